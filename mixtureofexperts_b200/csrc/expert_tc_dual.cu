// Grouped expert GEMMs, one CTA per SM working on TWO 128-row m-tiles against ONE weight tile.
//
// Same products, MMA shape (tcgen05.mma cta_group::1, M=128, N=256, K=16) and epilogue math as the
// single-CTA kernel (expert_tc.cu).  What changes is the operand traffic: the two m-tiles are the halves
// of a 256-row pair tile (same expert, same n-tile), so per K block the CTA stages two 16 KB A boxes and
// ONE 32 KB B box and issues the MMAs of both m-tiles from that B box: 64 KB from L2 per 8.4 MFLOP
// instead of 48 KB per 4.2 MFLOP.  The expert GEMMs run at the board's power limit on B200, so what a
// kernel moves per FLOP decides its speed; the cta_group::2 kernel saves the same L2 reads but its tensor
// cores fetch half of every B tile from the peer SM.  Measured on a Mixtral-shaped layer (4096 rows per
// expert): 3.2 % faster than the single-CTA kernel; the advantage is gone at 2048 rows per expert
// because 256-row tiles waste twice as much on an expert's ragged end.
//
// The price: two 128 x 256 FP32 accumulators are all 512 TMEM columns, so there is no second
// accumulator set for the next tile while the epilogue drains this one.  Eight epilogue warps (four per
// accumulator) keep that gap short, and each accumulator has its own "drained" barrier so the MMAs of
// the next tile start on the first accumulator while the second is still being read.  (GEMM 1's exposed
// epilogue is bound by the special-function unit: hence one such operation per element in tc::act_fast.)
//
// Structure (320 threads): warp 0 = TMA producer (3-stage ring of 64 KB, full/empty mbarriers), warp 1 =
// MMA issuer, warps 2..5 = epilogue of accumulator 0, warps 6..9 = epilogue of accumulator 1.  A pair
// tile whose second half holds no rows of the expert (ragged tail) skips that half's loads and MMAs.
// Tile order and bounded waits as in the other kernels; no clusters, no multicast, usable with expert
// parallelism (`p.tile_prefix` must count 256-row tiles).
#include "tc_common.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BM = TC_TILE_M;            // 128 rows per accumulator
constexpr int BM2 = TC_PAIR_TILE_M;      // 256 rows per tile
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int TMEM_COLS = 2 * BN;        // 512: both accumulators
constexpr int NUM_THREADS = 320;
constexpr int A_TILE_BYTES = BM * BK * 2;         // 16 KiB
constexpr int B_HALF_BYTES = 128 * BK * 2;        // 16 KiB
constexpr int B_STAGE_BYTES = 2 * B_HALF_BYTES;   // 32 KiB

struct __align__(1024) DualStorage {
    uint8_t a[STAGES][2][A_TILE_BYTES];
    uint8_t b[STAGES][B_STAGE_BYTES];
    uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t acc_full_bar;          // both accumulators of the tile are complete
    uint64_t acc_empty_bar[2];      // accumulator i has been read out (4 epilogue warps each)
    uint32_t tmem_base;
    volatile int abort_flag;
};

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
group_gemm_tc_dual_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                          const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_x,
                          const GroupGemmParams p, const int gm) {
    extern __shared__ uint8_t smem_raw[];
    DualStorage* ss = reinterpret_cast<DualStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    constexpr int TILE_N_OUT = (MODE == 1) ? 128 : 256;
    const int n_tiles = (p.N + TILE_N_OUT - 1) / TILE_N_OUT;
    const int num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ss->full_bar[s], 1);
            mbar_init(&ss->empty_bar[s], 1);
        }
        mbar_init(&ss->acc_full_bar, 1);
        mbar_init(&ss->acc_empty_bar[0], 4);
        mbar_init(&ss->acc_empty_bar[1], 4);
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&ss->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;
    chain_release();
    chain_wait();
    const int total_tiles = p.tile_prefix[p.E] * n_tiles;     // tile_prefix counts 256-row tiles

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;
            bool ok = true;
            for (int L = blockIdx.x; ok && L < total_tiles; L += gridDim.x) {
                const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E, BM2);
                const bool has2 = t.row0 + BM < t.row_end;
                const int brow0 = (MODE == 1) ? t.n_idx * 128 : t.n_idx * 256;
                const int brow1 = (MODE == 1) ? t.n_idx * 128 : t.n_idx * 256 + 128;
                const bool inplace = t.e < p.inplace_experts;
                const CUtensorMap* ma = inplace ? &map_x : &map_a;
                const int arow = inplace ? t.row0 - p.expert_offset[t.e] : t.row0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ss->full_bar[stage], (uint32_t)(B_STAGE_BYTES + (has2 ? 2 : 1) * A_TILE_BYTES));
                    tma_load_2d(ss->a[stage][0], ma, kb * BK, arow, &ss->full_bar[stage]);
                    if (has2) tma_load_2d(ss->a[stage][1], ma, kb * BK, arow + BM, &ss->full_bar[stage]);
                    tma_load_3d(ss->b[stage], &map_b0, kb * BK, brow0, t.e, &ss->full_bar[stage]);
                    tma_load_3d(ss->b[stage] + B_HALF_BYTES, &map_b1, kb * BK, brow1, t.e, &ss->full_bar[stage]);
                    armed |= 1u << stage;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || ss->abort_flag) {
                // leaving early: the copies already issued get a bounded time to land
                for (int s = 0; s < STAGES; ++s) {
                    if (!(armed & (1u << s))) continue;
                    const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(&ss->full_bar[s], par) && globaltimer_ns() - t0 < DRAIN_LIMIT_NS) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t aphase = 0;     // parity of the accumulators' "drained" barriers: flips every tile
            bool ok = true;
            for (int L = blockIdx.x; ok && L < total_tiles; L += gridDim.x) {
                const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E, BM2);
                const bool has2 = t.row0 + BM < t.row_end;
                if (!mbar_wait(&ss->acc_empty_bar[0], aphase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY)) break;
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->full_bar[stage], phase, &ss->abort_flag, p.status, DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da0 = make_smem_desc(smem_u32(ss->a[stage][0]));
                    const uint64_t da1 = make_smem_desc(smem_u32(ss->a[stage][1]));
                    const uint64_t db = make_smem_desc(smem_u32(ss->b[stage]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(tmem_base, da0 + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
                    if (kb == 0) {
                        // the second accumulator may still be read out while the first one is already being written
                        if (!mbar_wait(&ss->acc_empty_bar[1], aphase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                    }
                    if (has2) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16(tmem_base + (uint32_t)BN, da1 + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                      (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&ss->empty_bar[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(&ss->acc_full_bar);
                aphase ^= 1u;
            }
        }
    } else {
        // ------------------------------ epilogue (warps 2..5: accumulator 0, warps 6..9: accumulator 1) ----
        const int acc = (warp - 2) >> 2;
        const int lane_group = warp & 3;                 // TMEM lanes this warp may read
        const int row_in_tile = acc * BM + lane_group * 32 + lane;
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        uint32_t aphase = 0;
        for (int L = blockIdx.x; L < total_tiles; L += gridDim.x) {
            const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E, BM2);
            const bool mine = acc == 0 || t.row0 + BM < t.row_end;     // the tile has rows for this accumulator
            int ready = 1;
            if (lane == 0) ready = mbar_wait(&ss->acc_full_bar, aphase, &ss->abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            while (!mbar_try_wait(&ss->acc_full_bar, aphase)) {
            }  // already complete: returns at once, gives every lane its own acquire
            tc_fence_after();
            if (mine) {
                const int row = t.row0 + row_in_tile;
                const bool row_ok = row < t.row_end;
                __nv_bfloat16* dst_row = row_ok ? group_gemm_out_row<__nv_bfloat16>(p, t.e, row) : C;
                const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN);
                const int col_base = t.n_idx * TILE_N_OUT;
                if (MODE == 1) {
#pragma unroll 1
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t g[32], u[32];
                        tmem_ld32(taddr + (uint32_t)c, g);
                        tmem_ld32(taddr + (uint32_t)(128 + c), u);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            v[i] = act_fast(p.activation, __uint_as_float(g[i])) * __uint_as_float(u[i]);
                        if (row_ok) store_row32(dst_row, col_base + c, p.N, v, vec_ok);
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < 256; c += 32) {
                        uint32_t a[32];
                        tmem_ld32(taddr + (uint32_t)c, a);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(a[i]);
                        if (p.bias) {
                            const float* b = p.bias + (size_t)t.e * p.N + col_base + c;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (col_base + c + i < p.N) v[i] += b[i];
                        }
                        if (p.epilogue_act >= 0) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = act_fast(p.epilogue_act, v[i]);
                        }
                        if (row_ok && col_base + c < p.N) store_row32(dst_row, col_base + c, p.N, v, vec_ok);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ss->acc_empty_bar[acc]);
            aphase ^= 1u;
        }
    }

    // ------------------------------ teardown --------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

// Same contract as launch_group_gemm_tc; `p.tile_prefix` must have been built for TC_PAIR_TILE_M rows per tile.
int launch_group_gemm_tc_dual(const TcGemmPlan* plan, int stage, int mode, const GroupGemmParams& p, int max_tiles, int num_sms,
                              cudaStream_t s) {
    if (!plan->valid) return -1;
    if (max_tiles <= 0) return 0;
    const size_t smem = sizeof(DualStorage) + 1024;
    static bool attr_done[64] = {};     // the attribute belongs to a (kernel, device) pair
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(group_gemm_tc_dual_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(group_gemm_tc_dual_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return -1;
        attr_done[dev] = true;
    }
    const int gm = group_m_setting();
    const int grid = max_tiles < num_sms ? max_tiles : num_sms;
    cudaError_t err;
    if (mode == 1)
        err = launch_kernel(group_gemm_tc_dual_kernel<1>, dim3(grid), dim3(NUM_THREADS), smem, s, plan->map_xp, plan->map_w1,
                            plan->map_w3, plan->map_x, p, gm);
    else if (stage == 1)
        err = launch_kernel(group_gemm_tc_dual_kernel<2>, dim3(grid), dim3(NUM_THREADS), smem, s, plan->map_xp, plan->map_w1,
                            plan->map_w1, plan->map_x, p, gm);
    else
        err = launch_kernel(group_gemm_tc_dual_kernel<2>, dim3(grid), dim3(NUM_THREADS), smem, s, plan->map_h, plan->map_w2,
                            plan->map_w2, plan->map_h, p, gm);
    return err == cudaSuccess ? 1 : -1;
}

}  // namespace moe
