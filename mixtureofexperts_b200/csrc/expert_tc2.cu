// Grouped GatedExpert GEMM, CTA-pair variant (tcgen05 cta_group::2): a cluster of two CTAs on two
// SMs computes a 256-row x 256-column tile.  Each CTA stages its own 128 rows of A and HALF of the
// B tile (128 of the 256 weight rows); one thread of the leader CTA issues tcgen05.mma with M=256,
// which reads A and B from both CTAs' shared memory and writes each CTA's 128 rows of the
// accumulator into that CTA's TMEM.  Per 512 MMA cycles a CTA now pulls 32 KiB through its
// shared-memory port instead of 48 KiB, and the ring is 6 stages deep instead of 4.
//
// Same math, operands and outputs as expert_tc.cu (modes 1 and 2); used when experts have enough
// rows that rounding an expert up to 256-row tiles costs little.  In mode 1 the leader loads the
// W1 half and the peer the W3 half, so a thread still finds gate and up of a hidden unit in its
// own accumulator row.
//
// Synchronisation inside the pair:
//   full[s]       lives in the LEADER: its producer arms it for the bytes of both CTAs; both
//                 producers' TMA loads complete on it (the peer names it by its cluster address)
//   empty[s]      one per CTA; the leader's tcgen05.commit multicasts the arrival to both
//   tmem_full[a]  one per CTA, multicast commit after the last k-block of a tile
//   tmem_empty[a] lives in the leader, 8 arrivals: the four epilogue warps of each CTA
// No TMA load uses cluster multicast.  Every wait is bounded (see tc_common.cuh); the two cluster
// barriers (start-up, tear-down) are reached by every thread on every path.
#include "tc_common.cuh"

namespace moe {

namespace {

using namespace tc;

constexpr int BM_CTA = 128;     // rows per CTA
constexpr int BM_PAIR = TC_PAIR_TILE_M;  // 256 rows per CTA pair
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;
constexpr int NUM_THREADS = 192;
constexpr int A_STAGE_BYTES = BM_CTA * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = 128 * BK * 2;      // 16 KiB: this CTA's half of the B tile
constexpr uint32_t PAIR_TX_BYTES = 2 * (A_STAGE_BYTES + B_STAGE_BYTES);

struct __align__(1024) PairStorage {
    uint8_t a[STAGES][A_STAGE_BYTES];
    uint8_t b[STAGES][B_STAGE_BYTES];
    uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t tmem_full_bar[ACC_STAGES];
    uint64_t tmem_empty_bar[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t num_clusters_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();   // the aligned forms need the whole warp converged
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// Raise the abort flag of the other CTA of the pair too, so that it leaves its loops at its next
// check instead of when its own waits run out.
__device__ __forceinline__ void raise_peer_abort(volatile int* my_flag, uint32_t my_rank) {
    const uint32_t peer = map_to_cta(smem_u32(const_cast<int*>(my_flag)), my_rank ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"(1u) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA loads of the pair kernel: data lands in this CTA, completion is counted on `bar_cluster_addr`
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                             uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                             uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster_addr)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive, in both CTAs of the pair, on the barrier at this shared-memory offset once every MMA
// issued so far has completed.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
group_gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                      const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_x,
                      const GroupGemmParams p, const int gm) {
    extern __shared__ uint8_t smem_raw[];
    PairStorage* ss = reinterpret_cast<PairStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();      // 0 = leader
    const bool leader = rank == 0;

    constexpr int TILE_N_OUT = (MODE == 1) ? 128 : 256;
    const int n_tiles = (p.N + TILE_N_OUT - 1) / TILE_N_OUT;
    const int total_tiles = p.tile_prefix[p.E] * n_tiles;     // tile_prefix counts 256-row pair tiles
    const int num_kb = (p.K + BK - 1) / BK;
    const int tile0 = (int)cluster_id_x(), tile_step = (int)num_clusters_x();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ss->full_bar[s], 1);
            mbar_init(&ss->empty_bar[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(&ss->tmem_full_bar[s], 1);
            mbar_init(&ss->tmem_empty_bar[s], 8);   // four epilogue warps of each CTA
        }
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    cluster_sync_all();                               // both CTAs' barriers exist
    if (warp == 1) tmem_alloc2(&ss->tmem_base, TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();                               // both CTAs hold their TMEM columns
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer (one per CTA) -----------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;   // bit s: this CTA has issued copies into stage s that nobody consumed yet
            for (int L = tile0; L < total_tiles; L += tile_step) {
                const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E, BM_PAIR);
                // an expert that sees every token in token order reads the activations themselves
                const bool inplace = t.e < p.inplace_experts;
                const CUtensorMap* ma = inplace ? &map_x : &map_a;
                const int arow = t.row0 + (int)rank * BM_CTA - (inplace ? p.expert_offset[t.e] : 0);
                // this CTA's half of the weight tile
                const CUtensorMap* mb = (MODE == 1 && rank == 1) ? &map_b1 : &map_b0;
                const int brow = (MODE == 1) ? t.n_idx * 128 : t.n_idx * 256 + (int)rank * 128;
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full_leader = map_to_cta(smem_u32(&ss->full_bar[stage]), 0);
                    if (leader) mbar_expect_tx(&ss->full_bar[stage], PAIR_TX_BYTES);
                    tma2_load_2d(ss->a[stage], ma, kb * BK, arow, full_leader);
                    tma2_load_3d(ss->b[stage], mb, kb * BK, brow, t.e, full_leader);
                    armed |= 1u << stage;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
            }
            if (ss->abort_flag) {
                // Leaving early: tell the other CTA, then give the copies already issued a bounded time to
                // land so that none is still writing this CTA's shared memory when it exits.  The leader can
                // watch its full barriers (both CTAs' copies complete there); the peer has no barrier of its
                // own for them and simply waits out the limit.
                raise_peer_abort(&ss->abort_flag, rank);
                const unsigned long long t0 = globaltimer_ns();
                if (leader) {
                    for (int s2 = 0; s2 < STAGES; ++s2) {
                        if (!(armed & (1u << s2))) continue;
                        const uint32_t par = (s2 < stage) ? phase : (phase ^ 1u);
                        while (!mbar_try_wait(&ss->full_bar[s2], par) && globaltimer_ns() - t0 < DRAIN_LIMIT_NS) {
                        }
                    }
                } else if (armed) {
                    while (globaltimer_ns() - t0 < DRAIN_LIMIT_NS) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ---------------------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM_PAIR, BN);
            int stage = 0;
            uint32_t phase = 0;
            int as = 0;
            uint32_t aphase = 0;
            bool ok = true;
            for (int L = tile0; ok && L < total_tiles; L += tile_step) {
                if (!mbar_wait(&ss->tmem_empty_bar[as], aphase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_TMEM_EMPTY)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(as * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->full_bar[stage], phase, &ss->abort_flag, p.status, DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(ss->a[stage]));
                    const uint64_t db = make_smem_desc(smem_u32(ss->b[stage]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma2_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
                    umma2_commit_both(&ss->empty_bar[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma2_commit_both(&ss->tmem_full_bar[as]);
                if (++as == ACC_STAGES) {
                    as = 0;
                    aphase ^= 1u;
                }
            }
            if (ss->abort_flag) raise_peer_abort(&ss->abort_flag, rank);
        }
    } else {
        // ------------------------------ epilogue (warps 2..5 of each CTA) ----------------------
        const int lane_group = warp & 3;
        const int row_in_cta = lane_group * 32 + lane;
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        int as = 0;
        uint32_t aphase = 0;
        for (int L = tile0; L < total_tiles; L += tile_step) {
            const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E, BM_PAIR);
            int ready = 1;
            if (lane == 0) ready = mbar_wait(&ss->tmem_full_bar[as], aphase, &ss->abort_flag, p.status, DEV_TIMEOUT_TMEM_FULL);
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            while (!mbar_try_wait(&ss->tmem_full_bar[as], aphase)) {
            }
            tc_fence_after();
            const int row = t.row0 + (int)rank * BM_CTA + row_in_cta;
            const bool row_ok = row < t.row_end;
            __nv_bfloat16* dst_row = row_ok ? group_gemm_out_row<__nv_bfloat16>(p, t.e, row) : C;
            const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(as * BN);
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ss->tmem_empty_bar[as]), 0));
            if (++as == ACC_STAGES) {
                as = 0;
                aphase ^= 1u;
            }
        }
        if (lane == 0 && ss->abort_flag) raise_peer_abort(&ss->abort_flag, rank);
    }

    // ------------------------------ teardown --------------------------------------------------
    // Nobody leaves, and no TMEM is freed, before both CTAs are done: the peer's barriers, shared
    // memory and TMEM are targets of this CTA's MMAs, commits and arrivals.
    __syncwarp();                 // lanes that ran a role loop rejoin their warp before the aligned barrier
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, TMEM_COLS);
    }
}

}  // namespace

// Launch of the CTA-pair kernel; same contract as launch_group_gemm_tc.  `p.tile_prefix` must have
// been built for TC_PAIR_TILE_M rows per tile.
int launch_group_gemm_tc2(const TcGemmPlan* plan_c, int stage, int mode, const GroupGemmParams& p, int max_tiles,
                          int num_sms, cudaStream_t s) {
    TcGemmPlan* plan = const_cast<TcGemmPlan*>(plan_c);
    if (!plan->valid) return -1;
    if (max_tiles <= 0) return 0;
    const size_t smem = sizeof(PairStorage) + 1024;
    if (!plan->attr2_set) {
        if (cudaFuncSetAttribute(group_gemm_tc2_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
                cudaSuccess ||
            cudaFuncSetAttribute(group_gemm_tc2_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
                cudaSuccess)
            return -1;
        plan->attr2_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (plan->max_clusters == 0) {
        // how many CTA pairs the device keeps resident at once: a persistent grid must not exceed it
        cfg.gridDim = dim3(2 * (num_sms / 2));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, group_gemm_tc2_kernel<1>, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = num_sms / 2;
        }
        plan->max_clusters = n < num_sms / 2 ? n : num_sms / 2;
    }
    const int clusters = max_tiles < plan->max_clusters ? max_tiles : plan->max_clusters;
    cfg.gridDim = dim3(2 * clusters);
    const int gm = group_m_setting();
    cudaError_t e;
    if (mode == 1)
        e = cudaLaunchKernelEx(&cfg, group_gemm_tc2_kernel<1>, plan->map_xp, plan->map_w1, plan->map_w3, plan->map_x, p, gm);
    else if (stage == 1)
        e = cudaLaunchKernelEx(&cfg, group_gemm_tc2_kernel<2>, plan->map_xp, plan->map_w1, plan->map_w1, plan->map_x, p, gm);
    else
        e = cudaLaunchKernelEx(&cfg, group_gemm_tc2_kernel<2>, plan->map_h, plan->map_w2, plan->map_w2, plan->map_h, p, gm);
    return e == cudaSuccess ? 1 : -1;
}

}  // namespace moe
