// Grouped GatedExpert FFN on Blackwell tensor cores: BF16 operands, FP32 accumulation in TMEM.
//
//   mode 1:  h[r][j] = act(sum_d xp[r][d] W1[e][j][d]) * (sum_d xp[r][d] W3[e][j][d])   (BF16 out)
//   mode 2:  y[r][o] = sum_j h[r][j] W2[e][o][j]                                         (BF16 out)
//
// the three products of (expert::GatedExpert)(x) (src/experts/gated.jl:29-34) for every expert
// at once, on the rows the router sent to it only (src/cuda/experts.jl:28-57 ran three cuBLAS
// SGEMMs per expert on ALL tokens and masked afterwards).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128x64 A box and two 128x64 B boxes
//               per stage (128-byte swizzle), 4-stage ring guarded by full/empty mbarriers
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16, kind::f16) from
//               shared-memory descriptors into one of two 256-column TMEM accumulators;
//               tcgen05.commit releases ring stages and publishes finished accumulators
//   warps 2..5  epilogue: tcgen05.ld the accumulator (warp w owns TMEM lanes 32*(w%4)..+31),
//               apply act(gate)*up (mode 1), convert to BF16, 16-byte global stores; overlaps
//               the next tile's MMAs through the second accumulator
// In mode 1 the 256 accumulator columns are 128 W1 rows followed by the matching 128 W3 rows,
// so gate and up of one hidden unit meet in the same thread without interleaving the weights.
//
// Rows are grouped by expert (expert_offset); an expert's rows are cut into 128-row m-tiles
// (tile_prefix); a ragged last tile computes on whatever rows follow and masks its stores.
// Tiles are ordered expert-major, then in groups of m-tiles x n-tiles so that the CTAs running
// at the same time share A and B tiles through L2.
//
// Every mbarrier wait is bounded (globaltimer): on expiry the kernel records a DEV_TIMEOUT_*
// code in the status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include "activation.cuh"

namespace moe {

namespace {

constexpr int BM = TC_TILE_M;   // 128 rows per tile (UMMA M)
constexpr int BN = 256;         // accumulator columns per tile (UMMA N)
constexpr int BK = 64;          // K elements per stage: 128 bytes of BF16 = one swizzle atom
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = ACC_STAGES * BN;  // 512
constexpr int NUM_THREADS = 192;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_HALF_BYTES = 128 * BK * 2;        // 16 KiB
constexpr int B_STAGE_BYTES = 2 * B_HALF_BYTES;   // 32 KiB
constexpr uint32_t STAGE_TX_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait
constexpr unsigned long long DRAIN_LIMIT_NS = 2000000ull;    // 2 ms when draining after an abort

struct __align__(1024) SharedStorage {
    uint8_t a[STAGES][A_STAGE_BYTES];
    uint8_t b[STAGES][B_STAGE_BYTES];
    uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t tmem_full_bar[ACC_STAGES];
    uint64_t tmem_empty_bar[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the CTA is aborting or the limit expired (then it raises the
// abort flag and records `code`).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, SharedStorage* ss, int32_t* status,
                                          int32_t code, unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (ss->abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) {
                ss->abort_flag = 1;
                if (status) atomicCAS(status, DEV_OK, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, BF16 inputs, FP32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive FP32 columns: thread i of the warp receives lane (base_lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // bits [0,14): start address / 16
    d |= (uint64_t)1 << 16;                     // bits [16,30): leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;           // bits [32,46): stride byte offset / 16
    d |= (uint64_t)1 << 46;                     // bits [46,48): version
    d |= (uint64_t)2 << 61;                     // bits [61,64): SWIZZLE_128B
    return d;
}

// Instruction descriptor of kind::f16: FP32 accumulator, BF16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

struct TileCoord {
    int e;        // expert
    int row0;     // first permuted row of the tile
    int row_end;  // end of the expert's rows
    int n_idx;    // n-tile index
};

// Expert-major order; inside an expert, groups of `gm` m-tiles sweep all n-tiles (m fastest).
__device__ __forceinline__ TileCoord decode_tile(int L, int n_tiles, int gm, const int32_t* tile_prefix,
                                                 const int32_t* expert_offset, int E) {
    TileCoord t;
    const int e = find_segment(tile_prefix, E, L / n_tiles);
    const int m_tiles = tile_prefix[e + 1] - tile_prefix[e];
    const int local = L - tile_prefix[e] * n_tiles;
    const int g = local / (gm * n_tiles);
    const int rem = local - g * gm * n_tiles;
    const int gsz = min(gm, m_tiles - g * gm);
    const int m_local = g * gm + rem % gsz;
    t.e = e;
    t.n_idx = rem / gsz;
    t.row0 = expert_offset[e] + m_local * BM;
    t.row_end = expert_offset[e + 1];
    return t;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float act_fast(int act, float v) {
    switch (act) {
        case MOE_ACT_SILU:
            return __fdividef(v, 1.0f + __expf(-v));
        case MOE_ACT_GELU_TANH: {
            const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));  // tanh(u)
            return 0.5f * v * (1.0f + t);
        }
        case MOE_ACT_RELU:
            return fmaxf(v, 0.f);
        default:
            return v;
    }
}

// Store 32 consecutive BF16 columns of one row.
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst_row, int col0, int N, const float (&v)[32],
                                            bool vec_ok) {
    if (vec_ok && col0 + 32 <= N) {
        uint4* d = reinterpret_cast<uint4*>(dst_row + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            d[q] = u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < N) dst_row[col0 + i] = __float2bfloat16_rn(v[i]);
    }
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
group_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                     const __grid_constant__ CUtensorMap map_b1, const GroupGemmParams p, const int gm) {
    extern __shared__ uint8_t smem_raw[];
    SharedStorage* ss = reinterpret_cast<SharedStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                         ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // N_out columns per tile: mode 1 produces 128 hidden units (from 256 accumulator columns)
    constexpr int TILE_N_OUT = (MODE == 1) ? 128 : 256;
    const int n_tiles = (p.N + TILE_N_OUT - 1) / TILE_N_OUT;
    const int total_tiles = p.tile_prefix[p.E] * n_tiles;
    const int num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ss->full_bar[s], 1);
            mbar_init(&ss->empty_bar[s], 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(&ss->tmem_full_bar[s], 1);
            mbar_init(&ss->tmem_empty_bar[s], 4);  // one arrival per epilogue warp
        }
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&ss->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;  // bit s: stage s has a load in flight that nobody consumed yet
            bool ok = true;
            for (int L = blockIdx.x; ok && L < total_tiles; L += gridDim.x) {
                const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E);
                const int brow0 = (MODE == 1) ? t.n_idx * 128 : t.n_idx * 256;
                const int brow1 = (MODE == 1) ? t.n_idx * 128 : t.n_idx * 256 + 128;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1u, ss, p.status, DEV_TIMEOUT_SMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ss->full_bar[stage], STAGE_TX_BYTES);
                    tma_load_2d(ss->a[stage], &map_a, kb * BK, t.row0, &ss->full_bar[stage]);
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
                // Leaving early: give the copies already issued a bounded time to land so that
                // none is still writing this CTA's shared memory when it exits.
                for (int s = 0; s < STAGES; ++s) {
                    if (!(armed & (1u << s))) continue;
                    // stage s was last armed in the current phase if s < stage, else in the previous one
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
            int as = 0;
            uint32_t aphase = 0;
            bool ok = true;
            for (int L = blockIdx.x; ok && L < total_tiles; L += gridDim.x) {
                if (!mbar_wait(&ss->tmem_empty_bar[as], aphase ^ 1u, ss, p.status, DEV_TIMEOUT_TMEM_EMPTY)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(as * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->full_bar[stage], phase, ss, p.status, DEV_TIMEOUT_TMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(smem_u32(ss->a[stage]));
                    const uint64_t db = make_smem_desc(smem_u32(ss->b[stage]));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // +32 bytes along K inside the swizzle atom = +2 in the (addr/16) field
                        umma_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                  (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&ss->empty_bar[stage]);  // frees the stage once these MMAs finish
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                umma_commit(&ss->tmem_full_bar[as]);     // accumulator complete
                if (++as == ACC_STAGES) {
                    as = 0;
                    aphase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------ epilogue (warps 2..5) ---------------------------------
        const int lane_group = warp & 3;                 // TMEM lanes this warp may read
        const int row_in_tile = lane_group * 32 + lane;
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
        const bool vec_ok = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        int as = 0;
        uint32_t aphase = 0;
        for (int L = blockIdx.x; L < total_tiles; L += gridDim.x) {
            const TileCoord t = decode_tile(L, n_tiles, gm, p.tile_prefix, p.expert_offset, p.E);
            // lane 0 does the bounded wait and the warp follows its verdict, so the warp-wide
            // tcgen05.ld below is never reached by a part of the warp only
            int ready = 1;
            if (lane == 0) ready = mbar_wait(&ss->tmem_full_bar[as], aphase, ss, p.status, DEV_TIMEOUT_TMEM_FULL);
            ready = __shfl_sync(0xffffffffu, ready, 0);
            if (!ready) break;
            while (!mbar_try_wait(&ss->tmem_full_bar[as], aphase)) {
            }  // already complete: returns at once, gives every lane its own acquire
            tc_fence_after();
            const int row = t.row0 + row_in_tile;
            const bool row_ok = row < t.row_end;
            __nv_bfloat16* dst_row = C + (size_t)row * p.N;
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
                    if (row_ok && col_base + c < p.N) store_row32(dst_row, col_base + c, p.N, v, vec_ok);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ss->tmem_empty_bar[as]);
            if (++as == ACC_STAGES) {
                as = 0;
                aphase ^= 1u;
            }
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    return fn;
}

// rows x K BF16 matrix (K contiguous), optionally a stack of `batch` such matrices.
bool encode_map(CUtensorMap* map, const void* base, uint64_t K, uint64_t rows, uint64_t batch, bool three_d) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {K, rows, batch};
    cuuint64_t strides[2] = {K * 2, K * rows * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, 128u, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, three_d ? 3 : 2, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

struct TcGemmPlan {
    CUtensorMap map_xp, map_h, map_w1, map_w3, map_w2;
    bool valid = false;
    bool attr_set = false;
};

TcGemmPlan* tc_plan_create() { return new TcGemmPlan(); }
void tc_plan_destroy(TcGemmPlan* p) { delete p; }

int tc_plan_encode(TcGemmPlan* plan, const void* xp, const void* h, int64_t P_cap, int D, int H, int O, int E,
                   const void* w1, const void* w3, const void* w2, const char** out_msg) {
    plan->valid = false;
    if (D % 8 || H % 8) {
        *out_msg = "the BF16 tensor-core path needs input_dim and hidden_dim to be multiples of 8 (16-byte TMA strides)";
        return MOE_ERR_UNSUPPORTED;
    }
    if (!get_encode_fn()) {
        *out_msg = "cuTensorMapEncodeTiled is not available from this driver";
        return MOE_ERR_CUDA;
    }
    const bool ok = encode_map(&plan->map_xp, xp, (uint64_t)D, (uint64_t)P_cap, 1, false) &&
                    encode_map(&plan->map_h, h, (uint64_t)H, (uint64_t)P_cap, 1, false) &&
                    encode_map(&plan->map_w1, w1, (uint64_t)D, (uint64_t)H, (uint64_t)E, true) &&
                    encode_map(&plan->map_w3, w3, (uint64_t)D, (uint64_t)H, (uint64_t)E, true) &&
                    encode_map(&plan->map_w2, w2, (uint64_t)H, (uint64_t)O, (uint64_t)E, true);
    if (!ok) {
        *out_msg = "cuTensorMapEncodeTiled failed";
        return MOE_ERR_CUDA;
    }
    plan->valid = true;
    return MOE_OK;
}

int launch_group_gemm_tc(const TcGemmPlan* plan_c, int mode, const GroupGemmParams& p, int max_tiles, int num_sms,
                         cudaStream_t s) {
    TcGemmPlan* plan = const_cast<TcGemmPlan*>(plan_c);
    if (!plan->valid) return -1;
    if (max_tiles <= 0) return 0;
    const size_t smem = sizeof(SharedStorage) + 1024;
    if (!plan->attr_set) {
        if (cudaFuncSetAttribute(group_gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
                cudaSuccess ||
            cudaFuncSetAttribute(group_gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
                cudaSuccess)
            return -1;
        plan->attr_set = true;
    }
    static int gm_env = -1;
    if (gm_env < 0) {
        const char* e = getenv("MOE_B200_GROUP_M");
        gm_env = e ? atoi(e) : 0;
        if (gm_env < 0) gm_env = 0;
    }
    const int gm = gm_env > 0 ? gm_env : 16;
    const int grid = max_tiles < num_sms ? max_tiles : num_sms;
    if (mode == 1)
        group_gemm_tc_kernel<1><<<grid, NUM_THREADS, smem, s>>>(plan->map_xp, plan->map_w1, plan->map_w3, p, gm);
    else
        group_gemm_tc_kernel<2><<<grid, NUM_THREADS, smem, s>>>(plan->map_h, plan->map_w2, plan->map_w2, p, gm);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
