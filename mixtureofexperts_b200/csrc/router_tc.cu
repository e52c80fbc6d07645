// Router for wide gates (33..80 router rows) and BF16 activations: the gate GEMM on the tensor cores
// with an error-free split of the FP32 router matrix, then the per-token gating with an exact FP32
// re-evaluation of every token whose ranking the tensor-core rounding could have changed.
//
// Why: the FP32-FMA router kernel (router.cu) is bound by instruction issue once the router has
// more than ~32 rows (66 rows x 2048 inputs x 32768 tokens = 4.4 G FMAs: 0.45 ms, 4 % of the HBM
// roofline), while the gate GEMM is only 9 GFLOP.  Replaces the same reference code as router.cu:
// Router call + compute_gates (src/core/router.jl:25-46, src/gating/topk.jl:24-44,
// src/gating/advanced.jl:80-108).
//
//   kernel 1 (router_logits_tc_kernel)   logits[t][e] = sum_d x[t][d] * W[e][d]
//       x is BF16 already; W (FP32) is split once, when the router is set, into three BF16 matrices
//       W = Whi + Wmid + Wlo (8 + 8 + 8 mantissa bits: the split is exact up to 2^-27 |W|), stacked
//       as one K-major [3*E_PAD][D] operand.  Every BF16 x BF16 product is exact in FP32, so the
//       only rounding left is the accumulation.  One tcgen05.mma (M=128 tokens, N=3*E_PAD, K=16)
//       per K step; the accumulator is drained into FP32 registers every 128 K steps (two
//       accumulators alternate), where lo+mid+hi are added smallest first, so a TMEM accumulation
//       chain is never longer than 8 instructions.  TMA feeds a 4-stage ring; roles and bounded
//       waits as in the expert GEMM (expert_tc.cu).
//   kernel 2 (router_gate_kernel)        one warp per token on those logits
//       First the ranking is probed: if any two neighbours among the top k+1 selection logits are
//       closer than RECHECK_REL * max(1, largest |logit| of the token), the token is set aside and,
//       after the others, its logits are recomputed with FP32 FMAs (the eight warps of the CTA share
//       the router rows, lanes split K, fixed-order shuffle sum) before gate_token() runs.  The
//       tensor-core logits are within ~1.5e-6 of that scale of the float64 values (measured in the
//       tests: the same as the FP32-FMA kernel), far below RECHECK_REL = 3e-5, so a token that is not
//       re-evaluated has the same ranking under exact arithmetic, and ties within 1e-6 are always
//       decided on FP32-FMA values.
#include <cuda.h>

#include "router_gate.cuh"
#include "tc_common.cuh"

namespace moe {

namespace {

using namespace tc;
using namespace gating;

constexpr int BM = 128;                 // tokens per tile (UMMA M)
constexpr int BK = 64;                  // K per stage (one 128-byte swizzle atom of BF16)
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int CHUNK_KB = 2;             // K blocks per accumulator drain: 128 K steps = 8 MMAs
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = 512;          // two accumulators of up to 256 columns
constexpr int NUM_THREADS = 192;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr float RECHECK_REL = 3e-5f;     // re-evaluate when two ranked logits are closer than this times max(1, |logit|)

template <int E_PAD>
struct __align__(1024) RouterTcStorage {
    static constexpr int B_STAGE_BYTES = 3 * E_PAD * BK * 2;
    uint8_t a[STAGES][A_STAGE_BYTES];
    uint8_t b[STAGES][B_STAGE_BYTES];
    uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t tmem_full_bar[ACC_STAGES];
    uint64_t tmem_empty_bar[ACC_STAGES];
    uint32_t tmem_base;
    volatile int abort_flag;
};

// 32 lanes x 16 consecutive FP32 columns: thread i of the warp receives lane (base_lane + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// W (FP32 [E][D]) -> three BF16 matrices stacked as [3*E_PAD][D]: rows [0,E) hi, [E_PAD, E_PAD+E) mid,
// [2 E_PAD, 2 E_PAD + E) lo; padding rows zero.  hi + mid + lo == W up to 2^-27 |W|.
__global__ void router_split_kernel(const float* w, __nv_bfloat16* w3, int E, int D, int E_pad) {
    const size_t n = (size_t)E_pad * D;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int e = (int)(i / D);
        float v = e < E ? w[i] : 0.f;
        const __nv_bfloat16 hi = __float2bfloat16_rn(v);
        v = v - __bfloat162float(hi);              // exact
        const __nv_bfloat16 mid = __float2bfloat16_rn(v);
        v = v - __bfloat162float(mid);             // exact
        const __nv_bfloat16 lo = __float2bfloat16_rn(v);
        w3[i] = hi;
        w3[n + i] = mid;
        w3[2 * n + i] = lo;
    }
}

template <int E_PAD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
router_logits_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                        float* __restrict__ logits, const int64_t T, const int D, int32_t* status) {
    using Storage = RouterTcStorage<E_PAD>;
    constexpr int BN = 3 * E_PAD;
    constexpr uint32_t STAGE_TX_BYTES = A_STAGE_BYTES + Storage::B_STAGE_BYTES;
    static_assert(E_PAD % 16 == 0 && BN <= 256, "router width");
    extern __shared__ uint8_t smem_raw[];
    Storage* ss = reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = (int)((T + BM - 1) / BM);
    const int num_kb = (D + BK - 1) / BK;
    const int num_chunks = (num_kb + CHUNK_KB - 1) / CHUNK_KB;

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
            uint32_t phase = 0, armed = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1u, &ss->abort_flag, status, DEV_TIMEOUT_SMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&ss->full_bar[stage], STAGE_TX_BYTES);
                    tma_load_2d(ss->a[stage], &map_x, kb * BK, tile * BM, &ss->full_bar[stage]);
                    tma_load_2d(ss->b[stage], &map_w, kb * BK, 0, &ss->full_bar[stage]);
                    armed |= 1u << stage;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok || ss->abort_flag) {
                // leaving early: give the copies already issued a bounded time to land
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
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                for (int c = 0; ok && c < num_chunks; ++c) {
                    if (!mbar_wait(&ss->tmem_empty_bar[as], aphase ^ 1u, &ss->abort_flag, status, DEV_TIMEOUT_TMEM_EMPTY)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)(as * 256);
                    const int kb_end = min(num_kb, (c + 1) * CHUNK_KB);
                    for (int kb = c * CHUNK_KB; kb < kb_end; ++kb) {
                        if (!mbar_wait(&ss->full_bar[stage], phase, &ss->abort_flag, status, DEV_TIMEOUT_TMA_FULL)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint64_t da = make_smem_desc(smem_u32(ss->a[stage]));
                        const uint64_t db = make_smem_desc(smem_u32(ss->b[stage]));
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                      (kb != c * CHUNK_KB || k != 0) ? 1u : 0u);
                        umma_commit(&ss->empty_bar[stage]);
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    if (!ok) break;
                    umma_commit(&ss->tmem_full_bar[as]);
                    if (++as == ACC_STAGES) {
                        as = 0;
                        aphase ^= 1u;
                    }
                }
            }
        }
    } else {
        // ------------------------------ epilogue (warps 2..5) ---------------------------------
        const int lane_group = warp & 3;
        int as = 0;
        uint32_t aphase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < num_tiles; tile += gridDim.x) {
            float acc[E_PAD];
#pragma unroll
            for (int i = 0; i < E_PAD; ++i) acc[i] = 0.f;
            for (int c = 0; c < num_chunks; ++c) {
                int ready = 1;
                if (lane == 0) ready = mbar_wait(&ss->tmem_full_bar[as], aphase, &ss->abort_flag, status, DEV_TIMEOUT_TMEM_FULL);
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (!ready) {
                    alive = false;
                    break;
                }
                while (!mbar_try_wait(&ss->tmem_full_bar[as], aphase)) {
                }  // already complete: gives every lane its own acquire
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(as * 256);
#pragma unroll
                for (int g = 0; g < E_PAD / 16; ++g) {
                    uint32_t hi[16], mid[16], lo[16];
                    tmem_ld16(taddr + (uint32_t)(g * 16), hi);
                    tmem_ld16(taddr + (uint32_t)(E_PAD + g * 16), mid);
                    tmem_ld16(taddr + (uint32_t)(2 * E_PAD + g * 16), lo);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        acc[g * 16 + i] += (__uint_as_float(lo[i]) + __uint_as_float(mid[i])) + __uint_as_float(hi[i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ss->tmem_empty_bar[as]);
                if (++as == ACC_STAGES) {
                    as = 0;
                    aphase ^= 1u;
                }
            }
            if (!alive) break;
            const int64_t t = (int64_t)tile * BM + lane_group * 32 + lane;
            if (t < T) {
                float4* dst = reinterpret_cast<float4*>(logits + (size_t)t * E_PAD);
#pragma unroll
                for (int q = 0; q < E_PAD / 4; ++q) dst[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// NE logits of token t with FP32 FMAs by one warp: lanes split K in 16-byte pieces (8 products per
// piece into one accumulator per logit, at most D/32 products per lane), then fixed-order shuffle sums.
// The NE router rows are read side by side so that their loads are in flight together.
template <int NE>
__device__ __forceinline__ void exact_logits(const __nv_bfloat16* __restrict__ x, const float* const (&w)[NE], int D, int lane,
                                             float (&out)[NE]) {
    float s[NE];
#pragma unroll
    for (int i = 0; i < NE; ++i) s[i] = 0.f;
#pragma unroll 2
    for (int k0 = lane * 8; k0 < D; k0 += 256) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + k0);
        float4 w0[NE], w1[NE];
#pragma unroll
        for (int i = 0; i < NE; ++i) {
            w0[i] = *reinterpret_cast<const float4*>(w[i] + k0);
            w1[i] = *reinterpret_cast<const float4*>(w[i] + k0 + 4);
        }
        const float x0 = __uint_as_float(xv.x << 16), x1 = __uint_as_float(xv.x & 0xffff0000u),
                    x2 = __uint_as_float(xv.y << 16), x3 = __uint_as_float(xv.y & 0xffff0000u),
                    x4 = __uint_as_float(xv.z << 16), x5 = __uint_as_float(xv.z & 0xffff0000u),
                    x6 = __uint_as_float(xv.w << 16), x7 = __uint_as_float(xv.w & 0xffff0000u);
#pragma unroll
        for (int i = 0; i < NE; ++i) {
            s[i] = fmaf(x0, w0[i].x, s[i]);
            s[i] = fmaf(x1, w0[i].y, s[i]);
            s[i] = fmaf(x2, w0[i].z, s[i]);
            s[i] = fmaf(x3, w0[i].w, s[i]);
            s[i] = fmaf(x4, w1[i].x, s[i]);
            s[i] = fmaf(x5, w1[i].y, s[i]);
            s[i] = fmaf(x6, w1[i].z, s[i]);
            s[i] = fmaf(x7, w1[i].w, s[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < NE; ++i) out[i] = warp_sum(s[i]);
}

constexpr int GATE_THREADS = 256;
constexpr int GATE_WARPS = GATE_THREADS / 32;

// Phase 1: every warp gates its tokens of the tile from the tensor-core logits, except those whose
// ranking is too close to call; those are noted in a bit mask.  Phase 2: the noted tokens, in token
// order, get exact logits (all eight warps share the router rows of one token) and are then gated by
// warp 0.  The order of every floating-point sum is fixed, so two runs give the same bits.
template <int NJ>
__global__ void __launch_bounds__(GATE_THREADS) router_gate_kernel(const RouterParams p, const float* __restrict__ logits,
                                                                  const int ld, int32_t* __restrict__ recheck_count) {
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_psum[GATE_WARPS][MAX_EXPERTS];
    __shared__ float s_lse2[GATE_WARPS];
    __shared__ double s_ent[GATE_WARPS];
    __shared__ unsigned long long s_defer;            // tokens_per_cta <= 64
    __shared__ float s_exact[MAX_ROUTER_EXPERTS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < MAX_EXPERTS; i += GATE_THREADS) s_cnt[i] = 0;
    for (int i = tid; i < GATE_WARPS * MAX_EXPERTS; i += GATE_THREADS) (&s_psum[0][0])[i] = 0.f;
    if (tid == 0) s_defer = 0ull;
    __syncthreads();
    const int64_t tok0 = (int64_t)blockIdx.x * p.tokens_per_cta;
    const GateCtx c = make_ctx(p);
    float lse2 = 0.f;
    double ent = 0.0;
    for (int tok = warp; tok < p.tokens_per_cta; tok += GATE_WARPS) {
        const int64_t t = tok0 + tok;
        if (t >= p.T) break;
        float lg[NJ], nl[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane + 32 * j;
            lg[j] = e < p.E_router ? logits[(size_t)t * ld + e] : 0.f;
            nl[j] = 0.f;
        }
        // probe threshold: RECHECK_REL times max(1, largest |logit| of the token)
        float mag = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < p.E_router && fabsf(lg[j]) <= FLT_MAX) mag = fmaxf(mag, fabsf(lg[j]));
        mag = __int_as_float(__reduce_max_sync(0xffffffffu, __float_as_int(mag)));   // non-negative floats order like ints
        if (!gate_token<NJ, true>(c, t, lg, nl, lane, s_cnt, s_psum[warp], lse2, ent, RECHECK_REL * fmaxf(1.f, mag))) {
            if (lane == 0) atomicOr(&s_defer, 1ull << tok);
        }
    }
    __syncthreads();
    unsigned long long defer = s_defer;
    if (defer != 0ull && tid == 0 && recheck_count) atomicAdd(recheck_count, __popcll(defer));
    while (defer != 0ull) {
        const int tok = __ffsll((long long)defer) - 1;
        defer &= defer - 1ull;
        const int64_t t = tok0 + tok;
        const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x) + (size_t)t * p.D;
        // warp w owns router rows w, w + 8, w + 16, ...; four rows at a time
        for (int e0 = warp; e0 < p.E_router; e0 += 4 * GATE_WARPS) {
            const float* rows[4];
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) rows[i] = p.w + (size_t)min(e0 + i * GATE_WARPS, p.E_router - 1) * p.D;
            exact_logits<4>(x, rows, p.D, lane, v);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (lane == 0 && e0 + i * GATE_WARPS < p.E_router) s_exact[e0 + i * GATE_WARPS] = v[i];
        }
        __syncthreads();
        if (warp == 0) {
            float lg[NJ], nl[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int e = lane + 32 * j;
                lg[j] = e < p.E_router ? s_exact[e] : 0.f;
                nl[j] = 0.f;
            }
            gate_token<NJ, false>(c, t, lg, nl, lane, s_cnt, s_psum[0], lse2, ent);
        }
        __syncthreads();
    }
    if (lane == 0) {
        s_lse2[warp] = lse2;
        s_ent[warp] = ent;
    }
    __syncthreads();
    for (int e = tid; e < p.E; e += GATE_THREADS) p.cta_counts[(size_t)blockIdx.x * p.E + e] = s_cnt[e];
    for (int e = tid; e < p.E_probs; e += GATE_THREADS) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GATE_WARPS; ++w) s += s_psum[w][e];
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + e] = s;
    }
    if (tid == 0) {
        float s = 0.f;
        double d = 0.0;
        for (int w = 0; w < GATE_WARPS; ++w) {
            s += s_lse2[w];
            d += s_ent[w];
        }
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + p.E_probs] = s;
        p.cta_entropy[blockIdx.x] = d;
    }
}

template <int E_PAD>
int launch_logits(const CUtensorMap& mx, const CUtensorMap& mw, float* logits, int64_t T, int D, int32_t* status, int num_sms,
                  cudaStream_t s) {
    auto kern = router_logits_tc_kernel<E_PAD>;
    const size_t smem = sizeof(RouterTcStorage<E_PAD>) + 1024;
    static bool attr_done[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
        attr_done[dev] = true;
    }
    const int tiles = (int)((T + BM - 1) / BM);
    const int grid = tiles < num_sms ? tiles : num_sms;
    kern<<<grid, NUM_THREADS, smem, s>>>(mx, mw, logits, T, D, status);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

struct RouterTcPlan {
    CUtensorMap map_w;
    int e_pad = 0;
    bool valid = false;
};

RouterTcPlan* router_tc_plan_create() { return new RouterTcPlan(); }
void router_tc_plan_destroy(RouterTcPlan* p) { delete p; }

int router_tc_e_pad(int e_router) {
    // Up to 32 rows the FMA kernel is bound by reading x like this one (measured on 8 rows, 16384 tokens:
    // 0.097 ms against 0.100 ms); beyond 80 rows 3 * E_PAD accumulator columns no longer fit one tcgen05.mma.
    if (e_router <= 32 || e_router > 80) return 0;
    return e_router <= 48 ? 48 : (e_router <= 64 ? 64 : 80);
}

// Splits the router matrix into the stacked BF16 operand and encodes its tensor map.
int router_tc_plan_set(RouterTcPlan* plan, const float* w, void* w3, int e_router, int D, cudaStream_t s) {
    plan->valid = false;
    const int e_pad = router_tc_e_pad(e_router);
    if (!e_pad || D % 8) return 0;
    const size_t n = (size_t)e_pad * D;
    const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
    router_split_kernel<<<blocks, 256, 0, s>>>(w, reinterpret_cast<__nv_bfloat16*>(w3), e_router, D, e_pad);
    if (cudaGetLastError() != cudaSuccess) return -1;
    if (!tc_encode_bf16_2d(&plan->map_w, w3, (uint64_t)D, (uint64_t)(3 * e_pad), (uint32_t)(3 * e_pad))) return -1;
    plan->e_pad = e_pad;
    plan->valid = true;
    return 1;
}

bool router_tc_usable(const RouterTcPlan* plan, const void* x, int x_dtype, bool noise_network_armed, int e_router, int D,
                      int64_t T) {
    (void)T;
    return plan && plan->valid && x_dtype == MOE_DTYPE_BF16 && !noise_network_armed && D % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0 && router_tc_e_pad(e_router) == plan->e_pad;
}

int launch_router_tc(const RouterTcPlan* plan, const RouterParams& p, int num_cta, int num_sms, int32_t* status, cudaStream_t s) {
    CUtensorMap mx;
    if (!tc_encode_bf16_2d(&mx, p.x, (uint64_t)p.D, (uint64_t)p.T, 128u)) return -1;
    int n;
    switch (plan->e_pad) {
        case 48: n = launch_logits<48>(mx, plan->map_w, p.tc_logits, p.T, p.D, status, num_sms, s); break;
        case 64: n = launch_logits<64>(mx, plan->map_w, p.tc_logits, p.T, p.D, status, num_sms, s); break;
        case 80: n = launch_logits<80>(mx, plan->map_w, p.tc_logits, p.T, p.D, status, num_sms, s); break;
        default: return -1;
    }
    if (n < 0) return n;
    if (plan->e_pad <= 64)
        router_gate_kernel<2><<<num_cta, GATE_THREADS, 0, s>>>(p, p.tc_logits, plan->e_pad, p.tc_recheck_count);
    else
        router_gate_kernel<3><<<num_cta, GATE_THREADS, 0, s>>>(p, p.tc_logits, plan->e_pad, p.tc_recheck_count);
    return cudaGetLastError() == cudaSuccess ? n + 1 : -1;
}

}  // namespace moe
