// Fused router: gate GEMM (FP32 FMA, split-K + two-level summation for a short rounding chain) -> softmax -> top-k
// (k arg-max passes, ties to the lowest index) -> renormalised gates -> per-CTA expert
// histogram and per-CTA partial sums for the Switch loss, the z-loss and the routing entropy.
//
// Replaces Router.__call__ + compute_gates of the reference (src/core/router.jl:25-46,
// src/gating/topk.jl:24-44, src/gating/advanced.jl:80-108) and its GPU kernels
// (src/cuda/router.jl:5-71, src/cuda/kernels.jl:3-58).
//
// Bound: HBM (reads x once: T*D*sizeof(x); everything else is O(T*E)).
#include "common.cuh"
#include "router_gate.cuh"

#include <cfloat>
#include <cstdlib>
#include <climits>

namespace moe {

namespace {

using namespace gating;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// 16-byte async copy that reads only `src_bytes` (0..16) and zero-fills the rest.
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gmem_src), "r"(src_bytes)
                 : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}


template <typename XT> struct XElt;
template <> struct XElt<float> { static constexpr int PER16 = 4; };
template <> struct XElt<__nv_bfloat16> { static constexpr int PER16 = 8; };

// One pipeline stage: a [16*NI tokens][BK (+16 bytes pad)] tile of x in its own dtype and the
// [BK][E_PAD] block of the K-major router matrix.
template <int E_PAD, int BK, typename XT, int NI>
struct RouterStage {
    static constexpr int ROW_ELTS = BK + XElt<XT>::PER16;   // padded row, stays 16-byte aligned
    XT x[16 * NI][ROW_ELTS];
    float w[BK][E_PAD];
};

// ring depth: small token tiles keep more chunks in flight (the same bytes per CTA)
template <int NI> struct RouterRing { static constexpr int STAGES = NI == 4 ? 3 : (NI == 2 ? 4 : 6); };

template <int E_PAD, int BK, int KS, typename XT, int NI>
union RouterSmem {
    RouterStage<E_PAD, BK, XT, NI> st[RouterRing<NI>::STAGES];
    float red[KS * 16 * NI * E_PAD];  // [KS][tokens][E_PAD]
};

// Gate GEMM as a register-tiled FP32 FMA kernel: a CTA owns 16*NI tokens x E_PAD router rows
// (NI = 4, 2 or 1: small batches and narrow routers take small tiles, so that enough CTAs exist to
// keep every SM's memory pipeline busy); a thread owns NI tokens x 8 rows and 1/KS of every K chunk (16 * E_PAD/8 * KS threads), so the
// per-thread FP32 chain stays short; an inner accumulator is folded into an outer one every
// ~256 products (two-level summation) and the KS partials are added in a fixed order.  x (in
// its own dtype) and the K-major router matrix ([K][E_PAD], built once per set_router) stream
// through a 3-stage cp.async ring; every token row contributes BK contiguous elements per chunk.
template <int E_PAD, int BK, int KS, typename XT, int NI>
__global__ void __launch_bounds__(16 * (E_PAD / 8) * KS, (16 * (E_PAD / 8) * KS <= 320 ? 2 : 1))
router_kernel(const RouterParams p) {
    constexpr int RT_BT = 16 * NI;
    constexpr int RT_STAGES = RouterRing<NI>::STAGES;
    constexpr int EG = E_PAD / 8;
    constexpr int TG = 16;
    constexpr int NTHREADS = TG * EG * KS;
    constexpr int NWARPS = NTHREADS / 32;
    static_assert(NTHREADS % 32 == 0 && NWARPS <= ROUTER_MAX_WARPS, "thread layout");
    constexpr int KPT = BK / KS;
    constexpr int FOLD = (256 / KPT) > 0 ? (256 / KPT) : 1;
    constexpr int PER16 = XElt<XT>::PER16;
    constexpr int UPR = BK / PER16;                    // 16-byte units per token row per chunk
    constexpr int XUNITS = RT_BT * UPR;
    using Stage = RouterStage<E_PAD, BK, XT, NI>;
    static_assert(KPT >= 2 && KPT % 2 == 0, "tile configuration");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    RouterSmem<E_PAD, BK, KS, XT, NI>& sm = *reinterpret_cast<RouterSmem<E_PAD, BK, KS, XT, NI>*>(smem_raw);
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_psum[NWARPS][MAX_EXPERTS];
    __shared__ float s_lse2[NWARPS];
    __shared__ double s_ent[NWARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int eg = tid % EG, tg = (tid / EG) % TG, ks = tid / (EG * TG);
    for (int i = tid; i < MAX_EXPERTS; i += NTHREADS) s_cnt[i] = 0;
    for (int i = tid; i < NWARPS * MAX_EXPERTS; i += NTHREADS) (&s_psum[0][0])[i] = 0.f;
    chain_release();
    chain_wait();   // x may be the output of the caller's previous kernel; the id/gate buffers are read by the previous forward's combine

    const int64_t tok0 = (int64_t)blockIdx.x * RT_BT;
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const bool vec_x = (p.D % PER16 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
    const int nchunks = (p.D + BK - 1) / BK;

    auto issue_chunk = [&](int c) {
        if (c < nchunks) {
            Stage& st = sm.st[c % RT_STAGES];
            const int kbase = c * BK;
            if (vec_x) {
                for (int u = tid; u < XUNITS; u += NTHREADS) {
                    const int tok = u / UPR, q = u % UPR;
                    const int64_t t = tok0 + tok;
                    const int k0 = kbase + q * PER16;
                    int bytes = (t < p.T && k0 < p.D) ? 16 : 0;   // D % PER16 == 0: a unit is all in or all out
                    const XT* src = bytes ? x + (size_t)t * p.D + k0 : x;
                    cp_async16_zfill(&st.x[tok][q * PER16], src, bytes);
                }
            } else {
                for (int i = tid; i < RT_BT * BK; i += NTHREADS) {
                    const int tok = i / BK, kk = i % BK;
                    const int64_t t = tok0 + tok;
                    XT v = XT(0.f);
                    if (t < p.T && kbase + kk < p.D) v = x[(size_t)t * p.D + kbase + kk];
                    st.x[tok][kk] = v;
                }
            }
            // rows [kbase, kbase+BK) of the K-major router matrix: one contiguous block (rows past D are zero)
            const float* src = p.wt + (size_t)kbase * E_PAD;
            float* dst = &st.w[0][0];
            for (int u = tid; u < BK * E_PAD / 4; u += NTHREADS) cp_async16(dst + u * 4, src + u * 4);
        }
        cp_async_commit();   // always commit, so that group counting stays uniform
    };

    float acc[NI][8], outer[NI][8];
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[i][j] = 0.f;
            outer[i][j] = 0.f;
        }

#pragma unroll
    for (int s = 0; s < RT_STAGES - 1; ++s) issue_chunk(s);
    for (int c = 0; c < nchunks; ++c) {
        cp_async_wait<RT_STAGES - 2>();   // chunk c has landed (this thread's copies)
        __syncthreads();                  // ... and everybody's; everybody is also done with chunk c-1
        issue_chunk(c + RT_STAGES - 1);
        const Stage& st = sm.st[c % RT_STAGES];
#pragma unroll
        for (int kk = 0; kk < KPT; kk += 2) {
            const int k = ks * KPT + kk;
            float x0[NI], x1[NI];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                if constexpr (sizeof(XT) == 2) {
                    const uint32_t w2 = *reinterpret_cast<const uint32_t*>(&st.x[i * 16 + tg][k]);
                    x0[i] = __uint_as_float(w2 << 16);
                    x1[i] = __uint_as_float(w2 & 0xffff0000u);
                } else {
                    const float2 w2 = *reinterpret_cast<const float2*>(&st.x[i * 16 + tg][k]);
                    x0[i] = w2.x;
                    x1[i] = w2.y;
                }
            }
            const float4 a0 = *reinterpret_cast<const float4*>(&st.w[k][eg * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&st.w[k][E_PAD / 2 + eg * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&st.w[k + 1][eg * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&st.w[k + 1][E_PAD / 2 + eg * 4]);
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                acc[i][0] = fmaf(x0[i], a0.x, acc[i][0]);
                acc[i][1] = fmaf(x0[i], a0.y, acc[i][1]);
                acc[i][2] = fmaf(x0[i], a0.z, acc[i][2]);
                acc[i][3] = fmaf(x0[i], a0.w, acc[i][3]);
                acc[i][4] = fmaf(x0[i], a1.x, acc[i][4]);
                acc[i][5] = fmaf(x0[i], a1.y, acc[i][5]);
                acc[i][6] = fmaf(x0[i], a1.z, acc[i][6]);
                acc[i][7] = fmaf(x0[i], a1.w, acc[i][7]);
                acc[i][0] = fmaf(x1[i], b0.x, acc[i][0]);
                acc[i][1] = fmaf(x1[i], b0.y, acc[i][1]);
                acc[i][2] = fmaf(x1[i], b0.z, acc[i][2]);
                acc[i][3] = fmaf(x1[i], b0.w, acc[i][3]);
                acc[i][4] = fmaf(x1[i], b1.x, acc[i][4]);
                acc[i][5] = fmaf(x1[i], b1.y, acc[i][5]);
                acc[i][6] = fmaf(x1[i], b1.z, acc[i][6]);
                acc[i][7] = fmaf(x1[i], b1.w, acc[i][7]);
            }
        }
        if ((c % FOLD) == FOLD - 1) {
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    outer[i][j] += acc[i][j];
                    acc[i][j] = 0.f;
                }
        }
    }
    cp_async_wait<0>();
    __syncthreads();   // the ring is dead from here on; its memory becomes the reduction buffer
    // partial sums of this thread's K slices -> shared [ks][token][row]
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int tok = i * 16 + tg;
        float* dst = &sm.red[((size_t)ks * RT_BT + tok) * E_PAD];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dst[eg * 4 + j] = outer[i][j] + acc[i][j];
            dst[E_PAD / 2 + eg * 4 + j] = outer[i][4 + j] + acc[i][4 + j];
        }
    }
    __syncthreads();

    const GateCtx c = make_ctx(p);
    constexpr int NJ = (E_PAD + 31) / 32;
    float lse2 = 0.f;
    double ent = 0.0;
    // routers of at most 8 / 16 columns: four / two tokens of a warp are gated side by side
    constexpr int GW = (E_PAD <= 8) ? 8 : ((E_PAD <= 16) ? 16 : 32);
    constexpr int TPW = 32 / GW;
    for (int base = warp * TPW; base < RT_BT; base += NWARPS * TPW) {
        if (tok0 + base >= p.T) break;
        const int tok = base + lane / GW;
        const int64_t t = tok0 + tok;
        const bool active = t < p.T;
        float lg[NJ], nl[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int e = lane % GW + 32 * j;
            float s = 0.f, sn = 0.f;
            if (e < E_PAD) {
#pragma unroll
                for (int q = 0; q < KS; ++q) s += sm.red[((size_t)q * RT_BT + tok) * E_PAD + e];
            }
            if (p.noise_off > 0 && e < p.E_router) {
#pragma unroll
                for (int q = 0; q < KS; ++q) sn += sm.red[((size_t)q * RT_BT + tok) * E_PAD + p.noise_off + e];
            }
            lg[j] = s;
            nl[j] = sn;
        }
        gate_token<NJ, false, GW>(c, t, lg, nl, lane, s_cnt, s_psum[warp], lse2, ent, 0.f, active);
    }
    if (lane == 0) {
        s_lse2[warp] = lse2;
        s_ent[warp] = ent;
    }
    __syncthreads();
    for (int e = tid; e < p.E; e += NTHREADS) p.cta_counts[(size_t)blockIdx.x * p.E + e] = s_cnt[e];
    for (int e = tid; e < p.E_probs; e += NTHREADS) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) s += s_psum[w][e];
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + e] = s;
    }
    if (tid == 0) {
        float s = 0.f;
        double d = 0.0;
        for (int w = 0; w < NWARPS; ++w) {
            s += s_lse2[w];
            d += s_ent[w];
        }
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + p.E_probs] = s;
        p.cta_entropy[blockIdx.x] = d;
    }
}

// wt[k][e] = w[e][k] for k < D, e < E; zero elsewhere (k < D_pad, e < E_pad)
__global__ void router_transpose_kernel(const float* w, float* wt, int E, int D, int E_pad, int D_pad) {
    const size_t n = (size_t)E_pad * D_pad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i / E_pad), e = (int)(i % E_pad);
        wt[i] = (k < D && e < E) ? w[(size_t)e * D + k] : 0.f;
    }
}

// the same with the noise network's rows behind the router's: column E + e = nw[e]
__global__ void router_transpose_noise_kernel(const float* w, const float* nw, float* wt, int E, int D, int E_pad,
                                              int D_pad) {
    const size_t n = (size_t)E_pad * D_pad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i / E_pad), e = (int)(i % E_pad);
        float v = 0.f;
        if (k < D && e < E) v = w[(size_t)e * D + k];
        else if (k < D && e < 2 * E) v = nw[(size_t)(e - E) * D + k];
        wt[i] = v;
    }
}

// compute_gates as a stand-alone operator on given logits: one warp per token.
__global__ void __launch_bounds__(ROUTER_THREADS) gates_only_kernel(GateCtx c, const float* logits, const float* jitter_u,
                                                                     float eps, int64_t T) {
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_psum[ROUTER_WARPS][MAX_EXPERTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * ROUTER_WARPS + warp;
    if (t >= T) return;
    constexpr int NJ = MAX_ROUTER_EXPERTS / 32;
    float lg[NJ], nl[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        lg[j] = (e < c.E_router) ? logits[t * c.E_router + e] : 0.f;
        // JitterGating (src/gating/switch.jl:28-31): logits .* (1 .+ (2 .* rand .- 1) .* eps), each step rounded
        if (jitter_u && e < c.E_router) {
            const float u = jitter_u[t * c.E_router + e];
            lg[j] = __fmul_rn(lg[j], __fadd_rn(1.0f, __fmul_rn(__fsub_rn(__fmul_rn(2.0f, u), 1.0f), eps)));
        }
        nl[j] = 0.f;
    }
    float lse2 = 0.f;
    double ent = 0.0;
    gate_token<NJ, false>(c, t, lg, nl, lane, s_cnt, s_psum[warp], lse2, ent);
}

template <int E_PAD, int BK, int KS, typename XT, int NI>
int launch_router_n(const RouterParams& p, int num_cta, cudaStream_t s) {
    auto kern = router_kernel<E_PAD, BK, KS, XT, NI>;
    const size_t smem = sizeof(RouterSmem<E_PAD, BK, KS, XT, NI>);
    // the attribute belongs to a (kernel, device) pair: one flag per instantiation and device
    static bool attr_done[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
        attr_done[dev] = true;
    }
    return launch_kernel(kern, dim3(num_cta), dim3(16 * (E_PAD / 8) * KS), smem, s, p) == cudaSuccess ? 1 : -1;
}

template <int E_PAD, int BK, int KS, typename XT>
int launch_router_t(const RouterParams& p, int num_cta, cudaStream_t s) {
    switch (p.tokens_per_cta) {
        case 64: return launch_router_n<E_PAD, BK, KS, XT, 4>(p, num_cta, s);
        case 32: return launch_router_n<E_PAD, BK, KS, XT, 2>(p, num_cta, s);
        case 16: return launch_router_n<E_PAD, BK, KS, XT, 1>(p, num_cta, s);
        default: return -1;
    }
}

template <int E_PAD, int BK, int KS>
int launch_router_e(const RouterParams& p, int x_dtype, int num_cta, cudaStream_t s) {
    if (x_dtype == MOE_DTYPE_F32) return launch_router_t<E_PAD, BK, KS, float>(p, num_cta, s);
    return launch_router_t<E_PAD, BK, KS, __nv_bfloat16>(p, num_cta, s);
}

}  // namespace

// Token tile of the router and permute kernels for a batch of T tokens: the largest of 64/32/16 that
// still gives enough CTAs.  A narrow router (at most 32 padded rows) is latency-bound and wants every
// SM to have a CTA; a wide one is bound by FMA issue and loses more from re-reading the router
// matrix for fewer tokens (66 rows, 32768 tokens: 0.53 ms with 64-token tiles, 0.73 ms with 32, 1.42
// ms with 16) than from idle SMs, so it keeps large tiles until a quarter of the SMs would be idle.
int router_tokens_per_cta(int64_t T, int e_router, int num_sms) {
    static int forced = -1;     // MOE_B200_ROUTER_TILE = 16 / 32 / 64 forces the tile (experiments)
    if (forced < 0) {
        const char* e = getenv("MOE_B200_ROUTER_TILE");
        const int v = e ? atoi(e) : 0;
        forced = (v == 16 || v == 32 || v == 64) ? v : 0;
    }
    if (forced > 0) return forced;
    const int64_t want = router_e_pad(e_router) <= 32 ? (int64_t)num_sms : (int64_t)num_sms * 3 / 4;
    for (int bt = ROUTER_TOKENS_PER_CTA; bt > 16; bt >>= 1)
        if ((T + bt - 1) / bt >= want) return bt;
    return 16;
}

// Router rows are padded to one of these widths (multiples of 8 = the per-thread row tile).
int router_e_pad(int e_router) {
    static const int buckets[] = {8, 16, 24, 32, 48, 64, 72, 80, 96, 128};
    for (int b : buckets)
        if (e_router <= b) return b;
    return 128;
}

int router_d_pad(int D) { return (D + 127) / 128 * 128; }

int launch_router_transpose(const float* w, float* wt, int E, int D, cudaStream_t s) {
    const int e_pad = router_e_pad(E), d_pad = router_d_pad(D);
    const size_t n = (size_t)e_pad * d_pad;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    router_transpose_kernel<<<blocks, 256, 0, s>>>(w, wt, E, D, e_pad, d_pad);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_router_transpose_noise(const float* w, const float* nw, float* wt, int E, int D, cudaStream_t s) {
    const int e_pad = router_e_pad(2 * E), d_pad = router_d_pad(D);
    const size_t n = (size_t)e_pad * d_pad;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    router_transpose_noise_kernel<<<blocks, 256, 0, s>>>(w, nw, wt, E, D, e_pad, d_pad);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_router(const RouterParams& p, int x_dtype, int num_cta, int num_sms, cudaStream_t s) {
    // <E_PAD, BK, KS>: 16 * E_PAD/8 * KS threads; with a noise network the GEMM is 2*E_router wide
    switch (router_e_pad(p.noise_off > 0 ? 2 * p.E_router : p.E_router)) {
        case 8: return launch_router_e<8, 128, 16>(p, x_dtype, num_cta, s);
        case 16: return launch_router_e<16, 128, 8>(p, x_dtype, num_cta, s);
        case 24: return launch_router_e<24, 128, 4>(p, x_dtype, num_cta, s);
        case 32: return launch_router_e<32, 128, 4>(p, x_dtype, num_cta, s);
        case 48: return launch_router_e<48, 64, 2>(p, x_dtype, num_cta, s);
        case 64: return launch_router_e<64, 64, 2>(p, x_dtype, num_cta, s);
        case 72: return launch_router_e<72, 64, 2>(p, x_dtype, num_cta, s);
        case 80: return launch_router_e<80, 32, 2>(p, x_dtype, num_cta, s);
        case 96: return launch_router_e<96, 32, 2>(p, x_dtype, num_cta, s);
        case 128: return launch_router_e<128, 32, 1>(p, x_dtype, num_cta, s);
        default: return -1;
    }
}

int launch_gates_only(int gate_kind, int E, int S, int k, int index_base, const float* logits, const float* jitter_u,
                      float eps, int64_t T, int32_t* indices, float* gates, float* probs, cudaStream_t s) {
    // Scratch-free variant: idx/gate go straight to the caller's arrays.
    GateCtx c;
    const bool shared = gate_kind == MOE_GATE_SHARED_TOPK;
    c.E_router = E;
    c.S = shared ? S : 0;
    c.r0 = c.S;
    c.k = (gate_kind == MOE_GATE_SWITCH) ? 1 : k;
    c.k_tot = c.S + c.k;
    c.E = E;
    c.E_probs = E;
    c.shared_mode = shared ? MOE_SHARED_GATING : MOE_SHARED_NONE;
    c.bias_gates_only = 0;
    c.index_base = index_base;
    c.want_entropy = 0;
    c.bias = nullptr;
    // the layer-internal arrays are the caller's arrays here, with the caller's index base
    c.idx_base = index_base;
    c.noise = nullptr;
    c.noise_scale = 0.f;
    c.noise_net = 0;
    c.idx = indices;
    c.gate = gates;
    c.u_idx = nullptr;
    c.u_gate = nullptr;
    c.u_probs = probs;
    c.u_logits = nullptr;
    const int blocks = (int)((T + ROUTER_WARPS - 1) / ROUTER_WARPS);
    gates_only_kernel<<<blocks, ROUTER_THREADS, 0, s>>>(c, logits, jitter_u, eps, T);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
