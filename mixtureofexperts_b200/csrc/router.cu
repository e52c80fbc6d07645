// Fused router: gate GEMM (FP32, lane-split K for a short rounding chain) -> softmax -> top-k
// (k arg-max passes, ties to the lowest index) -> renormalised gates -> per-CTA expert
// histogram and per-CTA partial sums for the Switch loss, the z-loss and the routing entropy.
//
// Replaces Router.__call__ + compute_gates of the reference (src/core/router.jl:25-46,
// src/gating/topk.jl:24-44, src/gating/advanced.jl:80-108) and its GPU kernels
// (src/cuda/router.jl:5-71, src/cuda/kernels.jl:3-58).
//
// Bound: HBM (reads x once: T*D*sizeof(x); everything else is O(T*E)).
#include "common.cuh"

#include <cfloat>
#include <climits>

namespace moe {

namespace {

struct GateCtx {
    int E_router;     // columns of the incoming logits
    int r0;           // first routed column (S in GATING mode, else 0)
    int S, k, k_tot, E, E_probs;
    int shared_mode, bias_gates_only, index_base, want_entropy;
    int idx_base;     // base added to the ids stored through `idx` (0 inside the layer)
    const float* bias;
    int32_t* idx;
    float* gate;
    int32_t* u_idx;
    float* u_gate;
    float* u_probs;
    float* u_logits;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One token, one warp.  lg[j] is the raw logit of router column lane + 32*j.
// Accumulators (per warp, lane-owned columns): s_psum[e] += prob, returns lse^2 and entropy.
template <int NJ>
__device__ __forceinline__ void gate_token(const GateCtx& c, int64_t t, const float (&lg_in)[NJ], int lane,
                                           int* s_cnt, float* s_psum, float& lse2_acc, double& ent_acc) {
    float lsel[NJ], lprob[NJ];
    bool valid[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        const bool in = e < c.E_router;
        const float b = (in && c.bias) ? c.bias[e] : 0.f;
        lsel[j] = lg_in[j] + b;
        lprob[j] = c.bias_gates_only ? lg_in[j] : lsel[j];
        valid[j] = in && e >= c.r0;
        if (in && c.u_logits) c.u_logits[t * c.E_router + e] = lprob[j];
    }
    // logsumexp over every router column (src/balancing/losses.jl:103-114)
    {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < c.E_router) m = fmaxf(m, lprob[j]);
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < c.E_router) s += expf(lprob[j] - m);
        s = warp_sum(s);
        const float lse = m + logf(s);
        lse2_acc += lse * lse;
    }
    // softmax over the routed columns (NNlib.softmax: subtract max, exp, divide by the sum)
    float pr[NJ], psel[NJ];
    {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (valid[j]) m = fmaxf(m, lprob[j]);
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            pr[j] = valid[j] ? expf(lprob[j] - m) : 0.f;
            s += pr[j];
        }
        s = warp_sum(s);
#pragma unroll
        for (int j = 0; j < NJ; ++j) pr[j] = pr[j] / s;
    }
    if (c.bias && c.bias_gates_only) {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (valid[j]) m = fmaxf(m, lsel[j]);
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            psel[j] = valid[j] ? expf(lsel[j] - m) : 0.f;
            s += psel[j];
        }
        s = warp_sum(s);
#pragma unroll
        for (int j = 0; j < NJ; ++j) psel[j] = psel[j] / s;
    } else {
#pragma unroll
        for (int j = 0; j < NJ; ++j) psel[j] = pr[j];
    }
    // top-k of the probabilities: k passes of arg-max; among equal values the lowest column
    // wins (Base.partialsortperm rev=true is stable; src/cuda/kernels.jl:24 uses strict '>').
    bool taken[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) taken[j] = false;
    float my_v = 0.f;
    int my_i = 0;
    for (int s = 0; s < c.k; ++s) {
        float best = -2.f;
        int bi = INT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            // a NaN probability ranks below every number but stays selectable
            const float v = (psel[j] == psel[j]) ? psel[j] : -1.f;
            if (valid[j] && !taken[j] && v > best) {
                best = v;
                bi = lane + 32 * j;
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j == bi) taken[j] = true;
        if (lane == s) {
            my_v = best < 0.f ? nanf("") : best;
            my_i = bi;
        }
    }
    // gates = selected / sum(selected), summed in slot order like the reference
    float gsum = 0.f;
    for (int s = 0; s < c.k; ++s) gsum += __shfl_sync(0xffffffffu, my_v, s);
    const float g = my_v / gsum;

    const int n_shared_slots = (c.shared_mode == MOE_SHARED_NONE) ? 0 : c.S;
    if (lane < c.k && my_i != INT_MAX) {
        const int layer_id = my_i + (c.shared_mode == MOE_SHARED_LAYER_BLEND ? c.S : 0);
        float gi = g;
        if (c.shared_mode == MOE_SHARED_GATING) gi = (float)((double)g * (1.0 - (double)c.S / (double)c.k_tot));
        if (c.shared_mode == MOE_SHARED_LAYER_BLEND) gi = 0.5f * g;
        const int slot = n_shared_slots + lane;
        if (c.idx) c.idx[t * c.k_tot + slot] = layer_id + c.idx_base;
        if (c.gate) c.gate[t * c.k_tot + slot] = gi;
        atomicAdd(&s_cnt[layer_id], 1);
        if (c.shared_mode == MOE_SHARED_LAYER_BLEND) {
            if (c.u_idx) c.u_idx[t * c.k + lane] = layer_id + c.index_base;
            if (c.u_gate) c.u_gate[t * c.k + lane] = g;
        } else {
            if (c.u_idx) c.u_idx[t * c.k_tot + slot] = layer_id + c.index_base;
            if (c.u_gate) c.u_gate[t * c.k_tot + slot] = gi;
        }
    }
    if (lane < n_shared_slots) {
        const float gs = (c.shared_mode == MOE_SHARED_GATING) ? 1.0f / (float)c.k_tot : 0.5f / (float)c.S;
        if (c.idx) c.idx[t * c.k_tot + lane] = lane + c.idx_base;
        if (c.gate) c.gate[t * c.k_tot + lane] = gs;
        atomicAdd(&s_cnt[lane], 1);
        if (c.shared_mode == MOE_SHARED_GATING) {
            if (c.u_idx) c.u_idx[t * c.k_tot + lane] = lane + c.index_base;
            if (c.u_gate) c.u_gate[t * c.k_tot + lane] = gs;
        }
    }
    // probabilities as the reference returns them, their per-expert sums, and the entropy
    double ent = 0.0;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        if (e < c.E_probs) {
            float pv;
            if (c.shared_mode == MOE_SHARED_GATING) {
                pv = (e < c.S) ? 1.0f / (float)c.E
                               : (float)((double)pr[j] * (1.0 - (double)c.S / (double)c.E));
            } else {
                pv = pr[j];
            }
            if (c.u_probs) c.u_probs[t * c.E_probs + e] = pv;
            s_psum[e] += pv;
            if (c.want_entropy) ent -= (double)pv * log((double)pv + 1e-8);
        }
    }
    if (c.want_entropy) ent_acc += warp_sum_d(ent);
}

template <typename XT>
__device__ __forceinline__ float4 load_x4(const XT* row, int kk, int D, bool vec);

template <>
__device__ __forceinline__ float4 load_x4<float>(const float* row, int kk, int D, bool vec) {
    if (vec && kk + 3 < D) return *reinterpret_cast<const float4*>(row + kk);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kk + 0 < D) v.x = row[kk + 0];
    if (kk + 1 < D) v.y = row[kk + 1];
    if (kk + 2 < D) v.z = row[kk + 2];
    if (kk + 3 < D) v.w = row[kk + 3];
    return v;
}
template <>
__device__ __forceinline__ float4 load_x4<__nv_bfloat16>(const __nv_bfloat16* row, int kk, int D, bool vec) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vec && kk + 3 < D) {
        const uint2 u = *reinterpret_cast<const uint2*>(row + kk);
        v.x = __uint_as_float(u.x << 16);
        v.y = __uint_as_float(u.x & 0xffff0000u);
        v.z = __uint_as_float(u.y << 16);
        v.w = __uint_as_float(u.y & 0xffff0000u);
        return v;
    }
    if (kk + 0 < D) v.x = __bfloat162float(row[kk + 0]);
    if (kk + 1 < D) v.y = __bfloat162float(row[kk + 1]);
    if (kk + 2 < D) v.z = __bfloat162float(row[kk + 2]);
    if (kk + 3 < D) v.w = __bfloat162float(row[kk + 3]);
    return v;
}

__device__ __forceinline__ GateCtx make_ctx(const RouterParams& p) {
    GateCtx c;
    c.E_router = p.E_router;
    c.r0 = (p.shared_mode == MOE_SHARED_GATING) ? p.S : 0;
    c.S = p.S;
    c.k = p.k;
    c.k_tot = p.k_tot;
    c.E = p.E;
    c.E_probs = p.E_probs;
    c.shared_mode = p.shared_mode;
    c.bias_gates_only = p.bias_gates_only;
    c.index_base = p.index_base;
    c.want_entropy = p.want_entropy;
    c.idx_base = 0;
    c.bias = p.bias;
    c.idx = p.idx;
    c.gate = p.gate;
    c.u_idx = p.u_idx;
    c.u_gate = p.u_gate;
    c.u_probs = p.u_probs;
    c.u_logits = p.u_logits;
    return c;
}

// E_MAX: compile-time bound on router rows; TP: tokens a warp carries through the K loop.
template <int E_MAX, int TP, typename XT>
__global__ void __launch_bounds__(ROUTER_THREADS) router_kernel(const RouterParams p) {
    extern __shared__ float4 s_w[];  // [E_router][KC/4]
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_psum[ROUTER_WARPS][MAX_EXPERTS];
    __shared__ float s_lse2[ROUTER_WARPS];
    __shared__ double s_ent[ROUTER_WARPS];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < MAX_EXPERTS; i += ROUTER_THREADS) s_cnt[i] = 0;
    for (int i = threadIdx.x; i < ROUTER_WARPS * MAX_EXPERTS; i += ROUTER_THREADS) (&s_psum[0][0])[i] = 0.f;

    const int64_t tok0 = (int64_t)blockIdx.x * p.tokens_per_cta + (int64_t)warp * TP;
    const XT* x = reinterpret_cast<const XT*>(p.x);
    const bool vec_x = (p.D % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
    const bool vec_w = (p.D % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.w) & 15) == 0);

    float acc[TP][E_MAX];
#pragma unroll
    for (int a = 0; a < TP; ++a)
#pragma unroll
        for (int e = 0; e < E_MAX; ++e) acc[a][e] = 0.f;

    for (int kc = 0; kc < p.D; kc += ROUTER_KC) {
        __syncthreads();
        for (int i = threadIdx.x; i < p.E_router * (ROUTER_KC / 4); i += ROUTER_THREADS) {
            const int e = i / (ROUTER_KC / 4), c4 = i % (ROUTER_KC / 4);
            s_w[i] = load_x4<float>(p.w + (size_t)e * p.D, kc + c4 * 4, p.D, vec_w);
        }
        __syncthreads();
        float4 xv[TP];
#pragma unroll
        for (int a = 0; a < TP; ++a) {
            const int64_t t = tok0 + a;
            xv[a] = (t < p.T) ? load_x4<XT>(x + (size_t)t * p.D, kc + lane * 4, p.D, vec_x)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int e = 0; e < E_MAX; ++e) {
            if (e < p.E_router) {
                const float4 wv = s_w[e * (ROUTER_KC / 4) + lane];
#pragma unroll
                for (int a = 0; a < TP; ++a) {
                    float s = acc[a][e];
                    s = fmaf(xv[a].x, wv.x, s);
                    s = fmaf(xv[a].y, wv.y, s);
                    s = fmaf(xv[a].z, wv.z, s);
                    s = fmaf(xv[a].w, wv.w, s);
                    acc[a][e] = s;
                }
            }
        }
    }
    // butterfly all-reduce: every lane ends with the same full dot products
#pragma unroll
    for (int a = 0; a < TP; ++a)
#pragma unroll
        for (int e = 0; e < E_MAX; ++e) {
            if (e < p.E_router) {
                float v = acc[a][e];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[a][e] = v;
            }
        }

    const GateCtx c = make_ctx(p);
    constexpr int NJ = (E_MAX + 31) / 32;
    float lse2 = 0.f;
    double ent = 0.0;
#pragma unroll
    for (int a = 0; a < TP; ++a) {
        const int64_t t = tok0 + a;
        if (t < p.T) {
            float lg[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) lg[j] = 0.f;
#pragma unroll
            for (int e = 0; e < E_MAX; ++e)
                if ((e & 31) == lane) lg[e >> 5] = acc[a][e];
            gate_token<NJ>(c, t, lg, lane, s_cnt, s_psum[warp], lse2, ent);
        }
    }
    if (lane == 0) {
        s_lse2[warp] = lse2;
        s_ent[warp] = ent;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < p.E; e += ROUTER_THREADS) p.cta_counts[(size_t)blockIdx.x * p.E + e] = s_cnt[e];
    for (int e = threadIdx.x; e < p.E_probs; e += ROUTER_THREADS) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < ROUTER_WARPS; ++w) s += s_psum[w][e];
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + e] = s;
    }
    if (threadIdx.x == 0) {
        float s = 0.f;
        double d = 0.0;
        for (int w = 0; w < ROUTER_WARPS; ++w) {
            s += s_lse2[w];
            d += s_ent[w];
        }
        p.cta_psum[(size_t)blockIdx.x * (p.E_probs + 1) + p.E_probs] = s;
        p.cta_entropy[blockIdx.x] = d;
    }
}

// compute_gates as a stand-alone operator on given logits: one warp per token.
__global__ void __launch_bounds__(ROUTER_THREADS) gates_only_kernel(GateCtx c, const float* logits, int64_t T) {
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_psum[ROUTER_WARPS][MAX_EXPERTS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * ROUTER_WARPS + warp;
    if (t >= T) return;
    constexpr int NJ = MAX_ROUTER_EXPERTS / 32;
    float lg[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        lg[j] = (e < c.E_router) ? logits[t * c.E_router + e] : 0.f;
    }
    float lse2 = 0.f;
    double ent = 0.0;
    gate_token<NJ>(c, t, lg, lane, s_cnt, s_psum[warp], lse2, ent);
}

template <int E_MAX, int TP>
int launch_router_t(const RouterParams& p, int x_dtype, int num_cta, cudaStream_t s) {
    const size_t smem = (size_t)p.E_router * ROUTER_KC * sizeof(float);
    cudaError_t err;
    if (x_dtype == MOE_DTYPE_F32) {
        auto kern = router_kernel<E_MAX, TP, float>;
        if (smem > 32 * 1024) {
            err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess) return -1;
        }
        kern<<<num_cta, ROUTER_THREADS, smem, s>>>(p);
    } else {
        auto kern = router_kernel<E_MAX, TP, __nv_bfloat16>;
        if (smem > 32 * 1024) {
            err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess) return -1;
        }
        kern<<<num_cta, ROUTER_THREADS, smem, s>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int tokens_per_pass(int e_router) {
    if (e_router <= 16) return 8;
    if (e_router <= 32) return 4;
    if (e_router <= 72) return 2;
    return 1;
}

}  // namespace

int router_tokens_per_cta(int e_router) { return ROUTER_WARPS * tokens_per_pass(e_router); }

int launch_router(const RouterParams& p, int x_dtype, int num_cta, cudaStream_t s) {
    const int e = p.E_router;
    if (e <= 8) return launch_router_t<8, 8>(p, x_dtype, num_cta, s);
    if (e <= 16) return launch_router_t<16, 8>(p, x_dtype, num_cta, s);
    if (e <= 32) return launch_router_t<32, 4>(p, x_dtype, num_cta, s);
    if (e <= 64) return launch_router_t<64, 2>(p, x_dtype, num_cta, s);
    if (e <= 72) return launch_router_t<72, 2>(p, x_dtype, num_cta, s);
    return launch_router_t<128, 1>(p, x_dtype, num_cta, s);
}

int launch_gates_only(int gate_kind, int E, int S, int k, int index_base, const float* logits, int64_t T,
                      int32_t* indices, float* gates, float* probs, cudaStream_t s) {
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
    c.idx = indices;
    c.gate = gates;
    c.u_idx = nullptr;
    c.u_gate = nullptr;
    c.u_probs = probs;
    c.u_logits = nullptr;
    const int blocks = (int)((T + ROUTER_WARPS - 1) / ROUTER_WARPS);
    gates_only_kernel<<<blocks, ROUTER_THREADS, 0, s>>>(c, logits, T);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
