// Gating of one token by one warp, shared by the router kernels: softmax -> top-k (k arg-max
// passes, ties to the lowest index) -> renormalised gates -> histogram and partial sums for the
// Switch loss, the z-loss and the routing entropy.  Restates compute_gates of the reference
// (src/gating/topk.jl:24-44, src/gating/advanced.jl:80-108) and the noise / bias handling of
// Router and forward_standard (src/core/router.jl:32-41, src/core/moe_layer.jl:137-140).
#pragma once
#include <cfloat>
#include <climits>

#include "common.cuh"

namespace moe {
namespace gating {

struct GateCtx {
    int E_router;     // columns of the incoming logits
    int r0;           // first routed column (S in GATING mode, else 0)
    int S, k, k_tot, E, E_probs;
    int shared_mode, bias_gates_only, index_base, want_entropy;
    int idx_base;     // base added to the ids stored through `idx` (0 inside the layer)
    const float* noise;   // [T][E_router] standard-normal draws or null; scaled by noise_scale
    float noise_scale;
    int noise_net;        // draws are multiplied by softplus(noise-network logit) (src/core/router.jl:34-37)
    const float* bias;
    int32_t* idx;
    float* gate;
    int32_t* u_idx;
    float* u_gate;
    float* u_probs;
    float* u_logits;
};

// Reductions over groups of W consecutive lanes (W = 32: the whole warp).
template <int W = 32>
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = W / 2; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int W = 32>
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = W / 2; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Sum over the 32 / W lanes that hold the same column of different tokens (offsets W, 2W, ...).
template <int W>
__device__ __forceinline__ float across_tokens_sum(float v) {
#pragma unroll
    for (int o = W; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One token per group of W lanes (W = 32: one token per warp; W = 8 or 16, for routers of at most W
// columns: 4 or 2 tokens per warp side by side, NJ = 1).  lg[j] is the raw logit of router column
// (lane % W) + 32*j of the group's token `t`; `active` is false for a group past the last token: it
// runs along (the warp's shuffles need every lane) but leaves no trace.
// Accumulators (per warp, lane-owned columns): s_psum[e] += prob, returns lse^2 and entropy.
//
// PROBE = true (tensor-core router): the logits carry a rounding error of about 1.5e-6 times their
// scale, so the ranking is looked at before anything is written: one extra arg-max pass finds the
// (k+1)-th probability, and if two neighbours of the top k+1 are closer than probe_rel * max(1,
// largest |logit|) -- relative differences of probabilities are differences of logits -- the function
// returns false WITHOUT side effects and the caller gates the token again from exact logits.
template <int NJ, bool PROBE, int W = 32>
__device__ __forceinline__ bool gate_token(const GateCtx& c, int64_t t, const float (&lg_in)[NJ], const float (&nl)[NJ], int lane_in_warp,
                                           int* s_cnt, float* s_psum, float& lse2_acc, double& ent_acc, float probe_rel = 0.f,
                                           bool active = true) {
    static_assert(W == 32 || (NJ == 1 && !PROBE && (W == 8 || W == 16)), "several tokens per warp: narrow routers only");
    constexpr unsigned FULL = 0xffffffffu;
    const int lane = lane_in_warp % W;                     // column owner inside the token's lane group
    const unsigned GROUP = W == 32 ? FULL : (((1u << (W % 32)) - 1u) << ((lane_in_warp / W) * W));
    // Training-time router noise (src/core/router.jl:32-41): logits + noise_scale * randn (times
    // softplus(noise_weight x) when the router has a noise network, nl[] = those logits) feed the
    // gate and are the logits the router returns; the z-loss is computed by a second, noise-free
    // router pass in the reference (src/core/moe_layer.jl:117-121), hence from the clean logits.
    float lsel[NJ], lprob[NJ], lclean[NJ];
    bool valid[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        const bool in = e < c.E_router;
        const float b = (in && c.bias) ? c.bias[e] : 0.f;
        float nz = 0.f;
        if (in && c.noise && active) {
            float draw = c.noise[t * c.E_router + e];
            // NNlib.softplus(x) = log1p(exp(-|x|)) + relu(x)
            if (c.noise_net) draw *= log1pf(expf(-fabsf(nl[j]))) + fmaxf(nl[j], 0.f);
            nz = c.noise_scale * draw;
        }
        const float noisy = lg_in[j] + nz;
        lsel[j] = noisy + b;
        lprob[j] = c.bias_gates_only ? noisy : lsel[j];
        lclean[j] = c.bias_gates_only ? lg_in[j] : lg_in[j] + b;
        valid[j] = in && e >= c.r0;
    }
    // softmax over the routed columns (NNlib.softmax: subtract max, exp, divide by the sum)
    float pr[NJ], psel[NJ];
    float soft_m, soft_s;   // maximum and sum of exponentials of the probability softmax
    {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (valid[j]) m = fmaxf(m, lprob[j]);
        m = warp_max<W>(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            pr[j] = valid[j] ? expf(lprob[j] - m) : 0.f;
            s += pr[j];
        }
        s = warp_sum<W>(s);
        soft_m = m;
        soft_s = s;
#pragma unroll
        for (int j = 0; j < NJ; ++j) pr[j] = pr[j] / s;
    }
    if (c.bias && c.bias_gates_only) {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (valid[j]) m = fmaxf(m, lsel[j]);
        m = warp_max<W>(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            psel[j] = valid[j] ? expf(lsel[j] - m) : 0.f;
            s += psel[j];
        }
        s = warp_sum<W>(s);
#pragma unroll
        for (int j = 0; j < NJ; ++j) psel[j] = psel[j] / s;
    } else {
#pragma unroll
        for (int j = 0; j < NJ; ++j) psel[j] = pr[j];
    }
    // top-k of the probabilities: k passes of arg-max; among equal values the lowest column
    // wins (Base.partialsortperm rev=true is stable; src/cuda/kernels.jl:24 uses strict '>').
    // A probability is >= 0, so its bit pattern orders like a signed integer; a NaN probability is
    // keyed as -1.0f: it ranks below every number but stays selectable.  Two warp reductions per
    // pass: the largest key, then the lowest column that holds it.
    int key[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const float v = (psel[j] == psel[j]) ? psel[j] : -1.f;
        key[j] = valid[j] ? __float_as_int(v) : INT_MIN;
    }
    float my_v = 0.f;
    int my_i = 0;
    float prev = 0.f;
    bool close = false;
    const int passes = PROBE ? min(c.k + 1, c.E_router - c.r0) : c.k;
    for (int s = 0; s < passes; ++s) {
        int bk = INT_MIN, bj = 0;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (key[j] > bk) {
                bk = key[j];
                bj = j;
            }
        const int m = __reduce_max_sync(GROUP, bk);
        int bi = __reduce_min_sync(GROUP, (bk == m && m != INT_MIN) ? lane + 32 * bj : INT_MAX);
        const float best = m == INT_MIN ? -2.f : __int_as_float(m);
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j == bi) key[j] = INT_MIN;
        if (PROBE) {
            if (s > 0 && !(prev - best >= probe_rel * prev)) close = true;
            prev = best;
            if (s == c.k) break;          // the (k+1)-th value was only needed for the comparison
        }
        if (lane == s) {
            my_v = best < 0.f ? nanf("") : best;
            my_i = bi;
        }
    }
    if (PROBE && close) return false;

#pragma unroll
    for (int j = 0; j < NJ; ++j)
        if (active && lane + 32 * j < c.E_router && c.u_logits) c.u_logits[t * c.E_router + lane + 32 * j] = lprob[j];
    // logsumexp over every router column (src/balancing/losses.jl:103-114).  Without noise, without a
    // gates-only bias and with every column routed, these are the logits of the softmax above: its
    // maximum and sum are the same numbers, computed the same way.
    if (c.r0 == 0 && !c.noise && !(c.bias && c.bias_gates_only)) {
        const float lse = soft_m + logf(soft_s);
        lse2_acc += across_tokens_sum<W>(active ? lse * lse : 0.f);
    } else {
        float m = -FLT_MAX;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < c.E_router) m = fmaxf(m, lclean[j]);
        m = warp_max<W>(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < c.E_router) s += expf(lclean[j] - m);
        s = warp_sum<W>(s);
        const float lse = m + logf(s);
        lse2_acc += across_tokens_sum<W>(active ? lse * lse : 0.f);
    }
    // gates = selected / sum(selected), summed in slot order like the reference
    float gsum = 0.f;
    for (int s = 0; s < c.k; ++s) gsum += __shfl_sync(FULL, my_v, s, W);
    const float g = my_v / gsum;

    const int n_shared_slots = (c.shared_mode == MOE_SHARED_NONE) ? 0 : c.S;
    if (active && lane < c.k && my_i != INT_MAX) {
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
    if (active && lane < n_shared_slots) {
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
    // -sum p log(p + 1e-8) (src/core/moe_layer.jl:262: Float64 there because of the literal; FP32 here
    // agrees with it to ~1e-7 relative, the per-token sums are then accumulated in double)
    float ent = 0.f;
    const float shared_scale = (float)(1.0 - (double)c.S / (double)c.E);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        const bool has = e < c.E_probs;
        float pv = 0.f;
        if (has && active) {
            if (c.shared_mode == MOE_SHARED_GATING) {
                pv = (e < c.S) ? 1.0f / (float)c.E
                               : (float)((double)pr[j] * (1.0 - (double)c.S / (double)c.E));
            } else {
                pv = pr[j];
            }
            if (c.u_probs) c.u_probs[t * c.E_probs + e] = pv;
            if (c.want_entropy) ent -= pv * logf(pv + 1e-8f);
        }
        if (W == 32) {
            if (has) s_psum[e] += pv;
        } else {
            const float all = across_tokens_sum<W>(pv);      // the warp's tokens, always in the same order
            if (has && lane_in_warp < W) s_psum[e] += all;
        }
    }
    (void)shared_scale;
    if (c.want_entropy) ent_acc += (double)warp_sum<32>(ent);
    return true;
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
    c.noise = p.noise;
    c.noise_scale = p.noise_scale;
    c.noise_net = p.noise_off > 0;
    c.bias = p.bias;
    c.idx = p.idx;
    c.gate = p.gate;
    c.u_idx = p.u_idx;
    c.u_gate = p.u_gate;
    c.u_probs = p.u_probs;
    c.u_logits = p.u_logits;
    return c;
}

}  // namespace gating
}  // namespace moe
