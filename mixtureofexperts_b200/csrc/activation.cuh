// Activations of GatedExpert (MoEConfig.activation, src/core/moe_layer.jl:10;
// silu: src/experts/gated.jl:36 and src/llama2/inference.jl:159-162).
#pragma once
#include "common.cuh"

namespace moe {

__device__ __forceinline__ float apply_act(int act, float v) {
    switch (act) {
        case MOE_ACT_SILU:
            return v * (1.0f / (1.0f + expf(-v)));
        case MOE_ACT_GELU_TANH: {
            const float c = 0.7978845608028654f;  // sqrt(2/pi)
            return 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
        }
        case MOE_ACT_RELU:
            return fmaxf(v, 0.f);
        default:
            return v;
    }
}

// Binary search in a non-decreasing prefix array: largest e in [0, E) with prefix[e] <= v.
__device__ __forceinline__ int find_segment(const int32_t* prefix, int E, int v) {
    int lo = 0, hi = E;  // invariant: prefix[lo] <= v < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= v) lo = mid; else hi = mid;
    }
    return lo;
}

}  // namespace moe
