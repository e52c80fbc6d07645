// Scan + loss: one CTA turns the router's per-CTA histograms into (i) the exclusive prefix over
// CTAs that gives every (token, slot) pair a stable row in the permuted buffer, (ii) the
// per-expert row offsets and m-tile prefix the grouped GEMMs schedule from, and (iii) the
// Switch load-balancing loss, the z-loss and the routing entropy, reduced in a fixed order
// with warp shuffles so two runs are bit-identical.
//
// Replaces compute_loss(::SwitchTransformerLoss) and ZLoss (src/balancing/losses.jl:15-36,
// :103-114), the entropy of update_stats! (src/core/moe_layer.jl:250-264) and the GPU
// reductions of src/cuda/router.jl:73-99 (count_assignments_kernel!, three mapreduces).
#include "common.cuh"

namespace moe {
namespace {

constexpr int SCAN_THREADS = 1024;

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_loss_kernel(const ScanParams p) {
    __shared__ int s_count[MAX_EXPERTS];
    __shared__ float s_psum[MAX_EXPERTS + 1];
    __shared__ double s_ent;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NW = SCAN_THREADS / 32;
    chain_release();
    chain_wait();

    // (i) per expert: exclusive prefix of the per-CTA counts, in CTA (= token) order
    for (int e = warp; e < p.E; e += NW) {
        int run = 0;
        // eight independent loads in flight per lane, then the scans (the loads dominate: L2 latency)
        for (int c0 = 0; c0 < p.num_cta; c0 += 256) {
            int v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = c0 + j * 32 + lane;
                v[j] = (c < p.num_cta) ? p.cta_counts[(size_t)c * p.E + e] : 0;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = c0 + j * 32 + lane;
                const int inc = warp_incl_scan(v[j], lane);
                if (c < p.num_cta) p.cta_counts[(size_t)c * p.E + e] = run + inc - v[j];
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
        }
        // with a capacity constraint an expert keeps its first `capacity` pairs (token order)
        if (lane == 0) s_count[e] = (p.capacity >= 0 && run > p.capacity) ? p.capacity : run;
    }
    // per-expert probability sums (and the lse^2 sum in the last column): lanes stride the
    // CTAs, then a shuffle tree -- a fixed association order
    for (int e = warp; e <= p.E_probs; e += NW) {
        float s = 0.f;
        for (int c = lane; c < p.num_cta; c += 32) s += p.cta_psum[(size_t)c * (p.E_probs + 1) + e];
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) s_psum[e] = s;
    }
    if (warp == NW - 1) {
        double d = 0.0;
        for (int c = lane; c < p.num_cta; c += 32) d += p.cta_entropy[c];
#pragma unroll
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) s_ent = d;
    }
    __syncthreads();

    // (ii) offsets and tile prefix
    if (threadIdx.x == 0) {
        int off = 0, tiles = 0;
        for (int e = 0; e < p.E; ++e) {
            p.expert_offset[e] = off;
            p.tile_prefix[e] = tiles;
            p.expert_count[e] = s_count[e];
            off += s_count[e];
            tiles += (s_count[e] + p.tile_m - 1) / p.tile_m;
        }
        p.expert_offset[p.E] = off;
        p.tile_prefix[p.E] = tiles;
    }
    // sums_accumulate: this call is one chunk of a batch; chunks run in order on one stream, so the
    // running sums have a fixed order of additions
    const bool add = p.sums_accumulate != 0;
    for (int e = threadIdx.x; e < p.E; e += SCAN_THREADS)
        if (p.u_tokens_per_expert) p.u_tokens_per_expert[e] = (add ? p.u_tokens_per_expert[e] : 0) + (int64_t)s_count[e];
    if (p.ep_sums) {
        for (int e = threadIdx.x; e < p.E; e += SCAN_THREADS) p.ep_sums[e] = (add ? p.ep_sums[e] : 0.f) + (float)s_count[e];
        for (int e = threadIdx.x; e <= p.E_probs; e += SCAN_THREADS)
            p.ep_sums[p.E + e] = (add ? p.ep_sums[p.E + e] : 0.f) + s_psum[e];
        if (threadIdx.x == 0) {
            const int a = p.E + p.E_probs + 1;
            p.ep_sums[a] = (add ? p.ep_sums[a] : 0.f) + (float)p.T;
            p.ep_sums[a + 1] = (add ? p.ep_sums[a + 1] : 0.f) + (float)s_ent;
        }
    }

    if (p.ep_record) {
        for (int e = threadIdx.x; e < p.E; e += SCAN_THREADS) p.ep_record[e] = s_count[e];
        for (int e = threadIdx.x; e <= p.E_probs; e += SCAN_THREADS) p.ep_record[p.E + e] = __float_as_int(s_psum[e]);
        if (threadIdx.x == 0) {
            p.ep_record[p.E + p.E_probs + 1] = (int32_t)p.T;
            p.ep_record[p.E + p.E_probs + 2] = __float_as_int((float)s_ent);
        }
    }

    // (iii) loss = alpha * N * sum_i f_i P_i  (+ z_weight * mean lse^2), one warp
    if (warp == 0) {
        float acc = 0.f;
        const float inv_T = 1.0f / (float)p.T;
        if (p.shared_mode == MOE_SHARED_LAYER_BLEND) {
            // The reference counts ids shifted by +S against probabilities that only have
            // E-S rows (src/core/moe_layer.jl:172,182 with losses.jl:16,23): row j gets the
            // count of layer expert j, for S <= j < E-S; the denominator is k*T.
            const float denom = (float)((double)p.k * (double)p.T);
            for (int j = p.S + lane; j < p.E_probs; j += 32) {
                const float f = (float)s_count[j] / denom;
                acc += f * (s_psum[j] * inv_T);
            }
        } else {
            const float denom = (float)((double)p.k_tot * (double)p.T);
            for (int j = lane; j < p.E_probs; j += 32) {
                const float f = (float)s_count[j] / denom;
                acc += f * (s_psum[j] * inv_T);
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            float loss = 0.f;
            if (p.training) {
                loss = p.alpha * (float)p.E_probs * acc;
                if (p.z_weight > 0.f) loss += p.z_weight * (s_psum[p.E_probs] * inv_T);
            }
            *p.loss_internal = loss;
            if (p.u_loss) *p.u_loss = loss;
            if (p.u_entropy) *p.u_entropy = (float)(s_ent / (double)p.T);
        }
    }
}

// Stand-alone compute_loss on caller-provided indices/probs(/logits): one CTA.
__global__ void __launch_bounds__(SCAN_THREADS) loss_only_kernel(float alpha, float z_weight, int n_probs, int k,
                                                                 int index_base, const int32_t* indices,
                                                                 const float* probs, const float* logits,
                                                                 int n_logits, int64_t T, float* loss) {
    __shared__ int s_count[MAX_EXPERTS];
    __shared__ float s_p[MAX_EXPERTS];
    __shared__ float s_z[SCAN_THREADS / 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NW = SCAN_THREADS / 32;
    for (int i = threadIdx.x; i < MAX_EXPERTS; i += SCAN_THREADS) s_count[i] = 0;
    __syncthreads();
    for (int64_t i = threadIdx.x; i < T * k; i += SCAN_THREADS) {
        const int id = indices[i] - index_base;   // ids outside 1..N are skipped by the reference
        if (id >= 0 && id < n_probs) atomicAdd(&s_count[id], 1);
    }
    for (int e = warp; e < n_probs; e += NW) {
        float s = 0.f;
        for (int64_t t = lane; t < T; t += 32) s += probs[t * n_probs + e];
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) s_p[e] = s;
    }
    float z = 0.f;
    if (logits) {
        for (int64_t t = threadIdx.x; t < T; t += SCAN_THREADS) {
            float m = -3.4e38f;
            for (int e = 0; e < n_logits; ++e) m = fmaxf(m, logits[t * n_logits + e]);
            float s = 0.f;
            for (int e = 0; e < n_logits; ++e) s += expf(logits[t * n_logits + e] - m);
            const float lse = m + logf(s);
            z += lse * lse;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    if (lane == 0) s_z[warp] = z;
    __syncthreads();
    if (warp == 0) {
        float acc = 0.f;
        const float denom = (float)((double)k * (double)T);
        for (int j = lane; j < n_probs; j += 32) acc += ((float)s_count[j] / denom) * (s_p[j] / (float)T);
        float zz = s_z[lane];
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
            zz += __shfl_xor_sync(0xffffffffu, zz, o);
        }
        if (lane == 0) {
            float l = alpha * (float)n_probs * acc;
            if (logits && z_weight > 0.f) l += z_weight * (zz / (float)T);
            *loss = l;
        }
    }
}

// update_bias! (src/balancing/auxiliary_free.jl:36-71) from this call's per-expert counts.  One
// block; thread e owns expert e.  Arithmetic types follow Julia's promotion: the gradient and the
// momentum blend are Float64 (Int/Int target), rounded into the Float32 vectors; the bias step and
// the mean-centring are Float32.
__global__ void aux_free_update_kernel(const int32_t* expert_count, int E, float* bias, float* bias_momentum,
                                       float learning_rate, float momentum) {
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ float s_bias[MAX_EXPERTS];
    __shared__ long long s_total;
    __shared__ float s_mean;
    const int e = threadIdx.x;
    if (e < E) s_cnt[e] = expert_count[e];
    __syncthreads();
    if (e == 0) {
        long long t = 0;
        for (int i = 0; i < E; ++i) t += s_cnt[i];
        s_total = t;
    }
    __syncthreads();
    const long long total = s_total;
    if (total == 0) return;
    if (e < E) {
        const double target = (double)total / (double)E;
        const double grad = ((double)(float)s_cnt[e] - target) / (double)total;
        const float keep = __fmul_rn(momentum, bias_momentum[e]);
        const float bm = (float)((double)keep + (double)__fsub_rn(1.0f, momentum) * grad);
        bias_momentum[e] = bm;
        s_bias[e] = __fsub_rn(bias[e], __fmul_rn(learning_rate, bm));
    }
    __syncthreads();
    if (e == 0) {
        float sum = 0.f;
        for (int i = 0; i < E; ++i) sum = __fadd_rn(sum, s_bias[i]);
        s_mean = __fdiv_rn(sum, (float)E);
    }
    __syncthreads();
    if (e < E) bias[e] = __fsub_rn(s_bias[e], s_mean);
}

}  // namespace

int launch_aux_free_update(const int32_t* expert_count, int E, float* bias, float* bias_momentum, float learning_rate,
                           float momentum, cudaStream_t s) {
    aux_free_update_kernel<<<1, MAX_EXPERTS, 0, s>>>(expert_count, E, bias, bias_momentum, learning_rate, momentum);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_scan(const ScanParams& p, cudaStream_t s) {
    launch_kernel(scan_loss_kernel, dim3(1), dim3(SCAN_THREADS), 0, s, p);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_loss_only(float alpha, float z_weight, int n_probs, int k, int index_base, const int32_t* indices,
                     const float* probs, const float* logits, int n_logits, int64_t T, float* loss,
                     cudaStream_t s) {
    loss_only_kernel<<<1, SCAN_THREADS, 0, s>>>(alpha, z_weight, n_probs, k, index_base, indices, probs, logits,
                                                n_logits, T, loss);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
