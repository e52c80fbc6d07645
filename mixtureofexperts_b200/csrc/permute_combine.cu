// Token permute (dispatch) and weighted un-permute (combine).
//
// permute: every (token, slot) pair gets row  expert_offset[e] + (pairs of e in earlier CTAs) +
// (rank inside this CTA's token tile)  -- the ascending-token order of the reference's bucket
// pass (process_expert_forward!, src/core/moe_layer.jl:195-203) -- and the token's D-vector is
// copied there with 16-byte loads/stores: each token row is read once and written k_tot times.
// HBM bound: T*D*sizeof(x) read + pairs*D*sizeof(xp) written.
//
// combine: out[t] = sum over the token's slots, in ascending expert id (the order in which
// the reference's expert loop adds into a token, moe_layer.jl:205-218), of gate * y[row].
// Gather-style: every output element is written exactly once, no atomics, no memset
// (replaces apply_gates_kernel!, src/cuda/kernels.jl:60-81, launched E times with a device
// sync after each, and the zero fill of src/cuda/experts.jl:36).
// HBM bound: pairs*O*sizeof(y) read + T*O*4 written.
#include "common.cuh"
#include "permute_rows.cuh"

namespace moe {
namespace {

constexpr int PERM_THREADS = 256;
constexpr int PERM_MAX_PAIRS = 64 * MAX_KTOT;  // tokens_per_cta <= 64

using namespace rows;

template <typename XT, typename PT>
__global__ void __launch_bounds__(PERM_THREADS) permute_kernel(const PermuteParams p) {
    __shared__ int s_base[MAX_EXPERTS];
    __shared__ int s_pos[PERM_MAX_PAIRS];
    __shared__ int s_exp[PERM_MAX_PAIRS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tok0 = (int64_t)blockIdx.x * p.tokens_per_cta;
    const int ntok = (int)min((int64_t)p.tokens_per_cta, p.T - tok0);
    const int npairs = ntok * p.k_tot;
    chain_release();
    chain_wait();

    // s_base[e]: rank, inside expert e, of the first pair of this tile (pairs of earlier tiles)
    for (int e = threadIdx.x; e < p.E; e += PERM_THREADS) s_base[e] = p.cta_base[(size_t)blockIdx.x * p.E + e];
    __syncthreads();

    if (warp == 0) {
        // rank of each pair among the tile's pairs of the same expert, in (token, slot) order
        for (int q0 = 0; q0 < npairs; q0 += 32) {
            const int q = q0 + lane;
            const bool act = q < npairs;
            const int e = act ? p.idx[tok0 * p.k_tot + q] : -1 - lane;  // inactive lanes never match
            const unsigned m = __match_any_sync(0xffffffffu, e);
            const int rank = __popc(m & ((1u << lane) - 1u));
            int pos = -1;
            bool dropped = false;
            if (act && e >= 0 && e < p.E) {
                const int r = s_base[e] + rank;                      // rank inside the expert, token order
                dropped = p.capacity >= 0 && r >= p.capacity;        // first come, first served
                if (!dropped) pos = p.expert_offset[e] + r;
            }
            __syncwarp();
            if (act && e >= 0 && e < p.E && rank == 0) s_base[e] += __popc(m);
            __syncwarp();
            if (act) {
                if (!dropped && (pos < 0 || (int64_t)pos >= p.P_cap)) {
                    if (p.status) atomicCAS(p.status, DEV_OK, DEV_BAD_INDEX);
                    pos = -1;
                }
                s_pos[q] = pos;
                s_exp[q] = e;
                p.pair_pos[tok0 * p.k_tot + q] = pos;
                if (pos >= 0) p.row_token[pos] = (int)(tok0 + q / p.k_tot);
            }
        }
    }
    __syncthreads();
    if (p.capacity >= 0) {
        // apply_capacity_constraint (src/core/moe_layer.jl:239-244): dropped slots get id 0 and gate 0,
        // then the token's gates are divided by their sum (if positive)
        for (int tl = threadIdx.x; tl < ntok; tl += PERM_THREADS) {
            const int64_t base = (tok0 + tl) * p.k_tot;
            float sum = 0.f;
            for (int j = 0; j < p.k_tot; ++j)
                if (s_pos[tl * p.k_tot + j] >= 0) sum += p.gate_rw[base + j];
            for (int j = 0; j < p.k_tot; ++j) {
                const bool kept = s_pos[tl * p.k_tot + j] >= 0;
                float g = kept ? p.gate_rw[base + j] : 0.f;
                if (sum > 0.f) g = g / sum;
                p.gate_rw[base + j] = g;
                if (!kept) p.idx_rw[base + j] = -1;
                if (p.u_gate) p.u_gate[base + j] = g;
                if (p.u_idx && !kept) p.u_idx[base + j] = p.index_base - 1;
            }
        }
    }

    const XT* x = reinterpret_cast<const XT*>(p.x);
    PT* xp = reinterpret_cast<PT*>(p.xp);
    // (peer segments start at row boundaries of cudaMalloc'd buffers: 16-byte aligned when the rows are)
    const bool vec = (p.D * sizeof(XT)) % 16 == 0 && (p.D * sizeof(PT)) % 16 == 0 &&
                     ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.xp)) & 15) == 0;
    for (int tl = warp; tl < ntok; tl += PERM_THREADS / 32) {
        PT* dst[MAX_KTOT];
        int nd = 0;
        for (int j = 0; j < p.k_tot; ++j) {
            const int pos = s_pos[tl * p.k_tot + j];
            if (pos < 0 || s_exp[tl * p.k_tot + j] < p.inplace_experts) continue;
            if (p.expert_dst) {
                const int e = s_exp[tl * p.k_tot + j];
                dst[nd++] = reinterpret_cast<PT*>(p.expert_dst[e]) + (size_t)(pos - p.expert_offset[e]) * p.D;
            } else {
                dst[nd++] = xp + (size_t)pos * p.D;
            }
        }
        copy_row<XT, PT>(x + (size_t)(tok0 + tl) * p.D, dst, nd, p.D, lane, vec);
    }
}

template <typename YT>
__device__ __forceinline__ float4 ld_y4(const YT* p);
template <>
__device__ __forceinline__ float4 ld_y4<float>(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 ld_y4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <typename YT>
__device__ __forceinline__ float ld_y1(const YT* p);
template <>
__device__ __forceinline__ float ld_y1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_y1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

constexpr int COMB_THREADS = 256;

// One CTA per token; threads stride the O columns four at a time.
template <typename YT>
__global__ void __launch_bounds__(COMB_THREADS) combine_kernel(const CombineParams p) {
    __shared__ int s_row[MAX_KTOT];
    __shared__ const YT* s_ptr[MAX_KTOT];
    __shared__ float s_gate[MAX_KTOT];
    __shared__ int s_n;
    const int64_t t = blockIdx.x;
    // the token's slots: one thread per slot fetches (expert, row, gate), so the loads overlap ...
    __shared__ int s_id_in[MAX_KTOT], s_row_in[MAX_KTOT];
    __shared__ float s_gate_in[MAX_KTOT];
    chain_release();
    chain_wait();
    if (threadIdx.x < p.k_tot) {
        const int j = threadIdx.x;
        s_id_in[j] = p.idx[t * p.k_tot + j];
        s_row_in[j] = p.pair_pos[t * p.k_tot + j];
        s_gate_in[j] = p.gate[t * p.k_tot + j];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // ... then an insertion sort by expert id (k_tot <= 16)
        int ids[MAX_KTOT];
        int n = 0;
        for (int j = 0; j < p.k_tot; ++j) {
            const int e = s_id_in[j];
            const int r = s_row_in[j];
            const float g = s_gate_in[j];
            if (r < 0) continue;
            int i = n++;
            while (i > 0 && ids[i - 1] > e) {
                ids[i] = ids[i - 1];
                s_row[i] = s_row[i - 1];
                s_gate[i] = s_gate[i - 1];
                --i;
            }
            ids[i] = e;
            s_row[i] = r;
            s_gate[i] = g;
        }
        s_n = n;
        for (int i = 0; i < n; ++i) s_ptr[i] = reinterpret_cast<const YT*>(p.y) + (size_t)s_row[i] * p.O;
    }
    __syncthreads();
    const int n = s_n;
    float* out = p.out + (size_t)t * p.O;
    const bool vec = (p.O % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    bool done = false;
    if constexpr (sizeof(YT) == 2) {
        // BF16 rows: 16-byte loads (8 columns per thread), four rows in flight; the sum over a
        // token's experts keeps the ascending-expert order of the narrow path below
        if (vec && p.O % 8 == 0) {
            for (int c = threadIdx.x * 8; c < p.O; c += COMB_THREADS * 8) {
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                for (int j0 = 0; j0 < n; j0 += 4) {
                    uint4 q[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        if (j0 + jj < n) q[jj] = *reinterpret_cast<const uint4*>(s_ptr[j0 + jj] + c);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        if (j0 + jj < n) {
                            const float g = s_gate[j0 + jj];
                            const uint32_t u[4] = {q[jj].x, q[jj].y, q[jj].z, q[jj].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                acc[2 * i] += g * __uint_as_float(u[i] << 16);
                                acc[2 * i + 1] += g * __uint_as_float(u[i] & 0xffff0000u);
                            }
                        }
                    }
                }
                *reinterpret_cast<float4*>(out + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(out + c + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
            done = true;
        }
    }
    if (done) {
    } else if (vec) {
        for (int c = threadIdx.x * 4; c < p.O; c += COMB_THREADS * 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < n; ++j) {
                const float4 v = ld_y4<YT>(s_ptr[j] + c);
                const float g = s_gate[j];
                acc.x += g * v.x;
                acc.y += g * v.y;
                acc.z += g * v.z;
                acc.w += g * v.w;
            }
            *reinterpret_cast<float4*>(out + c) = acc;
        }
    } else {
        for (int c = threadIdx.x; c < p.O; c += COMB_THREADS) {
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc += s_gate[j] * ld_y1<YT>(s_ptr[j] + c);
            out[c] = acc;
        }
    }
}

}  // namespace

int launch_permute(const PermuteParams& p, int x_dtype, int xp_dtype, int num_cta, cudaStream_t s) {
    if (x_dtype == MOE_DTYPE_F32 && xp_dtype == MOE_DTYPE_F32)
        launch_kernel(permute_kernel<float, float>, dim3(num_cta), dim3(PERM_THREADS), 0, s, p);
    else if (x_dtype == MOE_DTYPE_BF16 && xp_dtype == MOE_DTYPE_BF16)
        launch_kernel(permute_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(num_cta), dim3(PERM_THREADS), 0, s, p);
    else if (x_dtype == MOE_DTYPE_F32 && xp_dtype == MOE_DTYPE_BF16)
        launch_kernel(permute_kernel<float, __nv_bfloat16>, dim3(num_cta), dim3(PERM_THREADS), 0, s, p);
    else
        launch_kernel(permute_kernel<__nv_bfloat16, float>, dim3(num_cta), dim3(PERM_THREADS), 0, s, p);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_combine(const CombineParams& p, int y_dtype, cudaStream_t s) {
    if (p.T == 0) return 0;
    if (y_dtype == MOE_DTYPE_F32)
        launch_kernel(combine_kernel<float>, dim3((unsigned)p.T), dim3(COMB_THREADS), 0, s, p);
    else
        launch_kernel(combine_kernel<__nv_bfloat16>, dim3((unsigned)p.T), dim3(COMB_THREADS), 0, s, p);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
