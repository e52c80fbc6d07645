// Grouped GatedExpert FFN in FP32 on CUDA cores (the 1e-5 parity class): real FP32 FMAs, no
// TF32/BF16 tensor cores.  Mode 1: h = act(A*W1^T) .* (A*W3^T); mode 2: y = h*W2^T -- the
// three products of (expert::GatedExpert)(x) (src/experts/gated.jl:29-34,
// src/llama2/inference.jl:154-167; src/cuda/experts.jl:20-26 ran them as three cuBLAS SGEMMs
// on ALL tokens for every expert).
//
// Rows of the permuted buffer are grouped by expert; an m-tile (F32_TILE_M rows) never spans
// two experts.  Weights are [E][N][K], K contiguous.  At the small per-expert row counts this
// path serves, the kernel is bound by streaming the expert weights from HBM once.
#include "activation.cuh"

namespace moe {
namespace {

constexpr int BM = F32_TILE_M;  // 16
constexpr int BN = 128;
constexpr int BK = 32;
constexpr int THREADS = 256;

__device__ __forceinline__ float4 ldg4(const float* row, int kk, int K, bool vec) {
    if (vec && kk + 3 < K) return __ldg(reinterpret_cast<const float4*>(row + kk));
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kk + 0 < K) v.x = row[kk + 0];
    if (kk + 1 < K) v.y = row[kk + 1];
    if (kk + 2 < K) v.z = row[kk + 2];
    if (kk + 3 < K) v.w = row[kk + 3];
    return v;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS) group_gemm_f32_kernel(const GroupGemmParams p) {
    constexpr int NB = (MODE == 1) ? 2 : 1;
    __shared__ float As[BM][BK];
    __shared__ float Bs[NB][BN][BK + 1];

    const int mtile = blockIdx.x;
    if (mtile >= p.tile_prefix[p.E]) return;
    const int e = find_segment(p.tile_prefix, p.E, mtile);
    const int row0 = p.expert_offset[e] + (mtile - p.tile_prefix[e]) * BM;
    const int row_end = p.expert_offset[e + 1];
    const int n0 = blockIdx.y * BN;

    const int tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const float* A = reinterpret_cast<const float*>(p.A);
    const float* Bm[2] = {reinterpret_cast<const float*>(p.B0) + (size_t)e * p.N * p.K,
                          MODE == 1 ? reinterpret_cast<const float*>(p.B1) + (size_t)e * p.N * p.K : nullptr};
    const bool vec = (p.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.A) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.B0) & 15) == 0) &&
                     (MODE != 1 || (reinterpret_cast<uintptr_t>(p.B1) & 15) == 0);

    // global -> register staging (prefetch of the next K block while the current one computes)
    float4 a_reg = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 b_reg[NB][4];
    const int a_row = tid >> 3, a_c4 = tid & 7;  // threads 0..127 load A: 16 rows x 8 float4
    auto load_tiles = [&](int k0) {
        if (tid < BM * (BK / 4)) {
            const int r = row0 + a_row;
            a_reg = (r < row_end) ? ldg4(A + (size_t)r * p.K, k0 + a_c4 * 4, p.K, vec)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * THREADS;
                const int n = n0 + (idx >> 3), c4 = idx & 7;
                b_reg[b][i] = (n < p.N) ? ldg4(Bm[b] + (size_t)n * p.K, k0 + c4 * 4, p.K, vec)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
            }
    };
    auto store_tiles = [&]() {
        if (tid < BM * (BK / 4)) {
            As[a_row][a_c4 * 4 + 0] = a_reg.x;
            As[a_row][a_c4 * 4 + 1] = a_reg.y;
            As[a_row][a_c4 * 4 + 2] = a_reg.z;
            As[a_row][a_c4 * 4 + 3] = a_reg.w;
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int idx = tid + i * THREADS;
                const int n = idx >> 3, c4 = idx & 7;
                Bs[b][n][c4 * 4 + 0] = b_reg[b][i].x;
                Bs[b][n][c4 * 4 + 1] = b_reg[b][i].y;
                Bs[b][n][c4 * 4 + 2] = b_reg[b][i].z;
                Bs[b][n][c4 * 4 + 3] = b_reg[b][i].w;
            }
    };

    float acc[NB][2][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[b][r][i] = 0.f;

    load_tiles(0);
    for (int k0 = 0; k0 < p.K; k0 += BK) {
        __syncthreads();
        store_tiles();
        __syncthreads();
        if (k0 + BK < p.K) load_tiles(k0 + BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float a0 = As[ty * 2 + 0][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float w = Bs[b][tx + 32 * i][k];
                    acc[b][0][i] = fmaf(a0, w, acc[b][0][i]);
                    acc[b][1][i] = fmaf(a1, w, acc[b][1][i]);
                }
        }
    }

    float* C = reinterpret_cast<float*>(p.C);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + ty * 2 + r;
        if (row >= row_end) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + tx + 32 * i;
            if (n >= p.N) continue;
            float v;
            if (MODE == 1) {
                v = apply_act(p.activation, acc[0][r][i]) * acc[NB - 1][r][i];
            } else {
                v = acc[0][r][i];
                if (p.bias) v += p.bias[(size_t)e * p.N + n];
                if (p.epilogue_act >= 0) v = apply_act(p.epilogue_act, v);
            }
            group_gemm_out_row<float>(p, e, row)[n] = v;
        }
    }
}

// ---- few rows per expert (decode, tiny batches): stream the weights once ------------------------
// One CTA owns (expert, 8*CW output columns); a warp owns CW columns; lanes split K in 16-byte
// pieces, so every weight load instruction of a warp is a contiguous 512-byte read and a lane keeps
// 2*CW (mode 1: 4*CW) of them in flight.  Four rows of the expert are held in registers per pass
// (further rows of the expert are taken by the CTAs of the other blockIdx.z planes, which read the
// same weight slice through L2 at the same time, or by further passes of this CTA); partial dot
// products are reduced with warp shuffles once per pass.  Bound: HBM, E*N*K*4 bytes of weights per GEMM.
constexpr int SK_ROWS = 4;
constexpr int SK_THREADS = 256;

__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

template <int MODE, int CW>
__global__ void __launch_bounds__(SK_THREADS) group_gemm_f32_skinny_kernel(const GroupGemmParams p) {
    constexpr int NB = (MODE == 1) ? 2 : 1;
    const int e = blockIdx.y;
    const int row_begin = p.expert_offset[e], row_end = p.expert_offset[e + 1];
    if (row_begin >= row_end) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_base = (blockIdx.x * (SK_THREADS / 32) + warp) * CW;
    if (n_base >= p.N) return;
    const float* A = reinterpret_cast<const float*>(p.A);
    const float* Bm[2] = {reinterpret_cast<const float*>(p.B0) + (size_t)e * p.N * p.K,
                          MODE == 1 ? reinterpret_cast<const float*>(p.B1) + (size_t)e * p.N * p.K : nullptr};
    float* C = reinterpret_cast<float*>(p.C);
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int r0 = row_begin + SK_ROWS * (int)blockIdx.z; r0 < row_end; r0 += SK_ROWS * (int)gridDim.z) {
        float acc[NB][CW][SK_ROWS];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = 0; c < CW; ++c)
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) acc[b][c][r] = 0.f;
        for (int kc = 0; kc < p.K; kc += 256) {
            const int k0 = kc + lane * 4, k1 = kc + 128 + lane * 4;   // K % 4 == 0: a piece is all in or all out
            float4 xa[SK_ROWS], xb[SK_ROWS];
#pragma unroll
            for (int r = 0; r < SK_ROWS; ++r) {
                const bool ok = r0 + r < row_end;
                const float* row = A + (size_t)(r0 + r) * p.K;
                xa[r] = (ok && k0 < p.K) ? *reinterpret_cast<const float4*>(row + k0) : zero4;
                xb[r] = (ok && k1 < p.K) ? *reinterpret_cast<const float4*>(row + k1) : zero4;
            }
            float4 wa[NB][CW], wb[NB][CW];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int c = 0; c < CW; ++c) {
                    const int n = n_base + c;
                    const float* wrow = Bm[b] + (size_t)n * p.K;
                    wa[b][c] = (n < p.N && k0 < p.K) ? __ldg(reinterpret_cast<const float4*>(wrow + k0)) : zero4;
                    wb[b][c] = (n < p.N && k1 < p.K) ? __ldg(reinterpret_cast<const float4*>(wrow + k1)) : zero4;
                }
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int c = 0; c < CW; ++c)
#pragma unroll
                    for (int r = 0; r < SK_ROWS; ++r)
                        acc[b][c][r] = dot4(wb[b][c], xb[r], dot4(wa[b][c], xa[r], acc[b][c][r]));
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = 0; c < CW; ++c)
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) {
                    float v = acc[b][c][r];
#pragma unroll
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    acc[b][c][r] = v;
                }
        // lane (c*SK_ROWS + r) writes element (row r, column c)
#pragma unroll
        for (int c = 0; c < CW; ++c)
#pragma unroll
            for (int r = 0; r < SK_ROWS; ++r) {
                if (lane == c * SK_ROWS + r) {
                    const int row = r0 + r, n = n_base + c;
                    if (row < row_end && n < p.N) {
                        float v;
                        if (MODE == 1) {
                            v = apply_act(p.activation, acc[0][c][r]) * acc[NB - 1][c][r];
                        } else {
                            v = acc[0][c][r];
                            if (p.bias) v += p.bias[(size_t)e * p.N + n];
                            if (p.epilogue_act >= 0) v = apply_act(p.epilogue_act, v);
                        }
                        group_gemm_out_row<float>(p, e, row)[n] = v;
                    }
                }
            }
    }
}

template <int MODE>
int launch_skinny(const GroupGemmParams& p, int64_t rows, int num_sms, cudaStream_t s) {
    // Row passes of an expert run side by side in the z planes of the grid instead of one after the
    // other in one CTA: about twice the average rows per expert, at most 8 planes (a CTA whose
    // plane has no rows left for its expert leaves at once).
    const int64_t avg = p.E > 0 ? (rows + p.E - 1) / p.E : 1;
    int planes = (int)((2 * avg + SK_ROWS - 1) / SK_ROWS);
    planes = planes < 1 ? 1 : (planes > 8 ? 8 : planes);
    // fewer columns per warp when the problem would otherwise leave SMs without a CTA
    const long ctas4 = (long)((p.N + 31) / 32) * p.E;
    if (ctas4 >= 2L * num_sms) {
        dim3 grid((p.N + 31) / 32, p.E, planes);
        group_gemm_f32_skinny_kernel<MODE, 4><<<grid, SK_THREADS, 0, s>>>(p);
    } else if (ctas4 * 2 >= 2L * num_sms) {
        dim3 grid((p.N + 15) / 16, p.E, planes);
        group_gemm_f32_skinny_kernel<MODE, 2><<<grid, SK_THREADS, 0, s>>>(p);
    } else {
        dim3 grid((p.N + 7) / 8, p.E, planes);
        group_gemm_f32_skinny_kernel<MODE, 1><<<grid, SK_THREADS, 0, s>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

int launch_group_gemm_f32(const GroupGemmParams& p, int mode, int max_mtiles, int64_t rows, int num_sms,
                          cudaStream_t s) {
    if (max_mtiles <= 0) return 0;
    const bool aligned = (p.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.A) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(p.B0) & 15) == 0) &&
                         (mode != 1 || (reinterpret_cast<uintptr_t>(p.B1) & 15) == 0);
    if (aligned && rows <= 16L * p.E) {
        // on average at most 16 rows per expert: weight streaming beats tiling
        return mode == 1 ? launch_skinny<1>(p, rows, num_sms, s) : launch_skinny<2>(p, rows, num_sms, s);
    }
    dim3 grid(max_mtiles, (p.N + BN - 1) / BN);
    if (mode == 1) group_gemm_f32_kernel<1><<<grid, THREADS, 0, s>>>(p);
    else group_gemm_f32_kernel<2><<<grid, THREADS, 0, s>>>(p);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace moe
