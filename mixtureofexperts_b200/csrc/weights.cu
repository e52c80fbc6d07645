// Weight repack: any of {FP32, BF16} x {in-contiguous, out-contiguous} source layouts into the
// handle's [out][in] (in contiguous = K-major) array of the compute dtype.  Stands in for the
// weight copy of to_cuda / create_synchronized_moe_pair (src/cuda/utils.jl:4-15,
// src/amdgpu/utils.jl:62-105), which copied Dense.weight verbatim.
#include "common.cuh"

namespace moe {
namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// dst[r][c] = src[r][c] (same layout) -- grid-stride convert
template <typename S, typename D>
__global__ void convert_kernel(const S* src, D* dst, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = from_f<D>(to_f<S>(src[i]));
}

// dst[r][c] = src[c][r]; dst is rows x cols, src is cols x rows; 32x32 tiles through smem
template <typename S, typename D>
__global__ void transpose_convert_kernel(const S* src, D* dst, int rows, int cols) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int c = c0 + j, r = r0 + threadIdx.x;   // src row = c, src col = r
        if (c < cols && r < rows) tile[j][threadIdx.x] = to_f<S>(src[(size_t)c * rows + r]);
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) dst[(size_t)r * cols + c] = from_f<D>(tile[threadIdx.x][j]);
    }
}

template <typename S, typename D>
int run(const void* src, void* dst, int rows, int cols, int transposed, cudaStream_t s) {
    if (!transposed) {
        const size_t n = (size_t)rows * cols;
        const int blocks = (int)((n + 255) / 256 < 65535 ? (n + 255) / 256 : 65535);
        convert_kernel<S, D><<<blocks, 256, 0, s>>>(reinterpret_cast<const S*>(src), reinterpret_cast<D*>(dst), n);
    } else {
        dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
        transpose_convert_kernel<S, D><<<grid, block, 0, s>>>(reinterpret_cast<const S*>(src),
                                                              reinterpret_cast<D*>(dst), rows, cols);
    }
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace

// dst: rows_out x cols_out, cols contiguous.  src_is_transposed: src is cols_out x rows_out.
int launch_transpose_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int rows_out, int cols_out,
                             int src_is_transposed, cudaStream_t s) {
    if (src_dtype == MOE_DTYPE_F32 && dst_dtype == MOE_DTYPE_F32)
        return run<float, float>(src, dst, rows_out, cols_out, src_is_transposed, s);
    if (src_dtype == MOE_DTYPE_F32 && dst_dtype == MOE_DTYPE_BF16)
        return run<float, __nv_bfloat16>(src, dst, rows_out, cols_out, src_is_transposed, s);
    if (src_dtype == MOE_DTYPE_BF16 && dst_dtype == MOE_DTYPE_F32)
        return run<__nv_bfloat16, float>(src, dst, rows_out, cols_out, src_is_transposed, s);
    return run<__nv_bfloat16, __nv_bfloat16>(src, dst, rows_out, cols_out, src_is_transposed, s);
}

}  // namespace moe
