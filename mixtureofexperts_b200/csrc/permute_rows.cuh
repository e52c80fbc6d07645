// Row copies of the token permute: one warp copies a token's D-vector to up to k_tot destination
// rows (16-byte loads and stores where the layout allows), converting between FP32 and BF16 when the
// activations and the expert GEMMs use different types.
#pragma once
#include "common.cuh"

namespace moe {
namespace rows {

template <typename T>
struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
};

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

template <typename XT, typename PT>
__device__ __forceinline__ void copy_row(const XT* src, PT* const* dst, int ndst, int D, int lane, bool vec);

// same type: straight 16-byte copies
template <typename T>
__device__ __forceinline__ void copy_row_same(const T* src, T* const* dst, int ndst, int D, int lane, bool vec) {
    constexpr int N = 16 / sizeof(T);
    if (vec) {
        // four 16-byte loads in flight per lane before the first store
        int c = lane * N;
        for (; c + 3 * 32 * N < D; c += 4 * 32 * N) {
            const uint4 v0 = ld16(src + c), v1 = ld16(src + c + 32 * N), v2 = ld16(src + c + 2 * 32 * N),
                        v3 = ld16(src + c + 3 * 32 * N);
            for (int j = 0; j < ndst; ++j) {
                st16(dst[j] + c, v0);
                st16(dst[j] + c + 32 * N, v1);
                st16(dst[j] + c + 2 * 32 * N, v2);
                st16(dst[j] + c + 3 * 32 * N, v3);
            }
        }
        for (; c < D; c += 32 * N) {
            const uint4 v = ld16(src + c);
            for (int j = 0; j < ndst; ++j) st16(dst[j] + c, v);
        }
    } else {
        for (int c = lane; c < D; c += 32) {
            const T v = src[c];
            for (int j = 0; j < ndst; ++j) dst[j][c] = v;
        }
    }
}

template <>
__device__ __forceinline__ void copy_row<float, float>(const float* s, float* const* d, int n, int D, int lane,
                                                       bool vec) {
    copy_row_same<float>(s, d, n, D, lane, vec);
}
template <>
__device__ __forceinline__ void copy_row<__nv_bfloat16, __nv_bfloat16>(const __nv_bfloat16* s,
                                                                       __nv_bfloat16* const* d, int n, int D,
                                                                       int lane, bool vec) {
    copy_row_same<__nv_bfloat16>(s, d, n, D, lane, vec);
}
template <>
__device__ __forceinline__ void copy_row<float, __nv_bfloat16>(const float* s, __nv_bfloat16* const* d, int n,
                                                               int D, int lane, bool vec) {
    if (vec) {
        // 8 columns per lane: two 16-byte loads, round to nearest even, one 16-byte store per destination
        for (int c = lane * 8; c < D; c += 32 * 8) {
            const float4 a = *reinterpret_cast<const float4*>(s + c), b = *reinterpret_cast<const float4*>(s + c + 4);
            const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w),
                                 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
            uint4 v;
            v.x = *reinterpret_cast<const uint32_t*>(&p0);
            v.y = *reinterpret_cast<const uint32_t*>(&p1);
            v.z = *reinterpret_cast<const uint32_t*>(&p2);
            v.w = *reinterpret_cast<const uint32_t*>(&p3);
            for (int j = 0; j < n; ++j) st16(d[j] + c, v);
        }
        return;
    }
    for (int c = lane; c < D; c += 32) {
        const __nv_bfloat16 v = __float2bfloat16_rn(s[c]);
        for (int j = 0; j < n; ++j) d[j][c] = v;
    }
}
template <>
__device__ __forceinline__ void copy_row<__nv_bfloat16, float>(const __nv_bfloat16* s, float* const* d, int n,
                                                               int D, int lane, bool) {
    for (int c = lane; c < D; c += 32) {
        const float v = __bfloat162float(s[c]);
        for (int j = 0; j < n; ++j) d[j][c] = v;
    }
}

}  // namespace rows
}  // namespace moe
