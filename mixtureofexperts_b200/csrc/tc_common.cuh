// PTX wrappers shared by the tcgen05 grouped-GEMM kernels (single-CTA and CTA-pair variants):
// mbarrier, TMA tensor loads, TMEM allocation, tcgen05.mma / commit / ld, descriptors.
#pragma once
#include <cuda.h>

#include "activation.cuh"

namespace moe {
namespace tc {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait
constexpr unsigned long long DRAIN_LIMIT_NS = 2000000ull;    // 2 ms when draining after an abort

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the CTA is aborting or the limit expired (then it raises the
// abort flag and records `code`).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int32_t code, unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    // the clock is first read after 64 failed attempts: most waits end well before that, and a read of
    // the global timer in front of every retry would sit between the barrier's completion and its notice
    unsigned long long t0 = 0;
    bool timed = false;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            const unsigned long long now = globaltimer_ns();
            if (!timed) {
                t0 = now;
                timed = true;
            } else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                if (status) atomicCAS(status, DEV_OK, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, BF16 inputs, FP32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive FP32 columns: thread i of the warp receives lane (base_lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // bits [0,14): start address / 16
    d |= (uint64_t)1 << 16;                     // bits [16,30): leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;           // bits [32,46): stride byte offset / 16
    d |= (uint64_t)1 << 46;                     // bits [46,48): version
    d |= (uint64_t)2 << 61;                     // bits [61,64): SWIZZLE_128B
    return d;
}

// Instruction descriptor of kind::f16: FP32 accumulator, BF16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}


struct TileCoord {
    int e;        // expert
    int row0;     // first permuted row of the tile
    int row_end;  // end of the expert's rows
    int n_idx;    // n-tile index
};

// Expert-major order; inside an expert, groups of `gm` m-tiles sweep all n-tiles (m fastest).
__device__ __forceinline__ TileCoord decode_tile(int L, int n_tiles, int gm, const int32_t* tile_prefix,
                                                 const int32_t* expert_offset, int E, int tile_rows) {
    TileCoord t;
    const int e = find_segment(tile_prefix, E, L / n_tiles);
    const int m_tiles = tile_prefix[e + 1] - tile_prefix[e];
    const int local = L - tile_prefix[e] * n_tiles;
    const int g = local / (gm * n_tiles);
    const int rem = local - g * gm * n_tiles;
    const int gsz = min(gm, m_tiles - g * gm);
    const int m_local = g * gm + rem % gsz;
    t.e = e;
    t.n_idx = rem / gsz;
    t.row0 = expert_offset[e] + m_local * tile_rows;
    t.row_end = expert_offset[e + 1];
    return t;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Activations of the BF16 epilogues.  One special-function operation per element: sigmoid(x) = 0.5 + 0.5 tanh(x/2)
// and the tanh of GELU's approximation both go through tanh.approx (absolute error below 2^-10.9, i.e. 2.6e-4 on
// the sigmoid, against the 2^-9 relative rounding of the BF16 result).  The exp-and-divide forms cost two, which
// the kernel whose epilogue is not hidden behind MMAs (expert_tc_dual.cu) felt; every tensor-core kernel uses
// this one function, so a layer gives the same bits whichever kernel a batch size selects.
__device__ __forceinline__ float tanh_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}
__device__ __forceinline__ float act_fast(int act, float v) {
    switch (act) {
        case MOE_ACT_SILU:
            return 0.5f * v * (1.0f + tanh_fast(0.5f * v));
        case MOE_ACT_GELU_TANH:
            return 0.5f * v * (1.0f + tanh_fast(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case MOE_ACT_RELU:
            return fmaxf(v, 0.f);
        default:
            return v;
    }
}

// Store 32 consecutive BF16 columns of one row.
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst_row, int col0, int N, const float (&v)[32],
                                            bool vec_ok) {
    if (vec_ok && col0 + 32 <= N) {
        uint4* d = reinterpret_cast<uint4*>(dst_row + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            u.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            u.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            u.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
            d[q] = u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < N) dst_row[col0 + i] = __float2bfloat16_rn(v[i]);
    }
}

}  // namespace tc

// Tensor maps of one layer's grouped GEMM pair (rows in boxes of 64 x 128, weights 64 x 128 x 1).
struct TcGemmPlan {
    CUtensorMap map_xp, map_h, map_w1, map_w3, map_w2;
    CUtensorMap map_x;      // this call's activations, for experts that read them in place (tc_plan_set_x)
    bool valid = false;
    bool attr_set = false;
    bool attr2_set = false;
    int max_clusters = 0;   // co-resident CTA pairs of the cta_group::2 kernel (0 = not queried)
};

int group_m_setting();   // m-tiles per group of the tile order (MOE_B200_GROUP_M or the default)

}  // namespace moe
