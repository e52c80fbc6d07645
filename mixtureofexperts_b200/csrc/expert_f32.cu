// Grouped GatedExpert FFN in FP32 on CUDA cores (the 1e-5 parity class): real FP32 FMAs, no
// TF32/BF16 tensor cores.  Mode 1: h = act(A*W1^T) .* (A*W3^T); mode 2: y = h*W2^T -- the
// three products of (expert::GatedExpert)(x) (src/experts/gated.jl:29-34,
// src/llama2/inference.jl:154-167; src/cuda/experts.jl:20-26 ran them as three cuBLAS SGEMMs
// on ALL tokens for every expert).
//
// Rows of the permuted buffer are grouped by expert; an m-tile (F32_TILE_M rows) never spans
// two experts.  Weights are [E][N][K], K contiguous.  At the small per-expert row counts this
// path serves, the kernel is bound by streaming the expert weights from HBM once.
#include "tc_common.cuh"

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
    chain_release();
    chain_wait();
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
// Bound: HBM, E*N*K*4 bytes of weights per GEMM.  A persistent CTA per SM walks work items (expert,
// block of 32 output columns, pass of up to 16 of the expert's rows); a producer thread streams each
// item as K tiles of 128 floats through a 4-stage shared-memory ring with TMA tensor loads (one
// 32 x 128 box per weight matrix and one 16 x 128 box of activation rows per stage, completion on an
// mbarrier; 1-D bulk copies, one per row piece, were tried first and were bound by the ~50 ns the
// TMA unit spends per copy), so ~160 KB per SM are in flight whatever the consumers do.
// Eight consumer warps own four columns each.  Lanes split a K tile in 16-byte pieces (conflict-free
// shared-memory reads), keep (matrices x 4 columns x 16 rows) accumulators in registers over the
// whole K loop, rows taken in groups of four, and finish with multi-value butterflies (31 shuffles
// for 32 sums, fixed order) that leave lane l with the sum for (column l / 16, row l % 16) of a
// column pair.  With two columns a warp the kernel was bound by shared-memory reads (every warp
// reads the whole activation tile of a stage: four bytes of it per weight byte) and packed
// two-wide FMAs changed nothing; one column a warp on sixteen warps was no faster either.  Every
// wait is bounded like in the tensor-core kernels.
constexpr int ST_CW = 4;             // output columns per consumer warp
constexpr int ST_COLS = 32;          // output columns per work item (8 consumer warps)
constexpr int ST_ROWS = 16;          // rows of an expert per pass
constexpr int ST_KT = 128;           // floats of K per ring stage: one float4 per lane
constexpr int ST_STAGES = 4;
constexpr int ST_CONSUMER_WARPS = 8;
// Three warpgroups: two of consumers, one whose first warp is the producer.  Registers are handed
// over at the start (setmaxnreg works on whole warpgroups): the producer group keeps 40 a thread,
// the consumers grow to 232, enough for the 128 accumulators, 8 weight and 4 activation vectors.
constexpr int ST_THREADS = (ST_CONSUMER_WARPS + 4) * 32;
constexpr int ST_REGS_PRODUCER = 40;
constexpr int ST_REGS_CONSUMER = 232;

template <int NB>
struct __align__(128) StreamStage {
    float w[NB][ST_COLS][ST_KT];
    float x[ST_ROWS][ST_KT];
};
template <int NB>
struct __align__(128) StreamStorage {
    StreamStage<NB> st[ST_STAGES];
    uint64_t full_bar[ST_STAGES];
    uint64_t empty_bar[ST_STAGES];
    volatile int abort_flag;
    int expert_offset[MAX_EXPERTS + 1];   // read once: a global load per work item would sit on every item's critical path
};

__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// 32 sums over the warp's lanes in 31 shuffles: after the call a[0] of lane l is the total of a[l].
__device__ __forceinline__ void warp_reduce32(float (&a)[32], int lane) {
    int n = 32;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        n >>= 1;
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < n) {
                const float send = up ? a[i] : a[i + n];
                const float keep = up ? a[i + n] : a[i];
                a[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
    }
}

template <int MODE>
__global__ void __launch_bounds__(ST_THREADS, 1)
group_gemm_f32_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                             const __grid_constant__ CUtensorMap map_b1, const GroupGemmParams p) {
    constexpr int NB = (MODE == 1) ? 2 : 1;
    using Storage = StreamStorage<NB>;
    extern __shared__ uint8_t smem_raw[];
    Storage* ss = reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncb = (p.N + ST_COLS - 1) / ST_COLS;
    const int num_items = p.E * ncb;
    const int nkt = (p.K + ST_KT - 1) / ST_KT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST_STAGES; ++s) {
            tc::mbar_init(&ss->full_bar[s], 1);
            tc::mbar_init(&ss->empty_bar[s], ST_CONSUMER_WARPS);
        }
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    chain_release();
    chain_wait();   // barriers are set up; everything below reads what the previous kernel wrote
    for (int e = threadIdx.x; e <= p.E; e += ST_THREADS) ss->expert_offset[e] = p.expert_offset[e];
    __syncthreads();

    int stage = 0;
    uint32_t phase = 0;
    if (warp >= ST_CONSUMER_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ST_REGS_PRODUCER));
        if (warp > ST_CONSUMER_WARPS) return;   // the group's other warps only give their registers away
        // ------------------------------ producer ----------------------------------------------
        uint32_t armed = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
            const int e = item / ncb, n0 = (item % ncb) * ST_COLS;
            const int row_begin = ss->expert_offset[e], row_end = ss->expert_offset[e + 1];
            for (int r0 = row_begin; ok && r0 < row_end; r0 += ST_ROWS) {
                for (int kt = 0; kt < nkt; ++kt) {
                    int go = 1;
                    if (lane == 0)
                        go = tc::mbar_wait(&ss->empty_bar[stage], phase ^ 1u, &ss->abort_flag, p.status, DEV_TIMEOUT_SMEM_EMPTY);
                    go = __shfl_sync(0xffffffffu, go, 0);
                    if (!go) {
                        ok = false;
                        break;
                    }
                    if (lane == 0) {
                        // boxes are always transferred whole (rows and columns past the tensor arrive as zeros)
                        StreamStage<NB>& st = ss->st[stage];
                        tc::mbar_expect_tx(&ss->full_bar[stage], (uint32_t)sizeof(StreamStage<NB>));
                        tc::tma_load_2d(&st.w[0][0][0], &map_b0, kt * ST_KT, e * p.N + n0, &ss->full_bar[stage]);
                        if (NB == 2) tc::tma_load_2d(&st.w[NB - 1][0][0], &map_b1, kt * ST_KT, e * p.N + n0, &ss->full_bar[stage]);
                        tc::tma_load_2d(&st.x[0][0], &map_a, kt * ST_KT, r0, &ss->full_bar[stage]);
                    }
                    armed |= 1u << stage;
                    if (++stage == ST_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        if ((!ok || ss->abort_flag) && lane == 0) {
            // leaving early: give the copies already issued a bounded time to land
            for (int s = 0; s < ST_STAGES; ++s) {
                if (!(armed & (1u << s))) continue;
                const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                const unsigned long long t0 = tc::globaltimer_ns();
                while (!tc::mbar_try_wait(&ss->full_bar[s], par) && tc::globaltimer_ns() - t0 < tc::DRAIN_LIMIT_NS) {
                }
            }
        }
        return;
    }

    // ------------------------------ consumers (warps 0..7): columns 4w .. 4w+3 of the item ----------
    // Shared memory bandwidth is what the consumers live on: every warp reads the whole activation tile
    // of a stage, so the more columns a warp owns the less of it is read per weight.  Four columns of
    // both matrices against sixteen rows are 128 accumulators a lane, which is what the registers taken
    // over from the producer group pay for.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ST_REGS_CONSUMER));
    const int c_lo = warp * ST_CW;
    bool alive = true;
    for (int item = blockIdx.x; alive && item < num_items; item += gridDim.x) {
        const int e = item / ncb, n0 = (item % ncb) * ST_COLS;
        const int row_begin = ss->expert_offset[e], row_end = ss->expert_offset[e + 1];
        for (int r0 = row_begin; alive && r0 < row_end; r0 += ST_ROWS) {
            const int rc = min(ST_ROWS, row_end - r0);
            float acc[NB][ST_CW / 2][32];            // [matrix][column pair][column (0/1) * 16 + row]
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int c = 0; c < ST_CW / 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[b][c][i] = 0.f;
            for (int kt = 0; kt < nkt; ++kt) {
                int ready = 1;
                if (lane == 0) ready = tc::mbar_wait(&ss->full_bar[stage], phase, &ss->abort_flag, p.status, DEV_TIMEOUT_TMA_FULL);
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (!ready) {
                    alive = false;
                    break;
                }
                while (!tc::mbar_try_wait(&ss->full_bar[stage], phase)) {
                }  // already complete: gives every lane its own acquire
                const StreamStage<NB>& st = ss->st[stage];
                const int k = lane * 4;
                if (k < p.K - kt * ST_KT) {
                    float4 w[NB][ST_CW];
#pragma unroll
                    for (int b = 0; b < NB; ++b)
#pragma unroll
                        for (int c = 0; c < ST_CW; ++c) w[b][c] = *reinterpret_cast<const float4*>(&st.w[b][c_lo + c][k]);
                    // rows in groups of four (a group past the pass's rows is skipped as a whole; rows past
                    // rc inside a group hold other experts' rows and their sums are never stored)
#pragma unroll
                    for (int g = 0; g < ST_ROWS / 4; ++g) {
                        if (g * 4 < rc) {
                            float4 xv[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) xv[q] = *reinterpret_cast<const float4*>(&st.x[g * 4 + q][k]);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int r = g * 4 + q;
#pragma unroll
                                for (int b = 0; b < NB; ++b)
#pragma unroll
                                    for (int c = 0; c < ST_CW; ++c)
                                        acc[b][c >> 1][(c & 1) * 16 + r] = dot4(w[b][c], xv[q], acc[b][c >> 1][(c & 1) * 16 + r]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&ss->empty_bar[stage]);
                if (++stage == ST_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!alive) break;
#pragma unroll
            for (int c = 0; c < ST_CW / 2; ++c) {
#pragma unroll
                for (int b = 0; b < NB; ++b) warp_reduce32(acc[b][c], lane);
                // lane l now holds (column c_lo + 2c + l / 16, row r0 + l % 16)
                const int n = n0 + c_lo + 2 * c + (lane >> 4), row = r0 + (lane & 15);
                if (n < p.N && (lane & 15) < rc) {
                    float v;
                    if (MODE == 1) {
                        v = apply_act(p.activation, acc[0][c][0]) * acc[NB - 1][c][0];
                    } else {
                        v = acc[0][c][0];
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
int launch_stream(const GroupGemmParams& p, int64_t rows, int num_sms, cudaStream_t s) {
    constexpr int NB = (MODE == 1) ? 2 : 1;
    auto kern = group_gemm_f32_stream_kernel<MODE>;
    const size_t smem = sizeof(StreamStorage<NB>) + 128;
    static bool attr_done[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
        attr_done[dev] = true;
    }
    CUtensorMap ma, mb0, mb1;
    if (!tc_encode_f32_2d(&ma, p.A, (uint64_t)p.K, (uint64_t)rows, ST_KT, ST_ROWS) ||
        !tc_encode_f32_2d(&mb0, p.B0, (uint64_t)p.K, (uint64_t)p.E * p.N, ST_KT, ST_COLS) ||
        !tc_encode_f32_2d(&mb1, NB == 2 ? p.B1 : p.B0, (uint64_t)p.K, (uint64_t)p.E * p.N, ST_KT, ST_COLS))
        return -1;
    const long items = (long)p.E * ((p.N + ST_COLS - 1) / ST_COLS);
    const int grid = (int)(items < num_sms ? items : num_sms);
    return launch_kernel(kern, dim3(grid), dim3(ST_THREADS), smem, s, ma, mb0, mb1, p) == cudaSuccess ? 1 : -1;
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
        return mode == 1 ? launch_stream<1>(p, rows, num_sms, s) : launch_stream<2>(p, rows, num_sms, s);
    }
    dim3 grid(max_mtiles, (p.N + BN - 1) / BN);
    const cudaError_t err = mode == 1 ? launch_kernel(group_gemm_f32_kernel<1>, grid, dim3(THREADS), 0, s, p)
                                      : launch_kernel(group_gemm_f32_kernel<2>, grid, dim3(THREADS), 0, s, p);
    return err == cudaSuccess ? 1 : -1;
}

}  // namespace moe
