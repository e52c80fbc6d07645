// Shared declarations of libmoe_b200: launch-parameter structs, device status codes and the
// host-side launcher prototypes of every kernel file.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/moe_b200.h"

namespace moe {

// ---- device status word (one int32 per handle) ---------------------------------------------
// 0 = clean.  Kernels never trap; a kernel that gives up writes one of these and returns.
enum : int32_t {
    DEV_OK = 0,
    DEV_TIMEOUT_TMA_FULL = 1,    // MMA warp waited too long for a TMA stage
    DEV_TIMEOUT_SMEM_EMPTY = 2,  // TMA warp waited too long for a free stage
    DEV_TIMEOUT_TMEM_FULL = 3,   // epilogue waited too long for an accumulator
    DEV_TIMEOUT_TMEM_EMPTY = 4,  // MMA warp waited too long for a drained accumulator
    DEV_BAD_INDEX = 5,           // an index check failed (recorded, access skipped)
    DEV_TIMEOUT_PEER = 6,        // expert parallel: a peer's flag (records, barrier) did not arrive in time
};

constexpr int ROUTER_THREADS = 256;
constexpr int ROUTER_WARPS = ROUTER_THREADS / 32;
constexpr int ROUTER_MAX_WARPS = 18;    // largest router CTA: 576 threads
constexpr int ROUTER_TOKENS_PER_CTA = 64;   // largest token tile; router_tokens_per_cta() picks per batch
constexpr int MAX_ROUTER_EXPERTS = 128; // upper bound on router rows
constexpr int MAX_EXPERTS = 256;        // upper bound on experts per layer
constexpr int MAX_KTOT = 16;            // upper bound on selected experts per token

// Tile height of the grouped GEMMs: an expert's rows are cut into tiles of this many rows.
constexpr int TC_TILE_M = 128;   // tcgen05 path, one CTA per tile
constexpr int TC_PAIR_TILE_M = 256;  // tcgen05 path, CTA pair per tile (cta_group::2)
constexpr int F32_TILE_M = 16;   // FP32 SIMT path

struct RouterParams {
    const void* x;            // [T][D]
    const float* w;           // [E_router][D]
    const float* wt;          // [D_pad][E_pad] K-major zero-padded copy (launch_router_transpose)
    const float* bias;        // [E_router] or null
    const float* noise = nullptr;   // [T][E_router] standard-normal draws for training-time router noise, or null
    float noise_scale = 0.f;
    int noise_off = 0;        // > 0: columns noise_off..noise_off+E_router-1 of wt hold the router's noise
                              // network and the draws are scaled by softplus of its logits; 0: no network
    int64_t T;
    int D;
    int E;                    // layer experts (shared included)
    int E_router;             // router rows
    int E_probs;              // columns of probs (E for NONE/GATING, E_router for LAYER_BLEND)
    int S;                    // shared experts
    int k;                    // routed experts per token
    int k_tot;                // S + k
    int shared_mode;
    int bias_gates_only;
    int index_base;
    int tokens_per_cta;       // 64, 32 or 16 (router_tokens_per_cta)
    int want_entropy;
    // internal results
    int32_t* idx;             // [T][k_tot] layer expert id, 0-based
    float* gate;              // [T][k_tot] combine-ready gate
    int32_t* cta_counts;      // [num_cta][E]
    float* cta_psum;          // [num_cta][E_probs + 1]: prob sums, then sum of lse^2
    double* cta_entropy;      // [num_cta]
    // user outputs (nullable)
    int32_t* u_idx;
    float* u_gate;
    float* u_probs;
    float* u_logits;
    // tensor-core router (router_tc.cu): scratch for the logits [T][E_PAD] and a counter of the tokens
    // whose logits were re-evaluated with FP32 FMAs; null = not available to this call
    float* tc_logits = nullptr;
    int32_t* tc_recheck_count = nullptr;
};

struct ScanParams {
    int64_t T;
    int E, E_probs, S, k, k_tot, shared_mode;
    int num_cta;
    int tile_m;
    int training;
    int capacity;             // rows an expert may keep (capacity constraint), -1 = unlimited
    float alpha, z_weight;
    int32_t* cta_counts;      // in: per-CTA counts; out: exclusive prefix over CTAs
    const float* cta_psum;
    const double* cta_entropy;
    int32_t* expert_count;    // [E]
    int32_t* expert_offset;   // [E+1] first permuted row of each expert
    int32_t* tile_prefix;     // [E+1] first m-tile of each expert
    float* loss_internal;     // [1]
    // user outputs (nullable, device)
    float* u_loss;
    int64_t* u_tokens_per_expert;
    float* u_entropy;
    // chunked host calls: when non-null the loss is finished later from the chunks' sums
    float* ep_sums;           // [E + E_probs + 3]: counts, prob sums, sum lse^2, T, entropy sum
    int sums_accumulate;      // 1: add into ep_sums / u_tokens_per_expert (chunks of one batch) instead of storing
    // expert-parallel: this rank's record of the call for the exchange with the other ranks,
    // [E + E_probs + 3] words = {int32 counts[E], float prob sums[E_probs], float lse^2 sum, int32 T, float entropy sum}
    int32_t* ep_record;
};

struct PermuteParams {
    const void* x;            // [T][D]
    void* xp;                 // [P][D]
    int64_t T;
    int D, E, k_tot;
    int tokens_per_cta;
    const int32_t* idx;
    const int32_t* cta_base;      // [num_cta][E] exclusive prefix over CTAs
    const int32_t* expert_offset; // [E+1]
    int32_t* pair_pos;            // [T][k_tot] permuted row of each pair
    int32_t* row_token;           // [P]
    int32_t* status;
    int64_t P_cap;
    // capacity constraint (capacity >= 0): pairs ranked >= capacity inside their expert are dropped,
    // gates renormalised per token; idx/gate (and the caller's copies) are rewritten
    int capacity;
    int index_base;
    int32_t* idx_rw;
    float* gate_rw;
    int32_t* u_idx;
    float* u_gate;
    // shared experts read the activations in place (experts below this id see every token, in token
    // order, so their block of xp would be a copy of x): their rows are numbered but not copied
    int inplace_experts = 0;
    // expert-parallel peer mode (else null): expert_dst[e] is where this rank's rows for expert e
    // start, possibly in another GPU's memory; row (pos - expert_offset[e]) of that segment is written
    void* const* expert_dst;
};

struct CombineParams {
    const void* y;            // [P][O]
    float* out;               // [T][O]
    int64_t T;
    int O, k_tot;
    const int32_t* idx;
    const float* gate;
    const int32_t* pair_pos;
};

// Grouped GEMM over the permuted rows: C[r][n] = sum_k A[r][k] * B[e(r)][n][k].
struct GroupGemmParams {
    const void* A;            // [P][K]
    const void* B0;           // [E][N][K]  (w1 for mode 1, w2 for mode 2)
    const void* B1;           // [E][N][K]  (w3 for mode 1, unused for mode 2)
    void* C;                  // [P][N]
    int N, K, E;
    int activation;           // mode 1: activation of the gate branch
    // mode 2 epilogue extras (StandardExpert, src/experts/standard.jl:38-55): C = act(A*B0^T + bias)
    const float* bias = nullptr;       // [E][N] FP32 or null
    int epilogue_act = -1;        // MOE_ACT_* applied after the bias, or -1 for none
    const int32_t* expert_offset; // [E+1]
    const int32_t* tile_prefix;   // [E+1]
    int32_t* status;
    // Scattered output (expert-parallel peer mode, GEMM 2; else seg_dst == null): the rows of expert e
    // form seg_per_expert consecutive segments, one per source rank; segment q starts at row
    // seg_start[e*seg_per_expert + q] and its rows are stored at seg_dst[e*seg_per_expert + q]
    // (a row-major [rows][N] block, possibly in another GPU's memory) instead of C.
    const int32_t* seg_start;
    void* const* seg_dst;
    int seg_per_expert;
    // GEMM 1 of the tensor-core path: experts below this id take their A rows from the activations x
    // themselves (row r of the expert = token r) through a second tensor map, instead of from A
    int inplace_experts = 0;
};

// Where row `row` of expert `e` of a grouped GEMM's output goes.
template <typename T>
__device__ __forceinline__ T* group_gemm_out_row(const GroupGemmParams& p, int e, int row) {
    if (!p.seg_dst) return reinterpret_cast<T*>(p.C) + (size_t)row * p.N;
    const int32_t* st = p.seg_start + (size_t)e * p.seg_per_expert;
    int q = 0;
    for (int i = 1; i < p.seg_per_expert; ++i)
        if (st[i] <= row) q = i;           // last segment starting at or before the row (empty ones skipped)
    return reinterpret_cast<T*>(p.seg_dst[(size_t)e * p.seg_per_expert + q]) + (size_t)(row - st[q]) * p.N;
}

// ---- chained launches (programmatic dependent launch) ------------------------------------------
// The kernels of a small forward are each a few microseconds long, so the time between the end of one
// and the start of the next is a large part of the call.  Launched as a chain, a kernel may be set up on
// the SMs (blocks scheduled, shared memory and barriers initialised) while its predecessor is still
// running; it calls chain_wait() before its first access to global memory, which returns when the
// predecessor has completed and its writes are visible, and chain_release() at its start lets its own
// successor be set up.  Both calls do nothing in a kernel that was launched the ordinary way.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Set by the forward call around its launches (per thread: a handle is driven by one thread at a time).
extern thread_local bool g_chain_launches;

template <class... P, class... A>
inline cudaError_t launch_kernel(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = g_chain_launches ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

// ---- launchers (each returns the number of kernels it launched, or <0 on a launch error) ---
int launch_router(const RouterParams& p, int x_dtype, int num_cta, int num_sms, cudaStream_t s);
int router_tokens_per_cta(int64_t T, int e_router, int num_sms);   // 64, 32 or 16
int router_e_pad(int e_router);          // router rows padded to a multiple of 8 (bucketed)
int router_d_pad(int D);                 // K rows of the K-major copy (multiple of 128)
int launch_router_transpose(const float* w, float* wt, int E, int D, cudaStream_t s);
// wt columns 0..E-1 = w, E..2E-1 = nw (the noise network), padded to router_e_pad(2E)
int launch_router_transpose_noise(const float* w, const float* nw, float* wt, int E, int D, cudaStream_t s);
int launch_scan(const ScanParams& p, cudaStream_t s);
// AuxiliaryFreeLoss.update_bias! on the device: bias/momentum [E] updated in place from expert_count [E]
int launch_aux_free_update(const int32_t* expert_count, int E, float* bias, float* bias_momentum, float learning_rate,
                           float momentum, cudaStream_t s);
int launch_permute(const PermuteParams& p, int x_dtype, int xp_dtype, int num_cta, cudaStream_t s);
int launch_combine(const CombineParams& p, int y_dtype, cudaStream_t s);
int launch_group_gemm_f32(const GroupGemmParams& p, int mode, int max_mtiles, int64_t rows, int num_sms,
                          cudaStream_t s);
int launch_gates_only(int gate_kind, int E, int S, int k, int index_base, const float* logits, const float* jitter_u,
                      float eps, int64_t T, int32_t* indices, float* gates, float* probs, cudaStream_t s);
int launch_loss_only(float alpha, float z_weight, int n_probs, int k, int index_base, const int32_t* indices,
                     const float* probs, const float* logits, int n_logits, int64_t T, float* loss,
                     cudaStream_t s);
int launch_transpose_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int rows_out,
                             int cols_out, int src_is_transposed, cudaStream_t s);

// tensor-core router for wide gates and BF16 activations (router_tc.cu)
struct RouterTcPlan;
RouterTcPlan* router_tc_plan_create();
void router_tc_plan_destroy(RouterTcPlan*);
int router_tc_e_pad(int e_router);       // padded router width of the tensor-core path, 0 = not offered for this width
// splits w (FP32 [E_router][D]) into w3 (BF16 [3*e_pad][D]) and encodes its tensor map; 1 = ready, 0 = not offered, <0 error
int router_tc_plan_set(RouterTcPlan*, const float* w, void* w3, int e_router, int D, cudaStream_t s);
// may this call take the tensor-core router?  (BF16 activations, 16-byte aligned, no noise network armed)
bool router_tc_usable(const RouterTcPlan*, const void* x, int x_dtype, bool noise_network_armed, int e_router, int D, int64_t T);
int launch_router_tc(const RouterTcPlan*, const RouterParams& p, int num_cta, int num_sms, int32_t* status, cudaStream_t s);
// K-major BF16 matrix [rows][K] as a 2-D tensor map with boxes of 64 x box_rows and 128-byte swizzle
bool tc_encode_bf16_2d(void* map, const void* base, uint64_t K, uint64_t rows, uint32_t box_rows);
// row-major FP32 matrix [rows][K] as a 2-D tensor map with plain boxes of box_k x box_rows (each <= 256)
bool tc_encode_f32_2d(void* map, const void* base, uint64_t K, uint64_t rows, uint32_t box_k, uint32_t box_rows);

// tcgen05 path (expert_tc.cu)
struct TcGemmPlan;  // tensor maps + geometry, owned by the handle
TcGemmPlan* tc_plan_create();
void tc_plan_destroy(TcGemmPlan*);
// (re)encodes the tensor maps; returns 0 or a negative MOE_ERR_* (message via out_msg)
int tc_plan_encode(TcGemmPlan*, const void* xp, const void* h, int64_t P_cap, int D, int H, int O, int E,
                   const void* w1, const void* w3, const void* w2, const char** out_msg);
// tensor map of this call's activations x [T][D] (BF16) for experts that read them in place; false if x does not qualify
bool tc_plan_set_x(TcGemmPlan*, const void* x, int64_t T, int D);
// stage 1: A = permuted rows, B = w1 (and w3 in mode 1); stage 2: A = hidden activations, B = w2.
// mode 1: gated pair with act(gate)*up epilogue; mode 2: single matrix (+ bias, + activation).
int launch_group_gemm_tc(const TcGemmPlan*, int stage, int mode, const GroupGemmParams& p, int max_tiles,
                         int num_sms, cudaStream_t s);
int launch_group_gemm_tc_dual(const TcGemmPlan*, int stage, int mode, const GroupGemmParams& p, int max_tiles, int num_sms,
                              cudaStream_t s);
int launch_group_gemm_tc2(const TcGemmPlan*, int stage, int mode, const GroupGemmParams& p, int max_tiles,
                          int num_sms, cudaStream_t s);
// one thread waits limit_us on an mbarrier nobody arrives on; 0 on success, the recorded status and waited time out
int run_bounded_wait_selftest(int limit_us, int32_t* status_out, int32_t* waited_us);

__host__ __device__ inline float bf16_bits_to_float(uint16_t b) {
    union { uint32_t u; float f; } v;
    v.u = ((uint32_t)b) << 16;
    return v.f;
}

}  // namespace moe
