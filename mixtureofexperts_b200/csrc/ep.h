// Expert-parallel exchange: all-to-all dispatch and combine of token rows between the ranks of
// one node over NCCL (NVLink 5 / NVSwitch).  The reference has no communication layer at all;
// the oracle for this path is the single-device layer on the concatenated batch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

struct EpState;

struct EpConfig {
    int rank, world;
    int E, E_probs, k_tot;
    int D, H, O;
    int elt;       // bytes per element of the row buffers (2 = BF16, 4 = FP32)
    int tile_m;    // m-tile height of the grouped GEMM that will run on the received rows
    int tile_m_alt;  // second tile height the caller may choose per call (0 = none)
    float alpha, z_weight;
};

struct EpCall {
    int64_t T;                     // local tokens
    int training;
    float* u_loss;                 // device, nullable
    float* u_entropy;              // device, nullable
    const void* xs;                // [pairs][D] rows grouped by global expert (send layout)
    void* y_back;                  // [pairs][O] expert outputs returned in the send layout
    const int32_t* expert_count;   // device [E], local counts per global expert
    const int32_t* expert_offset;  // device [E+1]
    cudaStream_t stream;
};

// Runs the expert GEMM pair on the received rows.
typedef int (*EpRunFn)(void* self, const void* a_in, void* h_buf, void* y_buf, const int32_t* expert_offset,
                       const int32_t* tile_prefix, int64_t rows, int n_experts, int64_t cap_rows, cudaStream_t s);

// Row layout of one rank's exchange from the all-gathered pair counts cnt[W][E] (host only).
// send_off[E+1]: first row, in this rank's permuted buffer, of the pairs routed to expert e.
// recv_off[per][W]: first received row of the pairs rank r sends to local expert el.
// local_off[per+1], tile_prefix[per+1]: the received rows grouped by local expert and their
// m-tile prefix (tile_m rows per tile).  Returns the number of rows this rank receives.
int64_t ep_plan_layout(const int32_t* cnt, int W, int E, int me, int tile_m, int64_t* send_off, int64_t* recv_off,
                       int32_t* local_off, int32_t* tile_prefix);
// Loss from summed statistics {counts[E], prob sums[E_probs], lse^2, T, entropy}: the Switch loss
// (+ z-loss) over all the tokens the sums cover.  Used for all ranks' tokens (expert parallel) and
// for all chunks of a chunked host call.
int launch_finish_loss(const float* sums, int E, int E_probs, int k_tot, float alpha, float z_weight, int training,
                       float* u_loss, float* u_entropy, cudaStream_t s);
int ep_unique_id(void* id128, char* err, size_t errlen);
int ep_create(EpState** out, const EpConfig& cfg, const void* id128, char* err, size_t errlen);
void ep_destroy(EpState*);
float* ep_sums_buffer(EpState*);   // device [E + E_probs + 3]: counts, prob sums, lse^2, T, entropy
int ep_exchange_and_run(EpState*, const EpCall&, EpRunFn run, void* self, int64_t* launches, char* err,
                        size_t errlen);
float ep_last_exchange_ms(EpState*);

// ---- peer-memory mode (default): rows cross NVLink inside the permute and combine kernels ----
// Every rank exports its receive buffers with CUDA IPC; the permute kernel stores each row
// straight into the owner GPU's buffer, and the GEMM 2 epilogue stores every output row straight into
// the buffer of the GPU that owns the token, tile by tile while the GEMM runs; the combine kernel then
// reads local memory only.  NCCL only carries the small control collectives (counts, the loss sums that
// double as a barrier, one more barrier).  MOE_B200_EP_MODE=nccl selects the send/recv path above.
struct EpPlan {
    int64_t rows;                     // rows this rank received
    int64_t rows_cap;                 // capacity (rows) of the receive buffers
    void* xr;                         // [rows_cap][D] received rows (this GPU's memory)
    void* hr;                         // [rows_cap][H]
    void* yb;                         // [pairs_cap][O] outputs of THIS rank's pairs, in its send (pair_pos) order;
                                      // written by the owners of the experts from their GEMM 2 epilogues
    const int32_t* d_seg_start;       // [per][world] first received row of the pairs of source rank s, expert el
    void* const* d_seg_dst;           // [per][world] where that segment's outputs go (rank s's yb)
    const int32_t* d_local_off;       // [per+1] received rows grouped by local expert
    const int32_t* d_tile_prefix;     // [per+1] for EpConfig.tile_m rows per tile
    const int32_t* d_tile_prefix_alt; // [per+1] for EpConfig.tile_m_alt rows per tile (0 = none)
    void* const* d_expert_dst;        // [E] where this rank's rows for expert e start (a peer's xr)
};
bool ep_peer_mode(const EpState*);
int ep_world(const EpState*);
// all-gather of the counts, host sync, layout, (collective) buffer growth, pointer tables
int ep_prepare(EpState*, const int32_t* d_expert_count, cudaStream_t s, EpPlan* plan, char* err, size_t errlen);
// all-reduce of the loss sums; completes only when every rank has issued it, i.e. after every
// rank's permute kernel: the barrier between dispatch and the expert GEMMs
int ep_sums_barrier(EpState*, cudaStream_t s, char* err, size_t errlen);
// barrier between the expert GEMMs and the combine kernels that read peers' outputs
int ep_barrier(EpState*, cudaStream_t s, char* err, size_t errlen);
int ep_finish_loss(EpState*, int training, float* u_loss, float* u_entropy, cudaStream_t s, int64_t* launches,
                   char* err, size_t errlen);
void ep_mark(EpState*, int i, cudaStream_t s);   // timing marks 0..3 around the two exchanges

}  // namespace moe
