// Expert-parallel exchange: all-to-all dispatch and combine of token rows between the ranks of
// one node over NVLink 5 / NVSwitch (peer stores from this library's own kernels by default, NCCL
// send/recv as the comparison mode).  The reference has no communication layer at all; the oracle
// for this path is the single-device layer on the concatenated batch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

struct EpState;

// Control block every rank exports to its peers (32-bit words): three rows of arrival flags
// (slot 0: rows dispatched, slot 1: expert outputs returned, slot 2: routing records posted), then
// two record tables (parity of the call number) with one record per rank.
constexpr int EP_MAX_WORLD = 32;
constexpr int EP_MAX_REC_WORDS = 272;     // >= num_experts + router rows + 3
constexpr int EP_CTL_FLAG_WORDS = 128;    // >= 3 * EP_MAX_WORLD
constexpr int EP_CTL_WORDS = EP_CTL_FLAG_WORDS + 2 * EP_MAX_WORLD * EP_MAX_REC_WORDS;

struct EpConfig {
    int rank, world;
    int E, E_probs, k_tot;
    int D, H, O;
    int elt;       // bytes per element of the row buffers (2 = BF16, 4 = FP32)
    int tile_m;    // m-tile height of the grouped GEMM that will run on the received rows
    int tile_m_alt;  // second tile height the caller may choose per call (0 = none)
    float alpha, z_weight;
    int32_t* status;   // the handle's device status word (bounded waits report DEV_TIMEOUT_PEER here)
};

struct EpCall {
    int64_t T;                     // local tokens
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
// Loss of a batch that was processed in chunks on one GPU, from the chunks' summed statistics:
// sums = {unused[E], prob sums[E_probs], lse^2 sum, unused, entropy sum} (FP32), the per-expert pair
// counts and T as integers, so that counts beyond 2^24 stay exact.
int launch_finish_loss(const float* sums, const int64_t* counts, int64_t T, int E, int E_probs, int k_tot, float alpha,
                       float z_weight, int training, float* u_loss, float* u_entropy, cudaStream_t s);
int ep_unique_id(void* id128, char* err, size_t errlen);
// Joins the group through a NON-BLOCKING NCCL communicator; the rendezvous is polled against
// timeout_ms (<= 0: the default of 30 s).  Every later wait on a collective uses the same deadline
// and ends in ncclCommAbort + MOE_ERR_TIMEOUT; after that the state refuses every call.
int ep_create(EpState** out, const EpConfig& cfg, const void* id128, int timeout_ms, char* err, size_t errlen);
void ep_destroy(EpState*);
int ep_set_timeout_ms(EpState*, int ms);
// device [E + E_probs + 3] words: this rank's record of the call = {int32 pair counts[E], float prob
// sums[E_probs], float lse^2 sum, int32 T, float entropy sum}; the scan kernel writes it
int32_t* ep_record_buffer(EpState*);
// nccl mode: records, dispatch, local experts (callback), combine
int ep_exchange_and_run(EpState*, const EpCall&, EpRunFn run, void* self, char* err, size_t errlen);
float ep_last_exchange_ms(EpState*);
// all ranks' largest local token count (collective, bounded)
int ep_max_tokens(EpState*, int64_t T_local, cudaStream_t s, int64_t* T_max, char* err, size_t errlen);

// ---- peer-memory mode (default): rows cross NVLink inside the permute and combine kernels ----
// Every rank exports its receive buffers with CUDA IPC; the permute kernel stores each row
// straight into the owner GPU's buffer, and the GEMM 2 epilogue stores every output row straight into
// the buffer of the GPU that owns the token, tile by tile while the GEMM runs; the combine kernel then
// reads local memory only.  Counts, statistics and the two barriers of a call travel through the
// exported control block (flag kernels with bounded waits); NCCL only carries the IPC handles when
// buffers grow.  MOE_B200_EP_MODE=nccl selects the send/recv path above.
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
// exchange of the records, host sync, layout, (collective) buffer growth, pointer tables
int ep_prepare(EpState*, int64_t T_local, cudaStream_t s, EpPlan* plan, char* err, size_t errlen);
// flag barrier over all ranks (one small kernel, bounded wait).  slot 0: after the permute kernel,
// "every rank's rows for my experts have landed"; slot 1: after GEMM 2, "the outputs of all my
// pairs have landed"
int ep_barrier(EpState*, int slot, cudaStream_t s, char* err, size_t errlen);
// Switch loss (+ z-loss) and entropy over all ranks' tokens from the gathered records.  chunk_mode:
// 0 = the call is a whole batch; 1 / 2 / 3 = first / middle / last chunk of a chunked host call
// (running totals are kept between the chunks, the last one writes the result)
int ep_finish_loss(EpState*, int training, int chunk_mode, float* u_loss, float* u_entropy, cudaStream_t s,
                   int64_t* launches, char* err, size_t errlen);
void ep_mark(EpState*, int i, cudaStream_t s);   // timing marks 0..3 around the two exchanges

}  // namespace moe
