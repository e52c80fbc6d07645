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
int ep_unique_id(void* id128, char* err, size_t errlen);
int ep_create(EpState** out, const EpConfig& cfg, const void* id128, char* err, size_t errlen);
void ep_destroy(EpState*);
float* ep_sums_buffer(EpState*);   // device [E + E_probs + 3]: counts, prob sums, lse^2, T, entropy
int ep_exchange_and_run(EpState*, const EpCall&, EpRunFn run, void* self, int64_t* launches, char* err,
                        size_t errlen);
float ep_last_exchange_ms(EpState*);

}  // namespace moe
