/*
 * moe_b200.h - C ABI of libmoe_b200.so: the MoE-layer forward pass of MixtureOfExperts.jl
 * (router -> top-k -> dispatch -> GatedExpert FFN -> weighted combine -> Switch balance
 * loss) as hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * The reference has no FFI today; its operator API is Julia multiple dispatch.  Each entry
 * point below names the reference interface it stands in for (paths are relative to the
 * reference project root).  Host bindings (Julia ccall, Python ctypes) sit on top of
 * exactly these symbols; signatures use plain pointers and sizes only.
 *
 * Conventions
 *   - Every function returns MOE_OK (0) or a negative MOE_ERR_* code; nothing throws, traps
 *     or aborts across the boundary.  moe_last_error() gives the message for the calling
 *     thread.
 *   - Matrices follow the reference's memory: Julia arrays are column-major, so the
 *     (input_dim x T) input is T contiguous token vectors, (k x T) index/gate arrays are
 *     [T][k], (E x T) probability/logit arrays are [T][E], and the (output_dim x T) output
 *     is [T][output_dim].
 *   - A handle is not thread-safe (the reference layer mutates its own training_stats,
 *     src/core/moe_layer.jl:153, so it is not re-entrant either); distinct handles are
 *     independent.
 *   - Device entry points enqueue all work on the caller's stream and return without
 *     synchronising unless documented otherwise.  Caller-owned buffers must stay valid
 *     until the stream reaches the end of the call.
 *   - There is no CPU fallback: without a usable CUDA device every compute call fails
 *     with MOE_ERR_CUDA.
 *
 * Environment switches (experiments and comparisons; defaults are what the measurements use).
 * The first three are read when a handle is created, the others once per process:
 *   MOE_B200_PAIR=0|1|2        force the single-CTA (128-row tiles), the CTA-pair (256-row tiles, cta_group::2)
 *                              or the two-accumulator (256-row tiles, one CTA) tensor-core GEMM kernels
 *                              instead of the per-batch choice
 *   MOE_B200_HOST_CHUNKS=n     moe_layer_forward_host cuts batches of 8192 tokens and more into n
 *                              equal chunks (1 = no chunking) instead of its default schedule of 2/12/10/6/2 thirty-seconds
 *   MOE_B200_HOST_TIMELINE=1   print every chunk's copy and compute times to stderr
 *   MOE_B200_GROUP_M=n         m-tiles per group of the GEMM tile order (default 32)
 *   MOE_B200_ROUTER_TILE=16|32|64   force the token tile of the router and permute kernels
 *   MOE_B200_INPLACE_SHARED=0  shared experts' rows are copied by the permute like everybody's instead of being
 *                              read from the activations in place (comparison; read at handle creation)
 *   MOE_B200_ROUTER_TC=0       keep the FP32-FMA router kernel for wide routers too (comparison; read at
 *                              handle creation)
 *   MOE_B200_GRAPHS=0          small batches launch their kernels one by one instead of replaying a captured
 *                              CUDA graph (comparison; read at handle creation)
 *   MOE_B200_CHAIN=0           small batches launch their kernels without programmatic dependent launch
 *                              (comparison; read at handle creation)
 *   MOE_B200_EP_MODE=nccl      expert parallelism moves token rows with ncclSend/ncclRecv instead of
 *                              peer stores from the library's own kernels (read by moe_ep_init)
 */
#ifndef MOE_B200_H
#define MOE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define MOE_OK                 0
#define MOE_ERR_INVALID       -1   /* bad argument (the reference raises ArgumentError / error()) */
#define MOE_ERR_CUDA          -2   /* a CUDA runtime/driver call failed or no device */
#define MOE_ERR_UNSUPPORTED   -3   /* valid request this build does not implement */
#define MOE_ERR_STATE         -4   /* weights not set, EP not initialised, ... */
#define MOE_ERR_TIMEOUT       -5   /* a bounded wait gave up: a device-side wait (status word set) or, with
                                      expert parallelism, a rank that did not join a collective in time */
#define MOE_ERR_NCCL          -6   /* an NCCL call failed */

/* ---- enums (int32 in moe_config_t) ------------------------------------------------- */
/* gate_kind: which compute_gates method runs after the router GEMM */
#define MOE_GATE_TOPK          0   /* TopKGating(k)            src/gating/topk.jl:16-44      */
#define MOE_GATE_SWITCH        1   /* SwitchGating() = top-1   src/gating/switch.jl:7-11     */
#define MOE_GATE_SHARED_TOPK   2   /* SharedExpertGating(S, TopKGating(k), E)
                                      src/gating/advanced.jl:74-108 */
/* activation of GatedExpert (MoEConfig.activation, src/core/moe_layer.jl:10) */
#define MOE_ACT_SILU           0   /* x*sigmoid(x)  src/experts/gated.jl:36 */
#define MOE_ACT_GELU_TANH      1   /* NNlib.gelu (tanh approximation) */
#define MOE_ACT_RELU           2
#define MOE_ACT_IDENTITY       3
/* element types */
#define MOE_DTYPE_F32          0
#define MOE_DTYPE_BF16         1
/* compute_dtype: MOE_DTYPE_F32  = FP32 FMA on CUDA cores (1e-5 parity class)
 *                MOE_DTYPE_BF16 = BF16 operands on tcgen05 tensor cores, FP32 accumulate */
/* shared_mode */
#define MOE_SHARED_NONE        0
#define MOE_SHARED_GATING      1   /* via SharedExpertGating: experts 1..S are always selected */
#define MOE_SHARED_LAYER_BLEND 2   /* MoEConfig.num_shared_experts>0:
                                      forward_with_shared_experts, src/core/moe_layer.jl:158-185 */
/* expert_kind */
#define MOE_EXPERT_GATED       0   /* GatedExpert: w2(act.(w1 x) .* (w3 x))            src/experts/gated.jl:29-34    */
#define MOE_EXPERT_STANDARD    1   /* StandardExpert: w2(act.(w1 x .+ b1)) .+ b2       src/experts/standard.jl:38-55 */
/* memory layout of a weight matrix W with logical shape (out x in), y = W*x */
#define MOE_LAYOUT_IN_CONTIG   0   /* [out][in], in fastest: Llama2.jl (in x out) column-major
                                      (src/llama2/conversion.jl:277-331), NumPy (out,in) C-order */
#define MOE_LAYOUT_OUT_CONTIG  1   /* [in][out], out fastest: Flux Dense.weight (out x in)
                                      column-major (src/experts/gated.jl:18-24) */

/* Mirror of the MoEConfig fields the forward pass reads (src/core/moe_layer.jl:4-29). */
typedef struct moe_config {
    int32_t num_experts;      /* E, shared experts included */
    int32_t num_shared;       /* S (0 unless shared_mode != NONE) */
    int32_t top_k;            /* k of the routed gate (gate_type.k; MoEConfig.top_k is not read) */
    int32_t input_dim;        /* D */
    int32_t hidden_dim;       /* H */
    int32_t output_dim;       /* O */
    int32_t gate_kind;        /* MOE_GATE_*   */
    int32_t activation;       /* MOE_ACT_*    */
    int32_t compute_dtype;    /* MOE_DTYPE_*  */
    int32_t shared_mode;      /* MOE_SHARED_* */
    float   balance_alpha;    /* SwitchTransformerLoss(alpha), src/balancing/losses.jl:11-36 */
    float   z_loss_weight;    /* MoEConfig.z_loss_weight (added when training), moe_layer.jl:117-121 */
    int32_t index_base;       /* 0 or 1: base of expert ids written to `indices` (Julia: 1) */
    int32_t bias_gates_only;  /* 1: logit_bias changes indices/gates but not probs (the
                                 AuxiliaryFreeLoss hook, moe_layer.jl:137-140); 0: bias is
                                 part of the logits (a Dense router with bias) */
    float   capacity_factor;  /* MoEConfig.capacity_factor */
    int32_t drop_tokens;      /* MoEConfig.drop_tokens: when set and training != 0, a forward applies
                                 apply_capacity_constraint (src/core/moe_layer.jl:221-248): per expert
                                 the first ceil(capacity_factor*T/E) (token, slot) pairs in token order
                                 keep their slot, later ones get id index_base-1 and gate 0, and every
                                 token's gates are renormalised.  Not with LAYER_BLEND or expert parallel. */
    int32_t expert_kind;      /* MOE_EXPERT_* (MoEConfig.expert_type :gated / :standard) */
} moe_config_t;

typedef struct moe_layer moe_layer_t;   /* opaque: one per (layer, device) */

/* Optional outputs of a forward call; every pointer may be NULL.  Device pointers for
 * moe_layer_forward, host pointers for moe_layer_forward_host. */
typedef struct moe_forward_outputs {
    float*   loss;               /* [1]   balance loss (+ z-loss), 0 when training==0          */
    int32_t* indices;            /* [T][k_tot] expert ids, index_base-based                   */
    float*   gates;              /* [T][k_tot]                                                 */
    float*   probs;              /* [T][E_probs]   router_probs                                */
    float*   logits;             /* [T][E_router]  router_logits                               */
    int64_t* tokens_per_expert;  /* [E]  counts of THIS call (training_stats[:tokens_per_expert]
                                         accumulates them, src/core/moe_layer.jl:250-264)      */
    float*   routing_entropy;    /* [1]  mean_t(-sum_i p*log(p+1e-8))                          */
} moe_forward_outputs_t;

/* ---- lifecycle --------------------------------------------------------------------- */

/* MoELayer(config) (src/core/moe_layer.jl:44-63) / create_cuda_moe (src/cuda/utils.jl).
 * Validates the config, binds the handle to CUDA device `device`, allocates weight storage. */
int moe_layer_create(const moe_config_t* cfg, int device, moe_layer_t** out);

/* Stands in for the weight copy of to_cuda / create_synchronized_moe_pair
 * (src/cuda/utils.jl:4-15, src/amdgpu/utils.jl:62-105): copies and repacks the three
 * matrices of expert `expert` (0-based) into the handle; the caller's arrays may be freed
 * after return.  w1,w3: (H x D); w2: (O x H).  src_dtype MOE_DTYPE_*; layout MOE_LAYOUT_*;
 * src_is_device != 0 if the pointers are device pointers on the handle's device; the call then
 * first waits for all work queued on the device, so sources still being produced on any of the
 * caller's streams are complete before they are read.  Synchronises before returning. */
int moe_layer_set_expert(moe_layer_t*, int expert, const void* w1, const void* w2, const void* w3,
                         int src_dtype, int layout, int src_is_device);

/* The same for a StandardExpert (src/experts/standard.jl:8-36; create_cuda_experts, src/cuda/types.jl):
 * w1 (H x D), w2 (O x H) in src_dtype/layout, b1 [H] and b2 [O] FP32 (NULL = no bias), all host or all
 * device pointers.  Dropout inside the expert is not offered (expert_dropout must be 0). */
int moe_layer_set_expert_standard(moe_layer_t*, int expert, const void* w1, const float* b1, const void* w2,
                                  const float* b2, int src_dtype, int layout, int src_is_device);

/* Weight image: everything serialize_moe_layer stores for one MoE layer (router_weight and every
 * expert's w1/w2/w3, src/llama2/utils.jl:258-303; plus biases and the noise network where the layer
 * has them) as ONE host blob in the library's own device layout and compute dtype.  A 128-byte
 * header ("MOEB200W", version, dtype, expert kind, dims, section offsets) is followed by 256-byte
 * aligned sections.  Import is a plain host->device copy per section, no repacking: it needs a
 * handle created with the same config (and the same expert-parallel split) and replaces
 * moe_layer_set_expert / moe_layer_set_router.  `bytes` is the size of the caller's buffer. */
int64_t moe_layer_weights_image_bytes(moe_layer_t*);          /* -1 on error (weights not all set) */
int moe_layer_export_weights(moe_layer_t*, void* dst_host, int64_t bytes);
int moe_layer_import_weights(moe_layer_t*, const void* src_host, int64_t bytes);

/* Router.weight (src/core/router.jl:14-23): FP32 (E_router x D), E_router = E - S.
 * (E_router = E in GATING mode: the first S rows are present but unused by the gate.)
 * logit_bias: optional FP32 [E_router] added to the logits (see bias_gates_only). */
int moe_layer_set_router(moe_layer_t*, const float* w, const float* logit_bias,
                         int layout, int src_is_device);

/* Training-time router noise (src/core/router.jl:32-41, noise_scale > 0 without a noise network):
 * `noise` is a caller-owned DEVICE array [T][E_router] of standard-normal draws (the caller keeps
 * its own random stream, as Julia's randn does in the reference); forward calls with training != 0
 * gate on logits + noise_scale*noise until it is replaced or cleared with NULL.  The z-loss still
 * comes from the noise-free logits, like the reference's second router pass. */
int moe_layer_set_router_noise(moe_layer_t*, const float* noise, float noise_scale);

/* AuxiliaryFreeLoss.update_bias! (src/balancing/auxiliary_free.jl:36-71) on the device: once enabled,
 * every training forward ends with a one-block kernel that turns the call's per-expert counts into
 * the momentum update of the logit bias (given to moe_layer_set_router) and mean-centres it, so
 * the next call selects with the new bias and no count ever travels to the host.  `bias_momentum`
 * (host, [E_router], NULL = zeros) and `update_counter` seed the state; update_freq as in the
 * reference.  Not with expert parallelism or num_shared_experts > 0.  enable = 0 switches it off. */
int moe_layer_set_aux_free(moe_layer_t*, int enable, float learning_rate, float momentum, int update_freq,
                           const float* bias_momentum, int64_t update_counter);
/* Reads the state back into HOST arrays (each nullable); synchronises the device. */
int moe_layer_aux_free_state(moe_layer_t*, float* bias, float* bias_momentum, int64_t* update_counter);

/* Router.noise_weight (src/core/router.jl:20, use_noise_network = true): an (E_router x D) FP32 matrix
 * in `layout`; once set, armed noise becomes logits + noise_scale * (noise .* softplus(noise_w x))
 * (router.jl:33-37), the second projection riding in the same gate GEMM.  Call after
 * moe_layer_set_router; needs 2*E_router <= 128.  NULL removes the network. */
int moe_layer_set_router_noise_network(moe_layer_t*, const float* noise_w, int layout, int src_is_device);

/* Number of values per token in indices/gates (k_tot), probs (E_probs), logits (E_router). */
int moe_layer_dims(const moe_layer_t*, int32_t* k_tot, int32_t* e_probs, int32_t* e_router);

/* (moe::MoELayer)(x; training) (src/core/moe_layer.jl:107-128) and cuda_moe_forward!
 * (src/cuda/layer.jl:3-32) on device buffers.  x: [T][D] of x_dtype; out: [T][O] FP32.
 * Workspace grows to the largest T seen (no 1024-token cap); growing it synchronises. */
int moe_layer_forward(moe_layer_t*, const void* x, int x_dtype, int64_t T, int training,
                      float* out, const moe_forward_outputs_t* opt, void* cuda_stream);

/* Same call with HOST buffers: stages x host->device, runs the layer, copies the results
 * back and synchronises.  This is the path the per-token Llama2 glue uses
 * (moe_ffn_forward!, src/llama2/inference.jl:58-121). */
int moe_layer_forward_host(moe_layer_t*, const void* x, int x_dtype, int64_t T, int training,
                           float* out, const moe_forward_outputs_t* opt);

/* compute_gates(gate, logits) (src/gating/base.jl:22, topk.jl:24-44, advanced.jl:80-108) as a
 * stand-alone device operator: logits [T][E] FP32 in; indices/gates/probs out (nullable). */
int moe_compute_gates(int gate_kind, int num_experts, int num_shared, int top_k, int index_base,
                      const float* logits, int64_t T,
                      int32_t* indices, float* gates, float* probs, void* cuda_stream);

/* compute_gates(JitterGating(base_gate, eps), logits; training = true) (src/gating/switch.jl:20-33):
 * the base gate on logits .* (1 .+ (2 .* u .- 1) .* eps), `jitter_u` [T][E] being the caller's
 * uniform [0,1) draws (device).  Inside the layer the reference's Router never passes `training`
 * to compute_gates, so a JitterGating layer routes exactly like its base gate; this operator serves
 * direct calls. */
int moe_compute_gates_jitter(int gate_kind, int num_experts, int num_shared, int top_k, int index_base,
                             const float* logits, const float* jitter_u, float eps, int64_t T,
                             int32_t* indices, float* gates, float* probs, void* cuda_stream);

/* compute_loss(SwitchTransformerLoss(alpha), indices, probs) (src/balancing/losses.jl:15-36)
 * plus z_weight * mean(logsumexp(logits)^2) when logits != NULL (losses.jl:103-114).
 * indices [T][k] (index_base-based), probs [T][n_probs]; writes one FP32 to `loss` (device). */
int moe_compute_loss(float alpha, float z_weight, int n_probs, int k, int index_base,
                     const int32_t* indices, const float* probs, const float* logits,
                     int n_logits, int64_t T, float* loss, void* cuda_stream);

/* Stage timing.  moe_layer_set_profiling(h, slots) keeps CUDA events for the last `slots`
 * forward calls (0 switches it off; it synchronises the device).  moe_layer_stage_ms gives the
 * device time in milliseconds of each stage of the call made `calls_back` calls ago (0 = the
 * last one), in order {router, scan+loss, permute, gemm1, gemm2, combine, exchange}; with
 * expert parallelism gemm1 includes the dispatch and `exchange` is dispatch + combine of the
 * last call.  It synchronises on that call's events. */
int moe_layer_set_profiling(moe_layer_t*, int slots);
int moe_layer_stage_ms(moe_layer_t*, int calls_back, float ms[7]);

/* Rows per m-tile of the expert GEMMs a forward of T local tokens takes on one GPU: 256 = CTA-pair
 * tensor-core kernel, 128 = single-CTA tensor-core kernel, 16 = FP32 kernels (no counterpart in the
 * reference: a profiling aid).  Negative = error. */
int moe_layer_tile_rows(moe_layer_t*, int64_t T);

/* Which tensor-core kernel a batch of T tokens gets on a layer without expert parallelism: 0 = single
 * CTAs on 128-row tiles, 1 = CTA pairs (cta_group::2) on 256-row tiles, 2 = single CTAs with two
 * accumulators sharing a weight tile on 256-row tiles; always 0 for FP32 layers.  A profiling aid
 * like moe_layer_tile_rows.  Negative = error. */
int moe_layer_gemm_kernel(moe_layer_t*, int64_t T);

/* Number of kernel launches of this library issued through the handle since creation. */
int64_t moe_layer_launch_count(const moe_layer_t*);

/* Routers with 33..80 rows fed BF16 activations run their gate GEMM on the tensor cores (an exact
 * three-way BF16 split of the FP32 router matrix, FP32 accumulation) and re-evaluate with FP32 FMAs
 * every token whose top-(k+1) ranking has two neighbours closer than 3e-5 * max(1, |logit|).  *tokens
 * receives how many tokens were re-evaluated through this handle since creation (0 for layers
 * that never take that path).  A diagnostic without counterpart in the reference; synchronises. */
int moe_layer_router_rechecks(moe_layer_t*, int64_t* tokens);

/* Small batches (T * selected experts per token <= 4096, no expert parallelism, no device bias
 * update, profiling off): the second forward call with the same arguments -- x, out and optional
 * output pointers, T, dtype, training flag, noise buffer -- is captured into a CUDA graph on a
 * stream of the handle and that call and later ones replay it on the caller's stream (one
 * launch instead of six; results are those of the same kernels).  A replay reads the buffers'
 * current contents.  Setters, workspace growth and moe_layer_set_profiling drop the graphs;
 * calls made while the caller's stream is itself being captured launch plainly into that
 * capture.  *replays receives the number of forward calls served by a replay since creation.
 * No counterpart in the reference. */
int moe_layer_graph_replays(const moe_layer_t*, int64_t* replays);

/* Value of the device status word after the last synchronising call (0 = clean). */
int moe_layer_device_status(moe_layer_t*, int32_t* status);

/* Self-test of the bounded waits the tensor-core kernels are built on (no counterpart in the
 * reference): launches one thread on `device` that waits on an mbarrier nobody ever arrives on,
 * with a limit of `limit_us` microseconds (1..1000000), through the same wait routine the GEMM
 * kernels use.  The wait must give up: *status_out receives the device status code it recorded
 * (1 = "waited too long for a TMA stage") and *waited_us how long the thread waited.  Nothing
 * faults or hangs; the context stays usable.  Synchronises the device. */
int moe_selftest_bounded_wait(int device, int limit_us, int32_t* status_out, int32_t* waited_us);

/* ---- expert parallelism (no counterpart in the reference: it has no communication layer) */

/* Fill `id128` (128 bytes) with a fresh NCCL unique id; rank 0 calls it and ships the
 * bytes to the other ranks by any host channel. */
int moe_ep_unique_id(void* id128);

/* Joins the handle to an expert-parallel group of `world` ranks (one process per GPU, at most 32).
 * Experts are block-partitioned: rank r owns experts [r*E/world, (r+1)*E/world); only those
 * need moe_layer_set_expert.  Tokens stay data-parallel; the router is replicated.
 * After this, moe_layer_forward dispatches token rows with an all-to-all over NVLink,
 * runs the local experts, returns the rows with a second all-to-all and combines them;
 * the balance loss is reduced over all ranks' tokens.
 *   - Every forward is a collective: all ranks call it the same number of times (a rank without
 *     tokens calls it with T = 0).  moe_layer_forward then SYNCHRONISES WITH THE HOST once per call
 *     (the routing counts of all ranks are read back to lay out the exchange), so it is not
 *     asynchronous under expert parallelism.
 *   - Per-expert pair counts travel as 32-bit integers and are summed in 64 bits: the loss is exact
 *     as long as one rank's pairs per call stay below 2^31.
 *   - Failure handling: the group is joined through a non-blocking NCCL communicator and every
 *     wait on another rank -- on the host or in a kernel -- is bounded by the timeout below.  A rank
 *     that does not arrive makes the call return MOE_ERR_TIMEOUT (or MOE_ERR_NCCL for an NCCL
 *     error); the communicator is aborted, the GPU stays usable, and every later expert-parallel
 *     call on the handle returns MOE_ERR_STATE.  A rank that cannot allocate its receive buffers
 *     still takes part in the exchange of that fact, so all ranks return MOE_ERR_CUDA together. */
int moe_ep_init(moe_layer_t*, const void* id128, int rank, int world);

/* Deadline, in milliseconds, of every wait on another rank (default 30000; device-side waits use
 * min(timeout, 10000)).  May be called before moe_ep_init (it then also bounds the rendezvous) or
 * after it.  All ranks should use the same value. */
int moe_ep_set_timeout_ms(moe_layer_t*, int timeout_ms);

/* Host-only helper (no CUDA, no NCCL): the row layout one rank uses for the dispatch and the
 * combine, from the all-gathered pair counts counts[world][num_experts].  send_off[E+1]: first
 * row, in the rank's permuted buffer, of its pairs for expert e; recv_off[E/world][world]:
 * first received row of the pairs rank r sends to local expert el; local_off[E/world+1] and
 * tile_prefix[E/world+1]: received rows grouped by local expert and their tile_m-row tile
 * prefix.  Returns the number of rows the rank receives, or a negative MOE_ERR_*.  A forward
 * call computes exactly this internally; it is exported so the exchange can be checked without
 * GPUs. */
int64_t moe_ep_layout(const int32_t* counts, int world, int num_experts, int rank, int tile_m,
                      int64_t* send_off, int64_t* recv_off, int32_t* local_off, int32_t* tile_prefix);

int moe_layer_destroy(moe_layer_t*);

/* ---- routing without any allocation -------------------------------------------------------
 * No counterpart in the reference.  For callers that cannot allocate device memory -- a
 * process that gives all of HBM to its own pools at start-up so that a later cudaMalloc fails,
 * or a latency-critical loop that cannot take the device-wide synchronisation an allocation or
 * free implies -- this runs the layer's fused router (gate GEMM, softmax, top-k, renormalised
 * gates) and its Switch + z loss with the kernels' scratch held in a file-scope device array
 * of moe_route_static_scratch_bytes() bytes (8 MiB, held by every GPU that loads the library
 * until the process exits).  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   x [T][input_dim] (x_dtype), router_w FP32 [num_experts][input_dim] (input contiguous),
 *   logit_bias FP32 [num_experts] or NULL: device pointers owned by the caller.
 *   indices/gates [T][k_tot] (k_tot = top_k, + num_shared for MOE_GATE_SHARED_TOPK), probs
 *   [T][num_experts] (nullable), loss [1] (nullable; 0 is written when training == 0): device.
 * Sizes whose scratch does not fit the array are rejected with MOE_ERR_INVALID (the message
 * says how much was needed); MoEConfig.num_shared_experts (LAYER_BLEND) is not offered here.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress) with
 * that device current; make that first call outside any stream capture.  All calls share the
 * one array, which keeps the previous call's contents (nothing in it needs clearing: every
 * region is rewritten before it is read); two calls whose kernels overlap on the GPU -- from
 * two streams or two threads -- race on it, so serialise them.  Errors of this entry point
 * are reported by moe_route_static_error(). */
int moe_route_static(int gate_kind, int num_experts, int num_shared, int top_k, int index_base,
                     const void* x, int x_dtype, int64_t T, int input_dim,
                     const float* router_w, const float* logit_bias,
                     float balance_alpha, float z_loss_weight, int training,
                     int32_t* indices, float* gates, float* probs, float* loss, void* cuda_stream);
int64_t moe_route_static_scratch_bytes(void);
const char* moe_route_static_error(void);

const char* moe_last_error(void);     /* thread-local message of the last failure */
const char* moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H */
