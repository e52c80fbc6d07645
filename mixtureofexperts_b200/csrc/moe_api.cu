// C ABI of libmoe_b200 (declared in include/moe_b200.h): handle lifecycle, weight repack,
// workspace management and the forward pipeline
//     router -> scan+loss -> permute -> grouped GEMM 1 (gate/up + act) -> grouped GEMM 2 -> combine
// that replaces (moe::MoELayer)(x; training) (src/core/moe_layer.jl:107-156) and
// cuda_moe_forward! (src/cuda/layer.jl:3-32).  No CPU fallback exists in this file: every
// compute entry point fails with MOE_ERR_CUDA when the device is unusable.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "ep.h"

namespace moe {
thread_local bool g_chain_launches = false;
}
using namespace moe;

namespace {

// Launches made while one of these is alive (and armed) are chained to their predecessors.
struct ChainScope {
    bool before;
    explicit ChainScope(bool on) : before(g_chain_launches) { g_chain_launches = on; }
    ~ChainScope() { g_chain_launches = before; }
};

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(expr)                                                                                   \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess) return fail(MOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

size_t dtype_size(int d) { return d == MOE_DTYPE_BF16 ? 2 : 4; }

template <typename T>
int dev_alloc(T** p, size_t n) {
    *p = nullptr;
    if (n == 0) n = 1;
    CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(p), n * sizeof(T)));
    return MOE_OK;
}
template <typename T>
void dev_free(T*& p) {
    if (p) cudaFree(p);
    p = nullptr;
}

}  // namespace

struct moe_layer {
    moe_config_t cfg;
    int device = 0;
    int num_sms = 0;
    int E = 0, S = 0, k = 0, k_tot = 0, E_router = 0, E_probs = 0;
    // expert range held by this handle ([0,E) unless expert-parallel)
    int e_lo = 0, e_hi = 0;

    // weights in the compute dtype, [E_local][out][in]
    void* w1 = nullptr;
    void* w3 = nullptr;
    void* w2 = nullptr;
    float* b1 = nullptr;         // [E_local][H] FP32, standard experts only
    float* b2 = nullptr;         // [E_local][O]
    float* router_w = nullptr;   // [E_router][D]
    float* router_wt = nullptr;  // [D_pad][E_pad] K-major zero-padded copy read by the router kernel
    float* router_nw = nullptr;  // [E_router][D] noise network (Router.noise_weight), or null
    float* router_wt_noise = nullptr;  // [D_pad][e_pad(2 E_router)]: router columns, then noise-network columns
    float* router_bias = nullptr;
    bool has_bias = false, router_set = false;
    // tensor-core router (wide gates, BF16 activations): split router matrix, its plan, scratch
    RouterTcPlan* rplan = nullptr;
    void* router_w3 = nullptr;      // BF16 [3*e_pad][D]: hi, mid, lo parts of router_w
    float* tc_logits = nullptr;     // workspace [T_cap][e_pad]
    int32_t* tc_recheck = nullptr;  // tokens re-evaluated with FP32 FMAs since creation
    bool router_tc_enabled = true;  // MOE_B200_ROUTER_TC=0 keeps the FP32-FMA router (comparison)
    bool inplace_shared = true;     // MOE_B200_INPLACE_SHARED=0: shared experts' rows are copied by the permute too
    // AuxiliaryFreeLoss.update_bias! on the device (moe_layer_set_aux_free)
    bool aux_free = false;
    float aux_lr = 0.f, aux_momentum = 0.f;
    int aux_freq = 1;
    int64_t aux_counter = 0;
    float* bias_momentum = nullptr;   // [E_router]
    const float* noise = nullptr;   // caller-owned device draws for the next training forward
    float noise_scale = 0.f;
    std::vector<char> expert_set;
    void* stage_w = nullptr;     // device staging for host-side weight sources
    size_t stage_w_bytes = 0;

    // workspace (sized for T_cap tokens)
    int64_t T_cap = 0;
    int64_t P_cap = 0;
    int32_t* idx = nullptr;
    float* gate = nullptr;
    int32_t* pair_pos = nullptr;
    int32_t* row_token = nullptr;
    int32_t* cta_counts = nullptr;
    float* cta_psum = nullptr;
    double* cta_entropy = nullptr;
    int32_t* expert_count = nullptr;
    int32_t* expert_offset = nullptr;
    int32_t* tile_prefix = nullptr;
    float* loss_dev = nullptr;
    void* xp = nullptr;
    void* h = nullptr;
    void* y = nullptr;
    int32_t* status = nullptr;
    TcGemmPlan* plan = nullptr;
    bool plan_dirty = true;
    const void* plan_a1 = nullptr;   // what the tensor maps were last encoded for
    const void* plan_a2 = nullptr;
    int64_t plan_rows = 0;

    // host-call staging
    cudaStream_t stream = nullptr;
    void* hx = nullptr;
    size_t hx_bytes = 0;
    float* hout = nullptr;
    size_t hout_bytes = 0;
    void* hopt = nullptr;
    size_t hopt_bytes = 0;
    // pinned host staging of small host calls: [status word, padded to 256 | x | out | optional outputs].
    // Copies between pageable memory and the device block the host one by one; through this block a
    // small call is one copy in, three copies out and a single wait.
    char* pin = nullptr;
    size_t pin_bytes = 0;
    // device side of small host calls: [status word, padded to 256 | out | optional outputs], one block
    // so that everything a small call returns comes back in a single copy (`status` points at its start)
    char* small_dev = nullptr;
    static constexpr size_t PIN_SMALL_CALL = 1 << 20;   // calls moving no more than this go through `pin`
    // chunked host calls: copy-in / compute / copy-out overlap on three streams
    static constexpr int MAX_CHUNKS = 8;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[MAX_CHUNKS] = {}, ev_done[MAX_CHUNKS] = {};
    // MOE_B200_HOST_TIMELINE=1: timed events around every chunk's copies, printed to stderr per call
    bool timeline = false;
    cudaEvent_t ev_t0 = nullptr, ev_in0[MAX_CHUNKS] = {}, ev_out1[MAX_CHUNKS] = {};
    float* chunk_acc = nullptr;      // [E + E_probs + 3] summed statistics of the chunks
    int64_t* chunk_tpe_acc = nullptr;  // [E]

    // profiling: a ring of event sets, one set per forward call
    int prof_slots = 0;
    std::vector<cudaEvent_t> ev;   // [prof_slots][8]
    int64_t prof_calls = 0;
    int prof_cur = 0;
    int64_t launches = 0;

    EpState* ep = nullptr;
    int ep_timeout_ms = 0;          // moe_ep_set_timeout_ms before moe_ep_init; 0 = default

    // Small batches: a forward call is a chain of six short launches whose host cost is larger than
    // their device time.  The second call with the same arguments (pointers, T, flags) is captured
    // into a CUDA graph on the handle's own stream and later calls replay it on the caller's stream.
    struct GraphEntry {
        const void* x = nullptr;
        int x_dtype = 0;
        int64_t T = 0;
        int training = 0;
        float* out = nullptr;
        moe_forward_outputs_t opt = {};   // loss / tokens_per_expert / routing_entropy: only whether they are wanted
        const float* noise = nullptr;
        float noise_scale = 0.f;
        cudaGraphExec_t exec = nullptr;
        bool refused = false;       // capture failed once: this key stays on plain launches
        int launches = 0;           // kernels inside the graph
        uint64_t tick = 0;          // last use (least recently used entry is replaced)
    };
    static constexpr int MAX_GRAPHS = 16;
    static constexpr int64_t GRAPH_MAX_PAIRS = 4096;   // T * k_tot above this: launches are no longer the cost
    std::vector<GraphEntry> graphs;
    // a graph writes loss, entropy and the per-expert counts into this block of the handle, and one
    // small kernel after the replay hands them to the caller's pointers (callers allocate those
    // afresh for every call, so they cannot be part of the key): [loss, entropy, pad, pad | int64 counts[E]]
    float* graph_small = nullptr;
    uint64_t graph_tick = 0;
    int64_t graph_replays = 0;
    bool graphs_enabled = true;     // MOE_B200_GRAPHS = 0: every call launches its kernels one by one
    bool chain_enabled = true;      // MOE_B200_CHAIN = 0: small batches launch their kernels without chaining
    bool capturing = false;         // forward_small is recording a graph: its launches are not chained

    // experiment switches of the environment, read once when the handle is created
    int force_pair = -1;            // MOE_B200_PAIR = 0 / 1 / 2: force the single-CTA / CTA-pair / two-accumulator GEMM kernels
    int host_chunks = 0;            // MOE_B200_HOST_CHUNKS = n: n equal chunks per large host call
    bool host_timeline = false;     // MOE_B200_HOST_TIMELINE = 1: print every chunk's copy/compute times
};

namespace {

int validate_config(const moe_config_t& c) {
    if (c.num_experts < 1 || c.num_experts > MAX_EXPERTS)
        return fail(MOE_ERR_INVALID, "num_experts must be in 1..%d (got %d)", MAX_EXPERTS, c.num_experts);
    if (c.input_dim < 1 || c.hidden_dim < 1 || c.output_dim < 1)
        return fail(MOE_ERR_INVALID, "input_dim, hidden_dim and output_dim must be positive");
    if (c.gate_kind < MOE_GATE_TOPK || c.gate_kind > MOE_GATE_SHARED_TOPK)
        return fail(MOE_ERR_INVALID, "unknown gate_kind %d", c.gate_kind);
    if (c.activation < MOE_ACT_SILU || c.activation > MOE_ACT_IDENTITY)
        return fail(MOE_ERR_INVALID, "unknown activation %d", c.activation);
    if (c.expert_kind != MOE_EXPERT_GATED && c.expert_kind != MOE_EXPERT_STANDARD)
        return fail(MOE_ERR_INVALID, "unknown expert_kind %d", c.expert_kind);
    if (c.compute_dtype != MOE_DTYPE_F32 && c.compute_dtype != MOE_DTYPE_BF16)
        return fail(MOE_ERR_INVALID, "unknown compute_dtype %d", c.compute_dtype);
    if (c.shared_mode < MOE_SHARED_NONE || c.shared_mode > MOE_SHARED_LAYER_BLEND)
        return fail(MOE_ERR_INVALID, "unknown shared_mode %d", c.shared_mode);
    if (c.index_base != 0 && c.index_base != 1) return fail(MOE_ERR_INVALID, "index_base must be 0 or 1");
    if ((c.gate_kind == MOE_GATE_SHARED_TOPK) != (c.shared_mode == MOE_SHARED_GATING))
        return fail(MOE_ERR_INVALID, "gate_kind SHARED_TOPK and shared_mode GATING go together");
    if (c.shared_mode == MOE_SHARED_NONE && c.num_shared != 0)
        return fail(MOE_ERR_INVALID, "num_shared must be 0 when shared_mode is NONE");
    if (c.shared_mode != MOE_SHARED_NONE && (c.num_shared < 1 || c.num_shared >= c.num_experts))
        return fail(MOE_ERR_INVALID, "num_shared must be in 1..num_experts-1 for this shared_mode");
    const int k = (c.gate_kind == MOE_GATE_SWITCH) ? 1 : c.top_k;
    const int e_router = c.shared_mode == MOE_SHARED_LAYER_BLEND ? c.num_experts - c.num_shared : c.num_experts;
    const int routed = c.shared_mode == MOE_SHARED_GATING ? c.num_experts - c.num_shared : e_router;
    if (k < 1 || k > routed) return fail(MOE_ERR_INVALID, "top_k must be in 1..%d (got %d)", routed, k);
    if (k + c.num_shared > MAX_KTOT)
        return fail(MOE_ERR_UNSUPPORTED, "more than %d selected experts per token", MAX_KTOT);
    if (e_router > MAX_ROUTER_EXPERTS)
        return fail(MOE_ERR_UNSUPPORTED, "more than %d router rows", MAX_ROUTER_EXPERTS);
    if (c.compute_dtype == MOE_DTYPE_BF16 && (c.input_dim % 8 || c.hidden_dim % 8))
        return fail(MOE_ERR_UNSUPPORTED,
                    "the BF16 tensor-core path needs input_dim and hidden_dim to be multiples of 8");
    if (c.drop_tokens && c.shared_mode == MOE_SHARED_LAYER_BLEND)
        return fail(MOE_ERR_INVALID, "drop_tokens does not apply to num_shared_experts > 0 (forward_with_shared_experts)");
    if (c.drop_tokens && !(c.capacity_factor > 0.f)) return fail(MOE_ERR_INVALID, "capacity_factor must be positive");
    return MOE_OK;
}

int ensure_weights(moe_layer* L) {
    if (L->w1) return MOE_OK;
    const size_t el = dtype_size(L->cfg.compute_dtype);
    const size_t n_local = (size_t)(L->e_hi - L->e_lo);
    const size_t D = L->cfg.input_dim, H = L->cfg.hidden_dim, O = L->cfg.output_dim;
    CUDA_TRY(cudaMalloc(&L->w1, n_local * H * D * el));
    CUDA_TRY(cudaMalloc(&L->w2, n_local * O * H * el));
    if (L->cfg.expert_kind == MOE_EXPERT_STANDARD) {
        CUDA_TRY(cudaMalloc(&L->b1, n_local * H * sizeof(float)));
        CUDA_TRY(cudaMalloc(&L->b2, n_local * O * sizeof(float)));
        CUDA_TRY(cudaMemset(L->b1, 0, n_local * H * sizeof(float)));
        CUDA_TRY(cudaMemset(L->b2, 0, n_local * O * sizeof(float)));
    } else {
        CUDA_TRY(cudaMalloc(&L->w3, n_local * H * D * el));
    }
    L->expert_set.assign(n_local, 0);
    L->plan_dirty = true;
    return MOE_OK;
}

// Graphs hold the addresses and kernel arguments of the call they were captured from: whatever
// changes the workspace or the layer's routing state drops them (callers synchronise first).
void drop_graphs(moe_layer* L) {
    bool any = false;
    for (auto& g : L->graphs) any = any || g.exec;
    if (any) cudaDeviceSynchronize();   // a replay may still be running on a caller's stream
    for (auto& g : L->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    L->graphs.clear();
}

void free_workspace(moe_layer* L) {
    drop_graphs(L);
    dev_free(L->idx);
    dev_free(L->gate);
    dev_free(L->pair_pos);
    dev_free(L->row_token);
    dev_free(L->cta_counts);
    dev_free(L->cta_psum);
    dev_free(L->cta_entropy);
    dev_free(L->xp);
    dev_free(L->h);
    dev_free(L->y);
    dev_free(L->tc_logits);
    L->T_cap = 0;
    L->P_cap = 0;
}

// Buffers whose size follows the number of local tokens.
int ensure_workspace(moe_layer* L, int64_t T) {
    if (T <= L->T_cap) return MOE_OK;
    CUDA_TRY(cudaDeviceSynchronize());
    free_workspace(L);
    const int64_t P = T * L->k_tot;
    const int64_t num_cta = (T + 15) / 16;   // the smallest token tile router_tokens_per_cta() may pick
    const size_t el = dtype_size(L->cfg.compute_dtype);
    int rc;
    if ((rc = dev_alloc(&L->idx, (size_t)P))) return rc;
    if ((rc = dev_alloc(&L->gate, (size_t)P))) return rc;
    if ((rc = dev_alloc(&L->pair_pos, (size_t)P))) return rc;
    if ((rc = dev_alloc(&L->row_token, (size_t)P))) return rc;
    if ((rc = dev_alloc(&L->cta_counts, (size_t)num_cta * L->E))) return rc;
    if ((rc = dev_alloc(&L->cta_psum, (size_t)num_cta * (L->E_probs + 1)))) return rc;
    if ((rc = dev_alloc(&L->cta_entropy, (size_t)num_cta))) return rc;
    if (L->rplan && (rc = dev_alloc(&L->tc_logits, (size_t)T * router_tc_e_pad(L->E_router)))) return rc;
    const bool peer = L->ep && ep_peer_mode(L->ep);
    if (!peer) {
        // (in peer mode rows go straight into the owners' receive buffers and come back from them)
        CUDA_TRY(cudaMalloc(&L->xp, (size_t)P * L->cfg.input_dim * el));
        CUDA_TRY(cudaMalloc(&L->y, (size_t)P * L->cfg.output_dim * el));
    }
    if (!L->ep) {
        // with expert parallelism the GEMMs run on the receive buffers owned by the EP state
        CUDA_TRY(cudaMalloc(&L->h, (size_t)P * L->cfg.hidden_dim * el));
    }
    L->T_cap = T;
    L->P_cap = P;
    L->plan_dirty = true;
    return MOE_OK;
}

int ensure_plan(moe_layer* L, const void* a1, const void* a2, int64_t rows) {
    if (L->cfg.compute_dtype != MOE_DTYPE_BF16) return MOE_OK;
    if (!L->plan) L->plan = tc_plan_create();
    if (!L->plan_dirty && L->plan_a1 == a1 && L->plan_a2 == a2 && L->plan_rows == rows) return MOE_OK;
    const char* msg = "";
    const int rc = tc_plan_encode(L->plan, a1, a2, rows, L->cfg.input_dim, L->cfg.hidden_dim, L->cfg.output_dim,
                                  L->e_hi - L->e_lo, L->w1, L->w3, L->w2, &msg);
    if (rc != MOE_OK) return fail(rc, "%s", msg);
    L->plan_dirty = false;
    L->plan_a1 = a1;
    L->plan_a2 = a2;
    L->plan_rows = rows;
    return MOE_OK;
}

inline void stage_mark(moe_layer* L, int i, cudaStream_t s) {
    if (L->prof_slots > 0) cudaEventRecord(L->ev[(size_t)L->prof_cur * 8 + i], s);
}

int check_ready(moe_layer* L) {
    if (!L->router_set) return fail(MOE_ERR_STATE, "router weights have not been set (moe_layer_set_router)");
    if (!L->w1) return fail(MOE_ERR_STATE, "no expert weights have been set (moe_layer_set_expert)");
    for (size_t i = 0; i < L->expert_set.size(); ++i)
        if (!L->expert_set[i])
            return fail(MOE_ERR_STATE, "expert %d has no weights (moe_layer_set_expert)", (int)i + L->e_lo);
    return MOE_OK;
}

// Which tensor-core kernel runs the expert GEMMs of a batch: 0 = single CTAs on 128-row tiles
// (expert_tc.cu), 1 = CTA pairs with cta_group::2 on 256-row tiles (expert_tc2.cu), 2 = single CTAs with
// two accumulators sharing a B tile on 256-row tiles (expert_tc_dual.cu).  Measured on B200, alternating
// in one call.  Long K (Mixtral widths: d_model 4096, ffn 14336, ~4096 rows per expert): 9.00-9.12 ms per
// layer with the two-accumulator kernel against 9.44 ms with single tiles and 9.65 ms with CTA pairs --
// the kernels run at the board's power limit and the two-accumulator kernel moves a third less from L2 per
// FLOP.  Short K (d 2048, hidden 1408, 66 experts): 4.07-4.10 ms with CTA pairs against 4.20-4.33 ms
// (two accumulators) and 4.28 ms (single): a K loop of 22-32 blocks ends before the three 64 KB stages of
// the two-accumulator kernel or the four of the single-CTA kernel have hidden the load latency, while the
// pair kernel's six stages do, and the epilogue gap of the two-accumulator kernel weighs more per tile.
// 256-row tiles waste half a tile per expert on average, twice what 128-row tiles do: with long K the
// two-accumulator kernel is ahead at 4096 rows per expert (-3.2 %), level at 2048, behind at 1024 (+3 %)
// and 512 (+8..14 %), so it takes experts of 3072 rows and more; the pair kernel needs an expert to fill
// two tiles.  MOE_B200_PAIR = 0 / 1 / 2 forces the choice.
int pick_gemm_kernel(const moe_layer* L, int64_t rows, int n_experts) {
    if (L->cfg.compute_dtype != MOE_DTYPE_BF16) return 0;
    if (L->force_pair >= 0) return L->force_pair;
    const int64_t per_expert = n_experts > 0 ? rows / n_experts : 0;
    if ((int64_t)L->cfg.input_dim + L->cfg.hidden_dim <= 6144) return per_expert >= 2 * TC_PAIR_TILE_M ? 1 : 0;
    return per_expert >= 12 * TC_PAIR_TILE_M ? 2 : 0;
}

int pick_tile_m(const moe_layer* L, int64_t rows, int n_experts) {
    if (L->cfg.compute_dtype != MOE_DTYPE_BF16) return F32_TILE_M;
    return pick_gemm_kernel(L, rows, n_experts) ? TC_PAIR_TILE_M : TC_TILE_M;
}

// The grouped GEMM pair on `rows_cap` rows described by (expert_offset, tile_prefix).
int run_experts(moe_layer* L, const void* a_in, void* h_buf, void* y_buf, const int32_t* expert_offset,
                const int32_t* tile_prefix, int64_t rows, int n_experts, cudaStream_t s, int ev_base, int tile_m,
                const int32_t* seg_start = nullptr, void* const* seg_dst = nullptr, int seg_per_expert = 0,
                int inplace_experts = 0) {
    const moe_config_t& c = L->cfg;
    GroupGemmParams g{};
    g.E = n_experts;
    g.activation = c.activation;
    g.expert_offset = expert_offset;
    g.tile_prefix = tile_prefix;
    g.status = L->status;
    g.seg_start = nullptr;
    g.seg_dst = nullptr;
    g.seg_per_expert = 0;
    const bool tc = c.compute_dtype == MOE_DTYPE_BF16;
    const bool pair = tc && tile_m == TC_PAIR_TILE_M;
    const int64_t max_mtiles64 = (rows + tile_m - 1) / tile_m + n_experts;
    if (max_mtiles64 > 0x7fffffff / 256) return fail(MOE_ERR_UNSUPPORTED, "too many row tiles");
    const int max_mtiles = (int)max_mtiles64;
    int n;
    const bool standard = c.expert_kind == MOE_EXPERT_STANDARD;
    // GEMM 1: gated h = act(a W1^T) .* (a W3^T); standard h = act(a W1^T + b1)
    const int mode1 = standard ? 2 : 1;
    const int ntile1 = standard ? (c.hidden_dim + 255) / 256 : (c.hidden_dim + 127) / 128;
    g.A = a_in;
    g.B0 = L->w1;
    g.B1 = standard ? nullptr : L->w3;
    g.C = h_buf;
    g.N = c.hidden_dim;
    g.K = c.input_dim;
    g.bias = standard ? L->b1 : nullptr;
    g.epilogue_act = standard ? c.activation : -1;
    g.inplace_experts = tc ? inplace_experts : 0;
    const bool dual = pair && pick_gemm_kernel(L, rows, n_experts) == 2;   // 256-row tiles on one CTA with two accumulators
    if (dual) n = launch_group_gemm_tc_dual(L->plan, 1, mode1, g, max_mtiles * ntile1, L->num_sms, s);
    else if (pair) n = launch_group_gemm_tc2(L->plan, 1, mode1, g, max_mtiles * ntile1, L->num_sms, s);
    else if (tc) n = launch_group_gemm_tc(L->plan, 1, mode1, g, max_mtiles * ntile1, L->num_sms, s);
    else n = launch_group_gemm_f32(g, mode1, max_mtiles, rows, L->num_sms, s);
    if (n < 0) return fail(MOE_ERR_CUDA, "expert GEMM 1 launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    stage_mark(L, ev_base, s);
    // GEMM 2: y = h W2^T (+ b2 for a standard expert)
    g.A = h_buf;
    g.B0 = L->w2;
    g.B1 = nullptr;
    g.bias = standard ? L->b2 : nullptr;
    g.epilogue_act = -1;
    g.inplace_experts = 0;
    g.C = y_buf;
    g.N = c.output_dim;
    g.K = c.hidden_dim;
    g.seg_start = seg_start;      // expert-parallel peer mode: rows go straight to the token owners
    g.seg_dst = seg_dst;
    g.seg_per_expert = seg_per_expert;
    if (dual) n = launch_group_gemm_tc_dual(L->plan, 2, 2, g, max_mtiles * ((c.output_dim + 255) / 256), L->num_sms, s);
    else if (pair) n = launch_group_gemm_tc2(L->plan, 2, 2, g, max_mtiles * ((c.output_dim + 255) / 256), L->num_sms, s);
    else if (tc) n = launch_group_gemm_tc(L->plan, 2, 2, g, max_mtiles * ((c.output_dim + 255) / 256), L->num_sms, s);
    else n = launch_group_gemm_f32(g, 2, max_mtiles, rows, L->num_sms, s);
    if (n < 0) return fail(MOE_ERR_CUDA, "expert GEMM 2 launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    stage_mark(L, ev_base + 1, s);
    return MOE_OK;
}

// A call that covers one chunk of a larger host batch.  Without expert parallelism the scan kernel adds
// its statistics into `sums` and the caller finishes loss and entropy from the total; with expert
// parallelism the records of every chunk are exchanged anyway and the running totals live in the EP
// state (ep_mode: 1 first, 2 middle, 3 last chunk).
struct ChunkCtx {
    float* sums = nullptr;
    int want_entropy = 0;
    int ep_mode = 0;
};

int forward_device(moe_layer* L, const void* x, int x_dtype, int64_t T, int training, float* out,
                   const moe_forward_outputs_t* opt, cudaStream_t s, const ChunkCtx* chunk = nullptr) {
    float* partial_sums = chunk ? chunk->sums : nullptr;
    const int partial_want_entropy = chunk ? chunk->want_entropy : 0;
    const bool chunked = chunk != nullptr;
    const moe_config_t& c = L->cfg;
    static const moe_forward_outputs_t none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    if (!opt) opt = &none;
    if (T < 0) return fail(MOE_ERR_INVALID, "T must be non-negative");
    if (x_dtype != MOE_DTYPE_F32 && x_dtype != MOE_DTYPE_BF16) return fail(MOE_ERR_INVALID, "unknown x_dtype");
    if (T > 0 && (!x || !out)) return fail(MOE_ERR_INVALID, "x and out must not be null");
    if (T * (int64_t)L->k_tot > 0x7fffffffLL) return fail(MOE_ERR_UNSUPPORTED, "T*k exceeds 2^31-1 rows");
    int rc = check_ready(L);
    if (rc) return rc;
    CUDA_TRY(cudaSetDevice(L->device));
    if (T == 0 && !L->ep) {
        if (opt->loss) CUDA_TRY(cudaMemsetAsync(opt->loss, 0, sizeof(float), s));
        if (opt->routing_entropy) CUDA_TRY(cudaMemsetAsync(opt->routing_entropy, 0, sizeof(float), s));
        if (opt->tokens_per_expert) CUDA_TRY(cudaMemsetAsync(opt->tokens_per_expert, 0, sizeof(int64_t) * L->E, s));
        return MOE_OK;
    }
    if ((rc = ensure_workspace(L, T > 0 ? T : 1))) return rc;
    if (!L->ep && L->plan_dirty && (rc = ensure_plan(L, L->xp, L->h, L->P_cap))) return rc;

    // the tensor-core router's gating kernel is latency-bound per token like a narrow router's: it takes the
    // narrow rule (enough CTAs for every SM) whatever the router width
    const bool noise_net_armed = training && L->noise_scale > 0.f && L->noise && L->router_nw;
    const bool use_tc_router = L->router_tc_enabled && L->tc_logits != nullptr &&
                               router_tc_usable(L->rplan, x, x_dtype, noise_net_armed, L->E_router, c.input_dim, T);
    const int tokens_per_cta = router_tokens_per_cta(T, use_tc_router ? 8 : L->E_router, L->num_sms);
    const int num_cta = (int)((T + tokens_per_cta - 1) / tokens_per_cta);
    if (L->prof_slots > 0) L->prof_cur = (int)(L->prof_calls++ % L->prof_slots);
    // small batches: every kernel may be set up on the SMs while its predecessor still runs
    // (plain launches only: measured on B200, a replayed graph is a little slower with chained nodes)
    const ChainScope chain(L->chain_enabled && !L->capturing && !L->ep && L->prof_slots == 0 &&
                           T * (int64_t)L->k_tot <= moe_layer::GRAPH_MAX_PAIRS);
    stage_mark(L, 0, s);

    RouterParams r{};
    r.x = x;
    r.w = L->router_w;
    r.wt = L->router_wt;
    r.bias = L->has_bias ? L->router_bias : nullptr;
    r.noise = (training && L->noise_scale > 0.f) ? L->noise : nullptr;
    r.noise_scale = L->noise_scale;
    r.noise_off = 0;
    if (r.noise && L->router_nw) {   // src/core/router.jl:33-37: the draws are scaled by softplus(noise_weight x)
        r.wt = L->router_wt_noise;
        r.noise_off = L->E_router;
    }
    r.T = T;
    r.D = c.input_dim;
    r.E = L->E;
    r.E_router = L->E_router;
    r.E_probs = L->E_probs;
    r.S = L->S;
    r.k = L->k;
    r.k_tot = L->k_tot;
    r.shared_mode = c.shared_mode;
    r.bias_gates_only = c.bias_gates_only;
    r.index_base = c.index_base;
    r.tokens_per_cta = tokens_per_cta;
    r.want_entropy = opt->routing_entropy != nullptr || partial_want_entropy;
    r.idx = L->idx;
    r.gate = L->gate;
    r.cta_counts = L->cta_counts;
    r.cta_psum = L->cta_psum;
    r.cta_entropy = L->cta_entropy;
    r.u_idx = opt->indices;
    r.u_gate = opt->gates;
    r.u_probs = opt->probs;
    r.u_logits = opt->logits;
    r.tc_logits = L->tc_logits;
    r.tc_recheck_count = L->tc_recheck;
    ScanParams sp{};
    sp.T = T;
    sp.E = L->E;
    sp.E_probs = L->E_probs;
    sp.S = L->S;
    sp.k = L->k;
    sp.k_tot = L->k_tot;
    sp.shared_mode = c.shared_mode;
    sp.num_cta = num_cta;
    const int tile_m_local = pick_tile_m(L, T * L->k_tot, L->E);   // non-expert-parallel GEMMs
    sp.tile_m = tile_m_local;
    sp.training = training;
    // capacity = ceil(Int, capacity_factor * T / E), evaluated in Float32 like the reference (moe_layer.jl:223)
    const int capacity = (c.drop_tokens && training) ? (int)ceilf(c.capacity_factor * (float)T / (float)L->E) : -1;
    if (capacity >= 0 && L->ep) return fail(MOE_ERR_UNSUPPORTED, "drop_tokens with expert parallelism is not implemented");
    sp.capacity = capacity;
    sp.alpha = c.balance_alpha;
    sp.z_weight = c.z_loss_weight;
    sp.cta_counts = L->cta_counts;
    sp.cta_psum = L->cta_psum;
    sp.cta_entropy = L->cta_entropy;
    sp.expert_count = L->expert_count;
    sp.expert_offset = L->expert_offset;
    sp.tile_prefix = L->tile_prefix;
    sp.loss_internal = L->loss_dev;
    sp.u_loss = (L->ep || chunked) ? nullptr : opt->loss;
    sp.u_tokens_per_expert = opt->tokens_per_expert;
    sp.u_entropy = (L->ep || chunked) ? nullptr : opt->routing_entropy;
    sp.ep_sums = L->ep ? nullptr : partial_sums;
    sp.sums_accumulate = chunked ? 1 : 0;
    sp.ep_record = L->ep ? ep_record_buffer(L->ep) : nullptr;

    PermuteParams pp{};
    pp.x = x;
    pp.xp = L->xp;
    pp.T = T;
    pp.D = c.input_dim;
    pp.E = L->E;
    pp.k_tot = L->k_tot;
    pp.tokens_per_cta = tokens_per_cta;
    pp.idx = L->idx;
    pp.cta_base = L->cta_counts;
    pp.expert_offset = L->expert_offset;
    pp.pair_pos = L->pair_pos;
    pp.row_token = L->row_token;
    pp.status = L->status;
    pp.P_cap = L->P_cap;
    pp.expert_dst = nullptr;
    pp.capacity = capacity;
    pp.index_base = c.index_base;
    pp.idx_rw = L->idx;
    pp.gate_rw = L->gate;
    pp.u_idx = opt->indices;
    pp.u_gate = opt->gates;
    // Shared experts (ids 0..S-1 of SharedExpertGating / num_shared_experts) see every token in token
    // order: on the tensor-core path GEMM 1 reads x itself for them and the permute copies nothing.
    int inplace_experts = 0;
    if (L->S > 0 && L->inplace_shared && !L->ep && capacity < 0 && c.compute_dtype == MOE_DTYPE_BF16 && x_dtype == MOE_DTYPE_BF16 && L->plan &&
        tc_plan_set_x(L->plan, x, T, c.input_dim))
        inplace_experts = L->S;
    pp.inplace_experts = inplace_experts;

    int n = 0;
    if (num_cta > 0) {
        if (use_tc_router)
            n = launch_router_tc(L->rplan, r, num_cta, L->num_sms, L->status, s);
        else
            n = launch_router(r, x_dtype, num_cta, L->num_sms, s);
        if (n < 0) return fail(MOE_ERR_CUDA, "router launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n;
    }
    stage_mark(L, 1, s);
    n = launch_scan(sp, s);
    if (n < 0) return fail(MOE_ERR_CUDA, "scan launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    stage_mark(L, 2, s);
    const bool peer = L->ep && ep_peer_mode(L->ep);
    EpPlan plan;
    const int ep_tile_m = L->cfg.compute_dtype == MOE_DTYPE_BF16 ? TC_TILE_M : F32_TILE_M;
    if (peer) {
        if ((rc = ep_prepare(L->ep, T, s, &plan, g_err, sizeof(g_err)))) return rc;
        pp.expert_dst = plan.d_expert_dst;
        ep_mark(L->ep, 0, s);
    }
    if (num_cta > 0) {
        n = launch_permute(pp, x_dtype, c.compute_dtype, num_cta, s);
        if (n < 0) return fail(MOE_ERR_CUDA, "permute launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n;
    }
    stage_mark(L, 3, s);

    if (!L->ep) {
        if ((rc = run_experts(L, L->xp, L->h, L->y, L->expert_offset, L->tile_prefix, T * L->k_tot, L->E, s, 4, tile_m_local,
                              nullptr, nullptr, 0, inplace_experts)))
            return rc;
    } else if (peer) {
        // flag barrier: every rank's permute kernel has written its rows into the owners' buffers
        if ((rc = ep_barrier(L->ep, 0, s, g_err, sizeof(g_err)))) return rc;
        L->launches += 1;
        ep_mark(L->ep, 1, s);
        if ((rc = ensure_plan(L, plan.xr, plan.hr, plan.rows_cap))) return rc;
        const int n_local = L->e_hi - L->e_lo;
        const bool pair = plan.d_tile_prefix_alt && pick_tile_m(L, plan.rows, n_local) == TC_PAIR_TILE_M;
        if ((rc = run_experts(L, plan.xr, plan.hr, nullptr, plan.d_local_off,
                              pair ? plan.d_tile_prefix_alt : plan.d_tile_prefix, plan.rows, n_local, s, 4,
                              pair ? TC_PAIR_TILE_M : ep_tile_m, plan.d_seg_start, plan.d_seg_dst, ep_world(L->ep))))
            return rc;
        ep_mark(L->ep, 2, s);
        // every rank's GEMM 2 has stored its rows into the token owners' buffers before anybody combines
        if ((rc = ep_barrier(L->ep, 1, s, g_err, sizeof(g_err)))) return rc;
        L->launches += 1;
    } else {
        EpCall call;
        call.T = T;
        call.xs = L->xp;
        call.y_back = L->y;
        call.expert_count = L->expert_count;
        call.expert_offset = L->expert_offset;
        call.stream = s;
        rc = ep_exchange_and_run(
            L->ep, call,
            [](void* self, const void* a_in, void* h_buf, void* y_buf, const int32_t* eo, const int32_t* tp,
               int64_t rows, int n_exp, int64_t cap_rows, cudaStream_t st) -> int {
                moe_layer* M = reinterpret_cast<moe_layer*>(self);
                int rc2 = ensure_plan(M, a_in, h_buf, cap_rows);
                if (rc2) return rc2;
                return run_experts(M, a_in, h_buf, y_buf, eo, tp, rows, n_exp, st, 4,
                                   M->cfg.compute_dtype == MOE_DTYPE_BF16 ? TC_TILE_M : F32_TILE_M);
            },
            L, g_err, sizeof(g_err));
        if (rc) return rc;
    }

    CombineParams cp{};
    cp.y = peer ? plan.yb : L->y;
    cp.out = out;
    cp.T = T;
    cp.O = c.output_dim;
    cp.k_tot = L->k_tot;
    cp.idx = L->idx;
    cp.gate = L->gate;
    cp.pair_pos = L->pair_pos;
    n = launch_combine(cp, c.compute_dtype, s);
    if (n < 0) return fail(MOE_ERR_CUDA, "combine launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    stage_mark(L, 6, s);
    // compute_loss(::AuxiliaryFreeLoss) first updates the bias the next call selects with
    // (src/balancing/auxiliary_free.jl:73-83); partial (chunked) calls are updated by their caller
    if (L->aux_free && training && !chunked) {
        ++L->aux_counter;
        if (L->aux_counter % L->aux_freq == 0) {
            n = launch_aux_free_update(L->expert_count, L->E_router, L->router_bias, L->bias_momentum, L->aux_lr,
                                       L->aux_momentum, s);
            if (n < 0) return fail(MOE_ERR_CUDA, "bias update launch failed: %s", cudaGetErrorString(cudaGetLastError()));
            L->launches += n;
        }
    }
    if (L->ep) {
        if (peer) ep_mark(L->ep, 3, s);
        if ((rc = ep_finish_loss(L->ep, training, chunk ? chunk->ep_mode : 0, opt->loss, opt->routing_entropy, s, &L->launches,
                                 g_err, sizeof(g_err))))
            return rc;
    }
    return MOE_OK;
}

__global__ void graph_small_outputs_kernel(const float* __restrict__ block, int E, float* loss, float* entropy,
                                           int64_t* tokens_per_expert) {
    const int i = threadIdx.x;
    if (i == 0 && loss) *loss = block[0];
    if (i == 0 && entropy) *entropy = block[1];
    if (tokens_per_expert) {
        const int64_t* counts = reinterpret_cast<const int64_t*>(block + 4);
        for (int e = i; e < E; e += blockDim.x) tokens_per_expert[e] = counts[e];
    }
}

int replay_graph(moe_layer* L, const moe_layer::GraphEntry& e, const moe_forward_outputs_t& o, cudaStream_t s) {
    CUDA_TRY(cudaGraphLaunch(e.exec, s));
    L->launches += e.launches;
    if (o.loss || o.routing_entropy || o.tokens_per_expert) {
        graph_small_outputs_kernel<<<1, 128, 0, s>>>(L->graph_small, L->E, o.loss, o.routing_entropy, o.tokens_per_expert);
        CUDA_TRY(cudaGetLastError());
        L->launches += 1;
    }
    ++L->graph_replays;
    return MOE_OK;
}

// Forward for batches small enough that launching costs more than computing: plain launches on
// the first call with a set of arguments, capture on the second, replay from then on.  The graph
// reads the same buffers as the launches would, so new contents of x (or of the noise buffer) are
// seen by a replay; anything else that differs makes a different key.
int forward_small(moe_layer* L, const void* x, int x_dtype, int64_t T, int training, float* out,
                  const moe_forward_outputs_t* opt, cudaStream_t s, bool allow_graph = true) {
    static const moe_forward_outputs_t none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    const moe_forward_outputs_t& o = opt ? *opt : none;
    const bool eligible = allow_graph && L->graphs_enabled && !L->ep && T > 0 && T * (int64_t)L->k_tot <= moe_layer::GRAPH_MAX_PAIRS &&
                          L->prof_slots == 0 && !(L->aux_free && training) && x && out && L->graph_small &&
                          (x_dtype == MOE_DTYPE_F32 || x_dtype == MOE_DTYPE_BF16);
    if (!eligible) return forward_device(L, x, x_dtype, T, training, out, opt, s);
    CUDA_TRY(cudaSetDevice(L->device));
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
        cudaGetLastError();   // the caller is building a graph of its own: its capture takes our launches
        return forward_device(L, x, x_dtype, T, training, out, opt, s);
    }
    const float* noise = (training && L->noise_scale > 0.f) ? L->noise : nullptr;
    moe_layer::GraphEntry* e = nullptr;
    for (auto& g : L->graphs)
        if (g.x == x && g.x_dtype == x_dtype && g.T == T && g.training == training && g.out == out &&
            !g.opt.loss == !o.loss && g.opt.indices == o.indices && g.opt.gates == o.gates && g.opt.probs == o.probs &&
            g.opt.logits == o.logits && !g.opt.tokens_per_expert == !o.tokens_per_expert &&
            !g.opt.routing_entropy == !o.routing_entropy && g.noise == noise && g.noise_scale == L->noise_scale) {
            e = &g;
            break;
        }
    if (e && e->exec) {
        int rc = check_ready(L);
        if (rc) return rc;
        e->tick = ++L->graph_tick;
        return replay_graph(L, *e, o, s);
    }
    if (!e) {   // first sighting: remember the key, run the launches (they also grow the workspace)
        if ((int)L->graphs.size() >= moe_layer::MAX_GRAPHS) {
            size_t victim = 0;
            for (size_t i = 1; i < L->graphs.size(); ++i)
                if (L->graphs[i].tick < L->graphs[victim].tick) victim = i;
            if (L->graphs[victim].exec) cudaGraphExecDestroy(L->graphs[victim].exec);
            L->graphs.erase(L->graphs.begin() + victim);
        }
        moe_layer::GraphEntry g;
        g.x = x;
        g.x_dtype = x_dtype;
        g.T = T;
        g.training = training;
        g.out = out;
        g.opt = o;
        g.noise = noise;
        g.noise_scale = L->noise_scale;
        g.tick = ++L->graph_tick;
        const int rc = forward_device(L, x, x_dtype, T, training, out, opt, s);   // may drop all graphs (growth)
        if (rc == MOE_OK) L->graphs.push_back(g);
        return rc;
    }
    e->tick = ++L->graph_tick;
    if (e->refused || T > L->T_cap) return forward_device(L, x, x_dtype, T, training, out, opt, s);
    // second sighting: record the same launches on the handle's stream instead of running them
    const int64_t launches_before = L->launches;
    if (cudaStreamBeginCapture(L->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        e->refused = true;
        return forward_device(L, x, x_dtype, T, training, out, opt, s);
    }
    moe_forward_outputs_t inside = o;
    inside.loss = o.loss ? L->graph_small : nullptr;
    inside.routing_entropy = o.routing_entropy ? L->graph_small + 1 : nullptr;
    inside.tokens_per_expert = o.tokens_per_expert ? reinterpret_cast<int64_t*>(L->graph_small + 4) : nullptr;
    L->capturing = true;
    const int rc = forward_device(L, x, x_dtype, T, training, out, &inside, L->stream);
    L->capturing = false;
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(L->stream, &graph);
    const int recorded = (int)(L->launches - launches_before);
    L->launches = launches_before;
    cudaGraphExec_t exec = nullptr;
    const bool ok = rc == MOE_OK && ce == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
    if (graph) cudaGraphDestroy(graph);
    if (!ok) {
        cudaGetLastError();
        e->refused = true;
        if (rc != MOE_OK) return rc;   // an argument error: nothing was recorded and nothing ran
        return forward_device(L, x, x_dtype, T, training, out, opt, s);
    }
    e->exec = exec;
    e->launches = recorded;
    return replay_graph(L, *e, o, s);
}

int grow(void** p, size_t* cap, size_t need) {
    if (need <= *cap) return MOE_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    CUDA_TRY(cudaMalloc(p, need));
    *cap = need;
    return MOE_OK;
}

int grow_pinned(char** p, size_t* cap, size_t need) {
    if (need <= *cap) return MOE_OK;
    if (*p) cudaFreeHost(*p);
    *p = nullptr;
    *cap = 0;
    CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(p), need, cudaHostAllocDefault));
    *cap = need;
    return MOE_OK;
}

int status_to_rc(moe_layer* L, int32_t st) {
    if (st == DEV_OK) return MOE_OK;
    cudaMemset(L->status, 0, sizeof(int32_t));
    return fail(st == DEV_BAD_INDEX ? MOE_ERR_INVALID : MOE_ERR_TIMEOUT, "device status %d after forward", st);
}

}  // namespace

extern "C" {

const char* moe_last_error(void) { return g_err; }
const char* moe_version(void) { return "moe_b200 0.1 (sm_100a)"; }

int moe_layer_create(const moe_config_t* cfg, int device, moe_layer_t** out) {
    if (!cfg || !out) return fail(MOE_ERR_INVALID, "cfg and out must not be null");
    *out = nullptr;
    int rc = validate_config(*cfg);
    if (rc) return rc;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return fail(MOE_ERR_CUDA, "no CUDA device is available (this library has no CPU path)");
    if (device < 0 || device >= ndev) return fail(MOE_ERR_INVALID, "device %d out of range (0..%d)", device, ndev - 1);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(MOE_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    moe_layer* L = new (std::nothrow) moe_layer();
    if (!L) return fail(MOE_ERR_INVALID, "out of host memory");
    L->cfg = *cfg;
    L->device = device;
    L->num_sms = prop.multiProcessorCount;
    L->E = cfg->num_experts;
    L->S = cfg->shared_mode == MOE_SHARED_NONE ? 0 : cfg->num_shared;
    L->k = cfg->gate_kind == MOE_GATE_SWITCH ? 1 : cfg->top_k;
    L->k_tot = L->k + L->S;
    L->E_router = cfg->shared_mode == MOE_SHARED_LAYER_BLEND ? L->E - L->S : L->E;
    L->E_probs = L->E_router;
    L->e_lo = 0;
    L->e_hi = L->E;
    if (const char* ev = getenv("MOE_B200_PAIR")) L->force_pair = atoi(ev) >= 2 ? 2 : (atoi(ev) > 0 ? 1 : 0);
    if (const char* ev = getenv("MOE_B200_HOST_CHUNKS")) L->host_chunks = atoi(ev) > 0 ? atoi(ev) : 0;
    if (const char* ev = getenv("MOE_B200_HOST_TIMELINE")) L->host_timeline = atoi(ev) > 0;
    if (const char* ev = getenv("MOE_B200_ROUTER_TC")) L->router_tc_enabled = atoi(ev) != 0;
    if (const char* ev = getenv("MOE_B200_INPLACE_SHARED")) L->inplace_shared = atoi(ev) != 0;
    if (const char* ev = getenv("MOE_B200_GRAPHS")) L->graphs_enabled = atoi(ev) != 0;
    if (const char* ev = getenv("MOE_B200_CHAIN")) L->chain_enabled = atoi(ev) != 0;
    auto cleanup = [&](int code) {
        moe_layer_destroy(L);
        return code;
    };
    if ((rc = dev_alloc(&L->router_w, (size_t)L->E_router * cfg->input_dim))) return cleanup(rc);
    if ((rc = dev_alloc(&L->router_wt, (size_t)router_e_pad(L->E_router) * router_d_pad(cfg->input_dim)))) return cleanup(rc);
    if ((rc = dev_alloc(&L->router_bias, (size_t)L->E_router))) return cleanup(rc);
    if ((rc = dev_alloc(&L->expert_count, (size_t)L->E))) return cleanup(rc);
    if ((rc = dev_alloc(&L->expert_offset, (size_t)L->E + 1))) return cleanup(rc);
    if ((rc = dev_alloc(&L->tile_prefix, (size_t)L->E + 1))) return cleanup(rc);
    if ((rc = dev_alloc(&L->loss_dev, 1))) return cleanup(rc);
    if (cudaMalloc(reinterpret_cast<void**>(&L->small_dev), 256 + moe_layer::PIN_SMALL_CALL) != cudaSuccess)
        return cleanup(fail(MOE_ERR_CUDA, "cudaMalloc failed"));
    L->status = reinterpret_cast<int32_t*>(L->small_dev);
    if (router_tc_e_pad(L->E_router) && cfg->input_dim % 8 == 0) {
        L->rplan = router_tc_plan_create();
        if (cudaMalloc(&L->router_w3, (size_t)3 * router_tc_e_pad(L->E_router) * cfg->input_dim * 2) != cudaSuccess)
            return cleanup(fail(MOE_ERR_CUDA, "cudaMalloc failed"));
        if ((rc = dev_alloc(&L->tc_recheck, 1))) return cleanup(rc);
        if (cudaMemset(L->tc_recheck, 0, sizeof(int32_t)) != cudaSuccess) return cleanup(fail(MOE_ERR_CUDA, "cudaMemset failed"));
    }
    if (cudaMemset(L->status, 0, sizeof(int32_t)) != cudaSuccess) return cleanup(fail(MOE_ERR_CUDA, "cudaMemset failed"));
    if ((rc = dev_alloc(&L->graph_small, (size_t)4 + 2 * L->E))) return cleanup(rc);
    if (cudaStreamCreateWithFlags(&L->stream, cudaStreamNonBlocking) != cudaSuccess)
        return cleanup(fail(MOE_ERR_CUDA, "cudaStreamCreate failed"));
    *out = L;
    return MOE_OK;
}

int moe_layer_destroy(moe_layer_t* L) {
    if (!L) return MOE_OK;
    cudaSetDevice(L->device);
    cudaDeviceSynchronize();
    if (L->ep) ep_destroy(L->ep);
    free_workspace(L);
    dev_free(L->w1);
    dev_free(L->w3);
    dev_free(L->w2);
    dev_free(L->b1);
    dev_free(L->b2);
    dev_free(L->router_w);
    dev_free(L->router_bias);
    dev_free(L->router_wt);
    dev_free(L->router_w3);
    dev_free(L->tc_recheck);
    if (L->rplan) router_tc_plan_destroy(L->rplan);
    dev_free(L->bias_momentum);
    dev_free(L->router_nw);
    dev_free(L->router_wt_noise);
    dev_free(L->stage_w);
    dev_free(L->expert_count);
    dev_free(L->expert_offset);
    dev_free(L->tile_prefix);
    dev_free(L->loss_dev);
    dev_free(L->small_dev);
    dev_free(L->graph_small);
    dev_free(L->hx);
    dev_free(L->hout);
    dev_free(L->hopt);
    if (L->pin) cudaFreeHost(L->pin);
    if (L->plan) tc_plan_destroy(L->plan);
    for (auto& e : L->ev) cudaEventDestroy(e);
    if (L->stream) cudaStreamDestroy(L->stream);
    if (L->s_in) cudaStreamDestroy(L->s_in);
    if (L->s_out) cudaStreamDestroy(L->s_out);
    for (auto& e : L->ev_in)
        if (e) cudaEventDestroy(e);
    for (auto e : {L->ev_t0})
        if (e) cudaEventDestroy(e);
    for (auto& e : L->ev_in0)
        if (e) cudaEventDestroy(e);
    for (auto& e : L->ev_out1)
        if (e) cudaEventDestroy(e);
    for (auto& e : L->ev_done)
        if (e) cudaEventDestroy(e);
    dev_free(L->chunk_acc);
    dev_free(L->chunk_tpe_acc);
    delete L;
    return MOE_OK;
}

int moe_layer_dims(const moe_layer_t* L, int32_t* k_tot, int32_t* e_probs, int32_t* e_router) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    // indices/gates hold k routed entries per token in LAYER_BLEND mode (the reference's
    // expert_indices there are the routed ones shifted by S), else k_tot.
    if (k_tot) *k_tot = L->cfg.shared_mode == MOE_SHARED_LAYER_BLEND ? L->k : L->k_tot;
    if (e_probs) *e_probs = L->E_probs;
    if (e_router) *e_router = L->E_router;
    return MOE_OK;
}

// shared body of the two expert setters: w3 == null for a standard expert (then b1/b2 may be given)
static int set_expert_impl(moe_layer_t* L, int expert, const void* w1, const void* w2, const void* w3, const float* b1,
                           const float* b2, int src_dtype, int layout, int src_is_device) {
    if (src_dtype != MOE_DTYPE_F32 && src_dtype != MOE_DTYPE_BF16) return fail(MOE_ERR_INVALID, "unknown src_dtype");
    if (layout != MOE_LAYOUT_IN_CONTIG && layout != MOE_LAYOUT_OUT_CONTIG) return fail(MOE_ERR_INVALID, "unknown layout");
    if (expert < 0 || expert >= L->E) return fail(MOE_ERR_INVALID, "expert %d out of range 0..%d", expert, L->E - 1);
    if (expert < L->e_lo || expert >= L->e_hi)
        return fail(MOE_ERR_INVALID, "expert %d is not held by this rank (it holds %d..%d)", expert, L->e_lo, L->e_hi - 1);
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    // Device sources may still be being written by work the caller queued on its own streams; the
    // repack below runs on the handle's stream, which is not ordered after them.
    if (src_is_device) CUDA_TRY(cudaDeviceSynchronize());
    int rc = ensure_weights(L);
    if (rc) return rc;
    const size_t D = L->cfg.input_dim, H = L->cfg.hidden_dim, O = L->cfg.output_dim;
    const size_t el = dtype_size(L->cfg.compute_dtype), sel = dtype_size(src_dtype);
    const size_t slot = (size_t)(expert - L->e_lo);
    struct Item { const void* src; void* dst; int rows, cols; };
    const Item items[3] = {
        {w1, (char*)L->w1 + slot * H * D * el, (int)H, (int)D},
        {w3, w3 ? (char*)L->w3 + slot * H * D * el : nullptr, (int)H, (int)D},
        {w2, (char*)L->w2 + slot * O * H * el, (int)O, (int)H},
    };
    for (const Item& it : items) {
        if (!it.src) continue;
        const void* src = it.src;
        const size_t bytes = (size_t)it.rows * it.cols * sel;
        if (!src_is_device) {
            if ((rc = grow(&L->stage_w, &L->stage_w_bytes, bytes))) return rc;
            CUDA_TRY(cudaMemcpyAsync(L->stage_w, it.src, bytes, cudaMemcpyHostToDevice, L->stream));
            src = L->stage_w;
        }
        const int n = launch_transpose_convert(src, src_dtype, it.dst, L->cfg.compute_dtype, it.rows, it.cols,
                                               layout == MOE_LAYOUT_OUT_CONTIG, L->stream);
        if (n < 0) return fail(MOE_ERR_CUDA, "weight repack launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n;
        CUDA_TRY(cudaStreamSynchronize(L->stream));
    }
    const cudaMemcpyKind kind = src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    if (L->b1) {
        if (b1) CUDA_TRY(cudaMemcpyAsync(L->b1 + slot * H, b1, H * sizeof(float), kind, L->stream));
        else CUDA_TRY(cudaMemsetAsync(L->b1 + slot * H, 0, H * sizeof(float), L->stream));
        if (b2) CUDA_TRY(cudaMemcpyAsync(L->b2 + slot * O, b2, O * sizeof(float), kind, L->stream));
        else CUDA_TRY(cudaMemsetAsync(L->b2 + slot * O, 0, O * sizeof(float), L->stream));
        CUDA_TRY(cudaStreamSynchronize(L->stream));
    }
    L->expert_set[slot] = 1;
    return MOE_OK;
}

int moe_layer_set_expert(moe_layer_t* L, int expert, const void* w1, const void* w2, const void* w3, int src_dtype,
                         int layout, int src_is_device) {
    if (!L || !w1 || !w2 || !w3) return fail(MOE_ERR_INVALID, "null argument");
    if (L->cfg.expert_kind != MOE_EXPERT_GATED)
        return fail(MOE_ERR_STATE, "this layer holds standard experts: use moe_layer_set_expert_standard");
    return set_expert_impl(L, expert, w1, w2, w3, nullptr, nullptr, src_dtype, layout, src_is_device);
}

int moe_layer_set_expert_standard(moe_layer_t* L, int expert, const void* w1, const float* b1, const void* w2,
                                  const float* b2, int src_dtype, int layout, int src_is_device) {
    if (!L || !w1 || !w2) return fail(MOE_ERR_INVALID, "null argument");
    if (L->cfg.expert_kind != MOE_EXPERT_STANDARD)
        return fail(MOE_ERR_STATE, "this layer holds gated experts: use moe_layer_set_expert");
    return set_expert_impl(L, expert, w1, w2, nullptr, b1, b2, src_dtype, layout, src_is_device);
}

int moe_layer_set_router(moe_layer_t* L, const float* w, const float* logit_bias, int layout, int src_is_device) {
    if (!L || !w) return fail(MOE_ERR_INVALID, "null argument");
    if (layout != MOE_LAYOUT_IN_CONTIG && layout != MOE_LAYOUT_OUT_CONTIG) return fail(MOE_ERR_INVALID, "unknown layout");
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    if (src_is_device) CUDA_TRY(cudaDeviceSynchronize());   // see moe_layer_set_expert
    const size_t bytes = (size_t)L->E_router * L->cfg.input_dim * sizeof(float);
    const void* src = w;
    int rc;
    if (!src_is_device) {
        if ((rc = grow(&L->stage_w, &L->stage_w_bytes, bytes))) return rc;
        CUDA_TRY(cudaMemcpyAsync(L->stage_w, w, bytes, cudaMemcpyHostToDevice, L->stream));
        src = L->stage_w;
    }
    const int n = launch_transpose_convert(src, MOE_DTYPE_F32, L->router_w, MOE_DTYPE_F32, L->E_router,
                                           L->cfg.input_dim, layout == MOE_LAYOUT_OUT_CONTIG, L->stream);
    if (n < 0) return fail(MOE_ERR_CUDA, "router repack launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    const int n2 = launch_router_transpose(L->router_w, L->router_wt, L->E_router, L->cfg.input_dim, L->stream);
    if (n2 < 0) return fail(MOE_ERR_CUDA, "router transpose launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n2;
    if (L->rplan) {
        const int n4 = router_tc_plan_set(L->rplan, L->router_w, L->router_w3, L->E_router, L->cfg.input_dim, L->stream);
        if (n4 < 0) return fail(MOE_ERR_CUDA, "router split failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n4;
    }
    if (L->router_nw) {
        const int n3 = launch_router_transpose_noise(L->router_w, L->router_nw, L->router_wt_noise, L->E_router,
                                                     L->cfg.input_dim, L->stream);
        if (n3 < 0) return fail(MOE_ERR_CUDA, "router transpose launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n3;
    }
    if (logit_bias) {
        CUDA_TRY(cudaMemcpyAsync(L->router_bias, logit_bias, sizeof(float) * L->E_router,
                                 src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, L->stream));
        L->has_bias = true;
    } else {
        L->has_bias = false;
    }
    CUDA_TRY(cudaStreamSynchronize(L->stream));
    L->router_set = true;
    return MOE_OK;
}

// ---- weight image: the layer's device-resident weights as one relocatable host blob ---------------------
namespace {

struct WeightImageHeader {       // 128 bytes, little-endian like the device
    char magic[8];               // "MOEB200W"
    int32_t version;             // 1
    int32_t compute_dtype, expert_kind;
    int32_t e_lo, e_hi;          // experts held (all of them without expert parallelism)
    int32_t input_dim, hidden_dim, output_dim;
    int32_t e_router, has_bias, has_noise_net;
    int32_t reserved0;
    int64_t total_bytes;
    int64_t off_w1, off_w3, off_w2, off_b1, off_b2, off_router, off_bias, off_noise;   // 0 = absent
};
static_assert(sizeof(WeightImageHeader) == 128, "weight image header layout");

struct WeightImageSection {
    int64_t WeightImageHeader::*off;
    void* ptr;
    size_t bytes;
};

// the sections present for this handle, in file order, and the header describing them
int weight_image_plan(moe_layer* L, WeightImageHeader* h, WeightImageSection (&sec)[8]) {
    const size_t el = dtype_size(L->cfg.compute_dtype);
    const size_t n = (size_t)(L->e_hi - L->e_lo);
    const size_t D = L->cfg.input_dim, H = L->cfg.hidden_dim, O = L->cfg.output_dim, R = L->E_router;
    const bool standard = L->cfg.expert_kind == MOE_EXPERT_STANDARD;
    memset(h, 0, sizeof(*h));
    memcpy(h->magic, "MOEB200W", 8);
    h->version = 1;
    h->compute_dtype = L->cfg.compute_dtype;
    h->expert_kind = L->cfg.expert_kind;
    h->e_lo = L->e_lo;
    h->e_hi = L->e_hi;
    h->input_dim = (int)D;
    h->hidden_dim = (int)H;
    h->output_dim = (int)O;
    h->e_router = (int)R;
    h->has_bias = L->has_bias ? 1 : 0;
    h->has_noise_net = L->router_nw ? 1 : 0;
    const WeightImageSection all[8] = {
        {&WeightImageHeader::off_w1, L->w1, n * H * D * el},
        {&WeightImageHeader::off_w3, standard ? nullptr : L->w3, n * H * D * el},
        {&WeightImageHeader::off_w2, L->w2, n * O * H * el},
        {&WeightImageHeader::off_b1, standard ? L->b1 : nullptr, n * H * sizeof(float)},
        {&WeightImageHeader::off_b2, standard ? L->b2 : nullptr, n * O * sizeof(float)},
        {&WeightImageHeader::off_router, L->router_w, R * D * sizeof(float)},
        {&WeightImageHeader::off_bias, L->has_bias ? L->router_bias : nullptr, R * sizeof(float)},
        {&WeightImageHeader::off_noise, L->router_nw, R * D * sizeof(float)},
    };
    int64_t off = sizeof(WeightImageHeader);
    for (int i = 0; i < 8; ++i) {
        sec[i] = all[i];
        if (!sec[i].ptr) continue;
        off = (off + 255) & ~(int64_t)255;
        h->*(sec[i].off) = off;
        off += (int64_t)sec[i].bytes;
    }
    h->total_bytes = off;
    return MOE_OK;
}

}  // namespace

int64_t moe_layer_weights_image_bytes(moe_layer_t* L) {
    if (!L) {
        fail(MOE_ERR_INVALID, "null handle");
        return -1;
    }
    if (check_ready(L)) return -1;
    WeightImageHeader h;
    WeightImageSection sec[8];
    weight_image_plan(L, &h, sec);
    return h.total_bytes;
}

int moe_layer_export_weights(moe_layer_t* L, void* dst, int64_t bytes) {
    if (!L || !dst) return fail(MOE_ERR_INVALID, "null argument");
    int rc = check_ready(L);
    if (rc) return rc;
    WeightImageHeader h;
    WeightImageSection sec[8];
    weight_image_plan(L, &h, sec);
    if (bytes < h.total_bytes) return fail(MOE_ERR_INVALID, "the image needs %lld bytes, got %lld", (long long)h.total_bytes, (long long)bytes);
    CUDA_TRY(cudaSetDevice(L->device));
    CUDA_TRY(cudaDeviceSynchronize());   // bias updates queued on the callers' streams
    memset(dst, 0, (size_t)h.total_bytes);
    memcpy(dst, &h, sizeof(h));
    for (const WeightImageSection& s : sec)
        if (s.ptr) CUDA_TRY(cudaMemcpy((char*)dst + h.*(s.off), s.ptr, s.bytes, cudaMemcpyDeviceToHost));
    return MOE_OK;
}

int moe_layer_import_weights(moe_layer_t* L, const void* src, int64_t bytes) {
    if (!L || !src) return fail(MOE_ERR_INVALID, "null argument");
    if (bytes < (int64_t)sizeof(WeightImageHeader)) return fail(MOE_ERR_INVALID, "not a weight image: too short");
    WeightImageHeader in;
    memcpy(&in, src, sizeof(in));
    if (memcmp(in.magic, "MOEB200W", 8) != 0) return fail(MOE_ERR_INVALID, "not a weight image: bad magic");
    if (in.version != 1) return fail(MOE_ERR_UNSUPPORTED, "weight image version %d is not supported", in.version);
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    int rc = ensure_weights(L);
    if (rc) return rc;
    if (in.compute_dtype != L->cfg.compute_dtype || in.expert_kind != L->cfg.expert_kind || in.e_lo != L->e_lo ||
        in.e_hi != L->e_hi || in.input_dim != L->cfg.input_dim || in.hidden_dim != L->cfg.hidden_dim ||
        in.output_dim != L->cfg.output_dim || in.e_router != L->E_router)
        return fail(MOE_ERR_INVALID,
                    "the weight image (dtype %d, kind %d, experts %d..%d, %d/%d/%d, %d router rows) does not match "
                    "this layer (dtype %d, kind %d, experts %d..%d, %d/%d/%d, %d router rows)",
                    in.compute_dtype, in.expert_kind, in.e_lo, in.e_hi - 1, in.input_dim, in.hidden_dim, in.output_dim,
                    in.e_router, L->cfg.compute_dtype, L->cfg.expert_kind, L->e_lo, L->e_hi - 1, L->cfg.input_dim,
                    L->cfg.hidden_dim, L->cfg.output_dim, L->E_router);
    if (in.has_noise_net && 2 * L->E_router > MAX_ROUTER_EXPERTS)
        return fail(MOE_ERR_UNSUPPORTED, "a router noise network needs 2*%d <= %d router rows", L->E_router, MAX_ROUTER_EXPERTS);
    // the image decides whether the bias and the noise network exist; lay the handle out like it first
    if (in.has_noise_net && !L->router_nw) {
        const size_t D = L->cfg.input_dim;
        if ((rc = dev_alloc(&L->router_nw, (size_t)L->E_router * D))) return rc;
        if ((rc = dev_alloc(&L->router_wt_noise, (size_t)router_e_pad(2 * L->E_router) * router_d_pad((int)D)))) return rc;
    } else if (!in.has_noise_net && L->router_nw) {
        CUDA_TRY(cudaDeviceSynchronize());
        dev_free(L->router_nw);
        dev_free(L->router_wt_noise);
        L->router_nw = L->router_wt_noise = nullptr;
    }
    L->has_bias = in.has_bias != 0;
    WeightImageHeader want;
    WeightImageSection sec[8];
    weight_image_plan(L, &want, sec);
    if (in.total_bytes != want.total_bytes || bytes < in.total_bytes)
        return fail(MOE_ERR_INVALID, "weight image is %lld bytes (buffer %lld), this layer's is %lld",
                    (long long)in.total_bytes, (long long)bytes, (long long)want.total_bytes);
    for (const WeightImageSection& s : sec) {
        if (!s.ptr) continue;
        if (in.*(s.off) != want.*(s.off)) return fail(MOE_ERR_INVALID, "weight image sections are laid out differently");
        CUDA_TRY(cudaMemcpyAsync(s.ptr, (const char*)src + in.*(s.off), s.bytes, cudaMemcpyHostToDevice, L->stream));
    }
    int n = launch_router_transpose(L->router_w, L->router_wt, L->E_router, L->cfg.input_dim, L->stream);
    if (n < 0) return fail(MOE_ERR_CUDA, "router transpose launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n;
    if (L->rplan) {
        n = router_tc_plan_set(L->rplan, L->router_w, L->router_w3, L->E_router, L->cfg.input_dim, L->stream);
        if (n < 0) return fail(MOE_ERR_CUDA, "router split failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n;
    }
    if (L->router_nw) {
        n = launch_router_transpose_noise(L->router_w, L->router_nw, L->router_wt_noise, L->E_router, L->cfg.input_dim, L->stream);
        if (n < 0) return fail(MOE_ERR_CUDA, "router transpose launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += n;
    }
    CUDA_TRY(cudaStreamSynchronize(L->stream));
    L->expert_set.assign(L->expert_set.size(), 1);
    L->router_set = true;
    return MOE_OK;
}

int moe_layer_set_aux_free(moe_layer_t* L, int enable, float learning_rate, float momentum, int update_freq,
                           const float* bias_momentum, int64_t update_counter) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    drop_graphs(L);
    if (!enable) {
        L->aux_free = false;
        return MOE_OK;
    }
    if (update_freq < 1) return fail(MOE_ERR_INVALID, "update_freq must be at least 1");
    if (L->ep) return fail(MOE_ERR_UNSUPPORTED, "the device bias update is not offered with expert parallelism");
    if (L->cfg.shared_mode == MOE_SHARED_LAYER_BLEND)
        return fail(MOE_ERR_UNSUPPORTED, "the device bias update is not offered with num_shared_experts > 0");
    if (!L->has_bias) return fail(MOE_ERR_STATE, "give the bias to moe_layer_set_router first");
    CUDA_TRY(cudaSetDevice(L->device));
    int rc;
    if (!L->bias_momentum && (rc = dev_alloc(&L->bias_momentum, (size_t)L->E_router))) return rc;
    if (bias_momentum)
        CUDA_TRY(cudaMemcpyAsync(L->bias_momentum, bias_momentum, sizeof(float) * L->E_router, cudaMemcpyHostToDevice, L->stream));
    else
        CUDA_TRY(cudaMemsetAsync(L->bias_momentum, 0, sizeof(float) * L->E_router, L->stream));
    CUDA_TRY(cudaStreamSynchronize(L->stream));
    L->aux_lr = learning_rate;
    L->aux_momentum = momentum;
    L->aux_freq = update_freq;
    L->aux_counter = update_counter;
    L->aux_free = true;
    return MOE_OK;
}

int moe_layer_aux_free_state(moe_layer_t* L, float* bias, float* bias_momentum, int64_t* update_counter) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    if (!L->aux_free) return fail(MOE_ERR_STATE, "the device bias update is not enabled (moe_layer_set_aux_free)");
    CUDA_TRY(cudaSetDevice(L->device));
    CUDA_TRY(cudaDeviceSynchronize());   // updates queued on the callers' streams
    if (bias) CUDA_TRY(cudaMemcpy(bias, L->router_bias, sizeof(float) * L->E_router, cudaMemcpyDeviceToHost));
    if (bias_momentum)
        CUDA_TRY(cudaMemcpy(bias_momentum, L->bias_momentum, sizeof(float) * L->E_router, cudaMemcpyDeviceToHost));
    if (update_counter) *update_counter = L->aux_counter;
    return MOE_OK;
}

int moe_layer_set_router_noise_network(moe_layer_t* L, const float* noise_w, int layout, int src_is_device) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    if (!noise_w) {   // back to plain Gaussian noise
        CUDA_TRY(cudaStreamSynchronize(L->stream));
        dev_free(L->router_nw);
        dev_free(L->router_wt_noise);
        L->router_nw = L->router_wt_noise = nullptr;
        return MOE_OK;
    }
    if (layout != MOE_LAYOUT_IN_CONTIG && layout != MOE_LAYOUT_OUT_CONTIG) return fail(MOE_ERR_INVALID, "unknown layout");
    if (!L->router_set) return fail(MOE_ERR_STATE, "set the router weights before its noise network");
    if (2 * L->E_router > MAX_ROUTER_EXPERTS)
        return fail(MOE_ERR_UNSUPPORTED, "a router noise network needs 2*%d <= %d router rows", L->E_router, MAX_ROUTER_EXPERTS);
    if (src_is_device) CUDA_TRY(cudaDeviceSynchronize());   // see moe_layer_set_expert
    const size_t D = L->cfg.input_dim;
    const size_t bytes = (size_t)L->E_router * D * sizeof(float);
    int rc;
    if (!L->router_nw) {
        if ((rc = dev_alloc(&L->router_nw, (size_t)L->E_router * D))) return rc;
        if ((rc = dev_alloc(&L->router_wt_noise, (size_t)router_e_pad(2 * L->E_router) * router_d_pad((int)D)))) return rc;
    }
    const void* src = noise_w;
    if (!src_is_device) {
        if ((rc = grow(&L->stage_w, &L->stage_w_bytes, bytes))) return rc;
        CUDA_TRY(cudaMemcpyAsync(L->stage_w, noise_w, bytes, cudaMemcpyHostToDevice, L->stream));
        src = L->stage_w;
    }
    const int n = launch_transpose_convert(src, MOE_DTYPE_F32, L->router_nw, MOE_DTYPE_F32, L->E_router, (int)D,
                                           layout == MOE_LAYOUT_OUT_CONTIG, L->stream);
    if (n < 0) return fail(MOE_ERR_CUDA, "router repack launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    const int n2 = launch_router_transpose_noise(L->router_w, L->router_nw, L->router_wt_noise, L->E_router, (int)D, L->stream);
    if (n2 < 0) return fail(MOE_ERR_CUDA, "router transpose launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    L->launches += n + n2;
    CUDA_TRY(cudaStreamSynchronize(L->stream));
    return MOE_OK;
}

int moe_layer_set_router_noise(moe_layer_t* L, const float* noise, float noise_scale) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    if (noise && !(noise_scale >= 0.f)) return fail(MOE_ERR_INVALID, "noise_scale must be non-negative");
    L->noise = noise;
    L->noise_scale = noise ? noise_scale : 0.f;
    return MOE_OK;
}

int moe_layer_forward(moe_layer_t* L, const void* x, int x_dtype, int64_t T, int training, float* out,
                      const moe_forward_outputs_t* opt, void* cuda_stream) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    return forward_small(L, x, x_dtype, T, training, out, opt, reinterpret_cast<cudaStream_t>(cuda_stream));
}

int moe_layer_forward_host(moe_layer_t* L, const void* x, int x_dtype, int64_t T, int training, float* out,
                           const moe_forward_outputs_t* opt) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    if (T < 0) return fail(MOE_ERR_INVALID, "T must be non-negative");
    if (x_dtype != MOE_DTYPE_F32 && x_dtype != MOE_DTYPE_BF16) return fail(MOE_ERR_INVALID, "unknown x_dtype");
    if (T > 0 && (!x || !out)) return fail(MOE_ERR_INVALID, "x and out must not be null");
    CUDA_TRY(cudaSetDevice(L->device));
    static const moe_forward_outputs_t none = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    if (!opt) opt = &none;
    int32_t ku = 0, ep = 0, er = 0;
    moe_layer_dims(L, &ku, &ep, &er);
    const size_t xb = (size_t)T * L->cfg.input_dim * dtype_size(x_dtype);
    const size_t ob = (size_t)T * L->cfg.output_dim * sizeof(float);
    // one device block for the optional outputs
    size_t off = 0;
    auto take = [&](bool want, size_t bytes) {
        const size_t o = off;
        if (want) off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_loss = take(opt->loss, 4), o_idx = take(opt->indices, (size_t)T * ku * 4),
                 o_gate = take(opt->gates, (size_t)T * ku * 4), o_probs = take(opt->probs, (size_t)T * ep * 4),
                 o_logits = take(opt->logits, (size_t)T * er * 4), o_tpe = take(opt->tokens_per_expert, (size_t)L->E * 8),
                 o_ent = take(opt->routing_entropy, 4);
    int rc;
    // small calls: status, output and optional outputs share one device block and one pinned block
    const size_t out_off = 256, opt_off = out_off + ((ob + 255) & ~(size_t)255), x_off = opt_off + ((off + 255) & ~(size_t)255);
    const bool small_call = !L->ep && x_off + xb <= moe_layer::PIN_SMALL_CALL;
    if ((rc = grow(&L->hx, &L->hx_bytes, xb))) return rc;
    if (!small_call) {
        if ((rc = grow(reinterpret_cast<void**>(&L->hout), &L->hout_bytes, ob))) return rc;
        if ((rc = grow(&L->hopt, &L->hopt_bytes, off))) return rc;
    }
    float* out_dev = small_call ? reinterpret_cast<float*>(L->small_dev + out_off) : L->hout;
    char* ob_dev = small_call ? L->small_dev + opt_off : reinterpret_cast<char*>(L->hopt);
    moe_forward_outputs_t d;
    d.loss = opt->loss ? reinterpret_cast<float*>(ob_dev + o_loss) : nullptr;
    d.indices = opt->indices ? reinterpret_cast<int32_t*>(ob_dev + o_idx) : nullptr;
    d.gates = opt->gates ? reinterpret_cast<float*>(ob_dev + o_gate) : nullptr;
    d.probs = opt->probs ? reinterpret_cast<float*>(ob_dev + o_probs) : nullptr;
    d.logits = opt->logits ? reinterpret_cast<float*>(ob_dev + o_logits) : nullptr;
    d.tokens_per_expert = opt->tokens_per_expert ? reinterpret_cast<int64_t*>(ob_dev + o_tpe) : nullptr;
    d.routing_entropy = opt->routing_entropy ? reinterpret_cast<float*>(ob_dev + o_ent) : nullptr;
    cudaStream_t s = L->stream;
    // Large batches are cut into token chunks: chunk c+1 is copied in and chunk c-1 copied out
    // while chunk c computes.  Tokens are independent, so outputs do not change; loss, entropy
    // and counts are finished from the statistics summed over the chunks.
    int nchunks = 1;
    int env_chunks = 0;   // MOE_B200_HOST_CHUNKS = n: n equal chunks (1 = off); unset: the default schedule
    // (not with the capacity constraint, whose capacity and first-come order span the whole batch)
    // With expert parallelism every chunk is a collective, so all ranks must cut alike: they decide from
    // the largest batch of any rank and every rank makes the same number of chunks (empty ones included).
    int64_t T_rule = T;
    if (L->ep && (rc = ep_max_tokens(L->ep, T, s, &T_rule, g_err, sizeof(g_err)))) return rc;
    if (L->cfg.shared_mode != MOE_SHARED_LAYER_BLEND && T_rule >= 8192 && !(L->cfg.drop_tokens && training) &&
        !(L->noise && training) && !(L->aux_free && training)) {
        env_chunks = L->host_chunks;
        nchunks = env_chunks > 0 ? env_chunks : 5;
        if (env_chunks <= 0) {
            // A chunk must still give every expert enough rows that its weights are not streamed for
            // nothing (every chunk reads all weights again): at least 512 rows per expert and chunk.
            const int world = L->ep ? ep_world(L->ep) : 1;
            const int64_t rows_per_expert = T_rule * world * L->k_tot / L->E;
            const int64_t fit = rows_per_expert / 512;
            if (fit < 5) {
                nchunks = fit < 1 ? 1 : (int)fit;
                env_chunks = nchunks;        // equal chunks
            }
        }
        if (nchunks > moe_layer::MAX_CHUNKS) nchunks = moe_layer::MAX_CHUNKS;
    }
    if (nchunks > 1) {
        const int nsum = L->E + L->E_probs + 3;
        if (!L->s_in) {
            CUDA_TRY(cudaStreamCreateWithFlags(&L->s_in, cudaStreamNonBlocking));
            CUDA_TRY(cudaStreamCreateWithFlags(&L->s_out, cudaStreamNonBlocking));
            L->timeline = L->host_timeline;
            const unsigned ev_flags = L->timeline ? cudaEventDefault : cudaEventDisableTiming;
            for (auto& e : L->ev_in) CUDA_TRY(cudaEventCreateWithFlags(&e, ev_flags));
            for (auto& e : L->ev_done) CUDA_TRY(cudaEventCreateWithFlags(&e, ev_flags));
            if (L->timeline) {
                CUDA_TRY(cudaEventCreate(&L->ev_t0));
                for (auto& e : L->ev_in0) CUDA_TRY(cudaEventCreate(&e));
                for (auto& e : L->ev_out1) CUDA_TRY(cudaEventCreate(&e));
            }
            if ((rc = dev_alloc(&L->chunk_acc, (size_t)nsum))) return rc;
            if ((rc = dev_alloc(&L->chunk_tpe_acc, (size_t)L->E))) return rc;
        }
        // Chunk boundaries (multiples of 64 tokens).  By default a small first chunk and a shrinking tail: only
        // the copy-in of the first and the copy-out of the last chunk are not hidden behind compute.
        std::vector<int64_t> bounds;
        bounds.push_back(0);
        if (env_chunks > 0) {
            const int64_t Tc = ((T + nchunks - 1) / nchunks + 63) / 64 * 64;
            for (int c = 1; c < nchunks; ++c) {
                const int64_t t = std::min<int64_t>(T, c * Tc);
                if (L->ep || (t > bounds.back() && t < T)) bounds.push_back(t);
            }
        } else {
            // thirty-seconds of the batch: the copy-out of a chunk must fit under the next chunk's compute
            // (the output is twice the input's bytes), so the chunks shrink towards the end
            static const int parts[] = {2, 12, 10, 6, 2};
            const int np = 5;
            nchunks = np;
            int64_t acc32 = 0;
            for (int i = 0; i + 1 < np; ++i) {
                acc32 += parts[i];
                const int64_t t = std::min<int64_t>(T, (T * acc32 / 32 + 63) / 64 * 64);
                if (L->ep || (t > bounds.back() && t < T)) bounds.push_back(t);
            }
        }
        bounds.push_back(T);
        const int n_bounds = (int)bounds.size();
        const size_t xrow = (size_t)L->cfg.input_dim * dtype_size(x_dtype), orow = (size_t)L->cfg.output_dim * 4;
        CUDA_TRY(cudaMemsetAsync(L->chunk_acc, 0, sizeof(float) * nsum, s));
        CUDA_TRY(cudaMemsetAsync(L->chunk_tpe_acc, 0, sizeof(int64_t) * L->E, s));
        if (L->timeline) CUDA_TRY(cudaEventRecord(L->ev_t0, L->s_in));
        for (int c = 0; c + 1 < (int)bounds.size(); ++c) {
            const int64_t t0 = bounds[c];
            const int64_t n = bounds[c + 1] - t0;
            if (L->timeline) CUDA_TRY(cudaEventRecord(L->ev_in0[c], L->s_in));
            if (n > 0)
                CUDA_TRY(cudaMemcpyAsync((char*)L->hx + t0 * xrow, (const char*)x + t0 * xrow, n * xrow,
                                         cudaMemcpyHostToDevice, L->s_in));
            CUDA_TRY(cudaEventRecord(L->ev_in[c], L->s_in));
            CUDA_TRY(cudaStreamWaitEvent(s, L->ev_in[c], 0));
            moe_forward_outputs_t dc = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
            if (d.indices) dc.indices = d.indices + t0 * ku;
            if (d.gates) dc.gates = d.gates + t0 * ku;
            if (d.probs) dc.probs = d.probs + t0 * ep;
            if (d.logits) dc.logits = d.logits + t0 * er;
            dc.tokens_per_expert = L->chunk_tpe_acc;       // the scan kernel adds every chunk's sums in place
            dc.loss = d.loss;                              // written by the last chunk only (expert parallel)
            dc.routing_entropy = d.routing_entropy;
            ChunkCtx cc;
            cc.sums = L->chunk_acc;
            cc.want_entropy = d.routing_entropy != nullptr;
            cc.ep_mode = c == 0 ? 1 : (c + 2 == n_bounds ? 3 : 2);
            if ((rc = forward_device(L, (char*)L->hx + t0 * xrow, x_dtype, n, training, L->hout + t0 * L->cfg.output_dim,
                                     &dc, s, &cc)))
                return rc;
            CUDA_TRY(cudaEventRecord(L->ev_done[c], s));
            CUDA_TRY(cudaStreamWaitEvent(L->s_out, L->ev_done[c], 0));
            if (n > 0)
                CUDA_TRY(cudaMemcpyAsync((char*)out + t0 * orow, (char*)L->hout + t0 * orow, n * orow, cudaMemcpyDeviceToHost,
                                         L->s_out));
            if (n == 0) {
                if (L->timeline) CUDA_TRY(cudaEventRecord(L->ev_out1[c], L->s_out));
                continue;
            }
            if (d.indices) CUDA_TRY(cudaMemcpyAsync(opt->indices + t0 * ku, dc.indices, (size_t)n * ku * 4, cudaMemcpyDeviceToHost, L->s_out));
            if (d.gates) CUDA_TRY(cudaMemcpyAsync(opt->gates + t0 * ku, dc.gates, (size_t)n * ku * 4, cudaMemcpyDeviceToHost, L->s_out));
            if (d.probs) CUDA_TRY(cudaMemcpyAsync(opt->probs + t0 * ep, dc.probs, (size_t)n * ep * 4, cudaMemcpyDeviceToHost, L->s_out));
            if (d.logits) CUDA_TRY(cudaMemcpyAsync(opt->logits + t0 * er, dc.logits, (size_t)n * er * 4, cudaMemcpyDeviceToHost, L->s_out));
            if (L->timeline) CUDA_TRY(cudaEventRecord(L->ev_out1[c], L->s_out));
        }
        if (!L->ep) {
            if (launch_finish_loss(L->chunk_acc, L->chunk_tpe_acc, T, L->E, L->E_probs, L->k_tot, L->cfg.balance_alpha,
                                   L->cfg.z_loss_weight, training, d.loss, d.routing_entropy, s) < 0)
                return fail(MOE_ERR_CUDA, "loss launch failed");
            L->launches += 1;
        }
        if (d.loss) CUDA_TRY(cudaMemcpyAsync(opt->loss, d.loss, 4, cudaMemcpyDeviceToHost, s));
        if (d.tokens_per_expert)
            CUDA_TRY(cudaMemcpyAsync(opt->tokens_per_expert, L->chunk_tpe_acc, (size_t)L->E * 8, cudaMemcpyDeviceToHost, s));
        if (d.routing_entropy) CUDA_TRY(cudaMemcpyAsync(opt->routing_entropy, d.routing_entropy, 4, cudaMemcpyDeviceToHost, s));
        CUDA_TRY(cudaStreamSynchronize(L->s_out));
        CUDA_TRY(cudaStreamSynchronize(s));
        if (L->timeline) {
            for (int c = 0; c + 1 < (int)bounds.size(); ++c) {
                float a = 0, b = 0, dn = 0, o = 0;
                cudaEventElapsedTime(&a, L->ev_t0, L->ev_in0[c]);
                cudaEventElapsedTime(&b, L->ev_t0, L->ev_in[c]);
                cudaEventElapsedTime(&dn, L->ev_t0, L->ev_done[c]);
                cudaEventElapsedTime(&o, L->ev_t0, L->ev_out1[c]);
                fprintf(stderr, "[moe_b200 timeline] chunk %d tokens %lld: copy-in %.3f..%.3f ms, compute done %.3f, copy-out done %.3f\n",
                        c, (long long)(bounds[c + 1] - bounds[c]), a, b, dn, o);
            }
        }
        int32_t stc = 0;
        CUDA_TRY(cudaMemcpy(&stc, L->status, sizeof(stc), cudaMemcpyDeviceToHost));
        return status_to_rc(L, stc);
    }
    if (small_call) {
        if ((rc = grow_pinned(&L->pin, &L->pin_bytes, x_off + xb))) return rc;
        if (xb) {
            memcpy(L->pin + x_off, x, xb);
            CUDA_TRY(cudaMemcpyAsync(L->hx, L->pin + x_off, xb, cudaMemcpyHostToDevice, s));
        }
        // Between a copy in and the copy out, chained plain launches beat a graph replay (measured on
        // B200, one position of a 512/1376 layer: 57 against 62-66 us per call): the first kernel starts
        // sooner after the copy than a graph does.  MOE_B200_CHAIN=0 brings the replay back.
        if ((rc = forward_small(L, L->hx, x_dtype, T, training, out_dev, &d, s, !L->chain_enabled))) return rc;
        CUDA_TRY(cudaMemcpyAsync(L->pin, L->small_dev, opt_off + off, cudaMemcpyDeviceToHost, s));
        CUDA_TRY(cudaStreamSynchronize(s));
        if (ob) memcpy(out, L->pin + out_off, ob);
        const char* po = L->pin + opt_off;
        if (opt->loss) memcpy(opt->loss, po + o_loss, 4);
        if (opt->indices && T) memcpy(opt->indices, po + o_idx, (size_t)T * ku * 4);
        if (opt->gates && T) memcpy(opt->gates, po + o_gate, (size_t)T * ku * 4);
        if (opt->probs && T) memcpy(opt->probs, po + o_probs, (size_t)T * ep * 4);
        if (opt->logits && T) memcpy(opt->logits, po + o_logits, (size_t)T * er * 4);
        if (opt->tokens_per_expert) memcpy(opt->tokens_per_expert, po + o_tpe, (size_t)L->E * 8);
        if (opt->routing_entropy) memcpy(opt->routing_entropy, po + o_ent, 4);
        int32_t st = 0;
        memcpy(&st, L->pin, sizeof(st));
        return status_to_rc(L, st);
    }
    if (xb) CUDA_TRY(cudaMemcpyAsync(L->hx, x, xb, cudaMemcpyHostToDevice, s));
    if ((rc = forward_small(L, L->hx, x_dtype, T, training, L->hout, &d, s))) return rc;
    if (ob) CUDA_TRY(cudaMemcpyAsync(out, L->hout, ob, cudaMemcpyDeviceToHost, s));
    if (d.loss) CUDA_TRY(cudaMemcpyAsync(opt->loss, d.loss, 4, cudaMemcpyDeviceToHost, s));
    if (d.indices && T) CUDA_TRY(cudaMemcpyAsync(opt->indices, d.indices, (size_t)T * ku * 4, cudaMemcpyDeviceToHost, s));
    if (d.gates && T) CUDA_TRY(cudaMemcpyAsync(opt->gates, d.gates, (size_t)T * ku * 4, cudaMemcpyDeviceToHost, s));
    if (d.probs && T) CUDA_TRY(cudaMemcpyAsync(opt->probs, d.probs, (size_t)T * ep * 4, cudaMemcpyDeviceToHost, s));
    if (d.logits && T) CUDA_TRY(cudaMemcpyAsync(opt->logits, d.logits, (size_t)T * er * 4, cudaMemcpyDeviceToHost, s));
    if (d.tokens_per_expert)
        CUDA_TRY(cudaMemcpyAsync(opt->tokens_per_expert, d.tokens_per_expert, (size_t)L->E * 8, cudaMemcpyDeviceToHost, s));
    if (d.routing_entropy) CUDA_TRY(cudaMemcpyAsync(opt->routing_entropy, d.routing_entropy, 4, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    int32_t st = 0;
    CUDA_TRY(cudaMemcpy(&st, L->status, sizeof(st), cudaMemcpyDeviceToHost));
    return status_to_rc(L, st);
}

static int compute_gates_impl(int gate_kind, int num_experts, int num_shared, int top_k, int index_base,
                              const float* logits, const float* jitter_u, float eps, int64_t T, int32_t* indices,
                              float* gates, float* probs, void* cuda_stream) {
    if (gate_kind < MOE_GATE_TOPK || gate_kind > MOE_GATE_SHARED_TOPK) return fail(MOE_ERR_INVALID, "unknown gate_kind");
    if (num_experts < 1 || num_experts > MAX_ROUTER_EXPERTS)
        return fail(MOE_ERR_UNSUPPORTED, "num_experts must be in 1..%d", MAX_ROUTER_EXPERTS);
    const int S = gate_kind == MOE_GATE_SHARED_TOPK ? num_shared : 0;
    const int k = gate_kind == MOE_GATE_SWITCH ? 1 : top_k;
    if (S < 0 || S >= num_experts) return fail(MOE_ERR_INVALID, "num_shared out of range");
    if (k < 1 || k > num_experts - S) return fail(MOE_ERR_INVALID, "top_k out of range");
    if (k + S > MAX_KTOT) return fail(MOE_ERR_UNSUPPORTED, "more than %d selected experts per token", MAX_KTOT);
    if (index_base != 0 && index_base != 1) return fail(MOE_ERR_INVALID, "index_base must be 0 or 1");
    if (T < 0 || (T > 0 && !logits)) return fail(MOE_ERR_INVALID, "bad logits/T");
    if (T == 0) return MOE_OK;
    if (launch_gates_only(gate_kind, num_experts, S, k, index_base, logits, jitter_u, eps, T, indices, gates, probs,
                          reinterpret_cast<cudaStream_t>(cuda_stream)) < 0)
        return fail(MOE_ERR_CUDA, "compute_gates launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return MOE_OK;
}

int moe_compute_gates(int gate_kind, int num_experts, int num_shared, int top_k, int index_base, const float* logits,
                      int64_t T, int32_t* indices, float* gates, float* probs, void* cuda_stream) {
    return compute_gates_impl(gate_kind, num_experts, num_shared, top_k, index_base, logits, nullptr, 0.f, T, indices,
                              gates, probs, cuda_stream);
}

int moe_compute_gates_jitter(int gate_kind, int num_experts, int num_shared, int top_k, int index_base,
                             const float* logits, const float* jitter_u, float eps, int64_t T, int32_t* indices,
                             float* gates, float* probs, void* cuda_stream) {
    if (T > 0 && !jitter_u) return fail(MOE_ERR_INVALID, "jitter_u must not be null");
    if (!(eps >= 0.f)) return fail(MOE_ERR_INVALID, "eps must be non-negative");
    return compute_gates_impl(gate_kind, num_experts, num_shared, top_k, index_base, logits, jitter_u, eps, T, indices,
                              gates, probs, cuda_stream);
}

int moe_compute_loss(float alpha, float z_weight, int n_probs, int k, int index_base, const int32_t* indices,
                     const float* probs, const float* logits, int n_logits, int64_t T, float* loss, void* cuda_stream) {
    if (n_probs < 1 || n_probs > MAX_EXPERTS) return fail(MOE_ERR_UNSUPPORTED, "n_probs must be in 1..%d", MAX_EXPERTS);
    if (k < 1 || T < 1 || !indices || !probs || !loss) return fail(MOE_ERR_INVALID, "bad argument");
    if (logits && n_logits < 1) return fail(MOE_ERR_INVALID, "n_logits must be positive");
    if (launch_loss_only(alpha, z_weight, n_probs, k, index_base, indices, probs, logits, n_logits, T, loss,
                         reinterpret_cast<cudaStream_t>(cuda_stream)) < 0)
        return fail(MOE_ERR_CUDA, "compute_loss launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return MOE_OK;
}

int moe_layer_set_profiling(moe_layer_t* L, int slots) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    if (slots < 0 || slots > 1024) return fail(MOE_ERR_INVALID, "slots must be in 0..1024");
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    CUDA_TRY(cudaDeviceSynchronize());
    for (auto& e : L->ev) cudaEventDestroy(e);
    L->ev.clear();
    L->prof_slots = 0;
    L->prof_calls = 0;
    L->prof_cur = 0;
    if (slots > 0) {
        L->ev.resize((size_t)slots * 8, nullptr);
        for (auto& e : L->ev) CUDA_TRY(cudaEventCreate(&e));
        L->prof_slots = slots;
    }
    return MOE_OK;
}

int moe_layer_stage_ms(moe_layer_t* L, int calls_back, float ms[7]) {
    if (!L || !ms) return fail(MOE_ERR_INVALID, "null argument");
    if (L->prof_slots <= 0) return fail(MOE_ERR_STATE, "profiling is not enabled");
    if (calls_back < 0 || calls_back >= L->prof_slots || calls_back >= L->prof_calls)
        return fail(MOE_ERR_INVALID, "that call is not in the profiling ring");
    CUDA_TRY(cudaSetDevice(L->device));
    const int slot = (int)((L->prof_calls - 1 - calls_back) % L->prof_slots);
    cudaEvent_t* ev = &L->ev[(size_t)slot * 8];
    CUDA_TRY(cudaEventSynchronize(ev[6]));
    // events: 0 start, 1 router, 2 scan, 3 permute, 4 gemm1, 5 gemm2, 6 combine
    for (int i = 0; i < 7; ++i) ms[i] = 0.f;
    for (int i = 0; i < 6; ++i) {
        float v = 0.f;
        if (cudaEventElapsedTime(&v, ev[i], ev[i + 1]) == cudaSuccess) ms[i] = v;
    }
    if (L->ep) ms[6] = ep_last_exchange_ms(L->ep);
    return MOE_OK;
}

int64_t moe_layer_launch_count(const moe_layer_t* L) { return L ? L->launches : 0; }

int moe_layer_router_rechecks(moe_layer_t* L, int64_t* tokens) {
    if (!L || !tokens) return fail(MOE_ERR_INVALID, "null argument");
    *tokens = 0;
    if (!L->tc_recheck) return MOE_OK;
    CUDA_TRY(cudaSetDevice(L->device));
    CUDA_TRY(cudaDeviceSynchronize());
    int32_t v = 0;
    CUDA_TRY(cudaMemcpy(&v, L->tc_recheck, sizeof(v), cudaMemcpyDeviceToHost));
    *tokens = v;
    return MOE_OK;
}

int moe_layer_tile_rows(moe_layer_t* L, int64_t T) {
    if (!L || T < 0) return fail(MOE_ERR_INVALID, "bad argument");
    return pick_tile_m(L, T * L->k_tot, L->E);
}

int moe_layer_gemm_kernel(moe_layer_t* L, int64_t T) {
    if (!L || T < 0) return fail(MOE_ERR_INVALID, "bad argument");
    return pick_gemm_kernel(L, T * L->k_tot, L->E);
}

int moe_layer_graph_replays(const moe_layer_t* L, int64_t* replays) {
    if (!L || !replays) return fail(MOE_ERR_INVALID, "null argument");
    *replays = L->graph_replays;
    return MOE_OK;
}

int moe_layer_device_status(moe_layer_t* L, int32_t* status) {
    if (!L || !status) return fail(MOE_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(L->device));
    CUDA_TRY(cudaMemcpy(status, L->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
    return MOE_OK;
}

int moe_selftest_bounded_wait(int device, int limit_us, int32_t* status_out, int32_t* waited_us) {
    if (!status_out || !waited_us) return fail(MOE_ERR_INVALID, "null argument");
    if (limit_us < 1 || limit_us > 1000000) return fail(MOE_ERR_INVALID, "limit_us must be in 1..1000000");
    CUDA_TRY(cudaSetDevice(device));
    if (run_bounded_wait_selftest(limit_us, status_out, waited_us) != 0)
        return fail(MOE_ERR_CUDA, "bounded-wait self-test failed to run: %s", cudaGetErrorString(cudaGetLastError()));
    return MOE_OK;
}

int moe_ep_unique_id(void* id128) { return ep_unique_id(id128, g_err, sizeof(g_err)); }

int64_t moe_ep_layout(const int32_t* counts, int world, int num_experts, int rank, int tile_m, int64_t* send_off,
                      int64_t* recv_off, int32_t* local_off, int32_t* tile_prefix) {
    if (!counts || !send_off || !recv_off || !local_off || !tile_prefix)
        return fail(MOE_ERR_INVALID, "null argument");
    if (world < 1 || rank < 0 || rank >= world || num_experts < 1 || num_experts % world || tile_m < 1)
        return fail(MOE_ERR_INVALID, "bad world/rank/num_experts/tile_m");
    return ep_plan_layout(counts, world, num_experts, rank, tile_m, send_off, recv_off, local_off, tile_prefix);
}

int moe_ep_set_timeout_ms(moe_layer_t* L, int timeout_ms) {
    if (!L) return fail(MOE_ERR_INVALID, "null handle");
    if (timeout_ms < 1) return fail(MOE_ERR_INVALID, "timeout_ms must be positive");
    L->ep_timeout_ms = timeout_ms;
    if (L->ep) return ep_set_timeout_ms(L->ep, timeout_ms);
    return MOE_OK;
}

int moe_ep_init(moe_layer_t* L, const void* id128, int rank, int world) {
    if (!L || !id128) return fail(MOE_ERR_INVALID, "null argument");
    if (world < 1 || rank < 0 || rank >= world) return fail(MOE_ERR_INVALID, "bad rank/world");
    if (L->E % world) return fail(MOE_ERR_INVALID, "num_experts (%d) must be divisible by the world size (%d)", L->E, world);
    if (L->cfg.shared_mode != MOE_SHARED_NONE)
        return fail(MOE_ERR_UNSUPPORTED, "expert parallelism with shared experts is not implemented");
    if (L->w1) return fail(MOE_ERR_STATE, "moe_ep_init must come before moe_layer_set_expert");
    if (L->ep) return fail(MOE_ERR_STATE, "expert parallelism is already initialised");
    CUDA_TRY(cudaSetDevice(L->device));
    drop_graphs(L);
    EpConfig ec;
    ec.rank = rank;
    ec.world = world;
    ec.E = L->E;
    ec.E_probs = L->E_probs;
    ec.k_tot = L->k_tot;
    ec.D = L->cfg.input_dim;
    ec.H = L->cfg.hidden_dim;
    ec.O = L->cfg.output_dim;
    ec.elt = (int)dtype_size(L->cfg.compute_dtype);
    ec.tile_m = L->cfg.compute_dtype == MOE_DTYPE_BF16 ? TC_TILE_M : F32_TILE_M;
    ec.tile_m_alt = L->cfg.compute_dtype == MOE_DTYPE_BF16 ? TC_PAIR_TILE_M : 0;
    ec.alpha = L->cfg.balance_alpha;
    ec.z_weight = L->cfg.z_loss_weight;
    ec.status = L->status;
    const int rc = ep_create(&L->ep, ec, id128, L->ep_timeout_ms, g_err, sizeof(g_err));
    if (rc) return rc;
    const int per = L->E / world;
    L->e_lo = rank * per;
    L->e_hi = L->e_lo + per;
    free_workspace(L);
    return MOE_OK;
}

}  // extern "C"
