// moe_route_static: the fused router + Switch/z-loss of the layer for callers that must not
// allocate device memory (a process that hands every byte of HBM to its own pools at start-up,
// or a latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply).  The per-CTA histograms and partial sums that the router kernel hands to
// the scan/loss kernel -- the only scratch this pair of kernels needs -- live in a file-scope
// device array instead of the handle's workspace.  Inputs and outputs stay caller-owned.
//
// The array is part of the loaded module: every GPU that loads the library holds
// MOE_ROUTE_STATIC_SCRATCH_BYTES of it until the process exits.
#include <cstdio>

#include "common.cuh"

namespace {

constexpr size_t SCRATCH_BYTES = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_route_scratch[SCRATCH_BYTES];

// In host code `g_route_scratch` is only a stand-in for the symbol, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, once per device.
constexpr int MAX_DEVICES = 64;
void* g_scratch_ptr[MAX_DEVICES] = {nullptr};
int g_num_sms[MAX_DEVICES] = {0};

thread_local char g_static_err[256] = "";

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

const char* moe_route_static_error(void) { return g_static_err; }

int64_t moe_route_static_scratch_bytes(void) { return (int64_t)SCRATCH_BYTES; }

int moe_route_static(int gate_kind, int num_experts, int num_shared, int top_k, int index_base, const void* x,
                     int x_dtype, int64_t T, int input_dim, const float* router_w, const float* logit_bias,
                     float balance_alpha, float z_loss_weight, int training, int32_t* indices, float* gates,
                     float* probs, float* loss, void* cuda_stream) {
    using namespace moe;
    auto fail = [](int code, const char* msg) {
        snprintf(g_static_err, sizeof(g_static_err), "%s", msg);
        return code;
    };
    if (gate_kind < MOE_GATE_TOPK || gate_kind > MOE_GATE_SHARED_TOPK) return fail(MOE_ERR_INVALID, "unknown gate_kind");
    if (num_experts < 1 || num_experts > MAX_ROUTER_EXPERTS)
        return fail(MOE_ERR_UNSUPPORTED, "num_experts must be in 1..128");
    const int S = gate_kind == MOE_GATE_SHARED_TOPK ? num_shared : 0;
    const int k = gate_kind == MOE_GATE_SWITCH ? 1 : top_k;
    if (S < 0 || S >= num_experts || (gate_kind == MOE_GATE_SHARED_TOPK && S < 1))
        return fail(MOE_ERR_INVALID, "num_shared out of range");
    if (k < 1 || k > num_experts - S) return fail(MOE_ERR_INVALID, "top_k out of range");
    if (k + S > MAX_KTOT) return fail(MOE_ERR_UNSUPPORTED, "more than 16 selected experts per token");
    if (index_base != 0 && index_base != 1) return fail(MOE_ERR_INVALID, "index_base must be 0 or 1");
    if (x_dtype != MOE_DTYPE_F32 && x_dtype != MOE_DTYPE_BF16) return fail(MOE_ERR_INVALID, "unknown x_dtype");
    if (T < 1 || input_dim < 1) return fail(MOE_ERR_INVALID, "T and input_dim must be positive");
    if (!x || !router_w || !indices || !gates) return fail(MOE_ERR_INVALID, "x, router_w, indices and gates must not be null");

    const int tpc = ROUTER_TOKENS_PER_CTA;   // the largest tile: the fewest per-CTA rows of scratch
    const int64_t num_cta64 = (T + tpc - 1) / tpc;
    const size_t b_counts = align256((size_t)num_cta64 * num_experts * sizeof(int32_t));
    const size_t b_psum = align256((size_t)num_cta64 * (num_experts + 1) * sizeof(float));
    const size_t b_ent = align256((size_t)num_cta64 * sizeof(double));
    const size_t b_tab = align256((size_t)(num_experts + 1) * sizeof(int32_t));
    const size_t b_wt = align256((size_t)router_e_pad(num_experts) * router_d_pad(input_dim) * sizeof(float));
    const size_t need = b_counts + b_psum + b_ent + 3 * b_tab + 256 + b_wt;
    if (need > SCRATCH_BYTES) {
        snprintf(g_static_err, sizeof(g_static_err),
                 "T=%lld with %d experts needs %zu bytes of scratch; the static array holds %zu "
                 "(use moe_layer_forward, which sizes its own workspace)",
                 (long long)T, num_experts, need, SCRATCH_BYTES);
        return MOE_ERR_INVALID;
    }

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return fail(MOE_ERR_CUDA, "cudaGetDevice failed (no current CUDA device)");
    if (!g_scratch_ptr[dev]) {
        // first call on this device: resolve the array's device address (with this device current)
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_route_scratch);
        if (e != cudaSuccess || !ptr) {
            snprintf(g_static_err, sizeof(g_static_err), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return MOE_ERR_CUDA;
        }
        g_scratch_ptr[dev] = ptr;
        if (cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_num_sms[dev] < 1)
            g_num_sms[dev] = 1;
    }
    unsigned char* base = reinterpret_cast<unsigned char*>(g_scratch_ptr[dev]);
    int32_t* cta_counts = reinterpret_cast<int32_t*>(base);
    float* cta_psum = reinterpret_cast<float*>(base + b_counts);
    double* cta_entropy = reinterpret_cast<double*>(base + b_counts + b_psum);
    int32_t* expert_count = reinterpret_cast<int32_t*>(base + b_counts + b_psum + b_ent);
    int32_t* expert_offset = reinterpret_cast<int32_t*>(base + b_counts + b_psum + b_ent + b_tab);
    int32_t* tile_prefix = reinterpret_cast<int32_t*>(base + b_counts + b_psum + b_ent + 2 * b_tab);
    float* loss_internal = reinterpret_cast<float*>(base + b_counts + b_psum + b_ent + 3 * b_tab);
    float* wt = reinterpret_cast<float*>(base + b_counts + b_psum + b_ent + 3 * b_tab + 256);
    // Nothing here has to start at zero: the transpose kernel writes the whole padded matrix,
    // the router kernel writes every per-CTA row before the scan kernel reads it, and the scan
    // kernel writes the tables and the loss it produces.

    cudaStream_t s = reinterpret_cast<cudaStream_t>(cuda_stream);
    // the router kernel reads a K-major, zero-padded copy of the router matrix: build it in the array
    if (launch_router_transpose(router_w, wt, num_experts, input_dim, s) < 0) {
        snprintf(g_static_err, sizeof(g_static_err), "router transpose launch failed: %s",
                 cudaGetErrorString(cudaGetLastError()));
        return MOE_ERR_CUDA;
    }
    RouterParams r{};
    r.x = x;
    r.w = router_w;
    r.wt = wt;
    r.bias = logit_bias;
    r.noise = nullptr;
    r.noise_scale = 0.f;
    r.noise_off = 0;
    r.T = T;
    r.D = input_dim;
    r.E = num_experts;
    r.E_router = num_experts;
    r.E_probs = num_experts;
    r.S = S;
    r.k = k;
    r.k_tot = k + S;
    r.shared_mode = S ? MOE_SHARED_GATING : MOE_SHARED_NONE;
    r.bias_gates_only = 0;
    r.index_base = index_base;
    r.tokens_per_cta = tpc;
    r.want_entropy = 0;
    r.idx = nullptr;
    r.gate = nullptr;
    r.cta_counts = cta_counts;
    r.cta_psum = cta_psum;
    r.cta_entropy = cta_entropy;
    r.u_idx = indices;
    r.u_gate = gates;
    r.u_probs = probs;
    r.u_logits = nullptr;
    if (launch_router(r, x_dtype, (int)num_cta64, g_num_sms[dev], s) < 0) {
        snprintf(g_static_err, sizeof(g_static_err), "router launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        return MOE_ERR_CUDA;
    }
    ScanParams sp{};
    sp.T = T;
    sp.E = num_experts;
    sp.E_probs = num_experts;
    sp.S = S;
    sp.k = k;
    sp.k_tot = k + S;
    sp.shared_mode = r.shared_mode;
    sp.num_cta = (int)num_cta64;
    sp.tile_m = TC_TILE_M;
    sp.training = training;
    sp.capacity = -1;
    sp.alpha = balance_alpha;
    sp.z_weight = z_loss_weight;
    sp.cta_counts = cta_counts;
    sp.cta_psum = cta_psum;
    sp.cta_entropy = cta_entropy;
    sp.expert_count = expert_count;
    sp.expert_offset = expert_offset;
    sp.tile_prefix = tile_prefix;
    sp.loss_internal = loss_internal;
    sp.u_loss = loss;
    sp.u_tokens_per_expert = nullptr;
    sp.u_entropy = nullptr;
    sp.ep_sums = nullptr;
    if (launch_scan(sp, s) < 0) {
        snprintf(g_static_err, sizeof(g_static_err), "scan launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        return MOE_ERR_CUDA;
    }
    return MOE_OK;
}

}  // extern "C"
