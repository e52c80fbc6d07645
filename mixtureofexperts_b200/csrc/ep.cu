// Expert-parallel dispatch/combine over NCCL (see ep.h).  NCCL is bound at run time with
// dlopen so that the library loads, and the single-GPU path works, without it; inside a
// process that already holds NCCL (for instance through torch.distributed) the same copy is
// reused.
//
// One forward call on every rank:
//   1. all-gather of the per-expert pair counts (E int32 per rank)          -> counts[world][E]
//   2. counts to the host (the one host synchronisation of the call): send/receive sizes,
//      the receive layout [local expert][source rank][rows] and its m-tile prefix
//   3. grouped ncclSend/ncclRecv of the permuted rows; rows for a rank's own experts are a
//      device-to-device copy
//   4. the expert GEMM pair on the received rows (callback)
//   5. grouped ncclSend/ncclRecv of the expert outputs back into the sender's row order
//   6. all-reduce of {counts, probability sums, lse^2 sum, T, entropy sum} and a one-warp kernel
//      that finishes the Switch loss over ALL ranks' tokens
// Received rows always land in this GPU's own memory before any TMA load touches them.
#include "ep.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/moe_b200.h"

namespace moe {

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi g_nccl;

int set_err(char* err, size_t n, int code, const char* msg, const char* detail = "") {
    if (err && n) snprintf(err, n, "%s%s", msg, detail);
    return code;
}

int load_nccl(char* err, size_t errlen) {
    if (g_nccl.lib) return MOE_OK;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return set_err(err, errlen, MOE_ERR_NCCL, "cannot load libnccl.so.2: ", dlerror());
#define BIND(field, sym)                                                                  \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(lib, sym));             \
    if (!g_nccl.field) return set_err(err, errlen, MOE_ERR_NCCL, "libnccl lacks symbol ", sym)
    BIND(GetUniqueId, "ncclGetUniqueId");
    BIND(CommInitRank, "ncclCommInitRank");
    BIND(CommDestroy, "ncclCommDestroy");
    BIND(GroupStart, "ncclGroupStart");
    BIND(GroupEnd, "ncclGroupEnd");
    BIND(Send, "ncclSend");
    BIND(Recv, "ncclRecv");
    BIND(AllGather, "ncclAllGather");
    BIND(AllReduce, "ncclAllReduce");
    BIND(GetErrorString, "ncclGetErrorString");
#undef BIND
    g_nccl.lib = lib;
    return MOE_OK;
}

// loss = alpha*N*sum_i f_i P_i (+ z*mean lse^2) from the all-reduced sums; one warp.
__global__ void ep_finish_loss_kernel(const float* sums, int E, int E_probs, int k_tot, float alpha, float z_weight,
                                      int training, float* u_loss, float* u_entropy) {
    const int lane = threadIdx.x;
    const float Tg = sums[E + E_probs + 1];
    float acc = 0.f;
    if (Tg > 0.f) {
        const float denom = (float)k_tot * Tg;
        for (int j = lane; j < E_probs; j += 32) acc += (sums[j] / denom) * (sums[E + j] / Tg);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float loss = 0.f;
        if (training && Tg > 0.f) {
            loss = alpha * (float)E_probs * acc;
            if (z_weight > 0.f) loss += z_weight * (sums[E + E_probs] / Tg);
        }
        if (u_loss) *u_loss = loss;
        if (u_entropy) *u_entropy = Tg > 0.f ? sums[E + E_probs + 2] / Tg : 0.f;
    }
}

}  // namespace

struct EpState {
    EpConfig cfg;
    ncclComm_t comm = nullptr;
    int per = 0;                    // experts per rank
    float* d_sums = nullptr;        // [E + E_probs + 3]
    int32_t* d_all_counts = nullptr;  // [world][E]
    int32_t* h_all_counts = nullptr;  // pinned
    int32_t* d_tables = nullptr;    // [2*(per+1)]: local expert_offset, local tile_prefix
    int32_t* h_tables = nullptr;    // pinned
    void* xr = nullptr;             // received rows       [rows_cap][D]
    void* hr = nullptr;             // hidden activations  [rows_cap][H]
    void* yr = nullptr;             // expert outputs      [rows_cap][O]
    int64_t rows_cap = 0;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    bool timed = false;
    // peer-memory mode
    bool peer_mode = true;
    std::vector<void*> peer_xr, peer_yb;   // [world] mapped buffers of every rank (own entry = local pointer)
    void* yb = nullptr;                    // [pairs_cap][O] outputs of this rank's pairs (written by the expert owners)
    int64_t pairs_cap = 0;
    int32_t* d_seg = nullptr;              // [per*world] segment starts
    int32_t* h_seg = nullptr;              // pinned
    void** d_segp = nullptr;               // [per*world] segment destinations
    void** h_segp = nullptr;               // pinned
    unsigned char* d_ipc = nullptr;        // [world][2 handles] staging for the handle all-gather
    unsigned char* h_ipc = nullptr;        // pinned
    void** d_ptrs = nullptr;               // [2E] expert_dst, expert_src
    void** h_ptrs = nullptr;               // pinned
    int32_t* d_flag = nullptr;             // barrier payload
};

int launch_finish_loss(const float* sums, int E, int E_probs, int k_tot, float alpha, float z_weight, int training,
                       float* u_loss, float* u_entropy, cudaStream_t s) {
    ep_finish_loss_kernel<<<1, 32, 0, s>>>(sums, E, E_probs, k_tot, alpha, z_weight, training, u_loss, u_entropy);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// Pure host arithmetic (no CUDA, no NCCL): see ep.h.
int64_t ep_plan_layout(const int32_t* cnt, int W, int E, int me, int tile_m, int64_t* send_off, int64_t* recv_off,
                       int32_t* local_off, int32_t* tile_prefix) {
    const int per = E / W;
    send_off[0] = 0;
    for (int e = 0; e < E; ++e) send_off[e + 1] = send_off[e] + cnt[(size_t)me * E + e];
    int64_t rows = 0;
    int64_t tiles = 0;
    for (int el = 0; el < per; ++el) {
        local_off[el] = (int32_t)rows;
        tile_prefix[el] = (int32_t)tiles;
        int64_t n_e = 0;
        for (int r = 0; r < W; ++r) {
            recv_off[(size_t)el * W + r] = rows + n_e;
            n_e += cnt[(size_t)r * E + me * per + el];
        }
        rows += n_e;
        tiles += (n_e + tile_m - 1) / tile_m;
    }
    local_off[per] = (int32_t)rows;
    tile_prefix[per] = (int32_t)tiles;
    return rows;
}

int ep_unique_id(void* id128, char* err, size_t errlen) {
    int rc = load_nccl(err, errlen);
    if (rc) return rc;
    ncclUniqueId id;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return set_err(err, errlen, MOE_ERR_NCCL, "ncclGetUniqueId: ", g_nccl.GetErrorString(r));
    memcpy(id128, &id, 128);
    return MOE_OK;
}

int ep_create(EpState** out, const EpConfig& cfg, const void* id128, char* err, size_t errlen) {
    *out = nullptr;
    int rc = load_nccl(err, errlen);
    if (rc) return rc;
    EpState* ep = new EpState();
    ep->cfg = cfg;
    ep->per = cfg.E / cfg.world;
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    const ncclResult_t r = g_nccl.CommInitRank(&ep->comm, cfg.world, id, cfg.rank);
    if (r != ncclSuccess) {
        delete ep;
        return set_err(err, errlen, MOE_ERR_NCCL, "ncclCommInitRank: ", g_nccl.GetErrorString(r));
    }
    bool ok = cudaMalloc(&ep->d_sums, sizeof(float) * (cfg.E + cfg.E_probs + 3)) == cudaSuccess &&
              cudaMalloc(&ep->d_all_counts, sizeof(int32_t) * cfg.world * cfg.E) == cudaSuccess &&
              cudaMallocHost(&ep->h_all_counts, sizeof(int32_t) * cfg.world * cfg.E) == cudaSuccess &&
              cudaMalloc(&ep->d_tables, sizeof(int32_t) * 3 * (ep->per + 1)) == cudaSuccess &&
              cudaMallocHost(&ep->h_tables, sizeof(int32_t) * 3 * (ep->per + 1)) == cudaSuccess;
    for (auto& e : ep->ev) ok = ok && cudaEventCreate(&e) == cudaSuccess;
    const char* mode = getenv("MOE_B200_EP_MODE");
    ep->peer_mode = !(mode && strcmp(mode, "nccl") == 0);
    ep->peer_xr.assign(cfg.world, nullptr);
    ep->peer_yb.assign(cfg.world, nullptr);
    const size_t ipc_bytes = (size_t)cfg.world * 2 * sizeof(cudaIpcMemHandle_t);
    ok = ok && cudaMalloc(&ep->d_ipc, ipc_bytes) == cudaSuccess && cudaMallocHost(&ep->h_ipc, ipc_bytes) == cudaSuccess &&
         cudaMalloc(&ep->d_ptrs, sizeof(void*) * 2 * cfg.E) == cudaSuccess &&
         cudaMallocHost(&ep->h_ptrs, sizeof(void*) * 2 * cfg.E) == cudaSuccess &&
         cudaMalloc(&ep->d_seg, sizeof(int32_t) * ep->per * cfg.world) == cudaSuccess &&
         cudaMallocHost(&ep->h_seg, sizeof(int32_t) * ep->per * cfg.world) == cudaSuccess &&
         cudaMalloc(&ep->d_segp, sizeof(void*) * ep->per * cfg.world) == cudaSuccess &&
         cudaMallocHost(&ep->h_segp, sizeof(void*) * ep->per * cfg.world) == cudaSuccess &&
         cudaMalloc(&ep->d_flag, sizeof(int32_t)) == cudaSuccess &&
         cudaMemset(ep->d_flag, 0, sizeof(int32_t)) == cudaSuccess;
    if (!ok) {
        ep_destroy(ep);
        return set_err(err, errlen, MOE_ERR_CUDA, "expert-parallel buffers: allocation failed");
    }
    *out = ep;
    return MOE_OK;
}

void ep_destroy(EpState* ep) {
    if (!ep) return;
    if (ep->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ep->comm);
    if (ep->d_sums) cudaFree(ep->d_sums);
    if (ep->d_all_counts) cudaFree(ep->d_all_counts);
    if (ep->h_all_counts) cudaFreeHost(ep->h_all_counts);
    if (ep->d_tables) cudaFree(ep->d_tables);
    if (ep->h_tables) cudaFreeHost(ep->h_tables);
    for (int r = 0; r < (int)ep->peer_xr.size(); ++r) {
        if (r == ep->cfg.rank) continue;
        if (ep->peer_xr[r]) cudaIpcCloseMemHandle(ep->peer_xr[r]);
        if (ep->peer_yb[r]) cudaIpcCloseMemHandle(ep->peer_yb[r]);
    }
    if (ep->yb) cudaFree(ep->yb);
    if (ep->d_seg) cudaFree(ep->d_seg);
    if (ep->h_seg) cudaFreeHost(ep->h_seg);
    if (ep->d_segp) cudaFree(ep->d_segp);
    if (ep->h_segp) cudaFreeHost(ep->h_segp);
    if (ep->xr) cudaFree(ep->xr);
    if (ep->hr) cudaFree(ep->hr);
    if (ep->yr) cudaFree(ep->yr);
    if (ep->d_ipc) cudaFree(ep->d_ipc);
    if (ep->h_ipc) cudaFreeHost(ep->h_ipc);
    if (ep->d_ptrs) cudaFree(ep->d_ptrs);
    if (ep->h_ptrs) cudaFreeHost(ep->h_ptrs);
    if (ep->d_flag) cudaFree(ep->d_flag);
    for (auto& e : ep->ev)
        if (e) cudaEventDestroy(e);
    delete ep;
}

float* ep_sums_buffer(EpState* ep) { return ep->d_sums; }

float ep_last_exchange_ms(EpState* ep) {
    if (!ep->timed) return 0.f;
    float a = 0.f, b = 0.f;
    if (cudaEventSynchronize(ep->ev[3]) != cudaSuccess) return 0.f;
    cudaEventElapsedTime(&a, ep->ev[0], ep->ev[1]);
    cudaEventElapsedTime(&b, ep->ev[2], ep->ev[3]);
    return a + b;
}

#define EP_CUDA(expr)                                                                  \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, #expr ": ", cudaGetErrorString(_e)); \
    } while (0)
#define EP_NCCL(expr)                                                                  \
    do {                                                                               \
        ncclResult_t _r = (expr);                                                      \
        if (_r != ncclSuccess) return set_err(err, errlen, MOE_ERR_NCCL, #expr ": ", g_nccl.GetErrorString(_r)); \
    } while (0)

int ep_exchange_and_run(EpState* ep, const EpCall& c, EpRunFn run, void* self, int64_t* launches, char* err,
                        size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank, per = ep->per, E = g.E;
    const ncclDataType_t row_t = g.elt == 2 ? ncclBfloat16 : ncclFloat32;
    cudaStream_t s = c.stream;

    EP_CUDA(cudaEventRecord(ep->ev[0], s));
    // 1-2. counts of every rank, to the host
    EP_NCCL(g_nccl.AllGather(c.expert_count, ep->d_all_counts, (size_t)E, ncclInt32, ep->comm, s));
    EP_CUDA(cudaMemcpyAsync(ep->h_all_counts, ep->d_all_counts, sizeof(int32_t) * W * E, cudaMemcpyDeviceToHost, s));
    EP_CUDA(cudaStreamSynchronize(s));
    const int32_t* cnt = ep->h_all_counts;  // cnt[r*E + e]

    // send layout (my rows grouped by global expert) and receive layout ([local expert][source])
    std::vector<int64_t> send_off((size_t)E + 1, 0);
    std::vector<int64_t> recv_off((size_t)per * W, 0);
    int32_t* h_off = ep->h_tables;
    int32_t* h_tp = ep->h_tables + (per + 1);
    const int64_t rows = ep_plan_layout(cnt, W, E, me, g.tile_m, send_off.data(), recv_off.data(), h_off, h_tp);
    if (rows > 0x7fffffffLL) return set_err(err, errlen, MOE_ERR_UNSUPPORTED, "more than 2^31-1 received rows");

    if (rows > ep->rows_cap) {
        const int64_t cap = rows + rows / 4 + g.tile_m;
        if (ep->xr) cudaFree(ep->xr);
        if (ep->hr) cudaFree(ep->hr);
        if (ep->yr) cudaFree(ep->yr);
        ep->xr = ep->hr = ep->yr = nullptr;
        ep->rows_cap = 0;
        EP_CUDA(cudaMalloc(&ep->xr, (size_t)cap * g.D * g.elt));
        EP_CUDA(cudaMalloc(&ep->hr, (size_t)cap * g.H * g.elt));
        EP_CUDA(cudaMalloc(&ep->yr, (size_t)cap * g.O * g.elt));
        ep->rows_cap = cap;
    }
    EP_CUDA(cudaMemcpyAsync(ep->d_tables, ep->h_tables, sizeof(int32_t) * 2 * (per + 1), cudaMemcpyHostToDevice, s));

    // 3. dispatch
    const char* xs = reinterpret_cast<const char*>(c.xs);
    char* xr = reinterpret_cast<char*>(ep->xr);
    EP_NCCL(g_nccl.GroupStart());
    for (int r = 0; r < W; ++r) {
        for (int el = 0; el < per; ++el) {
            const int e_dst = r * per + el;           // expert on rank r that my rows go to
            const int64_t n_send = cnt[(size_t)me * E + e_dst];
            const int e_mine = me * per + el;         // my expert that rank r's rows come to
            const int64_t n_recv = cnt[(size_t)r * E + e_mine];
            if (r == me) continue;
            if (n_send)
                EP_NCCL(g_nccl.Send(xs + (size_t)send_off[e_dst] * g.D * g.elt, (size_t)n_send * g.D, row_t, r,
                                    ep->comm, s));
            if (n_recv)
                EP_NCCL(g_nccl.Recv(xr + (size_t)recv_off[(size_t)el * W + r] * g.D * g.elt, (size_t)n_recv * g.D,
                                    row_t, r, ep->comm, s));
        }
    }
    EP_NCCL(g_nccl.GroupEnd());
    for (int el = 0; el < per; ++el) {
        const int e_mine = me * per + el;
        const int64_t n = cnt[(size_t)me * E + e_mine];
        if (n)
            EP_CUDA(cudaMemcpyAsync(xr + (size_t)recv_off[(size_t)el * W + me] * g.D * g.elt,
                                    xs + (size_t)send_off[e_mine] * g.D * g.elt, (size_t)n * g.D * g.elt,
                                    cudaMemcpyDeviceToDevice, s));
    }
    EP_CUDA(cudaEventRecord(ep->ev[1], s));

    // 4. local experts
    int rc = run(self, ep->xr, ep->hr, ep->yr, ep->d_tables, ep->d_tables + (per + 1), rows, per, ep->rows_cap, s);
    if (rc) return rc;

    // 5. combine: expert outputs back to the rank that owns the token
    EP_CUDA(cudaEventRecord(ep->ev[2], s));
    const char* yr = reinterpret_cast<const char*>(ep->yr);
    char* yb = reinterpret_cast<char*>(c.y_back);
    EP_NCCL(g_nccl.GroupStart());
    for (int r = 0; r < W; ++r) {
        for (int el = 0; el < per; ++el) {
            if (r == me) continue;
            const int e_mine = me * per + el;
            const int64_t n_send = cnt[(size_t)r * E + e_mine];   // rows of rank r that I computed
            const int e_dst = r * per + el;
            const int64_t n_recv = cnt[(size_t)me * E + e_dst];   // my rows that rank r computed
            if (n_send)
                EP_NCCL(g_nccl.Send(yr + (size_t)recv_off[(size_t)el * W + r] * g.O * g.elt, (size_t)n_send * g.O,
                                    row_t, r, ep->comm, s));
            if (n_recv)
                EP_NCCL(g_nccl.Recv(yb + (size_t)send_off[e_dst] * g.O * g.elt, (size_t)n_recv * g.O, row_t, r,
                                    ep->comm, s));
        }
    }
    EP_NCCL(g_nccl.GroupEnd());
    for (int el = 0; el < per; ++el) {
        const int e_mine = me * per + el;
        const int64_t n = cnt[(size_t)me * E + e_mine];
        if (n)
            EP_CUDA(cudaMemcpyAsync(yb + (size_t)send_off[e_mine] * g.O * g.elt,
                                    yr + (size_t)recv_off[(size_t)el * W + me] * g.O * g.elt, (size_t)n * g.O * g.elt,
                                    cudaMemcpyDeviceToDevice, s));
    }

    // 6. loss over all ranks' tokens
    EP_NCCL(g_nccl.AllReduce(ep->d_sums, ep->d_sums, (size_t)(E + g.E_probs + 3), ncclFloat32, ncclSum, ep->comm, s));
    ep_finish_loss_kernel<<<1, 32, 0, s>>>(ep->d_sums, E, g.E_probs, g.k_tot, g.alpha, g.z_weight, c.training,
                                           c.u_loss, c.u_entropy);
    if (cudaGetLastError() != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, "loss kernel launch failed");
    if (launches) *launches += 1;
    EP_CUDA(cudaEventRecord(ep->ev[3], s));
    ep->timed = true;
    return MOE_OK;
}

// ---- peer-memory mode ------------------------------------------------------------------------

bool ep_peer_mode(const EpState* ep) { return ep->peer_mode; }
int ep_world(const EpState* ep) { return ep->cfg.world; }

void ep_mark(EpState* ep, int i, cudaStream_t s) {
    cudaEventRecord(ep->ev[i], s);
    if (i == 3) ep->timed = true;
}

// Collective: every rank calls it with the same capacities (derived from the all-gathered counts).
// Order: drop the mappings of the peers' old buffers, allocate the new buffers, exchange their
// IPC handles (which also tells us every rank has dropped its old mappings), free the old
// buffers, map the peers' new ones.
static int ep_grow_peer_buffers(EpState* ep, int64_t cap, int64_t pairs_cap, cudaStream_t s, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank;
    for (int r = 0; r < W; ++r) {
        if (r != me) {
            if (ep->peer_xr[r]) cudaIpcCloseMemHandle(ep->peer_xr[r]);
            if (ep->peer_yb[r]) cudaIpcCloseMemHandle(ep->peer_yb[r]);
        }
        ep->peer_xr[r] = ep->peer_yb[r] = nullptr;
    }
    void *nxr = nullptr, *nhr = nullptr, *nyb = nullptr;
    EP_CUDA(cudaMalloc(&nxr, (size_t)cap * g.D * g.elt));
    EP_CUDA(cudaMalloc(&nhr, (size_t)cap * g.H * g.elt));
    EP_CUDA(cudaMalloc(&nyb, (size_t)pairs_cap * g.O * g.elt));
    cudaIpcMemHandle_t mine[2];
    EP_CUDA(cudaIpcGetMemHandle(&mine[0], nxr));
    EP_CUDA(cudaIpcGetMemHandle(&mine[1], nyb));
    const size_t hb = 2 * sizeof(cudaIpcMemHandle_t);
    EP_CUDA(cudaMemcpyAsync(ep->d_ipc + (size_t)me * hb, mine, hb, cudaMemcpyHostToDevice, s));
    EP_NCCL(g_nccl.AllGather(ep->d_ipc + (size_t)me * hb, ep->d_ipc, hb, ncclChar, ep->comm, s));
    EP_CUDA(cudaMemcpyAsync(ep->h_ipc, ep->d_ipc, hb * W, cudaMemcpyDeviceToHost, s));
    EP_CUDA(cudaStreamSynchronize(s));
    if (ep->xr) cudaFree(ep->xr);
    if (ep->hr) cudaFree(ep->hr);
    if (ep->yb) cudaFree(ep->yb);
    ep->xr = nxr;
    ep->hr = nhr;
    ep->yb = nyb;
    ep->rows_cap = cap;
    ep->pairs_cap = pairs_cap;
    for (int r = 0; r < W; ++r) {
        if (r == me) {
            ep->peer_xr[r] = nxr;
            ep->peer_yb[r] = nyb;
            continue;
        }
        cudaIpcMemHandle_t h[2];
        memcpy(h, ep->h_ipc + (size_t)r * hb, hb);
        EP_CUDA(cudaIpcOpenMemHandle(&ep->peer_xr[r], h[0], cudaIpcMemLazyEnablePeerAccess));
        EP_CUDA(cudaIpcOpenMemHandle(&ep->peer_yb[r], h[1], cudaIpcMemLazyEnablePeerAccess));
    }
    return MOE_OK;
}

int ep_prepare(EpState* ep, const int32_t* d_expert_count, cudaStream_t s, EpPlan* plan, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank, per = ep->per, E = g.E;
    EP_NCCL(g_nccl.AllGather(d_expert_count, ep->d_all_counts, (size_t)E, ncclInt32, ep->comm, s));
    EP_CUDA(cudaMemcpyAsync(ep->h_all_counts, ep->d_all_counts, sizeof(int32_t) * W * E, cudaMemcpyDeviceToHost, s));
    EP_CUDA(cudaStreamSynchronize(s));
    const int32_t* cnt = ep->h_all_counts;  // cnt[r*E + e]

    // rows every rank receives: the capacity decision must be the same on all ranks
    int64_t need = 0;
    std::vector<int64_t> expert_rows((size_t)E, 0);   // rows of expert e over all sources
    for (int e = 0; e < E; ++e)
        for (int r = 0; r < W; ++r) expert_rows[e] += cnt[(size_t)r * E + e];
    for (int r = 0; r < W; ++r) {
        int64_t rows_r = 0;
        for (int el = 0; el < per; ++el) rows_r += expert_rows[(size_t)r * per + el];
        if (rows_r > need) need = rows_r;
    }
    if (need > 0x7fffffffLL) return set_err(err, errlen, MOE_ERR_UNSUPPORTED, "more than 2^31-1 received rows");
    int64_t need_pairs = 0;                           // largest number of pairs any rank sends
    for (int r = 0; r < W; ++r) {
        int64_t pr = 0;
        for (int e = 0; e < E; ++e) pr += cnt[(size_t)r * E + e];
        if (pr > need_pairs) need_pairs = pr;
    }
    if (need > ep->rows_cap || need_pairs > ep->pairs_cap || !ep->xr) {
        const int64_t cap = need > ep->rows_cap ? need + need / 4 + g.tile_m : ep->rows_cap;
        const int64_t pcap = need_pairs > ep->pairs_cap ? need_pairs + need_pairs / 4 + 64 : ep->pairs_cap;
        const int rc = ep_grow_peer_buffers(ep, cap, pcap, s, err, errlen);
        if (rc) return rc;
    }

    // my receive layout (for the grouped GEMM)
    std::vector<int64_t> send_off((size_t)E + 1, 0), recv_off((size_t)per * W, 0);
    int32_t* h_off = ep->h_tables;
    int32_t* h_tp = ep->h_tables + (per + 1);
    const int64_t rows = ep_plan_layout(cnt, W, E, me, g.tile_m, send_off.data(), recv_off.data(), h_off, h_tp);
    int32_t* h_tp_alt = ep->h_tables + 2 * (per + 1);
    if (g.tile_m_alt > 0) {
        int32_t tiles = 0;
        for (int el = 0; el < per; ++el) {
            h_tp_alt[el] = tiles;
            tiles += (int32_t)((expert_rows[(size_t)me * per + el] + g.tile_m_alt - 1) / g.tile_m_alt);
        }
        h_tp_alt[per] = tiles;
    }
    EP_CUDA(cudaMemcpyAsync(ep->d_tables, ep->h_tables, sizeof(int32_t) * 3 * (per + 1), cudaMemcpyHostToDevice, s));

    // where my rows for expert e start inside its owner's receive buffer:
    //   (rows of the owner's earlier local experts) + (rows of expert e from lower ranks)
    for (int r = 0; r < W; ++r) {
        int64_t base = 0;
        for (int el = 0; el < per; ++el) {
            const int e = r * per + el;
            int64_t before_me = 0;
            for (int q = 0; q < me; ++q) before_me += cnt[(size_t)q * E + e];
            ep->h_ptrs[e] = reinterpret_cast<char*>(ep->peer_xr[r]) + (size_t)(base + before_me) * g.D * g.elt;
            base += expert_rows[e];
        }
    }
    EP_CUDA(cudaMemcpyAsync(ep->d_ptrs, ep->h_ptrs, sizeof(void*) * E, cudaMemcpyHostToDevice, s));
    // where the outputs of the rows I received go: segment (el, r) = rank r's pairs for my expert el,
    // stored at rank r's yb from its send offset of that expert (its pair_pos order)
    for (int r = 0; r < W; ++r) {
        int64_t send_off_r = 0;                       // rank r's send offset of expert e, e ascending
        for (int e = 0; e < me * per; ++e) send_off_r += cnt[(size_t)r * E + e];
        for (int el = 0; el < per; ++el) {
            const int e = me * per + el;
            ep->h_seg[(size_t)el * W + r] = (int32_t)recv_off[(size_t)el * W + r];
            ep->h_segp[(size_t)el * W + r] = reinterpret_cast<char*>(ep->peer_yb[r]) + (size_t)send_off_r * g.O * g.elt;
            send_off_r += cnt[(size_t)r * E + e];
        }
    }
    EP_CUDA(cudaMemcpyAsync(ep->d_seg, ep->h_seg, sizeof(int32_t) * per * W, cudaMemcpyHostToDevice, s));
    EP_CUDA(cudaMemcpyAsync(ep->d_segp, ep->h_segp, sizeof(void*) * per * W, cudaMemcpyHostToDevice, s));

    plan->rows = rows;
    plan->rows_cap = ep->rows_cap;
    plan->xr = ep->xr;
    plan->hr = ep->hr;
    plan->yb = ep->yb;
    plan->d_seg_start = ep->d_seg;
    plan->d_seg_dst = ep->d_segp;
    plan->d_local_off = ep->d_tables;
    plan->d_tile_prefix = ep->d_tables + (per + 1);
    plan->d_tile_prefix_alt = g.tile_m_alt > 0 ? ep->d_tables + 2 * (per + 1) : nullptr;
    plan->d_expert_dst = ep->d_ptrs;
    return MOE_OK;
}

int ep_sums_barrier(EpState* ep, cudaStream_t s, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    EP_NCCL(g_nccl.AllReduce(ep->d_sums, ep->d_sums, (size_t)(g.E + g.E_probs + 3), ncclFloat32, ncclSum, ep->comm, s));
    return MOE_OK;
}

int ep_barrier(EpState* ep, cudaStream_t s, char* err, size_t errlen) {
    EP_NCCL(g_nccl.AllReduce(ep->d_flag, ep->d_flag, 1, ncclInt32, ncclMax, ep->comm, s));
    return MOE_OK;
}

int ep_finish_loss(EpState* ep, int training, float* u_loss, float* u_entropy, cudaStream_t s, int64_t* launches,
                   char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    ep_finish_loss_kernel<<<1, 32, 0, s>>>(ep->d_sums, g.E, g.E_probs, g.k_tot, g.alpha, g.z_weight, training, u_loss,
                                           u_entropy);
    if (cudaGetLastError() != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, "loss kernel launch failed");
    if (launches) *launches += 1;
    return MOE_OK;
}

}  // namespace moe
