// Expert-parallel dispatch/combine between the ranks of one node (see ep.h).
//
// Peer-memory mode (default).  Every rank exports three buffers with CUDA IPC: its receive buffer
// xr, the buffer yb that collects the outputs of its own pairs, and a small control block (arrival
// flags + one record of routing statistics per rank and parity).  One forward call on every rank:
//   1. exchange kernel: this rank's record {per-expert pair counts, probability sums, lse^2 sum, T,
//      entropy sum} is stored into every peer's control block, followed by a release flag; the kernel
//      then waits (bounded) for every peer's flag                          -> records[world][...]
//   2. counts to the host (the one host synchronisation of the call): receive layout, capacity
//      decision (identical on all ranks, it only depends on the gathered counts), pointer tables
//   3. permute kernel: rows go straight into the owners' xr over NVLink
//   4. barrier kernel (flags): all rows for this rank's experts have landed
//   5. grouped GEMM pair on local memory; the GEMM 2 epilogue stores every output row into the yb
//      of the rank that owns the token
//   6. barrier kernel (flags): all outputs of this rank's pairs have landed; combine; one-block
//      kernel that finishes the Switch loss over ALL ranks' tokens from the gathered records
// NCCL is not on that path: it creates the group (non-blocking communicator, every call polled
// against a deadline) and carries the IPC handles when buffers are (re)allocated.  Every device-side
// wait is bounded by %globaltimer and reports through the handle's status word; every host-side
// wait on a collective is bounded and ends in ncclCommAbort, so a rank that stays away costs its
// peers a timeout, not a hang.
//
// MOE_B200_EP_MODE=nccl keeps the comparison path: records by ncclAllGather, rows by grouped
// ncclSend/ncclRecv into local buffers, outputs back the same way.
//
// NCCL is bound at run time with dlopen so that the library loads, and the single-GPU path works,
// without it; inside a process that already holds NCCL (for instance through torch.distributed)
// the same copy is reused.  Received rows always land in this GPU's own memory before any TMA
// load touches them.
#include "ep.h"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/moe_b200.h"
#include "common.cuh"

namespace moe {

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
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
    BIND(CommInitRankConfig, "ncclCommInitRankConfig");
    BIND(CommGetAsyncError, "ncclCommGetAsyncError");
    BIND(CommAbort, "ncclCommAbort");
    BIND(GroupStart, "ncclGroupStart");
    BIND(GroupEnd, "ncclGroupEnd");
    BIND(Send, "ncclSend");
    BIND(Recv, "ncclRecv");
    BIND(AllGather, "ncclAllGather");
    BIND(GetErrorString, "ncclGetErrorString");
#undef BIND
    g_nccl.lib = lib;
    return MOE_OK;
}

__device__ __forceinline__ unsigned long long ep_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Thread r < W: tell rank r that this rank has reached `epoch` at `slot`, then wait until rank r has
// told us the same.  Everything this rank stored before (earlier kernels of the stream, and this
// block's stores before the preceding fence + barrier) is ordered before the release store.  A wait
// that runs out records DEV_TIMEOUT_PEER and returns.
__device__ __forceinline__ void flag_exchange(int32_t* const* peer_ctl, int32_t* my_ctl, int slot, int W, int me, int epoch,
                                              unsigned long long limit_ns, int32_t* status) {
    const int r = threadIdx.x;
    if (r >= W) return;
    __threadfence_system();
    st_release_sys(peer_ctl[r] + slot * EP_MAX_WORLD + me, epoch);
    const int32_t* src = my_ctl + slot * EP_MAX_WORLD + r;
    const unsigned long long t0 = ep_timer_ns();
    unsigned spins = 0;
    while (ld_acquire_sys(src) - epoch < 0) {
        if ((++spins & 31u) == 0 && ep_timer_ns() - t0 > limit_ns) {
            if (status) atomicCAS(status, DEV_OK, DEV_TIMEOUT_PEER);
            break;
        }
    }
}

__global__ void __launch_bounds__(64) ep_barrier_kernel(int32_t* const* peer_ctl, int32_t* my_ctl, int slot, int W, int me,
                                                        int epoch, unsigned long long limit_ns, int32_t* status) {
    flag_exchange(peer_ctl, my_ctl, slot, W, me, epoch, limit_ns, status);
}

// Step 1 of a forward: copy this rank's record into slot `me` of every peer's record table (parity
// epoch & 1), flag, wait for everybody's flag.  256 threads; rec_words <= EP_MAX_REC_WORDS.
__global__ void __launch_bounds__(256) ep_exchange_records_kernel(const int32_t* my_record, int rec_words,
                                                                  int32_t* const* peer_ctl, int32_t* my_ctl, int W, int me,
                                                                  int epoch, unsigned long long limit_ns, int32_t* status) {
    const size_t rec_base = EP_CTL_FLAG_WORDS + ((size_t)(epoch & 1) * EP_MAX_WORLD + me) * EP_MAX_REC_WORDS;
    for (int r = 0; r < W; ++r) {
        int32_t* dst = peer_ctl[r] + rec_base;
        for (int i = threadIdx.x; i < rec_words; i += blockDim.x) dst[i] = my_record[i];
    }
    __threadfence_system();
    __syncthreads();
    flag_exchange(peer_ctl, my_ctl, 2, W, me, epoch, limit_ns, status);
}

// The loss over all ranks' tokens from their records: rec[r] = {int32 counts[E], float prob sums
// [E_probs], float lse^2 sum, int32 T, float entropy sum}.  Ranks are added in ascending order, so
// every rank computes the same bits.  Chunked host calls carry running totals in acc_i / acc_f:
// use_acc adds them in, store_acc writes the new totals back, emit writes loss and entropy.
__global__ void __launch_bounds__(256) ep_finish_loss_kernel(const int32_t* records, int rec_stride, int W, int E, int E_probs,
                                                             int k_tot, float alpha, float z_weight, int training, int use_acc,
                                                             int store_acc, int emit, long long* acc_i, float* acc_f,
                                                             float* u_loss, float* u_entropy) {
    __shared__ long long s_cnt[MAX_EXPERTS];
    __shared__ float s_p[MAX_EXPERTS + 2];
    __shared__ long long s_T;
    const int j = threadIdx.x;
    if (j < E) {
        long long c = use_acc ? acc_i[j] : 0;
        for (int r = 0; r < W; ++r) c += records[(size_t)r * rec_stride + j];
        s_cnt[j] = c;
        if (store_acc) acc_i[j] = c;
    }
    if (j <= E_probs + 1) {   // prob sums, lse^2 sum, entropy sum (the T word in between is an integer)
        const int w = j <= E_probs ? E + j : E + E_probs + 2;
        float v = use_acc ? acc_f[j] : 0.f;
        for (int r = 0; r < W; ++r) v += __int_as_float(records[(size_t)r * rec_stride + w]);
        s_p[j] = v;
        if (store_acc) acc_f[j] = v;
    }
    if (j == 0) {
        long long t = use_acc ? acc_i[E] : 0;
        for (int r = 0; r < W; ++r) t += records[(size_t)r * rec_stride + E + E_probs + 1];
        s_T = t;
        if (store_acc) acc_i[E] = t;
    }
    __syncthreads();
    if (!emit || j >= 32) return;
    const float Tg = (float)s_T;
    float acc = 0.f;
    if (s_T > 0) {
        const float denom = (float)((double)k_tot * (double)s_T);
        for (int i = j; i < E_probs; i += 32) acc += ((float)s_cnt[i] / denom) * (s_p[i] / Tg);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (j == 0) {
        float loss = 0.f;
        if (training && s_T > 0) {
            loss = alpha * (float)E_probs * acc;
            if (z_weight > 0.f) loss += z_weight * (s_p[E_probs] / Tg);
        }
        if (u_loss) *u_loss = loss;
        if (u_entropy) *u_entropy = s_T > 0 ? s_p[E_probs + 1] / Tg : 0.f;
    }
}

// The same from the summed statistics of the chunks of one batch (no expert parallelism): sums =
// {unused[E], prob sums[E_probs], lse^2 sum, unused, entropy sum}, integer counts and T on the side.
__global__ void chunk_finish_loss_kernel(const float* sums, const long long* counts, long long T, int E, int E_probs, int k_tot,
                                         float alpha, float z_weight, int training, float* u_loss, float* u_entropy) {
    const int lane = threadIdx.x;
    const float Tg = (float)T;
    float acc = 0.f;
    if (T > 0) {
        const float denom = (float)((double)k_tot * (double)T);
        for (int j = lane; j < E_probs; j += 32) acc += ((float)counts[j] / denom) * (sums[E + j] / Tg);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float loss = 0.f;
        if (training && T > 0) {
            loss = alpha * (float)E_probs * acc;
            if (z_weight > 0.f) loss += z_weight * (sums[E + E_probs] / Tg);
        }
        if (u_loss) *u_loss = loss;
        if (u_entropy) *u_entropy = T > 0 ? sums[E + E_probs + 2] / Tg : 0.f;
    }
}

using steady = std::chrono::steady_clock;

struct IpcRecord {
    cudaIpcMemHandle_t xr, yb, ctl;
    int32_t ok;          // 1: this rank allocated its buffers
    int32_t pad[3];
};

}  // namespace

struct EpState {
    EpConfig cfg;
    ncclComm_t comm = nullptr;
    bool dead = false;              // a collective failed or timed out: every later call is refused
    bool had_error = false;         // some call failed: tear the communicator down with abort, not destroy
    int timeout_ms = 30000;         // host-side deadline of every wait on a collective; device waits use min(this, 10 s)
    int per = 0;                    // experts per rank
    int rec_words = 0;              // 32-bit words of one rank's record
    int epoch = 0;                  // forward calls so far (the same on every rank)
    int32_t* d_record = nullptr;    // this rank's record, written by the scan kernel
    int32_t* d_gathered = nullptr;  // nccl all-gather target: [world][rec_words]
    int32_t* h_gathered = nullptr;  // pinned [world][EP_MAX_REC_WORDS]
    const int32_t* d_last_records = nullptr;   // where the current call's gathered records are on the device
    int last_stride = 0;
    long long* d_acc_i = nullptr;   // [E+1] running totals over the chunks of a host call
    float* d_acc_f = nullptr;       // [E_probs+2]
    int32_t* d_tables = nullptr;    // [3*(per+1)]: local expert_offset, tile_prefix, alternative tile_prefix
    int32_t* h_tables = nullptr;    // pinned
    void* xr = nullptr;             // received rows       [rows_cap][D]
    void* hr = nullptr;             // hidden activations  [rows_cap][H]
    void* yr = nullptr;             // nccl mode: expert outputs [rows_cap][O]
    int64_t rows_cap = 0;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t ev_sync = nullptr;
    bool timed = false;
    // peer-memory mode
    bool peer_mode = true;
    std::vector<void*> peer_xr, peer_yb, peer_ctl;   // [world] mapped buffers of every rank (own entry = local pointer)
    void* yb = nullptr;                    // [pairs_cap][O] outputs of this rank's pairs (written by the expert owners)
    int32_t* ctl = nullptr;                // control block: flags + record tables (EP_CTL_WORDS words)
    int64_t pairs_cap = 0;
    int32_t* d_seg = nullptr;              // [per*world] segment starts
    int32_t* h_seg = nullptr;              // pinned
    void** d_segp = nullptr;               // [per*world] segment destinations
    void** h_segp = nullptr;               // pinned
    unsigned char* d_ipc = nullptr;        // [world] IpcRecord staging for the handle all-gather
    unsigned char* h_ipc = nullptr;        // pinned
    void** d_ptrs = nullptr;               // [E] expert_dst
    void** h_ptrs = nullptr;               // pinned
    int32_t** d_ctl_ptrs = nullptr;        // [world] control blocks of every rank
};

namespace {

// Ends the group for this process: NCCL kernels that wait for a rank that will not come are torn down.
void ep_kill(EpState* ep) {
    if (ep->comm) {
        g_nccl.CommAbort(ep->comm);
        ep->comm = nullptr;
    }
    ep->dead = true;
}

unsigned long long device_limit_ns(const EpState* ep) {
    const int ms = ep->timeout_ms < 10000 ? ep->timeout_ms : 10000;
    return (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull;
}

// Result of a call on the non-blocking communicator: poll until the call has been processed.
int nccl_settle(EpState* ep, ncclResult_t r, const char* what, char* err, size_t errlen) {
    const auto deadline = steady::now() + std::chrono::milliseconds(ep->timeout_ms);
    while (r == ncclInProgress) {
        ncclResult_t q = ncclSuccess;
        if (g_nccl.CommGetAsyncError(ep->comm, &q) != ncclSuccess) {
            r = ncclSystemError;
            break;
        }
        r = q;
        if (r != ncclInProgress) break;
        if (steady::now() > deadline) {
            ep_kill(ep);
            if (err && errlen)
                snprintf(err, errlen, "%s did not complete within %d ms (a rank of the expert-parallel group is missing); "
                         "the communicator was aborted", what, ep->timeout_ms);
            return MOE_ERR_TIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (r != ncclSuccess) {
        const char* msg = g_nccl.GetErrorString(r);
        ep_kill(ep);
        if (err && errlen) snprintf(err, errlen, "%s: %s (the communicator was aborted)", what, msg);
        return MOE_ERR_NCCL;
    }
    return MOE_OK;
}

// Wait, against the deadline, for everything queued on `s` up to now; NCCL work is in there, so an
// asynchronous NCCL error or the deadline aborts the communicator (which ends its kernels).
int ep_stream_wait_nccl(EpState* ep, cudaStream_t s, const char* what, char* err, size_t errlen) {
    if (cudaEventRecord(ep->ev_sync, s) != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, "cudaEventRecord failed");
    const auto t0 = steady::now();
    const auto deadline = t0 + std::chrono::milliseconds(ep->timeout_ms);
    while (true) {
        const cudaError_t q = cudaEventQuery(ep->ev_sync);
        if (q == cudaSuccess) return MOE_OK;
        if (q != cudaErrorNotReady) return set_err(err, errlen, MOE_ERR_CUDA, "waiting for a collective: ", cudaGetErrorString(q));
        ncclResult_t ae = ncclSuccess;
        if (ep->comm && g_nccl.CommGetAsyncError(ep->comm, &ae) == ncclSuccess && ae != ncclSuccess && ae != ncclInProgress) {
            const char* msg = g_nccl.GetErrorString(ae);
            ep_kill(ep);
            cudaStreamSynchronize(s);
            if (err && errlen) snprintf(err, errlen, "%s: %s (the communicator was aborted)", what, msg);
            return MOE_ERR_NCCL;
        }
        const auto now = steady::now();
        if (now > deadline) {
            ep_kill(ep);
            cudaStreamSynchronize(s);   // the aborted collective's kernel ends; nothing else on the stream waits for a peer
            if (err && errlen)
                snprintf(err, errlen, "%s did not complete within %d ms (a rank of the expert-parallel group is missing); "
                         "the communicator was aborted", what, ep->timeout_ms);
            return MOE_ERR_TIMEOUT;
        }
        if (now - t0 > std::chrono::microseconds(500)) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
}

}  // namespace

int launch_finish_loss(const float* sums, const int64_t* counts, int64_t T, int E, int E_probs, int k_tot, float alpha,
                       float z_weight, int training, float* u_loss, float* u_entropy, cudaStream_t s) {
    static_assert(sizeof(long long) == sizeof(int64_t), "int64_t is long long");
    chunk_finish_loss_kernel<<<1, 32, 0, s>>>(sums, reinterpret_cast<const long long*>(counts), (long long)T, E, E_probs, k_tot,
                                              alpha, z_weight, training, u_loss, u_entropy);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// Pure host arithmetic (no CUDA, no NCCL): see ep.h.
int64_t ep_plan_layout(const int32_t* cnt, int W, int E, int me, int tile_m, int64_t* send_off, int64_t* recv_off,
                       int32_t* local_off, int32_t* tile_prefix) {
    const int per = E / W;
    for (size_t i = 0; i < (size_t)W * E; ++i)
        if (cnt[i] < 0) return MOE_ERR_INVALID;       // a count vector that cannot have come from a router
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
        if (rows > 0x7fffffffLL) return MOE_ERR_UNSUPPORTED;
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

int ep_create(EpState** out, const EpConfig& cfg, const void* id128, int timeout_ms, char* err, size_t errlen) {
    *out = nullptr;
    if (cfg.world > EP_MAX_WORLD) return set_err(err, errlen, MOE_ERR_UNSUPPORTED, "expert parallelism supports at most 32 ranks");
    int rc = load_nccl(err, errlen);
    if (rc) return rc;
    EpState* ep = new EpState();
    ep->cfg = cfg;
    ep->per = cfg.E / cfg.world;
    ep->rec_words = cfg.E + cfg.E_probs + 3;
    if (ep->rec_words > EP_MAX_REC_WORDS) {
        delete ep;
        return set_err(err, errlen, MOE_ERR_UNSUPPORTED, "too many experts for the expert-parallel record");
    }
    if (timeout_ms > 0) ep->timeout_ms = timeout_ms;
    if (cudaEventCreateWithFlags(&ep->ev_sync, cudaEventDisableTiming) != cudaSuccess) {
        delete ep;
        return set_err(err, errlen, MOE_ERR_CUDA, "cudaEventCreate failed");
    }
    // Non-blocking communicator: ncclCommInitRankConfig returns at once and the rendezvous with the
    // other ranks is polled against the deadline, so a rank that never calls moe_ep_init costs the
    // others a timeout instead of a hang.
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    ncclConfig_t ncfg = NCCL_CONFIG_INITIALIZER;
    ncfg.blocking = 0;
    const ncclResult_t r = g_nccl.CommInitRankConfig(&ep->comm, cfg.world, id, cfg.rank, &ncfg);
    if (r != ncclSuccess && r != ncclInProgress) {
        const char* msg = g_nccl.GetErrorString(r);
        ep->comm = nullptr;
        ep_destroy(ep);
        return set_err(err, errlen, MOE_ERR_NCCL, "ncclCommInitRankConfig: ", msg);
    }
    if ((rc = nccl_settle(ep, ncclInProgress, "joining the expert-parallel group (ncclCommInitRankConfig)", err, errlen))) {
        ep_destroy(ep);
        return rc;
    }
    const int W = cfg.world;
    bool ok = cudaMalloc(&ep->d_record, sizeof(int32_t) * ep->rec_words) == cudaSuccess &&
              cudaMalloc(&ep->d_gathered, sizeof(int32_t) * W * ep->rec_words) == cudaSuccess &&
              cudaMallocHost(&ep->h_gathered, sizeof(int32_t) * W * EP_MAX_REC_WORDS) == cudaSuccess &&
              cudaMalloc(&ep->d_acc_i, sizeof(long long) * (cfg.E + 1)) == cudaSuccess &&
              cudaMalloc(&ep->d_acc_f, sizeof(float) * (cfg.E_probs + 2)) == cudaSuccess &&
              cudaMalloc(&ep->d_tables, sizeof(int32_t) * 3 * (ep->per + 1)) == cudaSuccess &&
              cudaMallocHost(&ep->h_tables, sizeof(int32_t) * 3 * (ep->per + 1)) == cudaSuccess;
    for (auto& e : ep->ev) ok = ok && cudaEventCreate(&e) == cudaSuccess;
    const char* mode = getenv("MOE_B200_EP_MODE");
    ep->peer_mode = !(mode && strcmp(mode, "nccl") == 0);
    ep->peer_xr.assign(W, nullptr);
    ep->peer_yb.assign(W, nullptr);
    ep->peer_ctl.assign(W, nullptr);
    const size_t ipc_bytes = (size_t)W * sizeof(IpcRecord);
    ok = ok && cudaMalloc(&ep->d_ipc, ipc_bytes) == cudaSuccess && cudaMallocHost(&ep->h_ipc, ipc_bytes) == cudaSuccess &&
         cudaMalloc(&ep->d_ptrs, sizeof(void*) * cfg.E) == cudaSuccess &&
         cudaMallocHost(&ep->h_ptrs, sizeof(void*) * cfg.E) == cudaSuccess &&
         cudaMalloc(&ep->d_seg, sizeof(int32_t) * ep->per * W) == cudaSuccess &&
         cudaMallocHost(&ep->h_seg, sizeof(int32_t) * ep->per * W) == cudaSuccess &&
         cudaMalloc(&ep->d_segp, sizeof(void*) * ep->per * W) == cudaSuccess &&
         cudaMallocHost(&ep->h_segp, sizeof(void*) * ep->per * W) == cudaSuccess &&
         cudaMalloc(&ep->d_ctl_ptrs, sizeof(int32_t*) * W) == cudaSuccess &&
         cudaMalloc(&ep->ctl, sizeof(int32_t) * EP_CTL_WORDS) == cudaSuccess &&
         cudaMemset(ep->ctl, 0, sizeof(int32_t) * EP_CTL_WORDS) == cudaSuccess;
    if (!ok) {
        ep->had_error = true;
        ep_destroy(ep);
        return set_err(err, errlen, MOE_ERR_CUDA, "expert-parallel buffers: allocation failed");
    }
    *out = ep;
    return MOE_OK;
}

void ep_destroy(EpState* ep) {
    if (!ep) return;
    if (ep->comm) {
        // No operation of this communicator is outstanding here (every call that used it was waited
        // for), so nothing is lost by tearing it down with abort -- which, unlike a graceful
        // destroy, never waits for peers that may already be gone.
        g_nccl.CommAbort(ep->comm);
        ep->comm = nullptr;
    }
    for (int r = 0; r < (int)ep->peer_xr.size(); ++r) {
        if (r == ep->cfg.rank) continue;
        if (ep->peer_xr[r]) cudaIpcCloseMemHandle(ep->peer_xr[r]);
        if (ep->peer_yb[r]) cudaIpcCloseMemHandle(ep->peer_yb[r]);
        if (ep->peer_ctl[r]) cudaIpcCloseMemHandle(ep->peer_ctl[r]);
    }
    void* dev[] = {ep->d_record, ep->d_gathered, ep->d_acc_i, ep->d_acc_f, ep->d_tables, ep->yb, ep->ctl, ep->d_seg, ep->d_segp,
                   ep->xr, ep->hr, ep->yr, ep->d_ipc, ep->d_ptrs, ep->d_ctl_ptrs};
    for (void* p : dev)
        if (p) cudaFree(p);
    void* host[] = {ep->h_gathered, ep->h_tables, ep->h_seg, ep->h_segp, ep->h_ipc, ep->h_ptrs};
    for (void* p : host)
        if (p) cudaFreeHost(p);
    for (auto& e : ep->ev)
        if (e) cudaEventDestroy(e);
    if (ep->ev_sync) cudaEventDestroy(ep->ev_sync);
    delete ep;
}

int32_t* ep_record_buffer(EpState* ep) { return ep->d_record; }

int ep_set_timeout_ms(EpState* ep, int ms) {
    if (ms < 1) return MOE_ERR_INVALID;
    ep->timeout_ms = ms;
    return MOE_OK;
}

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
        if (_e != cudaSuccess) {                                                       \
            ep->had_error = true;                                                      \
            return set_err(err, errlen, MOE_ERR_CUDA, #expr ": ", cudaGetErrorString(_e)); \
        }                                                                              \
    } while (0)
// a call on the non-blocking communicator: settled before anything that depends on it is queued
#define EP_NCCL(expr)                                                                  \
    do {                                                                               \
        ncclResult_t _r = (expr);                                                      \
        if (_r != ncclSuccess) {                                                       \
            const int _rc = nccl_settle(ep, _r, #expr, err, errlen);                   \
            if (_rc) return _rc;                                                       \
        }                                                                              \
    } while (0)
// a call between ncclGroupStart and ncclGroupEnd: it is only queued; ncclGroupEnd is the call to settle
#define EP_NCCL_GROUPED(expr)                                                          \
    do {                                                                               \
        ncclResult_t _r = (expr);                                                      \
        if (_r != ncclSuccess && _r != ncclInProgress) {                               \
            const char* _m = g_nccl.GetErrorString(_r);                                \
            ep_kill(ep);                                                               \
            return set_err(err, errlen, MOE_ERR_NCCL, #expr ": ", _m);                 \
        }                                                                              \
    } while (0)

static int ep_refuse_if_dead(EpState* ep, char* err, size_t errlen) {
    if (!ep->dead) return MOE_OK;
    return set_err(err, errlen, MOE_ERR_STATE,
                   "the expert-parallel group of this handle is unusable after an earlier failure or timeout; create a new one");
}

// Every rank's record of this call, on the host and on the device.  nccl mode: one ncclAllGather.
// peer mode: the exchange kernel (own stores + flags).  The wait is bounded in both.
static int ep_gather_records(EpState* ep, cudaStream_t s, int64_t T_local, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world;
    ++ep->epoch;
    if (ep->peer_mode && ep->peer_ctl[g.rank]) {
        ep_exchange_records_kernel<<<1, 256, 0, s>>>(ep->d_record, ep->rec_words, ep->d_ctl_ptrs, ep->ctl, W, g.rank, ep->epoch,
                                                     device_limit_ns(ep), g.status);
        EP_CUDA(cudaGetLastError());
        const int32_t* tab = ep->ctl + EP_CTL_FLAG_WORDS + (size_t)(ep->epoch & 1) * EP_MAX_WORLD * EP_MAX_REC_WORDS;
        EP_CUDA(cudaMemcpyAsync(ep->h_gathered, tab, sizeof(int32_t) * W * EP_MAX_REC_WORDS, cudaMemcpyDeviceToHost, s));
        EP_CUDA(cudaStreamSynchronize(s));     // bounded: the kernel's own wait gives up after device_limit_ns
        int32_t st = 0;
        EP_CUDA(cudaMemcpy(&st, g.status, sizeof(st), cudaMemcpyDeviceToHost));
        if (st == DEV_TIMEOUT_PEER) {
            ep->dead = true;
            if (err && errlen)
                snprintf(err, errlen, "a rank of the expert-parallel group did not arrive within %llu ms (routing counts or a "
                         "barrier of the previous call)", device_limit_ns(ep) / 1000000ull);
            return MOE_ERR_TIMEOUT;
        }
        ep->d_last_records = tab;
        ep->last_stride = EP_MAX_REC_WORDS;
    } else {
        // (also the very first peer-mode call, before any control block has been exchanged)
        EP_NCCL(g_nccl.AllGather(ep->d_record, ep->d_gathered, (size_t)ep->rec_words, ncclInt32, ep->comm, s));
        EP_CUDA(cudaMemcpy2DAsync(ep->h_gathered, sizeof(int32_t) * EP_MAX_REC_WORDS, ep->d_gathered,
                                  sizeof(int32_t) * ep->rec_words, sizeof(int32_t) * ep->rec_words, W, cudaMemcpyDeviceToHost, s));
        const int rc = ep_stream_wait_nccl(ep, s, "the all-gather of the routing counts", err, errlen);
        if (rc) return rc;
        ep->d_last_records = ep->d_gathered;
        ep->last_stride = ep->rec_words;
    }
    // sanity of what arrived: this rank's own row must be what its router produced
    const int32_t* mine = ep->h_gathered + (size_t)g.rank * EP_MAX_REC_WORDS;
    int64_t pairs = 0;
    for (int e = 0; e < g.E; ++e) pairs += mine[e];
    if (mine[g.E + g.E_probs + 1] != (int32_t)T_local || pairs != T_local * g.k_tot) {
        ep->dead = true;
        return set_err(err, errlen, MOE_ERR_NCCL, "the gathered routing counts do not match this rank's own (corrupted exchange)");
    }
    return MOE_OK;
}

// counts of rank r, expert e in the gathered host table
static inline int32_t cnt_at(const EpState* ep, int r, int e) { return ep->h_gathered[(size_t)r * EP_MAX_REC_WORDS + e]; }

int ep_exchange_and_run(EpState* ep, const EpCall& c, EpRunFn run, void* self, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank, per = ep->per, E = g.E;
    const ncclDataType_t row_t = g.elt == 2 ? ncclBfloat16 : ncclFloat32;
    cudaStream_t s = c.stream;
    int rc = ep_refuse_if_dead(ep, err, errlen);
    if (rc) return rc;

    EP_CUDA(cudaEventRecord(ep->ev[0], s));
    // 1-2. records of every rank, counts to the host
    if ((rc = ep_gather_records(ep, s, c.T, err, errlen))) return rc;
    std::vector<int32_t> cnt((size_t)W * E);
    for (int r = 0; r < W; ++r)
        for (int e = 0; e < E; ++e) cnt[(size_t)r * E + e] = cnt_at(ep, r, e);

    // send layout (my rows grouped by global expert) and receive layout ([local expert][source])
    std::vector<int64_t> send_off((size_t)E + 1, 0);
    std::vector<int64_t> recv_off((size_t)per * W, 0);
    int32_t* h_off = ep->h_tables;
    int32_t* h_tp = ep->h_tables + (per + 1);
    const int64_t rows = ep_plan_layout(cnt.data(), W, E, me, g.tile_m, send_off.data(), recv_off.data(), h_off, h_tp);
    if (rows < 0) {
        ep->dead = true;
        return set_err(err, errlen, (int)rows, "the gathered routing counts are not a valid layout");
    }
    // capacity: the largest number of rows any rank receives, so that every rank grows in the same call
    int64_t need = 0;
    for (int r = 0; r < W; ++r) {
        int64_t rows_r = 0;
        for (int el = 0; el < per; ++el)
            for (int q = 0; q < W; ++q) rows_r += cnt[(size_t)q * E + r * per + el];
        if (rows_r > need) need = rows_r;
    }
    if (need > ep->rows_cap || !ep->xr) {
        const int64_t cap = need + need / 4 + g.tile_m;
        if (ep->xr) cudaFree(ep->xr);
        if (ep->hr) cudaFree(ep->hr);
        if (ep->yr) cudaFree(ep->yr);
        ep->xr = ep->hr = ep->yr = nullptr;
        ep->rows_cap = 0;
        const bool ok = cudaMalloc(&ep->xr, (size_t)cap * g.D * g.elt) == cudaSuccess &&
                        cudaMalloc(&ep->hr, (size_t)cap * g.H * g.elt) == cudaSuccess &&
                        cudaMalloc(&ep->yr, (size_t)cap * g.O * g.elt) == cudaSuccess;
        if (!ok) cudaGetLastError();
        // every rank learns whether every rank got its memory BEFORE any row is sent: a rank that failed
        // still joins this exchange, so nobody is left waiting in the grouped send/recv below
        int32_t flag = ok ? 1 : 0;
        EP_CUDA(cudaMemcpyAsync(ep->d_ipc + (size_t)me * sizeof(int32_t), &flag, sizeof(flag), cudaMemcpyHostToDevice, s));
        EP_NCCL(g_nccl.AllGather(ep->d_ipc + (size_t)me * sizeof(int32_t), ep->d_ipc, 1, ncclInt32, ep->comm, s));
        EP_CUDA(cudaMemcpyAsync(ep->h_ipc, ep->d_ipc, sizeof(int32_t) * W, cudaMemcpyDeviceToHost, s));
        if ((rc = ep_stream_wait_nccl(ep, s, "the exchange of allocation results", err, errlen))) return rc;
        for (int r = 0; r < W; ++r)
            if (reinterpret_cast<int32_t*>(ep->h_ipc)[r] != 1) {
                ep->dead = true;
                ep->had_error = true;
                if (err && errlen) snprintf(err, errlen, "rank %d could not allocate its receive buffers (%lld rows)", r, (long long)cap);
                return MOE_ERR_CUDA;
            }
        ep->rows_cap = cap;
    }
    EP_CUDA(cudaMemcpyAsync(ep->d_tables, ep->h_tables, sizeof(int32_t) * 2 * (per + 1), cudaMemcpyHostToDevice, s));

    // 3. dispatch
    const char* xs = reinterpret_cast<const char*>(c.xs);
    char* xr = reinterpret_cast<char*>(ep->xr);
    EP_NCCL_GROUPED(g_nccl.GroupStart());
    for (int r = 0; r < W; ++r) {
        for (int el = 0; el < per; ++el) {
            const int e_dst = r * per + el;           // expert on rank r that my rows go to
            const int64_t n_send = cnt[(size_t)me * E + e_dst];
            const int e_mine = me * per + el;         // my expert that rank r's rows come to
            const int64_t n_recv = cnt[(size_t)r * E + e_mine];
            if (r == me) continue;
            if (n_send)
                EP_NCCL_GROUPED(g_nccl.Send(xs + (size_t)send_off[e_dst] * g.D * g.elt, (size_t)n_send * g.D, row_t, r,
                                            ep->comm, s));
            if (n_recv)
                EP_NCCL_GROUPED(g_nccl.Recv(xr + (size_t)recv_off[(size_t)el * W + r] * g.D * g.elt, (size_t)n_recv * g.D,
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
    rc = run(self, ep->xr, ep->hr, ep->yr, ep->d_tables, ep->d_tables + (per + 1), rows, per, ep->rows_cap, s);
    if (rc) return rc;

    // 5. combine: expert outputs back to the rank that owns the token
    EP_CUDA(cudaEventRecord(ep->ev[2], s));
    const char* yr = reinterpret_cast<const char*>(ep->yr);
    char* yb = reinterpret_cast<char*>(c.y_back);
    EP_NCCL_GROUPED(g_nccl.GroupStart());
    for (int r = 0; r < W; ++r) {
        for (int el = 0; el < per; ++el) {
            if (r == me) continue;
            const int e_mine = me * per + el;
            const int64_t n_send = cnt[(size_t)r * E + e_mine];   // rows of rank r that I computed
            const int e_dst = r * per + el;
            const int64_t n_recv = cnt[(size_t)me * E + e_dst];   // my rows that rank r computed
            if (n_send)
                EP_NCCL_GROUPED(g_nccl.Send(yr + (size_t)recv_off[(size_t)el * W + r] * g.O * g.elt, (size_t)n_send * g.O,
                                            row_t, r, ep->comm, s));
            if (n_recv)
                EP_NCCL_GROUPED(g_nccl.Recv(yb + (size_t)send_off[e_dst] * g.O * g.elt, (size_t)n_recv * g.O, row_t, r,
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

// Collective: every rank calls it in the same forward with the same capacities (they derive from
// the gathered counts).  Order: drop the mappings of the peers' old buffers, allocate the new
// buffers, exchange their IPC handles together with "my allocation succeeded" (which also tells
// us every rank has dropped its old mappings), free the old buffers, map the peers' new ones.  A
// rank whose allocation fails still takes part in the exchange, so that all ranks leave with the
// same error instead of the others waiting for it.
static int ep_grow_peer_buffers(EpState* ep, int64_t cap, int64_t pairs_cap, cudaStream_t s, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank;
    for (int r = 0; r < W; ++r) {
        if (r != me) {
            if (ep->peer_xr[r]) cudaIpcCloseMemHandle(ep->peer_xr[r]);
            if (ep->peer_yb[r]) cudaIpcCloseMemHandle(ep->peer_yb[r]);
            if (ep->peer_ctl[r]) cudaIpcCloseMemHandle(ep->peer_ctl[r]);
        }
        ep->peer_xr[r] = ep->peer_yb[r] = ep->peer_ctl[r] = nullptr;
    }
    void *nxr = nullptr, *nhr = nullptr, *nyb = nullptr;
    IpcRecord mine;
    memset(&mine, 0, sizeof(mine));
    bool ok = cudaMalloc(&nxr, (size_t)cap * g.D * g.elt) == cudaSuccess && cudaMalloc(&nhr, (size_t)cap * g.H * g.elt) == cudaSuccess &&
              cudaMalloc(&nyb, (size_t)pairs_cap * g.O * g.elt) == cudaSuccess;
    ok = ok && cudaIpcGetMemHandle(&mine.xr, nxr) == cudaSuccess && cudaIpcGetMemHandle(&mine.yb, nyb) == cudaSuccess &&
         cudaIpcGetMemHandle(&mine.ctl, ep->ctl) == cudaSuccess;
    if (!ok) cudaGetLastError();   // the failure travels in the record
    mine.ok = ok ? 1 : 0;
    auto drop_new = [&]() {
        if (nxr) cudaFree(nxr);
        if (nhr) cudaFree(nhr);
        if (nyb) cudaFree(nyb);
    };
    const size_t hb = sizeof(IpcRecord);
    int rc = MOE_OK;
    do {
        if (cudaMemcpyAsync(ep->d_ipc + (size_t)me * hb, &mine, hb, cudaMemcpyHostToDevice, s) != cudaSuccess) {
            rc = set_err(err, errlen, MOE_ERR_CUDA, "staging the IPC handles failed");
            break;
        }
        ncclResult_t r = g_nccl.AllGather(ep->d_ipc + (size_t)me * hb, ep->d_ipc, hb, ncclChar, ep->comm, s);
        if (r != ncclSuccess && (rc = nccl_settle(ep, r, "ncclAllGather of the IPC handles", err, errlen))) break;
        if (cudaMemcpyAsync(ep->h_ipc, ep->d_ipc, hb * W, cudaMemcpyDeviceToHost, s) != cudaSuccess) {
            rc = set_err(err, errlen, MOE_ERR_CUDA, "reading the IPC handles back failed");
            break;
        }
        rc = ep_stream_wait_nccl(ep, s, "the exchange of the receive buffers' IPC handles", err, errlen);
    } while (false);
    if (rc) {
        drop_new();
        ep->had_error = true;
        ep->dead = true;
        return rc;
    }
    const IpcRecord* all = reinterpret_cast<const IpcRecord*>(ep->h_ipc);
    for (int r = 0; r < W; ++r)
        if (all[r].ok != 1) {
            drop_new();
            ep->dead = true;
            ep->had_error = true;
            if (err && errlen)
                snprintf(err, errlen, "rank %d could not allocate its expert-parallel buffers (%lld rows, %lld pairs)", r,
                         (long long)cap, (long long)pairs_cap);
            return MOE_ERR_CUDA;
        }
    if (ep->xr) cudaFree(ep->xr);
    if (ep->hr) cudaFree(ep->hr);
    if (ep->yb) cudaFree(ep->yb);
    ep->xr = nxr;
    ep->hr = nhr;
    ep->yb = nyb;
    ep->rows_cap = cap;
    ep->pairs_cap = pairs_cap;
    std::vector<int32_t*> ctl_ptrs(W, nullptr);
    for (int r = 0; r < W; ++r) {
        if (r == me) {
            ep->peer_xr[r] = nxr;
            ep->peer_yb[r] = nyb;
            ep->peer_ctl[r] = ep->ctl;
        } else {
            EP_CUDA(cudaIpcOpenMemHandle(&ep->peer_xr[r], all[r].xr, cudaIpcMemLazyEnablePeerAccess));
            EP_CUDA(cudaIpcOpenMemHandle(&ep->peer_yb[r], all[r].yb, cudaIpcMemLazyEnablePeerAccess));
            EP_CUDA(cudaIpcOpenMemHandle(&ep->peer_ctl[r], all[r].ctl, cudaIpcMemLazyEnablePeerAccess));
        }
        ctl_ptrs[r] = reinterpret_cast<int32_t*>(ep->peer_ctl[r]);
    }
    EP_CUDA(cudaMemcpy(ep->d_ctl_ptrs, ctl_ptrs.data(), sizeof(int32_t*) * W, cudaMemcpyHostToDevice));
    return MOE_OK;
}

int ep_prepare(EpState* ep, int64_t T_local, cudaStream_t s, EpPlan* plan, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    const int W = g.world, me = g.rank, per = ep->per, E = g.E;
    int rc = ep_refuse_if_dead(ep, err, errlen);
    if (rc) return rc;
    if ((rc = ep_gather_records(ep, s, T_local, err, errlen))) return rc;
    std::vector<int32_t> cntv((size_t)W * E);
    for (int r = 0; r < W; ++r)
        for (int e = 0; e < E; ++e) cntv[(size_t)r * E + e] = cnt_at(ep, r, e);
    const int32_t* cnt = cntv.data();  // cnt[r*E + e]

    // rows every rank receives: the capacity decision must be the same on all ranks
    int64_t need = 0;
    std::vector<int64_t> expert_rows((size_t)E, 0);   // rows of expert e over all sources
    for (int e = 0; e < E; ++e)
        for (int r = 0; r < W; ++r) {
            if (cnt[(size_t)r * E + e] < 0) {
                ep->dead = true;
                return set_err(err, errlen, MOE_ERR_NCCL, "a negative pair count arrived (corrupted exchange)");
            }
            expert_rows[e] += cnt[(size_t)r * E + e];
        }
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
        rc = ep_grow_peer_buffers(ep, cap, pcap, s, err, errlen);
        if (rc) return rc;
    }

    // my receive layout (for the grouped GEMM)
    std::vector<int64_t> send_off((size_t)E + 1, 0), recv_off((size_t)per * W, 0);
    int32_t* h_off = ep->h_tables;
    int32_t* h_tp = ep->h_tables + (per + 1);
    const int64_t rows = ep_plan_layout(cnt, W, E, me, g.tile_m, send_off.data(), recv_off.data(), h_off, h_tp);
    if (rows < 0) return set_err(err, errlen, (int)rows, "the gathered routing counts are not a valid layout");
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

int ep_barrier(EpState* ep, int slot, cudaStream_t s, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    ep_barrier_kernel<<<1, 64, 0, s>>>(ep->d_ctl_ptrs, ep->ctl, slot, g.world, g.rank, ep->epoch, device_limit_ns(ep), g.status);
    if (cudaGetLastError() != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, "barrier kernel launch failed");
    return MOE_OK;
}

int ep_finish_loss(EpState* ep, int training, int chunk_mode, float* u_loss, float* u_entropy, cudaStream_t s,
                   int64_t* launches, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    // chunk_mode: 0 = a whole batch; 1 = first chunk, 2 = middle chunk, 3 = last chunk of a host call
    const int use_acc = chunk_mode >= 2, store_acc = chunk_mode == 1 || chunk_mode == 2, emit = chunk_mode == 0 || chunk_mode == 3;
    ep_finish_loss_kernel<<<1, 256, 0, s>>>(ep->d_last_records, ep->last_stride, g.world, g.E, g.E_probs, g.k_tot, g.alpha,
                                            g.z_weight, training, use_acc, store_acc, emit, ep->d_acc_i, ep->d_acc_f, u_loss,
                                            u_entropy);
    if (cudaGetLastError() != cudaSuccess) return set_err(err, errlen, MOE_ERR_CUDA, "loss kernel launch failed");
    if (launches) *launches += 1;
    return MOE_OK;
}

// Largest T over the ranks (a host value, the same on every rank): lets all ranks of a host call
// decide together how to cut their batches.  One small all-gather, bounded like every collective.
int ep_max_tokens(EpState* ep, int64_t T_local, cudaStream_t s, int64_t* T_max, char* err, size_t errlen) {
    const EpConfig& g = ep->cfg;
    int rc = ep_refuse_if_dead(ep, err, errlen);
    if (rc) return rc;
    long long mine = T_local;
    static_assert(sizeof(IpcRecord) >= sizeof(long long), "staging slot");
    EP_CUDA(cudaMemcpyAsync(ep->d_ipc + (size_t)g.rank * sizeof(long long), &mine, sizeof(mine), cudaMemcpyHostToDevice, s));
    EP_NCCL(g_nccl.AllGather(ep->d_ipc + (size_t)g.rank * sizeof(long long), ep->d_ipc, sizeof(long long), ncclChar, ep->comm, s));
    EP_CUDA(cudaMemcpyAsync(ep->h_ipc, ep->d_ipc, sizeof(long long) * g.world, cudaMemcpyDeviceToHost, s));
    if ((rc = ep_stream_wait_nccl(ep, s, "the all-gather of the batch sizes", err, errlen))) return rc;
    long long mx = 0;
    for (int r = 0; r < g.world; ++r) {
        long long v;
        memcpy(&v, ep->h_ipc + (size_t)r * sizeof(long long), sizeof(v));
        if (v > mx) mx = v;
    }
    *T_max = mx;
    return MOE_OK;
}

}  // namespace moe
