// Tensor-parallel SwiGLU FFN over the GPUs of one node, driven by one host thread: the lifecycle a host without a
// process-per-GPU launcher binds (rlxq_tp_create / rlxq_tp_ffn_load / rlxq_tp_ffn_run / rlxq_tp_destroy).
//
// The reference has nothing to compare with: its CUDA context is a process-wide singleton on device 0
// (rlx-cuda/src/device.rs:44-60) and its collectives run on the host (rlx-driver/src/collective.rs:79-128), whose
// summation order (rank 0, 1, ...) the decode-sized all-reduce here keeps.  Every device gets a stream, its shards
// (gate / up rows stacked, the k-slice of down), scratch sized for the largest batch seen so far, and a buffer the
// other devices read directly (peer access inside one process needs no IPC handle).  A step is, per device:
// x host -> device, rlxq_tp_ffn_partial, then the sum of the partials -- rlxq_tp_allreduce_sum for up to 64 K values,
// NCCL (loaded at run time, one communicator per device from ncclCommInitAll) for prefill-sized partials -- and the
// result of device 0 back to the host.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <new>
#include <vector>

#include "../../../include/rlxq_tp.h"
#include "../common.cuh"
#include "../kernels.h"

namespace rlxq {

constexpr uint32_t kTpPeerElems = 1u << 16;       // partials up to this many values go through peer memory

struct NcclApi {
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    void* handle = nullptr;
    bool load() {
        if (handle) return true;
        handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!handle) return false;
        CommInitAll = reinterpret_cast<decltype(CommInitAll)>(dlsym(handle, "ncclCommInitAll"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(dlsym(handle, "ncclCommDestroy"));
        AllReduce = reinterpret_cast<decltype(AllReduce)>(dlsym(handle, "ncclAllReduce"));
        GroupStart = reinterpret_cast<decltype(GroupStart)>(dlsym(handle, "ncclGroupStart"));
        GroupEnd = reinterpret_cast<decltype(GroupEnd)>(dlsym(handle, "ncclGroupEnd"));
        GetErrorString = reinterpret_cast<decltype(GetErrorString)>(dlsym(handle, "ncclGetErrorString"));
        return CommInitAll && CommDestroy && AllReduce && GroupStart && GroupEnd && GetErrorString;
    }
};

struct TpRank {
    int dev = 0;
    cudaStream_t stream = nullptr;
    void* comm_buf = nullptr;             // rlxq_tp_comm_alloc: header + two parities of one slot per rank, written by the peers
    uint8_t* gate_up = nullptr;
    uint8_t* down = nullptr;
    uint8_t* x = nullptr;                 // [m, d_model] staging for the activations
    float* y = nullptr;                   // [m, d_model] partial, then the sum
    uint8_t* ws = nullptr;
    size_t x_bytes = 0, y_bytes = 0, ws_bytes = 0;
    ncclComm_t nccl = nullptr;
};

}  // namespace rlxq

using namespace rlxq;

struct rlxq_tp {
    std::vector<TpRank> ranks;
    uint32_t scheme = 0, d_model = 0, d_ffn = 0;
    bool loaded = false, peer_ok = false;
    NcclApi nccl;
    bool nccl_ready = false;
};

#define RLXQ_NCCL_TRY(t, expr)                                                                     \
    do {                                                                                           \
        ncclResult_t r__ = (expr);                                                                 \
        if (r__ != ncclSuccess) return ::rlxq::fail(RLXQ_E_NCCL, "%s: %s", #expr, (t)->nccl.GetErrorString(r__)); \
    } while (0)

static int tp_free_rank(TpRank& r) {
    cudaSetDevice(r.dev);
    if (r.stream) cudaStreamSynchronize(r.stream);
    for (void* p : {(void*)r.gate_up, (void*)r.down, (void*)r.x, (void*)r.y, (void*)r.ws})
        if (p) cudaFree(p);
    if (r.comm_buf) rlxq_tp_comm_free(r.comm_buf);
    if (r.stream) cudaStreamDestroy(r.stream);
    r = TpRank{};
    return RLXQ_OK;
}

extern "C" int rlxq_tp_destroy(rlxq_tp* t) {
    if (!t) return RLXQ_OK;
    for (TpRank& r : t->ranks) {
        if (r.nccl && t->nccl.CommDestroy) { cudaSetDevice(r.dev); t->nccl.CommDestroy(r.nccl); r.nccl = nullptr; }
        tp_free_rank(r);
    }
    delete t;
    return RLXQ_OK;
}

extern "C" int rlxq_tp_create(int ndev, const int* devs, rlxq_tp** out) {
    if (!out) return fail(RLXQ_E_NULL, "out is null");
    *out = nullptr;
    if (ndev < 1 || ndev > 8) return fail(RLXQ_E_ARG, "ndev=%d must be in [1, 8]", ndev);
    int have = 0;
    if (cudaGetDeviceCount(&have) != cudaSuccess || have <= 0) {
        (void)cudaGetLastError();
        return fail(RLXQ_E_CUDA, "no CUDA device available");
    }
    rlxq_tp* t = new (std::nothrow) rlxq_tp();
    if (!t) return fail(RLXQ_E_CUDA, "out of host memory");
    t->ranks.resize(ndev);
    for (int i = 0; i < ndev; ++i) {
        const int d = devs ? devs[i] : i;
        if (d < 0 || d >= have) { rlxq_tp_destroy(t); return fail(RLXQ_E_ARG, "device %d out of range (%d devices)", d, have); }
        for (int j = 0; j < i; ++j)
            if (t->ranks[j].dev == d) { rlxq_tp_destroy(t); return fail(RLXQ_E_ARG, "device %d listed twice", d); }
        t->ranks[i].dev = d;
    }
    int rc = RLXQ_OK;
    auto bail = [&](int code) { rlxq_tp_destroy(t); return code; };
    // every device can read every other one's buffers; without that the small all-reduce goes through NCCL too
    t->peer_ok = ndev > 1;
    for (int i = 0; i < ndev; ++i) {
        TpRank& r = t->ranks[i];
        if (cudaSetDevice(r.dev) != cudaSuccess) return bail(fail(RLXQ_E_CUDA, "cudaSetDevice(%d) failed", r.dev));
        rc = rlxq_init_device();
        if (rc) return bail(rc);
        if (cudaStreamCreateWithFlags(&r.stream, cudaStreamNonBlocking) != cudaSuccess) return bail(fail(RLXQ_E_CUDA, "stream creation failed on device %d", r.dev));
        for (int j = 0; j < ndev; ++j) {
            if (j == i) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, r.dev, t->ranks[j].dev) != cudaSuccess || !can) { t->peer_ok = false; continue; }
            const cudaError_t e = cudaDeviceEnablePeerAccess(t->ranks[j].dev, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
            else if (e != cudaSuccess) { (void)cudaGetLastError(); t->peer_ok = false; }
        }
        if (ndev > 1) {
            rc = rlxq_tp_comm_alloc(kTpPeerElems, &r.comm_buf);
            if (rc) return bail(rc);
        }
    }
    *out = t;
    return RLXQ_OK;
}

extern "C" int rlxq_tp_world(const rlxq_tp* t) { return t ? (int)t->ranks.size() : 0; }

extern "C" int rlxq_tp_ffn_load(rlxq_tp* t, uint32_t scheme, const void* gate, const void* up, const void* down,
                                uint32_t d_model, uint32_t d_ffn) {
    if (!t) return fail(RLXQ_E_NULL, "handle is null");
    if (!gate || !up || !down) return fail(RLXQ_E_NULL, "null weight buffer");
    const uint32_t world = (uint32_t)t->ranks.size();
    std::vector<uint8_t> slice;
    for (uint32_t i = 0; i < world; ++i) {
        TpRank& r = t->ranks[i];
        rlxq_tp_shard sh;
        int rc = rlxq_tp_shard_plan(scheme, d_model, d_ffn, world, i, &sh);
        if (rc) return rc;
        RLXQ_CUDA_TRY(cudaSetDevice(r.dev));
        RLXQ_CUDA_TRY(cudaStreamSynchronize(r.stream));
        if (r.gate_up) { cudaFree(r.gate_up); r.gate_up = nullptr; }
        if (r.down) { cudaFree(r.down); r.down = nullptr; }
        RLXQ_CUDA_TRY(cudaMalloc((void**)&r.gate_up, 2 * sh.gate_up_bytes));
        RLXQ_CUDA_TRY(cudaMalloc((void**)&r.down, sh.down_bytes));
        // column-parallel gate and up: the rank's rows are one contiguous byte range of each; stacked gate first
        RLXQ_CUDA_TRY(cudaMemcpy(r.gate_up, static_cast<const uint8_t*>(gate) + sh.gate_up_byte_offset, sh.gate_up_bytes, cudaMemcpyHostToDevice));
        RLXQ_CUDA_TRY(cudaMemcpy(r.gate_up + sh.gate_up_bytes, static_cast<const uint8_t*>(up) + sh.gate_up_byte_offset, sh.gate_up_bytes, cudaMemcpyHostToDevice));
        // row-parallel down: the rank's k-slice of every row, gathered on the host
        slice.resize(sh.down_bytes);
        rc = rlxq_tp_slice_k_host(scheme, down, d_model, d_ffn, sh.ffn_begin, sh.ffn_local, slice.data());
        if (rc) return rc;
        RLXQ_CUDA_TRY(cudaMemcpy(r.down, slice.data(), sh.down_bytes, cudaMemcpyHostToDevice));
    }
    t->scheme = scheme; t->d_model = d_model; t->d_ffn = d_ffn; t->loaded = true;
    return RLXQ_OK;
}

// Buffers for a batch of m rows, grown when a larger batch arrives (allocation: not for use under stream capture).
static int tp_reserve(rlxq_tp* t, uint32_t m, uint32_t x_dtype) {
    const uint32_t world = (uint32_t)t->ranks.size();
    const size_t xb = (size_t)m * t->d_model * (x_dtype == RLXQ_BF16 ? 2 : 4), yb = (size_t)m * t->d_model * 4;
    size_t need = 0;
    int rc = rlxq_tp_ffn_workspace_bytes(t->scheme, t->scheme, m, t->d_model, t->d_ffn / world, x_dtype, &need);
    if (rc) return rc;
    need += 256;
    for (TpRank& r : t->ranks) {
        RLXQ_CUDA_TRY(cudaSetDevice(r.dev));
        if (r.x_bytes < xb) { if (r.x) cudaFree(r.x); r.x = nullptr; RLXQ_CUDA_TRY(cudaMalloc((void**)&r.x, xb)); r.x_bytes = xb; }
        if (r.y_bytes < yb) { if (r.y) cudaFree(r.y); r.y = nullptr; RLXQ_CUDA_TRY(cudaMalloc((void**)&r.y, yb)); r.y_bytes = yb; }
        if (r.ws_bytes < need) { if (r.ws) cudaFree(r.ws); r.ws = nullptr; RLXQ_CUDA_TRY(cudaMalloc((void**)&r.ws, need)); r.ws_bytes = need; }
    }
    return RLXQ_OK;
}

static int tp_nccl_init(rlxq_tp* t) {
    if (t->nccl_ready) return RLXQ_OK;
    if (!t->nccl.load()) return fail(RLXQ_E_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror() ? dlerror() : "missing symbol");
    std::vector<int> devs;
    std::vector<ncclComm_t> comms(t->ranks.size());
    for (const TpRank& r : t->ranks) devs.push_back(r.dev);
    RLXQ_NCCL_TRY(t, t->nccl.CommInitAll(comms.data(), (int)devs.size(), devs.data()));
    for (size_t i = 0; i < comms.size(); ++i) t->ranks[i].nccl = comms[i];
    t->nccl_ready = true;
    return RLXQ_OK;
}

extern "C" int rlxq_tp_ffn_run(rlxq_tp* t, const void* x_host, uint32_t x_dtype, uint32_t m, float* y_host) {
    if (!t) return fail(RLXQ_E_NULL, "handle is null");
    if (!t->loaded) return fail(RLXQ_E_ARG, "rlxq_tp_ffn_run before rlxq_tp_ffn_load");
    if (x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (m == 0) return RLXQ_OK;
    if (!x_host || !y_host) return fail(RLXQ_E_NULL, "null buffer");
    const uint32_t world = (uint32_t)t->ranks.size(), f = t->d_ffn / world;
    const uint64_t elems64 = (uint64_t)m * t->d_model;
    if (elems64 > 0x7FFFFFFFull) return fail(RLXQ_E_LIMIT, "batch too large");
    const uint32_t elems = (uint32_t)elems64;
    const bool peer = world > 1 && t->peer_ok && elems <= kTpPeerElems && elems % 4 == 0;
    int rc = tp_reserve(t, m, x_dtype);
    if (rc) return rc;
    if (world > 1 && !peer) {
        rc = tp_nccl_init(t);
        if (rc) return rc;
    }
    const size_t xb = (size_t)elems * (x_dtype == RLXQ_BF16 ? 2 : 4);
    void* bufs[8] = {nullptr};
    for (uint32_t i = 0; i < world; ++i) bufs[i] = t->ranks[i].comm_buf;
    for (uint32_t i = 0; i < world; ++i) {
        TpRank& r = t->ranks[i];
        RLXQ_CUDA_TRY(cudaSetDevice(r.dev));
        RLXQ_CUDA_TRY(cudaMemcpyAsync(r.x, x_host, xb, cudaMemcpyHostToDevice, r.stream));
        uint8_t* ws = reinterpret_cast<uint8_t*>(((uintptr_t)r.ws + 255) & ~(uintptr_t)255);
        // decode sizes over peer memory: the step with the exchange inside (rlxq_tp_ffn_step); else the partial alone
        if (peer)
            rc = rlxq_tp_ffn_step((rlxq_stream_t)r.stream, t->scheme, t->scheme, r.x, x_dtype, r.gate_up, r.down, r.y, m,
                                  t->d_model, f, ws, r.ws_bytes - (size_t)(ws - r.ws), i, world, bufs, kTpPeerElems);
        else
            rc = rlxq_tp_ffn_partial((rlxq_stream_t)r.stream, t->scheme, t->scheme, r.x, x_dtype, r.gate_up, r.down, r.y, m,
                                     t->d_model, f, ws, r.ws_bytes - (size_t)(ws - r.ws));
        if (rc) return rc;
    }
    if (!peer && world > 1) {
        RLXQ_NCCL_TRY(t, t->nccl.GroupStart());
        for (TpRank& r : t->ranks) {
            const ncclResult_t nr = t->nccl.AllReduce(r.y, r.y, elems, ncclFloat, ncclSum, r.nccl, r.stream);
            if (nr != ncclSuccess) { t->nccl.GroupEnd(); return fail(RLXQ_E_NCCL, "ncclAllReduce: %s", t->nccl.GetErrorString(nr)); }
        }
        RLXQ_NCCL_TRY(t, t->nccl.GroupEnd());
    }
    // every rank holds the same sum: rank 0's goes back
    RLXQ_CUDA_TRY(cudaSetDevice(t->ranks[0].dev));
    RLXQ_CUDA_TRY(cudaMemcpyAsync(y_host, t->ranks[0].y, (size_t)elems * 4, cudaMemcpyDeviceToHost, t->ranks[0].stream));
    for (TpRank& r : t->ranks) {
        RLXQ_CUDA_TRY(cudaSetDevice(r.dev));
        RLXQ_CUDA_TRY(cudaStreamSynchronize(r.stream));
    }
    return RLXQ_OK;
}

// Bounded-wait status of every device of the group (rlxq_device_status per device): the first error wins.
extern "C" int rlxq_tp_status(rlxq_tp* t, int* device_error) {
    if (!t || !device_error) return fail(RLXQ_E_NULL, "null argument");
    *device_error = 0;
    for (TpRank& r : t->ranks) {
        RLXQ_CUDA_TRY(cudaSetDevice(r.dev));
        int code = 0;
        const int rc = rlxq_device_status(&code);
        if (rc) { *device_error = code; return rc; }
    }
    return RLXQ_OK;
}
