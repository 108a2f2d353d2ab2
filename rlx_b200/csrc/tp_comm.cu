// One-shot sum all-reduce of a small f32 vector over NVLink peer memory, one rank per GPU.
//
// The decode step of the tensor-parallel FFN ends with a sum of world partial rows [m, d_model] (32 KiB
// at m = 1).  For that size a library all-reduce is all latency (10-20 us); here every rank publishes its
// partial in a buffer the others have mapped (CUDA IPC), raises a flag in every peer's header, waits for
// the peers' flags, then reads all partials over NVLink and adds them in rank order -- the order of the
// reference's host collective (rlx-driver/src/collective.rs:107-127), so the result is the same on every
// rank and from run to run.  Plain peer loads and stores; no multimem, no TMA.
//
// Buffer of a rank: [header 256 B: epoch, flags[8]] [data slot 0] [data slot 1].  The epoch lives on the
// device and is advanced by the kernel, so a captured launch works on every replay; the two data slots
// alternate with it, which is what lets a fast rank start the next step while a slow one still reads.
// Every wait is bounded: a rank whose peer never arrives records an error word and returns.
#include "common.cuh"
#include "rlxq_tp.h"
#include "staged_common.cuh"

namespace rlxq {

constexpr uint32_t kCommMaxWorld = 8;
constexpr uint32_t kCommHeader = 256;
// Polls of a peer-written flag before a rank gives up: option "tp_spin_limit", default 2^24 (a few seconds).

struct CommParams {
    uint8_t* buf[kCommMaxWorld];     // buf[r]: rank r's buffer as mapped in this process (buf[rank] is local)
    const float* src;
    float* dst;
    int* err;
    uint32_t rank, world, elems, max_elems;
    uint32_t spin_limit;
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {       // no caching: another GPU wrote it
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(1024) tp_allreduce_kernel(const CommParams P) {
    __shared__ unsigned long long s_epoch;
    __shared__ int s_fail;
    griddep_launch_dependents();
    griddep_wait();                  // src comes from the kernel in front
    unsigned long long* hdr = reinterpret_cast<unsigned long long*>(P.buf[P.rank]);   // [0] epoch, [1..8] flags
    if (threadIdx.x == 0) {
        s_epoch = hdr[0] + 1ull;
        hdr[0] = s_epoch;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const size_t slot = (size_t)(epoch & 1ull) * P.max_elems;
    const uint32_t n4 = P.elems / 4;
    // 1. publish this rank's partial
    float4* mine = reinterpret_cast<float4*>(P.buf[P.rank] + kCommHeader) + slot / 4;
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) mine[i] = reinterpret_cast<const float4*>(P.src)[i];
    __syncthreads();                 // the release stores below, after this barrier, cover every thread's writes
    // 2. tell every peer, 3. wait for every peer (one thread per peer)
    if (threadIdx.x < P.world && threadIdx.x != P.rank) {
        const uint32_t p = threadIdx.x;
        st_release_sys(reinterpret_cast<unsigned long long*>(P.buf[p]) + 1 + P.rank, epoch);
        bool ok = false;
        for (uint32_t it = 0; it < P.spin_limit; ++it) {
            if (ld_acquire_sys(hdr + 1 + p) >= epoch) { ok = true; break; }
        }
        if (!ok) { s_fail = 1; atomicExch(P.err, 40 + (int)p); }
    }
    __syncthreads();
    if (s_fail) return;
    // 4. sum in rank order
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < P.world; ++r) {
            const float4* q = reinterpret_cast<const float4*>(P.buf[r] + kCommHeader) + slot / 4 + i;
            const float4 v = r == P.rank ? *q : ld_peer_f4(q);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(P.dst)[i] = acc;
    }
}

}  // namespace rlxq

using namespace rlxq;

extern "C" int rlxq_tp_comm_bytes(uint32_t max_elems, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    if (max_elems == 0 || max_elems % 4) return fail(RLXQ_E_SHAPE, "max_elems=%u must be a positive multiple of 4", max_elems);
    *bytes = kCommHeader + 2 * (size_t)max_elems * 4;
    return RLXQ_OK;
}

extern "C" int rlxq_tp_comm_alloc(uint32_t max_elems, void** buf) {
    if (!buf) return fail(RLXQ_E_NULL, "buf is null");
    size_t bytes = 0;
    int rc = rlxq_tp_comm_bytes(max_elems, &bytes);
    if (rc) return rc;
    RLXQ_CUDA_TRY(cudaMalloc(buf, bytes));          // an allocation of its own: IPC handles name whole allocations
    RLXQ_CUDA_TRY(cudaMemset(*buf, 0, bytes));
    RLXQ_CUDA_TRY(cudaDeviceSynchronize());
    return RLXQ_OK;
}

extern "C" int rlxq_tp_comm_free(void* buf) {
    if (buf) RLXQ_CUDA_TRY(cudaFree(buf));
    return RLXQ_OK;
}

extern "C" int rlxq_tp_ipc_export(const void* buf, uint8_t handle[64]) {
    if (!buf || !handle) return fail(RLXQ_E_NULL, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    RLXQ_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void*>(buf)));
    memcpy(handle, &h, 64);
    return RLXQ_OK;
}

extern "C" int rlxq_tp_ipc_open(const uint8_t handle[64], void** buf) {
    if (!buf || !handle) return fail(RLXQ_E_NULL, "null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    RLXQ_CUDA_TRY(cudaIpcOpenMemHandle(buf, h, cudaIpcMemLazyEnablePeerAccess));
    return RLXQ_OK;
}

extern "C" int rlxq_tp_ipc_close(void* buf) {
    if (buf) RLXQ_CUDA_TRY(cudaIpcCloseMemHandle(buf));
    return RLXQ_OK;
}

extern "C" int rlxq_tp_allreduce_sum(rlxq_stream_t stream, uint32_t rank, uint32_t world, void* const* bufs,
                                     uint32_t max_elems, const float* src, float* dst, uint32_t elems) {
    if (world < 1 || world > kCommMaxWorld || rank >= world) return fail(RLXQ_E_ARG, "bad rank %u of %u", rank, world);
    if (!bufs || !src || !dst) return fail(RLXQ_E_NULL, "null argument");
    if (elems == 0) return RLXQ_OK;
    if (elems % 4 || elems > max_elems) return fail(RLXQ_E_SHAPE, "elems=%u must be a multiple of 4 and at most %u", elems, max_elems);
    if (((uintptr_t)src | (uintptr_t)dst) & 15u) return fail(RLXQ_E_ALIGN, "src and dst must be 16-byte aligned");
    CommParams P{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!bufs[r]) return fail(RLXQ_E_NULL, "buffer of rank %u is null", r);
        P.buf[r] = reinterpret_cast<uint8_t*>(bufs[r]);
    }
    P.src = src; P.dst = dst; P.rank = rank; P.world = world; P.elems = elems; P.max_elems = max_elems;
    P.spin_limit = (uint32_t)options().tp_spin_limit.load();
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    int rc = launch_pdl(tp_allreduce_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, P);
    if (rc) return rc;
    count_launch();
    return check_launch("tp_allreduce_kernel");
}
