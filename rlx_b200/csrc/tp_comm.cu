// One-shot sum all-reduce of a small f32 vector over NVLink peer memory, one rank per GPU.
//
// The decode step of the tensor-parallel FFN ends with a sum of world partial rows [m, d_model] (32 KiB
// at m = 1).  For that size a library all-reduce is all latency (10-20 us).  Here every rank writes its
// partial straight into every peer's buffer (posted stores over NVLink: nobody waits for a read to come
// back), raises a flag in every peer's header behind them, waits for the peers' flags in its own header,
// and then adds the world partials that now sit in its own memory, in rank order -- the order of the
// reference's host collective (rlx-driver/src/collective.rs:107-127: put, barrier, fold from the identity),
// so the result is the same on every rank and from run to run.  Plain peer stores; no multimem, no TMA.
// (The first version pulled: publish locally, flag, then read every peer's partial.  Its sum loop over the
// ranks was not unrolled, so each thread paid one NVLink round trip per peer, one after the other: 33 us
// of a 53 us step on eight GPUs.)
//
// The vector is cut into kCommParts parts, one CTA each, every part with its own epoch and flags, so the
// parts never wait for one another: eight SMs push and add instead of one.
//
// Buffer of a rank: [header 1 KiB: epoch[part], flags[part][8]] [parity 0: world slots] [parity 1: world
// slots], a slot max_elems floats.  The epochs live on the device and are advanced by the kernel, so a
// captured launch works on every replay; the two parities alternate with them, which is what lets a fast
// rank push the next step while a slow one still adds the previous one (a rank cannot be two steps ahead:
// finishing a step takes every peer's flag of that step).  Every wait is bounded: a rank whose peer never
// arrives records an error word and returns without touching (that part of) dst.
#include "common.cuh"
#include "rlxq_tp.h"
#include "staged_common.cuh"
#include "tp_comm.cuh"

namespace rlxq {

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
__device__ __forceinline__ float4 ld_sys_f4(const float4* p) {        // no caching: another GPU wrote it
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_f4(float4* p, float4 v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__global__ void __launch_bounds__(512) tp_allreduce_kernel(const CommParams P) {
    __shared__ unsigned long long s_epoch;
    __shared__ int s_fail;
    griddep_launch_dependents();
    griddep_wait();                  // src comes from the kernel in front
    const uint32_t part = blockIdx.x;
    unsigned long long* hdr = reinterpret_cast<unsigned long long*>(P.buf[P.rank]);
    unsigned long long* my_flags = hdr + kCommParts + part * kCommMaxWorld;           // written by the peers
    if (threadIdx.x == 0) {
        s_epoch = hdr[part] + 1ull;
        hdr[part] = s_epoch;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const size_t parity = (size_t)(epoch & 1ull) * kCommMaxWorld * P.max_elems;      // floats
    // this CTA's share of the float4s
    const uint32_t n4 = P.elems / 4, per = (n4 + kCommParts - 1) / kCommParts;
    const uint32_t i0 = min(n4, part * per), i1 = min(n4, i0 + per);
    // 1. this rank's partial into its slot of every rank's buffer (its own included)
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(P.src)[i];
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world)
                st_sys_f4(reinterpret_cast<float4*>(P.buf[r] + kCommHeader) + (parity + (size_t)P.rank * P.max_elems) / 4 + i, v);
    }
    __syncthreads();                 // the release stores below, after this barrier, cover every thread's writes
    // 2. tell every peer, 3. wait for every peer (one thread per peer)
    if (threadIdx.x < P.world && threadIdx.x != P.rank) {
        const uint32_t p = threadIdx.x;
        st_release_sys(reinterpret_cast<unsigned long long*>(P.buf[p]) + kCommParts + part * kCommMaxWorld + P.rank, epoch);
        bool ok = false;
        for (uint32_t it = 0; it < P.spin_limit; ++it) {
            if (ld_acquire_sys(my_flags + p) >= epoch) { ok = true; break; }
        }
        if (!ok) { s_fail = 1; atomicExch(P.err, 40 + (int)p); }
    }
    __syncthreads();
    if (s_fail) return;
    // 4. sum in rank order, out of this rank's own memory; all loads of an element are issued before the first add
    const float4* mine = reinterpret_cast<const float4*>(P.buf[P.rank] + kCommHeader) + parity / 4;
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        float4 v[kCommMaxWorld];
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world) v[r] = ld_sys_f4(mine + (size_t)r * (P.max_elems / 4) + i);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
        reinterpret_cast<float4*>(P.dst)[i] = acc;
    }
}

}  // namespace rlxq

using namespace rlxq;

extern "C" int rlxq_tp_comm_bytes(uint32_t max_elems, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    if (max_elems == 0 || max_elems % 4) return fail(RLXQ_E_SHAPE, "max_elems=%u must be a positive multiple of 4", max_elems);
    *bytes = kCommHeader + 2 * (size_t)kCommMaxWorld * max_elems * 4;      // two parities of one slot per possible rank
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
    int rc = launch_pdl(tp_allreduce_kernel, dim3(kCommParts), dim3(512), 0, (cudaStream_t)stream, P);
    if (rc) return rc;
    count_launch();
    return check_launch("tp_allreduce_kernel");
}
