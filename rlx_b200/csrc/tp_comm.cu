// One-shot sum all-reduce of a small f32 vector over NVLink peer memory, one rank per GPU.
//
// The decode step of the tensor-parallel FFN ends with a sum of world partial rows [m, d_model] (32 KiB
// at m = 1).  For that size a library all-reduce is all latency (10-20 us).  Here every rank writes its
// partial straight into every peer's buffer (posted stores over NVLink: nobody waits for a read to come
// back) as 8-byte words {value, step tag}: a word is stored and loaded whole, so a reader that finds the tag
// of the current step in a word has the value that belongs to it.  No flag follows the data and no fence
// orders the two: a rank polls the words in its own memory (bounded) and adds the world partials in rank order
// -- the order of the reference's host collective (rlx-driver/src/collective.rs:107-127: put, barrier, fold
// from the identity), so the result is the same on every rank and from run to run.  Plain peer stores; no
// multimem, no TMA.
// (Earlier forms, per step on eight GPUs: pulling the peers' partials with a sum loop that was not unrolled,
// 33 us of a 53 us step; pushing floats and raising a flag behind them with st.release.sys, whose fence waits
// for every posted store to be acknowledged, 8.4 us of 27.8.)
//
// The vector is cut into kCommParts parts, one CTA each, every part with its own step counter, so the parts
// never wait for one another: eight SMs push and add instead of one.
//
// Buffer of a rank: [header 1 KiB: step counter per part, the words of the pushing down projection]
// [parity 0: a slot of max_elems tagged words per possible rank] [parity 1: the same] [the float slots of the
// pushing down projection, two parities].  The step counters live on the device and are advanced by the kernel,
// so a captured launch works on every replay; the two parities alternate with them, which is what lets a fast
// rank push the next step while a slow one still adds the previous one (a rank cannot be two steps ahead:
// finishing a step takes every peer's words of that step, which a peer sends only after it finished the step
// before).  Every wait is bounded: a rank whose peer never arrives records an error word and returns without
// touching (that part of) dst.
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

// a tagged word: stored and loaded as one 8-byte access
__device__ __forceinline__ void st_word_sys(void* p, float v, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_word_sys(const void* p) {        // no caching: another GPU wrote it
    uint2 w;
    asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
    return w;
}

__global__ void __launch_bounds__(512) tp_allreduce_kernel(const CommParams P) {
    __shared__ unsigned long long s_epoch;
    __shared__ int s_fail;
    griddep_launch_dependents();
    griddep_wait();                  // src comes from the kernel in front
    const uint32_t part = blockIdx.x;
    unsigned long long* hdr = reinterpret_cast<unsigned long long*>(P.buf[P.rank]);
    if (threadIdx.x == 0) {
        s_epoch = hdr[part] + 1ull;
        hdr[part] = s_epoch;
        s_fail = 0;
    }
    __syncthreads();
    const unsigned long long epoch = s_epoch;
    const uint32_t tag = (uint32_t)(epoch & 0x7FFFFFFFull) | 0x80000000u;        // never the zero of a fresh buffer
    const size_t parity = (size_t)(epoch & 1ull) * kCommMaxWorld * P.max_elems;   // words
    // this CTA's share of the elements
    const uint32_t per = (P.elems + kCommParts - 1) / kCommParts;
    const uint32_t i0 = min(P.elems, part * per), i1 = min(P.elems, i0 + per);
    // 1. this rank's partial, tagged, into its slot of every peer's buffer
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = P.src[i];
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world && r != P.rank)
                st_word_sys(reinterpret_cast<uint2*>(P.buf[r] + kCommHeader) + parity + (size_t)P.rank * P.max_elems + i, v, tag);
    }
    // 2. wait, bounded, until every peer's word of every element of this thread carries the tag: the words of all
    //    peers are loaded together (one trip through the memory system per attempt, not one per peer)
    const uint2* mine = reinterpret_cast<const uint2*>(P.buf[P.rank] + kCommHeader) + parity;
    bool ok = true;
    for (uint32_t i = i0 + threadIdx.x; i < i1 && ok; i += blockDim.x) {
        uint32_t late = 0;
        for (uint32_t it = 0; it < P.spin_limit; ++it) {
            uint32_t t[kCommMaxWorld];
#pragma unroll
            for (uint32_t r = 0; r < kCommMaxWorld; ++r)
                t[r] = (r < P.world && r != P.rank) ? ld_word_sys(mine + (size_t)r * P.max_elems + i).y : tag;
            late = 0;
#pragma unroll
            for (uint32_t r = 0; r < kCommMaxWorld; ++r)
                if (t[r] != tag) late |= 1u << r;
            if (late == 0) break;
        }
        if (late) { ok = false; s_fail = 1; atomicExch(P.err, 40 + (int)(__ffs(late) - 1)); }
    }
    __syncthreads();
    if (s_fail) return;
    // 3. sum in rank order (this rank's own partial straight from src); all loads of an element are issued
    //    before the first add
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        float v[kCommMaxWorld];
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world) v[r] = (r == P.rank) ? P.src[i] : __uint_as_float(ld_word_sys(mine + (size_t)r * P.max_elems + i).x);
        float acc = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < kCommMaxWorld; ++r)
            if (r < P.world) acc += v[r];
        P.dst[i] = acc;
    }
}

}  // namespace rlxq

using namespace rlxq;

extern "C" int rlxq_tp_comm_bytes(uint32_t max_elems, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    if (max_elems == 0 || max_elems % 4) return fail(RLXQ_E_SHAPE, "max_elems=%u must be a positive multiple of 4", max_elems);
    // two parities of one slot of tagged words per possible rank, then the float slots of the pushing down projection
    *bytes = comm_push_offset(max_elems) + 2 * (size_t)kCommMaxWorld * max_elems * 4;
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
