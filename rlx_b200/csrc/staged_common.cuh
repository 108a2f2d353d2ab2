// Pieces shared by the two staged GEMV kernels (tensor mode in gemv_staged.cu, integer mode in
// gemv_int.cu): per-format staging constants, the kernel parameter block, and the PTX wrappers
// for mbarriers, bulk async copies and named barriers.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"
#include "decode.cuh"

namespace rlxq {

// ---------------------------------------------------------------------------------------------
// Per-format constants
// ---------------------------------------------------------------------------------------------
template <uint32_t SCHEME> struct StagedTraits;
// UNIT_B : bytes of 256 consecutive weights of one row
// AG     : 256-weight units per 16-byte-aligned group (bulk copies move whole groups)
// CU     : units per stage chunk            STRIDE : shared-memory bytes between tile rows
// STAGES : ring depth                       SUB    : weights per activation-sum block
// BIAS   : constant removed per weight (fp16 "1024 + q" trick plus the format's own offset)
template <> struct StagedTraits<RLXQ_Q4_0> {
    static constexpr uint32_t UNIT_B = 144, AG = 1, CU = 4, STRIDE = 592, STAGES = 4, SUB = 32;
    static constexpr float BIAS = -1032.f;
};
template <> struct StagedTraits<RLXQ_Q8_0> {
    static constexpr uint32_t UNIT_B = 272, AG = 1, CU = 4, STRIDE = 1104, STAGES = 4, SUB = 32;
    static constexpr float BIAS = -1152.f;
};
template <> struct StagedTraits<RLXQ_Q4_K> {
    static constexpr uint32_t UNIT_B = 144, AG = 1, CU = 4, STRIDE = 672, STAGES = 4, SUB = 32;
    static constexpr float BIAS = -1024.f;
};
template <> struct StagedTraits<RLXQ_Q6_K> {
    static constexpr uint32_t UNIT_B = 210, AG = 8, CU = 8, STRIDE = 1680, STAGES = 3, SUB = 16;
    static constexpr float BIAS = -1056.f;
};

// Q5_K only runs in the integer GEMV (batch 1-2), which reads UNIT_B, AG and SUB; the rest mirrors Q4_K.
template <> struct StagedTraits<RLXQ_Q5_K> {
    static constexpr uint32_t UNIT_B = 176, AG = 1, CU = 4, STRIDE = 800, STAGES = 4, SUB = 32;
    static constexpr float BIAS = -1024.f;
};

// Q8_K, Q2_K, Q3_K only run in the integer GEMV with its integer-MMA units, which reads UNIT_B, AG and SUB
// (rows of 292-, 84- and 110-byte super-blocks are 16-byte aligned every 4, 4 and 8 of them).
// The 32-weight container types (20-, 22- and 24-byte blocks): integer-MMA units only, like the three below.
template <> struct StagedTraits<RLXQ_Q4_1> {
    static constexpr uint32_t UNIT_B = 160, AG = 1, CU = 8, STRIDE = 1296, STAGES = 4, SUB = 32;
    static constexpr float BIAS = 0.f;
};
template <> struct StagedTraits<RLXQ_Q5_0> {
    static constexpr uint32_t UNIT_B = 176, AG = 1, CU = 8, STRIDE = 1424, STAGES = 4, SUB = 32;
    static constexpr float BIAS = 0.f;
};
template <> struct StagedTraits<RLXQ_Q5_1> {
    static constexpr uint32_t UNIT_B = 192, AG = 1, CU = 8, STRIDE = 1552, STAGES = 4, SUB = 32;
    static constexpr float BIAS = 0.f;
};
template <> struct StagedTraits<RLXQ_Q8_K> {
    static constexpr uint32_t UNIT_B = 292, AG = 4, CU = 4, STRIDE = 1200, STAGES = 4, SUB = 32;
    static constexpr float BIAS = 0.f;
};
template <> struct StagedTraits<RLXQ_Q2_K> {
    static constexpr uint32_t UNIT_B = 84, AG = 4, CU = 8, STRIDE = 688, STAGES = 4, SUB = 16;
    static constexpr float BIAS = 0.f;
};
template <> struct StagedTraits<RLXQ_Q3_K> {
    static constexpr uint32_t UNIT_B = 110, AG = 8, CU = 8, STRIDE = 880, STAGES = 4, SUB = 16;
    static constexpr float BIAS = 0.f;
};

constexpr uint32_t kConsumerWarps = 4;
constexpr uint32_t kThreads = (kConsumerWarps + 1) * 32;
// A waiting thread is suspended by the hardware for up to kSuspendHintNs per attempt, so a wait
// costs a handful of instructions however long it lasts; kWaitLimit attempts bound it (seconds).
constexpr uint32_t kSuspendHintNs = 1000000u;
constexpr uint32_t kWaitLimit = 1u << 12;

struct StagedParams {
    const void* x;
    const uint8_t* w;
    void* y;
    float* partial;       // [ksl][m][n] when ksl > 1
    uint32_t* counters;   // [ntiles]     when ksl > 1
    int* err;             // device error word
    uint32_t m, k, n;
    uint32_t x_bf16, y_bf16;
    uint32_t row_bytes;   // bytes of one weight row
    uint32_t ntiles;      // ceil(n / 16)
    uint32_t rg;          // row groups: CTA (rgi, ks) owns tiles rgi, rgi + rg, ...
    uint32_t ksl;         // k slices
    uint32_t usl;         // 256-weight units per slice (the last slice may hold fewer)
    uint32_t xs_stride;   // halfs between activation rows in shared memory
    uint32_t mp;          // m rounded up to even
    uint32_t off_sxb, off_stage, off_scratch, off_red, off_bar;  // shared-memory layout
    uint32_t nstages;     // ring depth (runtime: whatever shared memory is left)
    const __half* xh_ws;  // [m][k] activations as fp16 after the row rescale (written by the converter kernel)
    const float* sxb_ws;  // [k / SUB][mp] block sums * BIAS
    const float* inv_ws;  // [8] 1 / row scale
};

// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(kSuspendHintNs) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out (the caller records an error and drains).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// A whole warp waiting on one barrier: one lane polls (every try_wait is a serialised operation on the barrier's
// word, and many warps share a stage barrier), the warp barrier hands the result and the memory ordering to the others.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, uint32_t lane) {
    uint32_t got = 1u;
    if (lane == 0) got = mbar_wait(bar, parity) ? 1u : 0u;
    __syncwarp();
    return __shfl_sync(0xFFFFFFFFu, got, 0) != 0u;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
template <uint32_t THREADS>
__device__ __forceinline__ void consumer_bar_n() {  // named barrier 1 over the first THREADS threads
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}
__device__ __forceinline__ void consumer_bar() {  // the four consumer warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}
__device__ __forceinline__ uint32_t lds_u32_2(const uint8_t* p) {  // 2-byte-aligned 32-bit read
    return lds_u16(p) | (lds_u16(p + 2) << 16);
}
__device__ __forceinline__ uint32_t lds_u32(const uint8_t* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}

__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with programmatic stream serialization (unless the "pdl" option is 0): the kernel may become
// resident while its predecessor drains; it orders itself with griddepcontrol.wait.
template <typename Kern, typename... Args>
static int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = options().pdl.load() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RLXQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
    return RLXQ_OK;
}

// One error word per device, allocated on first use (outside any capture), never freed.
int* device_error_word();
int* device_error_word_if_ready();   // never allocates; null if the device has none yet

}  // namespace rlxq
