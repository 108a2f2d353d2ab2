// The SwiGLU gate: out = up * silu(gate), silu(x) = x / (1 + exp(-x))
// (rlx-cpu/src/naive.rs:54-56; composition rlx-cuda/src/unfuse.rs:254-293).
#include "common.cuh"
#include "decode.cuh"
#include "host/session.hpp"
#include "kernels.h"
#include "staged_common.cuh"

namespace rlxq {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(256) swiglu_mul_kernel(const float* __restrict__ gate,
                                                         const float* __restrict__ up,
                                                         float* __restrict__ out, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = up[i] * silu_f(gate[i]);
}

int launch_swiglu_mul(cudaStream_t stream, const float* gate, const float* up, float* out, uint64_t n) {
    if (n == 0) return RLXQ_OK;
    uint64_t blocks = (n + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    swiglu_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>(gate, up, out, n);
    count_launch();
    return check_launch("swiglu_mul_kernel");
}

// Byte copy between a pinned host staging buffer and device memory (either direction), both 16-byte
// aligned.  A session in graph mode uses it for activations and outputs of a few KB: a kernel node
// starts sooner than a copy-engine node, and the bytes cross PCIe as plain loads / posted stores.
// Launched with programmatic stream serialization: the kernel behind an input copy becomes resident and
// requests its first weights while the input crosses PCIe, and an output copy is resident, waiting, when
// the kernel in front of it completes.
__global__ void __launch_bounds__(256) copy_bytes_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                                         uint64_t bytes) {
    griddep_launch_dependents();
    griddep_wait();                // every thread: whoever waits for this kernel has then waited for its predecessors
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t n16 = bytes / 16;
    for (uint64_t i = tid; i < n16; i += stride)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (uint64_t i = n16 * 16 + tid; i < bytes; i += stride) dst[i] = src[i];
}

int launch_copy_bytes(cudaStream_t stream, void* dst, const void* src, uint64_t bytes) {
    if (bytes == 0) return RLXQ_OK;
    if (((uintptr_t)dst | (uintptr_t)src) & 15u) return fail(RLXQ_E_ALIGN, "copy_bytes: buffers must be 16-byte aligned");
    uint64_t blocks = (bytes / 16 + 255) / 256;
    if (blocks == 0) blocks = 1;
    if (blocks > 64) blocks = 64;
    int rc = launch_pdl(copy_bytes_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (uint8_t*)dst, (const uint8_t*)src, bytes);
    if (rc) return rc;
    count_launch();
    return check_launch("copy_bytes_kernel");
}

// f32 activations for the tensor-core GEMM, whose operands are bf16: x = hi + lo with hi = bf16(x) and
// lo = bf16(x - hi), which leaves 2^-17 of x behind.  Rows [row0, row0 + rows) of x become rows [0, rows)
// (hi) and [rows, 2 rows) (lo) of `out`; the GEMM multiplies all 2 rows and add_halves_kernel adds the pairs.
__global__ void __launch_bounds__(256) split_hi_lo_kernel(const float* __restrict__ x, uint16_t* __restrict__ out,
                                                          uint64_t rows, uint64_t k) {
    const uint64_t total = rows * k / 4, stride = (uint64_t)gridDim.x * blockDim.x;     // k % 4 == 0
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint16_t h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[j] = (uint16_t)f32_to_bf16_bits(f[j]);
            const float rest = f[j] - __uint_as_float((uint32_t)h[j] << 16);     // exact; inf - inf = NaN stays NaN in y
            l[j] = (uint16_t)f32_to_bf16_bits(isfinite(f[j]) ? rest : 0.f);
        }
        reinterpret_cast<uint2*>(out)[i] = make_uint2(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16));
        reinterpret_cast<uint2*>(out + rows * k)[i] = make_uint2(l[0] | ((uint32_t)l[1] << 16), l[2] | ((uint32_t)l[3] << 16));
    }
}

__global__ void __launch_bounds__(256) add_halves_kernel(const float* __restrict__ y2, void* __restrict__ y, uint32_t y_bf16,
                                                         uint64_t rows, uint64_t n) {
    const uint64_t total = rows * n, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const float v = y2[i] + y2[total + i];
        if (y_bf16) reinterpret_cast<uint16_t*>(y)[i] = (uint16_t)f32_to_bf16_bits(v);
        else reinterpret_cast<float*>(y)[i] = v;
    }
}

int launch_split_hi_lo(cudaStream_t stream, const float* x, void* out, uint64_t rows, uint64_t k) {
    if (rows == 0 || k == 0) return RLXQ_OK;
    uint64_t blocks = (rows * k / 4 + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    split_hi_lo_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, reinterpret_cast<uint16_t*>(out), rows, k);
    count_launch();
    return check_launch("split_hi_lo_kernel");
}

int launch_add_halves(cudaStream_t stream, const float* y2, void* y, bool ybf, uint64_t rows, uint64_t n) {
    if (rows == 0 || n == 0) return RLXQ_OK;
    uint64_t blocks = (rows * n + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    add_halves_kernel<<<(unsigned)blocks, 256, 0, stream>>>(y2, y, ybf ? 1u : 0u, rows, n);
    count_launch();
    return check_launch("add_halves_kernel");
}

}  // namespace rlxq
