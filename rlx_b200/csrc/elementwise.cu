// The SwiGLU gate: out = up * silu(gate), silu(x) = x / (1 + exp(-x))
// (rlx-cpu/src/naive.rs:54-56; composition rlx-cuda/src/unfuse.rs:254-293).
#include "common.cuh"
#include "host/session.hpp"

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
__global__ void __launch_bounds__(256) copy_bytes_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                                         uint64_t bytes) {
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
    copy_bytes_kernel<<<(unsigned)blocks, 256, 0, stream>>>((uint8_t*)dst, (const uint8_t*)src, bytes);
    count_launch();
    return check_launch("copy_bytes_kernel");
}

}  // namespace rlxq
