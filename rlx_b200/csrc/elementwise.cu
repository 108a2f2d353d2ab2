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

}  // namespace rlxq
