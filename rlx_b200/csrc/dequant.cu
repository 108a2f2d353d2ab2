// Bit-exact block dequantisation to f32.
//
// Replaces the reference's `dequant_gguf` kernel (rlx-gpu-kernels/kernels/dequant_gguf.cu:46-244),
// which runs one thread per 256-element super-block, writes 1 KiB per thread with a stride,
// and lets the compiler contract d*q - m into an FMA.  Here each thread decodes four
// consecutive weights and stores one float4, so a warp writes 512 contiguous bytes; the
// arithmetic is the reference CPU decoder's, rounding by rounding.
#include "common.cuh"
#include "decode.cuh"

namespace rlxq {

template <uint32_t SCHEME>
__global__ void __launch_bounds__(256) dequant_f32_kernel(const uint8_t* __restrict__ w,
                                                          uint64_t n_quads, float4* __restrict__ out) {
    constexpr uint32_t E = SchemeTraits<SCHEME>::kElems, B = SchemeTraits<SCHEME>::kBytes;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t q = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_quads; q += stride) {
        const uint64_t e = q * 4;
        const uint64_t blk = e / E;
        const uint32_t t = (uint32_t)(e % E);
        out[q] = decode4_exact<SCHEME>(w + blk * B, t);
    }
}

int launch_dequant_f32(cudaStream_t stream, uint32_t scheme, const uint8_t* w, uint64_t n_elems,
                       float* out) {
    const uint64_t n_quads = n_elems / 4;
    if (n_quads == 0) return RLXQ_OK;
    const int threads = 256;
    uint64_t blocks = (n_quads + threads - 1) / threads;
    const uint64_t cap = (uint64_t)sm_count() * 8 * 4;  // grid-stride beyond a few waves
    if (blocks > cap) blocks = cap;
    float4* o = reinterpret_cast<float4*>(out);
    switch (scheme) {
        case RLXQ_Q8_0: dequant_f32_kernel<RLXQ_Q8_0><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q4_0: dequant_f32_kernel<RLXQ_Q4_0><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q4_K: dequant_f32_kernel<RLXQ_Q4_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q6_K: dequant_f32_kernel<RLXQ_Q6_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q5_K: dequant_f32_kernel<RLXQ_Q5_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q8_K: dequant_f32_kernel<RLXQ_Q8_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q2_K: dequant_f32_kernel<RLXQ_Q2_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q3_K: dequant_f32_kernel<RLXQ_Q3_K><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q4_1: dequant_f32_kernel<RLXQ_Q4_1><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q5_0: dequant_f32_kernel<RLXQ_Q5_0><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        case RLXQ_Q5_1: dequant_f32_kernel<RLXQ_Q5_1><<<(unsigned)blocks, threads, 0, stream>>>(w, n_quads, o); break;
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
    count_launch();
    return check_launch("dequant_f32_kernel");
}

}  // namespace rlxq
