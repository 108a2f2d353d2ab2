// Generic fused dequant + matmul kernel: one warp per weight row, any k that is a multiple
// of the block size, any m (processed eight activation rows at a time), 2-byte-aligned
// blocks.  It is the shape-agnostic path behind rlxq_matmul; the staged tensor-core GEMV
// and the tcgen05 GEMM take over for the shapes they support.
//
// Each lane decodes four consecutive weights at a time (the same decoders the bit-exact
// dequant kernel uses), multiplies them into up to eight f32 accumulators, and the warp
// finishes with a shuffle reduction.  Accumulation is f32; the summation order differs from
// the reference's sequential loop (rlx-cpu/src/gguf_matmul.rs:65-93), which the path's
// tolerance (1e-3 * |x| * |w_row|) covers.
#include "common.cuh"
#include "decode.cuh"

namespace rlxq {

template <bool XBF16>
__device__ __forceinline__ float4 load_x4(const void* x, uint64_t idx) {
    if constexpr (XBF16) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + idx);
        return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u),
                           __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
    } else {
        return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx);
    }
}

template <uint32_t SCHEME, int MT, bool XBF16, bool YBF16>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const void* __restrict__ x,
                                                           const uint8_t* __restrict__ w,
                                                           void* __restrict__ y, uint32_t m0,
                                                           uint32_t m, uint32_t k, uint32_t n) {
    constexpr uint32_t E = SchemeTraits<SCHEME>::kElems, B = SchemeTraits<SCHEME>::kBytes;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint64_t row_bytes = (uint64_t)(k / E) * B;
    const uint32_t mt = min((uint32_t)MT, m - m0);
    for (uint32_t row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < n;
         row += gridDim.x * warps_per_cta) {
        const uint8_t* wr = w + (uint64_t)row * row_bytes;
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; i++) acc[i] = 0.f;
        for (uint32_t e = lane * 4; e < k; e += 128) {
            const float4 wv = decode4_exact<SCHEME>(wr + (uint64_t)(e / E) * B, e % E);
#pragma unroll
            for (int i = 0; i < MT; i++) {
                if ((uint32_t)i < mt) {
                    const float4 xv = load_x4<XBF16>(x, (uint64_t)(m0 + i) * k + e);
                    acc[i] = fmaf(wv.x, xv.x, acc[i]);
                    acc[i] = fmaf(wv.y, xv.y, acc[i]);
                    acc[i] = fmaf(wv.z, xv.z, acc[i]);
                    acc[i] = fmaf(wv.w, xv.w, acc[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MT; i++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], o);
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < MT; i++) {
                if ((uint32_t)i < mt) {
                    const uint64_t o = (uint64_t)(m0 + i) * n + row;
                    if constexpr (YBF16)
                        reinterpret_cast<uint16_t*>(y)[o] = (uint16_t)f32_to_bf16_bits(acc[i]);
                    else
                        reinterpret_cast<float*>(y)[o] = acc[i];
                }
            }
        }
    }
}

template <uint32_t SCHEME, bool XBF16, bool YBF16>
static int launch_generic_t(cudaStream_t stream, const void* x, const uint8_t* w, void* y,
                            uint32_t m, uint32_t k, uint32_t n) {
    const int threads = 256, wpc = threads / 32;
    unsigned blocks = (n + wpc - 1) / wpc;
    const unsigned cap = (unsigned)sm_count() * 8 * 8;
    if (blocks > cap) blocks = cap;
    for (uint32_t m0 = 0; m0 < m; m0 += 8) {
        const uint32_t mt = (m - m0 < 8) ? (m - m0) : 8;
        if (mt == 1)
            gemv_generic_kernel<SCHEME, 1, XBF16, YBF16><<<blocks, threads, 0, stream>>>(x, w, y, m0, m, k, n);
        else if (mt <= 4)
            gemv_generic_kernel<SCHEME, 4, XBF16, YBF16><<<blocks, threads, 0, stream>>>(x, w, y, m0, m, k, n);
        else
            gemv_generic_kernel<SCHEME, 8, XBF16, YBF16><<<blocks, threads, 0, stream>>>(x, w, y, m0, m, k, n);
        count_launch();
    }
    return check_launch("gemv_generic_kernel");
}

template <uint32_t SCHEME>
static int launch_generic_s(cudaStream_t stream, const void* x, bool xbf, const uint8_t* w, void* y,
                            bool ybf, uint32_t m, uint32_t k, uint32_t n) {
    if (xbf && ybf) return launch_generic_t<SCHEME, true, true>(stream, x, w, y, m, k, n);
    if (xbf) return launch_generic_t<SCHEME, true, false>(stream, x, w, y, m, k, n);
    if (ybf) return launch_generic_t<SCHEME, false, true>(stream, x, w, y, m, k, n);
    return launch_generic_t<SCHEME, false, false>(stream, x, w, y, m, k, n);
}

int launch_matmul_generic(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf,
                          const uint8_t* w, void* y, bool ybf, uint32_t m, uint32_t k, uint32_t n) {
    switch (scheme) {
        case RLXQ_Q8_0: return launch_generic_s<RLXQ_Q8_0>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q4_0: return launch_generic_s<RLXQ_Q4_0>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q4_K: return launch_generic_s<RLXQ_Q4_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q6_K: return launch_generic_s<RLXQ_Q6_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q5_K: return launch_generic_s<RLXQ_Q5_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q8_K: return launch_generic_s<RLXQ_Q8_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q2_K: return launch_generic_s<RLXQ_Q2_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q3_K: return launch_generic_s<RLXQ_Q3_K>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q4_1: return launch_generic_s<RLXQ_Q4_1>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q5_0: return launch_generic_s<RLXQ_Q5_0>(stream, x, xbf, w, y, ybf, m, k, n);
        case RLXQ_Q5_1: return launch_generic_s<RLXQ_Q5_1>(stream, x, xbf, w, y, ybf, m, k, n);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
}

}  // namespace rlxq
