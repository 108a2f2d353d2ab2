// Kernel selection for rlxq_matmul: the counterpart of the reference's
// `use_gpu = dequant_scratch_off > 0 && blas.is_some()` branch and host fallback
// (rlx-cuda/src/backend.rs:5366-5405).  There is no host fallback here: every shape runs on
// the GPU, through the fastest kernel that supports it.
#include "common.cuh"
#include "kernels.h"

namespace rlxq {

size_t matmul_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t x_dtype,
                              uint32_t y_dtype) {
    (void)x_dtype; (void)y_dtype;
    if (m == 0 || n == 0 || k == 0) return 0;
    if (m <= 8) {
        // large enough for whichever GEMV kernel the dispatcher (or a forced option) picks
        const size_t a = staged_workspace_bytes(scheme, m, k, n);
        // (batch 5-8 of a format that only has the integer kernel runs it twice, four rows at a time)
        const size_t b = int_workspace_bytes(scheme, m <= 4 ? m : 4, k, n);
        // the tcgen05 GEMV (8-byte words for the parts of cut tiles) only runs when it is asked for
        const size_t c = options().gemv_kernel.load() == 4 ? gemv_tc_workspace_bytes(scheme, m, k, n) : 0;
        const size_t d = int_mma_workspace_bytes(scheme, m, k, n);
        const size_t ab = a > b ? a : b, cd = c > d ? c : d;
        return ab > cd ? ab : cd;
    }
    return gemm_tc_workspace_bytes(m, k, n);      // partial tiles of the stream-K split, when the shape wants it
}

int dispatch_matmul(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                    bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    if (k == 0) {
        // empty reduction: the reference zero-fills the output (rlx-cpu/src/gguf_matmul.rs:52)
        RLXQ_CUDA_TRY(cudaMemsetAsync(y, 0, (size_t)m * n * (ybf ? 2 : 4), stream));
        return RLXQ_OK;
    }
    if (!x || !w) return fail(RLXQ_E_NULL, "null input buffer");
    if ((uintptr_t)w & 1u) return fail(RLXQ_E_ALIGN, "w_blocks must be 2-byte aligned");
    if ((uintptr_t)x & 15u) return fail(RLXQ_E_ALIGN, "x must be 16-byte aligned");
    if ((uintptr_t)y & (ybf ? 1u : 3u)) return fail(RLXQ_E_ALIGN, "y must be aligned to its element size");
    if (m <= 8) {
        // 0 = automatic: the integer kernel with its dp4a units for batch 1-2, with its integer-MMA units for batch
        // 3-8 (and batch 2 of the formats with 32-weight blocks, where it already wins), then the staged tensor-mode
        // kernel, then the generic one.  The dp4a units also run batch 3-4, but only when asked for with gemv_kernel = 3.
        const int64_t force = options().gemv_kernel.load();
        const bool can_int = m <= 4 && int_supported(scheme, m, k, n, w, x);
        const bool can_tc = staged_supported(scheme, m, k, n, w, x, xbf);
        const bool can_tcg = gemv_tc_supported(scheme, m, k, n, w, x, xbf);
        if (force == 4) {
            if (!can_tcg) return fail(RLXQ_E_SHAPE, "tensor-core GEMV does not support scheme %u m=%u k=%u n=%u (or 16-byte alignment)", scheme, m, k, n);
            return launch_gemv_tc(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        }
        if (force == 5) {
            if (!int_mma_supported(scheme, m, k, n, w, x)) return fail(RLXQ_E_SHAPE, "integer-MMA GEMV does not support scheme %u m=%u k=%u n=%u (or 16-byte alignment)", scheme, m, k, n);
            return launch_gemv_int_mma(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        }
        if (force == 3 && !can_int)
            return fail(RLXQ_E_SHAPE, "integer GEMV does not support m=%u k=%u n=%u (or 16-byte alignment)", m, k, n);
        if (force == 2 && !can_tc)
            return fail(RLXQ_E_SHAPE, "staged GEMV does not support m=%u k=%u n=%u (or 16-byte alignment)", m, k, n);
        const bool mma_first = m >= 3 || (m == 2 && (scheme == RLXQ_Q4_0 || scheme == RLXQ_Q8_0));
        if (force == 0 && mma_first && int_mma_supported(scheme, m, k, n, w, x))
            return launch_gemv_int_mma(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        if (force == 3 || (force == 0 && can_int && m <= 2))
            return launch_gemv_int(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        if (force == 2 || (force == 0 && can_tc))
            return launch_gemv_staged(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        // A format with the integer kernel but no tensor-mode kernel (Q5_K): batch 3-4 in one pass, batch 5-8 in
        // two passes of four rows; streaming the weights twice still beats the warp-per-row kernel several times.
        if (force == 0 && can_int) return launch_gemv_int(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        if (force == 0 && m > 4 && int_supported(scheme, 4, k, n, w, x) && int_supported(scheme, m - 4, k, n, w, x)) {
            const size_t xrow = (size_t)k * (xbf ? 2 : 4), yrow = (size_t)n * (ybf ? 2 : 4);
            if ((4 * xrow) % 16 == 0) {
                int rc = launch_gemv_int(stream, scheme, x, xbf, w, y, ybf, 4, k, n, ws, ws_bytes);
                if (rc) return rc;
                return launch_gemv_int(stream, scheme, static_cast<const uint8_t*>(x) + 4 * xrow, xbf, w,
                                       static_cast<uint8_t*>(y) + 4 * yrow, ybf, m - 4, k, n, ws, ws_bytes);
            }
        }
        return launch_matmul_generic(stream, scheme, x, xbf, w, y, ybf, m, k, n);
    }
    // m > 8: tensor-memory GEMM for bf16 activations, the tiled generic kernel otherwise
    const int64_t gforce = options().gemm_kernel.load();
    const bool can = gemm_tc_supported(scheme, m, k, n, w, x, xbf);
    if (gforce == 2 && !can)
        return fail(RLXQ_E_SHAPE, "the tcgen05 GEMM needs bf16 activations, k %% 256 == 0 (2048 for Q6_K), one of Q4_0/Q8_0/Q4_K/Q5_K/Q6_K and 16-byte alignment");
    if (can && gforce != 1) return launch_gemm_tc(stream, scheme, x, w, y, ybf, m, k, n, ws, ws_bytes);
    return launch_matmul_generic(stream, scheme, x, xbf, w, y, ybf, m, k, n);
}

}  // namespace rlxq
