// Kernel selection for rlxq_matmul: the counterpart of the reference's
// `use_gpu = dequant_scratch_off > 0 && blas.is_some()` branch and host fallback
// (rlx-cuda/src/backend.rs:5366-5405).  There is no host fallback here: every shape runs on
// the GPU, through the fastest kernel that supports it.
#include "common.cuh"
#include "kernels.h"

namespace rlxq {

// Prefill with f32 activations: the tensor-core GEMM takes bf16 operands, so x goes in as hi + lo bf16 halves
// (twice the rows), `chunk` rows of x at a time, and the two partial results are added.  The scratch holds the
// 2 * chunk split rows, the 2 * chunk x n f32 partial results (kept under 128 MiB) and the GEMM's own workspace.
struct SplitPlan { bool ok; uint32_t chunk; size_t off_y2, off_gemm, bytes; };
static SplitPlan plan_f32_split(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n) {
    SplitPlan p{};
    if (m <= 8 || options().gemm_kernel.load() == 1) return p;
    uint64_t chunk = (128ull << 20) / (8ull * n) / 128 * 128;
    if (chunk < 128) chunk = 128;
    if (chunk > 2048) chunk = 2048;
    if (chunk > m) chunk = m;
    // the GEMM's own conditions, on an aligned stand-in for the pointers (dispatch checks the real ones)
    if (!gemm_tc_supported(scheme, 2 * (uint32_t)chunk, k, n, (const void*)256, (const void*)256, true)) return p;
    auto al = [](size_t v) { return (v + 255) / 256 * 256; };
    p.chunk = (uint32_t)chunk;
    p.off_y2 = al((size_t)2 * chunk * k * 2);
    p.off_gemm = p.off_y2 + al((size_t)2 * chunk * n * 4);
    p.bytes = p.off_gemm + al(gemm_tc_workspace_bytes(2 * (uint32_t)chunk, k, n));
    p.ok = true;
    return p;
}

size_t matmul_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t x_dtype,
                              uint32_t y_dtype) {
    (void)y_dtype;
    if (m == 0 || n == 0 || k == 0) return 0;
    if (m > 8 && x_dtype == RLXQ_F32) {
        const SplitPlan sp = plan_f32_split(scheme, m, k, n);
        return sp.ok ? sp.bytes : 0;
    }
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
        // 0 = automatic: the integer kernel with its dp4a units for batch 1, with its integer-MMA units for batch
        // 2-8 (measured at batch 2: level on Q4_K 4096 -> 14336, 5-15 % ahead elsewhere), then the dp4a units again
        // (batch 2, formats without an MMA unit), the staged tensor-mode kernel, the generic one.  The dp4a units
        // also run batch 3-4, but only when asked for with gemv_kernel = 3.
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
        const bool no_dp4a = scheme == RLXQ_Q8_K || scheme == RLXQ_Q2_K || scheme == RLXQ_Q3_K || scheme == RLXQ_Q4_1 ||
                             scheme == RLXQ_Q5_0 || scheme == RLXQ_Q5_1;                             // MMA units only
        if (force == 0 && (m >= 2 || no_dp4a) && int_mma_supported(scheme, m, k, n, w, x))
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
    // m > 8: tensor-memory GEMM for bf16 activations; for f32 activations the same GEMM on their hi + lo bf16
    // halves when the caller's workspace holds them; the tiled generic kernel otherwise
    const int64_t gforce = options().gemm_kernel.load();
    if (!xbf && gforce != 1 && !((uintptr_t)w & 15u) && !((uintptr_t)ws & 255u)) {
        const SplitPlan sp = plan_f32_split(scheme, m, k, n);
        if (sp.ok && ws && ws_bytes >= sp.bytes) {
            uint8_t* base = static_cast<uint8_t*>(ws);
            for (uint32_t r0 = 0; r0 < m; r0 += sp.chunk) {
                const uint32_t rows = m - r0 < sp.chunk ? m - r0 : sp.chunk;
                int rc = launch_split_hi_lo(stream, static_cast<const float*>(x) + (size_t)r0 * k, base, rows, k);
                if (rc) return rc;
                rc = launch_gemm_tc(stream, scheme, base, w, base + sp.off_y2, false, 2 * rows, k, n, base + sp.off_gemm,
                                    sp.bytes - sp.off_gemm);
                if (rc) return rc;
                rc = launch_add_halves(stream, reinterpret_cast<const float*>(base + sp.off_y2),
                                       static_cast<uint8_t*>(y) + (size_t)r0 * n * (ybf ? 2 : 4), ybf, rows, n);
                if (rc) return rc;
            }
            return RLXQ_OK;
        }
    }
    const bool can = gemm_tc_supported(scheme, m, k, n, w, x, xbf);
    if (gforce == 2 && !can)
        return fail(RLXQ_E_SHAPE, "the tcgen05 GEMM needs bf16 activations, k %% 256 == 0 (2048 for Q6_K), one of Q4_0/Q8_0/Q4_K/Q5_K/Q6_K and 16-byte alignment");
    if (can && gforce != 1) return launch_gemm_tc(stream, scheme, x, w, y, ybf, m, k, n, ws, ws_bytes);
    return launch_matmul_generic(stream, scheme, x, xbf, w, y, ybf, m, k, n);
}

}  // namespace rlxq
