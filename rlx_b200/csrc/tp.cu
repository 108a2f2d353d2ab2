// Tensor-parallel SwiGLU FFN pieces: the shard planner, the k-slice gather for the row-parallel
// down projection, and the per-rank forward pass  partial_y = down_r( up_r(x) * silu(gate_r(x)) ).
//
// The reference has no device-side parallelism at all (its collectives are host emulations,
// rlx-driver/src/collective.rs:79-128); the FFN composition is rlx-flow/src/blocks/swiglu.rs:48-52
// with silu from rlx-cpu/src/naive.rs:54-56.  Split: gate and up are column-parallel (rank r owns
// output rows [r*F/g, (r+1)*F/g) of W[F, D], one contiguous byte range), the product with silu is
// local, down is row-parallel (rank r owns k in [r*F/g, (r+1)*F/g) of every row of W[D, F], whole
// 256-weight groups), and the f32 partials [m, D] are summed across ranks by the caller's
// all-reduce (rank order 0..g-1 is the reference order, collective.rs:107-127).
#include <cstring>

#include "common.cuh"
#include "decode.cuh"
#include "host/session.hpp"
#include "kernels.h"
#include "tp_comm.cuh"
#include "../../include/rlxq_tp.h"

namespace rlxq {

// h[m, f] = up * silu(gate) where gu = [gate | up] per row: gu[m, 2f].  h is f32 for the decode
// path and bf16 (round to nearest even) when it feeds the tensor-core GEMM.
template <bool HBF16>
__global__ void __launch_bounds__(256) swiglu_pair_kernel(const float* __restrict__ gu, void* __restrict__ h,
                                                          uint32_t m, uint32_t f) {
    const uint64_t total = (uint64_t)m * f, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint64_t r = i / f, c = i - r * f;
        const float g = gu[r * 2 * f + c], u = gu[r * 2 * f + f + c];
        const float v = u * (g / (1.0f + expf(-g)));
        if (HBF16) reinterpret_cast<uint16_t*>(h)[i] = (uint16_t)f32_to_bf16_bits(v);
        else reinterpret_cast<float*>(h)[i] = v;
    }
}

// h[m, f] (f32) = up * silu(gate) of gu[m, 2f].
int launch_swiglu_pair(cudaStream_t stream, const float* gu, void* h, uint32_t m, uint32_t f) {
    const uint64_t total = (uint64_t)m * f;
    if (total == 0) return RLXQ_OK;
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    swiglu_pair_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(gu, h, m, f);
    count_launch();
    return check_launch("swiglu_pair_kernel");
}

}  // namespace rlxq

using namespace rlxq;

extern "C" {

int rlxq_tp_shard_plan(uint32_t scheme, uint32_t d_model, uint32_t d_ffn, uint32_t world, uint32_t rank,
                       rlxq_tp_shard* out) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (!out) return fail(RLXQ_E_NULL, "out is null");
    if (world == 0 || rank >= world) return fail(RLXQ_E_ARG, "rank %u of world %u", rank, world);
    if (d_model % g.elems || d_ffn % g.elems) return fail(RLXQ_E_SHAPE, "dimensions must be multiples of the block size %u", g.elems);
    // the row-parallel slice must hold whole 256-weight groups so that every rank's rows stay 16-byte aligned
    if (d_ffn % (256u * world)) return fail(RLXQ_E_SHAPE, "d_ffn=%u does not split into %u slices of whole 256-weight groups", d_ffn, world);
    const uint32_t f = d_ffn / world;
    out->ffn_local = f;
    out->ffn_begin = rank * f;
    out->gate_up_row_bytes = (uint64_t)d_model / g.elems * g.bytes;
    out->gate_up_byte_offset = (uint64_t)out->ffn_begin * out->gate_up_row_bytes;
    out->gate_up_bytes = (uint64_t)f * out->gate_up_row_bytes;
    out->down_row_bytes_full = (uint64_t)d_ffn / g.elems * g.bytes;
    out->down_row_bytes_local = (uint64_t)f / g.elems * g.bytes;
    out->down_row_byte_offset = (uint64_t)out->ffn_begin / g.elems * g.bytes;
    out->down_bytes = (uint64_t)d_model * out->down_row_bytes_local;
    return RLXQ_OK;
}

int rlxq_tp_slice_k_host(uint32_t scheme, const void* w_full, uint32_t n, uint32_t k, uint32_t k_begin,
                         uint32_t k_len, void* w_slice) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (k % g.elems || k_begin % g.elems || k_len % g.elems || (uint64_t)k_begin + k_len > k)
        return fail(RLXQ_E_SHAPE, "slice [%u, %u) of k=%u is not made of whole blocks", k_begin, k_begin + k_len, k);
    if (n == 0 || k_len == 0) return RLXQ_OK;
    if (!w_full || !w_slice) return fail(RLXQ_E_NULL, "null buffer");
    const size_t full = (size_t)k / g.elems * g.bytes, part = (size_t)k_len / g.elems * g.bytes;
    const size_t off = (size_t)k_begin / g.elems * g.bytes;
    const uint8_t* src = static_cast<const uint8_t*>(w_full);
    uint8_t* dst = static_cast<uint8_t*>(w_slice);
    for (uint32_t r = 0; r < n; ++r) memcpy(dst + (size_t)r * part, src + (size_t)r * full + off, part);
    return RLXQ_OK;
}

int rlxq_tp_ffn_workspace_bytes(uint32_t scheme_gate_up, uint32_t scheme_down, uint32_t m, uint32_t d_model,
                                uint32_t ffn_local, uint32_t x_dtype, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    size_t a = 0, b = 0;
    int rc = rlxq_workspace_bytes(scheme_gate_up, m, d_model, 2 * ffn_local, x_dtype, RLXQ_F32, &a);
    if (rc) return rc;
    rc = rlxq_workspace_bytes(scheme_down, m, ffn_local, d_model, RLXQ_F32, RLXQ_F32, &b);
    if (rc) return rc;
    const size_t mm = (a > b ? a : b);
    auto al = [](size_t v) { return (v + 255) / 256 * 256; };
    *bytes = al(mm) + al((size_t)m * 2 * ffn_local * 4) + al((size_t)m * ffn_local * 4);
    return RLXQ_OK;
}

// The per-rank forward pass.  tp (may be null): the group's exchange buffers; when the down projection runs on the
// integer GEMV it then pushes its tiles into them and finishes the sum itself, and *summed tells the caller so.
static int ffn_partial_impl(rlxq_stream_t stream, uint32_t scheme_gate_up, uint32_t scheme_down, const void* x,
                            uint32_t x_dtype, const void* gate_up_blocks, const void* down_blocks, float* y_partial,
                            uint32_t m, uint32_t d_model, uint32_t ffn_local, void* workspace, size_t workspace_bytes,
                            const TpPush* tp, bool* summed) {
    if (summed) *summed = false;
    size_t need = 0;
    int rc = rlxq_tp_ffn_workspace_bytes(scheme_gate_up, scheme_down, m, d_model, ffn_local, x_dtype, &need);
    if (rc) return rc;
    if (m == 0 || d_model == 0) return RLXQ_OK;
    if (!workspace || workspace_bytes < need) return fail(RLXQ_E_WORKSPACE, "FFN needs %zu workspace bytes, got %zu", need, workspace_bytes);
    if ((uintptr_t)workspace & 255u) return fail(RLXQ_E_ALIGN, "FFN workspace must be 256-byte aligned");
    auto al = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t a = 0, b = 0;
    rlxq_workspace_bytes(scheme_gate_up, m, d_model, 2 * ffn_local, x_dtype, RLXQ_F32, &a);
    rlxq_workspace_bytes(scheme_down, m, ffn_local, d_model, RLXQ_F32, RLXQ_F32, &b);
    const size_t mm = al(a > b ? a : b);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    float* gu = reinterpret_cast<float*>(ws + mm);
    void* h = ws + mm + al((size_t)m * 2 * ffn_local * 4);
    // prefill (m > 8): h goes to the tensor-core GEMM, which takes bf16 activations
    const bool h_bf16 = m > 8;
    // [gate_r ; up_r] are stored as one weight of 2*ffn_local rows: one matmul yields both
    rc = rlxq_matmul(stream, scheme_gate_up, x, x_dtype, gate_up_blocks, gu, RLXQ_F32, m, d_model, 2 * ffn_local, ws, mm);
    if (rc) return rc;
    // gu is [m, 2f] with gate in columns [0, f) and up in [f, 2f)
    if (options().gemv_kernel.load() == 0 &&
        ((m <= 2 && int_supported(scheme_down, m, ffn_local, d_model, down_blocks, gu)) ||
         (m >= 2 && m <= 8 && int_mma_supported(scheme_down, m, ffn_local, d_model, down_blocks, gu)))) {
        // decode: the down projection's activation quantiser forms up * silu(gate) itself
        const bool push = tp && (uint64_t)m * d_model <= tp->max_elems && int_push_supported(scheme_down);
        rc = launch_gemv_int_swiglu((cudaStream_t)stream, scheme_down, gu, (const uint8_t*)down_blocks, y_partial, false, m,
                                    ffn_local, d_model, ws, mm, push ? tp : nullptr);
        if (rc == RLXQ_OK && push && summed) *summed = true;
        return rc;
    }
    {
        const uint64_t total = (uint64_t)m * ffn_local;
        uint64_t blocks = (total + 255) / 256;
        const uint64_t cap = (uint64_t)sm_count() * 8;
        if (blocks > cap) blocks = cap;
        if (h_bf16) swiglu_pair_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(gu, h, m, ffn_local);
        else swiglu_pair_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(gu, h, m, ffn_local);
        count_launch();
        rc = check_launch("swiglu_pair_kernel");
        if (rc) return rc;
    }
    return rlxq_matmul(stream, scheme_down, h, h_bf16 ? RLXQ_BF16 : RLXQ_F32, down_blocks, y_partial, RLXQ_F32, m,
                       ffn_local, d_model, ws, mm);
}

int rlxq_tp_ffn_partial(rlxq_stream_t stream, uint32_t scheme_gate_up, uint32_t scheme_down, const void* x,
                        uint32_t x_dtype, const void* gate_up_blocks, const void* down_blocks, float* y_partial,
                        uint32_t m, uint32_t d_model, uint32_t ffn_local, void* workspace, size_t workspace_bytes) {
    return ffn_partial_impl(stream, scheme_gate_up, scheme_down, x, x_dtype, gate_up_blocks, down_blocks, y_partial, m,
                            d_model, ffn_local, workspace, workspace_bytes, nullptr, nullptr);
}

int rlxq_tp_ffn_step(rlxq_stream_t stream, uint32_t scheme_gate_up, uint32_t scheme_down, const void* x, uint32_t x_dtype,
                     const void* gate_up_blocks, const void* down_blocks, float* y, uint32_t m, uint32_t d_model,
                     uint32_t ffn_local, void* workspace, size_t workspace_bytes, uint32_t rank, uint32_t world,
                     void* const* bufs, uint32_t max_elems) {
    if (world < 1 || world > kCommMaxWorld || rank >= world) return fail(RLXQ_E_ARG, "bad rank %u of %u", rank, world);
    if (!bufs) return fail(RLXQ_E_NULL, "bufs is null");
    const uint64_t elems = (uint64_t)m * d_model;
    if (elems > max_elems || elems % 4) return fail(RLXQ_E_SHAPE, "m * d_model = %llu must be a multiple of 4 and at most %u", (unsigned long long)elems, max_elems);
    TpPush tp{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!bufs[r]) return fail(RLXQ_E_NULL, "buffer of rank %u is null", r);
        tp.buf[r] = static_cast<uint8_t*>(bufs[r]);
    }
    tp.world = world; tp.rank = rank; tp.max_elems = max_elems;
    tp.spin_limit = (uint32_t)options().tp_spin_limit.load();
    bool summed = false;
    int rc = ffn_partial_impl(stream, scheme_gate_up, scheme_down, x, x_dtype, gate_up_blocks, down_blocks, y, m, d_model,
                              ffn_local, workspace, workspace_bytes, options().tp_fused.load() ? &tp : nullptr, &summed);
    if (rc || summed || m == 0 || d_model == 0) return rc;
    return rlxq_tp_allreduce_sum(stream, rank, world, bufs, max_elems, y, y, (uint32_t)elems);
}

}  // extern "C"
