// Fused GGUF dequant + grouped matmul for MoE expert stacks (Op::DequantGroupedMatMul).
//
// Replaces the reference's host-sorted lowering (rlx-cuda/src/gguf_gpu.rs:142-280): D2H of x and the
// expert ids, counting sort on the CPU, per-expert dequantise + sgemm, H2D of the result.  Here:
//   moe_sort_kernel     one CTA: rows per expert (shared-memory atomics), exclusive scan, row
//                       permutation grouped by expert -- grouped_moe_sort_plan
//                       (rlx-cpu/src/gguf_matmul.rs:178-205) without the copy of x: the matmul
//                       kernel reads the rows through the permutation instead
//   moe_grouped_kernel  grid (weight-row tiles, experts): a warp owns one weight row of one expert,
//                       decodes it four weights per lane at a time (the bit-exact decoders) and
//                       multiplies it into up to eight of that expert's activation rows per pass;
//                       results go straight to the rows' original positions (the unpermute of
//                       grouped_moe_unpermute_out, gguf_matmul.rs:207-218, is the store address)
// Accumulation is f32 in a different order from the CPU loop; same tolerance as the general kernel.
//
// Prefill-sized batches (32 rows and more, the tensor-core GEMM's formats and shapes) go through the tcgen05
// GEMM in its grouped form instead of moe_grouped_kernel:
//   moe_tiles_kernel    the table of 128- or 256-row activation tiles, one list per expert, from the sorted offsets
//   moe_gather_kernel   the rows of every expert, gathered next to each other as bf16 (f32 activations as
//                       bf16 hi rows followed by the expert's lo rows, so nothing of x is lost)
//   gemm_tcgen05_kernel every tile against its expert's slab of the stack (gemm_tcgen05.cu, GemmParams::groups)
//   moe_scatter_kernel  results (hi + lo) to the rows' original positions
// The weight operand is bf16(d * q) there, as in the dense GEMM: same tolerance as that kernel.
//
// Decode (m <= 8 rows, Q4_0 / Q8_0 / Q4_K / Q6_K, k a multiple of 256 up to 12288) skips both kernels:
// every row is one launch of the streaming integer GEMV over the whole stack seen as an
// [experts * n, k] matrix, with the slab picked on the device from expert_idx[i] (gemv_int.cu,
// expert-indirect mode), so a routed expert's weights come through the TMA ring at GEMV speed.
#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "rlxq_moe.h"

namespace rlxq {

constexpr uint32_t kMoeInvalid = 0xFFFFFFFFu;

// offsets[0..E] (exclusive scan of the counts), perm[sorted position] = original row.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const float* __restrict__ expert_idx, uint32_t m, uint32_t E,
                                                        uint32_t* __restrict__ offsets, uint32_t* __restrict__ cursor,
                                                        uint32_t* __restrict__ perm) {
    extern __shared__ uint32_t cnt[];          // [E]
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0u;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
        uint32_t e;
        if (expert_of_row(expert_idx[i], E, &e)) atomicAdd(&cnt[e], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {                    // E is small (tens to hundreds): a serial scan is enough
        uint32_t run = 0;
        for (uint32_t e = 0; e < E; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += cnt[e];
        }
        offsets[E] = run;
    }
    __syncthreads();
    __threadfence_block();
    // cursor lives in global memory (this CTA is its only user); atomics hand out the slots
    for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) {
        uint32_t e;
        if (expert_of_row(expert_idx[i], E, &e)) perm[atomicAdd(&cursor[e], 1u)] = i;
    }
}

template <bool XBF16>
__device__ __forceinline__ float4 moe_load_x4(const void* x, uint64_t idx) {
    if constexpr (XBF16) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + idx);
        return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u),
                           __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
    } else {
        return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + idx);
    }
}

template <uint32_t SCHEME, bool XBF16, bool YBF16>
__global__ void __launch_bounds__(256) moe_grouped_kernel(const void* __restrict__ x, const uint8_t* __restrict__ w,
                                                          void* __restrict__ y, const uint32_t* __restrict__ offsets,
                                                          const uint32_t* __restrict__ perm, uint32_t k, uint32_t n) {
    constexpr uint32_t E = SchemeTraits<SCHEME>::kElems, B = SchemeTraits<SCHEME>::kBytes;
    constexpr int MT = 8;
    const uint32_t e = blockIdx.y;
    const uint32_t r0 = offsets[e], r1 = offsets[e + 1];
    if (r0 == r1) return;                                   // nobody routed here: the slab is never read
    const uint32_t lane = threadIdx.x & 31u, wpc = blockDim.x >> 5;
    const uint64_t row_bytes = (uint64_t)(k / E) * B;
    const uint8_t* slab = w + (uint64_t)e * n * row_bytes;
    for (uint32_t row = blockIdx.x * wpc + (threadIdx.x >> 5); row < n; row += gridDim.x * wpc) {
        const uint8_t* wr = slab + (uint64_t)row * row_bytes;
        for (uint32_t c0 = r0; c0 < r1; c0 += MT) {         // eight of the expert's rows per pass
            const uint32_t mt = min((uint32_t)MT, r1 - c0);
            uint32_t src[MT];
            float acc[MT];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                src[i] = (uint32_t)i < mt ? perm[c0 + i] : 0u;
                acc[i] = 0.f;
            }
            for (uint32_t el = lane * 4; el < k; el += 128) {
                const float4 wv = decode4_exact<SCHEME>(wr + (uint64_t)(el / E) * B, el % E);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    if ((uint32_t)i < mt) {
                        const float4 xv = moe_load_x4<XBF16>(x, (uint64_t)src[i] * k + el);
                        acc[i] = fmaf(wv.x, xv.x, acc[i]);
                        acc[i] = fmaf(wv.y, xv.y, acc[i]);
                        acc[i] = fmaf(wv.z, xv.z, acc[i]);
                        acc[i] = fmaf(wv.w, xv.w, acc[i]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < MT; ++i) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], o);
            }
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    if ((uint32_t)i < mt) {
                        const uint64_t o = (uint64_t)src[i] * n + row;
                        if constexpr (YBF16) reinterpret_cast<uint16_t*>(y)[o] = (uint16_t)f32_to_bf16_bits(acc[i]);
                        else reinterpret_cast<float*>(y)[o] = acc[i];
                    }
                }
            }
        }
    }
}

template <uint32_t SCHEME>
static void launch_grouped_s(cudaStream_t s, dim3 grid, bool xbf, bool ybf, const void* x, const uint8_t* w, void* y,
                             const uint32_t* offsets, const uint32_t* perm, uint32_t k, uint32_t n) {
    if (xbf && ybf) moe_grouped_kernel<SCHEME, true, true><<<grid, 256, 0, s>>>(x, w, y, offsets, perm, k, n);
    else if (xbf) moe_grouped_kernel<SCHEME, true, false><<<grid, 256, 0, s>>>(x, w, y, offsets, perm, k, n);
    else if (ybf) moe_grouped_kernel<SCHEME, false, true><<<grid, 256, 0, s>>>(x, w, y, offsets, perm, k, n);
    else moe_grouped_kernel<SCHEME, false, false><<<grid, 256, 0, s>>>(x, w, y, offsets, perm, k, n);
}

constexpr uint32_t kMoeDecodeRows = 8;      // up to this many rows go row by row through the streaming GEMV

// ---- prefill-sized batches on the tensor-core GEMM ------------------------------------------------------------

// activation rows per GEMM tile in grouped mode: 256 when the experts get about that many gathered rows each
// (a weight tile is then decoded once for all of them), else 128
static uint32_t moe_tile_rows(uint32_t gathered_rows, uint32_t E) { return gathered_rows / E >= 160u ? 256u : 128u; }
constexpr uint32_t kMoeTcMinRows = 32;      // smaller batches stay on moe_grouped_kernel

// table[t] = {first gathered row, rows, expert, 0} for the tiles in use, {0, 0, 0, 0} up to `bound`.
// mult = gathered rows per activation row (2 for f32 activations: hi and lo halves).
__global__ void moe_tiles_kernel(const uint32_t* __restrict__ offsets, uint32_t E, uint32_t mult, uint4* __restrict__ table,
                                 uint32_t bound, uint32_t tile_rows) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        uint32_t t = 0;
        for (uint32_t e = 0; e < E; ++e) {
            const uint32_t base = mult * offsets[e], rows = mult * (offsets[e + 1] - offsets[e]);
            for (uint32_t r = 0; r < rows && t < bound; r += tile_rows, ++t)
                table[t] = make_uint4(base + r, min(tile_rows, rows - r), e, 0u);
        }
        for (; t < bound; ++t) table[t] = make_uint4(0u, 0u, 0u, 0u);
    }
}

// One CTA per sorted position i: row perm[i] of x goes to row mult * offsets[e] + j of xg (j = position inside
// the expert's group), and for f32 activations its lo half to row mult * offsets[e] + count_e + j.
template <bool XBF16>
__global__ void __launch_bounds__(256) moe_gather_kernel(const void* __restrict__ x, const float* __restrict__ expert_idx,
                                                         const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ perm,
                                                         uint32_t E, uint32_t k, uint16_t* __restrict__ xg) {
    const uint32_t i = blockIdx.x;
    if (i >= offsets[E]) return;
    const uint32_t src = perm[i];
    uint32_t e = 0;
    expert_of_row(expert_idx[src], E, &e);
    const uint32_t j = i - offsets[e], cnt = offsets[e + 1] - offsets[e];
    if constexpr (XBF16) {
        const uint2* in = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + (size_t)src * k);
        uint2* out = reinterpret_cast<uint2*>(xg + (size_t)(offsets[e] + j) * k);
        for (uint32_t c = threadIdx.x; c < k / 4; c += blockDim.x) out[c] = in[c];
    } else {
        const float4* in = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)src * k);
        uint2* hi = reinterpret_cast<uint2*>(xg + (size_t)(2 * offsets[e] + j) * k);
        uint2* lo = reinterpret_cast<uint2*>(xg + (size_t)(2 * offsets[e] + cnt + j) * k);
        for (uint32_t c = threadIdx.x; c < k / 4; c += blockDim.x) {
            const float4 v = in[c];
            const float f[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[4], l[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                h[q] = f32_to_bf16_bits(f[q]) & 0xFFFFu;
                const float rest = f[q] - __uint_as_float(h[q] << 16);
                l[q] = f32_to_bf16_bits(isfinite(f[q]) ? rest : 0.f) & 0xFFFFu;
            }
            hi[c] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
            lo[c] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
        }
    }
}

// One CTA per sorted position: y[perm[i]] = y2[hi row] (+ y2[lo row]).
template <bool YBF16>
__global__ void __launch_bounds__(256) moe_scatter_kernel(const float* __restrict__ y2, const float* __restrict__ expert_idx,
                                                          const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ perm,
                                                          uint32_t E, uint32_t n, uint32_t mult, void* __restrict__ y) {
    const uint32_t i = blockIdx.x;
    if (i >= offsets[E]) return;
    const uint32_t dst = perm[i];
    uint32_t e = 0;
    expert_of_row(expert_idx[dst], E, &e);
    const uint32_t j = i - offsets[e], cnt = offsets[e + 1] - offsets[e];
    const float* a = y2 + (size_t)(mult * offsets[e] + j) * n;
    const float* b = a + (size_t)cnt * n;
    for (uint32_t c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = mult == 2 ? a[c] + b[c] : a[c];
        if constexpr (YBF16) reinterpret_cast<uint16_t*>(y)[(size_t)dst * n + c] = (uint16_t)f32_to_bf16_bits(v);
        else reinterpret_cast<float*>(y)[(size_t)dst * n + c] = v;
    }
}

struct MoeTcPlan { bool ok; uint32_t mult, rows, tiles, tile_rows; size_t off_table, off_xg, off_y2, bytes; };

// The scratch of the tensor-core path behind the sort's arrays (which end at `base`): tile table, gathered
// activations, result rows.  Not taken (ok = false) for small batches, other formats or shapes, or when it would
// need more than 4 GiB.
static MoeTcPlan plan_moe_tc(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t E, bool xbf, size_t base) {
    MoeTcPlan p{};
    if (m < kMoeTcMinRows || options().gemm_kernel.load() == 1) return p;
    if (!gemm_tc_supported(scheme, m, k, n, (const void*)256, (const void*)256, true)) return p;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    p.mult = xbf ? 1u : 2u;
    p.rows = p.mult * m;
    p.tile_rows = moe_tile_rows(p.rows, E);
    p.tiles = (p.rows + 127) / 128 + E;      // enough for either tile size
    p.off_table = up(base);
    p.off_xg = p.off_table + up((size_t)p.tiles * 16);
    p.off_y2 = p.off_xg + up((size_t)p.rows * k * 2);
    p.bytes = p.off_y2 + up((size_t)p.rows * n * 4);
    p.ok = p.bytes <= (4ull << 30) && (uint64_t)n * E <= 0x7FFFFFFFull;
    return p;
}

static size_t grouped_ws(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t E, bool xbf, size_t* off_cursor,
                         size_t* off_perm, MoeTcPlan* tc) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t off = up(((size_t)E + 1) * 4);
    if (off_cursor) *off_cursor = off;
    off += up((size_t)E * 4);
    if (off_perm) *off_perm = off;
    off += up((size_t)m * 4);
    const MoeTcPlan p = plan_moe_tc(scheme, m, k, n, E, xbf, off);
    if (tc) *tc = p;
    if (p.ok) off = p.bytes;
    const size_t gemv = m <= kMoeDecodeRows ? up(int_workspace_bytes(scheme, 1, k, n)) : 0;   // the decode path's scratch
    return off > gemv ? off : gemv;
}

}  // namespace rlxq

using namespace rlxq;

extern "C" int rlxq_grouped_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t num_experts,
                                            size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (k == 0 || k % g.elems) return fail(RLXQ_E_SHAPE, "k=%u is not a positive multiple of the block size %u", k, g.elems);
    if (num_experts == 0 || num_experts > 8192) return fail(RLXQ_E_LIMIT, "num_experts=%u must be in [1, 8192]", num_experts);
    // sized for f32 activations (two gathered rows per row); bf16 activations need less of it
    *bytes = grouped_ws(scheme, m, k, n, num_experts, false, nullptr, nullptr, nullptr);
    return RLXQ_OK;
}

extern "C" int rlxq_grouped_matmul(rlxq_stream_t stream, uint32_t scheme, const void* x, uint32_t x_dtype,
                                   const void* w_blocks, const float* expert_idx, void* y, uint32_t y_dtype, uint32_t m,
                                   uint32_t k, uint32_t n, uint32_t num_experts, void* workspace, size_t workspace_bytes) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if ((x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) || (y_dtype != RLXQ_F32 && y_dtype != RLXQ_BF16))
        return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (k == 0 || k % g.elems) return fail(RLXQ_E_SHAPE, "k=%u is not a positive multiple of the block size %u", k, g.elems);
    if (num_experts == 0 || num_experts > 8192) return fail(RLXQ_E_LIMIT, "num_experts=%u must be in [1, 8192]", num_experts);
    if (m == 0 || n == 0) return RLXQ_OK;
    if (!x || !w_blocks || !expert_idx || !y || !workspace) return fail(RLXQ_E_NULL, "null buffer");
    if (((uintptr_t)x & 15u) || ((uintptr_t)workspace & 15u)) return fail(RLXQ_E_ALIGN, "x and workspace must be 16-byte aligned");
    if ((uintptr_t)w_blocks & 1u) return fail(RLXQ_E_ALIGN, "w_blocks must be 2-byte aligned");
    if ((uintptr_t)y & (y_dtype == RLXQ_BF16 ? 1u : 3u)) return fail(RLXQ_E_ALIGN, "y must be aligned to its element size");
    size_t off_cursor = 0, off_perm = 0;
    const bool xbf = x_dtype == RLXQ_BF16, ybf = y_dtype == RLXQ_BF16;
    MoeTcPlan tc{};
    size_t need = grouped_ws(scheme, m, k, n, num_experts, xbf, &off_cursor, &off_perm, &tc);
    // the tensor-core path is taken when the workspace holds its arrays; a smaller one still runs the general kernel
    if (tc.ok && (workspace_bytes < tc.bytes || ((uintptr_t)workspace & 255u) || ((uintptr_t)w_blocks & 15u))) {
        tc.ok = false;
        need = off_perm + ((size_t)m * 4 + 255) / 256 * 256;
    }
    if (workspace_bytes < need) return fail(RLXQ_E_WORKSPACE, "grouped matmul needs %zu workspace bytes, got %zu", need, workspace_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    uint32_t* offsets = reinterpret_cast<uint32_t*>(ws);
    uint32_t* cursor = reinterpret_cast<uint32_t*>(ws + off_cursor);
    uint32_t* perm = reinterpret_cast<uint32_t*>(ws + off_perm);
    // rows with an id of num_experts or more are in no group: their outputs stay zero
    RLXQ_CUDA_TRY(cudaMemsetAsync(y, 0, (size_t)m * n * (ybf ? 2 : 4), s));
    const uint8_t* wst = (const uint8_t*)w_blocks;
    const size_t xes = xbf ? 2 : 4, yes = ybf ? 2 : 4;
    if (m <= kMoeDecodeRows && options().gemv_kernel.load() != 1 && ((size_t)k * xes) % 16 == 0 &&
        (uint64_t)n * num_experts <= 0x7FFFFFFFull && int_expert_supported(scheme, k, n, wst, x)) {
        for (uint32_t i = 0; i < m; ++i) {
            int rc = launch_gemv_int_expert(s, scheme, (const uint8_t*)x + (size_t)i * k * xes, xbf, wst,
                                            (uint8_t*)y + (size_t)i * n * yes, ybf, k, n, num_experts, expert_idx + i,
                                            workspace, workspace_bytes);
            if (rc) return rc;
        }
        return RLXQ_OK;
    }
    moe_sort_kernel<<<1, 1024, num_experts * sizeof(uint32_t), s>>>(expert_idx, m, num_experts, offsets, cursor, perm);
    count_launch();
    if (tc.ok) {
        uint4* table = reinterpret_cast<uint4*>(ws + tc.off_table);
        uint16_t* xg = reinterpret_cast<uint16_t*>(ws + tc.off_xg);
        float* y2 = reinterpret_cast<float*>(ws + tc.off_y2);
        moe_tiles_kernel<<<1, 32, 0, s>>>(offsets, num_experts, tc.mult, table, tc.tiles, tc.tile_rows);
        count_launch();
        if (xbf) moe_gather_kernel<true><<<m, 256, 0, s>>>(x, expert_idx, offsets, perm, num_experts, k, xg);
        else moe_gather_kernel<false><<<m, 256, 0, s>>>(x, expert_idx, offsets, perm, num_experts, k, xg);
        count_launch();
        int rc = check_launch("moe_gather_kernel");
        if (rc) return rc;
        rc = launch_gemm_grouped(s, scheme, xg, tc.rows, wst, num_experts, y2, k, n, table, tc.tiles, tc.tile_rows);
        if (rc) return rc;
        if (ybf) moe_scatter_kernel<true><<<m, 256, 0, s>>>(y2, expert_idx, offsets, perm, num_experts, n, tc.mult, y);
        else moe_scatter_kernel<false><<<m, 256, 0, s>>>(y2, expert_idx, offsets, perm, num_experts, n, tc.mult, y);
        count_launch();
        return check_launch("moe_scatter_kernel");
    }
    const uint32_t wpc = 8;
    unsigned gx = (n + wpc - 1) / wpc;
    const unsigned cap = (unsigned)sm_count() * 8;
    if (gx > cap) gx = cap;
    const dim3 grid(gx, num_experts);
    const uint8_t* w = (const uint8_t*)w_blocks;
    switch (scheme) {
        case RLXQ_Q4_K: launch_grouped_s<RLXQ_Q4_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q5_K: launch_grouped_s<RLXQ_Q5_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q6_K: launch_grouped_s<RLXQ_Q6_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q8_K: launch_grouped_s<RLXQ_Q8_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q2_K: launch_grouped_s<RLXQ_Q2_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q3_K: launch_grouped_s<RLXQ_Q3_K>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q4_1: launch_grouped_s<RLXQ_Q4_1>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q5_0: launch_grouped_s<RLXQ_Q5_0>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q5_1: launch_grouped_s<RLXQ_Q5_1>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q4_0: launch_grouped_s<RLXQ_Q4_0>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        case RLXQ_Q8_0: launch_grouped_s<RLXQ_Q8_0>(s, grid, xbf, ybf, x, w, y, offsets, perm, k, n); break;
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
    count_launch();
    return check_launch("moe_grouped_kernel");
}
