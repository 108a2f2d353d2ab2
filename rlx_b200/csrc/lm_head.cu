// Greedy / top-k selection over a GGUF-packed tied LM head.
//
// Replaces gguf_tied_lm_argmax (rlx-cpu/src/lm_head.rs:223-251) and gguf_tied_lm_topk (:172-199).
// logits = hidden . W^T is one batch-1 call of the streaming GEMV (the vocabulary is the output
// dimension: 128 k rows x 4096 columns of Q4_K is 295 MB, i.e. pure HBM streaming).  Selection:
//   lm_select_kernel  one CTA per 2048 logits keeps its C best (value desc, token id asc)
//   lm_merge_kernel   one CTA merges the (sorted) per-slice lists into the C best overall
//   lm_exact_kernel   (RLXQ_LM_EXACT) one CTA per candidate recomputes its logit exactly as the
//                     reference does: f32 products in column order, multiply and add rounded
//                     separately (row_dot_gguf, lm_head.rs:46-76), decoders bit-exact
//   lm_final_kernel   ranks the C candidates by the (exact) values and writes the first `cap`
// C = cap + 8 spare candidates, so the exact re-ranking can repair any reordering the GEMV's
// rounding (15-bit activations, different summation order) causes among near-equal logits.
#include <math_constants.h>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "rlxq_lm.h"
#include "staged_common.cuh"

namespace rlxq {

constexpr uint32_t kLmSlice = 2048;       // logits per CTA of the selection kernel
constexpr uint32_t kLmThreads = 256;
constexpr uint32_t kLmSpare = 8;          // candidates beyond cap
constexpr uint32_t kLmNone = 0xFFFFFFFFu; // "no token"
constexpr uint32_t kLmChunk = 4096;       // products staged per pass of the exact kernel

// Order-preserving map of f32 onto u32 (larger float <-> larger integer); NaN maps to 0, below -inf.
__device__ __forceinline__ uint32_t ord_of(float v) {
    if (!(v == v)) return 0u;
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord_to_float(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7FFFFFFFu) : ~o);
}

// Best (value desc, id asc) over the block of the per-thread candidates (ord, id); a thread with nothing
// to offer passes ord = 0.  Two warp-wide integer reductions (redux.sync) per warp, then every thread
// reads the eight warp results: one barrier per call, on alternating halves of `sh`.
struct Best { uint32_t ord, id; };
__device__ __forceinline__ Best block_best(uint32_t ord, uint32_t id, uint32_t (*sh)[2][kLmThreads / 32], uint32_t parity) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t wmax = __reduce_max_sync(0xFFFFFFFFu, ord);
    const uint32_t wid = __reduce_min_sync(0xFFFFFFFFu, ord == wmax ? id : kLmNone);
    if (lane == 0) { sh[parity][0][warp] = wmax; sh[parity][1][warp] = wid; }
    __syncthreads();
    Best b{0u, kLmNone};
#pragma unroll
    for (uint32_t w = 0; w < kLmThreads / 32; ++w) {
        const uint32_t o = sh[parity][0][w], i = sh[parity][1][w];
        if (o > b.ord || (o == b.ord && i < b.id)) b = Best{o, i};
    }
    if (b.ord == 0u) b.id = kLmNone;      // nothing selectable in the whole block
    return b;
}

__global__ void __launch_bounds__(kLmThreads) lm_select_kernel(const float* __restrict__ logits, uint32_t n,
                                                               uint32_t C, float* __restrict__ cv,
                                                               uint32_t* __restrict__ ci) {
    __shared__ uint32_t red[2][2][kLmThreads / 32];
    griddep_launch_dependents();      // the next small kernel may become resident already
    griddep_wait();                   // the logits come from the kernel in front
    const uint32_t base = blockIdx.x * kLmSlice;
    // eight logits per thread, in registers, as order-preserving integers (0 = cannot be chosen)
    uint32_t o[kLmSlice / kLmThreads];
#pragma unroll
    for (uint32_t r = 0; r < kLmSlice / kLmThreads; ++r) {
        const uint32_t j = base + r * kLmThreads + threadIdx.x;
        o[r] = j < n ? ord_of(logits[j]) : 0u;
    }
    for (uint32_t c = 0; c < C; ++c) {
        uint32_t bo = 0u, bi = kLmNone;
#pragma unroll
        for (uint32_t r = 0; r < kLmSlice / kLmThreads; ++r)      // ids grow with r: '>' keeps the lowest id of equals
            if (o[r] > bo) { bo = o[r]; bi = base + r * kLmThreads + threadIdx.x; }
        const Best b = block_best(bo, bi, red, c & 1u);
        if (threadIdx.x == 0) {
            cv[blockIdx.x * C + c] = b.id != kLmNone ? ord_to_float(b.ord) : -CUDART_INF_F;
            ci[blockIdx.x * C + c] = b.id;
        }
        if (b.id != kLmNone && bi == b.id) {                      // the owner retires it
#pragma unroll
            for (uint32_t r = 0; r < kLmSlice / kLmThreads; ++r)
                if (base + r * kLmThreads + threadIdx.x == b.id) o[r] = 0u;
        }
    }
}

constexpr uint32_t kLmMaxLists = 2048;      // per-slice lists the merge kernel tracks (2048 * 2048 = 4 M tokens)

// a before b: larger value, then smaller token id.  NaN is never before anything.
__device__ __forceinline__ bool before(float av, uint32_t ai, float bv, uint32_t bi) {
    return av > bv || (av == bv && ai < bi);
}

// Merges the per-slice lists (each sorted best first) into the C best overall: a C-step merge over the
// list heads, which live in shared memory; only the list a winner came from reads a new head.
__global__ void __launch_bounds__(kLmThreads) lm_merge_kernel(const float* __restrict__ cv, const uint32_t* __restrict__ ci,
                                                              uint32_t nlists, uint32_t C, float* __restrict__ sv,
                                                              uint32_t* __restrict__ si) {
    __shared__ uint32_t red[2][2][kLmThreads / 32];
    __shared__ uint32_t ho[kLmMaxLists], hi[kLmMaxLists], hp[kLmMaxLists];   // head: ord, token id, position
    griddep_launch_dependents();
    griddep_wait();
    for (uint32_t s = threadIdx.x; s < nlists; s += kLmThreads) {
        const uint32_t id = ci[s * C];
        hp[s] = 0u;
        hi[s] = id;
        ho[s] = id != kLmNone ? ord_of(cv[s * C]) : 0u;
    }
    __syncthreads();
    for (uint32_t c = 0; c < C; ++c) {
        uint32_t bo = 0u, bi = kLmNone;
        for (uint32_t s = threadIdx.x; s < nlists; s += kLmThreads)      // ids grow with s
            if (ho[s] > bo) { bo = ho[s]; bi = hi[s]; }
        const Best b = block_best(bo, bi, red, c & 1u);
        if (threadIdx.x == 0) {
            sv[c] = b.id != kLmNone ? ord_to_float(b.ord) : -CUDART_INF_F;
            si[c] = b.id;
        }
        if (b.id != kLmNone) {
            const uint32_t s = b.id / kLmSlice;                           // the list this token came from
            if (threadIdx.x == (s % kLmThreads)) {
                const uint32_t pos = hp[s] + 1u;
                hp[s] = pos;
                const uint32_t id = pos < C ? ci[s * C + pos] : kLmNone;
                hi[s] = id;
                ho[s] = id != kLmNone ? ord_of(cv[s * C + pos]) : 0u;
            }
        }
        __syncthreads();
    }
}

template <uint32_t SCHEME>
__global__ void __launch_bounds__(kLmThreads) lm_exact_kernel(const void* __restrict__ hidden, uint32_t h_bf16,
                                                              const uint8_t* __restrict__ w, uint32_t k,
                                                              const uint32_t* __restrict__ si, float* __restrict__ ev) {
    constexpr uint32_t E = SchemeTraits<SCHEME>::kElems, B = SchemeTraits<SCHEME>::kBytes;
    __shared__ __align__(16) float prod[kLmChunk];
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t row = si[blockIdx.x];
    if (row == kLmNone) {
        if (threadIdx.x == 0) ev[blockIdx.x] = -CUDART_INF_F;
        return;
    }
    const uint8_t* wrow = w + (uint64_t)row * (k / E) * B;
    float acc = 0.0f;
    for (uint32_t base = 0; base < k; base += kLmChunk) {
        const uint32_t chunk = min(kLmChunk, k - base);                // a multiple of 32
#pragma unroll 4
        for (uint32_t q = threadIdx.x; q < chunk / 4; q += kLmThreads) {   // independent iterations: loads overlap
            const uint32_t e = base + 4 * q;
            const float4 wv = decode4_exact<SCHEME>(wrow + (uint64_t)(e / E) * B, e % E);
            float h[4];
            if (h_bf16) {
                const uint2 hb = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(hidden) + e);
                h[0] = __uint_as_float(hb.x << 16); h[1] = __uint_as_float(hb.x & 0xFFFF0000u);
                h[2] = __uint_as_float(hb.y << 16); h[3] = __uint_as_float(hb.y & 0xFFFF0000u);
            } else {
                const float4 hv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(hidden) + e);
                h[0] = hv.x; h[1] = hv.y; h[2] = hv.z; h[3] = hv.w;
            }
            prod[4 * q + 0] = __fmul_rn(h[0], wv.x);
            prod[4 * q + 1] = __fmul_rn(h[1], wv.y);
            prod[4 * q + 2] = __fmul_rn(h[2], wv.z);
            prod[4 * q + 3] = __fmul_rn(h[3], wv.w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // the reference's order: one running f32 sum over the columns.  A serial chain of adds:
            // the next 32 products are read from shared memory while the current 32 are added.
            const float4* pv = reinterpret_cast<const float4*>(prod);
            float4 cur[8], nxt[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = pv[i];
            for (uint32_t p = 0; p < chunk; p += 32) {
                if (p + 32 < chunk) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) nxt[i] = pv[(p + 32) / 4 + i];
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    acc = __fadd_rn(acc, cur[i].x);
                    acc = __fadd_rn(acc, cur[i].y);
                    acc = __fadd_rn(acc, cur[i].z);
                    acc = __fadd_rn(acc, cur[i].w);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) ev[blockIdx.x] = acc;
}

__global__ void __launch_bounds__(64) lm_final_kernel(const float* __restrict__ v, const uint32_t* __restrict__ si,
                                                      uint32_t C, uint32_t cap, uint32_t argmax_mode,
                                                      uint32_t* __restrict__ out_i, float* __restrict__ out_v) {
    const uint32_t t = threadIdx.x;
    griddep_launch_dependents();
    griddep_wait();
    if (t < cap) { out_i[t] = kLmNone; out_v[t] = -CUDART_INF_F; }
    __syncthreads();
    if (t < C) {
        const float mv = v[t];
        const uint32_t mi = si[t];
        if (mi != kLmNone && mv == mv) {
            uint32_t rank = 0;
            for (uint32_t j = 0; j < C; ++j) {
                const float ov = v[j];
                const uint32_t oi = si[j];
                if (oi != kLmNone && ov == ov && before(ov, oi, mv, mi)) ++rank;
            }
            if (rank < cap) { out_i[rank] = mi; out_v[rank] = mv; }
        }
    }
    __syncthreads();
    // the reference's greedy scan starts from (0, -inf) and only moves on a strictly larger logit
    if (argmax_mode && t == 0 && !(out_v[0] > -CUDART_INF_F)) { out_i[0] = 0u; out_v[0] = -CUDART_INF_F; }
}

struct LmPlan {
    uint32_t nslices, C;
    size_t off_cv, off_ci, off_sv, off_si, off_ev, off_mm, mm_bytes, total;
};

static LmPlan plan_lm(uint32_t scheme, uint32_t n_embd, uint32_t n_vocab, uint32_t x_dtype, uint32_t cap) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    LmPlan p{};
    p.nslices = (n_vocab + kLmSlice - 1) / kLmSlice;
    p.C = cap + kLmSpare;
    if (p.C > RLXQ_LM_MAX_CAP) p.C = RLXQ_LM_MAX_CAP;
    size_t off = up((size_t)n_vocab * 4);                       // logits first
    p.off_cv = off; off += up((size_t)p.nslices * p.C * 4);
    p.off_ci = off; off += up((size_t)p.nslices * p.C * 4);
    p.off_sv = off; off += up((size_t)p.C * 4);
    p.off_si = off; off += up((size_t)p.C * 4);
    p.off_ev = off; off += up((size_t)p.C * 4);
    p.off_mm = off;
    p.mm_bytes = matmul_workspace_bytes(scheme, 1, n_embd, n_vocab, x_dtype, RLXQ_F32);
    p.total = off + up(p.mm_bytes);
    return p;
}

template <uint32_t SCHEME>
static void launch_exact(cudaStream_t s, uint32_t C, const void* hidden, bool hbf, const uint8_t* w, uint32_t k,
                         const uint32_t* si, float* ev) {
    (void)launch_pdl(lm_exact_kernel<SCHEME>, dim3(C), dim3(kLmThreads), 0, s, hidden, hbf ? 1u : 0u, w, k, si, ev);
}

static int lm_run(cudaStream_t stream, uint32_t scheme, const void* hidden, uint32_t x_dtype, const void* w_blocks,
                  uint32_t n_embd, uint32_t n_vocab, uint32_t cap, uint32_t flags, bool argmax_mode, void* workspace,
                  size_t workspace_bytes, uint32_t* idx_out, float* val_out) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (n_embd == 0 || n_embd % g.elems) return fail(RLXQ_E_SHAPE, "n_embd=%u is not a positive multiple of the block size %u", n_embd, g.elems);
    if (n_vocab == 0) return fail(RLXQ_E_SHAPE, "n_vocab is zero");
    if (n_vocab > kLmMaxLists * kLmSlice) return fail(RLXQ_E_LIMIT, "n_vocab=%u beyond %u", n_vocab, kLmMaxLists * kLmSlice);
    if (cap == 0 || cap > RLXQ_LM_MAX_CAP || cap > n_vocab)
        return fail(RLXQ_E_ARG, "cap=%u must be in [1, min(%u, n_vocab)]", cap, RLXQ_LM_MAX_CAP);
    if (flags & ~(uint32_t)RLXQ_LM_EXACT) return fail(RLXQ_E_ARG, "unknown flags 0x%x", flags);
    if (!hidden || !w_blocks || !idx_out || !val_out || !workspace) return fail(RLXQ_E_NULL, "null buffer");
    if (((uintptr_t)hidden & 15u) || ((uintptr_t)workspace & 15u)) return fail(RLXQ_E_ALIGN, "hidden and workspace must be 16-byte aligned");
    if ((uintptr_t)w_blocks & 1u) return fail(RLXQ_E_ALIGN, "w_blocks must be 2-byte aligned");
    const LmPlan p = plan_lm(scheme, n_embd, n_vocab, x_dtype, cap);
    if (workspace_bytes < p.total)
        return fail(RLXQ_E_WORKSPACE, "LM head needs %zu workspace bytes, got %zu", p.total, workspace_bytes);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    float* logits = reinterpret_cast<float*>(ws);
    float* cv = reinterpret_cast<float*>(ws + p.off_cv);
    uint32_t* ci = reinterpret_cast<uint32_t*>(ws + p.off_ci);
    float* sv = reinterpret_cast<float*>(ws + p.off_sv);
    uint32_t* si = reinterpret_cast<uint32_t*>(ws + p.off_si);
    float* ev = reinterpret_cast<float*>(ws + p.off_ev);
    const bool hbf = x_dtype == RLXQ_BF16;
    const bool exact = (flags & RLXQ_LM_EXACT) != 0;
    const uint32_t C = exact ? p.C : cap;

    int rc = dispatch_matmul(stream, scheme, hidden, hbf, (const uint8_t*)w_blocks, logits, false, 1, n_embd, n_vocab,
                             p.mm_bytes ? ws + p.off_mm : nullptr, p.mm_bytes);
    if (rc) return rc;
    // programmatic dependent launch: each kernel is resident before its predecessor ends and orders
    // itself with griddepcontrol.wait, so the four small launches cost a microsecond each, not three
    rc = launch_pdl(lm_select_kernel, dim3(p.nslices), dim3(kLmThreads), 0, stream, (const float*)logits, n_vocab, C, cv, ci);
    if (rc) return rc;
    count_launch();
    rc = launch_pdl(lm_merge_kernel, dim3(1), dim3(kLmThreads), 0, stream, (const float*)cv, (const uint32_t*)ci, p.nslices, C, sv, si);
    if (rc) return rc;
    count_launch();
    if (exact) {
        const uint8_t* w = (const uint8_t*)w_blocks;
        switch (scheme) {
            case RLXQ_Q4_K: launch_exact<RLXQ_Q4_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q5_K: launch_exact<RLXQ_Q5_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q6_K: launch_exact<RLXQ_Q6_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q8_K: launch_exact<RLXQ_Q8_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q2_K: launch_exact<RLXQ_Q2_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q3_K: launch_exact<RLXQ_Q3_K>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q4_1: launch_exact<RLXQ_Q4_1>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q5_0: launch_exact<RLXQ_Q5_0>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q5_1: launch_exact<RLXQ_Q5_1>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q4_0: launch_exact<RLXQ_Q4_0>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            case RLXQ_Q8_0: launch_exact<RLXQ_Q8_0>(stream, C, hidden, hbf, w, n_embd, si, ev); break;
            default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
        }
        count_launch();
    }
    rc = launch_pdl(lm_final_kernel, dim3(1), dim3(64), 0, stream, (const float*)(exact ? ev : sv), (const uint32_t*)si, C, cap,
                    argmax_mode ? 1u : 0u, idx_out, val_out);
    if (rc) return rc;
    count_launch();
    return check_launch("lm_head kernels");
}

}  // namespace rlxq

using namespace rlxq;

extern "C" int rlxq_lm_head_workspace_bytes(uint32_t scheme, uint32_t n_embd, uint32_t n_vocab, uint32_t x_dtype,
                                            uint32_t cap, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (n_embd == 0 || n_embd % g.elems || n_vocab == 0) return fail(RLXQ_E_SHAPE, "bad LM head shape %u x %u", n_vocab, n_embd);
    if (cap == 0 || cap > RLXQ_LM_MAX_CAP) return fail(RLXQ_E_ARG, "cap=%u must be in [1, %u]", cap, RLXQ_LM_MAX_CAP);
    *bytes = plan_lm(scheme, n_embd, n_vocab, x_dtype, cap).total;
    return RLXQ_OK;
}

extern "C" int rlxq_lm_head_topk(rlxq_stream_t stream, uint32_t scheme, const void* hidden, uint32_t x_dtype,
                                 const void* w_blocks, uint32_t n_embd, uint32_t n_vocab, uint32_t cap, uint32_t flags,
                                 void* workspace, size_t workspace_bytes, uint32_t* idx_out, float* val_out) {
    return lm_run((cudaStream_t)stream, scheme, hidden, x_dtype, w_blocks, n_embd, n_vocab, cap, flags, false, workspace,
                  workspace_bytes, idx_out, val_out);
}

extern "C" int rlxq_lm_head_argmax(rlxq_stream_t stream, uint32_t scheme, const void* hidden, uint32_t x_dtype,
                                   const void* w_blocks, uint32_t n_embd, uint32_t n_vocab, uint32_t flags,
                                   void* workspace, size_t workspace_bytes, uint32_t* idx_out, float* val_out) {
    return lm_run((cudaStream_t)stream, scheme, hidden, x_dtype, w_blocks, n_embd, n_vocab, 1, flags, true, workspace,
                  workspace_bytes, idx_out, val_out);
}
