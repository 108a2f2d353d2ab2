// rlxq_matmul_chain: a chain of dependent matmuls (each layer's input is the previous layer's output, or the
// SwiGLU product of its [gate | up] halves) behind one call.  For batch 1-2 of the streaming formats the whole
// chain runs as one cooperative kernel (gemv_int.cu, gemv_chain_kernel); everything else runs layer by layer
// through the same kernels rlxq_matmul uses.  The reference executes such a chain as consecutive steps of its
// compiled graph (rlx-cuda/src/backend.rs:5366-5405 per step) with the SwiGLU product as its own fused step
// (rlx-cuda/src/unfuse.rs:254-293).
#include "common.cuh"
#include "kernels.h"
#include "../../include/rlxq.h"

namespace rlxq {

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

struct SeqPlan { size_t mm, off_a, off_b, off_h, bytes; };

// Scratch of the layer-by-layer path: the matmuls' own workspace, two alternating output buffers, one buffer for
// a SwiGLU product.
static SeqPlan plan_sequential(uint32_t scheme, const rlxq_chain_layer* L, uint32_t nl, uint32_t m, uint32_t x_dtype) {
    SeqPlan p{};
    size_t ymax = 0, hmax = 0;
    for (uint32_t i = 0; i < nl; ++i) {
        const uint32_t xd = (i == 0 && !L[i].swiglu) ? x_dtype : (uint32_t)RLXQ_F32;
        const size_t w = matmul_workspace_bytes(scheme, m, L[i].k, L[i].n, xd, RLXQ_F32);
        p.mm = w > p.mm ? w : p.mm;
        if (i + 1 < nl) ymax = ymax > (size_t)m * L[i].n * 4 ? ymax : (size_t)m * L[i].n * 4;
        if (L[i].swiglu) hmax = hmax > (size_t)m * L[i].k * 4 ? hmax : (size_t)m * L[i].k * 4;
    }
    p.mm = up256(p.mm);
    p.off_a = p.mm;
    p.off_b = p.off_a + up256(ymax);
    p.off_h = p.off_b + up256(ymax);
    p.bytes = p.off_h + up256(hmax);
    return p;
}

static bool chain_layers(const rlxq_chain_layer* L, uint32_t nl, ChainLayer* out) {
    if (nl > 3) return false;
    for (uint32_t i = 0; i < nl; ++i) out[i] = ChainLayer{static_cast<const uint8_t*>(L[i].w_blocks), L[i].k, L[i].n, L[i].swiglu};
    return true;
}

}  // namespace rlxq

using namespace rlxq;

static int check_layers(uint32_t scheme, const rlxq_chain_layer* L, uint32_t nl) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (!L || nl == 0) return fail(RLXQ_E_NULL, "no layers");
    if (nl > 8) return fail(RLXQ_E_LIMIT, "at most 8 layers per chain");
    for (uint32_t i = 0; i < nl; ++i) {
        if (L[i].k == 0 || L[i].k % g.elems) return fail(RLXQ_E_SHAPE, "layer %u: k=%u is not a positive multiple of the block size %u", i, L[i].k, g.elems);
        if (L[i].n == 0) return fail(RLXQ_E_SHAPE, "layer %u: n is zero", i);
        if (i == 0 && L[i].swiglu) return fail(RLXQ_E_SHAPE, "the first layer has no [gate | up] input to combine");
        if (i > 0 && L[i - 1].n != (L[i].swiglu ? 2 * L[i].k : L[i].k))
            return fail(RLXQ_E_SHAPE, "layer %u takes %u values per row, layer %u yields %u", i, L[i].swiglu ? 2 * L[i].k : L[i].k, i - 1, L[i - 1].n);
    }
    return RLXQ_OK;
}

extern "C" int rlxq_chain_workspace_bytes(uint32_t scheme, const rlxq_chain_layer* layers, uint32_t nlayers, uint32_t m,
                                          uint32_t x_dtype, size_t* bytes) {
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    int rc = check_layers(scheme, layers, nlayers);
    if (rc) return rc;
    ChainLayer cl[3];
    size_t fused = 0;
    if (m >= 1 && m <= 2 && nlayers >= 2 && chain_layers(layers, nlayers, cl)) fused = chain_workspace_bytes(scheme, cl, nlayers, m);
    const size_t seq = plan_sequential(scheme, layers, nlayers, m, x_dtype).bytes;
    *bytes = fused > seq ? fused : seq;
    return RLXQ_OK;
}

extern "C" int rlxq_matmul_chain(rlxq_stream_t stream, uint32_t scheme, const rlxq_chain_layer* layers, uint32_t nlayers,
                                 const void* x, uint32_t x_dtype, void* y, uint32_t y_dtype, uint32_t m, void* workspace,
                                 size_t workspace_bytes) {
    int rc = check_layers(scheme, layers, nlayers);
    if (rc) return rc;
    if ((x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) || (y_dtype != RLXQ_F32 && y_dtype != RLXQ_BF16)) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (m == 0) return RLXQ_OK;
    if (!x || !y) return fail(RLXQ_E_NULL, "null buffer");
    for (uint32_t i = 0; i < nlayers; ++i)
        if (!layers[i].w_blocks) return fail(RLXQ_E_NULL, "layer %u: w_blocks is null", i);
    if ((uintptr_t)workspace & 255u) return fail(RLXQ_E_ALIGN, "chain workspace must be 256-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const bool xbf = x_dtype == RLXQ_BF16, ybf = y_dtype == RLXQ_BF16;
    // one cooperative kernel for the whole chain, when the shapes and the workspace allow it
    ChainLayer cl[3];
    if (options().gemv_chain.load() && m <= 2 && nlayers >= 2 && chain_layers(layers, nlayers, cl)) {
        bool aligned = ((uintptr_t)x & 15u) == 0;
        for (uint32_t i = 0; i < nlayers; ++i) aligned = aligned && ((uintptr_t)cl[i].w & 15u) == 0;
        const size_t need = aligned ? chain_workspace_bytes(scheme, cl, nlayers, m) : 0;
        if (need && workspace && workspace_bytes >= need) {
            rc = launch_gemv_chain(s, scheme, cl, nlayers, x, xbf, y, ybf, m, workspace, workspace_bytes);
            if (rc != RLXQ_E_SHAPE) return rc;        // a device whose grid cannot be co-resident: layer by layer below
        }
    }
    const SeqPlan sp = plan_sequential(scheme, layers, nlayers, m, x_dtype);
    if (!workspace || workspace_bytes < sp.bytes) return fail(RLXQ_E_WORKSPACE, "the chain needs %zu workspace bytes, got %zu", sp.bytes, workspace_bytes);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    const void* cur = x;
    bool cur_bf = xbf;
    for (uint32_t i = 0; i < nlayers; ++i) {
        const rlxq_chain_layer& Li = layers[i];
        const bool last = i + 1 == nlayers;
        void* out = last ? y : static_cast<void*>(base + ((i & 1u) ? sp.off_b : sp.off_a));
        if (Li.swiglu) {
            const uint8_t* w = static_cast<const uint8_t*>(Li.w_blocks);
            // decode sizes: the integer GEMV's activation quantiser forms up * silu(gate) itself
            if (options().gemv_kernel.load() == 0 &&
                ((m <= 2 && int_supported(scheme, m, Li.k, Li.n, w, cur)) ||
                 (m >= 2 && m <= 8 && int_mma_supported(scheme, m, Li.k, Li.n, w, cur)))) {
                rc = launch_gemv_int_swiglu(s, scheme, static_cast<const float*>(cur), w, out, last && ybf, m, Li.k, Li.n, base, sp.mm);
                if (rc) return rc;
                cur = out;
                cur_bf = false;
                continue;
            }
            rc = launch_swiglu_pair(s, static_cast<const float*>(cur), base + sp.off_h, m, Li.k);
            if (rc) return rc;
            cur = base + sp.off_h;
            cur_bf = false;
        }
        rc = dispatch_matmul(s, scheme, cur, cur_bf, static_cast<const uint8_t*>(Li.w_blocks), out, last && ybf, m, Li.k, Li.n, base, sp.mm);
        if (rc) return rc;
        cur = out;
        cur_bf = false;
    }
    return RLXQ_OK;
}
