// Graph / Session / CompiledGraph for the quantized-matmul path, and their C handles.
#include "session.hpp"

#include <cstring>
#include <new>

#include "../../../include/rlxq_session.h"
#include "../../../include/rlxq_moe.h"
#include "../../../include/rlxq_tp.h"
#include "../common.cuh"
#include "../kernels.h"

namespace rlxq {

constexpr uint64_t kGraphIoLimit = 256u << 10;   // staged bytes up to which a captured graph carries its own I/O copies

static uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
static uint32_t dtype_size(uint32_t d) { return d == RLXQ_BF16 ? 2u : 4u; }

// ------------------------------------------------------------------ Graph
int Graph::input(const std::string& name, uint32_t m, uint32_t k, uint32_t dtype) {
    if (dtype != RLXQ_F32 && dtype != RLXQ_BF16) return fail(RLXQ_E_DTYPE, "input '%s': unknown dtype", name.c_str());
    Node nd;
    nd.op = OpKind::Input; nd.name = name; nd.rows = m; nd.cols = k; nd.dtype = dtype;
    nd.bytes = (uint64_t)m * k * dtype_size(dtype);
    nodes_.push_back(nd);
    return (int)nodes_.size() - 1;
}

int Graph::param(const std::string& name, uint64_t bytes) {
    Node nd;
    nd.op = OpKind::Param; nd.name = name; nd.bytes = bytes;
    nodes_.push_back(nd);
    return (int)nodes_.size() - 1;
}

int Graph::dequant_matmul(int x, int w, uint32_t scheme, uint32_t n, uint32_t out_dtype) {
    if (x < 0 || w < 0 || x >= (int)nodes_.size() || w >= (int)nodes_.size())
        return fail(RLXQ_E_ARG, "dequant_matmul: bad input node id");
    const Node& xn = nodes_[x];
    const Node& wn = nodes_[w];
    if (wn.op != OpKind::Param) return fail(RLXQ_E_ARG, "dequant_matmul: weight must be a U8 param node");
    if (xn.op == OpKind::Param) return fail(RLXQ_E_ARG, "dequant_matmul: x must be a value node");
    if (out_dtype != RLXQ_F32 && out_dtype != RLXQ_BF16) return fail(RLXQ_E_DTYPE, "dequant_matmul: unknown dtype");
    uint64_t need = 0;
    int rc = rlxq_packed_bytes(scheme, xn.cols, n, &need);   // also checks scheme and k % block
    if (rc) return rc;
    if (need != wn.bytes)
        return fail(RLXQ_E_SHAPE, "dequant_matmul: param '%s' holds %llu bytes, W[%u,%u] needs %llu",
                    wn.name.c_str(), (unsigned long long)wn.bytes, n, xn.cols, (unsigned long long)need);
    Node nd;
    nd.op = OpKind::DequantMatMul; nd.rows = xn.rows; nd.cols = n; nd.dtype = out_dtype; nd.scheme = scheme;
    nd.in0 = x; nd.in1 = w;
    nd.bytes = (uint64_t)nd.rows * n * dtype_size(out_dtype);
    nodes_.push_back(nd);
    return (int)nodes_.size() - 1;
}

int Graph::swiglu_mul(int gate, int up) {
    if (gate < 0 || up < 0 || gate >= (int)nodes_.size() || up >= (int)nodes_.size())
        return fail(RLXQ_E_ARG, "swiglu_mul: bad input node id");
    const Node& a = nodes_[gate];
    const Node& b = nodes_[up];
    if (a.op == OpKind::Param || b.op == OpKind::Param || a.dtype != RLXQ_F32 || b.dtype != RLXQ_F32)
        return fail(RLXQ_E_DTYPE, "swiglu_mul: operands must be f32 value nodes");
    if (a.rows != b.rows || a.cols != b.cols) return fail(RLXQ_E_SHAPE, "swiglu_mul: shape mismatch");
    Node nd;
    nd.op = OpKind::SwigluMul; nd.rows = a.rows; nd.cols = a.cols; nd.dtype = RLXQ_F32;
    nd.in0 = gate; nd.in1 = up; nd.bytes = (uint64_t)a.rows * a.cols * 4;
    nodes_.push_back(nd);
    return (int)nodes_.size() - 1;
}

// Op::DequantGroupedMatMul (rlx-ir/src/op.rs:860-871): inputs [x, packed expert stack, expert_idx].
int Graph::dequant_grouped_matmul(int x, int w, int idx, uint32_t scheme, uint32_t n, uint32_t num_experts) {
    const int nn = (int)nodes_.size();
    if (x < 0 || w < 0 || idx < 0 || x >= nn || w >= nn || idx >= nn)
        return fail(RLXQ_E_ARG, "dequant_grouped_matmul: bad input node id");
    const Node& xn = nodes_[x];
    const Node& wn = nodes_[w];
    const Node& in = nodes_[idx];
    if (wn.op != OpKind::Param) return fail(RLXQ_E_ARG, "dequant_grouped_matmul: weight must be a U8 param node");
    if (xn.op == OpKind::Param || in.op == OpKind::Param)
        return fail(RLXQ_E_ARG, "dequant_grouped_matmul: x and expert_idx must be value nodes");
    if (in.dtype != RLXQ_F32 || (uint64_t)in.rows * in.cols != xn.rows)
        return fail(RLXQ_E_SHAPE, "dequant_grouped_matmul: expert_idx must hold one f32 per row of x");
    if (num_experts == 0) return fail(RLXQ_E_ARG, "dequant_grouped_matmul: no experts");
    uint64_t slab = 0;
    int rc = rlxq_packed_bytes(scheme, xn.cols, n, &slab);
    if (rc) return rc;
    if (slab * num_experts != wn.bytes)
        return fail(RLXQ_E_SHAPE, "dequant_grouped_matmul: param '%s' holds %llu bytes, %u slabs of W[%u,%u] need %llu",
                    wn.name.c_str(), (unsigned long long)wn.bytes, num_experts, n, xn.cols,
                    (unsigned long long)(slab * num_experts));
    Node nd;
    nd.op = OpKind::DequantGroupedMatMul; nd.rows = xn.rows; nd.cols = n; nd.dtype = RLXQ_F32; nd.scheme = scheme;
    nd.in0 = x; nd.in1 = w; nd.in2 = idx; nd.experts = num_experts;
    nd.bytes = (uint64_t)nd.rows * n * 4;
    nodes_.push_back(nd);
    return (int)nodes_.size() - 1;
}

int Graph::set_output(int node) {
    if (node < 0 || node >= (int)nodes_.size() || nodes_[node].op == OpKind::Param)
        return fail(RLXQ_E_ARG, "set_output: bad node id");
    output_ = node;
    return RLXQ_OK;
}

// The SwiGLU FFN pattern (rlx-flow/src/blocks/swiglu.rs:48-52; the reference's CUDA backend fuses the product as
// `FusedSwiGLU`, rlx-cuda/src/unfuse.rs:254-293): gate = dequant_matmul(x, Wg), up = dequant_matmul(x, Wu) on the same x
// with the same scheme and width, h = swiglu_mul(gate, up), y = dequant_matmul(h, Wd), all f32, none of the three
// intermediate values read by anything else or returned.
void CompiledGraph::find_fused_ffns() {
    const int nn = (int)nodes_.size();
    fused_role_.assign(nn, -1);
    fused_index_.assign(nn, -1);
    if (!options().graph_fuse_ffn.load()) return;
    std::vector<int> uses(nn, 0);
    for (const Node& nd : nodes_)
        for (int in : {nd.in0, nd.in1, nd.in2})
            if (in >= 0) ++uses[in];
    if (output_ >= 0) ++uses[output_];
    for (int d = 0; d < nn; ++d) {
        const Node& dn = nodes_[d];
        if (dn.op != OpKind::DequantMatMul || dn.dtype != RLXQ_F32 || dn.in0 < 0) continue;
        const int s = dn.in0;
        const Node& sn = nodes_[s];
        if (sn.op != OpKind::SwigluMul || uses[s] != 1 || fused_role_[s] != -1) continue;
        const int gm = sn.in0, um = sn.in1;
        const Node& gn = nodes_[gm];
        const Node& un = nodes_[um];
        if (gm == um || gn.op != OpKind::DequantMatMul || un.op != OpKind::DequantMatMul) continue;
        if (uses[gm] != 1 || uses[um] != 1 || fused_role_[gm] != -1 || fused_role_[um] != -1) continue;
        if (gn.in0 != un.in0 || gn.scheme != un.scheme || gn.cols != un.cols || gn.dtype != RLXQ_F32 || un.dtype != RLXQ_F32) continue;
        if (gn.in1 == un.in1 || uses[gn.in1] != 1 || uses[un.in1] != 1) continue;     // the two weights become one stacked slot
        if (nodes_[gn.in1].bytes % 256) continue;                                      // up must start where gate ends, aligned
        fused_index_[d] = (int)fused_.size();
        fused_.push_back({gm, um, s, d});
        fused_role_[gm] = fused_role_[um] = fused_role_[s] = 0;
        fused_role_[d] = 1;
    }
}

// ------------------------------------------------------------------ Session::compile
int Session::compile(const Graph& g, ExecMode mode, CompiledGraph** out) {
    if (!out) return fail(RLXQ_E_NULL, "out is null");
    *out = nullptr;
    if (g.output() < 0) return fail(RLXQ_E_ARG, "graph '%s' has no output", g.name().c_str());
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
        (void)cudaGetLastError();
        // Session::new(Device::Cuda) asserts availability (rlx-runtime/src/session.rs:48-55)
        return fail(RLXQ_E_CUDA, "no CUDA device available: Device::Cuda sessions cannot be created");
    }
    if (device_ < 0 || device_ >= ndev) return fail(RLXQ_E_ARG, "device %d out of range (%d devices)", device_, ndev);
    RLXQ_CUDA_TRY(cudaSetDevice(device_));
    int rc = staged_prepare_device();
    if (rc) return rc;

    CompiledGraph* c = new (std::nothrow) CompiledGraph();
    if (!c) return fail(RLXQ_E_CUDA, "out of host memory");
    c->device_ = device_;
    c->mode_ = mode;
    c->nodes_ = g.nodes();
    c->output_ = g.output();
    c->find_fused_ffns();
    // a fused FFN reads [gate rows ; up rows] as one weight: the up param's slot follows the gate param's directly
    std::vector<int> follows(c->nodes_.size(), -1);       // node -> the node whose slot it must follow
    std::vector<char> deferred(c->nodes_.size(), 0);
    for (const auto& f : c->fused_) {
        const int wg = c->nodes_[f.gate_mm].in1, wu = c->nodes_[f.up_mm].in1;
        follows[wu] = wg;
        deferred[wu] = 1;
    }
    uint64_t off = 0, ws = 0, stage = 0;
    c->offsets_.assign(c->nodes_.size(), 0);
    for (size_t ni = 0; ni < c->nodes_.size(); ++ni) {
        const Node& nd = c->nodes_[ni];
        if (deferred[ni]) continue;                        // placed right behind its gate param below
        c->offsets_[ni] = off;
        off += align_up(nd.bytes ? nd.bytes : 1, 256);
        for (size_t nj = 0; nj < c->nodes_.size(); ++nj)
            if (follows[nj] == (int)ni) {
                c->offsets_[nj] = c->offsets_[ni] + nd.bytes;      // nd.bytes is a multiple of 256 (checked when fusing)
                off = c->offsets_[nj] + align_up(c->nodes_[nj].bytes ? c->nodes_[nj].bytes : 1, 256);
            }
    }
    for (size_t ni = 0; ni < c->nodes_.size(); ++ni) {
        const Node& nd = c->nodes_[ni];
        if (c->fused_role_[ni] == 1) {
            const auto& f = c->fused_[c->fused_index_[ni]];
            const Node& gn = c->nodes_[f.gate_mm];
            const Node& xn = c->nodes_[gn.in0];
            size_t need = 0;
            rc = rlxq_tp_ffn_workspace_bytes(gn.scheme, nd.scheme, nd.rows, xn.cols, gn.cols, xn.dtype, &need);
            if (rc) { delete c; return rc; }
            if (need > ws) ws = need;
        }
        if (nd.op == OpKind::DequantMatMul && c->fused_role_[ni] == -1) {
            size_t need = 0;
            const Node& xn = c->nodes_[nd.in0];
            rc = rlxq_workspace_bytes(nd.scheme, nd.rows, xn.cols, nd.cols, xn.dtype, nd.dtype, &need);
            if (rc) { delete c; return rc; }
            if (need > ws) ws = need;
        }
        if (nd.op == OpKind::DequantGroupedMatMul) {
            size_t need = 0;
            rc = rlxq_grouped_workspace_bytes(nd.scheme, nd.rows, c->nodes_[nd.in0].cols, nd.cols, nd.experts, &need);
            if (rc) { delete c; return rc; }
            if (need > ws) ws = need;
        }
        if (nd.op == OpKind::Input) stage += align_up(nd.bytes, 256);
    }
    stage += align_up(c->nodes_[c->output_].bytes, 256);
    c->ws_off_ = off;
    c->ws_bytes_ = ws;
    c->arena_bytes_ = off + align_up(ws, 256);
    cudaError_t e = cudaMalloc((void**)&c->arena_, c->arena_bytes_);
    if (e != cudaSuccess) { delete c; return fail(RLXQ_E_CUDA, "arena cudaMalloc(%llu): %s", (unsigned long long)c->arena_bytes_, cudaGetErrorString(e)); }
    e = cudaMemset(c->arena_, 0, c->arena_bytes_);   // Arena::from_plan uses alloc_zeros
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream_, cudaStreamNonBlocking);
    if (e == cudaSuccess) { c->pinned_bytes_ = stage; e = cudaHostAlloc(&c->pinned_, stage, cudaHostAllocDefault); }
    if (e != cudaSuccess) { delete c; return fail(RLXQ_E_CUDA, "compile: %s", cudaGetErrorString(e)); }

    if (mode == ExecMode::Graph) {
        // Small inputs and outputs travel inside the captured graph, through the pinned staging buffer:
        // a run is then one graph launch and one synchronize instead of five driver calls, which matters
        // when the kernels of a decode step last 20 us.  Large tensors keep their direct copies (a host
        // memcpy into the staging buffer would cost more than the calls it saves).
        c->io_in_graph_ = stage <= kGraphIoLimit;
        cudaGraph_t graph = nullptr;
        e = cudaStreamBeginCapture(c->stream_, cudaStreamCaptureModeThreadLocal);
        if (e == cudaSuccess) {
            uint64_t so = 0;
            if (c->io_in_graph_)
                for (size_t i = 0; i < c->nodes_.size() && e == cudaSuccess; ++i) {
                    const Node& nd = c->nodes_[i];
                    if (nd.op != OpKind::Input) continue;
                    if (nd.bytes && !rc) rc = launch_copy_bytes(c->stream_, c->arena_ + c->offsets_[i], (uint8_t*)c->pinned_ + so, nd.bytes);
                    so += align_up(nd.bytes, 256);
                }
            const uint64_t launches_before = g_launches.load(std::memory_order_relaxed);
            if (!rc) rc = c->enqueue_steps(c->stream_);
            const Node& on = c->nodes_[c->output_];
            if (c->io_in_graph_ && on.bytes && !rc)
                rc = launch_copy_bytes(c->stream_, (uint8_t*)c->pinned_ + so, c->arena_ + c->offsets_[c->output_], on.bytes);
            // what one replay of the captured graph launches (the I/O copy kernels are counted below)
            c->captured_launches_ = g_launches.load(std::memory_order_relaxed) - launches_before;
            cudaError_t e2 = cudaStreamEndCapture(c->stream_, &graph);
            if (e == cudaSuccess) e = e2;
            if (rc) { if (graph) cudaGraphDestroy(graph); delete c; return rc; }
        }
        if (e == cudaSuccess) e = cudaGraphInstantiate(&c->graph_exec_, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        if (e != cudaSuccess) { delete c; return fail(RLXQ_E_CUDA, "graph capture: %s", cudaGetErrorString(e)); }
    }
    *out = c;
    return RLXQ_OK;
}

CompiledGraph::~CompiledGraph() {
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    if (stream_) cudaStreamDestroy(stream_);
    if (pinned_) cudaFreeHost(pinned_);
    if (arena_) cudaFree(arena_);
}

int CompiledGraph::enqueue_steps(cudaStream_t s) {
    for (size_t i = 0; i < nodes_.size(); ++i) {
        const Node& nd = nodes_[i];
        if (fused_role_[i] == 0) continue;          // computed inside the fused FFN below
        if (fused_role_[i] == 1) {
            const FusedFfn& f = fused_[fused_index_[i]];
            const Node& gn = nodes_[f.gate_mm];
            const Node& xn = nodes_[gn.in0];
            int rc = rlxq_tp_ffn_partial((rlxq_stream_t)s, gn.scheme, nd.scheme, arena_ + offsets_[gn.in0], xn.dtype,
                                         arena_ + offsets_[gn.in1], arena_ + offsets_[nd.in1], (float*)(arena_ + offsets_[i]),
                                         nd.rows, xn.cols, gn.cols, arena_ + ws_off_, ws_bytes_);
            if (rc) return rc;
            continue;
        }
        if (nd.op == OpKind::DequantMatMul) {
            const Node& xn = nodes_[nd.in0];
            int rc = rlxq_matmul((rlxq_stream_t)s, nd.scheme, arena_ + offsets_[nd.in0], xn.dtype,
                                 arena_ + offsets_[nd.in1], arena_ + offsets_[i], nd.dtype, nd.rows,
                                 xn.cols, nd.cols, ws_bytes_ ? arena_ + ws_off_ : nullptr, ws_bytes_);
            if (rc) return rc;
        } else if (nd.op == OpKind::DequantGroupedMatMul) {
            const Node& xn = nodes_[nd.in0];
            int rc = rlxq_grouped_matmul((rlxq_stream_t)s, nd.scheme, arena_ + offsets_[nd.in0], xn.dtype,
                                         arena_ + offsets_[nd.in1], (const float*)(arena_ + offsets_[nd.in2]),
                                         arena_ + offsets_[i], nd.dtype, nd.rows, xn.cols, nd.cols, nd.experts,
                                         arena_ + ws_off_, ws_bytes_);
            if (rc) return rc;
        } else if (nd.op == OpKind::SwigluMul) {
            int rc = launch_swiglu_mul(s, (const float*)(arena_ + offsets_[nd.in0]),
                                       (const float*)(arena_ + offsets_[nd.in1]),
                                       (float*)(arena_ + offsets_[i]), (uint64_t)nd.rows * nd.cols);
            if (rc) return rc;
        }
    }
    return RLXQ_OK;
}

int CompiledGraph::set_param_typed(const std::string& name, const void* data, uint64_t len) {
    for (size_t i = 0; i < nodes_.size(); ++i) {
        if (nodes_[i].op == OpKind::Param && nodes_[i].name == name) {
            if (len != nodes_[i].bytes)
                return fail(RLXQ_E_SHAPE, "set_param_typed('%s'): %llu bytes given, %llu declared", name.c_str(),
                            (unsigned long long)len, (unsigned long long)nodes_[i].bytes);
            if (len && !data) return fail(RLXQ_E_NULL, "set_param_typed: data is null");
            RLXQ_CUDA_TRY(cudaSetDevice(device_));
            RLXQ_CUDA_TRY(cudaMemcpyAsync(arena_ + offsets_[i], data, len, cudaMemcpyHostToDevice, stream_));
            RLXQ_CUDA_TRY(cudaStreamSynchronize(stream_));
            return RLXQ_OK;
        }
    }
    return fail(RLXQ_E_ARG, "set_param_typed: no param named '%s'", name.c_str());
}

int CompiledGraph::clear_scratch() {
    RLXQ_CUDA_TRY(cudaSetDevice(device_));
    if (ws_bytes_) RLXQ_CUDA_TRY(cudaMemsetAsync(arena_ + ws_off_, 0, arena_bytes_ - ws_off_, stream_));
    RLXQ_CUDA_TRY(cudaStreamSynchronize(stream_));
    return RLXQ_OK;
}

static bool is_pinned(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}

int CompiledGraph::run_typed(uint32_t n_inputs, const char* const* names, const void* const* data,
                             const uint64_t* bytes, const uint32_t* dtypes, void* out, uint64_t out_bytes,
                             uint32_t out_dtype) {
    RLXQ_CUDA_TRY(cudaSetDevice(device_));
    const Node& on = nodes_[output_];
    if (out_dtype != on.dtype) return fail(RLXQ_E_DTYPE, "run: output node is declared with another dtype");
    if (out_bytes != on.bytes) return fail(RLXQ_E_SHAPE, "run: output holds %llu bytes, %llu given",
                                           (unsigned long long)on.bytes, (unsigned long long)out_bytes);
    if (on.bytes && !out) return fail(RLXQ_E_NULL, "run: out is null");
    uint64_t stage_off = 0;
    uint32_t bound = 0;
    for (size_t i = 0; i < nodes_.size(); ++i) {
        const Node& nd = nodes_[i];
        if (nd.op != OpKind::Input) continue;
        int found = -1;
        for (uint32_t j = 0; j < n_inputs; ++j)
            if (names[j] && nd.name == names[j]) found = (int)j;
        if (found < 0) return fail(RLXQ_E_ARG, "run: input '%s' not supplied", nd.name.c_str());
        if (dtypes[found] != nd.dtype) return fail(RLXQ_E_DTYPE, "run: input '%s' dtype differs from the graph's", nd.name.c_str());
        if (bytes[found] != nd.bytes) return fail(RLXQ_E_SHAPE, "run: input '%s' has %llu bytes, graph expects %llu",
                                                  nd.name.c_str(), (unsigned long long)bytes[found], (unsigned long long)nd.bytes);
        const void* src = data[found];
        if (nd.bytes && !src) return fail(RLXQ_E_NULL, "run: input '%s' is null", nd.name.c_str());
        if (io_in_graph_) {                  // the captured graph copies from the staging buffer
            if (nd.bytes) memcpy((uint8_t*)pinned_ + stage_off, src, nd.bytes);
            stage_off += align_up(nd.bytes, 256);
            ++bound;
            continue;
        }
        if (nd.bytes && !is_pinned(src)) {   // pageable: stage through pinned memory so the copy is async
            memcpy((uint8_t*)pinned_ + stage_off, src, nd.bytes);
            src = (uint8_t*)pinned_ + stage_off;
        }
        stage_off += align_up(nd.bytes, 256);
        if (nd.bytes) RLXQ_CUDA_TRY(cudaMemcpyAsync(arena_ + offsets_[i], src, nd.bytes, cudaMemcpyHostToDevice, stream_));
        ++bound;
    }
    if (bound != n_inputs) return fail(RLXQ_E_ARG, "run: %u inputs supplied, graph has %u", n_inputs, bound);
    if (mode_ == ExecMode::Graph) {
        RLXQ_CUDA_TRY(cudaGraphLaunch(graph_exec_, stream_));
        // the captured launches were counted at capture time; count the replays too
        count_launch(captured_launches_);
    } else {
        int rc = enqueue_steps(stream_);
        if (rc) return rc;
    }
    if (io_in_graph_) {
        RLXQ_CUDA_TRY(cudaStreamSynchronize(stream_));
        if (on.bytes) memcpy(out, (uint8_t*)pinned_ + stage_off, on.bytes);
        return RLXQ_OK;
    }
    void* dst = out;
    const bool direct = !on.bytes || is_pinned(out);
    if (!direct) dst = (uint8_t*)pinned_ + stage_off;
    if (on.bytes) RLXQ_CUDA_TRY(cudaMemcpyAsync(dst, arena_ + offsets_[output_], on.bytes, cudaMemcpyDeviceToHost, stream_));
    RLXQ_CUDA_TRY(cudaStreamSynchronize(stream_));
    if (!direct) memcpy(out, dst, on.bytes);
    return RLXQ_OK;
}

}  // namespace rlxq

// ------------------------------------------------------------------ C handles
using namespace rlxq;

struct rlxq_graph { Graph g; explicit rlxq_graph(const char* n) : g(n ? n : "") {} };
struct rlxq_compiled { CompiledGraph* c; };

extern "C" {

rlxq_graph* rlxq_graph_new(const char* name) { return new (std::nothrow) rlxq_graph(name); }
void rlxq_graph_free(rlxq_graph* g) { delete g; }

int rlxq_graph_input(rlxq_graph* g, const char* name, uint32_t m, uint32_t k, uint32_t dtype) {
    if (!g || !name) return fail(RLXQ_E_NULL, "null argument");
    return g->g.input(name, m, k, dtype);
}
int rlxq_graph_param_u8(rlxq_graph* g, const char* name, uint64_t bytes) {
    if (!g || !name) return fail(RLXQ_E_NULL, "null argument");
    return g->g.param(name, bytes);
}
int rlxq_graph_dequant_matmul(rlxq_graph* g, int x_node, int w_node, uint32_t scheme, uint32_t n, uint32_t out_dtype) {
    if (!g) return fail(RLXQ_E_NULL, "null argument");
    return g->g.dequant_matmul(x_node, w_node, scheme, n, out_dtype);
}
int rlxq_graph_swiglu_mul(rlxq_graph* g, int gate_node, int up_node) {
    if (!g) return fail(RLXQ_E_NULL, "null argument");
    return g->g.swiglu_mul(gate_node, up_node);
}
int rlxq_graph_dequant_grouped_matmul(rlxq_graph* g, int x_node, int w_node, int expert_idx_node, uint32_t scheme,
                                      uint32_t n, uint32_t num_experts) {
    if (!g) return fail(RLXQ_E_NULL, "null argument");
    return g->g.dequant_grouped_matmul(x_node, w_node, expert_idx_node, scheme, n, num_experts);
}
int rlxq_graph_set_output(rlxq_graph* g, int node) {
    if (!g) return fail(RLXQ_E_NULL, "null argument");
    return g->g.set_output(node);
}

int rlxq_session_compile(const rlxq_graph* g, int device, int exec_mode, rlxq_compiled** out) {
    if (!g || !out) return fail(RLXQ_E_NULL, "null argument");
    *out = nullptr;
    if (exec_mode != 0 && exec_mode != 1) return fail(RLXQ_E_ARG, "unknown exec mode %d", exec_mode);
    CompiledGraph* c = nullptr;
    Session s(device);
    int rc = s.compile(g->g, exec_mode ? ExecMode::Graph : ExecMode::Stream, &c);
    if (rc) return rc;
    rlxq_compiled* h = new (std::nothrow) rlxq_compiled{c};
    if (!h) { delete c; return fail(RLXQ_E_CUDA, "out of host memory"); }
    *out = h;
    return RLXQ_OK;
}
void rlxq_compiled_free(rlxq_compiled* c) { if (c) { delete c->c; delete c; } }

int rlxq_compiled_set_param_typed(rlxq_compiled* c, const char* name, const void* data, uint64_t len) {
    if (!c || !name) return fail(RLXQ_E_NULL, "null argument");
    return c->c->set_param_typed(name, data, len);
}

int rlxq_compiled_run(rlxq_compiled* c, uint32_t n_inputs, const char* const* names, const float* const* data,
                      const uint64_t* elems, float* out, uint64_t out_elems) {
    if (!c || (n_inputs && (!names || !data || !elems))) return fail(RLXQ_E_NULL, "null argument");
    if (n_inputs > 16) return fail(RLXQ_E_LIMIT, "at most 16 inputs");
    uint64_t bytes[16];
    uint32_t dts[16];
    const void* ptrs[16];
    for (uint32_t i = 0; i < n_inputs; ++i) { bytes[i] = elems[i] * 4; dts[i] = RLXQ_F32; ptrs[i] = data[i]; }
    return c->c->run_typed(n_inputs, names, ptrs, bytes, dts, out, out_elems * 4, RLXQ_F32);
}

int rlxq_compiled_run_typed(rlxq_compiled* c, uint32_t n_inputs, const char* const* names, const void* const* data,
                            const uint64_t* bytes, const uint32_t* dtypes, void* out, uint64_t out_bytes,
                            uint32_t out_dtype) {
    if (!c || (n_inputs && (!names || !data || !bytes || !dtypes))) return fail(RLXQ_E_NULL, "null argument");
    return c->c->run_typed(n_inputs, names, data, bytes, dtypes, out, out_bytes, out_dtype);
}

uint64_t rlxq_compiled_arena_bytes(const rlxq_compiled* c) { return c ? c->c->arena_bytes() : 0; }

uint32_t rlxq_compiled_fused_ffn_count(const rlxq_compiled* c) { return c ? c->c->fused_ffn_count() : 0; }

int rlxq_compiled_clear_scratch(rlxq_compiled* c) {
    if (!c) return fail(RLXQ_E_NULL, "null argument");
    return c->c->clear_scratch();
}

}  // extern "C"
