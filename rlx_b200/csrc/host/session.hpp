// Host-side mirror of the reference's Graph / Session / CompiledGraph for the quantized-matmul
// path (C++; the reference's are Rust: rlx-ir/src/graph.rs, rlx-runtime/src/session.rs:42-87,
// rlx-runtime/src/compiled.rs:55-63,192-205, rlx-cuda/src/backend.rs:2327-2358,3923-3994).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace rlxq {

enum class OpKind { Input, Param, DequantMatMul, SwigluMul, DequantGroupedMatMul };

struct Node {
    OpKind op;
    std::string name;      // inputs and params only
    uint32_t rows = 0;     // m
    uint32_t cols = 0;     // k for inputs, n for compute nodes
    uint32_t dtype = 0;    // RLXQ_F32 / RLXQ_BF16 (element type of the node's value)
    uint32_t scheme = 0;   // DequantMatMul
    uint64_t bytes = 0;    // size of the node's device slot
    int in0 = -1, in1 = -1, in2 = -1;
    uint32_t experts = 0;  // DequantGroupedMatMul
};

class Graph {
public:
    explicit Graph(std::string name) : name_(std::move(name)) {}
    int input(const std::string& name, uint32_t m, uint32_t k, uint32_t dtype);
    int param(const std::string& name, uint64_t bytes);                    // Shape([bytes], U8)
    int dequant_matmul(int x, int w, uint32_t scheme, uint32_t n, uint32_t out_dtype);
    int swiglu_mul(int gate, int up);
    int dequant_grouped_matmul(int x, int w, int expert_idx, uint32_t scheme, uint32_t n, uint32_t num_experts);
    int set_output(int node);
    const std::vector<Node>& nodes() const { return nodes_; }
    int output() const { return output_; }
    const std::string& name() const { return name_; }

private:
    std::string name_;
    std::vector<Node> nodes_;
    int output_ = -1;
};

enum class ExecMode { Stream = 0, Graph = 1 };

class CompiledGraph {
public:
    ~CompiledGraph();
    CompiledGraph(const CompiledGraph&) = delete;
    CompiledGraph& operator=(const CompiledGraph&) = delete;

    int set_param_typed(const std::string& name, const void* data, uint64_t len);
    // inputs: host pointers to each named input in its declared dtype; out: host pointer
    int run_typed(uint32_t n_inputs, const char* const* names, const void* const* data,
                  const uint64_t* bytes, const uint32_t* dtypes, void* out, uint64_t out_bytes,
                  uint32_t out_dtype);
    uint64_t arena_bytes() const { return arena_bytes_; }
    int clear_scratch();
    uint32_t fused_ffn_count() const { return (uint32_t)fused_.size(); }

private:
    friend class Session;
    CompiledGraph() = default;
    int enqueue_steps(cudaStream_t s);
    void find_fused_ffns();

    // down(up(x) * silu(gate(x))) recognised at compile time and lowered to one stacked gate / up matmul, the
    // SwiGLU product formed inside the down projection's activation step, and the down projection.
    struct FusedFfn { int gate_mm, up_mm, swiglu, down_mm; };
    std::vector<FusedFfn> fused_;
    std::vector<int> fused_role_;     // per node: -1 not fused, 0 absorbed (nothing to launch), 1 the down matmul of fused_[idx]
    std::vector<int> fused_index_;

    int device_ = 0;
    ExecMode mode_ = ExecMode::Stream;
    std::vector<Node> nodes_;
    std::vector<uint64_t> offsets_;   // arena byte offset of every node's slot
    int output_ = -1;
    uint8_t* arena_ = nullptr;
    uint64_t arena_bytes_ = 0;
    uint64_t ws_off_ = 0, ws_bytes_ = 0;
    cudaStream_t stream_ = nullptr;
    cudaGraphExec_t graph_exec_ = nullptr;
    void* pinned_ = nullptr;          // staging for pageable host buffers
    uint64_t pinned_bytes_ = 0;
    uint64_t captured_launches_ = 0;  // Graph mode: kernels one replay of the captured graph launches
    bool io_in_graph_ = false;        // Graph mode, small I/O: the captured graph copies to and from pinned_
};

class Session {
public:
    explicit Session(int device) : device_(device) {}   // Session::new(Device::Cuda)
    int compile(const Graph& g, ExecMode mode, CompiledGraph** out);

private:
    int device_;
};

int launch_swiglu_mul(cudaStream_t stream, const float* gate, const float* up, float* out, uint64_t n);
int launch_copy_bytes(cudaStream_t stream, void* dst, const void* src, uint64_t bytes);

}  // namespace rlxq
