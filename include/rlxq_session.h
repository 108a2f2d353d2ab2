/*
 * rlxq_session — host-side mirror of the reference's Graph / Session / CompiledGraph API for
 * the quantized-matmul path, as plain C handles.
 *
 * The reference's user-facing contract on this path is (rlx-runtime/tests/dequant_matmul_gguf.rs:
 * 212-227): build a Graph with an input x, a U8 param holding the packed weight, and one
 * Op::DequantMatMul{scheme} node; Session::new(Device::Cuda).compile(g); set_param_typed(name,
 * bytes, DType::U8); run(&[("x", &x)]) -> Vec<Vec<f32>>.  The functions below are that contract
 * with C linkage; the C++ classes behind them (rlx_b200/csrc/host/session.hpp) carry the same
 * names.  Host pointers in, host pointers out: the calls copy to and from the device themselves,
 * like CudaExecutable::run (rlx-cuda/src/backend.rs:3976-3994, 6675-6693).
 */
#ifndef RLXQ_SESSION_H
#define RLXQ_SESSION_H

#include <stddef.h>
#include <stdint.h>

#include "rlxq.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rlxq_graph rlxq_graph;
typedef struct rlxq_compiled rlxq_compiled;

/* Graph::new(name) — rlx-ir/src/graph.rs.  Returns NULL on allocation failure. */
RLXQ_API rlxq_graph* rlxq_graph_new(const char* name);
RLXQ_API void rlxq_graph_free(rlxq_graph* g);

/* Graph::input(name, Shape[m,k], dtype) — returns the node id (>= 0) or a negative status.
 * dtype is the host-facing element type of the input: RLXQ_F32 (run) or RLXQ_BF16 (run_typed). */
RLXQ_API int rlxq_graph_input(rlxq_graph* g, const char* name, uint32_t m, uint32_t k, uint32_t dtype);

/* Graph::param(name, Shape([bytes], U8)) — the packed weight node
 * (rlx-ir/src/ops/linalg.rs:79-91 documents the [bytes] U8 convention). */
RLXQ_API int rlxq_graph_param_u8(rlxq_graph* g, const char* name, uint64_t bytes);

/* Op::DequantMatMul{scheme} with inputs [x, packed_w] and output Shape[m,n] of out_dtype
 * (RLXQ_F32 as in the reference's tests, or RLXQ_BF16 for run_typed graphs)
 * (rlx-ir/src/op.rs:736-752; Graph::dequant_matmul_packed, rlx-ir/src/ops/linalg.rs:79-91). */
RLXQ_API int rlxq_graph_dequant_matmul(rlxq_graph* g, int x_node, int w_node, uint32_t scheme, uint32_t n,
                              uint32_t out_dtype);

/* The SwiGLU gate of rlx-flow/src/blocks/swiglu.rs:48-52 after unfusing
 * (rlx-cuda/src/unfuse.rs:254-293): out = up * silu(gate), elementwise on two [m,n] f32 nodes. */
RLXQ_API int rlxq_graph_swiglu_mul(rlxq_graph* g, int gate_node, int up_node);

/* g.add_node(Op::DequantGroupedMatMul{scheme}, [x, w_packed, expert_idx], Shape([m, n], F32))
 * (rlx-ir/src/op.rs:860-871; usage rlx-runtime/tests/dequant_grouped_matmul_gguf.rs:92-105): w_node is
 * a U8 param holding num_experts packed [n, k] slabs, expert_idx_node an f32 input with one id per
 * row of x.  Output dtype is f32. */
RLXQ_API int rlxq_graph_dequant_grouped_matmul(rlxq_graph* g, int x_node, int w_node, int expert_idx_node,
                                               uint32_t scheme, uint32_t n, uint32_t num_experts);

/* Graph::set_outputs — one output node. */
RLXQ_API int rlxq_graph_set_output(rlxq_graph* g, int node);

/* Session::new(Device::Cuda).compile(graph) — rlx-runtime/src/session.rs:42-87.  Plans one device
 * arena (byte-accurate slots, 256-byte aligned; the reference sizes every slot elems*4,
 * rlx-cuda/src/arena.rs:93-95), allocates it, and records the step schedule.  `device` is the
 * CUDA device ordinal (the reference hard-wires 0, rlx-cuda/src/device.rs:44-60).
 * exec_mode: 0 = ExecMode::Stream, 1 = ExecMode::Graph (steps captured once into a CUDA graph
 * and replayed, rlx-cuda/src/backend.rs:4015-4037). */
RLXQ_API int rlxq_session_compile(const rlxq_graph* g, int device, int exec_mode, rlxq_compiled** out);
RLXQ_API void rlxq_compiled_free(rlxq_compiled* c);

/* CompiledGraph::set_param_typed(name, bytes, DType::U8) — rlx-runtime/src/compiled.rs:192-194 →
 * CudaExecutable::set_param_bytes (rlx-cuda/src/backend.rs:3937-3945).  One plain host-to-device
 * copy of the raw block bytes; len must equal the declared param size. */
RLXQ_API int rlxq_compiled_set_param_typed(rlxq_compiled* c, const char* name, const void* data, uint64_t len);

/* CompiledGraph::run(&[("x", &[f32])]) — rlx-runtime/src/compiled.rs:61-63.  Copies each named
 * f32 input to the device, runs the schedule, copies the f32 output back, and returns when the
 * output is in `out` (out_elems must equal m*n of the output node). */
RLXQ_API int rlxq_compiled_run(rlxq_compiled* c, uint32_t n_inputs, const char* const* names,
                      const float* const* data, const uint64_t* elems, float* out, uint64_t out_elems);

/* run_typed — rlx-runtime/src/backend.rs:2181-2206: inputs and output as raw bytes of the given
 * dtype (RLXQ_F32 or RLXQ_BF16).  bf16 inputs are consumed as bf16 by the kernels (the reference
 * widens them to f32 on the host first; the values are identical); a bf16 output is the f32
 * accumulator rounded to nearest even, as narrow_f32_to_bytes does (:66-89). */
RLXQ_API int rlxq_compiled_run_typed(rlxq_compiled* c, uint32_t n_inputs, const char* const* names,
                            const void* const* data, const uint64_t* bytes, const uint32_t* dtypes,
                            void* out, uint64_t out_bytes, uint32_t out_dtype);

/* Bytes of device memory the compiled graph holds (arena incl. workspace). */
RLXQ_API uint64_t rlxq_compiled_arena_bytes(const rlxq_compiled* c);

/* How many SwiGLU FFNs the compiler recognised and fused in this graph: gate = dequant_matmul(x, Wg),
 * up = dequant_matmul(x, Wu), h = swiglu_mul(gate, up), y = dequant_matmul(h, Wd), all f32, with the three
 * intermediate values used nowhere else.  Such a group runs as one matmul over the stacked [Wg ; Wu] (their arena
 * slots are placed back to back), the product up * silu(gate) formed inside the down projection's activation
 * step, and the down projection: what rlxq_tp_ffn_partial does for one rank.  The reference's CUDA backend
 * fuses the product as FusedSwiGLU (rlx-cuda/src/unfuse.rs:254-293).  Option "graph_fuse_ffn" = 0 turns it off. */
RLXQ_API uint32_t rlxq_compiled_fused_ffn_count(const rlxq_compiled* c);

/* Zeroes the kernels' scratch region of the arena (not the params, inputs or outputs) and waits for it.
 * Call it after rlxq_device_status reported RLXQ_E_TIMEOUT and before the next run: a wait that ran out
 * can leave a half-finished tile exchange behind.  The reference has no counterpart: its executable
 * panics on a failed synchronize (rlx-cuda/src/backend.rs:6675-6693) and is rebuilt. */
RLXQ_API int rlxq_compiled_clear_scratch(rlxq_compiled* c);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_SESSION_H */
