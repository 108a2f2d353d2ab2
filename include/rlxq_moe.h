/*
 * rlxq — fused GGUF dequant + grouped matmul for MoE expert stacks, on the GPU.
 *
 * Replaces run_dequant_grouped_matmul_gguf_gpu (rlx-cuda/src/gguf_gpu.rs:142-280), the lowering of
 * Op::DequantGroupedMatMul (rlx-ir/src/op.rs:860-871; CPU semantics gguf_grouped_matmul_bt,
 * rlx-cpu/src/gguf_matmul.rs:102-139): y[i,:] = x[i,:] . W_e^T with e = expert_idx[i], where
 * w_blocks holds num_experts contiguous packed slabs, expert e at [e*slab, (e+1)*slab), each slab a
 * [n,k] matrix in the layout rlxq_matmul takes.  The reference copies x and the expert ids to the
 * host, counting-sorts the rows there, runs dequantise + sgemm per expert and copies back; here the
 * counting sort (grouped_moe_sort_plan, gguf_matmul.rs:178-205) runs on the device and one kernel
 * walks every expert's rows, so nothing crosses PCIe and nothing synchronises.  Up to 8 rows (decode)
 * go row by row through the streaming GEMV, the expert picked on the device.  From 32 rows on, for the
 * formats and shapes the tensor-core GEMM takes (every format; k a multiple of 256, 1024 for Q2_K and Q8_K, 2048 for Q3_K and
 * Q6_K; 16-byte aligned stack), every expert's rows are gathered next to each other as bf16 (f32 activations
 * as hi + lo halves) and one launch of the GEMM in its grouped form multiplies each 128- or 256-row tile by its
 * expert's slab; the weight operand is bf16(d * q) there, as in rlxq_matmul for m > 8.
 */
#ifndef RLXQ_MOE_H
#define RLXQ_MOE_H

#include "rlxq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Scratch for rlxq_grouped_matmul: expert offsets, the row permutation, per-expert cursors, or (decode
 * sizes) the streaming GEMV's own scratch.  For the tensor-core path also the tile table, the gathered
 * activations (2 m rows of k bf16) and their results (2 m rows of n f32): 2 m (2 k + 4 n) bytes, 256-byte
 * aligned.  A call given less than that (but enough for the sort) runs the general kernel instead. */
RLXQ_API int rlxq_grouped_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t num_experts,
                                          size_t* bytes);

/* x: [m,k] f32 or bf16; expert_idx: [m] f32-encoded expert ids, as the reference's graph input
 * (rlx-runtime/tests/dequant_grouped_matmul_gguf.rs:92-105); y: [m,n] f32 or bf16.  A row whose id
 * is read as the reference's `expert_idx[i] as usize` reads it (rlx-cpu/src/gguf_matmul.rs:187,198: a
 * saturating cast, so NaN, negative values and fractions below 1 mean expert 0); a row whose id is
 * num_experts or more, which indexes out of bounds in the reference, gets zeros.
 * k must be a multiple of the block size and k*n of it too (whole blocks per slab row). */
RLXQ_API int rlxq_grouped_matmul(rlxq_stream_t stream, uint32_t scheme, const void* x, uint32_t x_dtype,
                                 const void* w_blocks, const float* expert_idx, void* y, uint32_t y_dtype,
                                 uint32_t m, uint32_t k, uint32_t n, uint32_t num_experts,
                                 void* workspace, size_t workspace_bytes);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_MOE_H */
