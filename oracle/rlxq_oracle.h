/*
 * CPU oracle for the GGUF quantized-weight linear layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's CPU algorithm for the path
 * (rlx-gguf block decoders + rlx-cpu fused dequant matmul).  It is the checker
 * the CUDA kernels are compared with and the timed CPU baseline; nothing in the
 * shipped library (rlx_b200/) links, imports or calls it.
 *
 * Parity status: PINNED against the reference's own known-answer vectors for
 * the decoders (rlx-gguf/src/lib.rs:1188-1291) and the fused-equals-dequant-then-dot
 * property (rlx-cpu/src/gguf_matmul.rs:238-277).  The reference holds no vector
 * for Q8_0/Q4_0 matmul, Q4_K sub-blocks 4..7 with non-zero scales, or Q6_K with
 * negative sub-scales; for those the oracle is cross-checked against an
 * independent formula-level decoder written in numpy (tests/test_oracle.py).
 * The reference itself is Rust and cannot be compiled in this image (no cargo /
 * rustc), so no oracle/_ref build exists.
 *
 * Build: gcc -O2 -ffp-contract=off (never -ffast-math): Rust does not contract
 * a*b+c into an FMA, so neither may this file.
 */
#ifndef RLXQ_ORACLE_H
#define RLXQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Scheme ids shared with include/rlxq.h: 0 = Q4_K and 2 = Q6_K keep the values of
 * rlx-cuda/src/gguf_host.rs:24-34; 6 = Q4_0 and 7 = Q8_0 are new (the reference's
 * CUDA backend has no id for them). */
/* 0..5 are the ids of gguf_scheme_id (rlx-cuda/src/gguf_host.rs:24-34) */
enum { RLXO_Q4_K = 0, RLXO_Q5_K = 1, RLXO_Q6_K = 2, RLXO_Q8_K = 3, RLXO_Q2_K = 4, RLXO_Q3_K = 5, RLXO_Q4_0 = 6, RLXO_Q8_0 = 7,
       RLXO_Q4_1 = 8, RLXO_Q5_0 = 9, RLXO_Q5_1 = 10 };

/* rlx-ir/src/quant.rs:138-164 — block geometry. Returns 0, or -1 for an unknown scheme. */
int rlxo_scheme_geometry(uint32_t scheme, uint32_t* block_elems, uint32_t* block_bytes);

/* half 2.7.1 conversions used at rlx-gguf/src/lib.rs:569-571 and
 * rlx-runtime/src/backend.rs:36-58,66-89. */
float    rlxo_f16_to_f32(uint16_t h);
uint16_t rlxo_f32_to_f16(float f);   /* round to nearest even (generator side only) */
float    rlxo_bf16_to_f32(uint16_t h);
uint16_t rlxo_f32_to_bf16(float f);  /* round to nearest even, NaN kept quiet */

/* Full-tensor decoders: rlx-gguf/src/lib.rs:600-633 (Q8_0, Q4_0), :974-1013 (Q4_K),
 * :1070-1114 (Q6_K, signed sub-scales).  n_elems must be a multiple of the block size.
 * q6k_unsigned_scales != 0 reproduces the per-block decoder at :819-845, which reads
 * the sub-scales as u8; it exists only to document that difference in a test. */
int rlxo_dequant(uint32_t scheme, const uint8_t* blocks, uint64_t n_elems, float* out);
int rlxo_dequant_q6k_unsigned(const uint8_t* blocks, uint64_t n_elems, float* out);

/* rlx-cpu/src/gguf_matmul.rs:40-95 — out[m,n] = x[m,k] . W^T, W packed [n,k] row-major by
 * blocks; out zeroed, then accumulated block by block in storage order with a separate
 * multiply and add.  Single-threaded like the reference. */
int rlxo_matmul_bt(const float* x, const uint8_t* w, float* out,
                   uint64_t m, uint64_t k, uint64_t n, uint32_t scheme);

/* Same arithmetic and per-output accumulation order, rows of W split over `threads`
 * pthreads (k must be a multiple of the block size so blocks do not straddle rows).
 * Bit-identical to rlxo_matmul_bt; used for the all-cores CPU baseline.  Computes only
 * output columns [n0, n1). */
int rlxo_matmul_bt_mt(const float* x, const uint8_t* w, float* out,
                      uint64_t m, uint64_t k, uint64_t n, uint32_t scheme,
                      uint64_t n0, uint64_t n1, int threads);

/* rlx-cpu/src/naive.rs:54-56 */
float rlxo_silu(float x);

/* SwiGLU FFN of rlx-flow/src/blocks/swiglu.rs:48-52 with packed weights:
 * h = up(x) * silu(gate(x)); y = down(h).  x [m,d_model] f32, y [m,d_model] f32.
 * h_out (optional, may be NULL) receives h [m,d_ffn]. */
int rlxo_ffn_swiglu(const float* x, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                    float* y, float* h_out, uint64_t m, uint64_t d_model, uint64_t d_ffn,
                    uint32_t scheme_gate_up, uint32_t scheme_down, int threads);

/* rlx-driver/src/collective.rs:79-128 — sum all-reduce: acc = 0, then acc += rank r's
 * value for r = 0..ranks-1.  parts is [ranks][elems]; out is [elems]. */
void rlxo_allreduce_sum(const float* parts, uint64_t ranks, uint64_t elems, float* out);

/* Seeded synthetic tensors with the value distributions of the benchmark configurations.
 * Counter-based (splitmix64 of seed and block index), so any sub-range can be generated
 * independently and in parallel.  fill_blocks writes n_blocks blocks starting at block
 * index first_block of the stream identified by seed. */
int  rlxo_fill_blocks(uint32_t scheme, uint64_t seed, uint64_t first_block, uint64_t n_blocks,
                      uint8_t* out);
void rlxo_fill_normal_f32(uint64_t seed, uint64_t first, uint64_t count, float* out);

/* Q4_K scale field: inverse of get_scale_min_k4 (rlx-gguf/src/lib.rs:743-751). */
void rlxo_q4k_pack_scales(const uint8_t sc[8], const uint8_t mn[8], uint8_t packed[12]);
void rlxo_q4k_unpack_scale_min(int j, const uint8_t packed[12], uint8_t* sc, uint8_t* mn);

#ifdef __cplusplus
}
#endif
#endif
