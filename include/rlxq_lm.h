/*
 * rlxq — greedy / top-k selection over a GGUF-packed tied LM head, on the GPU.
 *
 * Replaces gguf_tied_lm_argmax (rlx-cpu/src/lm_head.rs:223-251) and gguf_tied_lm_topk
 * (rlx-cpu/src/lm_head.rs:172-199): logits[j] = hidden . W[j,:] over the packed embedding
 * W[n_vocab, n_embd] (the same raw block stream rlxq_matmul takes), then the best token or the
 * `cap` best.  The reference streams the rows on one CPU thread (with a Cauchy-bound early exit for
 * top-k); here the logits come from the streaming GEMV of rlxq_matmul (batch 1) and the selection
 * from a few small kernels.  Nothing is copied to the host and nothing synchronises: the results
 * are written to device memory on the caller's stream.
 */
#ifndef RLXQ_LM_H
#define RLXQ_LM_H

#include "rlxq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Largest `cap` rlxq_lm_head_topk accepts. */
#define RLXQ_LM_MAX_CAP 64u

/* flags */
enum rlxq_lm_flags {
    /* Re-evaluate the leading candidates in the reference's own arithmetic (f32, products added in
     * column order, multiply and add rounded separately: row_dot_gguf, rlx-cpu/src/lm_head.rs:46-76)
     * and rank them by those values.  The returned logits are then bit-identical to the reference's
     * and so is the chosen token unless more rows than the spare candidates (8) lie within the
     * GEMV's rounding (about 1e-6 relative) of the winner.  Costs one serial pass over n_embd. */
    RLXQ_LM_EXACT = 1u
};

/* Bytes of scratch the two calls below need (logits, candidate lists, the GEMV's own workspace). */
RLXQ_API int rlxq_lm_head_workspace_bytes(uint32_t scheme, uint32_t n_embd, uint32_t n_vocab,
                                          uint32_t x_dtype, uint32_t cap, size_t* bytes);

/* Top-`cap` tokens: idx_out[0..cap) and val_out[0..cap) (device memory), best first; equal logits
 * are ordered by token id (the reference leaves that order to an unstable selection).  Rows whose
 * logit is NaN are never chosen; if fewer than `cap` rows can be chosen the remaining entries are
 * (0xFFFFFFFF, -inf).  hidden: [n_embd] f32 or bf16, 16-byte aligned.  1 <= cap <= RLXQ_LM_MAX_CAP
 * and cap <= n_vocab (the reference clamps cap the same way, lm_head.rs:181). */
RLXQ_API int rlxq_lm_head_topk(rlxq_stream_t stream, uint32_t scheme, const void* hidden, uint32_t x_dtype,
                               const void* w_blocks, uint32_t n_embd, uint32_t n_vocab, uint32_t cap,
                               uint32_t flags, void* workspace, size_t workspace_bytes,
                               uint32_t* idx_out, float* val_out);

/* The best token and its logit: strict '>' scan from token 0 as in the reference, so the lowest id
 * wins a tie and (0, -inf) comes back when no logit exceeds -inf. */
RLXQ_API int rlxq_lm_head_argmax(rlxq_stream_t stream, uint32_t scheme, const void* hidden, uint32_t x_dtype,
                                 const void* w_blocks, uint32_t n_embd, uint32_t n_vocab, uint32_t flags,
                                 void* workspace, size_t workspace_bytes, uint32_t* idx_out, float* val_out);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_LM_H */
