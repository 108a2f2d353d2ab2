/*
 * rlxq_tp — tensor-parallel SwiGLU FFN over packed GGUF weights, one rank per GPU.
 *
 * The reference has no counterpart: its CUDA context is a process-wide singleton on device 0
 * (rlx-cuda/src/device.rs:44-60) and its collectives are host emulations
 * (rlx-driver/src/collective.rs:79-128).  These entry points are what a multi-device helper beside
 * CudaExecutable would bind.  The FFN itself is the reference's: y = down(up(x) * silu(gate(x)))
 * (rlx-flow/src/blocks/swiglu.rs:48-52; silu: rlx-cpu/src/naive.rs:54-56).
 *
 * gate and up [d_ffn, d_model] are column-parallel (each rank owns d_ffn/world consecutive output
 * rows), down [d_model, d_ffn] is row-parallel (each rank owns d_ffn/world consecutive k of every
 * row).  A rank computes an f32 partial [m, d_model]; the caller sums the partials with its
 * all-reduce (NCCL through the process group the ranks already have).
 */
#ifndef RLXQ_TP_H
#define RLXQ_TP_H

#include "rlxq.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rlxq_tp_shard {
    uint32_t ffn_local;              /* d_ffn / world */
    uint32_t ffn_begin;              /* rank * ffn_local */
    uint64_t gate_up_row_bytes;      /* bytes of one row of gate / up (k = d_model) */
    uint64_t gate_up_byte_offset;    /* this rank's rows start here in the full gate / up */
    uint64_t gate_up_bytes;          /* ... and span this many bytes (contiguous) */
    uint64_t down_row_bytes_full;    /* bytes of one full row of down (k = d_ffn) */
    uint64_t down_row_bytes_local;   /* bytes of this rank's k-slice of one row */
    uint64_t down_row_byte_offset;   /* offset of the slice inside every full row */
    uint64_t down_bytes;             /* d_model * down_row_bytes_local */
} rlxq_tp_shard;

/* Where rank `rank` of `world` finds its shards.  d_ffn must split into `world` slices of whole
 * 256-weight groups (so every sliced row keeps 16-byte alignment); RLXQ_E_SHAPE otherwise. */
RLXQ_API int rlxq_tp_shard_plan(uint32_t scheme, uint32_t d_model, uint32_t d_ffn, uint32_t world,
                                uint32_t rank, rlxq_tp_shard* out);

/* Host-side gather of the k-slice [k_begin, k_begin + k_len) of every row of a packed W[n, k] into
 * a packed W'[n, k_len] (run once at load time). */
RLXQ_API int rlxq_tp_slice_k_host(uint32_t scheme, const void* w_full, uint32_t n, uint32_t k,
                                  uint32_t k_begin, uint32_t k_len, void* w_slice);

/* Scratch for rlxq_tp_ffn_partial. */
RLXQ_API int rlxq_tp_ffn_workspace_bytes(uint32_t scheme_gate_up, uint32_t scheme_down, uint32_t m,
                                         uint32_t d_model, uint32_t ffn_local, uint32_t x_dtype, size_t* bytes);

/* One rank's share of the FFN on the caller's stream:
 *   gu = x . [gate_r ; up_r]^T   (one matmul: gate_up_blocks holds the rank's gate rows followed by
 *                                 its up rows, 2*ffn_local rows of k = d_model)
 *   h  = up * silu(gate)         (f32 for m <= 8; rounded to bf16 for m > 8, where it feeds the
 *                                 tensor-core GEMM, which takes bf16 activations)
 *   y_partial = h . down_r^T     (down_blocks: d_model rows of k = ffn_local)
 * x: [m, d_model] f32 or bf16; y_partial: [m, d_model] f32.  workspace 256-byte aligned.
 * No synchronisation, no allocation: capture-safe like rlxq_matmul. */
RLXQ_API int rlxq_tp_ffn_partial(rlxq_stream_t stream, uint32_t scheme_gate_up, uint32_t scheme_down,
                                 const void* x, uint32_t x_dtype, const void* gate_up_blocks,
                                 const void* down_blocks, float* y_partial, uint32_t m, uint32_t d_model,
                                 uint32_t ffn_local, void* workspace, size_t workspace_bytes);

/* ---- sum all-reduce of a small f32 vector over peer memory (NVLink), for the decode step ----
 *
 * No counterpart in the reference (its collectives run on the host, rlx-driver/src/collective.rs:79-128;
 * the summation order here is theirs: rank 0, 1, ... world-1).  One process per GPU.  Set-up, once:
 * every rank allocates a buffer with rlxq_tp_comm_alloc, exports its handle, the ranks exchange the
 * handles through whatever channel they share (torch.distributed, MPI, a file) and open each other's
 * with rlxq_tp_ipc_open.  Per step: rlxq_tp_allreduce_sum on every rank.  world <= 8.
 * A buffer holds a 1 KiB header, twice one slot of max_elems 8-byte words {value, step tag} per possible rank,
 * and twice one slot of max_elems floats per possible rank for rlxq_tp_ffn_step's pushing form (192 * max_elems
 * + 1024 bytes; rlxq_tp_comm_bytes says): every rank stores its partial, tagged with the step, into its slot of
 * every peer's buffer and adds the slots of its own buffer once every word carries the tag of the step (eight
 * CTAs, an eighth of the vector each; no flag and no fence between data and flag: a word arrives whole). */
RLXQ_API int rlxq_tp_comm_bytes(uint32_t max_elems, size_t* bytes);
RLXQ_API int rlxq_tp_comm_alloc(uint32_t max_elems, void** buf);       /* cudaMalloc + zero; not capture-safe */
RLXQ_API int rlxq_tp_comm_free(void* buf);
RLXQ_API int rlxq_tp_ipc_export(const void* buf, uint8_t handle[64]);  /* cudaIpcGetMemHandle */
RLXQ_API int rlxq_tp_ipc_open(const uint8_t handle[64], void** buf);   /* cudaIpcOpenMemHandle, peer access enabled */
RLXQ_API int rlxq_tp_ipc_close(void* buf);

/* dst[i] = sum over ranks r = 0..world-1 of src_r[i], the same bits on every rank.  bufs: host array of
 * `world` device pointers, bufs[rank] this rank's own buffer, the others as opened through IPC.  elems a
 * multiple of 4, at most the max_elems the buffers were allocated for; src, dst 16-byte aligned; src and
 * dst may be the same.  One kernel on the caller's stream, capture-safe (the step counter lives in the
 * buffer).  A rank whose peer does not arrive within a bounded wait records a device error (reported by
 * rlxq_device_status) and leaves dst unwritten; it never hangs. */
RLXQ_API int rlxq_tp_allreduce_sum(rlxq_stream_t stream, uint32_t rank, uint32_t world, void* const* bufs,
                                   uint32_t max_elems, const float* src, float* dst, uint32_t elems);

/* One step of the sharded FFN on this rank, exchange included: y[m, d_model] = sum over ranks of the partials of
 * rlxq_tp_ffn_partial, in rank order, the same bits on every rank (every rank calls it with its own shard).  bufs,
 * max_elems as for rlxq_tp_allreduce_sum; m * d_model <= max_elems and a multiple of 4.  By default this is
 * rlxq_tp_ffn_partial followed by rlxq_tp_allreduce_sum.  With option "tp_fused" = 1, for batch 1-8 of Q4_0, Q8_0,
 * Q4_K, Q5_K and Q6_K, the down projection is the collective: its finisher warps store every finished 16-row tile
 * into this rank's slot of every rank's buffer (plain peer stores) while later tiles are still being multiplied,
 * each CTA counts itself in on its own rank behind its stores, the CTA that completes the count tells every rank
 * (one red.release.sys each), and a few CTAs wait, bounded, until all ranks are in and add the world slots out of
 * their own rank's memory.  One launch fewer, no copy of the partial; measured slower than the default all the
 * same (2 GPUs, 70B FFN shard, batch 1: 54 us against 47 us a step), because the stand-alone all-reduce leaves the
 * SMs free for the next kernel to fetch its first weights while the exchange completes.  All ranks must make the
 * same sequence of calls with the same shapes and the same option.  No counterpart in the reference (rlx-driver/src/collective.rs:79-128 is its host-side exchange). */
RLXQ_API int rlxq_tp_ffn_step(rlxq_stream_t stream, uint32_t scheme_gate_up, uint32_t scheme_down, const void* x,
                              uint32_t x_dtype, const void* gate_up_blocks, const void* down_blocks, float* y,
                              uint32_t m, uint32_t d_model, uint32_t ffn_local, void* workspace, size_t workspace_bytes,
                              uint32_t rank, uint32_t world, void* const* bufs, uint32_t max_elems);

/* ---- the whole layer from one host thread: create / load / run / destroy ----
 *
 * For a host that drives all GPUs of a node from one process (the reference's CudaExecutable lives in one
 * process; rlx-cuda/src/device.rs:44-60 is what would grow a device list).  No counterpart in the reference.
 * The library owns what it creates here: one stream per device, the shards, scratch that grows with the largest
 * batch seen, the peer buffers of the decode-sized all-reduce, and (created on the first prefill-sized step) one
 * NCCL communicator per device; libnccl.so.2 is loaded at run time, so the library has no link-time dependency
 * on it and a host that only ever runs decode batches never touches it.
 *
 * rlxq_tp_create: devs = ndev device ordinals (null: 0 .. ndev-1), 1 <= ndev <= 8.  Enables peer access between
 *   them where the hardware allows it.
 * rlxq_tp_ffn_load: gate, up [d_ffn, d_model] and down [d_model, d_ffn] as packed blocks in HOST memory; every
 *   device receives its shard (rlxq_tp_shard_plan) with one upload per tensor.  May be called again to replace
 *   the weights.
 * rlxq_tp_ffn_run: x [m, d_model] (f32 or bf16) and y [m, d_model] (f32) in HOST memory.  Per device: copy of x,
 *   rlxq_tp_ffn_partial, then the sum of the partials -- rlxq_tp_allreduce_sum when m * d_model <= 65536 and every
 *   device can read its peers, NCCL's all-reduce otherwise -- and device 0's result back to y.  Returns after all
 *   devices have finished.  RLXQ_E_NCCL when NCCL is needed and cannot be loaded or fails.  Allocates on the first
 *   call for a batch size (and for any larger one later): not for use inside a stream capture.
 * rlxq_tp_status: rlxq_device_status on every device of the group.
 * One thread at a time per handle. */
typedef struct rlxq_tp rlxq_tp;
RLXQ_API int rlxq_tp_create(int ndev, const int* devs, rlxq_tp** out);
RLXQ_API int rlxq_tp_world(const rlxq_tp* t);
RLXQ_API int rlxq_tp_ffn_load(rlxq_tp* t, uint32_t scheme, const void* gate, const void* up, const void* down,
                              uint32_t d_model, uint32_t d_ffn);
RLXQ_API int rlxq_tp_ffn_run(rlxq_tp* t, const void* x_host, uint32_t x_dtype, uint32_t m, float* y_host);
RLXQ_API int rlxq_tp_status(rlxq_tp* t, int* device_error);
RLXQ_API int rlxq_tp_destroy(rlxq_tp* t);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_TP_H */
