/*
 * rlxq — B200 (sm_100a) kernels for RLX's GGUF quantized-weight linear layer, behind a C ABI.
 *
 * This is the boundary RLX's Rust `rlx-cuda` backend binds in place of its
 * dequant-to-f32-scratch + cublasSgemm lowering of `Op::DequantMatMul` (GGUF schemes).
 * Every entry point takes plain pointers and sizes; device pointers are "arena base +
 * byte offset" exactly as the reference computes them (rlx-cuda/src/gguf_gpu.rs:105-111).
 *
 * Conventions
 *  - Return value: 0 on success, a negative rlxq_status otherwise.  Nothing aborts.  The
 *    reference panics on failure (`.expect(...)`, rlx-cuda/src/gguf_gpu.rs:99-103,132); a
 *    Rust shim keeps that behaviour by `expect`-ing a zero status.
 *  - Work is enqueued on the caller's stream; no entry point that takes a stream
 *    synchronises, allocates, or reads device memory from the host, so they may be called
 *    on a capturing stream (the reference captures its step loop in ExecMode::Graph,
 *    rlx-cuda/src/backend.rs:4015-4037).
 *  - `w_blocks` is the raw GGUF block stream of a weight W[n,k], row-major by blocks,
 *    `n*k/block_elems*block_bytes` bytes, as uploaded by set_param_bytes
 *    (rlx-cuda/src/backend.rs:3937-3945).  k must be a multiple of block_elems.
 *  - Matrices: x is [m,k] row-major, y is [m,n] row-major: y = x . W^T
 *    (rlx-cpu/src/gguf_matmul.rs:40-95).
 */
#ifndef RLXQ_H
#define RLXQ_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define RLXQ_API __attribute__((visibility("default")))
#else
#define RLXQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* rlxq_stream_t; /* a cudaStream_t / CUstream */

enum rlxq_status {
    RLXQ_OK = 0,
    RLXQ_E_SCHEME = -1,    /* unknown scheme id */
    RLXQ_E_SHAPE = -2,     /* k not a multiple of the block size, zero-sized where not allowed, overflow */
    RLXQ_E_NULL = -3,      /* null pointer for a non-empty buffer */
    RLXQ_E_DTYPE = -4,     /* unknown activation / output dtype */
    RLXQ_E_WORKSPACE = -5, /* workspace smaller than rlxq_workspace_bytes reports */
    RLXQ_E_CUDA = -6,      /* a CUDA call failed; rlxq_last_error() has the text */
    RLXQ_E_NCCL = -7,      /* an NCCL call failed */
    RLXQ_E_TIMEOUT = -8,   /* a bounded device- or host-side wait ran out */
    RLXQ_E_ALIGN = -9,     /* pointer alignment below what the entry point states */
    RLXQ_E_ARG = -10,      /* other invalid argument (unknown option, bad rank, name not found) */
    RLXQ_E_LIMIT = -11     /* size beyond a stated fixed maximum */
};

/* Scheme ids.  0..5 keep the values of gguf_scheme_id (rlx-cuda/src/gguf_host.rs:24-34);
 * Q4_0 and Q8_0 have no id there (that function panics on them) and get 6 and 7.  Q4_K, Q6_K,
 * Q4_0 and Q8_0 have the streaming GEMV and the tensor-core GEMM; so has the rest of
 * QuantScheme::is_gguf (rlx-ir/src/quant.rs:170-182): Q5_K, and Q2_K, Q8_K / Q3_K where k is a multiple
 * of 1024 / 2048; every shape these kernels do not take runs through the
 * general kernel, so every GGUF scheme the reference lowers runs on the GPU without its host fallback.  Q4_1, Q5_0 and Q5_1 (8, 9, 10)
 * are container types the reference only decodes to f32 when a file is loaded (GgufFile::tensor_f32,
 * rlx-gguf/src/lib.rs:323-353, decoders :635-729) and no QuantScheme names; here they dequantise bit-exactly
 * and multiply through the streaming GEMV (m <= 8) and the tensor-core GEMM (m > 8) like the others, so such
 * a tensor can stay packed on the device as well. */
enum rlxq_scheme {
    RLXQ_Q4_K = 0, RLXQ_Q5_K = 1, RLXQ_Q6_K = 2, RLXQ_Q8_K = 3, RLXQ_Q2_K = 4, RLXQ_Q3_K = 5,
    RLXQ_Q4_0 = 6, RLXQ_Q8_0 = 7, RLXQ_Q4_1 = 8, RLXQ_Q5_0 = 9, RLXQ_Q5_1 = 10
};

/* Activation / output element types: the two the reference's typed I/O carries on this
 * path (run_typed, rlx-runtime/src/backend.rs:2181-2206). */
enum rlxq_dtype { RLXQ_F32 = 0, RLXQ_BF16 = 1 };

/* Library version (major*10000 + minor*100 + patch). */
RLXQ_API int rlxq_version(void);

/* Static text for a status code. */
RLXQ_API const char* rlxq_status_string(int status);

/* Thread-local text of the most recent failure in this thread ("" if none). */
RLXQ_API const char* rlxq_last_error(void);

/* Replaces QuantScheme::gguf_block_size / gguf_block_bytes (rlx-ir/src/quant.rs:138-164). */
RLXQ_API int rlxq_scheme_geometry(uint32_t scheme, uint32_t* block_elems, uint32_t* block_bytes);

/* Replaces slab_bytes_for (rlx-cuda/src/gguf_gpu.rs:29-33): bytes of a packed W[n,k]. */
RLXQ_API int rlxq_packed_bytes(uint32_t scheme, uint64_t k, uint64_t n, uint64_t* bytes);

/* Replaces dequant_gguf_scratch_bytes (rlx-cuda/src/gguf_gpu.rs:35-59) at plan time: the
 * scratch rlxq_matmul needs for this shape.  For m <= 8 that is the converted activations
 * (a few bytes per element of x), the partial output tiles of CTAs that share a row tile and
 * their counters: tens to hundreds of KiB (up to 4.9 MB while the option gemv_kernel is 4).  The tensor-core GEMM needs none for most shapes; for few
 * output tiles and a long k it asks for two partial 128 x 256 f32 tiles per SM (39 MB on a 148-SM
 * part) for its stream-K split; without them it runs whole tiles.  With f32 activations and m > 8 the GEMM runs
 * on their bf16 hi + lo halves, a chunk of rows at a time: the split rows and the two partial results need up to
 * about 150 MB (256-byte aligned); without that workspace such a call runs the tiled generic kernel, some 40 times
 * slower.  The reference reserves k*n*4 bytes. */
RLXQ_API int rlxq_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n,
                         uint32_t x_dtype, uint32_t y_dtype, size_t* bytes);

/* Replaces the `dequant_gguf` kernel launch (rlx-cuda/src/gguf_gpu.rs:81-103;
 * rlx-gpu-kernels/kernels/dequant_gguf.cu:46-244): decode n_elems weights to f32, bit-identical
 * to rlx_gguf::dequant_{q8_0,q4_0,q4_k,q6_k} (rlx-gguf/src/lib.rs:600-633,974-1013,1070-1114).
 * `out` must be 16-byte aligned; w_blocks 2-byte aligned. */
RLXQ_API int rlxq_dequant_f32(rlxq_stream_t stream, uint32_t scheme, const void* w_blocks,
                     uint64_t n_elems, float* out);

/* Replaces run_dequant_matmul_gguf_gpu (rlx-cuda/src/gguf_gpu.rs:62-134) and the host fallback
 * run_dequant_matmul_gguf (rlx-cuda/src/gguf_host.rs:90-128): y = x . W^T with the blocks
 * decoded inside the kernel.  m <= 8 runs the streaming GEMV; larger m runs the tensor-core
 * GEMM when the shape allows it (rlxq_workspace_bytes tells what it needs; f32 activations enter it as two bf16
 * halves whose results are added, so no activation bit is lost), else a tiled kernel.
 * x: f32 or bf16 [m,k]; y: f32 or bf16 [m,n]; accumulation is f32, a bf16 y is its round-to-nearest-even
 * narrowing (a NaN result of the GEMM is stored as the canonical quiet NaN).  x must be 16-byte aligned, y
 * aligned to its element size, w_blocks to 2 bytes (16 bytes enables the bulk-copy fast paths).
 * workspace: rlxq_workspace_bytes(...) bytes, 16-byte aligned, contents irrelevant on entry; it is
 * private to the call while the kernels run (two calls in flight must not share it). */
RLXQ_API int rlxq_matmul(rlxq_stream_t stream, uint32_t scheme,
                const void* x, uint32_t x_dtype, const void* w_blocks,
                void* y, uint32_t y_dtype, uint32_t m, uint32_t k, uint32_t n,
                void* workspace, size_t workspace_bytes);

/* A chain of dependent matmuls behind one call: y_i[m, n_i] = in_i[m, k_i] . W_i^T with in_0 = x and in_i = y_(i-1),
 * or, with swiglu != 0, in_i = up * silu(gate) of y_(i-1) = [gate | up] ([m, 2 k_i]; silu(g) = g / (1 + exp(-g)),
 * rlx-cpu/src/naive.rs:54-56).  Two plain layers are the up / down pair of a decode step, a plain layer over the
 * stacked [gate ; up] weight followed by a swiglu layer is a SwiGLU FFN (rlx-flow/src/blocks/swiglu.rs:48-52).
 * The reference runs such a chain as consecutive steps of its compiled graph (rlx-cuda/src/backend.rs:5366-5405),
 * the product as FusedSwiGLU (rlx-cuda/src/unfuse.rs:254-293).  By default the layers run one after the other
 * through the kernels rlxq_matmul uses (the SwiGLU product in a kernel of its own).  With option "gemv_chain" = 1,
 * m <= 2 and up to 3 layers of the streaming formats (k a multiple of 256, 2048 for Q6_K; 16-byte aligned x and
 * weights; every layer's tiles cut at most once by the CTA ranges) the whole chain is ONE cooperative kernel: the
 * weight stream never stops between layers and a layer waits only for a grid-wide barrier on its input (bounded:
 * RLXQ_E_TIMEOUT code 8 through rlxq_device_status).  That needs every CTA of the grid resident at once, so
 * nothing else may occupy the GPU's SMs meanwhile.  It is off by default because it is slower than the separate
 * launches on the shapes measured (24 us against 16 us for the Q4_0 4096 -> 11008 -> 4096 pair): every CTA
 * quantises the whole input of every layer behind the barrier, and programmatic dependent launch already hides
 * most of a launch boundary.  Same results either way up to f32 summation order.  Intermediate outputs are f32
 * and live in the workspace.  y: f32 or bf16 [m, n_last].
 * workspace: rlxq_chain_workspace_bytes(...) bytes, 256-byte aligned, contents irrelevant on entry. */
typedef struct rlxq_chain_layer {
    const void* w_blocks;     /* packed W_i[n, k] */
    uint32_t k, n;
    uint32_t swiglu;          /* input is the SwiGLU product of the previous layer's output (never for layer 0) */
} rlxq_chain_layer;
RLXQ_API int rlxq_chain_workspace_bytes(uint32_t scheme, const rlxq_chain_layer* layers, uint32_t nlayers, uint32_t m,
                                        uint32_t x_dtype, size_t* bytes);
RLXQ_API int rlxq_matmul_chain(rlxq_stream_t stream, uint32_t scheme, const rlxq_chain_layer* layers, uint32_t nlayers,
                               const void* x, uint32_t x_dtype, void* y, uint32_t y_dtype, uint32_t m,
                               void* workspace, size_t workspace_bytes);

/* y = x . W^T for batch 1 and 2 (the streaming decode GEMV) without any device allocation and
 * without a caller workspace.  This entry point has no counterpart in the reference.
 *
 * It is meant for callers that cannot obtain device memory when they need the result: a decode
 * loop that runs after the process has frozen its allocations, a host whose device budget belongs
 * entirely to another allocator, or code that must stay free of cudaMalloc / cudaFree after
 * start-up.  The scratch rlxq_matmul would take from `workspace` (quantised activations, a few
 * partial tiles, tile counters) lives instead in a fixed 2 MiB array inside this library's device
 * image; every GPU that loads the library carries those 2 MiB until the process ends.
 *
 * Same arguments, results and alignment rules as rlxq_matmul with m <= 2 (k a multiple of 256,
 * 2048 for Q6_K; x and w_blocks 16-byte aligned).  RLXQ_E_SHAPE for m > 2 or an unsupported k,
 * RLXQ_E_LIMIT when the shape would need more scratch than the array holds (very large n * k/2048).
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call before any stream capture.  Later calls only launch.
 * All calls on a device share the one array, which keeps whatever the previous call left; each call
 * rewrites or zeroes what it depends on, so calls issued one after the other (same stream, or
 * ordered by events) are independent, but two calls whose kernels may overlap on the GPU race on it
 * and must not be issued.
 * A bounded wait that runs out inside this entry point is recorded in the device's regular error
 * word when the process already has one (rlxq_init_device at start-up creates it), otherwise in a
 * word inside the library image; rlxq_device_status reads both, and allocates nothing when only
 * allocation-free calls have been made on the device. */
RLXQ_API int rlxq_matmul_static_scratch(rlxq_stream_t stream, uint32_t scheme,
                                        const void* x, uint32_t x_dtype, const void* w_blocks,
                                        void* y, uint32_t y_dtype, uint32_t m, uint32_t k, uint32_t n);

/* Once per device, with that device current and outside any stream capture: allocates the
 * library's per-device error word (4 bytes).  The reference creates its per-process device state
 * in cuda_context() (rlx-cuda/src/device.rs:44-60).  rlxq_matmul calls it lazily if it was not. */
RLXQ_API int rlxq_init_device(void);

/* Synchronises the current device and reports whether any kernel of this library gave up on a
 * bounded wait since the last call (RLXQ_E_TIMEOUT, *device_error = which wait).  Every spin in
 * the kernels has an iteration limit, so a lost copy or a missing signal ends as this error, not
 * as a hung GPU.  Not capture-safe (it synchronises); the reference's equivalent is the
 * stream.synchronize() + panic in CudaExecutable::run (rlx-cuda/src/backend.rs:6675-6693).
 * After RLXQ_E_TIMEOUT the outputs of the calls since the last check are undefined, and the
 * workspace those calls used (or the built-in scratch of rlxq_matmul_static_scratch) may hold a
 * half-finished tile exchange: zero it (cudaMemsetAsync) before the next call or graph replay that
 * uses it (rlxq_compiled_clear_scratch for a compiled graph's arena). */
RLXQ_API int rlxq_device_status(int* device_error);

/* Number of kernels this library has launched in this process (all threads). */
RLXQ_API uint64_t rlxq_launch_count(void);

/* Tuning / dispatch override, the counterpart of the reference's RLX_KERNEL_DISPATCH and
 * RLX_CUDA_* environment keys (rlx-ir/src/env.rs:57-104).  Keys:
 *   "gemv_kernel": 0 = automatic (integer kernel: dp4a units for m = 1, integer-MMA units for m = 2 .. 8 where the
 *                  format and shape have them, else dp4a units for m = 2 and the staged tensor-mode kernel above),
 *                  1 = force the generic warp-per-row kernel, 2 = force the staged tensor-mode
 *                  GEMV, 3 = force the integer GEMV with its dp4a units (m <= 4), 4 = force the tcgen05 GEMV (m <= 8;
 *                  Q4_0, Q8_0, Q4_K; k a multiple of 256), 5 = force the integer GEMV with its integer-MMA units
 *                  (m <= 8; Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, Q4_1, Q5_0, Q5_1 with k a multiple of 256, 2048 for Q6_K; Q8_K, Q2_K with k a
 *                  multiple of 1024, Q3_K of 2048: whole 16-byte groups of super-blocks per row).  2 to 5: error if the shape does not allow it.  The tcgen05 GEMV is
 *                  correct but slower than the others on the shapes measured so far, hence not automatic.
 *   "gemv_tc_ctas": CTAs per SM of the tcgen05 GEMV, 2 (default) or 1
 *   "tp_fused": 1 = rlxq_tp_ffn_step lets the down projection push its tiles to the peers and finish the sum
 *                  itself (rlxq_tp.h), 0 (default) = partial, then the stand-alone all-reduce kernel.  The pushing
 *                  form is one launch shorter but measured slower on NVLink (its CTAs hold their SMs while the
 *                  exchange completes, so the next kernel cannot fetch its first weights meanwhile)
 *   "gemv_chain": 1 = rlxq_matmul_chain runs a chain as one cooperative kernel where it can, 0 (default) = always
 *                  layer by layer
 *   "gemm_kernel": 0 = automatic, 1 = force the tiled generic kernel, 2 = force the tcgen05 GEMM
 *   "gemm_streamk": 0 = automatic (split the k dimension across SMs when that saves at least 36
 *                  256-wide k steps on the busiest SM and a workspace is given), 1 = never,
 *                  2 = whenever a workspace is given
 *   "gemm_pair": the tcgen05 GEMM with two CTAs per MMA (a cluster of two SMs on 256 weight rows x 256 activation
 *                  rows, each CTA loading half of the activation tile): 0 = automatic (n a multiple of 256, at
 *                  least one tile pair per resident cluster, not Q6_K or Q3_K, no k split chosen), 1 = never, 2 = wherever
 *                  n is a multiple of 256.  Same bits as the single-CTA kernel.  "gemm_pair_clusters" (read only):
 *                  clusters the device keeps resident, 0 until the paired kernel has run
 *   "gemm_tile_x": 0 = automatic, 128 or 256 = activation rows per tile of the tcgen05 GEMM
 *   "gemv_inline_q": 0 = automatic, 1 = the integer GEMV always runs its activation quantiser as a
 *                  kernel of its own, 2 = the streaming kernel quantises the activations itself
 *                  whenever the shape allows it
 *   "gemv_kslices": 0 = automatic, n > 0 = split k over n CTAs per row tile in the staged GEMV
 *   "tp_spin_limit": polls of a peer's flag before rlxq_tp_allreduce_sum's kernel gives up and reports
 *          RLXQ_E_TIMEOUT (device_error = 40 + the peer's rank); default 2^24, a few seconds
 *   "graph_fuse_ffn": 1 (default) = the Session mirror lowers a SwiGLU FFN pattern to the fused form (rlxq_session.h),
 *          0 = every node runs as its own kernels
 *   "pdl": 1 (default) = launch the GEMV kernels with programmatic stream serialization so a
 *          kernel's weight prefetch overlaps the tail of its predecessor, 0 = plain launches
 * Returns RLXQ_E_ARG for an unknown key. */
RLXQ_API int rlxq_set_option(const char* key, int64_t value);
RLXQ_API int rlxq_get_option(const char* key, int64_t* value);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_H */
