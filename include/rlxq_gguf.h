/*
 * rlxq — reading packed weights out of a GGUF container and putting them on the device.
 *
 * Replaces, for this path, GgufFile::from_path / from_reader, GgufFile::get and
 * GgufFile::tensor_bytes (rlx-gguf/src/lib.rs:205-209, 246-318, 320-326, 355-371) followed by
 * set_param_bytes (rlx-cuda/src/backend.rs:3937-3945).  The reference reads the whole data
 * segment into a Vec, slices the tensor out of it and uploads the slice through its f32-typed
 * arena; here only the header is parsed at open, and a tensor goes file -> pinned staging ->
 * device in chunks, the read of one chunk overlapping the copy of the previous one, straight
 * into the byte-exact slot rlxq_matmul reads.
 */
#ifndef RLXQ_GGUF_H
#define RLXQ_GGUF_H

#include "rlxq.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rlxq_gguf rlxq_gguf;

/* One entry of the tensor table (GgufTensor, rlx-gguf/src/lib.rs:179-194). */
typedef struct rlxq_gguf_tensor {
    uint32_t ggml_type;   /* GgmlType as stored in the file (rlx-gguf/src/lib.rs:55-99) */
    int32_t scheme;       /* rlxq_scheme of that type, or -1 (F32, F16, BF16: not block formats) */
    uint32_t n_dims;
    uint64_t dims[4];     /* GGML order, innermost first, verbatim; a weight W[n,k] is stored as {k, n} */
    uint64_t offset;      /* within the data segment */
    uint64_t bytes;       /* bytes_for(dtype, n_elements) (rlx-gguf/src/lib.rs:393-419); 0 if the type's size is unknown */
} rlxq_gguf_tensor;

/* Parses magic, version (1..3), metadata and the tensor table; the data segment starts at the next
 * multiple of general.alignment (default 32).  Errors: RLXQ_E_ARG (cannot open, not a GGUF file,
 * unsupported version, malformed or truncated header). */
RLXQ_API int rlxq_gguf_open(const char* path, rlxq_gguf** out);
RLXQ_API void rlxq_gguf_close(rlxq_gguf* f);

RLXQ_API uint32_t rlxq_gguf_version(const rlxq_gguf* f);
RLXQ_API uint64_t rlxq_gguf_alignment(const rlxq_gguf* f);
RLXQ_API uint64_t rlxq_gguf_tensor_count(const rlxq_gguf* f);
RLXQ_API uint64_t rlxq_gguf_data_start(const rlxq_gguf* f);

/* Name of tensor `index` in file order (the pointer lives as long as the handle). */
RLXQ_API int rlxq_gguf_tensor_name(const rlxq_gguf* f, uint64_t index, const char** name);
/* GgufFile::get: RLXQ_E_ARG if there is no such tensor. */
RLXQ_API int rlxq_gguf_find(const rlxq_gguf* f, const char* name, rlxq_gguf_tensor* info);

/* Scalar metadata (MetaValue::as_u64 / as_str, rlx-gguf/src/lib.rs:153-175); arrays are skipped at
 * open (a tokenizer's vocabulary is not needed to load weights).  RLXQ_E_ARG if absent or of another kind. */
RLXQ_API int rlxq_gguf_meta_u64(const rlxq_gguf* f, const char* key, uint64_t* value);
RLXQ_API int rlxq_gguf_meta_str(const rlxq_gguf* f, const char* key, const char** value);

/* GgufFile::tensor_bytes into caller memory: exactly `bytes` == info.bytes bytes.  RLXQ_E_SHAPE if the
 * size differs or the tensor reaches past the end of the file. */
RLXQ_API int rlxq_gguf_read_tensor(const rlxq_gguf* f, const char* name, void* host_dst, uint64_t bytes);

/* The same into device memory on `stream`: chunks of the file are read into pinned staging buffers
 * owned by the handle (two per reader; tensors of 64 MiB and more are read by four threads) and copied
 * with cudaMemcpyAsync while the next chunks are being read.  Not for a capturing stream.
 * Returns after the last copy has been enqueued and its staging buffer released (the call waits on
 * events of its own copies only). */
RLXQ_API int rlxq_gguf_upload_tensor(rlxq_gguf* f, const char* name, void* device_dst, uint64_t bytes,
                                     rlxq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RLXQ_GGUF_H */
