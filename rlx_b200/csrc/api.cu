// C ABI of the rlxq library: argument checking and kernel selection.  The kernels live in
// dequant.cu, gemv_generic.cu, gemv_staged.cu and gemm_tcgen05.cu.
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace rlxq {

std::atomic<uint64_t> g_launches{0};

char* last_error_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return status;
}

Options& options() {
    static Options o;
    return o;
}

int sm_count() {
    // One query per device, cached; cudaDeviceGetAttribute does not synchronise.
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

static bool dtype_ok(uint32_t d) { return d == RLXQ_F32 || d == RLXQ_BF16; }

}  // namespace rlxq

using namespace rlxq;

extern "C" {

int rlxq_version(void) { return 100; }

const char* rlxq_status_string(int s) {
    switch (s) {
        case RLXQ_OK: return "ok";
        case RLXQ_E_SCHEME: return "unknown quantisation scheme";
        case RLXQ_E_SHAPE: return "bad shape";
        case RLXQ_E_NULL: return "null pointer";
        case RLXQ_E_DTYPE: return "unknown dtype";
        case RLXQ_E_WORKSPACE: return "workspace too small";
        case RLXQ_E_CUDA: return "CUDA error";
        case RLXQ_E_NCCL: return "NCCL error";
        case RLXQ_E_TIMEOUT: return "timed out";
        case RLXQ_E_ALIGN: return "misaligned pointer";
        case RLXQ_E_ARG: return "invalid argument";
        case RLXQ_E_LIMIT: return "size beyond the fixed maximum";
        default: return "unknown status";
    }
}

const char* rlxq_last_error(void) { return last_error_buf(); }

int rlxq_scheme_geometry(uint32_t scheme, uint32_t* block_elems, uint32_t* block_bytes) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (block_elems) *block_elems = g.elems;
    if (block_bytes) *block_bytes = g.bytes;
    return RLXQ_OK;
}

int rlxq_packed_bytes(uint32_t scheme, uint64_t k, uint64_t n, uint64_t* bytes) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    if (k % g.elems) return fail(RLXQ_E_SHAPE, "k=%llu is not a multiple of the block size %u",
                                 (unsigned long long)k, g.elems);
    if (n != 0 && k / g.elems > (UINT64_MAX / g.bytes) / n) return fail(RLXQ_E_SHAPE, "size overflow");
    *bytes = (k / g.elems) * n * g.bytes;
    return RLXQ_OK;
}

int rlxq_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, uint32_t x_dtype,
                         uint32_t y_dtype, size_t* bytes) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (!bytes) return fail(RLXQ_E_NULL, "bytes is null");
    if (k % g.elems) return fail(RLXQ_E_SHAPE, "k=%u is not a multiple of the block size %u", k, g.elems);
    *bytes = matmul_workspace_bytes(scheme, m, k, n, x_dtype, y_dtype);
    return RLXQ_OK;
}

int rlxq_dequant_f32(rlxq_stream_t stream, uint32_t scheme, const void* w_blocks, uint64_t n_elems,
                     float* out) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (n_elems % g.elems) return fail(RLXQ_E_SHAPE, "n_elems=%llu is not a multiple of the block size %u",
                                       (unsigned long long)n_elems, g.elems);
    if (n_elems == 0) return RLXQ_OK;
    if (!w_blocks || !out) return fail(RLXQ_E_NULL, "null buffer");
    if ((uintptr_t)w_blocks & 1u) return fail(RLXQ_E_ALIGN, "w_blocks must be 2-byte aligned");
    if ((uintptr_t)out & 15u) return fail(RLXQ_E_ALIGN, "out must be 16-byte aligned");
    return launch_dequant_f32((cudaStream_t)stream, scheme, (const uint8_t*)w_blocks, n_elems, out);
}

int rlxq_matmul(rlxq_stream_t stream, uint32_t scheme, const void* x, uint32_t x_dtype,
                const void* w_blocks, void* y, uint32_t y_dtype, uint32_t m, uint32_t k, uint32_t n,
                void* workspace, size_t workspace_bytes) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (k % g.elems) return fail(RLXQ_E_SHAPE, "k=%u is not a multiple of the block size %u", k, g.elems);
    if (m == 0 || n == 0) return RLXQ_OK;  // empty output
    if (!y) return fail(RLXQ_E_NULL, "y is null");
    return dispatch_matmul((cudaStream_t)stream, scheme, x, x_dtype == RLXQ_BF16, (const uint8_t*)w_blocks,
                           y, y_dtype == RLXQ_BF16, m, k, n, workspace, workspace_bytes);
}

int rlxq_device_status(int* device_error) {
    if (!device_error) return fail(RLXQ_E_NULL, "device_error is null");
    int rc = staged_device_error(device_error);
    if (rc) return rc;
    if (*device_error) return fail(RLXQ_E_TIMEOUT, "a bounded device-side wait ran out (code %d)", *device_error);
    return RLXQ_OK;
}

int rlxq_init_device(void) { return staged_prepare_device(); }

uint64_t rlxq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int rlxq_set_option(const char* key, int64_t value) {
    if (!key) return fail(RLXQ_E_NULL, "key is null");
    if (!strcmp(key, "gemv_kernel")) { options().gemv_kernel = value; return RLXQ_OK; }
    if (!strcmp(key, "gemm_kernel")) { options().gemm_kernel = value; return RLXQ_OK; }
    if (!strcmp(key, "gemv_kslices")) { options().gemv_kslices = value; return RLXQ_OK; }
    if (!strcmp(key, "pdl")) { options().pdl = value; return RLXQ_OK; }
    if (!strcmp(key, "graph_fuse_ffn")) { options().graph_fuse_ffn = value ? 1 : 0; return RLXQ_OK; }
    if (!strcmp(key, "gemv_tc_ctas")) { options().gemv_tc_ctas = value < 1 ? 1 : (value > 2 ? 2 : value); return RLXQ_OK; }
    if (!strcmp(key, "gemv_chain")) { options().gemv_chain = value ? 1 : 0; return RLXQ_OK; }
    if (!strcmp(key, "tp_fused")) { options().tp_fused = value ? 1 : 0; return RLXQ_OK; }
    if (!strcmp(key, "gemm_pair")) {
        if (value < 0 || value > 2) return fail(RLXQ_E_ARG, "gemm_pair is 0, 1 or 2");
        options().gemm_pair = value;
        return RLXQ_OK;
    }
    if (!strcmp(key, "tp_spin_limit")) {
        if (value < 1 || value > (1ll << 30)) return fail(RLXQ_E_ARG, "tp_spin_limit must be in [1, 2^30]");
        options().tp_spin_limit = value;
        return RLXQ_OK;
    }
    if (!strcmp(key, "gemv_early")) { options().gemv_early = value < 0 ? 0 : value; return RLXQ_OK; }
    if (!strcmp(key, "gemv_inline_q")) {
        if (value < 0 || value > 2) return fail(RLXQ_E_ARG, "gemv_inline_q must be 0, 1 or 2");
        options().gemv_inline_q = value;
        return RLXQ_OK;
    }
    if (!strcmp(key, "gemm_streamk")) {
        if (value < 0 || value > 2) return fail(RLXQ_E_ARG, "gemm_streamk must be 0, 1 or 2");
        options().gemm_streamk = value;
        return RLXQ_OK;
    }
    if (!strcmp(key, "gemm_tile_x")) {
        if (value != 0 && value != 128 && value != 256) return fail(RLXQ_E_ARG, "gemm_tile_x must be 0, 128 or 256");
        options().gemm_tile_x = value;
        return RLXQ_OK;
    }
    return fail(RLXQ_E_ARG, "unknown option '%s'", key);
}

int rlxq_get_option(const char* key, int64_t* value) {
    if (!key || !value) return fail(RLXQ_E_NULL, "null argument");
    if (!strcmp(key, "gemv_kernel")) { *value = options().gemv_kernel; return RLXQ_OK; }
    if (!strcmp(key, "gemm_kernel")) { *value = options().gemm_kernel; return RLXQ_OK; }
    if (!strcmp(key, "gemv_kslices")) { *value = options().gemv_kslices; return RLXQ_OK; }
    if (!strcmp(key, "pdl")) { *value = options().pdl; return RLXQ_OK; }
    if (!strcmp(key, "graph_fuse_ffn")) { *value = options().graph_fuse_ffn; return RLXQ_OK; }
    if (!strcmp(key, "gemv_tc_ctas")) { *value = options().gemv_tc_ctas; return RLXQ_OK; }
    if (!strcmp(key, "gemv_chain")) { *value = options().gemv_chain; return RLXQ_OK; }
    if (!strcmp(key, "tp_fused")) { *value = options().tp_fused; return RLXQ_OK; }
    if (!strcmp(key, "gemm_pair")) { *value = options().gemm_pair; return RLXQ_OK; }
    if (!strcmp(key, "gemm_pair_clusters")) { *value = options().gemm_pair_clusters; return RLXQ_OK; }
    if (!strcmp(key, "tp_spin_limit")) { *value = options().tp_spin_limit; return RLXQ_OK; }
    if (!strcmp(key, "gemv_early")) { *value = options().gemv_early; return RLXQ_OK; }
    if (!strcmp(key, "gemv_inline_q")) { *value = options().gemv_inline_q; return RLXQ_OK; }
    if (!strcmp(key, "gemm_streamk")) { *value = options().gemm_streamk; return RLXQ_OK; }
    if (!strcmp(key, "gemm_tile_x")) { *value = options().gemm_tile_x; return RLXQ_OK; }
    return fail(RLXQ_E_ARG, "unknown option '%s'", key);
}

}  // extern "C"
