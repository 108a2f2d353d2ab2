// Shared host-side plumbing for the rlxq library: status codes, error text, launch counting.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/rlxq.h"

namespace rlxq {

// Per-thread failure text returned by rlxq_last_error().
char* last_error_buf();
int fail(int status, const char* fmt, ...);

// Every kernel launch made by the library goes through this counter.
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Options set through rlxq_set_option.
struct Options {
    std::atomic<int64_t> gemv_kernel{0};
    std::atomic<int64_t> gemm_kernel{0};
    std::atomic<int64_t> gemv_kslices{0};
    std::atomic<int64_t> pdl{1};
    std::atomic<int64_t> gemm_tile_x{0};
    std::atomic<int64_t> gemm_streamk{0};
    std::atomic<int64_t> gemv_inline_q{0};
    std::atomic<int64_t> gemv_early{2};
    std::atomic<int64_t> tp_spin_limit{1 << 24};
    std::atomic<int64_t> gemv_tc_ctas{2};
    std::atomic<int64_t> gemm_pair{0};        // tcgen05 GEMM, two CTAs per MMA (cta_group::2): 0 = where it pays, 1 = never, 2 = wherever the shape allows
    std::atomic<int64_t> gemm_pair_clusters{0};   // read-only: clusters of two CTAs the device keeps resident (0 until the paired GEMM ran)
    std::atomic<int64_t> tp_fused{0};         // rlxq_tp_ffn_step: the down projection pushes its tiles and finishes the sum
    std::atomic<int64_t> gemv_chain{0};       // 1: rlxq_matmul_chain runs a chain as one cooperative kernel where it can
    std::atomic<int64_t> graph_fuse_ffn{1};
};
Options& options();

struct Geometry { uint32_t elems, bytes; };
inline bool geometry(uint32_t scheme, Geometry* g) {
    switch (scheme) {
        case RLXQ_Q4_K: *g = {256, 144}; return true;
        case RLXQ_Q6_K: *g = {256, 210}; return true;
        case RLXQ_Q4_0: *g = {32, 18}; return true;
        case RLXQ_Q8_0: *g = {32, 34}; return true;
        case RLXQ_Q5_K: *g = {256, 176}; return true;
        case RLXQ_Q8_K: *g = {256, 292}; return true;
        case RLXQ_Q2_K: *g = {256, 84}; return true;
        case RLXQ_Q3_K: *g = {256, 110}; return true;
        case RLXQ_Q4_1: *g = {32, 20}; return true;
        case RLXQ_Q5_0: *g = {32, 22}; return true;
        case RLXQ_Q5_1: *g = {32, 24}; return true;
        default: return false;
    }
}

// Checks the launch itself (not the execution): never synchronises.
inline int check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(RLXQ_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    return RLXQ_OK;
}

#define RLXQ_CUDA_TRY(expr)                                                              \
    do {                                                                                 \
        cudaError_t e__ = (expr);                                                        \
        if (e__ != cudaSuccess)                                                          \
            return ::rlxq::fail(RLXQ_E_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// Cached per-device properties (SM count), looked up without synchronising.
int sm_count();

}  // namespace rlxq
