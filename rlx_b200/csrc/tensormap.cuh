// Tiled tensor maps for TMA (cp.async.bulk.tensor), encoded through the driver entry point so
// the library links against the CUDA runtime only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace rlxq {

// A packed weight W[n, row_bytes] seen as a 2-D array of 8-byte elements; one box is `box_rows`
// rows by `box_elems` elements (box_elems * 8 a multiple of 16, box_elems <= 256).  Elements
// outside the array read as zero, which is what tail tiles and tail chunks rely on.
int encode_weight_map(CUtensorMap* map, const void* base, uint64_t n_rows, uint64_t row_bytes,
                      uint32_t box_elems, uint32_t box_rows);

// A bf16 matrix X[rows, cols] (row-major) with 128-byte swizzled boxes of box_rows x 64 elements,
// the K-major operand layout of tcgen05.mma.
int encode_bf16_kmajor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

#if defined(__CUDACC__)
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(mbar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
#endif

}  // namespace rlxq
