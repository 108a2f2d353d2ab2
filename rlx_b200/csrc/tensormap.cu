#include "tensormap.cuh"

#include <mutex>

namespace rlxq {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

int encode_weight_map(CUtensorMap* map, const void* base, uint64_t n_rows, uint64_t row_bytes,
                      uint32_t box_elems, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((uintptr_t)base & 15u) return fail(RLXQ_E_ALIGN, "TMA needs a 16-byte aligned weight");
    if (row_bytes % 16 || box_elems > 256 || box_rows > 256 || (box_elems * 8) % 16)
        return fail(RLXQ_E_SHAPE, "weight rows of %llu bytes cannot be tiled for TMA", (unsigned long long)row_bytes);
    const cuuint64_t dims[2] = {row_bytes / 8, n_rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_elems, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    return RLXQ_OK;
}

int encode_bf16_kmajor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((uintptr_t)base & 15u) return fail(RLXQ_E_ALIGN, "TMA needs a 16-byte aligned matrix");
    if ((cols * 2) % 16 || box_rows > 256) return fail(RLXQ_E_SHAPE, "matrix cannot be tiled for TMA");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled(bf16) failed with %d", (int)r);
    return RLXQ_OK;
}

}  // namespace rlxq
