#include "tensormap.cuh"

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace rlxq {

// Encoded maps are kept per (kind, base address, extents, box): a weight is multiplied thousands of times with the
// same map, and in stream mode (no graph replay) every call would otherwise pay the driver's encoder again.  A map
// holds no reference to the memory it describes, only its address and shape, so an entry stays valid when the
// buffer is freed and an identical one is later allocated at the same address.
namespace {
struct MapKey {
    uint64_t kind, base, d0, d1, b0, b1;
    bool operator==(const MapKey& o) const { return !memcmp(this, &o, sizeof(MapKey)); }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = 0x9E3779B97F4A7C15ull;
        const uint64_t v[6] = {k.kind, k.base, k.d0, k.d1, k.b0, k.b1};
        for (uint64_t x : v) { h ^= x + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); }
        return (size_t)h;
    }
};
constexpr size_t kMapCacheEntries = 8192;   // 128 bytes each; emptied when full
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash>& map_cache() {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> c;
    return c;
}
bool cache_lookup(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> g(g_map_mutex);
    auto it = map_cache().find(k);
    if (it == map_cache().end()) return false;
    *out = it->second;
    return true;
}
void cache_store(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> g(g_map_mutex);
    if (map_cache().size() >= kMapCacheEntries) map_cache().clear();
    map_cache()[k] = m;
}
}  // namespace

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
    const MapKey key{1, (uint64_t)(uintptr_t)base, row_bytes, n_rows, box_elems, box_rows};
    if (cache_lookup(key, map)) return RLXQ_OK;
    const cuuint64_t dims[2] = {row_bytes / 8, n_rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_elems, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    cache_store(key, *map);
    return RLXQ_OK;
}

int encode_bf16_kmajor_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if ((uintptr_t)base & 15u) return fail(RLXQ_E_ALIGN, "TMA needs a 16-byte aligned matrix");
    if ((cols * 2) % 16 || box_rows > 256) return fail(RLXQ_E_SHAPE, "matrix cannot be tiled for TMA");
    const MapKey key{2, (uint64_t)(uintptr_t)base, cols, rows, 64, box_rows};
    if (cache_lookup(key, map)) return RLXQ_OK;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RLXQ_E_CUDA, "cuTensorMapEncodeTiled(bf16) failed with %d", (int)r);
    cache_store(key, *map);
    return RLXQ_OK;
}

}  // namespace rlxq
