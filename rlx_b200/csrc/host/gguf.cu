// GGUF container reader and file -> device upload (host code; see include/rlxq_gguf.h).
//
// Mirrors GgufFile::from_reader (rlx-gguf/src/lib.rs:246-318): magic, version 1..3 (v1 has 32-bit
// counts, string lengths and dimensions), kv_count metadata pairs, tensor_count table entries,
// data segment at the next multiple of general.alignment.  Unlike the reference the data segment
// is not read at open: tensors are fetched with pread when asked for.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <new>
#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "../../../include/rlxq_gguf.h"
#include "../common.cuh"

namespace rlxq {

constexpr uint32_t kGgufMagic = 0x46554747u;        // "GGUF"
constexpr uint64_t kGgufDefaultAlignment = 32;
constexpr size_t kStageBytes = 8u << 20;             // per pinned staging buffer
constexpr int kReaders = 4;                          // reader threads of a large upload (two buffers each)

struct MetaScalar { int kind; uint64_t u; int64_t i; double d; std::string s; };   // kind: 0 u, 1 i, 2 f, 3 bool, 4 str

// bytes_for (rlx-gguf/src/lib.rs:393-419): block elements / block bytes per GGML type, 0 = unknown size.
static bool ggml_block(uint32_t t, uint32_t* elems, uint32_t* bytes, int32_t* scheme) {
    *scheme = -1;
    switch (t) {
        case 0: *elems = 1; *bytes = 4; return true;                       // F32
        case 1: case 30: *elems = 1; *bytes = 2; return true;              // F16, BF16
        case 2: *elems = 32; *bytes = 18; *scheme = RLXQ_Q4_0; return true;
        case 3: *elems = 32; *bytes = 20; *scheme = RLXQ_Q4_1; return true;
        case 6: *elems = 32; *bytes = 22; *scheme = RLXQ_Q5_0; return true;
        case 7: *elems = 32; *bytes = 24; *scheme = RLXQ_Q5_1; return true;
        case 8: *elems = 32; *bytes = 34; *scheme = RLXQ_Q8_0; return true;
        case 10: *elems = 256; *bytes = 84; *scheme = RLXQ_Q2_K; return true;
        case 11: *elems = 256; *bytes = 110; *scheme = RLXQ_Q3_K; return true;
        case 12: *elems = 256; *bytes = 144; *scheme = RLXQ_Q4_K; return true;
        case 13: *elems = 256; *bytes = 176; *scheme = RLXQ_Q5_K; return true;
        case 14: *elems = 256; *bytes = 210; *scheme = RLXQ_Q6_K; return true;
        case 15: *elems = 256; *bytes = 292; *scheme = RLXQ_Q8_K; return true;
        default: return false;
    }
}

// GgmlType::from_u32 (rlx-gguf/src/lib.rs:101-139): the ids the reference accepts.
static bool ggml_type_known(uint32_t t) {
    return t <= 3 || (t >= 6 && t <= 30) || t == 34 || t == 35 || (t >= 39 && t <= 41);
}

struct Reader {
    int fd;
    uint64_t pos, size;
    bool ok = true;
    bool read(void* dst, size_t n) {
        if (!ok || pos + n > size) { ok = false; return false; }
        size_t got = 0;
        while (got < n) {
            const ssize_t r = pread(fd, (char*)dst + got, n - got, (off_t)(pos + got));
            if (r <= 0) { ok = false; return false; }
            got += (size_t)r;
        }
        pos += n;
        return true;
    }
    template <typename T> T get() { T v{}; read(&v, sizeof(T)); return v; }     // little-endian host
    uint64_t len(uint32_t version) { return version == 1 ? get<uint32_t>() : get<uint64_t>(); }
    std::string str(uint32_t version) {
        const uint64_t n = len(version);
        if (!ok || n > size - pos) { ok = false; return {}; }
        std::string s((size_t)n, '\0');
        read(s.data(), (size_t)n);
        return s;
    }
};

static const size_t kScalarSize[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

}  // namespace rlxq

using namespace rlxq;

struct rlxq_gguf {
    int fd = -1;
    uint64_t file_size = 0, data_start = 0, alignment = kGgufDefaultAlignment;
    uint32_t version = 0;
    std::vector<std::string> names;
    std::map<std::string, rlxq_gguf_tensor> tensors;
    std::map<std::string, MetaScalar> meta;
    void* stage[2 * kReaders] = {};
    cudaEvent_t done[2 * kReaders] = {};
    ~rlxq_gguf() {
        for (int i = 0; i < 2 * kReaders; ++i) {
            if (done[i]) cudaEventDestroy(done[i]);
            if (stage[i]) cudaFreeHost(stage[i]);
        }
        if (fd >= 0) close(fd);
    }
};

static bool read_scalar(Reader& r, uint32_t ty, uint32_t version, MetaScalar* out) {
    switch (ty) {
        case 0: *out = {0, r.get<uint8_t>(), 0, 0, {}}; break;
        case 1: *out = {1, 0, r.get<int8_t>(), 0, {}}; break;
        case 2: *out = {0, r.get<uint16_t>(), 0, 0, {}}; break;
        case 3: *out = {1, 0, r.get<int16_t>(), 0, {}}; break;
        case 4: *out = {0, r.get<uint32_t>(), 0, 0, {}}; break;
        case 5: *out = {1, 0, r.get<int32_t>(), 0, {}}; break;
        case 6: *out = {2, 0, 0, r.get<float>(), {}}; break;
        case 7: *out = {3, (uint64_t)(r.get<uint8_t>() != 0), 0, 0, {}}; break;
        case 8: *out = {4, 0, 0, 0, r.str(version)}; break;
        case 10: *out = {0, r.get<uint64_t>(), 0, 0, {}}; break;
        case 11: *out = {1, 0, r.get<int64_t>(), 0, {}}; break;
        case 12: *out = {2, 0, 0, r.get<double>(), {}}; break;
        default: return false;
    }
    return r.ok;
}

extern "C" int rlxq_gguf_open(const char* path, rlxq_gguf** out) {
    if (!path || !out) return fail(RLXQ_E_NULL, "null argument");
    *out = nullptr;
    rlxq_gguf* f = new (std::nothrow) rlxq_gguf();
    if (!f) return fail(RLXQ_E_ARG, "out of host memory");
    f->fd = open(path, O_RDONLY);
    struct stat st;
    if (f->fd < 0 || fstat(f->fd, &st) != 0) { delete f; return fail(RLXQ_E_ARG, "cannot open %s", path); }
    f->file_size = (uint64_t)st.st_size;
    Reader r{f->fd, 0, f->file_size};
    const uint32_t magic = r.get<uint32_t>();
    if (!r.ok || magic != kGgufMagic) { delete f; return fail(RLXQ_E_ARG, "%s is not a GGUF file (magic %#x)", path, magic); }
    f->version = r.get<uint32_t>();
    if (!r.ok || f->version < 1 || f->version > 3) { const uint32_t v = f->version; delete f; return fail(RLXQ_E_ARG, "unsupported GGUF version %u", v); }
    const uint64_t tensor_count = r.len(f->version), kv_count = r.len(f->version);
    for (uint64_t i = 0; i < kv_count && r.ok; ++i) {
        const std::string key = r.str(f->version);
        const uint32_t ty = r.get<uint32_t>();
        if (!r.ok) break;
        if (ty == 9) {                                   // array: element type, count, elements (not nested)
            const uint32_t inner = r.get<uint32_t>();
            const uint64_t n = r.len(f->version);
            if (inner == 9 || inner > 12) { delete f; return fail(RLXQ_E_ARG, "metadata '%s': bad array element type %u", key.c_str(), inner); }
            if (inner == 8) {
                for (uint64_t j = 0; j < n && r.ok; ++j) {
                    const uint64_t l = r.len(f->version);
                    if (l > r.size - r.pos) r.ok = false; else r.pos += l;
                }
            } else {
                uint64_t bytes = 0;      // a count that wraps the product is a malformed header, not a short array
                if (__builtin_mul_overflow(n, (uint64_t)kScalarSize[inner], &bytes) || bytes > r.size - r.pos) r.ok = false;
                else r.pos += bytes;
            }
        } else {
            MetaScalar v;
            if (!read_scalar(r, ty, f->version, &v)) {
                if (r.ok) { delete f; return fail(RLXQ_E_ARG, "metadata '%s': unknown value type %u", key.c_str(), ty); }
                break;
            }
            f->meta[key] = v;
        }
    }
    auto al = f->meta.find("general.alignment");       // MetaValue::as_u64 of general.alignment, else 32
    if (al != f->meta.end() && (al->second.kind == 0 || (al->second.kind == 1 && al->second.i >= 0))) {
        const uint64_t a = al->second.kind == 0 ? al->second.u : (uint64_t)al->second.i;
        if (a) f->alignment = a;
    }
    for (uint64_t i = 0; i < tensor_count && r.ok; ++i) {
        const std::string name = r.str(f->version);
        rlxq_gguf_tensor t{};
        t.n_dims = r.get<uint32_t>();
        if (!r.ok || t.n_dims > 4) { delete f; return fail(RLXQ_E_ARG, "tensor '%s': %u dimensions", name.c_str(), t.n_dims); }
        uint64_t elems = 1;
        bool wraps = false;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = r.len(f->version);
            wraps = __builtin_mul_overflow(elems, t.dims[d], &elems) || wraps;
        }
        t.ggml_type = r.get<uint32_t>();
        t.offset = r.get<uint64_t>();
        if (!r.ok) break;
        if (!ggml_type_known(t.ggml_type)) { delete f; return fail(RLXQ_E_ARG, "tensor '%s': unknown ggml type %u", name.c_str(), t.ggml_type); }
        if (wraps) { delete f; return fail(RLXQ_E_ARG, "tensor '%s': element count overflows 64 bits (malformed GGUF header)", name.c_str()); }
        uint32_t be = 0, bb = 0;
        if (ggml_block(t.ggml_type, &be, &bb, &t.scheme) && elems % be == 0 &&
            __builtin_mul_overflow(elems / be, (uint64_t)bb, &t.bytes)) {
            delete f;
            return fail(RLXQ_E_ARG, "tensor '%s': byte size overflows 64 bits (malformed GGUF header)", name.c_str());
        }
        // a repeated name replaces the earlier entry, as inserting into the reference's map does
        // (rlx-gguf/src/lib.rs:246-318); it is listed once
        if (f->tensors.find(name) == f->tensors.end()) f->names.push_back(name);
        f->tensors[name] = t;
    }
    if (!r.ok) { delete f; return fail(RLXQ_E_ARG, "%s: truncated or malformed GGUF header", path); }
    f->data_start = (r.pos + f->alignment - 1) / f->alignment * f->alignment;
    *out = f;
    return RLXQ_OK;
}

extern "C" void rlxq_gguf_close(rlxq_gguf* f) { delete f; }
extern "C" uint32_t rlxq_gguf_version(const rlxq_gguf* f) { return f ? f->version : 0; }
extern "C" uint64_t rlxq_gguf_alignment(const rlxq_gguf* f) { return f ? f->alignment : 0; }
extern "C" uint64_t rlxq_gguf_tensor_count(const rlxq_gguf* f) { return f ? f->names.size() : 0; }
extern "C" uint64_t rlxq_gguf_data_start(const rlxq_gguf* f) { return f ? f->data_start : 0; }

extern "C" int rlxq_gguf_tensor_name(const rlxq_gguf* f, uint64_t index, const char** name) {
    if (!f || !name) return fail(RLXQ_E_NULL, "null argument");
    if (index >= f->names.size()) return fail(RLXQ_E_ARG, "tensor index %llu out of range", (unsigned long long)index);
    *name = f->names[index].c_str();
    return RLXQ_OK;
}

extern "C" int rlxq_gguf_find(const rlxq_gguf* f, const char* name, rlxq_gguf_tensor* info) {
    if (!f || !name || !info) return fail(RLXQ_E_NULL, "null argument");
    auto it = f->tensors.find(name);
    if (it == f->tensors.end()) return fail(RLXQ_E_ARG, "tensor not found: %s", name);
    *info = it->second;
    return RLXQ_OK;
}

extern "C" int rlxq_gguf_meta_u64(const rlxq_gguf* f, const char* key, uint64_t* value) {
    if (!f || !key || !value) return fail(RLXQ_E_NULL, "null argument");
    auto it = f->meta.find(key);
    if (it == f->meta.end()) return fail(RLXQ_E_ARG, "no metadata key '%s'", key);
    const MetaScalar& v = it->second;
    if (v.kind == 0 || v.kind == 3) { *value = v.u; return RLXQ_OK; }
    if (v.kind == 1 && v.i >= 0) { *value = (uint64_t)v.i; return RLXQ_OK; }
    return fail(RLXQ_E_ARG, "metadata '%s' is not a non-negative integer", key);
}

extern "C" int rlxq_gguf_meta_str(const rlxq_gguf* f, const char* key, const char** value) {
    if (!f || !key || !value) return fail(RLXQ_E_NULL, "null argument");
    auto it = f->meta.find(key);
    if (it == f->meta.end() || it->second.kind != 4) return fail(RLXQ_E_ARG, "no string metadata '%s'", key);
    *value = it->second.s.c_str();
    return RLXQ_OK;
}

// tensor_bytes (rlx-gguf/src/lib.rs:355-371): range check against the data segment
static int tensor_range(const rlxq_gguf* f, const char* name, uint64_t bytes, uint64_t* file_off) {
    auto it = f->tensors.find(name);
    if (it == f->tensors.end()) return fail(RLXQ_E_ARG, "tensor not found: %s", name);
    const rlxq_gguf_tensor& t = it->second;
    if (t.bytes == 0) return fail(RLXQ_E_SHAPE, "tensor %s: element count not aligned to its block, or a type without a known size", name);
    if (bytes != t.bytes) return fail(RLXQ_E_SHAPE, "tensor %s holds %llu bytes, %llu asked for", name, (unsigned long long)t.bytes, (unsigned long long)bytes);
    const uint64_t start = f->data_start + t.offset;
    if (start < f->data_start || start + bytes < start || start + bytes > f->file_size)
        return fail(RLXQ_E_SHAPE, "tensor %s extends past the data segment", name);
    *file_off = start;
    return RLXQ_OK;
}

static int pread_all(int fd, void* dst, size_t n, uint64_t off) {
    size_t got = 0;
    while (got < n) {
        const ssize_t r = pread(fd, (char*)dst + got, n - got, (off_t)(off + got));
        if (r <= 0) return fail(RLXQ_E_ARG, "read failed at offset %llu", (unsigned long long)(off + got));
        got += (size_t)r;
    }
    return RLXQ_OK;
}

extern "C" int rlxq_gguf_read_tensor(const rlxq_gguf* f, const char* name, void* host_dst, uint64_t bytes) {
    if (!f || !name || (!host_dst && bytes)) return fail(RLXQ_E_NULL, "null argument");
    uint64_t off = 0;
    int rc = tensor_range(f, name, bytes, &off);
    if (rc) return rc;
    return pread_all(f->fd, host_dst, (size_t)bytes, off);
}

// One reader: chunks c = first, first + step, ... of the tensor, through its own pair of staging buffers.
static int upload_chunks(rlxq_gguf* f, int dev, int reader, uint64_t first, uint64_t step, uint64_t off, uint64_t bytes,
                         uint8_t* device_dst, cudaStream_t s) {
    RLXQ_CUDA_TRY(cudaSetDevice(dev));
    bool used[2] = {false, false};
    int b = 0;
    for (uint64_t c = first; c * kStageBytes < bytes; c += step, b ^= 1) {
        const uint64_t pos = c * kStageBytes;
        const size_t n = (size_t)((bytes - pos < kStageBytes) ? bytes - pos : kStageBytes);
        const int slot = 2 * reader + b;
        if (used[b]) RLXQ_CUDA_TRY(cudaEventSynchronize(f->done[slot]));   // the copy out of this buffer has finished
        int rc = pread_all(f->fd, f->stage[slot], n, off + pos);           // overlaps the copies out of the other buffers
        if (rc) return rc;
        RLXQ_CUDA_TRY(cudaMemcpyAsync(device_dst + pos, f->stage[slot], n, cudaMemcpyHostToDevice, s));
        RLXQ_CUDA_TRY(cudaEventRecord(f->done[slot], s));
        used[b] = true;
    }
    for (b = 0; b < 2; ++b)
        if (used[b]) RLXQ_CUDA_TRY(cudaEventSynchronize(f->done[2 * reader + b]));   // staging may be reused by the next call
    return RLXQ_OK;
}

extern "C" int rlxq_gguf_upload_tensor(rlxq_gguf* f, const char* name, void* device_dst, uint64_t bytes,
                                       rlxq_stream_t stream) {
    if (!f || !name || (!device_dst && bytes)) return fail(RLXQ_E_NULL, "null argument");
    uint64_t off = 0;
    int rc = tensor_range(f, name, bytes, &off);
    if (rc) return rc;
    // a single reader saturates at the speed of one core copying out of the page cache (about 10 GB/s);
    // large tensors are read by several threads, each feeding its own copies into the caller's stream
    const int readers = bytes >= 8 * kStageBytes ? kReaders : 1;
    for (int i = 0; i < 2 * readers; ++i) {
        if (!f->stage[i]) RLXQ_CUDA_TRY(cudaHostAlloc(&f->stage[i], kStageBytes, cudaHostAllocDefault));
        if (!f->done[i]) RLXQ_CUDA_TRY(cudaEventCreateWithFlags(&f->done[i], cudaEventDisableTiming));
    }
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    cudaStream_t s = (cudaStream_t)stream;
    if (readers == 1) return upload_chunks(f, dev, 0, 0, 1, off, bytes, (uint8_t*)device_dst, s);
    std::atomic<int> status{RLXQ_OK};
    char first_error[512] = {0};
    std::vector<std::thread> pool;
    for (int t = 0; t < readers; ++t)
        pool.emplace_back([&, t]() {
            const int r = upload_chunks(f, dev, t, (uint64_t)t, (uint64_t)readers, off, bytes, (uint8_t*)device_dst, s);
            int expect = RLXQ_OK;
            if (r && status.compare_exchange_strong(expect, r)) strncpy(first_error, rlxq_last_error(), sizeof(first_error) - 1);
        });
    for (auto& th : pool) th.join();
    if (status.load()) return fail(status.load(), "%s", first_error);
    return RLXQ_OK;
}
