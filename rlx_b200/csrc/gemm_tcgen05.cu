// Prefill GEMM (m >= 128 activation rows) on the 5th-generation tensor cores: tcgen05.mma with
// the accumulator AND the dequantised weight operand in tensor memory, activations by TMA.
//
// y[m,n] = x[m,k] . W^T is computed transposed, tile by tile: D[128 weight rows, 256 activation
// rows] += A[128, 64] . B[256, 64]^T per 64-wide k block.
//   * A (weights) never exists in memory.  The raw GGUF blocks of 128 rows x 256 weights arrive in
//     shared memory through one 2-D TMA box; eight decode warps, twelve for Q6_K (one thread per weight row, which
//     is also that thread's tensor-memory lane) turn 64 weights at a time into bf16(d * q) in
//     registers and store them to tensor memory with tcgen05.st.  d * q is formed in f32 exactly as
//     the reference decoder does (rlx-gguf/src/lib.rs:574-597, 974-1013) and rounded once to bf16.
//   * B (activations, bf16, K-major) comes through TMA with the 128-byte swizzle the MMA's
//     shared-memory descriptor expects.
//   * One thread issues four tcgen05.mma (k = 16 each) per stage and tcgen05.commit releases the
//     stage's shared memory and tensor-memory columns through an mbarrier.
//   * Four epilogue warps read the 128 x 256 f32 accumulator with tcgen05.ld and write y (f32 or
//     bf16, round to nearest even); consecutive lanes hold consecutive n, so stores coalesce.
// Persistent CTAs, one per SM, walk the tiles with the activation tile index fastest so that the
// CTAs working at any moment share a handful of weight tiles (L2 reuse) and x stays L2 resident.
//
// Every wait is bounded: on a timeout the kernel records an error word, stops issuing, lets the
// copies in flight land, frees its tensor memory and returns.
//
// Replaces the reference's dequantise-to-f32-scratch + cublasSgemm for m > 8
// (rlx-cuda/src/gguf_gpu.rs:62-134), which also reads the scratch with the wrong leading
// dimension for n > 1.
#include <cuda_bf16.h>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "staged_common.cuh"
#include "tc_common.cuh"
#include "tensormap.cuh"

namespace rlxq {

constexpr uint32_t kGemmTileW = 128;    // weight rows per tile (MMA M, tensor-memory lanes)
// activation rows per tile (MMA N): a template parameter, 256, or 128 when that fills more SMs
constexpr uint32_t kGemmBK = 64;        // k per pipeline stage (one 128-byte swizzled row of bf16)
constexpr uint32_t kGemmMaxStages = 6;  // B shared-memory stages == A tensor-memory stages (4 or 5, by format)
constexpr uint32_t kGemmRawStages = 2;  // raw weight boxes (256 weights of 128 rows each)

// Instruction descriptor: f32 accumulator, bf16 A and B, both K-major, M = 128, N = 256.
template <uint32_t TX> struct GemmIdesc {
    static constexpr uint32_t value = (1u << 4) | (1u << 7) | (1u << 10) | ((TX >> 3) << 17) | ((kGemmTileW >> 4) << 24);
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);       // .x (low half) = lo
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- weight decode: 64 consecutive weights of one row -> 32 bf16 pairs ------------------------
// The raw box holds 256 weights of 128 rows; RAW_ROW bytes per row (an odd number of 16-byte
// chunks, so one-row-per-lane 128-bit reads do not conflict).  `S` = which 64 of the 256.
template <uint32_t SCHEME> struct GemmRaw;
// GROUPS: decode warp groups (four warps each).  Two keep pace with the MMA for the cheap decoders (more only
// add contention: measured 917 against 950 TFLOP/s for Q8_0); Q6_K's decoder is the slow one and gains 10 % from three.
template <> struct GemmRaw<RLXQ_Q4_0> { static constexpr uint32_t ROW = 144, STAGES = 5, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q8_0> { static constexpr uint32_t ROW = 272, STAGES = 4, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q4_K> { static constexpr uint32_t ROW = 144, STAGES = 5, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q5_K> { static constexpr uint32_t ROW = 176, STAGES = 4, GROUPS = 2; };
// Q6_K super-blocks are 210 bytes: group g of a row starts at byte 210 g, which is only 2-byte aligned.
// The box starts at the 16-byte boundary below it and is 240 bytes wide (15 chunks: conflict-free, and
// 14 + 210 <= 240); the decoder is compiled for each of the eight possible offsets 2 (g mod 8).
template <> struct GemmRaw<RLXQ_Q6_K> { static constexpr uint32_t ROW = 240, STAGES = 4, GROUPS = 3; };
// Q2_K super-blocks are 84 bytes (group g starts 4 (g mod 4) bytes past a 16-byte boundary: a 112-byte box covers
// 12 + 84), Q3_K's 110 bytes (2-byte aligned only, like Q6_K: a 144-byte box covers 14 + 110).
template <> struct GemmRaw<RLXQ_Q2_K> { static constexpr uint32_t ROW = 112, STAGES = 5, GROUPS = 2; };
// The 32-weight container types: Q4_1 (20-byte blocks: 160 bytes per 256 weights, fetched as 176 so that a row of the
// box is an odd number of 16-byte chunks), Q5_0 (22: 176), Q5_1 (24: 192, fetched as 208).
template <> struct GemmRaw<RLXQ_Q4_1> { static constexpr uint32_t ROW = 176, STAGES = 5, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q5_0> { static constexpr uint32_t ROW = 176, STAGES = 4, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q5_1> { static constexpr uint32_t ROW = 208, STAGES = 4, GROUPS = 2; };
// Q8_K: 292 bytes (f32 d, 256 int8, 16 int16 block sums that the decoder does not read); 4 (g mod 4) bytes past a
// boundary, a 304-byte box (19 chunks) covers 12 + 292.
template <> struct GemmRaw<RLXQ_Q8_K> { static constexpr uint32_t ROW = 304, STAGES = 4, GROUPS = 2; };
template <> struct GemmRaw<RLXQ_Q3_K> { static constexpr uint32_t ROW = 144, STAGES = 5, GROUPS = 3; };
template <uint32_t SCHEME> __device__ __forceinline__ uint32_t gemm_raw_x(uint32_t g) {   // box start, 8-byte elements
    if (SCHEME == RLXQ_Q6_K) return ((210u * g) & ~15u) / 8u;
    if (SCHEME == RLXQ_Q2_K) return ((84u * g) & ~15u) / 8u;
    if (SCHEME == RLXQ_Q8_K) return ((292u * g) & ~15u) / 8u;
    if (SCHEME == RLXQ_Q4_1) return g * (160u / 8u);
    if (SCHEME == RLXQ_Q5_1) return g * (192u / 8u);
    if (SCHEME == RLXQ_Q3_K) return ((110u * g) & ~15u) / 8u;
    return g * (GemmRaw<SCHEME>::ROW / 8u);
}

// float(b) for b in 0..255 without the conversion unit: 0x4B000000 | b is 2^23 + b
__device__ __forceinline__ float u8_to_f32(uint32_t b) { return __uint_as_float(0x4B000000u | b) - 8388608.0f; }
// float(b) - OFF in one exact subtraction (OFF a small integer)
template <int OFF>
__device__ __forceinline__ float u8_minus(uint32_t b) { return __uint_as_float(0x4B000000u | b) - (8388608.0f + (float)OFF); }

// The decoders are bound by instruction issue (two decode warps share a scheduler with the MMA pace of one
// k block per 512 cycles), so they work on pairs: one byte-permute per weight builds the float 2^23 + byte
// straight from the raw word, and the arithmetic uses the packed two-float instructions of this architecture.
// Every step rounds exactly as the scalar f32 expression it replaces.
__device__ __forceinline__ uint64_t f32x2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f32x2_splat(float f) { return f32x2(__float_as_uint(f), __float_as_uint(f)); }
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// two floats -> bf16 pair, the first in the low half
__device__ __forceinline__ uint32_t bf16x2_of(uint64_t v) {
    uint32_t lo, hi, d;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
    return d;
}
// bytes 2 H and 2 H + 1 of u -> (2^23 + byte, 2^23 + byte)
template <int H> __device__ __forceinline__ uint64_t magic_pair(uint32_t u) {
    return f32x2(__byte_perm(u, 0x4B000000u, 0x7440 + 2 * H), __byte_perm(u, 0x4B000000u, 0x7441 + 2 * H));
}
// (byte - OFF) * scale for bytes 2 H, 2 H + 1 of u, as a bf16 pair
template <int H> __device__ __forceinline__ uint32_t scaled_pair(uint32_t u, uint64_t neg_off, uint64_t scale) {
    return bf16x2_of(mul_f32x2(add_f32x2(magic_pair<H>(u), neg_off), scale));
}

template <uint32_t SCHEME, int S> struct Decode64;

template <int S> struct Decode64<RLXQ_Q4_0, S> {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        // blocks 2S and 2S+1 = bytes [36 S, 36 S + 36): read the 16-byte chunks that cover them
        constexpr int B0 = 36 * S, C0 = B0 / 16, C1 = (B0 + 36 + 15) / 16, W0 = B0 / 4 - 4 * C0;
        uint32_t w[4 * (C1 - C0) + 1];
#pragma unroll
        for (int c = C0; c < C1; ++c) {
            const uint4 t = *reinterpret_cast<const uint4*>(row + 16 * c);
            w[4 * (c - C0)] = t.x; w[4 * (c - C0) + 1] = t.y; w[4 * (c - C0) + 2] = t.z; w[4 * (c - C0) + 3] = t.w;
        }
        w[4 * (C1 - C0)] = 0;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            uint32_t qs[4], dbits;
            if (blk == 0) {   // starts on word W0: d in the low half, quants shifted by two bytes
                dbits = w[W0] & 0xFFFFu;
#pragma unroll
                for (int i = 0; i < 4; ++i) qs[i] = __funnelshift_r(w[W0 + i], w[W0 + i + 1], 16);
            } else {          // starts two bytes into word W0 + 4
                dbits = w[W0 + 4] >> 16;
#pragma unroll
                for (int i = 0; i < 4; ++i) qs[i] = w[W0 + 5 + i];
            }
            const uint64_t d2 = f32x2_splat(f16_bits_to_f32(dbits)), off = f32x2_splat(-(8388608.0f + 8.0f));
#pragma unroll
            for (int i = 0; i < 4; ++i) {   // weights 4i..4i+3: low nibbles of bytes 4i..; weights 16+4i..: high nibbles
                const uint32_t lo = qs[i] & 0x0F0F0F0Fu, hi = (qs[i] >> 4) & 0x0F0F0F0Fu;
                v[16 * blk + 2 * i] = scaled_pair<0>(lo, off, d2);
                v[16 * blk + 2 * i + 1] = scaled_pair<1>(lo, off, d2);
                v[16 * blk + 8 + 2 * i] = scaled_pair<0>(hi, off, d2);
                v[16 * blk + 8 + 2 * i + 1] = scaled_pair<1>(hi, off, d2);
            }
        }
    }
};

template <int S> struct Decode64<RLXQ_Q8_0, S> {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        // blocks 2S and 2S+1 = bytes [68 S, 68 S + 68)
        constexpr int B0 = 68 * S, C0 = B0 / 16, C1 = (B0 + 68 + 15) / 16, W0 = B0 / 4 - 4 * C0;
        uint32_t w[4 * (C1 - C0) + 1];
#pragma unroll
        for (int c = C0; c < C1; ++c) {
            const uint4 t = *reinterpret_cast<const uint4*>(row + 16 * c);
            w[4 * (c - C0)] = t.x; w[4 * (c - C0) + 1] = t.y; w[4 * (c - C0) + 2] = t.z; w[4 * (c - C0) + 3] = t.w;
        }
        w[4 * (C1 - C0)] = 0;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            uint32_t q[8], dbits;
            if (blk == 0) {
                dbits = w[W0] & 0xFFFFu;
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[W0 + i], w[W0 + i + 1], 16);
            } else {
                dbits = w[W0 + 8] >> 16;
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = w[W0 + 9 + i];
            }
            const uint64_t d2 = f32x2_splat(f16_bits_to_f32(dbits)), off = f32x2_splat(-(8388608.0f + 128.0f));
#pragma unroll
            for (int i = 0; i < 8; ++i) {   // int8 -> (q + 128) unsigned -> float, minus 128
                const uint32_t u = q[i] ^ 0x80808080u;
                v[16 * blk + 2 * i] = scaled_pair<0>(u, off, d2);
                v[16 * blk + 2 * i + 1] = scaled_pair<1>(u, off, d2);
            }
        }
    }
};

template <int S> struct Decode64<RLXQ_Q4_K, S> {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        const uint4 hd = *reinterpret_cast<const uint4*>(row);   // d, dmin, 12 scale bytes
        const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
        // sub-blocks 2S (low nibbles) and 2S+1 (high nibbles) of bytes [16 + 32 S, +32)
        uint32_t sc[2], mn[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = 2 * S + i;
            if (j < 4) {
                sc[i] = (hd.y >> (8 * j)) & 63u;
                mn[i] = (hd.z >> (8 * j)) & 63u;
            } else {
                sc[i] = ((hd.w >> (8 * (j - 4))) & 0x0Fu) | (((hd.y >> (8 * (j - 4) + 6)) & 3u) << 4);
                mn[i] = ((hd.w >> (8 * (j - 4) + 4)) & 0x0Fu) | (((hd.z >> (8 * (j - 4) + 6)) & 3u) << 4);
            }
        }
        const float dl = d * (float)sc[0], ml = dmin * (float)mn[0];
        const float dh = d * (float)sc[1], mh = dmin * (float)mn[1];
        const uint4 a = *reinterpret_cast<const uint4*>(row + 16 + 32 * S);
        const uint4 b = *reinterpret_cast<const uint4*>(row + 32 + 32 * S);
        const uint32_t qs[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const uint64_t off = f32x2_splat(-8388608.0f);
        const uint64_t dl2 = f32x2_splat(dl), ml2 = f32x2_splat(-ml), dh2 = f32x2_splat(dh), mh2 = f32x2_splat(-mh);
#pragma unroll
        for (int i = 0; i < 8; ++i) {       // scale * nibble - min, rounded after each step as the dequantiser does
            const uint32_t lo = qs[i] & 0x0F0F0F0Fu, hi = (qs[i] >> 4) & 0x0F0F0F0Fu;
            v[2 * i] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<0>(lo), off)), ml2));
            v[2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<1>(lo), off)), ml2));
            v[16 + 2 * i] = bf16x2_of(add_f32x2(mul_f32x2(dh2, add_f32x2(magic_pair<0>(hi), off)), mh2));
            v[16 + 2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(dh2, add_f32x2(magic_pair<1>(hi), off)), mh2));
        }
    }
};

// Q5_K: d | dmin | 12 scale bytes | qh[32] | qs[128] (rlx-gguf/src/lib.rs:1019-1068): Q4_K with bit j of
// qh[l] adding 16 to weight l of sub-block j.
template <int S> struct Decode64<RLXQ_Q5_K, S> {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        const uint4 hd = *reinterpret_cast<const uint4*>(row);
        const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
        uint32_t sc[2], mn[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int j = 2 * S + i;
            if (j < 4) {
                sc[i] = (hd.y >> (8 * j)) & 63u;
                mn[i] = (hd.z >> (8 * j)) & 63u;
            } else {
                sc[i] = ((hd.w >> (8 * (j - 4))) & 0x0Fu) | (((hd.y >> (8 * (j - 4) + 6)) & 3u) << 4);
                mn[i] = ((hd.w >> (8 * (j - 4) + 4)) & 0x0Fu) | (((hd.z >> (8 * (j - 4) + 6)) & 3u) << 4);
            }
        }
        const float dl = d * (float)sc[0], ml = dmin * (float)mn[0];
        const float dh = d * (float)sc[1], mh = dmin * (float)mn[1];
        const uint4 ha = *reinterpret_cast<const uint4*>(row + 16), hb = *reinterpret_cast<const uint4*>(row + 32);
        const uint4 a = *reinterpret_cast<const uint4*>(row + 48 + 32 * S);
        const uint4 b = *reinterpret_cast<const uint4*>(row + 64 + 32 * S);
        const uint32_t qs[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const uint32_t qh[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
        const uint64_t off = f32x2_splat(-8388608.0f);
        const uint64_t dl2 = f32x2_splat(dl), ml2 = f32x2_splat(-ml), dh2 = f32x2_splat(dh), mh2 = f32x2_splat(-mh);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lo = (qs[i] & 0x0F0F0F0Fu) | (((qh[i] >> (2 * S)) & 0x01010101u) << 4);
            const uint32_t hi = ((qs[i] >> 4) & 0x0F0F0F0Fu) | (((qh[i] >> (2 * S + 1)) & 0x01010101u) << 4);
            v[2 * i] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<0>(lo), off)), ml2));
            v[2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<1>(lo), off)), ml2));
            v[16 + 2 * i] = bf16x2_of(add_f32x2(mul_f32x2(dh2, add_f32x2(magic_pair<0>(hi), off)), mh2));
            v[16 + 2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(dh2, add_f32x2(magic_pair<1>(hi), off)), mh2));
        }
    }
};

// Words of a row buffer at compile-time byte offsets: loads the 16-byte chunks covering [B0, B0 + LEN)
// and hands out the 32-bit little-endian word at any even byte offset inside.
template <int B0, int LEN> struct Span {
    static constexpr int C0 = B0 / 16, C1 = (B0 + LEN + 15) / 16;
    uint32_t w[4 * (C1 - C0) + 1];
    __device__ __forceinline__ void load(const uint8_t* row) {
#pragma unroll
        for (int c = C0; c < C1; ++c) {
            const uint4 t = *reinterpret_cast<const uint4*>(row + 16 * c);
            w[4 * (c - C0)] = t.x; w[4 * (c - C0) + 1] = t.y; w[4 * (c - C0) + 2] = t.z; w[4 * (c - C0) + 3] = t.w;
        }
        w[4 * (C1 - C0)] = 0;
    }
    template <int B> __device__ __forceinline__ uint32_t word() const {
        constexpr int rel = B - 16 * C0;
        if (rel % 4 == 0) return w[rel / 4];
        return __funnelshift_r(w[rel / 4], w[rel / 4 + 1], 16);
    }
};

// S = which 64 of the 256 weights, O = byte offset of the super-block inside the 240-byte row buffer.
// Layout ql[128] | qh[64] | sc[16] (i8) | d (f16) and element order as rlx-gguf/src/lib.rs:1070-1114.
template <int S, int O> struct Decode64Q6 {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        constexpr int h = S / 2;
        Span<O + 64 * h, 64> ql;
        Span<O + 128 + 32 * h, 32> qh;
        Span<O + 192 + 8 * h + 4 * (S % 2), 4> sc;
        Span<O + 208, 2> dd;
        ql.load(row); qh.load(row); sc.load(row); dd.load(row);
        const float d = f16_bits_to_f32(dd.template word<O + 208>() & 0xFFFFu);
        const uint32_t scw = sc.template word<O + 192 + 8 * h + 4 * (S % 2)>();   // scales 2 g4, 2 g4 + 1 of both groups
        const float s00 = d * (float)(int8_t)(scw & 0xFFu), s01 = d * (float)(int8_t)((scw >> 8) & 0xFFu);
        const float s10 = d * (float)(int8_t)((scw >> 16) & 0xFFu), s11 = d * (float)(int8_t)(scw >> 24);
#pragma unroll
        for (int gsel = 0; gsel < 2; ++gsel) {
            const int g4 = 2 * (S % 2) + gsel;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t qlw = gsel == 0 ? word_ql<0>(ql, i) : word_ql<1>(ql, i);
                const uint32_t qhw = word_qh(qh, i);
                const uint32_t lo = (qlw >> (4 * (g4 >> 1))) & 0x0F0F0F0Fu;
                const uint32_t hi = (g4 < 2 ? (qhw << (4 - 2 * g4)) : (qhw >> (2 * g4 - 4))) & 0x30303030u;
                const uint32_t mw = lo | hi;
                const uint64_t ds = f32x2_splat(gsel == 0 ? (i < 4 ? s00 : s01) : (i < 4 ? s10 : s11));
                const uint64_t off = f32x2_splat(-(8388608.0f + 32.0f));
                v[16 * gsel + 2 * i] = scaled_pair<0>(mw, off, ds);
                v[16 * gsel + 2 * i + 1] = scaled_pair<1>(mw, off, ds);
            }
        }
    }
    // word i (0..7) of the 32 ql bytes of group (g4 & 1) = GSEL (within this half) / of the 32 qh bytes
    template <int GSEL> __device__ static __forceinline__ uint32_t word_ql(const Span<O + 64 * (S / 2), 64>& ql, int i) {
        constexpr int base = O + 64 * (S / 2) + 32 * GSEL;
        switch (i) {
            case 0: return ql.template word<base>();      case 1: return ql.template word<base + 4>();
            case 2: return ql.template word<base + 8>();  case 3: return ql.template word<base + 12>();
            case 4: return ql.template word<base + 16>(); case 5: return ql.template word<base + 20>();
            case 6: return ql.template word<base + 24>(); default: return ql.template word<base + 28>();
        }
    }
    __device__ static __forceinline__ uint32_t word_qh(const Span<O + 128 + 32 * (S / 2), 32>& qh, int i) {
        constexpr int base = O + 128 + 32 * (S / 2);
        switch (i) {
            case 0: return qh.template word<base>();      case 1: return qh.template word<base + 4>();
            case 2: return qh.template word<base + 8>();  case 3: return qh.template word<base + 12>();
            case 4: return qh.template word<base + 16>(); case 5: return qh.template word<base + 20>();
            case 6: return qh.template word<base + 24>(); default: return qh.template word<base + 28>();
        }
    }
};

// Q2_K as the reference reads it (rlx-gguf/src/lib.rs:857-886): d, dmin (f16) | 16 scale bytes (low nibble scale,
// high nibble min) | 64 quant bytes.  Weights [64 S, 64 S + 64) are two 2-bit planes (shift 4 (S % 2), + 2) of the
// 32 quant bytes of half S / 2, sixteen weights per scale byte: w = (d * sc) * q - dmin * mn, product and
// difference rounded separately.  O = byte offset of the super-block in the row buffer (a multiple of 4).
template <int S, int O> struct Decode64Q2 {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        constexpr int h = S / 2;
        Span<O, 4> hd;
        Span<O + 4 + 8 * h + 4 * (S % 2), 4> sc;
        Span<O + 20 + 32 * h, 32> qs;
        hd.load(row); sc.load(row); qs.load(row);
        const uint32_t hw = hd.template word<O>();
        const float d = f16_bits_to_f32(hw & 0xFFFFu), dmin = f16_bits_to_f32(hw >> 16);
        const uint32_t scw = sc.template word<O + 4 + 8 * h + 4 * (S % 2)>();    // scale bytes of (plane, sixteen) = (0,0) (0,1) (1,0) (1,1)
        const uint64_t off = f32x2_splat(-8388608.0f);
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) {
            const int shift = 4 * (S % 2) + 2 * pl;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t sb = (scw >> (16 * pl + 8 * (i >> 2))) & 0xFFu;
                const uint64_t dl2 = f32x2_splat(d * (float)(sb & 0xFu)), ml2 = f32x2_splat(-(dmin * (float)(sb >> 4)));
                const uint32_t q = (word_at(qs, i) >> shift) & 0x03030303u;
                v[16 * pl + 2 * i] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<0>(q), off)), ml2));
                v[16 * pl + 2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(dl2, add_f32x2(magic_pair<1>(q), off)), ml2));
            }
        }
    }
    __device__ static __forceinline__ uint32_t word_at(const Span<O + 20 + 32 * (S / 2), 32>& qs, int i) {
        constexpr int base = O + 20 + 32 * (S / 2);
        switch (i) {
            case 0: return qs.template word<base>();      case 1: return qs.template word<base + 4>();
            case 2: return qs.template word<base + 8>();  case 3: return qs.template word<base + 12>();
            case 4: return qs.template word<base + 16>(); case 5: return qs.template word<base + 20>();
            case 6: return qs.template word<base + 24>(); default: return qs.template word<base + 28>();
        }
    }
};
template <int S>
__device__ __forceinline__ void decode64_q2(const uint8_t* row, uint32_t g, uint32_t (&v)[32]) {
    switch (g & 3u) {      // 84 g mod 16 = 4 (g mod 4)
        case 0: Decode64Q2<S, 0>::run(row, v); break;   case 1: Decode64Q2<S, 4>::run(row, v); break;
        case 2: Decode64Q2<S, 8>::run(row, v); break;   default: Decode64Q2<S, 12>::run(row, v); break;
    }
}

// The 32-bit word at even byte offset `rel` of a word array (offsets are constants once the loops are unrolled).
__device__ __forceinline__ uint32_t word_of(const uint32_t* w, int rel) {
    return (rel % 4 == 0) ? w[rel / 4] : __funnelshift_r(w[rel / 4], w[rel / 4 + 1], 16);
}
// four bits -> bit 0 of four bytes
__device__ __forceinline__ uint32_t spread4(uint32_t x) { return ((x & 0xFu) * 0x00204081u) & 0x01010101u; }

// Q4_1 / Q5_0 / Q5_1 (rlx-gguf/src/lib.rs:635-729): blocks of 32 weights, d (f16) [m (f16)] [qh (u32)] 16 nibble
// bytes; low nibbles are weights 0..15, high nibbles 16..31, bit j (j + 16) of qh the fifth bit of weight j (16 + j).
// Q4_1, Q5_1: d * q + m (product and sum rounded separately); Q5_0: d * (q - 16).
template <int S, int BB, bool HAS_M, bool HAS_H> struct Decode64Blk32 {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        constexpr int B0 = 2 * BB * S;
        Span<B0, 2 * BB> sp;
        sp.load(row);
        constexpr int R0 = B0 - 16 * Span<B0, 2 * BB>::C0;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const int base = R0 + BB * blk;
            const uint32_t hw = word_of(sp.w, base);
            const uint64_t d2 = f32x2_splat(f16_bits_to_f32(hw & 0xFFFFu));
            const uint64_t m2 = HAS_M ? f32x2_splat(f16_bits_to_f32(hw >> 16)) : 0ull;
            const int oh = HAS_M ? 4 : 2, oq = oh + (HAS_H ? 4 : 0);
            const uint32_t qh = HAS_H ? word_of(sp.w, base + oh) : 0u;
            const uint64_t off = f32x2_splat(HAS_M ? -8388608.0f : -(8388608.0f + 16.0f));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t q = word_of(sp.w, base + oq + 4 * i);
                uint32_t lo = q & 0x0F0F0F0Fu, hi = (q >> 4) & 0x0F0F0F0Fu;
                if (HAS_H) { lo |= spread4(qh >> (4 * i)) << 4; hi |= spread4(qh >> (16 + 4 * i)) << 4; }
                if (HAS_M) {
                    v[16 * blk + 2 * i] = bf16x2_of(add_f32x2(mul_f32x2(d2, add_f32x2(magic_pair<0>(lo), off)), m2));
                    v[16 * blk + 2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(d2, add_f32x2(magic_pair<1>(lo), off)), m2));
                    v[16 * blk + 8 + 2 * i] = bf16x2_of(add_f32x2(mul_f32x2(d2, add_f32x2(magic_pair<0>(hi), off)), m2));
                    v[16 * blk + 8 + 2 * i + 1] = bf16x2_of(add_f32x2(mul_f32x2(d2, add_f32x2(magic_pair<1>(hi), off)), m2));
                } else {
                    v[16 * blk + 2 * i] = scaled_pair<0>(lo, off, d2);
                    v[16 * blk + 2 * i + 1] = scaled_pair<1>(lo, off, d2);
                    v[16 * blk + 8 + 2 * i] = scaled_pair<0>(hi, off, d2);
                    v[16 * blk + 8 + 2 * i + 1] = scaled_pair<1>(hi, off, d2);
                }
            }
        }
    }
};
template <int S> struct Decode64<RLXQ_Q4_1, S> : Decode64Blk32<S, 20, true, false> {};
template <int S> struct Decode64<RLXQ_Q5_0, S> : Decode64Blk32<S, 22, false, true> {};
template <int S> struct Decode64<RLXQ_Q5_1, S> : Decode64Blk32<S, 24, true, true> {};

// Q8_K (rlx-gguf/src/lib.rs:848-854, 1121-1140): w = d * q with an f32 d.
template <int S, int O> struct Decode64Q8K {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        Span<O, 4> hd;
        Span<O + 4 + 64 * S, 64> qs;
        hd.load(row); qs.load(row);
        const uint64_t d2 = f32x2_splat(__uint_as_float(hd.template word<O>())), off = f32x2_splat(-(8388608.0f + 128.0f));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t u = qs.w[(O + 4 + 64 * S) / 4 - 4 * Span<O + 4 + 64 * S, 64>::C0 + i] ^ 0x80808080u;   // int8 -> q + 128
            v[2 * i] = scaled_pair<0>(u, off, d2);
            v[2 * i + 1] = scaled_pair<1>(u, off, d2);
        }
    }
};
template <int S>
__device__ __forceinline__ void decode64_q8k(const uint8_t* row, uint32_t g, uint32_t (&v)[32]) {
    switch (g & 3u) {      // 292 g mod 16 = 4 (g mod 4)
        case 0: Decode64Q8K<S, 0>::run(row, v); break;   case 1: Decode64Q8K<S, 4>::run(row, v); break;
        case 2: Decode64Q8K<S, 8>::run(row, v); break;   default: Decode64Q8K<S, 12>::run(row, v); break;
    }
}

// Q3_K as the reference reads it (rlx-gguf/src/lib.rs:889-930): d (f16) | 12 scale bytes (sixteen 6-bit scales) |
// 32 high-mask bytes | 64 quant bytes.  Weights [64 S, 64 S + 64): planes 2 (S % 2), + 1 of the 32 quant bytes of
// half S / 2; weight = (d * (scale - 32)) * (q - (mask bit ? 0 : 4)), mask bit 4 (S / 2) + plane of the weight's
// mask byte.  The four scales of the group are the bytes of word S of the unpacked scale words.
template <int S, int O> struct Decode64Q3 {
    __device__ static __forceinline__ void run(const uint8_t* row, uint32_t (&v)[32]) {
        constexpr int h = S / 2;
        Span<O, 14> hd;
        Span<O + 14, 32> hm;
        Span<O + 46 + 32 * h, 32> qs;
        hd.load(row); hm.load(row); qs.load(row);
        const float d = f16_bits_to_f32(hd.template word<O>() & 0xFFFFu);
        const uint32_t a0 = hd.template word<O + 2>(), a1 = hd.template word<O + 6>(), tmp = hd.template word<O + 10>();
        uint32_t scw;
        if (S == 0) scw = (a0 & 0x0F0F0F0Fu) | ((tmp & 0x03030303u) << 4);
        else if (S == 1) scw = (a1 & 0x0F0F0F0Fu) | (((tmp >> 2) & 0x03030303u) << 4);
        else if (S == 2) scw = ((a0 >> 4) & 0x0F0F0F0Fu) | (((tmp >> 4) & 0x03030303u) << 4);
        else scw = ((a1 >> 4) & 0x0F0F0F0Fu) | (((tmp >> 6) & 0x03030303u) << 4);
        const uint64_t off = f32x2_splat(-(8388608.0f + 4.0f));
#pragma unroll
        for (int pl = 0; pl < 2; ++pl) {
            const int plane = 2 * (S % 2) + pl;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int sb = (int)((scw >> (16 * pl + 8 * (i >> 2))) & 0xFFu) - 32;
                const uint64_t dl2 = f32x2_splat(d * (float)sb);
                const uint32_t q = (word_q(qs, i) >> (2 * plane)) & 0x03030303u;
                const uint32_t hb = (word_h(hm, i) >> (4 * h + plane)) & 0x01010101u;
                const uint32_t u = q | (hb << 2);                 // q + 4 where the mask bit is set: weight = u - 4
                v[16 * pl + 2 * i] = scaled_pair<0>(u, off, dl2);
                v[16 * pl + 2 * i + 1] = scaled_pair<1>(u, off, dl2);
            }
        }
    }
    __device__ static __forceinline__ uint32_t word_q(const Span<O + 46 + 32 * (S / 2), 32>& qs, int i) {
        constexpr int base = O + 46 + 32 * (S / 2);
        switch (i) {
            case 0: return qs.template word<base>();      case 1: return qs.template word<base + 4>();
            case 2: return qs.template word<base + 8>();  case 3: return qs.template word<base + 12>();
            case 4: return qs.template word<base + 16>(); case 5: return qs.template word<base + 20>();
            case 6: return qs.template word<base + 24>(); default: return qs.template word<base + 28>();
        }
    }
    __device__ static __forceinline__ uint32_t word_h(const Span<O + 14, 32>& hm, int i) {
        constexpr int base = O + 14;
        switch (i) {
            case 0: return hm.template word<base>();      case 1: return hm.template word<base + 4>();
            case 2: return hm.template word<base + 8>();  case 3: return hm.template word<base + 12>();
            case 4: return hm.template word<base + 16>(); case 5: return hm.template word<base + 20>();
            case 6: return hm.template word<base + 24>(); default: return hm.template word<base + 28>();
        }
    }
};
template <int S>
__device__ __forceinline__ void decode64_q3(const uint8_t* row, uint32_t g, uint32_t (&v)[32]) {
    switch (g & 7u) {      // 110 g mod 16 = (16 - 2 (g mod 8)) mod 16
        case 0: Decode64Q3<S, 0>::run(row, v); break;   case 1: Decode64Q3<S, 14>::run(row, v); break;
        case 2: Decode64Q3<S, 12>::run(row, v); break;  case 3: Decode64Q3<S, 10>::run(row, v); break;
        case 4: Decode64Q3<S, 8>::run(row, v); break;   case 5: Decode64Q3<S, 6>::run(row, v); break;
        case 6: Decode64Q3<S, 4>::run(row, v); break;   default: Decode64Q3<S, 2>::run(row, v); break;
    }
}

// Dispatch on the (warp-uniform) offset of group g inside its row buffer.
template <int S>
__device__ __forceinline__ void decode64_q6(const uint8_t* row, uint32_t g, uint32_t (&v)[32]) {
    switch (g & 7u) {
        case 0: Decode64Q6<S, 0>::run(row, v); break;   case 1: Decode64Q6<S, 2>::run(row, v); break;
        case 2: Decode64Q6<S, 4>::run(row, v); break;   case 3: Decode64Q6<S, 6>::run(row, v); break;
        case 4: Decode64Q6<S, 8>::run(row, v); break;   case 5: Decode64Q6<S, 10>::run(row, v); break;
        case 6: Decode64Q6<S, 12>::run(row, v); break;  default: Decode64Q6<S, 14>::run(row, v); break;
    }
}

template <uint32_t SCHEME, int S>
__device__ __forceinline__ void decode64(const uint8_t* row, uint32_t g, uint32_t (&v)[32]) {
    if constexpr (SCHEME == RLXQ_Q6_K) decode64_q6<S>(row, g, v);
    else if constexpr (SCHEME == RLXQ_Q2_K) decode64_q2<S>(row, g, v);
    else if constexpr (SCHEME == RLXQ_Q8_K) decode64_q8k<S>(row, g, v);
    else if constexpr (SCHEME == RLXQ_Q3_K) decode64_q3<S>(row, g, v);
    else Decode64<SCHEME, S>::run(row, v);
}

// ---- kernel -----------------------------------------------------------------------------------
constexpr uint32_t kGemmMaxDecodeGroups = 3;
constexpr uint32_t kGemmMaxBlock = (4 + 4 * kGemmMaxDecodeGroups + 4) * 32;   // B TMA, MMA, raw TMA, spare | decode | epilogue
// warp roles: 0 = activation (B) TMA producer, 1 = MMA issuer and tensor-memory owner,
// 2 = raw weight TMA producer, 3 = idle, then GROUPS x 4 decode warps (tensor-memory lane quarter =
// warp % 4; group (warp - 4) / 4 takes the 64-wide k blocks whose running index is its number modulo
// GROUPS), then 4 epilogue warps (lane quarter = warp % 4).

struct GemmParams {
    CUtensorMap xmap;      // x[m, k] bf16, box 256 rows x 64 columns, 128-byte swizzle
    CUtensorMap wmap;      // W[n, row_bytes / 8] eight-byte elements, box 128 rows x one 256-weight group
    void* y;
    int* err;
    uint32_t m, n, k, y_bf16, y_vec;      // y_vec: y rows can be written in aligned 16-byte pieces
    uint32_t wtiles, xtiles;
    // Work split.  streamk == 0: CTA c takes whole tiles c, c + grid, ...  streamk == 1: the units
    // (tile, 256-weight k group), tile-major, are dealt as contiguous ranges of units_q units (the first
    // units_r CTAs one more), so every SM gets the same work however many tiles there are; a tile cut
    // by range boundaries is completed by the last of its contributors to arrive (partial tiles in
    // `partial`, one slot per CTA and end of its range; arrival counters in `counters`, zeroed by the host).
    uint32_t streamk, kgroups, units_q, units_r;
    float* partial;
    uint32_t* counters;
    // Grouped mode (MoE expert stacks; null = one dense matrix): W is a stack of [n, k] slabs and activation
    // tile xt is described by groups[xt] = {first row in x, rows (0 = no such tile), expert, -}: the tile
    // multiplies those rows by slab `expert`.  The table is written on the device by the kernel in front, and
    // xtiles is only an upper bound of the tiles in use.  Never combined with the k split.
    const uint4* groups;
};

// Where tile `tile` reads and writes: activation rows [xrow0, xlim), weight rows from wrow0 (in the stack).
struct GemmTileRows { uint32_t xrow0, xlim, wrow0; };
template <uint32_t TX>
__device__ __forceinline__ bool gemm_tile_rows(const GemmParams& P, uint32_t tile, GemmTileRows& t) {
    const uint32_t wt = tile / P.xtiles, xt = tile % P.xtiles;
    if (P.groups) {
        const uint4 g = __ldg(&P.groups[xt]);
        t.xrow0 = g.x; t.xlim = g.x + g.y; t.wrow0 = g.z * P.n + wt * kGemmTileW;
        return g.y != 0u;
    }
    t.xrow0 = xt * TX; t.xlim = P.m; t.wrow0 = wt * kGemmTileW;
    return true;
}


struct GemmSeg { uint32_t tile, g0, g1; };     // k groups [g0, g1) of one tile

__device__ __forceinline__ uint32_t gemm_range_start(const GemmParams& P, uint32_t c) {
    return c * P.units_q + min(c, P.units_r);
}
// The CTA whose range holds unit u.
__device__ __forceinline__ uint32_t gemm_owner(const GemmParams& P, uint32_t u) {
    const uint32_t big = P.units_r * (P.units_q + 1);
    return u < big ? u / (P.units_q + 1) : P.units_r + (u - big) / P.units_q;
}
// Iteration over this CTA's segments, in the order every warp role walks them.
__device__ __forceinline__ void gemm_seg_init(const GemmParams& P, uint32_t& cur, uint32_t& lim) {
    if (P.streamk) { cur = gemm_range_start(P, blockIdx.x); lim = gemm_range_start(P, blockIdx.x + 1); }
    else { cur = blockIdx.x; lim = P.wtiles * P.xtiles; }
}
__device__ __forceinline__ bool gemm_seg_next(const GemmParams& P, uint32_t& cur, uint32_t lim, GemmSeg& sg) {
    if (cur >= lim) return false;
    if (P.streamk) {
        sg.tile = cur / P.kgroups;
        sg.g0 = cur - sg.tile * P.kgroups;
        sg.g1 = min(P.kgroups, sg.g0 + (lim - cur));
        cur += sg.g1 - sg.g0;
    } else {
        sg.tile = cur; sg.g0 = 0; sg.g1 = P.kgroups;
        cur += gridDim.x;
    }
    return true;
}

// Where an epilogue pass writes: y (bf16 or f32, row pitch n) or a partial tile (f32, row pitch 128).
struct GemmDst {
    uint8_t* base;
    size_t ld;                        // elements per activation row
    uint32_t m0, mlim, n0, nlim;      // first row / column of the tile in the destination, and its extents
};
constexpr uint32_t kGemmEpiStage = 2 * 8192;   // two 8 KB transposition buffers

// Thirty-two accumulator columns (activation rows 32 c ..) of the 128 weight rows -> destination.  A thread
// owns one weight row, so its values lie one destination row apart; written directly, a warp's store is
// 64 or 128 bytes and each thread issues one store per value.  Here the columns are transposed through
// shared memory 8 KB at a time and leave as 16-byte pieces, a warp covering whole 256- or 512-byte row
// segments.  One named barrier per pass: the two buffers alternate, and a thread can only write a
// buffer again after the barrier of the pass in between, which everybody reaches after reading it.
template <bool F32>
__device__ __forceinline__ void gemm_store_vec(uint8_t* stage, uint32_t epi_tid, uint32_t row, const uint32_t (&v)[32],
                                               const GemmDst& d, uint32_t c) {
    constexpr uint32_t ES = F32 ? 4u : 2u, CP = 8192u / (kGemmTileW * ES), PR = kGemmTileW * ES / 16u, NPASS = 32u / CP;
#pragma unroll
    for (uint32_t h = 0; h < NPASS; ++h) {
        uint8_t* buf = stage + ((NPASS == 1u ? c : h) & 1u) * 8192u;
        if (F32) {
#pragma unroll
            for (uint32_t j = 0; j < CP; ++j) *reinterpret_cast<uint32_t*>(buf + (j * kGemmTileW + row) * 4u) = v[h * CP + j];
        } else {
            // one conversion instruction per two values (round to nearest even; a NaN becomes the canonical
            // quiet NaN), the halves stored to the two output rows they belong to
#pragma unroll
            for (uint32_t j = 0; j < CP; j += 2) {
                const uint32_t pr = bf16x2_of(f32x2(v[h * CP + j], v[h * CP + j + 1]));
                *reinterpret_cast<uint16_t*>(buf + (j * kGemmTileW + row) * 2u) = (uint16_t)pr;
                *reinterpret_cast<uint16_t*>(buf + ((j + 1) * kGemmTileW + row) * 2u) = (uint16_t)(pr >> 16);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            const uint32_t p = epi_tid + 128u * q, j = p / PR, pc = p % PR;
            const uint32_t mi = d.m0 + 32u * c + h * CP + j, ni = d.n0 + pc * (16u / ES);
            if (mi < d.mlim && ni < d.nlim) {
                const uint4 t = *reinterpret_cast<const uint4*>(buf + j * (kGemmTileW * ES) + pc * 16u);
                *reinterpret_cast<uint4*>(d.base + ((size_t)mi * d.ld + ni) * ES) = t;
            }
        }
    }
}

// Four values of activation row mi, weight rows ni .. ni + 3, into y.
__device__ __forceinline__ void gemm_store4(const GemmParams& P, uint32_t mi, uint32_t ni, float4 a) {
    if (mi >= P.m || ni >= P.n) return;
    const size_t o = (size_t)mi * P.n + ni;
    if (P.y_vec) {                       // n is a multiple of 4 at least and the rows are aligned
        if (P.y_bf16) {
            uint2 t;
            t.x = bf16x2_of(f32x2(__float_as_uint(a.x), __float_as_uint(a.y)));
            t.y = bf16x2_of(f32x2(__float_as_uint(a.z), __float_as_uint(a.w)));
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(P.y) + o) = t;
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(P.y) + o) = a;
        }
        return;
    }
    const float e[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        if (ni + i < P.n) {
            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o + i] = (uint16_t)bf16x2_of(f32x2(__float_as_uint(e[i]), 0u));
            else reinterpret_cast<float*>(P.y)[o + i] = e[i];
        }
    }
}

// Thirty-two accumulator columns plus the same columns of another contributor's published part -> y.  The
// other part's 16-byte pieces follow the piece order of the transposition buffers: piece p of a 16-column
// pass is floats [4 p, 4 p + 4) of that pass, in the buffer and in the part alike.
__device__ __forceinline__ void gemm_add_store(uint8_t* stage, uint32_t epi_tid, uint32_t row, const uint32_t (&v)[32],
                                               const uint4* other, const GemmParams& P, uint32_t m0, uint32_t n0) {
#pragma unroll
    for (uint32_t h = 0; h < 2; ++h) {
        uint8_t* buf = stage + h * 8192u;
#pragma unroll
        for (uint32_t j = 0; j < 16; ++j) *reinterpret_cast<uint32_t*>(buf + (j * kGemmTileW + row) * 4u) = v[16 * h + j];
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            const uint32_t p = epi_tid + 128u * q;
            const float4 own = *reinterpret_cast<const float4*>(buf + p * 16u);
            const uint4 ot = __ldcg(other + 512u * h + p);
            float4 r;
            r.x = own.x + __uint_as_float(ot.x); r.y = own.y + __uint_as_float(ot.y);
            r.z = own.z + __uint_as_float(ot.z); r.w = own.w + __uint_as_float(ot.w);
            gemm_store4(P, m0 + 16 * h + (p >> 5), n0 + 4 * (p & 31u), r);
        }
    }
}

// The last contributor of a cut tile adds all parts in contributor order (its own included, re-read from
// memory: the sum then never depends on who came last).  Sixteen activation rows (8 KB of every part) at a
// time, in 16-byte pieces: a warp reads 512 contiguous bytes of each part.  Kept out of line: it runs once
// per cut tile and would otherwise raise the register need of the whole kernel.
__device__ __noinline__ void gemm_reduce_parts(const GemmParams& P, uint32_t tile_x, uint32_t c_first, uint32_t c_last,
                                               uint32_t u0, uint32_t m0, uint32_t n0, uint32_t epi_tid) {
    for (uint32_t col0 = 0; col0 < tile_x && m0 + col0 < P.m; col0 += 16) {
        float4 acc[4];
        for (uint32_t cc = c_first; cc <= c_last; ++cc) {
            const uint32_t sid = 2 * cc + (gemm_range_start(P, cc) > u0 ? 0u : 1u);
            const uint4* src = reinterpret_cast<const uint4*>(P.partial + (size_t)sid * (kGemmTileW * tile_x) + (size_t)col0 * kGemmTileW) + epi_tid;
            uint4 pv[4];
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) pv[q] = __ldcg(src + 128u * q);
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                const float4 f = make_float4(__uint_as_float(pv[q].x), __uint_as_float(pv[q].y), __uint_as_float(pv[q].z), __uint_as_float(pv[q].w));
                if (cc == c_first) acc[q] = f;
                else { acc[q].x += f.x; acc[q].y += f.y; acc[q].z += f.z; acc[q].w += f.w; }
            }
        }
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            const uint32_t p = epi_tid + 128u * q;
            gemm_store4(P, m0 + col0 + (p >> 5), n0 + 4 * (p & 31u), acc[q]);
        }
    }
}

struct GemmBars {
    uint64_t b_full[kGemmMaxStages], a_full[kGemmMaxStages], stage_free[kGemmMaxStages];
    uint64_t raw_full[kGemmRawStages], raw_empty[kGemmRawStages];
    uint64_t d_full, d_free;
    uint32_t tmem_base, abort_flag, epi_prev, epi_prev1;   // epi_prev, epi_prev1: arrival counts of alternate segments
};

template <uint32_t SCHEME, uint32_t kGemmTileX>
__global__ void __launch_bounds__(kGemmMaxBlock, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams P) {
    constexpr uint32_t RAW_ROW = GemmRaw<SCHEME>::ROW;
    constexpr uint32_t kGemmStages = GemmRaw<SCHEME>::STAGES;   // shared memory left after the raw boxes decides
    constexpr uint32_t kGemmDecodeGroups = GemmRaw<SCHEME>::GROUPS;
    constexpr uint32_t RAW_BYTES = kGemmTileW * RAW_ROW;
    constexpr uint32_t B_BYTES = kGemmTileX * kGemmBK * 2;           // 32 KB
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* b_stage = smem;                                          // kGemmStages x 32 KB, 1024-aligned
    uint8_t* raw_stage = smem + kGemmStages * B_BYTES;                // kGemmRawStages x RAW_BYTES (128-aligned)
    GemmBars* bars = reinterpret_cast<GemmBars*>(raw_stage + kGemmRawStages * ((RAW_BYTES + 127) / 128 * 128));
    constexpr uint32_t RAW_STRIDE = (RAW_BYTES + 127) / 128 * 128;
    uint8_t* epi_stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bars + 1) + 15) & ~(uintptr_t)15);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    volatile uint32_t* abort_flag = &bars->abort_flag;

    if (tid == 0) {
        for (uint32_t s = 0; s < kGemmStages; ++s) {
            mbar_init(smem_u32(&bars->b_full[s]), 1);
            mbar_init(smem_u32(&bars->a_full[s]), 4);
            mbar_init(smem_u32(&bars->stage_free[s]), 1);
        }
        for (uint32_t r = 0; r < kGemmRawStages; ++r) {
            mbar_init(smem_u32(&bars->raw_full[r]), 1);
            mbar_init(smem_u32(&bars->raw_empty[r]), 4 * kGemmDecodeGroups);
        }
        mbar_init(smem_u32(&bars->d_full), 1);
        mbar_init(smem_u32(&bars->d_free), 4);
        bars->abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {               // the whole warp allocates all 512 columns: 256 accumulator + up to 8 x 32 weight stages
        tmem_alloc(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t tmem_d = tmem_base, tmem_a = tmem_base + 256;
    auto give_up = [&](int code) {
        if (lane == 0) { atomicExch(P.err, code); *abort_flag = 1u; }
    };

    if (warp == 0) {
        // ---------------- activation tiles (B operand) ----------------
        if (lane == 0) {
            tma_prefetch_desc(&P.xmap);
            uint32_t s = 0, ph = 1;      // parity to wait for on stage_free (1 passes on a fresh barrier)
            uint32_t cur, lim;
            gemm_seg_init(P, cur, lim);
            GemmSeg sg;
            while (!*abort_flag && gemm_seg_next(P, cur, lim, sg)) {
                GemmTileRows tr;
                if (!gemm_tile_rows<kGemmTileX>(P, sg.tile, tr)) continue;
                bool ok = true;
                for (uint32_t kb = 4 * sg.g0; kb < 4 * sg.g1; ++kb) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->stage_free[s]), ph)) { give_up(11); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->b_full[s]);
                    mbar_arrive_expect_tx(full, B_BYTES);
                    tma_load_2d(smem_u32(b_stage + s * B_BYTES), &P.xmap, (int32_t)(kb * kGemmBK), (int32_t)tr.xrow0, full);
                    if (++s == kGemmStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 2) {
        // ---------------- raw weight groups ----------------
        if (lane == 0) {
            tma_prefetch_desc(&P.wmap);
            uint32_t r = 0, ph = 1;
            uint32_t cur, lim;
            gemm_seg_init(P, cur, lim);
            GemmSeg sg;
            while (!*abort_flag && gemm_seg_next(P, cur, lim, sg)) {
                GemmTileRows tr;
                if (!gemm_tile_rows<kGemmTileX>(P, sg.tile, tr)) continue;
                bool ok = true;
                for (uint32_t g = sg.g0; g < sg.g1; ++g) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_empty[r]), ph)) { give_up(12); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->raw_full[r]);
                    mbar_arrive_expect_tx(full, RAW_BYTES);
                    tma_load_2d(smem_u32(raw_stage + r * RAW_STRIDE), &P.wmap, (int32_t)gemm_raw_x<SCHEME>(g), (int32_t)tr.wrow0, full);
                    if (++r == kGemmRawStages) { r = 0; ph ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, dph = 1;   // dph: parity to wait for on d_free (1 passes the first time)
            uint32_t cur, lim;
            gemm_seg_init(P, cur, lim);
            GemmSeg sg;
            while (!*abort_flag && gemm_seg_next(P, cur, lim, sg)) {
                { GemmTileRows tr; if (!gemm_tile_rows<kGemmTileX>(P, sg.tile, tr)) continue; }
                if (!mbar_wait(smem_u32(&bars->d_free), dph)) { give_up(13); break; }
                dph ^= 1u;
                tc_fence_after();
                bool ok = true;
                for (uint32_t kb = 0; kb < 4 * (sg.g1 - sg.g0); ++kb) {    // the first MMA of a segment overwrites the accumulator
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->b_full[s]), ph) ||
                        !mbar_wait(smem_u32(&bars->a_full[s]), ph)) { give_up(14); ok = false; break; }
                    tc_fence_after();
                    const uint64_t bdesc = kmajor_sw128_desc(smem_u32(b_stage + s * B_BYTES));
#pragma unroll
                    for (uint32_t j = 0; j < kGemmBK / 16; ++j)
                        tc_mma_ts(tmem_d, tmem_a + 32 * s + 8 * j, bdesc + 2 * j, GemmIdesc<kGemmTileX>::value, (kb | j) ? 1u : 0u);
                    tc_commit(smem_u32(&bars->stage_free[s]));     // frees the B stage and the A columns when the MMAs retire
                    if (++s == kGemmStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                tc_commit(smem_u32(&bars->d_full));
            }
        }
    } else if (warp >= 4 && warp < 4 + 4 * kGemmDecodeGroups) {
        // ---------------- decode: raw blocks -> bf16 rows in tensor memory ----------------
        // Group grp takes the k blocks whose running index is grp modulo the number of groups, so the
        // groups alternate whatever the number of 64-wide blocks per raw group (4) is.
        const uint32_t quarter = warp & 3u, grp = (warp - 4) >> 2;
        const uint32_t row = quarter * 32 + lane;                       // weight row of the tile == tensor-memory lane
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t r = 0, rph = 0, kbg0 = 0;   // kbg0: k blocks this CTA has gone through before the current group
        bool ok = true;
        uint32_t cur, lim;
        gemm_seg_init(P, cur, lim);
        GemmSeg sg;
        while (ok && !*abort_flag && gemm_seg_next(P, cur, lim, sg)) {
            { GemmTileRows tr; if (!gemm_tile_rows<kGemmTileX>(P, sg.tile, tr)) continue; }
            for (uint32_t g = sg.g0; g < sg.g1 && ok; ++g, kbg0 += 4) {
                if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_full[r]), rph)) { give_up(15); ok = false; break; }
                const uint8_t* rp = raw_stage + r * RAW_STRIDE + row * RAW_ROW;
#pragma unroll
                for (uint32_t sub = 0; sub < 4; ++sub) {                 // which 64 weights of the group
                    const uint32_t kbg = kbg0 + sub;                     // running k-block index -> owner, ring slot, phase
                    if (kbg % kGemmDecodeGroups != grp) continue;
                    const uint32_t s = kbg % kGemmStages, fph = ((kbg / kGemmStages) & 1u) ^ 1u;
                    // decode into registers first: only the store needs the stage's tensor-memory columns,
                    // so the arithmetic stays off the free -> store -> MMA chain
                    uint32_t v[32];
                    if (sub == 0) decode64<SCHEME, 0>(rp, g, v);
                    else if (sub == 1) decode64<SCHEME, 1>(rp, g, v);
                    else if (sub == 2) decode64<SCHEME, 2>(rp, g, v);
                    else decode64<SCHEME, 3>(rp, g, v);
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->stage_free[s]), fph)) { give_up(16); ok = false; break; }
                    tc_fence_after();
                    tmem_st32(tmem_a + lane_addr + 32 * s, v);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->a_full[s]));
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->raw_empty[r]));
                if (++r == kGemmRawStages) { r = 0; rph ^= 1u; }
            }
        }
    } else if (warp >= 4 + 4 * kGemmDecodeGroups) {
        // ---------------- epilogue: accumulator -> y (or -> a partial tile, completed by the last contributor) ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t lane_addr = (quarter * 32) << 16;
        const uint32_t row = quarter * 32 + lane;
        const uint32_t epi_tid = (warp - (4 + 4 * kGemmDecodeGroups)) * 32 + lane;
        uint32_t dph = 0, nseg = 0;
        uint32_t cur, lim;
        gemm_seg_init(P, cur, lim);
        GemmSeg sg;
        while (!*abort_flag && gemm_seg_next(P, cur, lim, sg)) {
            const uint32_t wt = sg.tile / P.xtiles, xt = sg.tile % P.xtiles;
            GemmTileRows tr;
            if (!gemm_tile_rows<kGemmTileX>(P, sg.tile, tr)) continue;
            if (!mbar_wait(smem_u32(&bars->d_full), dph)) { give_up(17); break; }
            dph ^= 1u;
            tc_fence_after();
            const uint32_t n_idx = wt * kGemmTileW + row;
            const bool whole = sg.g0 == 0 && sg.g1 == P.kgroups;
            // a cut tile: this CTA's part goes to its head slot when its range begins inside the tile
            // (only a first segment can), to its tail slot otherwise; layout [activation row][weight row]
            const uint32_t u0 = sg.tile * P.kgroups;
            uint32_t c_first = 0, c_last = 0;
            float* slot = nullptr;
            const float* other = nullptr;     // two contributors and the other one has already published
            if (!whole) {
                slot = P.partial + (size_t)(2 * blockIdx.x + ((nseg == 0 && sg.g0 != 0) ? 0u : 1u)) * (kGemmTileW * kGemmTileX);
                c_first = gemm_owner(P, u0);
                c_last = gemm_owner(P, u0 + P.kgroups - 1);
                if (c_last - c_first == 1u) {
                    // a + b == b + a: with two parts the sum does not depend on who adds, so the second one
                    // to arrive adds the published part to its own registers and never publishes
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (epi_tid == 0) (&bars->epi_prev)[nseg & 1u] = *reinterpret_cast<volatile uint32_t*>(&P.counters[sg.tile]);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (reinterpret_cast<volatile uint32_t*>(&bars->epi_prev)[nseg & 1u] == 1u) {
                        __threadfence();
                        const uint32_t oc = blockIdx.x == c_first ? c_last : c_first;
                        const uint32_t sid = 2 * oc + (gemm_range_start(P, oc) > u0 ? 0u : 1u);
                        other = P.partial + (size_t)sid * (kGemmTileW * kGemmTileX);
                    }
                }
            }
#pragma unroll 1
            for (uint32_t c = 0; c < kGemmTileX / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_d + lane_addr + 32 * c, v);
                tmem_ld_wait();
                if (c == kGemmTileX / 32 - 1) {      // everything is in registers: the accumulator may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->d_free));
                }
                if (other) {
                    gemm_add_store(epi_stage, epi_tid, row, v, reinterpret_cast<const uint4*>(other + (size_t)(32 * c) * kGemmTileW),
                                   P, xt * kGemmTileX + 32 * c, wt * kGemmTileW);
                } else if (!whole) {
                    const GemmDst d{reinterpret_cast<uint8_t*>(slot), kGemmTileW, 0u, kGemmTileX, 0u, kGemmTileW};
                    gemm_store_vec<true>(epi_stage, epi_tid, row, v, d, c);
                } else if (P.y_vec) {
                    const GemmDst d{reinterpret_cast<uint8_t*>(P.y), P.n, tr.xrow0, tr.xlim, wt * kGemmTileW, P.n};
                    if (P.y_bf16) gemm_store_vec<false>(epi_stage, epi_tid, row, v, d, c);
                    else gemm_store_vec<true>(epi_stage, epi_tid, row, v, d, c);
                } else if (n_idx < P.n) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        const uint32_t m_idx = tr.xrow0 + 32 * c + j;
                        if (m_idx < tr.xlim) {
                            const size_t o = (size_t)m_idx * P.n + n_idx;
                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)bf16x2_of(f32x2(v[j], 0u));
                            else reinterpret_cast<float*>(P.y)[o] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            if (!whole && !other) {
                // publish, count, and let the last contributor add all parts in contributor order (its own
                // included, re-read from memory: the sum then never depends on who came last)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (epi_tid == 0) (&bars->epi_prev)[nseg & 1u] = atomicAdd(&P.counters[sg.tile], 1u);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const uint32_t prev = reinterpret_cast<volatile uint32_t*>(&bars->epi_prev)[nseg & 1u];
                if (prev == c_last - c_first) {
                    __threadfence();
                    gemm_reduce_parts(P, kGemmTileX, c_first, c_last, u0, xt * kGemmTileX, wt * kGemmTileW, epi_tid);
                }
            }
            ++nseg;
        }
    }
    // everybody meets here, also after a timeout, so the tensor memory is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- the same GEMM, two CTAs per MMA (cta_group::2) --------------------------------------------
// A pair of CTAs (a cluster of two, on neighbouring SMs) works on 256 weight rows x 256 activation rows: each CTA
// decodes its own 128 weight rows into its own tensor memory and owns their accumulators, exactly as above, but
// loads only HALF of the activation tile (128 rows) into its shared memory; one tcgen05.mma.cta_group::2, issued by
// the first CTA of the pair, reads both halves.  A CTA therefore takes 16 KB of activations per k block from L2
// instead of 32 KB, so a stage of the same size holds a k block of 128 instead of 64: eight MMAs per round of
// barrier hand-overs instead of four.  That is what the pair buys here: the hand-overs of one round (stage freed ->
// refill and decode -> full -> issue -> commit) cost about 0.42 us whatever the ring depth and whatever else runs
// (measured with everything but the barriers switched off), against 0.35 us of tensor time for four MMAs.
//   barriers: the first CTA's b_full[s] collects its own TMA and the other CTA's (forwarded by a warp that waits
//   on that CTA's own barrier), its a_full[s] the decode warps of both CTAs, its d_free the epilogue warps of
//   both; one tcgen05.commit with a CTA mask signals stage_free[s] / d_full in both CTAs.
// Whole tiles only, n a multiple of 256, no expert groups; everything else runs the single-CTA kernel.
constexpr uint32_t kPairRound = 2;                        // 64-wide k blocks per stage (per round of hand-overs); 4 with two stages measured the same
constexpr uint32_t kPairStages = 8 / kPairRound;          // 8 x 32 tensor-memory columns of A, 8 x 16 KB of B, whatever the round
constexpr uint32_t kPairHalf = 128;                       // activation rows a CTA loads
constexpr uint32_t kPairSubBytes = kPairHalf * kGemmBK * 2;   // one 64-wide swizzled box: 16 KB
constexpr uint32_t kPairBBytes = kPairRound * kPairSubBytes;  // a stage: kPairRound boxes
constexpr uint32_t kPairIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);

struct PairBars {
    uint64_t b_full[kPairStages], b_own[kPairStages], a_full[kPairStages], stage_free[kPairStages];
    uint64_t raw_full[kGemmRawStages], raw_empty[kGemmRawStages];
    uint64_t d_full, d_free;
    uint32_t tmem_base, abort_flag;
};

// How a decode warp waits.  Where the decoders keep pace with the MMA they spend their time waiting, and one polling
// lane per warp keeps the barrier word free (every lane polling serialises on it).  Q6_K's decoders are the pacing
// part (Q3_K's too) and hardly ever find a barrier closed: there the single instruction of an all-lane poll is the
// cheaper form.
template <uint32_t SCHEME>
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, uint32_t lane) {
    if constexpr (SCHEME == RLXQ_Q6_K || SCHEME == RLXQ_Q3_K) return mbar_wait(bar, parity);
    else return mbar_wait_warp(bar, parity, lane);
}

template <uint32_t SCHEME>
__global__ void __launch_bounds__(kGemmMaxBlock, 1) gemm_pair_kernel(const __grid_constant__ GemmParams P) {
    constexpr uint32_t RAW_ROW = GemmRaw<SCHEME>::ROW;
    constexpr uint32_t kGemmDecodeGroups = GemmRaw<SCHEME>::GROUPS;
    constexpr uint32_t RAW_BYTES = kGemmTileW * RAW_ROW;
    constexpr uint32_t RAW_STRIDE = (RAW_BYTES + 127) / 128 * 128;
    constexpr uint32_t TX = 256;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* b_stage = smem;                                          // kPairStages x 32 KB, 1024-aligned
    uint8_t* raw_stage = smem + kPairStages * kPairBBytes;
    PairBars* bars = reinterpret_cast<PairBars*>(raw_stage + kGemmRawStages * RAW_STRIDE);
    uint8_t* epi_stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bars + 1) + 15) & ~(uintptr_t)15);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rank = cluster_cta_rank();            // 0 issues the MMAs
    volatile uint32_t* abort_flag = &bars->abort_flag;

    if (tid == 0) {
        for (uint32_t s = 0; s < kPairStages; ++s) {
            mbar_init(smem_u32(&bars->b_full[s]), 2);        // own TMA (with its bytes) + the other CTA's, forwarded
            mbar_init(smem_u32(&bars->b_own[s]), 1);
            mbar_init(smem_u32(&bars->a_full[s]), 8 * kPairRound);   // per 64-wide block four decode warps, of each CTA
            mbar_init(smem_u32(&bars->stage_free[s]), 1);
        }
        for (uint32_t r = 0; r < kGemmRawStages; ++r) {
            mbar_init(smem_u32(&bars->raw_full[r]), 1);
            mbar_init(smem_u32(&bars->raw_empty[r]), 4 * kGemmDecodeGroups);
        }
        mbar_init(smem_u32(&bars->d_full), 1);
        mbar_init(smem_u32(&bars->d_free), 8);               // four epilogue warps of each CTA
        bars->abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {               // the same warp of both CTAs: all 512 columns in each
        tmem_alloc_pair(smem_u32(&bars->tmem_base), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // the other CTA's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const uint32_t tmem_d = tmem_base, tmem_a = tmem_base + 256;
    auto give_up = [&](int code) {
        if (lane == 0) { atomicExch(P.err, code); *abort_flag = 1u; }
    };
    // the pair's tiles: 256 weight rows (pair index wp) x 256 activation rows (xt), xt fastest
    const uint32_t pt0 = blockIdx.x >> 1, pstep = gridDim.x >> 1, plim = (P.wtiles >> 1) * P.xtiles;
    const uint32_t rounds = 4 * P.kgroups / kPairRound;  // rounds of a tile

    if (warp == 0) {
        // ---------------- this CTA's half of the activation tile ----------------
        if (lane == 0) {
            tma_prefetch_desc(&P.xmap);
            uint32_t s = 0, ph = 1;
            bool ok = true;
            for (uint32_t pt = pt0; ok && pt < plim && !*abort_flag; pt += pstep) {
                const uint32_t xrow = (pt % P.xtiles) * TX + rank * kPairHalf;
                for (uint32_t kb = 0; kb < rounds; ++kb) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->stage_free[s]), ph)) { give_up(21); ok = false; break; }
                    const uint32_t full = smem_u32(rank == 0 ? &bars->b_full[s] : &bars->b_own[s]);
                    mbar_arrive_expect_tx(full, kPairBBytes);
#pragma unroll
                    for (uint32_t q = 0; q < kPairRound; ++q)
                        tma_load_2d(smem_u32(b_stage + s * kPairBBytes + q * kPairSubBytes), &P.xmap,
                                    (int32_t)((kb * kPairRound + q) * kGemmBK), (int32_t)xrow, full);
                    if (++s == kPairStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 3) {
        // ---------------- second CTA: tell the first that this half has landed ----------------
        if (lane == 0 && rank == 1) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t pt = pt0; ok && pt < plim && !*abort_flag; pt += pstep) {
                for (uint32_t kb = 0; kb < rounds; ++kb) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->b_own[s]), ph)) { give_up(22); ok = false; break; }
                    mbar_arrive_cluster(cluster_map(smem_u32(&bars->b_full[s]), 0));
                    if (++s == kPairStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 2) {
        // ---------------- raw weight groups of this CTA's 128 rows ----------------
        if (lane == 0) {
            tma_prefetch_desc(&P.wmap);
            uint32_t r = 0, ph = 1;
            bool ok = true;
            for (uint32_t pt = pt0; ok && pt < plim && !*abort_flag; pt += pstep) {
                const uint32_t wrow0 = (2 * (pt / P.xtiles) + rank) * kGemmTileW;
                for (uint32_t g = 0; g < P.kgroups; ++g) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_empty[r]), ph)) { give_up(23); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->raw_full[r]);
                    mbar_arrive_expect_tx(full, RAW_BYTES);
                    tma_load_2d(smem_u32(raw_stage + r * RAW_STRIDE), &P.wmap, (int32_t)gemm_raw_x<SCHEME>(g), (int32_t)wrow0, full);
                    if (++r == kGemmRawStages) { r = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the first CTA, for both ----------------
        if (lane == 0 && rank == 0) {
            uint32_t s = 0, ph = 0, dph = 1;
            bool ok = true;
            for (uint32_t pt = pt0; ok && pt < plim && !*abort_flag; pt += pstep) {
                if (!mbar_wait(smem_u32(&bars->d_free), dph)) { give_up(24); break; }
                dph ^= 1u;
                tc_fence_after();
                for (uint32_t kb = 0; kb < rounds; ++kb) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->b_full[s]), ph) ||
                        !mbar_wait(smem_u32(&bars->a_full[s]), ph)) { give_up(25); ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t j = 0; j < kPairRound * kGemmBK / 16; ++j) {
                        const uint64_t bdesc = kmajor_sw128_desc(smem_u32(b_stage + s * kPairBBytes + (j >> 2) * kPairSubBytes));
                        tc_mma_ts_pair(tmem_d, tmem_a + 32 * kPairRound * s + 8 * j, bdesc + 2 * (j & 3u), kPairIdesc, (kb | j) ? 1u : 0u);
                    }
                    tc_commit_pair_both(smem_u32(&bars->stage_free[s]), 3);     // frees the stage in both CTAs
                    if (++s == kPairStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                tc_commit_pair_both(smem_u32(&bars->d_full), 3);
            }
        }
    } else if (warp >= 4 && warp < 4 + 4 * kGemmDecodeGroups) {
        // ---------------- decode: raw blocks -> bf16 rows in this CTA's tensor memory ----------------
        const uint32_t quarter = warp & 3u, grp = (warp - 4) >> 2;
        const uint32_t row = quarter * 32 + lane;
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t r = 0, rph = 0, kbg0 = 0;
        bool ok = true;
        for (uint32_t pt = pt0; ok && pt < plim && !*abort_flag; pt += pstep) {
            for (uint32_t g = 0; g < P.kgroups && ok; ++g, kbg0 += 4) {
                if (*abort_flag || !pair_wait<SCHEME>(smem_u32(&bars->raw_full[r]), rph, lane)) { give_up(26); ok = false; break; }
                const uint8_t* rp = raw_stage + r * RAW_STRIDE + row * RAW_ROW;
#pragma unroll
                for (uint32_t sub = 0; sub < 4; ++sub) {
                    const uint32_t kbg = kbg0 + sub;
                    if (kbg % kGemmDecodeGroups != grp) continue;
                    // 64-wide block kbg is part kbg % kPairRound of round kbg / kPairRound
                    const uint32_t rd = kbg / kPairRound, s = rd % kPairStages, fph = ((rd / kPairStages) & 1u) ^ 1u;
                    uint32_t v[32];
                    if (sub == 0) decode64<SCHEME, 0>(rp, g, v);
                    else if (sub == 1) decode64<SCHEME, 1>(rp, g, v);
                    else if (sub == 2) decode64<SCHEME, 2>(rp, g, v);
                    else decode64<SCHEME, 3>(rp, g, v);
                    if (*abort_flag || !pair_wait<SCHEME>(smem_u32(&bars->stage_free[s]), fph, lane)) { give_up(27); ok = false; break; }
                    tc_fence_after();
                    tmem_st32(tmem_a + lane_addr + 32 * (kPairRound * s + kbg % kPairRound), v);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0) mbar_arrive(smem_u32(&bars->a_full[s]));
                        else mbar_arrive_cluster(cluster_map(smem_u32(&bars->a_full[s]), 0));
                    }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->raw_empty[r]));
                if (++r == kGemmRawStages) { r = 0; rph ^= 1u; }
            }
        }
    } else if (warp >= 4 + 4 * kGemmDecodeGroups) {
        // ---------------- epilogue: this CTA's 128 weight rows x 256 activation rows -> y ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t lane_addr = (quarter * 32) << 16;
        const uint32_t row = quarter * 32 + lane;
        const uint32_t epi_tid = (warp - (4 + 4 * kGemmDecodeGroups)) * 32 + lane;
        uint32_t dph = 0;
        for (uint32_t pt = pt0; pt < plim && !*abort_flag; pt += pstep) {
            const uint32_t wt = 2 * (pt / P.xtiles) + rank, xrow0 = (pt % P.xtiles) * TX;
            if (!mbar_wait_warp(smem_u32(&bars->d_full), dph, lane)) { give_up(28); break; }
            dph ^= 1u;
            tc_fence_after();
            const uint32_t n_idx = wt * kGemmTileW + row;
#pragma unroll 1
            for (uint32_t c = 0; c < TX / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_d + lane_addr + 32 * c, v);
                tmem_ld_wait();
                if (c == TX / 32 - 1) {          // everything is in registers: the accumulator may be overwritten
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0) mbar_arrive(smem_u32(&bars->d_free));
                        else mbar_arrive_cluster(cluster_map(smem_u32(&bars->d_free), 0));
                    }
                }
                if (P.y_vec) {
                    const GemmDst d{reinterpret_cast<uint8_t*>(P.y), P.n, xrow0, P.m, wt * kGemmTileW, P.n};
                    if (P.y_bf16) gemm_store_vec<false>(epi_stage, epi_tid, row, v, d, c);
                    else gemm_store_vec<true>(epi_stage, epi_tid, row, v, d, c);
                } else if (n_idx < P.n) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        const uint32_t m_idx = xrow0 + 32 * c + j;
                        if (m_idx < P.m) {
                            const size_t o = (size_t)m_idx * P.n + n_idx;
                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)bf16x2_of(f32x2(v[j], 0u));
                            else reinterpret_cast<float*>(P.y)[o] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
        }
    }
    // both CTAs meet here, also after a timeout: neither returns its tensor memory while the other may still use it
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ---- host side --------------------------------------------------------------------------------
bool gemm_tc_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf) {
    if (!xbf || m == 0 || n == 0 || k == 0 || k % 256) return false;
    if (scheme != RLXQ_Q4_0 && scheme != RLXQ_Q8_0 && scheme != RLXQ_Q4_K && scheme != RLXQ_Q6_K && scheme != RLXQ_Q5_K &&
        scheme != RLXQ_Q2_K && scheme != RLXQ_Q3_K && scheme != RLXQ_Q8_K && scheme != RLXQ_Q4_1 && scheme != RLXQ_Q5_0 &&
        scheme != RLXQ_Q5_1) return false;
    if ((scheme == RLXQ_Q6_K || scheme == RLXQ_Q3_K) && k % 2048) return false;   // rows must stay 16-byte aligned
    if ((scheme == RLXQ_Q2_K || scheme == RLXQ_Q8_K) && k % 1024) return false;
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    return true;
}

// The k split ("stream-K") evens the work out over the SMs, at the price of exchanging partial tiles through
// memory, which costs about as much as 36 steps of one 256-wide k group.  It is chosen when it saves at
// least that many steps on the busiest SM against whole tiles (of the width they would be given): few
// tiles and a long k, e.g. the down projection of a tensor-parallel shard at a small batch.
static bool gemm_wants_streamk(uint32_t m, uint32_t k, uint32_t n) {
    const int64_t opt = options().gemm_streamk.load();
    if (opt == 1) return false;
    if (opt == 2) return true;
    const uint64_t sms = (uint64_t)sm_count(), wt = (n + kGemmTileW - 1) / kGemmTileW, kgroups = k / 256;
    const uint64_t ntiles256 = wt * ((m + 255) / 256), ntiles128 = wt * ((m + 127) / 128);
    const uint64_t whole_tiles = ntiles256 * 4 < sms * 3 ? ntiles128 : ntiles256;
    const uint64_t steps_whole = (whole_tiles + sms - 1) / sms * kgroups;
    const uint64_t steps_split = (ntiles256 * kgroups + sms - 1) / sms;
    return steps_whole >= steps_split + 36;
}
static size_t gemm_streamk_bytes(uint32_t ntiles, size_t* off_partial) {
    const size_t counters = ((size_t)ntiles * 4 + 255) / 256 * 256;
    if (off_partial) *off_partial = counters;
    return counters + 2 * (size_t)sm_count() * kGemmTileW * 256 * 4;     // two partial tiles per CTA
}

// Scratch the GEMM would use for this shape (0 when whole tiles fill the SMs well enough).
size_t gemm_tc_workspace_bytes(uint32_t m, uint32_t k, uint32_t n) {
    if (m <= 8 || k == 0 || k % 256) return 0;
    const uint32_t ntiles = ((n + kGemmTileW - 1) / kGemmTileW) * ((m + 255) / 256);
    return gemm_wants_streamk(m, k, n) ? gemm_streamk_bytes(ntiles, nullptr) : 0;
}

template <uint32_t SCHEME, uint32_t TX>
static int launch_gemm_t(cudaStream_t stream, const void* x, const uint8_t* w, void* y, bool ybf, uint32_t m,
                         uint32_t k, uint32_t n, void* ws, bool streamk, const uint4* groups = nullptr,
                         uint32_t group_tiles = 0, uint32_t num_slabs = 1) {
    constexpr uint32_t RAW_ROW = GemmRaw<SCHEME>::ROW;
    constexpr uint32_t RAW_STRIDE = (kGemmTileW * RAW_ROW + 127) / 128 * 128;
    Geometry g;
    geometry(SCHEME, &g);
    GemmParams P{};
    int rc = encode_bf16_kmajor_map(&P.xmap, x, m, k, TX);
    if (rc) return rc;
    rc = encode_weight_map(&P.wmap, w, (uint64_t)n * num_slabs, (uint64_t)k / g.elems * g.bytes, RAW_ROW / 8, kGemmTileW);
    if (rc) return rc;
    P.y = y; P.m = m; P.n = n; P.k = k; P.y_bf16 = ybf;
    P.groups = groups;
    P.y_vec = (((uintptr_t)y & 15u) == 0 && n % (ybf ? 8u : 4u) == 0) ? 1u : 0u;
    P.wtiles = (n + kGemmTileW - 1) / kGemmTileW;
    P.xtiles = groups ? group_tiles : (m + TX - 1) / TX;
    P.kgroups = k / 256;
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    const size_t smem = 1024 + (size_t)GemmRaw<SCHEME>::STAGES * TX * kGemmBK * 2 + (size_t)kGemmRawStages * RAW_STRIDE +
                        sizeof(GemmBars) + 64 + kGemmEpiStage;
    static std::atomic<uint32_t> attr_set[64];
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<SCHEME, TX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev].store(1);
    }
    uint32_t grid = (uint32_t)sm_count();
    const uint32_t ntiles = P.wtiles * P.xtiles;
    if (streamk) {
        const uint64_t units = (uint64_t)ntiles * P.kgroups;
        if (units > 0xFFFFFFFFull) return fail(RLXQ_E_LIMIT, "GEMM too large for the stream-K split");
        if (grid > units) grid = (uint32_t)units;
        size_t off_partial = 0;
        gemm_streamk_bytes(ntiles, &off_partial);
        P.streamk = 1;
        P.units_q = (uint32_t)(units / grid);
        P.units_r = (uint32_t)(units % grid);
        P.counters = reinterpret_cast<uint32_t*>(ws);
        P.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + off_partial);
        RLXQ_CUDA_TRY(cudaMemsetAsync(P.counters, 0, (size_t)ntiles * 4, stream));
    } else if (grid > ntiles) {
        grid = ntiles;
    }
    gemm_tcgen05_kernel<SCHEME, TX><<<grid, (4 + 4 * GemmRaw<SCHEME>::GROUPS + 4) * 32, smem, stream>>>(P);
    count_launch();
    return check_launch("gemm_tcgen05_kernel");
}

// The two-CTA form: whole 256 x 256 tile pairs dealt round-robin to as many clusters as are resident at once.
static bool gemm_pair_fits(uint32_t m, uint32_t k, uint32_t n) {
    return n % 256 == 0 && m >= 1 && k % 256 == 0;
}
// Chosen by itself where it measured faster: at least one 256 x 256 tile pair per resident cluster, and a format
// whose decoder keeps pace with two groups of decode warps (Q6_K and Q3_K, with three groups, lose 5-12 % in the
// paired form on large shapes).
template <uint32_t SCHEME>
static bool gemm_wants_pair(uint32_t m, uint32_t k, uint32_t n) {
    const int64_t opt = options().gemm_pair.load();
    if (opt == 1 || !gemm_pair_fits(m, k, n)) return false;
    if (opt == 2) return true;
    if (SCHEME == RLXQ_Q6_K || SCHEME == RLXQ_Q3_K) return false;
    return (uint64_t)(n / 256) * ((m + 255) / 256) >= (uint64_t)sm_count() / 2;
}
template <uint32_t SCHEME>
static int launch_gemm_pair_t(cudaStream_t stream, const void* x, const uint8_t* w, void* y, bool ybf, uint32_t m,
                              uint32_t k, uint32_t n) {
    constexpr uint32_t RAW_ROW = GemmRaw<SCHEME>::ROW;
    constexpr uint32_t RAW_STRIDE = (kGemmTileW * RAW_ROW + 127) / 128 * 128;
    Geometry g;
    geometry(SCHEME, &g);
    GemmParams P{};
    int rc = encode_bf16_kmajor_map(&P.xmap, x, m, k, kPairHalf);
    if (rc) return rc;
    rc = encode_weight_map(&P.wmap, w, n, (uint64_t)k / g.elems * g.bytes, RAW_ROW / 8, kGemmTileW);
    if (rc) return rc;
    P.y = y; P.m = m; P.n = n; P.k = k; P.y_bf16 = ybf;
    P.y_vec = (((uintptr_t)y & 15u) == 0 && n % (ybf ? 8u : 4u) == 0) ? 1u : 0u;
    P.wtiles = n / kGemmTileW;
    P.xtiles = (m + 255) / 256;
    P.kgroups = k / 256;
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    const size_t smem = 1024 + (size_t)kPairStages * kPairBBytes + (size_t)kGemmRawStages * RAW_STRIDE + sizeof(PairBars) + 64 +
                        kGemmEpiStage;
    const uint32_t threads = (4 + 4 * GemmRaw<SCHEME>::GROUPS + 4) * 32;
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static std::atomic<int> clusters_of[64];        // resident clusters per device, found once (0 = not yet)
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    int clusters = (dev >= 0 && dev < 64) ? clusters_of[dev].load() : 0;
    if (clusters == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cfg.gridDim = dim3((unsigned)sm_count() & ~1u);
        RLXQ_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<SCHEME>, &cfg));
        if (clusters < 1) return fail(RLXQ_E_CUDA, "no cluster of two CTAs of the paired GEMM fits this device");
        if (dev >= 0 && dev < 64) clusters_of[dev].store(clusters);
        options().gemm_pair_clusters = clusters;
    }
    const uint32_t ptiles = (P.wtiles / 2) * P.xtiles;
    uint32_t pairs = (uint32_t)clusters;
    if (pairs > (uint32_t)sm_count() / 2) pairs = (uint32_t)sm_count() / 2;
    if (pairs > ptiles) pairs = ptiles;
    cfg.gridDim = dim3(2 * pairs);
    RLXQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<SCHEME>, P));
    count_launch();
    return check_launch("gemm_pair_kernel");
}

// 256-row activation tiles halve the activation traffic per FLOP.  When whole tiles would fill the SMs
// badly the k dimension is split as well (stream-K, needs the workspace); without a workspace, 128-row
// tiles are used when the wider ones would leave more than a quarter of the SMs without a tile.
template <uint32_t SCHEME>
static int launch_gemm_s(cudaStream_t stream, const void* x, const uint8_t* w, void* y, bool ybf, uint32_t m,
                         uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    const uint32_t wt = (n + kGemmTileW - 1) / kGemmTileW, sms = (uint32_t)sm_count();
    const int64_t force = options().gemm_tile_x.load();
    const uint32_t ntiles256 = wt * ((m + 255) / 256);
    if (options().gemm_pair.load() == 2 && gemm_pair_fits(m, k, n))               // forced: two CTAs per MMA
        return launch_gemm_pair_t<SCHEME>(stream, x, w, y, ybf, m, k, n);
    if (force != 128 && gemm_wants_streamk(m, k, n) && ws && !((uintptr_t)ws & 15u) &&
        ws_bytes >= gemm_streamk_bytes(ntiles256, nullptr))
        return launch_gemm_t<SCHEME, 256>(stream, x, w, y, ybf, m, k, n, ws, true);
    const bool narrow = force ? force == 128 : (ntiles256 * 4 < sms * 3);
    if (narrow) return launch_gemm_t<SCHEME, 128>(stream, x, w, y, ybf, m, k, n, nullptr, false);
    if (force == 0 && gemm_wants_pair<SCHEME>(m, k, n)) return launch_gemm_pair_t<SCHEME>(stream, x, w, y, ybf, m, k, n);
    return launch_gemm_t<SCHEME, 256>(stream, x, w, y, ybf, m, k, n, nullptr, false);
}

// Grouped form for MoE expert stacks: x holds x_rows gathered bf16 activation rows, w a stack of num_slabs
// [n, k] slabs, groups[0 .. group_tiles) the device-side table of activation tiles of tile_rows (128 or 256) rows
// (GemmParams::groups), y2 the f32 result rows in the order of x.
template <uint32_t SCHEME>
static int launch_gemm_grouped_s(cudaStream_t stream, const void* x, uint32_t x_rows, const uint8_t* w, uint32_t num_slabs,
                                 float* y2, uint32_t k, uint32_t n, const uint4* gt, uint32_t group_tiles, uint32_t tile_rows) {
    if (tile_rows == 256) return launch_gemm_t<SCHEME, 256>(stream, x, w, y2, false, x_rows, k, n, nullptr, false, gt, group_tiles, num_slabs);
    return launch_gemm_t<SCHEME, 128>(stream, x, w, y2, false, x_rows, k, n, nullptr, false, gt, group_tiles, num_slabs);
}

int launch_gemm_grouped(cudaStream_t stream, uint32_t scheme, const void* x, uint32_t x_rows, const uint8_t* w,
                        uint32_t num_slabs, float* y2, uint32_t k, uint32_t n, const void* groups, uint32_t group_tiles,
                        uint32_t tile_rows) {
    const uint4* gt = static_cast<const uint4*>(groups);
    if ((uint64_t)n * num_slabs > 0x7FFFFFFFull) return fail(RLXQ_E_LIMIT, "expert stack too tall for a tensor map");
    if (tile_rows != 128 && tile_rows != 256) return fail(RLXQ_E_ARG, "activation tiles are 128 or 256 rows");
    switch (scheme) {
        case RLXQ_Q4_0: return launch_gemm_grouped_s<RLXQ_Q4_0>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q8_0: return launch_gemm_grouped_s<RLXQ_Q8_0>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q4_K: return launch_gemm_grouped_s<RLXQ_Q4_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q5_K: return launch_gemm_grouped_s<RLXQ_Q5_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q2_K: return launch_gemm_grouped_s<RLXQ_Q2_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q8_K: return launch_gemm_grouped_s<RLXQ_Q8_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q4_1: return launch_gemm_grouped_s<RLXQ_Q4_1>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q5_0: return launch_gemm_grouped_s<RLXQ_Q5_0>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q5_1: return launch_gemm_grouped_s<RLXQ_Q5_1>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q3_K: return launch_gemm_grouped_s<RLXQ_Q3_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        case RLXQ_Q6_K: return launch_gemm_grouped_s<RLXQ_Q6_K>(stream, x, x_rows, w, num_slabs, y2, k, n, gt, group_tiles, tile_rows);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme");
    }
}

int launch_gemm_tc(cudaStream_t stream, uint32_t scheme, const void* x, const uint8_t* w, void* y, bool ybf,
                   uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    switch (scheme) {
        case RLXQ_Q4_0: return launch_gemm_s<RLXQ_Q4_0>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q8_0: return launch_gemm_s<RLXQ_Q8_0>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q4_K: return launch_gemm_s<RLXQ_Q4_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q5_K: return launch_gemm_s<RLXQ_Q5_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q2_K: return launch_gemm_s<RLXQ_Q2_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q8_K: return launch_gemm_s<RLXQ_Q8_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q4_1: return launch_gemm_s<RLXQ_Q4_1>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q5_0: return launch_gemm_s<RLXQ_Q5_0>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q5_1: return launch_gemm_s<RLXQ_Q5_1>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q3_K: return launch_gemm_s<RLXQ_Q3_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q6_K: return launch_gemm_s<RLXQ_Q6_K>(stream, x, w, y, ybf, m, k, n, ws, ws_bytes);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme");
    }
}

}  // namespace rlxq
