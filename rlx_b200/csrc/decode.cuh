// Device-side GGUF block decoders shared by every kernel in the library.
//
// Semantics follow rlx-gguf/src/lib.rs: Q8_0 :574-581, Q4_0 :584-597, the 6-bit scale/min
// unpack :743-751, Q4_K :974-1013, Q6_K :1070-1114 (signed sub-scales).  Where a kernel
// must reproduce the reference's f32 values bit for bit it uses the *_exact functions,
// which spell every rounding with __fmul_rn / __fsub_rn so nvcc cannot contract a
// multiply and a subtract into one FMA (Rust never does).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace rlxq {

// Expert id of a row as the reference reads it, `expert_idx[i] as usize` (rlx-cpu/src/gguf_matmul.rs:187,198):
// a saturating cast, so NaN and every value below 1 select expert 0.  An id of num_experts or more indexes
// out of bounds in the reference; here such a row is in no group (false) and its output stays zero.
__device__ __forceinline__ bool expert_of_row(float f, uint32_t num_experts, uint32_t* e) {
    if (!(f >= 1.0f)) { *e = 0u; return true; }
    if (f >= (float)num_experts) return false;
    *e = (uint32_t)f;
    return true;
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) {
    // Exact for every fp16 value, subnormals included (rlx-gguf/src/lib.rs:569-571).
    return __half2float(__ushort_as_half((unsigned short)bits));
}

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);  // blocks are always 2-byte aligned
}

// Unaligned-safe 32-bit read built from two 16-bit reads.
__device__ __forceinline__ uint32_t ld_u32_2(const uint8_t* p) {
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}

// 6-bit (scale, min) pair j of a Q4_K super-block; q points at the 12 scale bytes.
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, uint32_t& sc, uint32_t& mn) {
    if (j < 4) {
        sc = q[j] & 63u;
        mn = q[j + 4] & 63u;
    } else {
        sc = (q[j + 4] & 0x0Fu) | ((uint32_t)(q[j - 4] >> 6) << 4);
        mn = ((uint32_t)q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
}

// Decode 4 consecutive weights starting at element t (t % 4 == 0) of the block at `b`.
// Bit-identical to the reference decoders.
template <uint32_t SCHEME>
__device__ __forceinline__ float4 decode4_exact(const uint8_t* b, uint32_t t);

template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q8_0>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t w = ld_u32_2(b + 2 + t);
    float4 r;
    r.x = __fmul_rn(d, (float)(int8_t)(w & 0xFF));
    r.y = __fmul_rn(d, (float)(int8_t)((w >> 8) & 0xFF));
    r.z = __fmul_rn(d, (float)(int8_t)((w >> 16) & 0xFF));
    r.w = __fmul_rn(d, (float)(int8_t)(w >> 24));
    return r;
}

template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q4_0>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    // elements 0..15 are the low nibbles of qs[0..15], 16..31 the high nibbles
    const uint32_t w = ld_u32_2(b + 2 + (t & 15u)) >> ((t & 16u) ? 4 : 0);
    float4 r;
    r.x = __fmul_rn(d, (float)((int)(w & 0xF) - 8));
    r.y = __fmul_rn(d, (float)((int)((w >> 8) & 0xF) - 8));
    r.z = __fmul_rn(d, (float)((int)((w >> 16) & 0xF) - 8));
    r.w = __fmul_rn(d, (float)((int)((w >> 24) & 0xF) - 8));
    return r;
}

template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q4_K>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const float dmin = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t pair = t >> 6;         // 64 weights per (low, high) sub-block pair
    const uint32_t within = t & 63u;
    const uint32_t hi = within >> 5;      // 0: low nibbles (sub-block 2*pair), 1: high nibbles
    uint32_t sc, mn;
    q4k_scale_min((int)(2 * pair + hi), b + 4, sc, mn);
    const float dj = __fmul_rn(d, (float)sc);
    const float mj = __fmul_rn(dmin, (float)mn);
    const uint32_t w = ld_u32_2(b + 16 + 32 * pair + (within & 31u)) >> (hi ? 4 : 0);
    float4 r;
    r.x = __fsub_rn(__fmul_rn(dj, (float)(w & 0xF)), mj);
    r.y = __fsub_rn(__fmul_rn(dj, (float)((w >> 8) & 0xF)), mj);
    r.z = __fsub_rn(__fmul_rn(dj, (float)((w >> 16) & 0xF)), mj);
    r.w = __fsub_rn(__fmul_rn(dj, (float)((w >> 24) & 0xF)), mj);
    return r;
}

template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q6_K>(const uint8_t* b, uint32_t t) {
    // layout: ql[128] | qh[64] | sc[16] (i8) | d (f16)
    const uint32_t h = t >> 7;            // half of the super-block
    const uint32_t r7 = t & 127u;
    const uint32_t g = r7 >> 5;           // which of the four interleaved 32-element groups
    const uint32_t l = r7 & 31u;
    const float d = f16_bits_to_f32(ld_u16(b + 208));
    const int sc = (int)(int8_t)b[192 + 8 * h + (l >> 4) + 2 * g];
    const float ds = __fmul_rn(d, (float)sc);
    const uint32_t lo = ld_u32_2(b + 64 * h + l + ((g & 1u) ? 32u : 0u)) >> ((g & 2u) ? 4 : 0);
    const uint32_t hi = ld_u32_2(b + 128 + 32 * h + l) >> (2 * g);
    float4 r;
    r.x = __fmul_rn(ds, (float)((int)((lo & 0xF) | ((hi & 3u) << 4)) - 32));
    r.y = __fmul_rn(ds, (float)((int)(((lo >> 8) & 0xF) | (((hi >> 8) & 3u) << 4)) - 32));
    r.z = __fmul_rn(ds, (float)((int)(((lo >> 16) & 0xF) | (((hi >> 16) & 3u) << 4)) - 32));
    r.w = __fmul_rn(ds, (float)((int)(((lo >> 24) & 0xF) | (((hi >> 24) & 3u) << 4)) - 32));
    return r;
}

// Q5_K (rlx-gguf/src/lib.rs:783-816, 1019-1068): d | dmin | 12 scale bytes | qh[32] | qs[128].
// Sub-block j = 2*pair + hi takes nibble hi of qs[32*pair + l] plus 16 if bit j of qh[l] is set.
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q5_K>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const float dmin = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t pair = t >> 6, within = t & 63u, hi = within >> 5, l = within & 31u;
    uint32_t sc, mn;
    q4k_scale_min((int)(2 * pair + hi), b + 4, sc, mn);
    const float dj = __fmul_rn(d, (float)sc);
    const float mj = __fmul_rn(dmin, (float)mn);
    const uint32_t w = ld_u32_2(b + 48 + 32 * pair + l) >> (hi ? 4 : 0);
    const uint32_t hb = ld_u32_2(b + 16 + l) >> (2 * pair + hi);
    float4 r;
    r.x = __fsub_rn(__fmul_rn(dj, (float)((w & 0xF) + ((hb & 1u) << 4))), mj);
    r.y = __fsub_rn(__fmul_rn(dj, (float)(((w >> 8) & 0xF) + (((hb >> 8) & 1u) << 4))), mj);
    r.z = __fsub_rn(__fmul_rn(dj, (float)(((w >> 16) & 0xF) + (((hb >> 16) & 1u) << 4))), mj);
    r.w = __fsub_rn(__fmul_rn(dj, (float)(((w >> 24) & 0xF) + (((hb >> 24) & 1u) << 4))), mj);
    return r;
}

// Q8_K (rlx-gguf/src/lib.rs:848-854, 1121-1140): f32 d | 256 i8 | 16 i16 block sums (not read).
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q8_K>(const uint8_t* b, uint32_t t) {
    const float d = __uint_as_float(ld_u32_2(b));
    const uint32_t w = ld_u32_2(b + 4 + t);
    float4 r;
    r.x = __fmul_rn(d, (float)(int8_t)(w & 0xFF));
    r.y = __fmul_rn(d, (float)(int8_t)((w >> 8) & 0xFF));
    r.z = __fmul_rn(d, (float)(int8_t)((w >> 16) & 0xFF));
    r.w = __fmul_rn(d, (float)(int8_t)(w >> 24));
    return r;
}

// Q2_K as the reference reads it (rlx-gguf/src/lib.rs:857-886): d | dmin | 16 scale bytes | q[64].
// Per 128-weight half four 2-bit planes of 32 bytes; 16 weights share a (scale, min) nibble pair.
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q2_K>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const float mn = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t half = t >> 7, r7 = t & 127u, plane = r7 >> 5, within = r7 & 31u, sub = within >> 4, l = within & 15u;
    const uint32_t sc = b[4 + 8 * half + 2 * plane + sub];
    const float dl = __fmul_rn(d, (float)(sc & 0xFu));
    const float ml = __fmul_rn(mn, (float)(sc >> 4));
    const uint32_t w = ld_u32_2(b + 20 + 32 * half + 16 * sub + l) >> (2 * plane);
    float4 r;
    r.x = __fsub_rn(__fmul_rn(dl, (float)(w & 3u)), ml);
    r.y = __fsub_rn(__fmul_rn(dl, (float)((w >> 8) & 3u)), ml);
    r.z = __fsub_rn(__fmul_rn(dl, (float)((w >> 16) & 3u)), ml);
    r.w = __fsub_rn(__fmul_rn(dl, (float)((w >> 24) & 3u)), ml);
    return r;
}

// Q3_K as the reference reads it (rlx-gguf/src/lib.rs:889-930): d | 12 scale bytes | hmask[32] | q[64].
// Sixteen 6-bit scales: scale i has its low four bits in nibble (i >> 3) of byte (i & 7) and its high
// two bits at position 2 * (i >> 2) of byte 8 + (i & 3).  Weight = ((q >> 2*plane) & 3) - (mask bit ? 0 : 4).
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q3_K>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t half = t >> 7, r7 = t & 127u, plane = r7 >> 5, within = r7 & 31u, sub = within >> 4, l = within & 15u;
    const uint32_t is = 8 * half + 2 * plane + sub;
    const uint32_t low4 = (b[2 + (is & 7u)] >> (4 * (is >> 3))) & 0xFu;
    const uint32_t high2 = (b[10 + (is & 3u)] >> (2 * (is >> 2))) & 3u;
    const float dl = __fmul_rn(d, (float)((int)(low4 | (high2 << 4)) - 32));
    const uint32_t w = ld_u32_2(b + 46 + 32 * half + 16 * sub + l) >> (2 * plane);
    const uint32_t hm = ld_u32_2(b + 14 + 16 * sub + l) >> (4 * half + plane);
    float4 r;
    r.x = __fmul_rn(dl, (float)((int)(w & 3u) - ((hm & 1u) ? 0 : 4)));
    r.y = __fmul_rn(dl, (float)((int)((w >> 8) & 3u) - (((hm >> 8) & 1u) ? 0 : 4)));
    r.z = __fmul_rn(dl, (float)((int)((w >> 16) & 3u) - (((hm >> 16) & 1u) ? 0 : 4)));
    r.w = __fmul_rn(dl, (float)((int)((w >> 24) & 3u) - (((hm >> 24) & 1u) ? 0 : 4)));
    return r;
}

// Q4_1 (rlx-gguf/src/lib.rs:635-660): f16 d | f16 m | 16 bytes; weight j = low nibble of byte j, 16 + j = high nibble;
// value d * q + m, the product rounded before the sum as in the reference's `d * v0 + m`.
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q4_1>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b)), mn = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t w = ld_u32_2(b + 4 + (t & 15u)) >> (4 * (t >> 4));
    float4 r;
    r.x = __fadd_rn(__fmul_rn(d, (float)(w & 0xFu)), mn);
    r.y = __fadd_rn(__fmul_rn(d, (float)((w >> 8) & 0xFu)), mn);
    r.z = __fadd_rn(__fmul_rn(d, (float)((w >> 16) & 0xFu)), mn);
    r.w = __fadd_rn(__fmul_rn(d, (float)((w >> 24) & 0xFu)), mn);
    return r;
}

// Q5_0 (rlx-gguf/src/lib.rs:662-694): f16 d | u32 qh | 16 bytes; bit j (+16 for the high nibbles) of qh is the
// fifth bit of the quant; value d * (q - 16).
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q5_0>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t qh = ld_u32_2(b + 2) >> t;                       // bit i: fifth bit of weight t + i
    const uint32_t w = ld_u32_2(b + 6 + (t & 15u)) >> (4 * (t >> 4));
    float4 r;
    r.x = __fmul_rn(d, (float)((int)((w & 0xFu) | ((qh & 1u) << 4)) - 16));
    r.y = __fmul_rn(d, (float)((int)(((w >> 8) & 0xFu) | (((qh >> 1) & 1u) << 4)) - 16));
    r.z = __fmul_rn(d, (float)((int)(((w >> 16) & 0xFu) | (((qh >> 2) & 1u) << 4)) - 16));
    r.w = __fmul_rn(d, (float)((int)(((w >> 24) & 0xFu) | (((qh >> 3) & 1u) << 4)) - 16));
    return r;
}

// Q5_1 (rlx-gguf/src/lib.rs:696-729): f16 d | f16 m | u32 qh | 16 bytes; value d * q + m with the five-bit q.
template <>
__device__ __forceinline__ float4 decode4_exact<RLXQ_Q5_1>(const uint8_t* b, uint32_t t) {
    const float d = f16_bits_to_f32(ld_u16(b)), mn = f16_bits_to_f32(ld_u16(b + 2));
    const uint32_t qh = ld_u32_2(b + 4) >> t;
    const uint32_t w = ld_u32_2(b + 8 + (t & 15u)) >> (4 * (t >> 4));
    float4 r;
    r.x = __fadd_rn(__fmul_rn(d, (float)((w & 0xFu) | ((qh & 1u) << 4))), mn);
    r.y = __fadd_rn(__fmul_rn(d, (float)(((w >> 8) & 0xFu) | (((qh >> 1) & 1u) << 4))), mn);
    r.z = __fadd_rn(__fmul_rn(d, (float)(((w >> 16) & 0xFu) | (((qh >> 2) & 1u) << 4))), mn);
    r.w = __fadd_rn(__fmul_rn(d, (float)(((w >> 24) & 0xFu) | (((qh >> 3) & 1u) << 4))), mn);
    return r;
}

template <uint32_t SCHEME> struct SchemeTraits;
template <> struct SchemeTraits<RLXQ_Q4_1> { static constexpr uint32_t kElems = 32, kBytes = 20; };
template <> struct SchemeTraits<RLXQ_Q5_0> { static constexpr uint32_t kElems = 32, kBytes = 22; };
template <> struct SchemeTraits<RLXQ_Q5_1> { static constexpr uint32_t kElems = 32, kBytes = 24; };
template <> struct SchemeTraits<RLXQ_Q5_K> { static constexpr uint32_t kElems = 256, kBytes = 176; };
template <> struct SchemeTraits<RLXQ_Q8_K> { static constexpr uint32_t kElems = 256, kBytes = 292; };
template <> struct SchemeTraits<RLXQ_Q2_K> { static constexpr uint32_t kElems = 256, kBytes = 84; };
template <> struct SchemeTraits<RLXQ_Q3_K> { static constexpr uint32_t kElems = 256, kBytes = 110; };
template <> struct SchemeTraits<RLXQ_Q8_0> { static constexpr uint32_t kElems = 32, kBytes = 34; };
template <> struct SchemeTraits<RLXQ_Q4_0> { static constexpr uint32_t kElems = 32, kBytes = 18; };
template <> struct SchemeTraits<RLXQ_Q4_K> { static constexpr uint32_t kElems = 256, kBytes = 144; };
template <> struct SchemeTraits<RLXQ_Q6_K> { static constexpr uint32_t kElems = 256, kBytes = 210; };

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits) { return __uint_as_float(bits << 16); }

// Round-to-nearest-even f32 -> bf16 bits, NaN kept quiet (half::bf16::from_f32, used by
// narrow_f32_to_bytes at rlx-runtime/src/backend.rs:66-89).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint32_t x = __float_as_uint(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (x >> 16) | 0x40u;
    const uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return x >> 16;
}

}  // namespace rlxq
