/*
 * CPU oracle for the GGUF quantized-weight linear layer.  TEST INFRASTRUCTURE ONLY:
 * see rlxq_oracle.h for what it restates, how it is pinned, and who may call it.
 */
#include "rlxq_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* geometry — rlx-ir/src/quant.rs:138-164                              */
/* ------------------------------------------------------------------ */
int rlxo_scheme_geometry(uint32_t scheme, uint32_t* block_elems, uint32_t* block_bytes) {
    uint32_t e, b;
    switch (scheme) {
        case RLXO_Q4_K: e = 256; b = 144; break; /* f16 d, f16 dmin, 12 scale bytes, 128 nibble bytes */
        case RLXO_Q6_K: e = 256; b = 210; break; /* 128 ql, 64 qh, 16 i8 scales, f16 d */
        case RLXO_Q4_0: e = 32;  b = 18;  break; /* f16 d, 16 nibble bytes */
        case RLXO_Q8_0: e = 32;  b = 34;  break; /* f16 d, 32 i8 */
        case RLXO_Q5_K: e = 256; b = 176; break; /* f16 d, f16 dmin, 12 scale bytes, 32 high-bit bytes, 128 nibble bytes */
        case RLXO_Q8_K: e = 256; b = 292; break; /* f32 d, 256 i8, 16 i16 block sums */
        case RLXO_Q2_K: e = 256; b = 84;  break; /* as the reference reads it: f16 d, f16 dmin, 16 scale bytes, 64 quant bytes */
        case RLXO_Q3_K: e = 256; b = 110; break; /* as the reference reads it: f16 d, 12 scale bytes, 32 high-mask bytes, 64 quant bytes */
        case RLXO_Q4_1: e = 32;  b = 20;  break; /* f16 d, f16 m, 16 nibble bytes (rlx-gguf/src/lib.rs:405) */
        case RLXO_Q5_0: e = 32;  b = 22;  break; /* f16 d, u32 fifth bits, 16 nibble bytes (:406) */
        case RLXO_Q5_1: e = 32;  b = 24;  break; /* f16 d, f16 m, u32 fifth bits, 16 nibble bytes (:407) */
        default: return -1;
    }
    if (block_elems) *block_elems = e;
    if (block_bytes) *block_bytes = b;
    return 0;
}

/* ------------------------------------------------------------------ */
/* 16-bit float conversions (IEEE exact / round-to-nearest-even)       */
/* ------------------------------------------------------------------ */
static float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float rlxo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        /* subnormal: value = man * 2^-24, exact in f32 */
        float v = (float)man * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7F800000u | (man << 13)); /* inf / NaN kept */
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

uint16_t rlxo_f32_to_f16(float f) {
    uint32_t x = f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

float rlxo_bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

uint16_t rlxo_f32_to_bf16(float f) {
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u); /* quiet NaN */
    uint32_t round_bit = 0x8000u;
    if ((x & round_bit) != 0 && (x & (3u * round_bit - 1u)) != 0) return (uint16_t)((x >> 16) + 1u);
    return (uint16_t)(x >> 16);
}

static float read_f16_le(const uint8_t* b) { /* rlx-gguf/src/lib.rs:569-571 */
    return rlxo_f16_to_f32((uint16_t)(b[0] | ((uint16_t)b[1] << 8)));
}

/* ------------------------------------------------------------------ */
/* block decoders                                                      */
/* ------------------------------------------------------------------ */

/* rlx-gguf/src/lib.rs:574-581 */
static void dequant_q8_0_block(const uint8_t* block, float* out) {
    float d = read_f16_le(block);
    const uint8_t* qs = block + 2;
    for (int i = 0; i < 32; i++) out[i] = d * (float)(int8_t)qs[i];
}

/* rlx-gguf/src/lib.rs:584-597 — low nibbles fill the first half of the block. */
static void dequant_q4_0_block(const uint8_t* block, float* out) {
    float d = read_f16_le(block);
    const uint8_t* qs = block + 2;
    for (int j = 0; j < 16; j++) {
        int v0 = (int)(qs[j] & 0x0F) - 8;
        out[j] = d * (float)v0;
    }
    for (int j = 0; j < 16; j++) {
        int v1 = (int)(qs[j] >> 4) - 8;
        out[16 + j] = d * (float)v1;
    }
}

/* rlx-gguf/src/lib.rs:743-751 */
void rlxo_q4k_unpack_scale_min(int j, const uint8_t q[12], uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

void rlxo_q4k_pack_scales(const uint8_t sc[8], const uint8_t mn[8], uint8_t q[12]) {
    for (int i = 0; i < 4; i++) {
        q[i]     = (uint8_t)((sc[i] & 63) | ((sc[4 + i] >> 4) << 6));
        q[4 + i] = (uint8_t)((mn[i] & 63) | ((mn[4 + i] >> 4) << 6));
        q[8 + i] = (uint8_t)((sc[4 + i] & 0x0F) | ((mn[4 + i] & 0x0F) << 4));
    }
}

/* rlx-gguf/src/lib.rs:974-1013 (identical arithmetic to the block form at :754-780):
 * d0 = d*sc and m0 = dmin*m are rounded once, then each element is mul, then sub. */
static void dequant_q4_k_block(const uint8_t* block, float* out) {
    float d = read_f16_le(block);
    float dmin = read_f16_le(block + 2);
    const uint8_t* scales = block + 4;
    const uint8_t* qs = block + 16;
    int is = 0, oi = 0;
    for (int j = 0; j < 8; j += 2) {
        uint8_t sc0, m0, sc1, m1;
        rlxo_q4k_unpack_scale_min(j, scales, &sc0, &m0);
        rlxo_q4k_unpack_scale_min(j + 1, scales, &sc1, &m1);
        float d0 = d * (float)sc0;
        float m0f = dmin * (float)m0;
        float d1 = d * (float)sc1;
        float m1f = dmin * (float)m1;
        for (int l = 0; l < 32; l++) {
            float t = d0 * (float)(qs[is + l] & 0x0F);
            out[oi++] = t - m0f;
        }
        for (int l = 0; l < 32; l++) {
            float t = d1 * (float)(qs[is + l] >> 4);
            out[oi++] = t - m1f;
        }
        is += 32;
    }
}

/* rlx-gguf/src/lib.rs:1070-1114.  `d * sc * q` groups as (d*sc)*q. */
static void dequant_q6_k_block_impl(const uint8_t* block, float* out, int unsigned_scales) {
    const uint8_t* ql = block;
    const uint8_t* qh = block + 128;
    const uint8_t* sc = block + 192;
    float d = read_f16_le(block + 208);
    for (int h = 0; h < 2; h++) {
        int dst = h * 128, ql_off = h * 64, qh_off = h * 32, sc_off = h * 8;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            uint8_t qb = qh[qh_off + l];
            float q1 = (float)((int)((ql[ql_off + l] & 0x0F) | ((qb & 3) << 4)) - 32);
            float q2 = (float)((int)((ql[ql_off + l + 32] & 0x0F) | (((qb >> 2) & 3) << 4)) - 32);
            float q3 = (float)((int)((ql[ql_off + l] >> 4) | (((qb >> 4) & 3) << 4)) - 32);
            float q4 = (float)((int)((ql[ql_off + l + 32] >> 4) | (((qb >> 6) & 3) << 4)) - 32);
            float s1, s2, s3, s4;
            if (unsigned_scales) {
                s1 = (float)sc[sc_off + is];     s2 = (float)sc[sc_off + is + 2];
                s3 = (float)sc[sc_off + is + 4]; s4 = (float)sc[sc_off + is + 6];
            } else {
                s1 = (float)(int8_t)sc[sc_off + is];     s2 = (float)(int8_t)sc[sc_off + is + 2];
                s3 = (float)(int8_t)sc[sc_off + is + 4]; s4 = (float)(int8_t)sc[sc_off + is + 6];
            }
            float t1 = d * s1, t2 = d * s2, t3 = d * s3, t4 = d * s4;
            out[dst + l]      = t1 * q1;
            out[dst + l + 32] = t2 * q2;
            out[dst + l + 64] = t3 * q3;
            out[dst + l + 96] = t4 * q4;
        }
    }
}

/* rlx-gguf/src/lib.rs:783-816: Q4_K's scales and nibbles plus a fifth bit per weight from the
 * 32-byte plane qh (bit 2*pair for the low-nibble sub-block, bit 2*pair+1 for the high one);
 * per element one multiply and one subtract, each rounded. */
static void dequant_q5_k_block(const uint8_t* block, float* out) {
    float d = read_f16_le(block), dmin = read_f16_le(block + 2);
    const uint8_t* scales = block + 4;
    const uint8_t* qh = block + 16;
    const uint8_t* qs = block + 48;
    int is = 0, oi = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < 8; j += 2) {
        uint8_t sc0, m0, sc1, m1;
        rlxo_q4k_unpack_scale_min(j, scales, &sc0, &m0);
        rlxo_q4k_unpack_scale_min(j + 1, scales, &sc1, &m1);
        float d0 = d * (float)sc0, m0f = dmin * (float)m0;
        float d1 = d * (float)sc1, m1f = dmin * (float)m1;
        for (int l = 0; l < 32; l++) {
            int q = (qs[is + l] & 0x0F) + ((qh[l] & u1) ? 16 : 0);
            float t = d0 * (float)q;
            out[oi++] = t - m0f;
        }
        for (int l = 0; l < 32; l++) {
            int q = (qs[is + l] >> 4) + ((qh[l] & u2) ? 16 : 0);
            float t = d1 * (float)q;
            out[oi++] = t - m1f;
        }
        is += 32;
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

/* rlx-gguf/src/lib.rs:848-854 (block) and :1121-1140 (tensor): f32 scale, 256 i8; the 16 i16
 * block sums at the end are not read. */
static void dequant_q8_k_block(const uint8_t* block, float* out) {
    float d;
    memcpy(&d, block, 4);   /* little-endian host */
    for (int i = 0; i < 256; i++) out[i] = d * (float)(int8_t)block[4 + i];
}

/* rlx-gguf/src/lib.rs:857-886.  Layout as that decoder reads it: f16 d at 0, f16 dmin at 2,
 * 16 scale bytes (low nibble scale, high nibble min) at 4, 64 quant bytes at 20.  Two halves of
 * 128 weights; in each, four 2-bit planes (shift 0, 2, 4, 6) of 32 bytes, 16 weights per scale. */
static void dequant_q2_k_block(const uint8_t* block, float* out) {
    float d = read_f16_le(block), mn = read_f16_le(block + 2);
    const uint8_t* q = block + 20;
    int is = 0, oi = 0;
    for (int half = 0; half < 2; half++) {
        for (int shift = 0; shift < 8; shift += 2) {
            uint8_t sc = block[4 + is++];
            float dl = d * (float)(sc & 0xF), ml = mn * (float)(sc >> 4);
            for (int l = 0; l < 16; l++) {
                float t = dl * (float)((q[l] >> shift) & 3);
                out[oi++] = t - ml;
            }
            sc = block[4 + is++];
            dl = d * (float)(sc & 0xF);
            ml = mn * (float)(sc >> 4);
            for (int l = 0; l < 16; l++) {
                float t = dl * (float)((q[l + 16] >> shift) & 3);
                out[oi++] = t - ml;
            }
        }
        q += 32;
    }
}

/* rlx-gguf/src/lib.rs:889-930.  f16 d at 0, 12 scale bytes at 2 (sixteen 6-bit scales: low four
 * bits in bytes 0..7, high two bits in bytes 8..11), 32 high-mask bytes at 14, 64 quant bytes at
 * 46.  A weight is ((q >> shift) & 3) - (mask bit set ? 0 : 4), scaled by d * (scale - 32). */
static void dequant_q3_k_block(const uint8_t* block, float* out) {
    const uint32_t KMASK1 = 0x03030303u, KMASK2 = 0x0f0f0f0fu;
    float d_all = read_f16_le(block);
    const uint8_t* hm = block + 14;
    const uint8_t* q = block + 46;
    uint32_t aux[4];
    for (int i = 0; i < 3; i++)
        aux[i] = (uint32_t)block[2 + 4 * i] | ((uint32_t)block[3 + 4 * i] << 8) |
                 ((uint32_t)block[4 + 4 * i] << 16) | ((uint32_t)block[5 + 4 * i] << 24);
    uint32_t tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & KMASK2) | (((tmp >> 4) & KMASK1) << 4);
    aux[3] = ((aux[1] >> 4) & KMASK2) | (((tmp >> 6) & KMASK1) << 4);
    aux[0] = (aux[0] & KMASK2) | ((tmp & KMASK1) << 4);
    aux[1] = (aux[1] & KMASK2) | (((tmp >> 2) & KMASK1) << 4);
    int8_t scales[16];
    for (int i = 0; i < 16; i++) scales[i] = (int8_t)((aux[i >> 2] >> (8 * (i & 3))) & 0xFF);
    int is = 0, oi = 0;
    uint8_t m = 1;
    for (int half = 0; half < 2; half++) {
        for (int shift = 0; shift < 8; shift += 2) {
            float dl = d_all * (float)(int8_t)(scales[is++] - 32);
            for (int l = 0; l < 16; l++) {
                int h = (hm[l] & m) ? 0 : 4;
                out[oi++] = dl * (float)(int8_t)((int8_t)((q[l] >> shift) & 3) - h);
            }
            dl = d_all * (float)(int8_t)(scales[is++] - 32);
            for (int l = 0; l < 16; l++) {
                int h = (hm[l + 16] & m) ? 0 : 4;
                out[oi++] = dl * (float)(int8_t)((int8_t)((q[l + 16] >> shift) & 3) - h);
            }
            m = (uint8_t)(m << 1);
        }
        q += 32;
    }
}

/* rlx-gguf/src/lib.rs:635-660: d * q + m, product and sum rounded separately. */
static void dequant_q4_1_block(const uint8_t* b, float* out) {
    float d = rlxo_f16_to_f32((uint16_t)(b[0] | (b[1] << 8))), m = rlxo_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
    const uint8_t* qs = b + 4;
    for (int j = 0; j < 16; j++) { float v0 = (float)(qs[j] & 0x0F); float p = d * v0; out[j] = p + m; }
    for (int j = 0; j < 16; j++) { float v1 = (float)(qs[j] >> 4); float p = d * v1; out[16 + j] = p + m; }
}

/* rlx-gguf/src/lib.rs:662-694: bit j of qh (j + 16 for the high nibbles) is the fifth bit; d * (q - 16). */
static void dequant_q5_0_block(const uint8_t* b, float* out) {
    float d = rlxo_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
    uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    const uint8_t* qs = b + 6;
    for (int j = 0; j < 16; j++) {
        uint8_t xh0 = (uint8_t)(((qh >> j) & 1u) << 4);
        int v0 = (int)((qs[j] & 0x0F) | xh0) - 16;
        out[j] = d * (float)v0;
    }
    for (int j = 0; j < 16; j++) {
        uint8_t xh1 = (uint8_t)(((qh >> (j + 16)) & 1u) << 4);
        int v1 = (int)((qs[j] >> 4) | xh1) - 16;
        out[16 + j] = d * (float)v1;
    }
}

/* rlx-gguf/src/lib.rs:696-729: d * q + m with the five-bit q. */
static void dequant_q5_1_block(const uint8_t* b, float* out) {
    float d = rlxo_f16_to_f32((uint16_t)(b[0] | (b[1] << 8))), m = rlxo_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
    uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
    const uint8_t* qs = b + 8;
    for (int j = 0; j < 16; j++) {
        uint8_t xh0 = (uint8_t)(((qh >> j) & 1u) << 4);
        float v0 = (float)((qs[j] & 0x0F) | xh0);
        float p = d * v0;
        out[j] = p + m;
    }
    for (int j = 0; j < 16; j++) {
        uint8_t xh1 = (uint8_t)(((qh >> (j + 16)) & 1u) << 4);
        float v1 = (float)((qs[j] >> 4) | xh1);
        float p = d * v1;
        out[16 + j] = p + m;
    }
}

/* rlx-cpu/src/gguf_matmul.rs:25-37 with the Q6_K arm taken from the signed full-tensor
 * decoder (the per-block decoder the reference calls there reads the scales unsigned). */
static void dequant_block(uint32_t scheme, const uint8_t* block, float* out) {
    switch (scheme) {
        case RLXO_Q4_K: dequant_q4_k_block(block, out); break;
        case RLXO_Q6_K: dequant_q6_k_block_impl(block, out, 0); break;
        case RLXO_Q4_0: dequant_q4_0_block(block, out); break;
        case RLXO_Q8_0: dequant_q8_0_block(block, out); break;
        case RLXO_Q5_K: dequant_q5_k_block(block, out); break;
        case RLXO_Q8_K: dequant_q8_k_block(block, out); break;
        case RLXO_Q2_K: dequant_q2_k_block(block, out); break;
        case RLXO_Q3_K: dequant_q3_k_block(block, out); break;
        case RLXO_Q4_1: dequant_q4_1_block(block, out); break;
        case RLXO_Q5_0: dequant_q5_0_block(block, out); break;
        case RLXO_Q5_1: dequant_q5_1_block(block, out); break;
        default: break;
    }
}

int rlxo_dequant(uint32_t scheme, const uint8_t* blocks, uint64_t n_elems, float* out) {
    uint32_t be, bb;
    if (rlxo_scheme_geometry(scheme, &be, &bb)) return -1;
    if (n_elems % be) return -2;
    uint64_t nb = n_elems / be;
    for (uint64_t i = 0; i < nb; i++) dequant_block(scheme, blocks + i * bb, out + i * be);
    return 0;
}

int rlxo_dequant_q6k_unsigned(const uint8_t* blocks, uint64_t n_elems, float* out) {
    if (n_elems % 256) return -2;
    for (uint64_t i = 0; i < n_elems / 256; i++)
        dequant_q6_k_block_impl(blocks + i * 210, out + i * 256, 1);
    return 0;
}

/* ------------------------------------------------------------------ */
/* fused dequant + matmul — rlx-cpu/src/gguf_matmul.rs:40-95            */
/* ------------------------------------------------------------------ */
int rlxo_matmul_bt(const float* x, const uint8_t* w, float* out,
                   uint64_t m, uint64_t k, uint64_t n, uint32_t scheme) {
    uint32_t be, bb;
    if (rlxo_scheme_geometry(scheme, &be, &bb)) return -1;
    uint64_t total = k * n;
    if (total % be) return -2;
    uint64_t nb = total / be;
    memset(out, 0, (size_t)(m * n) * sizeof(float));
    float blockf[256];
    for (uint64_t bi = 0; bi < nb; bi++) {
        dequant_block(scheme, w + bi * bb, blockf);
        uint64_t idx0 = bi * be;
        for (uint32_t t = 0; t < be; t++) {
            uint64_t idx = idx0 + t;
            uint64_t j = idx / k, p = idx % k;
            float wv = blockf[t];
            for (uint64_t mi = 0; mi < m; mi++) {
                float prod = x[mi * k + p] * wv;
                out[mi * n + j] = out[mi * n + j] + prod;
            }
        }
    }
    return 0;
}

typedef struct {
    const float* x; const uint8_t* w; float* out;
    uint64_t m, k, n, j0, j1; uint32_t scheme, be, bb;
} mt_job;

static void* mt_worker(void* arg) {
    mt_job* jb = (mt_job*)arg;
    float blockf[256];
    uint64_t bpr = jb->k / jb->be; /* blocks per row */
    for (uint64_t j = jb->j0; j < jb->j1; j++) {
        for (uint64_t mi = 0; mi < jb->m; mi++) jb->out[mi * jb->n + j] = 0.0f;
        for (uint64_t b = 0; b < bpr; b++) {
            dequant_block(jb->scheme, jb->w + (j * bpr + b) * jb->bb, blockf);
            uint64_t p0 = b * jb->be;
            for (uint32_t t = 0; t < jb->be; t++) {
                float wv = blockf[t];
                for (uint64_t mi = 0; mi < jb->m; mi++) {
                    float prod = jb->x[mi * jb->k + p0 + t] * wv;
                    jb->out[mi * jb->n + j] = jb->out[mi * jb->n + j] + prod;
                }
            }
        }
    }
    return NULL;
}

int rlxo_matmul_bt_mt(const float* x, const uint8_t* w, float* out,
                      uint64_t m, uint64_t k, uint64_t n, uint32_t scheme,
                      uint64_t n0, uint64_t n1, int threads) {
    uint32_t be, bb;
    if (rlxo_scheme_geometry(scheme, &be, &bb)) return -1;
    if (k % be) return -2;
    if (n1 > n || n0 > n1) return -3;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    uint64_t rows = n1 - n0;
    if ((uint64_t)threads > rows) threads = rows ? (int)rows : 1;
    pthread_t th[256];
    mt_job jobs[256];
    for (int t = 0; t < threads; t++) {
        mt_job jb = { x, w, out, m, k, n, n0 + rows * (uint64_t)t / (uint64_t)threads,
                      n0 + rows * (uint64_t)(t + 1) / (uint64_t)threads, scheme, be, bb };
        jobs[t] = jb;
    }
    if (threads == 1) { mt_worker(&jobs[0]); return 0; }
    for (int t = 0; t < threads; t++) pthread_create(&th[t], NULL, mt_worker, &jobs[t]);
    for (int t = 0; t < threads; t++) pthread_join(th[t], NULL);
    return 0;
}

/* ------------------------------------------------------------------ */
/* SwiGLU FFN and all-reduce                                           */
/* ------------------------------------------------------------------ */
float rlxo_silu(float x) { return x / (1.0f + expf(-x)); } /* rlx-cpu/src/naive.rs:54-56 */

int rlxo_ffn_swiglu(const float* x, const uint8_t* gate, const uint8_t* up, const uint8_t* down,
                    float* y, float* h_out, uint64_t m, uint64_t d_model, uint64_t d_ffn,
                    uint32_t scheme_gate_up, uint32_t scheme_down, int threads) {
    size_t hn = (size_t)(m * d_ffn);
    float* g = (float*)malloc(hn * sizeof(float));
    float* u = (float*)malloc(hn * sizeof(float));
    if (!g || !u) { free(g); free(u); return -4; }
    int rc = rlxo_matmul_bt_mt(x, gate, g, m, d_model, d_ffn, scheme_gate_up, 0, d_ffn, threads);
    if (!rc) rc = rlxo_matmul_bt_mt(x, up, u, m, d_model, d_ffn, scheme_gate_up, 0, d_ffn, threads);
    if (!rc) {
        /* rlx-cuda/src/unfuse.rs:254-293: out = up * silu(gate) */
        for (size_t i = 0; i < hn; i++) u[i] = u[i] * rlxo_silu(g[i]);
        if (h_out) memcpy(h_out, u, hn * sizeof(float));
        rc = rlxo_matmul_bt_mt(u, down, y, m, d_ffn, d_model, scheme_down, 0, d_model, threads);
    }
    free(g); free(u);
    return rc;
}

void rlxo_allreduce_sum(const float* parts, uint64_t ranks, uint64_t elems, float* out) {
    for (uint64_t i = 0; i < elems; i++) {
        float acc = 0.0f;
        for (uint64_t r = 0; r < ranks; r++) acc = acc + parts[r * elems + i];
        out[i] = acc;
    }
}

/* ------------------------------------------------------------------ */
/* seeded synthetic inputs                                             */
/* ------------------------------------------------------------------ */
static uint64_t splitmix64(uint64_t* s) {
    uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static uint64_t stream_state(uint64_t seed, uint64_t idx) {
    uint64_t s = seed ^ (idx * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull);
    (void)splitmix64(&s);
    return s;
}
static float u01(uint64_t r) { return (float)(r >> 40) * (1.0f / 16777216.0f); } /* [0,1) */
static uint16_t gen_scale_f16(uint64_t* s) {                   /* fp16(U[1e-3, 1e-2]) */
    return rlxo_f32_to_f16(1e-3f + 9e-3f * u01(splitmix64(s)));
}
static void gen_bytes(uint64_t* s, uint8_t* out, int n) {
    for (int i = 0; i < n; i += 8) {
        uint64_t r = splitmix64(s);
        for (int b = 0; b < 8 && i + b < n; b++) out[i + b] = (uint8_t)(r >> (8 * b));
    }
}
static void put_u16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

int rlxo_fill_blocks(uint32_t scheme, uint64_t seed, uint64_t first_block, uint64_t n_blocks,
                     uint8_t* out) {
    uint32_t be, bb;
    if (rlxo_scheme_geometry(scheme, &be, &bb)) return -1;
    for (uint64_t i = 0; i < n_blocks; i++) {
        uint64_t s = stream_state(seed, first_block + i);
        uint8_t* b = out + i * bb;
        switch (scheme) {
            case RLXO_Q8_0: {
                put_u16(b, gen_scale_f16(&s));
                for (int j = 0; j < 32; j += 2) {
                    /* uniform over the 255 values -127..127, two per draw */
                    uint64_t r = splitmix64(&s);
                    int q0 = (int)((((r >> 32) * 255ull) >> 32)) - 127;
                    int q1 = (int)((((r & 0xFFFFFFFFull) * 255ull) >> 32)) - 127;
                    b[2 + j] = (uint8_t)(int8_t)q0;
                    b[3 + j] = (uint8_t)(int8_t)q1;
                }
                break;
            }
            case RLXO_Q4_0:
                put_u16(b, gen_scale_f16(&s));
                gen_bytes(&s, b + 2, 16);
                break;
            case RLXO_Q4_K:
                put_u16(b, gen_scale_f16(&s));
                put_u16(b + 2, gen_scale_f16(&s));
                /* 12 random bytes are a bijection onto sixteen independent 6-bit values */
                gen_bytes(&s, b + 4, 12);
                gen_bytes(&s, b + 16, 128);
                break;
            case RLXO_Q6_K:
                gen_bytes(&s, b, 192);
                gen_bytes(&s, b + 192, 16);
                for (int j = 0; j < 16; j++) /* i8 in [-64, 63] */
                    b[192 + j] = (uint8_t)(int8_t)((int)(b[192 + j] & 127) - 64);
                put_u16(b + 208, gen_scale_f16(&s));
                break;
            case RLXO_Q5_K:
                put_u16(b, gen_scale_f16(&s));
                put_u16(b + 2, gen_scale_f16(&s));
                gen_bytes(&s, b + 4, 12 + 32 + 128);   /* scales, fifth-bit plane, nibbles: all uniform */
                break;
            case RLXO_Q8_K: {
                float d = 1e-3f + 9e-3f * u01(splitmix64(&s));
                memcpy(b, &d, 4);
                gen_bytes(&s, b + 4, 256);
                for (int g = 0; g < 16; g++) {          /* block sums, as a quantiser would have written them */
                    int sum = 0;
                    for (int l = 0; l < 16; l++) sum += (int8_t)b[4 + 16 * g + l];
                    put_u16(b + 260 + 2 * g, (uint16_t)(int16_t)sum);
                }
                break;
            }
            case RLXO_Q2_K:
                put_u16(b, gen_scale_f16(&s));
                put_u16(b + 2, gen_scale_f16(&s));
                gen_bytes(&s, b + 4, 16 + 64);
                break;
            case RLXO_Q3_K:
                put_u16(b, gen_scale_f16(&s));
                gen_bytes(&s, b + 2, 12 + 32 + 64);
                break;
            case RLXO_Q4_1:          /* d and m like the other scales, quants uniform */
                put_u16(b, gen_scale_f16(&s));
                put_u16(b + 2, gen_scale_f16(&s));
                gen_bytes(&s, b + 4, 16);
                break;
            case RLXO_Q5_0:
                put_u16(b, gen_scale_f16(&s));
                gen_bytes(&s, b + 2, 4 + 16);
                break;
            case RLXO_Q5_1:
                put_u16(b, gen_scale_f16(&s));
                put_u16(b + 2, gen_scale_f16(&s));
                gen_bytes(&s, b + 4, 4 + 16);
                break;
            default: return -1;
        }
    }
    return 0;
}

void rlxo_fill_normal_f32(uint64_t seed, uint64_t first, uint64_t count, float* out) {
    /* Box-Muller on counter-based uniforms; element e depends only on (seed, e). */
    for (uint64_t i = 0; i < count; i++) {
        uint64_t e = first + i;
        uint64_t s = stream_state(seed ^ 0xA5A5A5A5DEADBEEFull, e >> 1);
        float u1 = u01(splitmix64(&s)) + (1.0f / 33554432.0f);
        float u2 = u01(splitmix64(&s));
        float r = sqrtf(-2.0f * logf(u1));
        float a = 6.28318530717958647692f * u2;
        out[i] = (e & 1) ? r * sinf(a) : r * cosf(a);
    }
}
