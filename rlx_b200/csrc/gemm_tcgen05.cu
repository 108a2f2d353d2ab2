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
#include "tensormap.cuh"

namespace rlxq {

constexpr uint32_t kGemmTileW = 128;    // weight rows per tile (MMA M, tensor-memory lanes)
constexpr uint32_t kGemmTileXMax = 256; // activation rows per tile (MMA N): 256, or 128 when that fills more SMs
constexpr uint32_t kGemmBK = 64;        // k per pipeline stage (one 128-byte swizzled row of bf16)
constexpr uint32_t kGemmMaxStages = 6;  // B shared-memory stages == A tensor-memory stages (4 or 5, by format)
constexpr uint32_t kGemmRawStages = 2;  // raw weight boxes (256 weights of 128 rows each)

// ---- tcgen05 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem descriptor]^T, bf16 inputs, f32 accumulate
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 operand stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes for a 64-element-wide box): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);           // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                  // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                  // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                                  // 128-byte swizzle
    return d;
}
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
// Q6_K super-blocks are 210 bytes: group g of a row starts at byte 210 g, which is only 2-byte aligned.
// The box starts at the 16-byte boundary below it and is 240 bytes wide (15 chunks: conflict-free, and
// 14 + 210 <= 240); the decoder is compiled for each of the eight possible offsets 2 (g mod 8).
template <> struct GemmRaw<RLXQ_Q6_K> { static constexpr uint32_t ROW = 240, STAGES = 4, GROUPS = 3; };
template <uint32_t SCHEME> __device__ __forceinline__ uint32_t gemm_raw_x(uint32_t g) {   // box start, 8-byte elements
    if (SCHEME == RLXQ_Q6_K) return ((210u * g) & ~15u) / 8u;
    return g * (GemmRaw<SCHEME>::ROW / 8u);
}

// float(b) for b in 0..255 without the conversion unit: 0x4B000000 | b is 2^23 + b
__device__ __forceinline__ float u8_to_f32(uint32_t b) { return __uint_as_float(0x4B000000u | b) - 8388608.0f; }
// float(b) - OFF in one exact subtraction (OFF a small integer)
template <int OFF>
__device__ __forceinline__ float u8_minus(uint32_t b) { return __uint_as_float(0x4B000000u | b) - (8388608.0f + (float)OFF); }

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
            const float d = f16_bits_to_f32(dbits);
#pragma unroll
            for (int p = 0; p < 8; ++p) {   // weights 2p, 2p+1: low nibbles of bytes 2p, 2p+1; 16+2p..: high nibbles
                const uint32_t word = qs[p >> 1] >> (16 * (p & 1));
                const float l0 = d * u8_minus<8>(word & 0xFu), l1 = d * u8_minus<8>((word >> 8) & 0xFu);
                const float h0 = d * u8_minus<8>((word >> 4) & 0xFu), h1 = d * u8_minus<8>((word >> 12) & 0xFu);
                v[16 * blk + p] = pack_bf16(l0, l1);
                v[16 * blk + 8 + p] = pack_bf16(h0, h1);
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
            const float d = f16_bits_to_f32(dbits);
#pragma unroll
            for (int p = 0; p < 16; ++p) {  // int8 -> (q + 128) unsigned -> float, minus 128
                const uint32_t u = (q[p >> 1] ^ 0x80808080u) >> (16 * (p & 1));
                v[16 * blk + p] = pack_bf16(d * u8_minus<128>(u & 0xFFu), d * u8_minus<128>((u >> 8) & 0xFFu));
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
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            const uint32_t word = qs[p >> 1] >> (16 * (p & 1));
            v[p] = pack_bf16(fmaf(dl, u8_to_f32(word & 0xFu), -ml), fmaf(dl, u8_to_f32((word >> 8) & 0xFu), -ml));
            v[16 + p] = pack_bf16(fmaf(dh, u8_to_f32((word >> 4) & 0xFu), -mh), fmaf(dh, u8_to_f32((word >> 12) & 0xFu), -mh));
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
                const float ds = gsel == 0 ? (i < 4 ? s00 : s01) : (i < 4 ? s10 : s11);
                v[16 * gsel + 2 * i] = pack_bf16(ds * u8_minus<32>(mw & 0xFFu), ds * u8_minus<32>((mw >> 8) & 0xFFu));
                v[16 * gsel + 2 * i + 1] = pack_bf16(ds * u8_minus<32>((mw >> 16) & 0xFFu), ds * u8_minus<32>(mw >> 24));
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
    uint32_t m, n, k, y_bf16;
    uint32_t wtiles, xtiles;
};

struct GemmBars {
    uint64_t b_full[kGemmMaxStages], a_full[kGemmMaxStages], stage_free[kGemmMaxStages];
    uint64_t raw_full[kGemmRawStages], raw_empty[kGemmRawStages];
    uint64_t d_full, d_free;
    uint32_t tmem_base, abort_flag;
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

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t kblocks = P.k / kGemmBK, kgroups = P.k / 256;
    const uint32_t ntiles = P.wtiles * P.xtiles;
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
            for (uint32_t t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                const uint32_t xt = t % P.xtiles;
                bool ok = true;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->stage_free[s]), ph)) { give_up(11); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->b_full[s]);
                    mbar_arrive_expect_tx(full, B_BYTES);
                    tma_load_2d(smem_u32(b_stage + s * B_BYTES), &P.xmap, (int32_t)(kb * kGemmBK), (int32_t)(xt * kGemmTileX), full);
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
            for (uint32_t t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                const uint32_t wt = t / P.xtiles;
                bool ok = true;
                for (uint32_t g = 0; g < kgroups; ++g) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_empty[r]), ph)) { give_up(12); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->raw_full[r]);
                    mbar_arrive_expect_tx(full, RAW_BYTES);
                    tma_load_2d(smem_u32(raw_stage + r * RAW_STRIDE), &P.wmap, (int32_t)gemm_raw_x<SCHEME>(g), (int32_t)(wt * kGemmTileW), full);
                    if (++r == kGemmRawStages) { r = 0; ph ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, dph = 1;   // dph: parity to wait for on d_free (1 passes the first time)
            for (uint32_t t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
                if (!mbar_wait(smem_u32(&bars->d_free), dph)) { give_up(13); break; }
                dph ^= 1u;
                tc_fence_after();
                bool ok = true;
                for (uint32_t kb = 0; kb < kblocks; ++kb) {
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
        for (uint32_t t = blockIdx.x; t < ntiles && ok && !*abort_flag; t += gridDim.x) {
            for (uint32_t g = 0; g < kgroups && ok; ++g, kbg0 += 4) {
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
        // ---------------- epilogue: accumulator -> y ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t lane_addr = (quarter * 32) << 16;
        uint32_t dph = 0;
        for (uint32_t t = blockIdx.x; t < ntiles && !*abort_flag; t += gridDim.x) {
            const uint32_t wt = t / P.xtiles, xt = t % P.xtiles;
            if (!mbar_wait(smem_u32(&bars->d_full), dph)) { give_up(17); break; }
            dph ^= 1u;
            tc_fence_after();
            const uint32_t n_idx = wt * kGemmTileW + quarter * 32 + lane;
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
                if (n_idx < P.n) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        const uint32_t m_idx = xt * kGemmTileX + 32 * c + j;
                        if (m_idx < P.m) {
                            const size_t o = (size_t)m_idx * P.n + n_idx;
                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(__uint_as_float(v[j]));
                            else reinterpret_cast<float*>(P.y)[o] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
        }
    }
    // everybody meets here, also after a timeout, so the tensor memory is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- host side --------------------------------------------------------------------------------
bool gemm_tc_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf) {
    if (!xbf || m == 0 || n == 0 || k == 0 || k % 256) return false;
    if (scheme != RLXQ_Q4_0 && scheme != RLXQ_Q8_0 && scheme != RLXQ_Q4_K && scheme != RLXQ_Q6_K) return false;
    if (scheme == RLXQ_Q6_K && k % 2048) return false;   // rows must stay 16-byte aligned
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    return true;
}

template <uint32_t SCHEME, uint32_t TX>
static int launch_gemm_t(cudaStream_t stream, const void* x, const uint8_t* w, void* y, bool ybf, uint32_t m,
                         uint32_t k, uint32_t n) {
    constexpr uint32_t RAW_ROW = GemmRaw<SCHEME>::ROW;
    constexpr uint32_t RAW_STRIDE = (kGemmTileW * RAW_ROW + 127) / 128 * 128;
    Geometry g;
    geometry(SCHEME, &g);
    GemmParams P{};
    int rc = encode_bf16_kmajor_map(&P.xmap, x, m, k, TX);
    if (rc) return rc;
    rc = encode_weight_map(&P.wmap, w, n, (uint64_t)k / g.elems * g.bytes, RAW_ROW / 8, kGemmTileW);
    if (rc) return rc;
    P.y = y; P.m = m; P.n = n; P.k = k; P.y_bf16 = ybf;
    P.wtiles = (n + kGemmTileW - 1) / kGemmTileW;
    P.xtiles = (m + TX - 1) / TX;
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    const size_t smem = 1024 + (size_t)GemmRaw<SCHEME>::STAGES * TX * kGemmBK * 2 + (size_t)kGemmRawStages * RAW_STRIDE +
                        sizeof(GemmBars) + 64;
    static std::atomic<uint32_t> attr_set[64];
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<SCHEME, TX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev].store(1);
    }
    uint32_t grid = (uint32_t)sm_count();
    const uint32_t ntiles = P.wtiles * P.xtiles;
    if (grid > ntiles) grid = ntiles;
    gemm_tcgen05_kernel<SCHEME, TX><<<grid, (4 + 4 * GemmRaw<SCHEME>::GROUPS + 4) * 32, smem, stream>>>(P);
    count_launch();
    return check_launch("gemm_tcgen05_kernel");
}

// 256-row activation tiles halve the activation traffic per FLOP; 128-row tiles are used when the
// wider ones would leave more than a quarter of the SMs without a tile.
template <uint32_t SCHEME>
static int launch_gemm_s(cudaStream_t stream, const void* x, const uint8_t* w, void* y, bool ybf, uint32_t m,
                         uint32_t k, uint32_t n) {
    const uint32_t wt = (n + kGemmTileW - 1) / kGemmTileW, sms = (uint32_t)sm_count();
    const int64_t force = options().gemm_tile_x.load();
    const bool narrow = force ? force == 128 : (wt * ((m + 255) / 256) * 4 < sms * 3);
    if (narrow) return launch_gemm_t<SCHEME, 128>(stream, x, w, y, ybf, m, k, n);
    return launch_gemm_t<SCHEME, 256>(stream, x, w, y, ybf, m, k, n);
}

int launch_gemm_tc(cudaStream_t stream, uint32_t scheme, const void* x, const uint8_t* w, void* y, bool ybf,
                   uint32_t m, uint32_t k, uint32_t n) {
    switch (scheme) {
        case RLXQ_Q4_0: return launch_gemm_s<RLXQ_Q4_0>(stream, x, w, y, ybf, m, k, n);
        case RLXQ_Q8_0: return launch_gemm_s<RLXQ_Q8_0>(stream, x, w, y, ybf, m, k, n);
        case RLXQ_Q4_K: return launch_gemm_s<RLXQ_Q4_K>(stream, x, w, y, ybf, m, k, n);
        case RLXQ_Q6_K: return launch_gemm_s<RLXQ_Q6_K>(stream, x, w, y, ybf, m, k, n);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme");
    }
}

}  // namespace rlxq
