// Streaming decode GEMV (m <= 8) for GGUF block formats on sm_100a.
//
// y[m,n] = x[m,k] . W^T with W's raw blocks streamed from HBM exactly once.
//
// Data movement.  A persistent CTA owns a set of 16-row weight tiles and one k-slice.  A
// producer warp streams the tile's rows through a ring of shared-memory stages with 1-D bulk
// async copies (cp.async.bulk, completion counted on an mbarrier): each copy is one row's
// 16-byte-aligned run of whole blocks, so HBM sees long contiguous bursts and no load
// instruction is spent on it.  Four consumer warps split every stage by 256-weight units.
//
// Arithmetic, batch 1-2 (integer mode).  Each CTA quantises its activation slice once to two
// int8 limbs per value (15 bits, one f32 scale per 32 values, exact block sums alongside).
// Weights stay integers: nibbles are masked out four at a time and multiplied with dp4a, which
// accumulates exactly in int32; one int->float conversion and one FMA per 32-weight block apply
// d_block * s_block.  Error: only the activation quantisation, |err| <= 1.7e-4 * |x| * |w_row|
// worst case (about 1e-6 typical), plus f32 accumulation across blocks.
//
// Arithmetic, batch 3-8 (tensor mode).  Block quants are small integers, so they are exact in fp16: a byte-permute
// builds the fp16 pair (1024 + q) from a raw byte and the constant 0x64, two weights per
// instruction, and mma.sync.m16n8k16 (f16 x f16 -> f32) multiplies a 16-row tile by the
// activation columns.  The activations are converted once per CTA to fp16 after an exact
// power-of-two rescale of each row; the "+1024" and the format's own offset (-8, -128, -32,
// or Q4_K's min term) are removed through per-block activation sums that seed the MMA
// accumulator.  Per block the f32 accumulator is scaled by the block's fp16 scale with one
// FMA per output.  All block decoding therefore happens in registers; nothing dequantised
// ever touches memory.  Error: the only rounding besides f32 accumulation is x -> fp16
// (relative 2^-12), i.e. |y - y_exact| <= 2.5e-4 * |x| * |w_row|, inside the path's 1e-3 bound.
//
// Reduction.  Warps of a CTA combine through shared memory in a fixed order.  When k is
// split over several CTAs (to keep the activation slice in shared memory or to fill the
// machine), each CTA writes its partial tile to the workspace and the CTA that arrives last
// at the tile's counter adds the partials in slice order, so the result is deterministic
// and no CTA ever waits for another.
//
// Replaces the reference's per-call "dequantise all of W to f32, then cublasSgemm"
// (rlx-cuda/src/gguf_gpu.rs:62-134), which moves about 8 bytes per weight; this kernel moves
// the packed 0.56-1.06 bytes per weight.
#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "staged_common.cuh"
#include "tensormap.cuh"

namespace rlxq {

// fp16 pair (1024 + byte i, 1024 + byte j) of v: 0x64 in the high byte is 1024 with ulp 1.
__device__ __forceinline__ uint32_t pair01(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4140); }
__device__ __forceinline__ uint32_t pair23(uint32_t v) { return __byte_perm(v, 0x64646464u, 0x4342); }

// Per-thread view of the tile a warp is working on.
struct Lane {
    const uint8_t* stage;   // first row of the stage
    const uint8_t* row_lo;  // stage row g      (g = lane / 4)
    const uint8_t* row_hi;  // stage row g + 8
    const __half* xrow;     // activation row min(g, m-1)... see below
    const float* sxb;       // activation block sums * BIAS, [block][mp]
    uint32_t t;             // lane % 4
    uint32_t mp;
};

// All fragment loads are unconditional.  Columns of the MMA are independent, so a lane whose
// column does not exist (g >= m) may feed any finite-or-not data: it reads activation row 0 and
// whatever follows its block's sums; the garbage stays in accumulator columns that are never
// stored.  Conditional loads here cost a branch each and serialise the unrolled blocks.
__device__ __forceinline__ uint2 ld_b64(const Lane& L, uint32_t k) {  // 4 activations at k
    return *reinterpret_cast<const uint2*>(L.xrow + k);
}
__device__ __forceinline__ uint4 ld_b128(const Lane& L, uint32_t k) {  // 8 activations at k
    return *reinterpret_cast<const uint4*>(L.xrow + k);
}
__device__ __forceinline__ float2 ld_sx(const Lane& L, uint32_t block) {
    return *reinterpret_cast<const float2*>(L.sxb + block * L.mp + 2 * L.t);
}

// ---------------------------------------------------------------------------------------------
// One 256-weight unit x 16 rows per warp.  `u_off` = byte offset of the unit inside a stage
// row, `kb` = k offset of the unit inside the CTA's activation slice.
// tot[0..3] = (row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1).
// ---------------------------------------------------------------------------------------------
template <uint32_t SCHEME> struct Unit;

template <> struct Unit<RLXQ_Q4_0> {
    __device__ static __forceinline__ void run(const Lane& L, uint32_t u_off, uint32_t kb, float* scratch,
                                               uint32_t lane, float (&tot)[4]) {
        (void)scratch; (void)lane;
#pragma unroll
        for (uint32_t b = 0; b < 8; ++b) {
            const uint8_t* pl = L.row_lo + u_off + 18 * b;
            const uint8_t* ph = L.row_hi + u_off + 18 * b;
            const uint32_t wl = lds_u32_2(pl + 2 + 4 * L.t), wh = lds_u32_2(ph + 2 + 4 * L.t);
            const float dl = f16_bits_to_f32(lds_u16(pl)), dh = f16_bits_to_f32(lds_u16(ph));
            const uint32_t k0 = kb + 32 * b + 4 * L.t;
            const uint2 x0 = ld_b64(L, k0), x1 = ld_b64(L, k0 + 16);
            const float2 sx = ld_sx(L, (kb >> 5) + b);
            float c[4] = {sx.x, sx.y, sx.x, sx.y};
            const uint32_t ll = wl & 0x0F0F0F0Fu, lh = wh & 0x0F0F0F0Fu;
            mma16816(c, pair01(ll), pair01(lh), pair23(ll), pair23(lh), x0.x, x0.y);
            const uint32_t hl = (wl >> 4) & 0x0F0F0F0Fu, hh = (wh >> 4) & 0x0F0F0F0Fu;
            mma16816(c, pair01(hl), pair01(hh), pair23(hl), pair23(hh), x1.x, x1.y);
            tot[0] = fmaf(dl, c[0], tot[0]);
            tot[1] = fmaf(dl, c[1], tot[1]);
            tot[2] = fmaf(dh, c[2], tot[2]);
            tot[3] = fmaf(dh, c[3], tot[3]);
        }
    }
};

template <> struct Unit<RLXQ_Q8_0> {
    __device__ static __forceinline__ void run(const Lane& L, uint32_t u_off, uint32_t kb, float* scratch,
                                               uint32_t lane, float (&tot)[4]) {
        (void)scratch; (void)lane;
#pragma unroll
        for (uint32_t b = 0; b < 8; ++b) {
            const uint8_t* pl = L.row_lo + u_off + 34 * b;
            const uint8_t* ph = L.row_hi + u_off + 34 * b;
            const float dl = f16_bits_to_f32(lds_u16(pl)), dh = f16_bits_to_f32(lds_u16(ph));
            const float2 sx = ld_sx(L, (kb >> 5) + b);
            float c[4] = {sx.x, sx.y, sx.x, sx.y};
#pragma unroll
            for (uint32_t j = 0; j < 2; ++j) {
                // int8 q -> unsigned q + 128 by flipping the sign bit of every byte
                const uint32_t wl = lds_u32_2(pl + 2 + 16 * j + 4 * L.t) ^ 0x80808080u;
                const uint32_t wh = lds_u32_2(ph + 2 + 16 * j + 4 * L.t) ^ 0x80808080u;
                const uint2 xv = ld_b64(L, kb + 32 * b + 16 * j + 4 * L.t);
                mma16816(c, pair01(wl), pair01(wh), pair23(wl), pair23(wh), xv.x, xv.y);
            }
            tot[0] = fmaf(dl, c[0], tot[0]);
            tot[1] = fmaf(dl, c[1], tot[1]);
            tot[2] = fmaf(dh, c[2], tot[2]);
            tot[3] = fmaf(dh, c[3], tot[3]);
        }
    }
};

template <> struct Unit<RLXQ_Q4_K> {
    // scratch: per warp [16 rows][8 sub-blocks] float2 = (d * sc, dmin * m / 1024)
    __device__ static __forceinline__ void run(const Lane& L, uint32_t u_off, uint32_t kb, float* scratch,
                                               uint32_t lane, float (&tot)[4]) {
        const uint32_t g = lane >> 2;
        __syncwarp();
        {   // lanes 0..15 unpack sub-blocks 0..3 of row (lane & 15), lanes 16..31 sub-blocks 4..7
            const uint32_t r = lane & 15u, half = lane >> 4;
            const uint8_t* base = L.stage + r * StagedTraits<RLXQ_Q4_K>::STRIDE + u_off;
            const uint32_t dd = lds_u32(base);
            const float d = f16_bits_to_f32(dd & 0xFFFFu), dmin = f16_bits_to_f32(dd >> 16);
            const uint32_t w0 = lds_u32(base + 4), w1 = lds_u32(base + 8), w2 = lds_u32(base + 12);
            uint32_t scb, mnb;
            if (half == 0) {
                scb = w0 & 0x3F3F3F3Fu;
                mnb = w1 & 0x3F3F3F3Fu;
            } else {
                scb = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
                mnb = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
            }
            float2* dst = reinterpret_cast<float2*>(scratch) + r * 8 + half * 4;
            const float dm = dmin * (1.0f / 1024.0f);
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
                dst[i] = make_float2(d * (float)((scb >> (8 * i)) & 0xFFu), dm * (float)((mnb >> (8 * i)) & 0xFFu));
        }
        __syncwarp();
        const float2* sc_lo = reinterpret_cast<const float2*>(scratch) + g * 8;
        const float2* sc_hi = sc_lo + 64;
#pragma unroll
        for (uint32_t p = 0; p < 4; ++p) {
            const uint2 ql = *reinterpret_cast<const uint2*>(L.row_lo + u_off + 16 + 32 * p + 8 * L.t);
            const uint2 qh = *reinterpret_cast<const uint2*>(L.row_hi + u_off + 16 + 32 * p + 8 * L.t);
#pragma unroll
            for (uint32_t nib = 0; nib < 2; ++nib) {   // sub-block 2p (low nibbles), 2p+1 (high)
                const uint32_t j = 2 * p + nib;
                const uint4 xv = ld_b128(L, kb + 32 * j + 8 * L.t);
                const float2 sx = ld_sx(L, (kb >> 5) + j);
                float c[4] = {sx.x, sx.y, sx.x, sx.y};
                const uint32_t a_l = (ql.x >> (4 * nib)) & 0x0F0F0F0Fu, a_h = (qh.x >> (4 * nib)) & 0x0F0F0F0Fu;
                mma16816(c, pair01(a_l), pair01(a_h), pair23(a_l), pair23(a_h), xv.x, xv.y);
                const uint32_t b_l = (ql.y >> (4 * nib)) & 0x0F0F0F0Fu, b_h = (qh.y >> (4 * nib)) & 0x0F0F0F0Fu;
                mma16816(c, pair01(b_l), pair01(b_h), pair23(b_l), pair23(b_h), xv.z, xv.w);
                const float2 sl = sc_lo[j], sh = sc_hi[j];
                tot[0] = fmaf(sl.x, c[0], fmaf(sl.y, sx.x, tot[0]));
                tot[1] = fmaf(sl.x, c[1], fmaf(sl.y, sx.y, tot[1]));
                tot[2] = fmaf(sh.x, c[2], fmaf(sh.y, sx.x, tot[2]));
                tot[3] = fmaf(sh.x, c[3], fmaf(sh.y, sx.y, tot[3]));
            }
        }
    }
};

template <> struct Unit<RLXQ_Q6_K> {
    // scratch: per warp [16 rows][16 sub-blocks] float = d * sc
    __device__ static __forceinline__ void run(const Lane& L, uint32_t u_off, uint32_t kb, float* scratch,
                                               uint32_t lane, float (&tot)[4]) {
        const uint32_t g = lane >> 2;
        __syncwarp();
        {
            const uint32_t r = lane & 15u, half = lane >> 4;
            const uint8_t* base = L.stage + r * StagedTraits<RLXQ_Q6_K>::STRIDE + u_off;
            const float d = f16_bits_to_f32(lds_u16(base + 208));
            float* dst = scratch + r * 16 + half * 8;
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                const uint32_t s2 = lds_u16(base + 192 + 8 * half + 2 * i);
                dst[2 * i] = d * (float)(int8_t)(s2 & 0xFFu);
                dst[2 * i + 1] = d * (float)(int8_t)(s2 >> 8);
            }
        }
        __syncwarp();
        const float* sc_lo = scratch + g * 16;
        const float* sc_hi = sc_lo + 128;
        const uint8_t* bl = L.row_lo + u_off;
        const uint8_t* bh = L.row_hi + u_off;
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
#pragma unroll
            for (uint32_t i = 0; i < 2; ++i) {
                const uint32_t qh_l = lds_u32_2(bl + 128 + 32 * h + 16 * i + 4 * L.t);
                const uint32_t qh_h = lds_u32_2(bh + 128 + 32 * h + 16 * i + 4 * L.t);
#pragma unroll
                for (uint32_t ps = 0; ps < 2; ++ps) {
                    const uint32_t ql_l = lds_u32_2(bl + 64 * h + 32 * ps + 16 * i + 4 * L.t);
                    const uint32_t ql_h = lds_u32_2(bh + 64 * h + 32 * ps + 16 * i + 4 * L.t);
#pragma unroll
                    for (uint32_t nib = 0; nib < 2; ++nib) {
                        const uint32_t g4 = ps + 2 * nib;  // which 32-element group of the half
                        // bits 2*g4, 2*g4+1 of every qh byte moved to bits 4, 5
                        const uint32_t h_l = (g4 < 2 ? (qh_l << (4 - 2 * g4)) : (qh_l >> (2 * g4 - 4))) & 0x30303030u;
                        const uint32_t h_h = (g4 < 2 ? (qh_h << (4 - 2 * g4)) : (qh_h >> (2 * g4 - 4))) & 0x30303030u;
                        const uint32_t a_l = ((ql_l >> (4 * nib)) & 0x0F0F0F0Fu) | h_l;
                        const uint32_t a_h = ((ql_h >> (4 * nib)) & 0x0F0F0F0Fu) | h_h;
                        const uint32_t ke = kb + 128 * h + 32 * g4 + 16 * i;  // first k of this 16-block
                        const uint2 xv = ld_b64(L, ke + 4 * L.t);
                        const float2 sx = ld_sx(L, ke >> 4);
                        float c[4] = {sx.x, sx.y, sx.x, sx.y};
                        mma16816(c, pair01(a_l), pair01(a_h), pair23(a_l), pair23(a_h), xv.x, xv.y);
                        const uint32_t si = 8 * h + 2 * g4 + i;
                        const float sl = sc_lo[si], sh = sc_hi[si];
                        tot[0] = fmaf(sl, c[0], tot[0]);
                        tot[1] = fmaf(sl, c[1], tot[1]);
                        tot[2] = fmaf(sh, c[2], tot[2]);
                        tot[3] = fmaf(sh, c[3], tot[3]);
                    }
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Activation slice -> fp16 in shared memory, with per-block sums.
// ---------------------------------------------------------------------------------------------
// One CTA per activation row (plus one for the zero column when m is odd).  Two passes over the
// row: its maximum, then the exact power-of-two rescale, the fp16 conversion and the sums per
// SUB-weight block.  Also clears the split-k tile counters of the main kernel.
template <uint32_t SUB>
__global__ void __launch_bounds__(1024) convert_x_f16_kernel(const void* __restrict__ x, uint32_t x_bf16, uint32_t m,
                                                             uint32_t mp, uint32_t k, float bias, __half* __restrict__ xh,
                                                             float* __restrict__ sxb, float* __restrict__ inv,
                                                             uint32_t* __restrict__ counters, uint32_t ncounters) {
    griddep_launch_dependents();
    griddep_wait();
    __shared__ uint32_t rowmax;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid & 31u;
    if (r == 0) for (uint32_t i = tid; i < ncounters; i += blockDim.x) counters[i] = 0u;
    const uint32_t groups = k / 8;
    if (r >= m) {   // padding column of the block sums
        for (uint32_t b = tid; b < k / SUB; b += blockDim.x) sxb[(size_t)b * mp + r] = 0.f;
        return;
    }
    if (tid == 0) rowmax = 0u;
    __syncthreads();
    auto load8 = [&](uint32_t g, float (&f)[8]) {
        if (x_bf16) {
            const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (size_t)r * k + 8 * g);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) { f[2 * q] = __uint_as_float(w[q] << 16); f[2 * q + 1] = __uint_as_float(w[q] & 0xFFFF0000u); }
        } else {
            const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)r * k + 8 * g);
            const float4 a = p[0], b = p[1];
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
        }
    };
    uint32_t mx = 0;
    for (uint32_t g = tid; g < groups; g += blockDim.x) {
        float f[8];
        load8(g, f);
#pragma unroll
        for (int q = 0; q < 8; ++q) mx = max(mx, __float_as_uint(f[q]) & 0x7FFFFFFFu);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0 && mx) atomicMax(&rowmax, mx);
    __syncthreads();
    // exact power-of-two rescale so that the row maximum lands in [2^14, 2^15)
    const uint32_t e = rowmax >> 23;
    uint32_t sf = 127u;                       // scale = 1 for an all-zero or non-finite row
    if (e != 0u && e != 255u) sf = min(253u, max(1u, 268u - e));
    const float sc = __uint_as_float(sf << 23);
    if (tid == 0) inv[r] = __uint_as_float((254u - sf) << 23);
    if (r == 0 && tid >= m && tid < 8) inv[tid] = 1.0f;
    // groups is a multiple of 32, so whole warps stay together and the lanes of one block are adjacent
    for (uint32_t g = tid; g < groups; g += blockDim.x) {
        float f[8];
        load8(g, f);
        __half2 h[4];
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            h[q] = __floats2half2_rn(f[2 * q] * sc, f[2 * q + 1] * sc);
            const float2 back = __half22float2(h[q]);
            sum += back.x + back.y;
        }
        uint4 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&h[0]); pk.y = *reinterpret_cast<uint32_t*>(&h[1]);
        pk.z = *reinterpret_cast<uint32_t*>(&h[2]); pk.w = *reinterpret_cast<uint32_t*>(&h[3]);
        *reinterpret_cast<uint4*>(xh + (size_t)r * k + 8 * g) = pk;
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        if (SUB == 32) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if ((lane & (SUB / 8 - 1)) == 0) sxb[(size_t)(8 * g / SUB) * mp + r] = bias * sum;
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
struct StagedArgs { CUtensorMap wmap; StagedParams p; };

template <uint32_t SCHEME>
__global__ void __launch_bounds__(kThreads) gemv_staged_kernel(const __grid_constant__ StagedArgs A) {
    const StagedParams& P = A.p;
    using T = StagedTraits<SCHEME>;
    extern __shared__ __align__(128) uint8_t smem[];
    __half* xs = reinterpret_cast<__half*>(smem);
    float* sxb = reinterpret_cast<float*>(smem + P.off_sxb);
    uint8_t* stages = smem + P.off_stage;
    float* scratch_all = reinterpret_cast<float*>(smem + P.off_scratch);
    float* red = reinterpret_cast<float*>(smem + P.off_red);      // [2][4 warps][16][8]
    const uint32_t NS = P.nstages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P.off_bar);  // full[NS], empty[NS], xbar
    uint32_t* misc = reinterpret_cast<uint32_t*>(bars + 2 * NS + 1);
    volatile uint32_t* abort_flag = misc;
    volatile uint32_t* last_flag = misc + 1;
    griddep_launch_dependents();

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t ks = blockIdx.x % P.ksl, rgi = blockIdx.x / P.ksl;
    const uint32_t ku = P.k / 256;
    const uint32_t u0 = ks * P.usl;
    const uint32_t units = min(P.usl, ku - u0);          // 256-weight units in this CTA's slice
    const uint32_t nchunks = (units + T::CU - 1) / T::CU;
    const uint32_t stage_bytes = 16 * T::STRIDE;

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[NS + s]), kConsumerWarps);
        }
        mbar_init(smem_u32(&bars[2 * NS]), 1);
        *abort_flag = 0u;
        *last_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Everyone converts the activation slice once; weights for the first stages are requested
    // first so the copies overlap the conversion.
    uint32_t prod_it = 0;
    const uint32_t my_tiles = (P.ntiles > rgi) ? (P.ntiles - rgi + P.rg - 1) / P.rg : 0u;
    const uint32_t total_it = my_tiles * nchunks;
    auto produce = [&](uint32_t it) {
        // one 2-D TMA box per stage: 16 rows x (CU units + pad); rows past n and bytes past the row
        // end arrive as zeros (scale 0: they add nothing)
        const uint32_t tile = rgi + (it / nchunks) * P.rg, chunk = it % nchunks;
        const uint32_t s = it % NS;
        const uint32_t full = smem_u32(&bars[s]);
        if (lane == 0) {
            mbar_arrive_expect_tx(full, stage_bytes);
            tma_load_2d(smem_u32(stages + s * stage_bytes), &A.wmap, (int32_t)(((u0 + chunk * T::CU) * T::UNIT_B) / 8),
                        (int32_t)(tile * 16), full);
        }
    };
    if (warp == kConsumerWarps) {
        // weights never change: fill the ring before waiting for the previous kernel
        if (lane == 0) tma_prefetch_desc(&A.wmap);
        for (; prod_it < total_it && prod_it < NS; ++prod_it) produce(prod_it);
        griddep_wait();
        // this CTA's slice of the converted activations and of their block sums, by bulk copy
        const uint32_t klen = units * 256, nblk = klen / T::SUB;
        const uint32_t xbar = smem_u32(&bars[2 * NS]);
        if (lane == 0) mbar_arrive_expect_tx(xbar, P.m * klen * 2 + nblk * P.mp * 4);
        __syncwarp();
        if (lane < P.m)
            bulk_g2s(smem_u32(xs + (size_t)lane * P.xs_stride), P.xh_ws + (size_t)lane * P.k + (size_t)u0 * 256, klen * 2, xbar);
        if (lane == 31)
            bulk_g2s(smem_u32(sxb), P.sxb_ws + (size_t)(u0 * 256 / T::SUB) * P.mp, nblk * P.mp * 4, xbar);
    }

    if (warp == kConsumerWarps) {
        // ---------------- producer warp ----------------
        bool dead = false;
        for (; prod_it < total_it; ++prod_it) {
            const uint32_t s = prod_it % NS;
            const uint32_t ph = ((prod_it / NS) & 1u) ^ 1u;
            if (!dead && (*abort_flag || !mbar_wait(smem_u32(&bars[NS + s]), ph))) {
                dead = true;
                if (lane == 0) { atomicExch(P.err, 1); *abort_flag = 1u; }
            }
            if (dead) break;
            produce(prod_it);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const uint32_t g = lane >> 2, t = lane & 3u;
    Lane L;
    L.t = t;
    L.mp = P.mp;
    L.xrow = xs + (size_t)(g < P.m ? g : 0u) * P.xs_stride;
    L.sxb = sxb;
    float* scratch = scratch_all + warp * 512;  // 2 KB per warp
    bool dead = false;
    griddep_wait();
    if (!mbar_wait(smem_u32(&bars[2 * NS]), 0)) {
        dead = true;
        if (lane == 0) { atomicExch(P.err, 8); *abort_flag = 1u; }
    }
    uint32_t it = 0;
    for (uint32_t ti = 0; ti < my_tiles; ++ti) {
        const uint32_t tile = rgi + ti * P.rg;
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t chunk = 0; chunk < nchunks; ++chunk, ++it) {
            const uint32_t s = it % NS, ph = (it / NS) & 1u;
            if (!dead && (*abort_flag || !mbar_wait(smem_u32(&bars[s]), ph))) {
                dead = true;
                if (lane == 0) { atomicExch(P.err, 2); *abort_flag = 1u; }
            }
            if (dead) continue;
            const uint32_t cu = min(T::CU, units - chunk * T::CU);
            L.stage = stages + s * stage_bytes;
            L.row_lo = L.stage + g * T::STRIDE;
            L.row_hi = L.row_lo + 8 * T::STRIDE;
            for (uint32_t u = warp; u < cu; u += kConsumerWarps)
                Unit<SCHEME>::run(L, u * T::UNIT_B, (chunk * T::CU + u) * 256, scratch, lane, tot);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[NS + s]));
        }
        // cross-warp reduction, fixed order
        float* rbuf = red + (ti & 1u) * (kConsumerWarps * 128);
        {
            float* mine = rbuf + warp * 128;
            mine[g * 8 + 2 * t] = tot[0];
            mine[g * 8 + 2 * t + 1] = tot[1];
            mine[(g + 8) * 8 + 2 * t] = tot[2];
            mine[(g + 8) * 8 + 2 * t + 1] = tot[3];
        }
        consumer_bar();
        const uint32_t col = tid >> 4, rrow = tid & 15u;   // tid < 128
        const uint32_t orow = tile * 16 + rrow;
        float v = 0.f;
#pragma unroll
        for (uint32_t wv = 0; wv < kConsumerWarps; ++wv) v += rbuf[wv * 128 + rrow * 8 + col];
        const bool live = col < P.m && orow < P.n;
        v *= __ldg(P.inv_ws + col);
        if (P.ksl == 1) {
            if (live) {
                const size_t o = (size_t)col * P.n + orow;
                if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(v);
                else reinterpret_cast<float*>(P.y)[o] = v;
            }
        } else {
            // split-k: publish the partial, the last CTA to arrive for this tile reduces
            if (live) P.partial[((size_t)ks * P.m + col) * P.n + orow] = v;
            __threadfence();
            consumer_bar();
            if (tid == 0) {
                const uint32_t prev = atomicAdd(&P.counters[tile], 1u);
                *last_flag = (prev == P.ksl - 1) ? 1u : 0u;
            }
            consumer_bar();
            if (*last_flag) {
                __threadfence();
                if (live) {
                    float acc = 0.f;
                    for (uint32_t s2 = 0; s2 < P.ksl; ++s2)
                        acc += __ldcg(&P.partial[((size_t)s2 * P.m + col) * P.n + orow]);
                    const size_t o = (size_t)col * P.n + orow;
                    if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(acc);
                    else reinterpret_cast<float*>(P.y)[o] = acc;
                }
                if (tid == 0) P.counters[tile] = 0u;
            }
            consumer_bar();   // last_flag is rewritten by the next tile
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host side: shape support, tiling plan, launch
// ---------------------------------------------------------------------------------------------
struct StagedPlan {
    bool ok;
    uint32_t ksl, usl, rg, ntiles, xs_stride, mp, nstages;
    uint32_t off_sxb, off_stage, off_scratch, off_red, off_bar, smem_bytes;
    size_t ws_partial_bytes, ws_counter_bytes, ws_xh_bytes, ws_sxb_bytes, ws_bytes;
};

template <uint32_t SCHEME>
static StagedPlan plan_staged(uint32_t m, uint32_t k, uint32_t n, int64_t force_ksl) {
    using T = StagedTraits<SCHEME>;
    StagedPlan pl{};
    pl.ok = false;
    if (m == 0 || m > 8 || n == 0 || k == 0 || k % (256 * T::AG)) return pl;
    const uint32_t ku = k / 256;
    const uint32_t sms = (uint32_t)sm_count();
    pl.ntiles = (n + 15) / 16;
    pl.mp = (m + 1) & ~1u;
    // padding between activation rows: 64-bit fragment reads want a stride of 32 bytes mod 128,
    // 128-bit reads (Q4_K) 64 bytes mod 128
    const uint32_t pad_halfs = (SCHEME == RLXQ_Q4_K) ? 32u : 16u;
    auto usl_for = [&](uint32_t ksl) {
        uint32_t usl = (ku + ksl - 1) / ksl;
        usl = (usl + T::AG - 1) / T::AG * T::AG;
        return usl;
    };
    auto xs_bytes_for = [&](uint32_t usl) { return (size_t)m * (usl * 256 + pad_halfs) * 2; };
    uint32_t ksl = 1;
    if (force_ksl > 0) {
        ksl = (uint32_t)force_ksl;
    } else {
        while (xs_bytes_for(usl_for(ksl)) > 64 * 1024 && ksl < ku) ++ksl;
        // fill the machine when there are few row tiles, but keep slices at least two chunks long
        while (pl.ntiles * ksl < 2 * sms && usl_for(ksl * 2) >= 2 * T::CU && ksl < 8) ksl *= 2;
    }
    if (ksl > ku) ksl = ku;
    pl.usl = usl_for(ksl);
    pl.ksl = (ku + pl.usl - 1) / pl.usl;
    if (xs_bytes_for(pl.usl) > 96 * 1024) return pl;
    pl.xs_stride = pl.usl * 256 + pad_halfs;
    uint32_t off = (uint32_t)xs_bytes_for(pl.usl);
    auto align = [](uint32_t v, uint32_t a) { return (v + a - 1) / a * a; };
    off = align(off, 128);
    pl.off_sxb = off;
    off += (pl.usl * 256 / T::SUB) * pl.mp * 4;
    off = align(off, 128);
    pl.off_stage = off;
    // the ring takes what is left of half an SM's shared memory (two CTAs per SM) when that gives
    // at least three stages, else of a whole one
    const uint32_t stage_bytes = 16 * T::STRIDE;
    const uint32_t tail = kConsumerWarps * 2048 + 2 * kConsumerWarps * 128 * 4 + 1024;
    uint32_t budget = 112u * 1024u;
    if (off + tail + 3 * stage_bytes > budget) budget = 224u * 1024u;
    if (off + tail + 2 * stage_bytes > budget) return pl;
    pl.nstages = (budget - off - tail) / stage_bytes;
    if (pl.nstages > 16) pl.nstages = 16;
    off += pl.nstages * stage_bytes;
    off = align(off, 128);
    pl.off_scratch = off;
    off += kConsumerWarps * 2048;
    pl.off_red = off;
    off += 2 * kConsumerWarps * 128 * 4;
    pl.off_bar = off;
    off += (2 * pl.nstages + 1) * 8 + 64;
    pl.smem_bytes = off;
    if (pl.smem_bytes > 226 * 1024) return pl;
    uint32_t occ = (226u * 1024u) / (pl.smem_bytes + 1024u);
    if (occ > 4) occ = 4;
    if (occ < 1) occ = 1;
    uint32_t rg = (sms * occ) / pl.ksl;
    if (rg < 1) rg = 1;
    if (rg > pl.ntiles) rg = pl.ntiles;
    pl.rg = rg;
    auto al = [](size_t v) { return (v + 255) / 256 * 256; };
    pl.ws_partial_bytes = pl.ksl > 1 ? al((size_t)pl.ksl * m * n * 4) : 0;
    pl.ws_counter_bytes = al((size_t)pl.ntiles * 4);
    pl.ws_xh_bytes = al((size_t)m * k * 2);
    pl.ws_sxb_bytes = al((size_t)(k / T::SUB) * pl.mp * 4);
    pl.ws_bytes = pl.ws_partial_bytes + pl.ws_counter_bytes + pl.ws_xh_bytes + pl.ws_sxb_bytes + 256;
    pl.ok = true;
    return pl;
}

template <uint32_t SCHEME>
static int launch_staged_t(cudaStream_t stream, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf,
                           uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes,
                           const StagedPlan& pl) {
    using T = StagedTraits<SCHEME>;
    Geometry g;
    geometry(SCHEME, &g);
    StagedParams P{};
    P.x = x; P.w = w; P.y = y;
    P.m = m; P.k = k; P.n = n;
    P.x_bf16 = xbf; P.y_bf16 = ybf;
    P.row_bytes = k / g.elems * g.bytes;
    P.ntiles = pl.ntiles; P.rg = pl.rg; P.ksl = pl.ksl; P.usl = pl.usl;
    P.xs_stride = pl.xs_stride; P.mp = pl.mp;
    P.off_sxb = pl.off_sxb; P.off_stage = pl.off_stage; P.off_scratch = pl.off_scratch;
    P.off_red = pl.off_red; P.off_bar = pl.off_bar;
    P.nstages = pl.nstages;
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(RLXQ_E_WORKSPACE, "tensor-mode GEMV needs %zu workspace bytes, got %zu", pl.ws_bytes, ws_bytes);
    if ((uintptr_t)ws & 15u) return fail(RLXQ_E_ALIGN, "workspace must be 16-byte aligned");
    uint8_t* wsb = reinterpret_cast<uint8_t*>(ws);
    P.partial = reinterpret_cast<float*>(wsb);
    P.counters = reinterpret_cast<uint32_t*>(wsb + pl.ws_partial_bytes);
    __half* xh = reinterpret_cast<__half*>(wsb + pl.ws_partial_bytes + pl.ws_counter_bytes);
    float* sxb = reinterpret_cast<float*>(wsb + pl.ws_partial_bytes + pl.ws_counter_bytes + pl.ws_xh_bytes);
    float* inv = reinterpret_cast<float*>(wsb + pl.ws_partial_bytes + pl.ws_counter_bytes + pl.ws_xh_bytes + pl.ws_sxb_bytes);
    P.xh_ws = xh; P.sxb_ws = sxb; P.inv_ws = inv;
    StagedArgs A{};
    A.p = P;
    int rc = encode_weight_map(&A.wmap, w, n, P.row_bytes, T::STRIDE / 8, 16);
    if (rc) return rc;
    static std::atomic<uint32_t> attr_set[64];
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemv_staged_kernel<SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev].store(1);
    }
    rc = launch_pdl(convert_x_f16_kernel<T::SUB>, dim3(pl.mp), dim3(1024), 0, stream, x, (uint32_t)xbf, m, pl.mp, k,
                    (float)T::BIAS, xh, sxb, inv, P.counters, pl.ksl > 1 ? pl.ntiles : 0u);
    if (rc) return rc;
    count_launch();
    rc = launch_pdl(gemv_staged_kernel<SCHEME>, dim3(pl.rg * pl.ksl), dim3(kThreads), pl.smem_bytes, stream, A);
    if (rc) return rc;
    count_launch();
    return check_launch("gemv_staged_kernel");
}

static std::atomic<int*> g_error_words[64];

int* device_error_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* p = g_error_words[dev].load();
    if (!p) {
        int* fresh = nullptr;
        if (cudaMalloc(&fresh, sizeof(int)) != cudaSuccess) return nullptr;
        if (cudaMemset(fresh, 0, sizeof(int)) != cudaSuccess) return nullptr;
        int* expected = nullptr;
        if (g_error_words[dev].compare_exchange_strong(expected, fresh)) p = fresh;
        else { cudaFree(fresh); p = expected; }
    }
    return p;
}

// The word if this device already has one, else null; never allocates.
int* device_error_word_if_ready() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return g_error_words[dev].load();
}

// Reads (and clears) the error words kernels on this device may have written: the allocated one, and the
// one inside the library image that rlxq_matmul_static_scratch uses while the device has no allocated
// word.  A process that has only ever made allocation-free calls has just the second, and this function
// then allocates nothing either; with neither present nothing can have been recorded, and the regular
// word is created so that later launches have one.
int staged_device_error(int* value) {
    int* p = device_error_word_if_ready();
    int* sp = static_error_word_if_resolved();
    if (!p && !sp) {
        p = device_error_word();
        if (!p) return fail(RLXQ_E_CUDA, "device error word unavailable");
    }
    RLXQ_CUDA_TRY(cudaDeviceSynchronize());
    *value = 0;
    int* words[2] = {p, sp};
    for (int* w : words) {
        if (!w) continue;
        int v = 0;
        RLXQ_CUDA_TRY(cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost));
        if (v) {
            RLXQ_CUDA_TRY(cudaMemset(w, 0, sizeof(int)));
            if (!*value) *value = v;
        }
    }
    return RLXQ_OK;
}

int staged_prepare_device() { return device_error_word() ? RLXQ_OK : fail(RLXQ_E_CUDA, "device error word unavailable"); }

bool staged_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x,
                      bool xbf) {
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    (void)xbf;
    const int64_t f = options().gemv_kslices.load();
    switch (scheme) {
        case RLXQ_Q4_0: return plan_staged<RLXQ_Q4_0>(m, k, n, f).ok;
        case RLXQ_Q8_0: return plan_staged<RLXQ_Q8_0>(m, k, n, f).ok;
        case RLXQ_Q4_K: return plan_staged<RLXQ_Q4_K>(m, k, n, f).ok;
        case RLXQ_Q6_K: return plan_staged<RLXQ_Q6_K>(m, k, n, f).ok;
        default: return false;
    }
}

size_t staged_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n) {
    const int64_t f = options().gemv_kslices.load();
    StagedPlan pl{};
    switch (scheme) {
        case RLXQ_Q4_0: pl = plan_staged<RLXQ_Q4_0>(m, k, n, f); break;
        case RLXQ_Q8_0: pl = plan_staged<RLXQ_Q8_0>(m, k, n, f); break;
        case RLXQ_Q4_K: pl = plan_staged<RLXQ_Q4_K>(m, k, n, f); break;
        case RLXQ_Q6_K: pl = plan_staged<RLXQ_Q6_K>(m, k, n, f); break;
        default: break;
    }
    return pl.ok ? pl.ws_bytes : 0;
}

int launch_gemv_staged(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w,
                       void* y, bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    const int64_t f = options().gemv_kslices.load();
    switch (scheme) {
        case RLXQ_Q4_0: return launch_staged_t<RLXQ_Q4_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, plan_staged<RLXQ_Q4_0>(m, k, n, f));
        case RLXQ_Q8_0: return launch_staged_t<RLXQ_Q8_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, plan_staged<RLXQ_Q8_0>(m, k, n, f));
        case RLXQ_Q4_K: return launch_staged_t<RLXQ_Q4_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, plan_staged<RLXQ_Q4_K>(m, k, n, f));
        case RLXQ_Q6_K: return launch_staged_t<RLXQ_Q6_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, plan_staged<RLXQ_Q6_K>(m, k, n, f));
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
}

}  // namespace rlxq
