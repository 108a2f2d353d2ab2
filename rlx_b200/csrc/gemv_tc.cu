// Streaming decode GEMV for batch 1-8 on the 5th-generation tensor cores.
//
// y[m,n] = x[m,k] . W^T with m <= 8 is computed transposed, 128 weight rows at a time:
// D[128 weight rows, 16] += A[128, 16 k] . B[16, 16 k]^T, tcgen05.mma with M = 128, N = 16, K = 16.
//   * A (weights) never exists in memory.  The raw GGUF blocks of 128 rows x 256 weights arrive in
//     shared memory through one 2-D TMA box; eight decode warps (one thread per weight row, which is also
//     that thread's tensor-memory lane) turn them into fp16 values of d * q, about two instructions per
//     weight on packed fp16 pairs, and store them to tensor memory (tcgen05.st).  The integer part of a
//     weight is exact in fp16 and d is an fp16 number, so a weight is rounded once, to 11 significant bits.
//   * B (activations) holds the m rows twice, as fp16 like the weights (the MMA takes one 16-bit format for both
//     operands): rows 0..7 are h = fp16(x), rows 8..15 are fp16((x - h) * 2^11), so an f32 activation keeps 22
//     significant bits; the two halves of an output meet in the epilogue, the second scaled by 2^-11.
//     Activations are clamped to the fp16 range (+-65504) and lose precision below about 1e-7 in magnitude;
//     the reference's f32 path has no such limits.  The B operand of the CTA's first units is built straight
//     from global memory by five warps as soon as the kernel in front has finished (that latency is on the
//     critical path of a decode step); for long ranges the rest comes through a staging ring filled by bulk copies.
//     The order of the k values inside a 64-wide group follows the order the decoders produce (low nibbles and
//     high nibbles of a word side by side), which costs nothing on the B side and saves byte shuffles on the A side.
//   * Issuing one tcgen05.mma occupies its thread for about 115 cycles whatever the tile's width (measured: 114.7
//     cycles per instruction from one thread for N = 16 .. 128, 28.7 aggregate from four warps; two lanes of one warp
//     issuing together take 155).  A 128 x 16 x 16 MMA covers 2048 weights, so one issuing thread feeds 18 weights per
//     clock where a 4-bit format needs 41 per SM at HBM speed.  Here four streams issue, two lanes in each of two
//     warps: stream q takes k block q of every unit into its own accumulator (fp16 x fp16 into f32).  tcgen05.commit
//     releases stages, B slabs and accumulators through mbarriers.  Four epilogue warps read the accumulators
//     (tcgen05.ld) and add the four streams in order.
// Status: correct for batch 1-8 (Q4_0, Q8_0, Q4_K) and selectable with the option gemv_kernel = 4, but not the
// default: with three tensor-memory stages per decode group the decode -> MMA -> free loop is a latency chain, and
// the kernel is slower than the integer kernel (batch 1-2) and the mma.sync kernel (batch 3-8) on every shape measured.
// The work list is (row tile, 256-wide k group) units, tile-major, dealt to the CTAs as equal contiguous
// ranges so every SM streams the same bytes whatever n and k are.  A tile cut by range boundaries is
// completed by its first contributor, the CTA whose range ends inside the tile: that tile is the last
// thing it works on, while for every other contributor it is the first.  The others publish each value
// as one 8-byte word (f32 value, call token), a single store that is valid by itself; the first contributor
// reads the words (polling, bounded, a word whose token is not there yet), adds them to its own values in
// contributor order, writes y and clears the words for a replay of the same captured launch.  The grid
// never exceeds the number of CTAs the device holds at once, so every contributor is running or about to.
// Two CTAs per SM; all weights are requested before the dependency wait (programmatic dependent launch),
// only the activations wait for the kernel in front.
//
// Every wait is bounded: on a timeout the kernel records an error word, stops issuing, lets the copies in
// flight land, frees its tensor memory and returns.
//
// Replaces, for m <= 8, the reference's dequantise-everything + cublasSgemm (rlx-cuda/src/gguf_gpu.rs:62-134);
// semantics of the product: rlx-cpu/src/gguf_matmul.rs:40-95.
#include <chrono>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "staged_common.cuh"
#include "tc_common.cuh"
#include "tensormap.cuh"

namespace rlxq {

constexpr uint32_t kTcTileW = 128;          // weight rows per tile (MMA M, tensor-memory lanes)
constexpr uint32_t kTcN = 16;               // MMA N: 8 activation rows x (high part, low part)
constexpr uint32_t kTcGroups = 2;           // decode warp groups (four warps each), one MMA issuer per group
constexpr uint32_t kTcGroupStages = 3;      // 64-wide k blocks of decoded weights in tensor memory per group (32 columns each)
constexpr uint32_t kTcAStages = kTcGroups * kTcGroupStages;
constexpr uint32_t kTcCols = 256;           // tensor-memory columns per CTA: 2 x 2 accumulators of 16 + 6 x 32 weights
constexpr uint32_t kTcThreads = (4 + 4 * kTcGroups + 4) * 32;
constexpr uint32_t kTcBSlab = 8192;         // B operand of one unit: 4 k blocks x 16 rows x 128 bytes
constexpr uint32_t kTcMaxRing = 8;
constexpr uint32_t kTcMaxB = 6;             // B slabs: the whole range of a CTA when it is that short
constexpr uint32_t kTcBThreads = 160;       // warp 3 and the four epilogue warps build the first B slabs together
constexpr uint32_t kTcSmemBudget = 113u * 1024u;   // two CTAs per SM
constexpr uint32_t kTcPollLimit = 1u << 22;          // polls (200 ns apart) of a word another CTA of the grid has yet to publish

// warp roles: 0 = raw weight TMA producer, 1-2 = MMA issuers (one per decode group), 3 = activations (B operand),
// 4-11 = decode (lane quarter = warp % 4, group = (warp - 4) / 4), 12-15 = epilogue (they first help warp 3).

// Instruction descriptor: f32 accumulator, fp16 A and B, both K-major, M = 128, N = 16.
constexpr uint32_t kTcIdesc = (1u << 4) | (0u << 7) | (0u << 10) | ((kTcN >> 3) << 17) | ((kTcTileW >> 4) << 24);

// Raw bytes of 256 weights of one row inside a TMA box (an odd number of 16-byte chunks, so one-row-per-lane
// 128-bit reads do not conflict).
template <uint32_t SCHEME> struct TcRaw;
template <> struct TcRaw<RLXQ_Q4_0> { static constexpr uint32_t ROW = 144; };
template <> struct TcRaw<RLXQ_Q8_0> { static constexpr uint32_t ROW = 272; };
template <> struct TcRaw<RLXQ_Q4_K> { static constexpr uint32_t ROW = 144; };

struct TcParams {
    CUtensorMap wmap;      // W[n, row_bytes / 8] eight-byte elements, box 128 rows x one 256-weight group
    const void* x;
    void* y;
    int* err;
    unsigned long long* parts;    // [2 * grid][m][128] words (value, token) of cut tiles: slot 2c = head of CTA c's range, 2c + 1 = tail
    uint32_t token;               // odd, different for every call
    uint32_t m, n, k, x_bf16, y_bf16;
    uint32_t ntiles, kgroups, units_q, units_r;
    uint32_t nraw, nb, nxs;                   // ring depths: raw boxes, B slabs, activation staging (0: no range is longer than nb)
    uint32_t off_xs, off_raw, off_bar;        // shared-memory offsets from the 1024-byte aligned base
    uint32_t xs_row_bytes, xs_stage_bytes;    // staging: 256 activations of one row / of all m rows
};

struct TcBars {
    uint64_t raw_full[kTcMaxRing], raw_empty[kTcMaxRing];
    uint64_t a_full[kTcAStages], a_free[kTcAStages];
    uint64_t b_full[kTcMaxB], b_free[kTcMaxB], xs_full[4], xs_free[4];
    uint64_t d_full[2], d_free[2];
    uint32_t tmem_base, abort_flag;
};

struct TcSeg { uint32_t tile, g0, g1; };     // k groups [g0, g1) of one row tile


__device__ __forceinline__ uint32_t tc_range_start(const TcParams& P, uint32_t c) { return c * P.units_q + min(c, P.units_r); }
__device__ __forceinline__ uint32_t tc_owner(const TcParams& P, uint32_t u) {
    const uint32_t big = P.units_r * (P.units_q + 1);
    return u < big ? u / (P.units_q + 1) : P.units_r + (u - big) / P.units_q;
}
__device__ __forceinline__ bool tc_seg_next(const TcParams& P, uint32_t& cur, uint32_t lim, TcSeg& sg) {
    if (cur >= lim) return false;
    sg.tile = cur / P.kgroups;
    sg.g0 = cur - sg.tile * P.kgroups;
    sg.g1 = min(P.kgroups, sg.g0 + (lim - cur));
    cur += sg.g1 - sg.g0;
    return true;
}

// ---- packed fp16 arithmetic on 32-bit registers -------------------------------------------------
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) { uint32_t d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
// (f, f) as an fp16 pair, round to nearest even
__device__ __forceinline__ uint32_t h2splat(float f) { uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %1;" : "=r"(d) : "f"(f)); return d; }
constexpr uint32_t kMagic = 0x64646464u;    // 0x64xx as fp16 is 1024 + xx for xx < 256
// bytes 0,1 / 2,3 of u -> the fp16 pair (1024 + byte, 1024 + byte)
__device__ __forceinline__ uint32_t magic01(uint32_t u) { return __byte_perm(u, kMagic, 0x5140); }
__device__ __forceinline__ uint32_t magic23(uint32_t u) { return __byte_perm(u, kMagic, 0x5342); }

// 32-bit words of a row buffer at compile-time byte offsets (multiples of 4): loads the 16-byte chunks that
// cover [B0, B0 + LEN).
template <int B0, int LEN> struct TcWords {
    static_assert(B0 % 4 == 0, "word aligned");
    static constexpr int C0 = B0 / 16, C1 = (B0 + LEN + 15) / 16;
    uint32_t w[4 * (C1 - C0)];
    __device__ __forceinline__ void load(const uint8_t* row) {
#pragma unroll
        for (int c = C0; c < C1; ++c) {
            const uint4 t = *reinterpret_cast<const uint4*>(row + 16 * c);
            w[4 * (c - C0)] = t.x; w[4 * (c - C0) + 1] = t.y; w[4 * (c - C0) + 2] = t.z; w[4 * (c - C0) + 3] = t.w;
        }
    }
    // word i counted from byte B0
    __device__ __forceinline__ uint32_t at(int i) const { return w[(B0 - 16 * C0) / 4 + i]; }
};

// ---- decoders: 32 weights (half H of the 64-wide k block S of a 256-weight group) -> 16 fp16 pairs --------
// The pairs are in the order of the B operand's k slots: see tc_xoff.
template <uint32_t SCHEME, int S> struct TcStage;

// Q4_0 (rlx-gguf/src/lib.rs:584-597): block = fp16 d | 16 bytes; weight j = low nibble of byte j, weight 16 + j = high
// nibble, value d * (q - 8).  Half H is block 2S + H at byte 36 S + 18 H of the row buffer.  Slot order of a block:
// for i = 0..3: weights 4i..4i+3, then 16+4i..16+4i+3.
template <int S> struct TcStage<RLXQ_Q4_0, S> {
    __device__ __forceinline__ void prep(const uint8_t*) {}
    template <int H> __device__ __forceinline__ void half(const uint8_t* row, uint32_t (&v)[16]) const {
        constexpr int B0 = 36 * S + 18 * H, A0 = B0 & ~3;
        TcWords<A0, 20> ws;
        ws.load(row);
        uint32_t lo[5], hi[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) { lo[j] = ws.at(j) & 0x0F0F0F0Fu; hi[j] = (ws.at(j) >> 4) & 0x0F0F0F0Fu; }
        // an even block starts on a word: d, then the quants from byte 2; an odd one has d in the upper half of word 0
        const uint32_t d2 = __byte_perm(ws.at(0), 0u, H == 0 ? 0x1010 : 0x3232);
        const uint32_t off = 0x64086408u;   // 1032 = 1024 + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t a, b, c, e;
            if (H == 0) { a = magic23(lo[i]); b = magic01(lo[i + 1]); c = magic23(hi[i]); e = magic01(hi[i + 1]); }
            else { a = magic01(lo[i + 1]); b = magic23(lo[i + 1]); c = magic01(hi[i + 1]); e = magic23(hi[i + 1]); }
            v[4 * i] = h2mul(h2sub(a, off), d2);
            v[4 * i + 1] = h2mul(h2sub(b, off), d2);
            v[4 * i + 2] = h2mul(h2sub(c, off), d2);
            v[4 * i + 3] = h2mul(h2sub(e, off), d2);
        }
    }
};

// Q8_0 (rlx-gguf/src/lib.rs:574-581): block = fp16 d | 32 int8, value d * q.  Half H is block 2S + H at byte
// 68 S + 34 H.  Natural slot order.
template <int S> struct TcStage<RLXQ_Q8_0, S> {
    __device__ __forceinline__ void prep(const uint8_t*) {}
    template <int H> __device__ __forceinline__ void half(const uint8_t* row, uint32_t (&v)[16]) const {
        constexpr int B0 = 68 * S + 34 * H, A0 = B0 & ~3;
        TcWords<A0, 36> ws;
        ws.load(row);
        const uint32_t d2 = __byte_perm(ws.at(0), 0u, H == 0 ? 0x1010 : 0x3232);
        const uint32_t off = 0x64806480u;   // 1152 = 1024 + 128: the int8 is read as q + 128
#pragma unroll
        for (int p = 0; p < 16; ++p) {      // pair p = quants 2p, 2p + 1 = stream bytes 2 + 2p, 3 + 2p counted from A0 (H == 0) or 4 + 2p (H == 1)
            const int byte = (H == 0 ? 2 : 4) + 2 * p;
            const uint32_t u = ws.at(byte / 4) ^ 0x80808080u;
            v[p] = h2mul(h2sub((byte % 4) ? magic23(u) : magic01(u), off), d2);
        }
    }
};

// Q4_K (rlx-gguf/src/lib.rs:974-1013): super-block = fp16 d | fp16 dmin | 12 scale bytes | 128 bytes; the 32 bytes
// [32 S, 32 S + 32) hold sub-block 2S in their low nibbles and 2S + 1 in their high nibbles; value
// (d * sc) * q - dmin * mn.  Half H takes words 4H..4H+3 of the eight.  Slot order of a 64-wide block: for word
// c = 0..7: weights 4c..4c+3 of sub-block 2S, then of sub-block 2S + 1.
template <int S> struct TcStage<RLXQ_Q4_K, S> {
    uint32_t dl2, nml2, dh2, nmh2;
    __device__ __forceinline__ void prep(const uint8_t* row) {
        const uint4 hd = *reinterpret_cast<const uint4*>(row);   // d, dmin, 12 scale bytes
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
        dl2 = h2splat(d * (float)sc[0]);  nml2 = h2splat(-(dmin * (float)mn[0]));
        dh2 = h2splat(d * (float)sc[1]);  nmh2 = h2splat(-(dmin * (float)mn[1]));
    }
    template <int H> __device__ __forceinline__ void half(const uint8_t* row, uint32_t (&v)[16]) const {
        const uint4 q = *reinterpret_cast<const uint4*>(row + 16 + 32 * S + 16 * H);
        const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
        const uint32_t off = 0x64006400u;   // 1024
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = qs[i] & 0x0F0F0F0Fu, hi = (qs[i] >> 4) & 0x0F0F0F0Fu;
            v[4 * i] = h2fma(h2sub(magic01(lo), off), dl2, nml2);
            v[4 * i + 1] = h2fma(h2sub(magic23(lo), off), dl2, nml2);
            v[4 * i + 2] = h2fma(h2sub(magic01(hi), off), dh2, nmh2);
            v[4 * i + 3] = h2fma(h2sub(magic23(hi), off), dh2, nmh2);
        }
    }
};

// Where the eight k slots of chunk t (0..31) of a 256-weight unit come from: activations [offA, offA + 4) then
// [offB, offB + 4), offsets inside the unit.  Chunk t belongs to the 64-wide k block t / 8, position t % 8.
template <uint32_t SCHEME> __device__ __forceinline__ void tc_xoff(uint32_t t, uint32_t& offA, uint32_t& offB) {
    if (SCHEME == RLXQ_Q4_0) { offA = 8u * t - 4u * (t & 3u); offB = offA + 16u; }        // block t / 4, word t % 4
    else if (SCHEME == RLXQ_Q8_0) { offA = 8u * t; offB = offA + 4u; }
    else { offA = 64u * (t >> 3) + 4u * (t & 7u); offB = offA + 32u; }                    // Q4_K
}

// Two activations -> fp16 pairs of their high parts h = fp16(clamp(x)) and low parts fp16((x - h) * 2^11); the
// first value in the low half.  x - h is exact in f32 and so is the scaling.
__device__ __forceinline__ void f16_hi_lo(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    x0 = fminf(fmaxf(x0, -65504.0f), 65504.0f);
    x1 = fminf(fmaxf(x1, -65504.0f), 65504.0f);
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x1), "f"(x0));
    float h0, h1;
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}" : "=f"(h0), "=f"(h1) : "r"(hi));
    const float r0 = (x0 - h0) * 2048.0f, r1 = (x1 - h1) * 2048.0f;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(r1), "f"(r0));
}
// Has the phase of this parity completed?  Never suspends.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_sc_gpu() { asm volatile("fence.sc.gpu;" ::: "memory"); }
__device__ __forceinline__ unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One chunk (eight k slots) of the B operand: activations [offA, offA + 4) and [offB, offB + 4) of row r of a unit
// as fp16 high and low parts, at their swizzled places in the unit's slab.
__device__ __forceinline__ void tc_store_chunk(uint8_t* slab, uint32_t r, uint32_t t, const float (&f)[8]) {
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f16_hi_lo(f[2 * i], f[2 * i + 1], hi[i], lo[i]);
    uint8_t* blk = slab + (t >> 3) * 2048u;                   // 64-wide k block
    const uint32_t chunk = ((t & 7u) ^ r) * 16u;              // 128-byte swizzle: chunk ^ (row % 8), the same for rows r and 8 + r
    *reinterpret_cast<uint4*>(blk + r * 128u + chunk) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4*>(blk + 1024u + r * 128u + chunk) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}
__device__ __forceinline__ void tc_widen_bf16(uint2 a, uint2 b, float (&f)[8]) {
    const uint32_t wv[4] = {a.x, a.y, b.x, b.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(wv[i] << 16);
        f[2 * i + 1] = __uint_as_float(wv[i] & 0xFFFF0000u);
    }
}

template <uint32_t SCHEME>
__global__ void __launch_bounds__(kTcThreads, 2) gemv_tc_kernel(const __grid_constant__ TcParams P) {
    constexpr uint32_t RAW_ROW = TcRaw<SCHEME>::ROW;
    constexpr uint32_t RAW_BYTES = kTcTileW * RAW_ROW;
    constexpr uint32_t RAW_STRIDE = (RAW_BYTES + 127) / 128 * 128;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* b_ring = smem;                                  // nb x 8 KB, 1024-aligned
    uint8_t* xs_ring = smem + P.off_xs;
    uint8_t* raw_ring = smem + P.off_raw;
    TcBars* bars = reinterpret_cast<TcBars*>(smem + P.off_bar);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    volatile uint32_t* abort_flag = &bars->abort_flag;
    griddep_launch_dependents();
    if (tid == 0) {
        tma_prefetch_desc(&P.wmap);
        for (uint32_t i = 0; i < P.nraw; ++i) { mbar_init(smem_u32(&bars->raw_full[i]), 1); mbar_init(smem_u32(&bars->raw_empty[i]), 4 * kTcGroups); }
        for (uint32_t i = 0; i < kTcAStages; ++i) { mbar_init(smem_u32(&bars->a_full[i]), 4); mbar_init(smem_u32(&bars->a_free[i]), 1); }
        for (uint32_t i = 0; i < kTcMaxB; ++i) { mbar_init(smem_u32(&bars->b_full[i]), 1); mbar_init(smem_u32(&bars->b_free[i]), 4); }
        for (uint32_t i = 0; i < 4; ++i) { mbar_init(smem_u32(&bars->xs_full[i]), 1); mbar_init(smem_u32(&bars->xs_free[i]), 1); }
        for (uint32_t i = 0; i < 2; ++i) { mbar_init(smem_u32(&bars->d_full[i]), 4); mbar_init(smem_u32(&bars->d_free[i]), 4); }
        bars->abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars->tmem_base), kTcCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    // accumulators: one per 64-wide k block of a unit (issue stream q at column 16 q); weight stages from column 64
    const uint32_t tmem_d = tmem_base, tmem_a = tmem_base + 64;
    auto give_up = [&](int code) {
        if (lane == 0) { atomicExch(P.err, code); *abort_flag = 1u; }
    };
    const uint32_t cur0 = tc_range_start(P, blockIdx.x), lim = tc_range_start(P, blockIdx.x + 1);
    const uint32_t nunits = lim - cur0;
    const uint32_t nb1 = min(nunits, P.nb);                 // units whose B slab is built directly from global memory

    if (warp == 0) {
        // ---------------- raw weight groups: everything is requested as soon as its stage is free ----------------
        if (lane == 0) {
            uint32_t cur = cur0, u = 0;
            TcSeg sg;
            bool ok = true;
            while (ok && !*abort_flag && tc_seg_next(P, cur, lim, sg)) {
                for (uint32_t g = sg.g0; g < sg.g1; ++g, ++u) {
                    const uint32_t r = u % P.nraw, rd = u / P.nraw;
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_empty[r]), (rd & 1u) ^ 1u)) { give_up(51); ok = false; break; }
                    const uint32_t full = smem_u32(&bars->raw_full[r]);
                    mbar_arrive_expect_tx(full, RAW_BYTES);
                    tma_load_2d(smem_u32(raw_ring + r * RAW_STRIDE), &P.wmap, (int32_t)(g * (RAW_ROW / 8u)), (int32_t)(sg.tile * kTcTileW), full);
                }
            }
            if (!ok || *abort_flag) {
                // let the copies in flight land before the CTA's shared memory goes away
                for (uint32_t i = 0; i < min(u, P.nraw); ++i) {
                    const uint32_t uu = u - 1 - i;
                    (void)mbar_wait(smem_u32(&bars->raw_full[uu % P.nraw]), (uu / P.nraw) & 1u);
                }
            }
        }
    } else if (warp < 3) {
        // ---------------- MMA issuers: four issue streams, two lanes in each of two warps ----------------
        // Stream q = 2 * issuer warp + lane takes k block q of every unit (decode group q % 2 produces it) into its own
        // accumulator.  A tcgen05.mma executed by two lanes costs 155 cycles against 115 for one, so the pair issues
        // two MMAs in the time of 1.35.
        if (lane < 2) {
            const uint32_t iss = warp - 1u, q = 2u * iss + lane;
            uint32_t cur = cur0, u = 0, segi = 0;
            TcSeg sg;
            bool ok = true;
            auto fail_now = [&](int code) { atomicExch(P.err, code); *abort_flag = 1u; };
            while (ok && !*abort_flag && tc_seg_next(P, cur, lim, sg)) {
                // one set of accumulators: the epilogue must have read the segment before
                if (!mbar_wait(smem_u32(&bars->d_free[0]), (segi & 1u) ^ 1u)) { fail_now(52); break; }
                tc_fence_after();
                bool first = true;
                for (uint32_t g = sg.g0; g < sg.g1 && ok; ++g, ++u) {
                    const uint32_t bs = u % P.nb;
                    const uint32_t lsb = 2u * u + iss;                  // running index of this k block within its decode group
                    const uint32_t s = lane + kTcGroups * (lsb % kTcGroupStages);
                    if (*abort_flag || !mbar_wait(smem_u32(&bars->b_full[bs]), (u / P.nb) & 1u)) { fail_now(53); ok = false; }
                    if (ok && (*abort_flag || !mbar_wait(smem_u32(&bars->a_full[s]), (lsb / kTcGroupStages) & 1u))) { fail_now(54); ok = false; }
                    ok = __all_sync(0x3u, ok);                          // the two lanes stay together
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = kmajor_sw128_desc(smem_u32(b_ring + bs * kTcBSlab + q * 2048u));
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        tc_mma_ts(tmem_d + 16u * q, tmem_a + 32u * s + 8u * j, bdesc + 2u * j, kTcIdesc, (first && j == 0) ? 0u : 1u);
                    first = false;
                    tc_commit(smem_u32(&bars->a_free[s]));
                    if (P.nxs) tc_commit(smem_u32(&bars->b_free[bs]));      // slabs are only reused by a long range
                }
                if (!ok) break;
                tc_commit(smem_u32(&bars->d_full[0]));
                ++segi;
            }
        }
    } else if (warp == 3 || warp >= 4 + 4 * kTcGroups) {
        // ---------------- activations (warp 3, helped at first by the epilogue warps), then the epilogue ----------------
        const uint32_t pid = warp == 3 ? lane : 32u + (tid - (4u + 4u * kTcGroups) * 32u);    // 0..159
        {   // rows m..7 and 8+m..15 of every slab stay zero for the whole kernel
            uint4* z = reinterpret_cast<uint4*>(b_ring);
            for (uint32_t i = pid; i < P.nb * kTcBSlab / 16u; i += kTcBThreads) z[i] = make_uint4(0u, 0u, 0u, 0u);
            asm volatile("bar.sync 2, 160;" ::: "memory");
        }
        griddep_wait();               // x comes from the kernel in front; y and the scratch may still be in use by it
        {
            // The first nb1 units straight from global memory: every load of a thread's batch is issued before the first
            // value is used, so the whole B operand of a short range costs one trip to L2.
            const uint32_t per_unit = 32u * P.m, total = nb1 * per_unit;
            // task q -> unit j of the range, activation row r, chunk t; its eight values sit at base + offA .. and base + offB ..
            auto locate = [&](uint32_t q, uint32_t& j, uint32_t& r, uint32_t& t, size_t& base, uint32_t& offA, uint32_t& offB) {
                j = q / per_unit;
                const uint32_t rem = q - j * per_unit;
                r = rem >> 5; t = rem & 31u;
                tc_xoff<SCHEME>(t, offA, offB);
                base = (size_t)r * P.k + (size_t)((cur0 + j) % P.kgroups) * 256u;
            };
            if (P.x_bf16) {
                for (uint32_t q0 = pid; q0 < total; q0 += 8u * kTcBThreads) {
                    uint2 ra[8], rb[8];
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        const uint32_t q = q0 + i * kTcBThreads;
                        if (q < total) {
                            uint32_t j, r, t, offA, offB; size_t base;
                            locate(q, j, r, t, base, offA, offB);
                            const uint16_t* xp = reinterpret_cast<const uint16_t*>(P.x) + base;
                            ra[i] = __ldcg(reinterpret_cast<const uint2*>(xp + offA));
                            rb[i] = __ldcg(reinterpret_cast<const uint2*>(xp + offB));
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        const uint32_t q = q0 + i * kTcBThreads;
                        if (q < total) {
                            uint32_t j, r, t, offA, offB; size_t base;
                            locate(q, j, r, t, base, offA, offB);
                            float f[8];
                            tc_widen_bf16(ra[i], rb[i], f);
                            tc_store_chunk(b_ring + j * kTcBSlab, r, t, f);
                        }
                    }
                }
            } else {
                for (uint32_t q0 = pid; q0 < total; q0 += 4u * kTcBThreads) {
                    float4 ra[4], rb[4];
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t q = q0 + i * kTcBThreads;
                        if (q < total) {
                            uint32_t j, r, t, offA, offB; size_t base;
                            locate(q, j, r, t, base, offA, offB);
                            const float* xp = reinterpret_cast<const float*>(P.x) + base;
                            ra[i] = __ldcg(reinterpret_cast<const float4*>(xp + offA));
                            rb[i] = __ldcg(reinterpret_cast<const float4*>(xp + offB));
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t q = q0 + i * kTcBThreads;
                        if (q < total) {
                            uint32_t j, r, t, offA, offB; size_t base;
                            locate(q, j, r, t, base, offA, offB);
                            const float f[8] = {ra[i].x, ra[i].y, ra[i].z, ra[i].w, rb[i].x, rb[i].y, rb[i].z, rb[i].w};
                            tc_store_chunk(b_ring + j * kTcBSlab, r, t, f);
                        }
                    }
                }
            }
            fence_proxy_async_smem();
            asm volatile("bar.sync 2, 160;" ::: "memory");
            if (pid == 0)
                for (uint32_t j = 0; j < nb1; ++j) mbar_arrive(smem_u32(&bars->b_full[j]));
        }
        if (warp == 3) {
            // ---------------- the rest of a long range: global -> staging ring (bulk copies) -> B slabs ----------------
            if (nunits > nb1) {
                const uint32_t esz = P.x_bf16 ? 2u : 4u;
                uint32_t iu = nb1;                               // next unit to request
                auto issue_next = [&]() -> bool {
                    if (iu >= nunits) return false;
                    const uint32_t v = iu - nb1, sl = v % P.nxs, rd = v / P.nxs;
                    if (!mbar_wait(smem_u32(&bars->xs_free[sl]), (rd & 1u) ^ 1u)) return false;
                    const uint32_t g = (cur0 + iu) % P.kgroups;
                    const uint32_t full = smem_u32(&bars->xs_full[sl]);
                    mbar_arrive_expect_tx(full, P.m * P.xs_row_bytes);
                    for (uint32_t r = 0; r < P.m; ++r)
                        bulk_g2s(smem_u32(xs_ring + sl * P.xs_stage_bytes + r * P.xs_row_bytes),
                                 reinterpret_cast<const uint8_t*>(P.x) + ((size_t)r * P.k + (size_t)g * 256u) * esz, P.xs_row_bytes, full);
                    ++iu;
                    return true;
                };
                if (lane == 0)
                    for (uint32_t i = 0; i < P.nxs; ++i)
                        if (!issue_next()) break;
                bool ok = true;
                const uint32_t ntask = 32u * P.m;
                for (uint32_t u = nb1; u < nunits && ok && !*abort_flag; ++u) {
                    const uint32_t v = u - nb1, sl = v % P.nxs, bs = u % P.nb;
                    if (!mbar_wait(smem_u32(&bars->xs_full[sl]), (v / P.nxs) & 1u) ||
                        !mbar_wait(smem_u32(&bars->b_free[bs]), ((u / P.nb) & 1u) ^ 1u)) { give_up(55); ok = false; break; }
                    const uint8_t* xs = xs_ring + sl * P.xs_stage_bytes;
                    for (uint32_t q = lane; q < ntask; q += 32u) {
                        const uint32_t r = q >> 5, t = q & 31u;
                        uint32_t offA, offB;
                        tc_xoff<SCHEME>(t, offA, offB);
                        float f[8];
                        if (P.x_bf16) {
                            tc_widen_bf16(*reinterpret_cast<const uint2*>(xs + r * P.xs_row_bytes + offA * 2u),
                                          *reinterpret_cast<const uint2*>(xs + r * P.xs_row_bytes + offB * 2u), f);
                        } else {
                            const float4 a = *reinterpret_cast<const float4*>(xs + r * P.xs_row_bytes + offA * 4u);
                            const float4 b = *reinterpret_cast<const float4*>(xs + r * P.xs_row_bytes + offB * 4u);
                            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
                        }
                        tc_store_chunk(b_ring + bs * kTcBSlab, r, t, f);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(smem_u32(&bars->b_full[bs])); mbar_arrive(smem_u32(&bars->xs_free[sl])); (void)issue_next(); }
                    __syncwarp();
                }
                if (lane == 0 && (!ok || *abort_flag)) {
                    // copies in flight must land before the CTA ends
                    for (uint32_t i = 0; i < min(iu - nb1, P.nxs); ++i) {
                        const uint32_t v = iu - nb1 - 1 - i;
                        (void)mbar_wait(smem_u32(&bars->xs_full[v % P.nxs]), (v / P.nxs) & 1u);
                    }
                }
            }
        } else {
            // ---------------- epilogue: accumulators -> y, or -> this CTA's part of a cut tile ----------------
            const uint32_t quarter = warp & 3u;
            const uint32_t lane_addr = (quarter * 32u) << 16;
            const uint32_t row = quarter * 32u + lane;
            uint32_t cur = cur0, segi = 0;
            TcSeg sg;
            while (!*abort_flag && tc_seg_next(P, cur, lim, sg)) {
                if (!mbar_wait(smem_u32(&bars->d_full[0]), segi & 1u)) { give_up(58); break; }
                tc_fence_after();
                float val[8];
                {
                    uint32_t dv[32];
                    tmem_ld32(tmem_d + lane_addr, dv);                  // streams 0 and 1
                    tmem_ld_wait();
                    float hi[8], lo[8];
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        hi[r] = __uint_as_float(dv[r]) + __uint_as_float(dv[16 + r]);
                        lo[r] = __uint_as_float(dv[8 + r]) + __uint_as_float(dv[24 + r]);
                    }
                    tmem_ld32(tmem_d + lane_addr + 32u, dv);            // streams 2 and 3
                    tmem_ld_wait();
#pragma unroll
                    for (int r = 0; r < 8; ++r) {    // the four streams in order, then high part + low part * 2^-11
                        hi[r] = (hi[r] + __uint_as_float(dv[r])) + __uint_as_float(dv[16 + r]);
                        lo[r] = (lo[r] + __uint_as_float(dv[8 + r])) + __uint_as_float(dv[24 + r]);
                        val[r] = fmaf(lo[r], 1.0f / 2048.0f, hi[r]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->d_free[0]));
                const uint32_t n_idx = sg.tile * kTcTileW + row;
                if (sg.g0 == 0 && sg.g1 == P.kgroups) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        if ((uint32_t)r < P.m && n_idx < P.n) {
                            const size_t o = (size_t)r * P.n + n_idx;
                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(val[r]);
                            else reinterpret_cast<float*>(P.y)[o] = val[r];
                        }
                    }
                } else {
                    // A cut tile.  Its first contributor (the CTA whose range ends inside the tile: this is the last thing
                    // it does) completes it; the others, for whom the tile is the first thing they do, only publish their
                    // values: one 8-byte word (value, call token) per output, a single store, valid by itself.
                    const uint32_t u0 = sg.tile * P.kgroups;
                    const uint32_t c_first = tc_owner(P, u0), c_last = tc_owner(P, u0 + P.kgroups - 1u);
                    const size_t slot_words = (size_t)P.m * kTcTileW;
                    if (blockIdx.x != c_first) {
                        unsigned long long* mine = P.parts + (size_t)(2u * blockIdx.x) * slot_words + row;   // head slot: the range begins inside the tile
                        const unsigned long long tok = (unsigned long long)P.token << 32;
#pragma unroll
                        for (int r = 0; r < 8; ++r)
                            if ((uint32_t)r < P.m) st_relaxed_gpu_u64(mine + r * kTcTileW, tok | __float_as_uint(val[r]));
                    } else {
                        // Word i of the list is (output row i / nother, contributor c_first + 1 + i % nother).  Sixteen words at
                        // a time, every load issued before the first value is used; a word whose token is not there yet
                        // is polled (bounded).  The sum runs in contributor order, this CTA's value first.
                        const uint32_t nother = c_last - c_first, total = P.m * nother;
                        unsigned long long* col = P.parts + (size_t)(2u * (c_first + 1u)) * slot_words + row;
                        uint32_t lr = 0, lc = 0, pr = 0, pc = 0;          // (output row, contributor) of the next word to load / to use
                        float sum = val[0];
                        bool ok = true;
                        for (uint32_t base = 0; base < total && ok; base += 16u) {
                            unsigned long long wv[16];
#pragma unroll
                            for (uint32_t i = 0; i < 16; ++i) {
                                if (base + i < total) {
                                    wv[i] = ld_relaxed_gpu_u64(col + (size_t)(2u * lc) * slot_words + lr * kTcTileW);
                                    if (++lc == nother) { lc = 0; ++lr; }
                                }
                            }
#pragma unroll
                            for (uint32_t i = 0; i < 16; ++i) {
                                if (base + i < total && ok) {
                                    unsigned long long* wp = col + (size_t)(2u * pc) * slot_words + pr * kTcTileW;
                                    for (uint32_t spin = 0; (uint32_t)(wv[i] >> 32) != P.token; ++spin) {
                                        if (spin >= kTcPollLimit || *abort_flag) { ok = false; break; }
                                        __nanosleep(200);
                                        wv[i] = ld_relaxed_gpu_u64(wp);
                                    }
                                    if (!ok) break;
                                    st_relaxed_gpu_u64(wp, 0ull);          // left at zero for a replay of the same captured launch (same token)
                                    sum += __uint_as_float((uint32_t)wv[i]);
                                    if (++pc == nother) {
                                        if (n_idx < P.n) {
                                            const size_t o = (size_t)pr * P.n + n_idx;
                                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(sum);
                                            else reinterpret_cast<float*>(P.y)[o] = sum;
                                        }
                                        pc = 0; ++pr;
                                        sum = pr < 8u ? val[pr & 7u] : 0.f;
                                    }
                                }
                            }
                        }
                        if (!ok) { atomicExch(P.err, 59); *abort_flag = 1u; }
                    }
                }
                ++segi;
            }
        }
    } else {
        // ---------------- decode: raw blocks -> fp16 rows in tensor memory ----------------
        const uint32_t quarter = warp & 3u, grp = (warp - 4u) >> 2;
        const uint32_t row = quarter * 32u + lane;                  // weight row of the tile == tensor-memory lane
        const uint32_t lane_addr = (quarter * 32u) << 16;
        uint32_t cur = cur0, u = 0, lsb = 0;
        TcSeg sg;
        bool ok = true;
        constexpr uint32_t kNoStage = 0xFFFFFFFFu;
        uint32_t pending = kNoStage;                                // stage stored to but not yet handed to the issuer
        auto publish = [&](uint32_t s) {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->a_full[s]));
        };
        while (ok && !*abort_flag && tc_seg_next(P, cur, lim, sg)) {
            for (uint32_t g = sg.g0; g < sg.g1 && ok; ++g, ++u) {
                const uint32_t r = u % P.nraw;
                // a block stored but not yet handed over must not sit through a wait for a box that is still on its way
                if (pending != kNoStage && !mbar_test(smem_u32(&bars->raw_full[r]), (u / P.nraw) & 1u)) { publish(pending); pending = kNoStage; }
                if (*abort_flag || !mbar_wait(smem_u32(&bars->raw_full[r]), (u / P.nraw) & 1u)) { give_up(56); ok = false; break; }
                const uint8_t* rp = raw_ring + r * RAW_STRIDE + row * RAW_ROW;
#pragma unroll
                for (uint32_t sub = 0; sub < 4; ++sub) {
                    if ((sub & (kTcGroups - 1u)) != grp) continue;      // group g takes k blocks g and g + 2 of every unit
                    const uint32_t s = grp + kTcGroups * (lsb % kTcGroupStages);
                    uint32_t v[16];
                    auto run = [&](auto stage) {
                        stage.prep(rp);
                        stage.template half<0>(rp, v);
                        // the stores of the block before this one have had the time of half a decode to land
                        if (pending != kNoStage) { publish(pending); pending = kNoStage; }
                        if (*abort_flag || !mbar_wait(smem_u32(&bars->a_free[s]), ((lsb / kTcGroupStages) & 1u) ^ 1u)) { give_up(57); ok = false; return; }
                        tc_fence_after();
                        tmem_st16(tmem_a + lane_addr + 32u * s, v);
                        stage.template half<1>(rp, v);
                        tmem_st16(tmem_a + lane_addr + 32u * s + 16u, v);
                        pending = s;
                    };
                    if (sub == 0) run(TcStage<SCHEME, 0>());
                    else if (sub == 1) run(TcStage<SCHEME, 1>());
                    else if (sub == 2) run(TcStage<SCHEME, 2>());
                    else run(TcStage<SCHEME, 3>());
                    if (!ok) break;
                    ++lsb;
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->raw_empty[r]));
            }
        }
        if (pending != kNoStage) publish(pending);
    }
    // everybody meets here, also after a timeout, so the tensor memory is always returned
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, kTcCols);
}

// ---- host side --------------------------------------------------------------------------------
struct TcPlan {
    bool ok;
    uint32_t grid, ntiles, kgroups, nraw, nb, nxs, off_xs, off_raw, off_bar, smem_bytes, xs_row_bytes, xs_stage_bytes;
    size_t ws_bytes;
};

template <uint32_t SCHEME>
static TcPlan plan_tc(uint32_t m, uint32_t k, uint32_t n, bool xbf) {
    constexpr uint32_t RAW_STRIDE = (kTcTileW * TcRaw<SCHEME>::ROW + 127) / 128 * 128;
    TcPlan pl{};
    if (m == 0 || m > 8 || n == 0 || k == 0 || k % 256) return pl;
    pl.ntiles = (n + kTcTileW - 1) / kTcTileW;
    pl.kgroups = k / 256;
    const uint64_t units = (uint64_t)pl.ntiles * pl.kgroups;
    if (units > 0x7FFFFFFFull) return pl;
    pl.grid = (uint32_t)(options().gemv_tc_ctas.load() > 0 ? options().gemv_tc_ctas.load() : 1) * (uint32_t)sm_count();
    if (pl.grid > units) pl.grid = (uint32_t)units;
    const uint32_t longest = (uint32_t)((units + pl.grid - 1) / pl.grid);     // units of the longest range
    pl.xs_row_bytes = 256u * (xbf ? 2u : 4u);
    pl.xs_stage_bytes = m * pl.xs_row_bytes;
    const uint32_t bars = (uint32_t)((sizeof(TcBars) + 127) / 128 * 128);
    // A short range keeps its whole B operand (no staging); a long one gets four slabs and two staging stages.
    // Whatever is left holds raw boxes: at least two, and slabs are given up for a third.
    uint32_t nb = longest <= kTcMaxB ? longest : 4u, nxs = longest <= kTcMaxB ? 0u : 2u;
    for (;;) {
        const uint32_t fixed = nb * kTcBSlab + (nxs * pl.xs_stage_bytes + 127u) / 128u * 128u + 1024u + bars;
        const uint32_t nraw = fixed < kTcSmemBudget ? (kTcSmemBudget - fixed) / RAW_STRIDE : 0u;
        if (nraw >= 3 || (nraw == 2 && nb <= 2)) { pl.nb = nb; pl.nxs = nxs; pl.nraw = nraw > kTcMaxRing ? kTcMaxRing : nraw; break; }
        if (nb <= 2) return pl;
        --nb;
        if (nb < longest && nxs == 0) nxs = 2u;
    }
    pl.off_xs = pl.nb * kTcBSlab;
    pl.off_raw = pl.off_xs + (pl.nxs * pl.xs_stage_bytes + 127u) / 128u * 128u;
    pl.off_bar = pl.off_raw + pl.nraw * RAW_STRIDE;
    pl.smem_bytes = 1024u + pl.off_bar + bars;
    pl.ws_bytes = ((size_t)2 * pl.grid * m * kTcTileW * 8 + 255) / 256 * 256;
    pl.ok = pl.smem_bytes <= kTcSmemBudget;
    return pl;
}

static TcPlan plan_tc_any(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, bool xbf) {
    switch (scheme) {
        case RLXQ_Q4_0: return plan_tc<RLXQ_Q4_0>(m, k, n, xbf);
        case RLXQ_Q8_0: return plan_tc<RLXQ_Q8_0>(m, k, n, xbf);
        case RLXQ_Q4_K: return plan_tc<RLXQ_Q4_K>(m, k, n, xbf);
        default: return TcPlan{};
    }
}

bool gemv_tc_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x, bool xbf) {
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    return plan_tc_any(scheme, m, k, n, xbf).ok;
}

// The scratch does not depend on the activation type.
size_t gemv_tc_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n) {
    const TcPlan a = plan_tc_any(scheme, m, k, n, false);
    return a.ok ? a.ws_bytes : 0;
}

// Odd 32-bit values, a different one for every call of this process (they repeat after 2^31 calls); the starting
// point differs from process to process.
static uint32_t tc_next_token() {
    static std::atomic<uint32_t> epoch{
        (uint32_t)(((unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9E3779B97F4A7C15ull) >> 33)};
    return (epoch.fetch_add(1) << 1) | 1u;
}

template <uint32_t SCHEME>
static int launch_tc_t(cudaStream_t stream, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf, uint32_t m,
                       uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    constexpr uint32_t RAW_ROW = TcRaw<SCHEME>::ROW;
    const TcPlan pl = plan_tc<SCHEME>(m, k, n, xbf);
    if (!pl.ok) return fail(RLXQ_E_SHAPE, "tensor-core GEMV does not support m=%u k=%u n=%u", m, k, n);
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(RLXQ_E_WORKSPACE, "tensor-core GEMV needs %zu workspace bytes, got %zu", pl.ws_bytes, ws_bytes);
    if ((uintptr_t)ws & 15u) return fail(RLXQ_E_ALIGN, "workspace must be 16-byte aligned");
    Geometry g;
    geometry(SCHEME, &g);
    TcParams P{};
    int rc = encode_weight_map(&P.wmap, w, n, (uint64_t)k / g.elems * g.bytes, RAW_ROW / 8, kTcTileW);
    if (rc) return rc;
    P.x = x; P.y = y; P.m = m; P.n = n; P.k = k; P.x_bf16 = xbf ? 1u : 0u; P.y_bf16 = ybf ? 1u : 0u;
    P.ntiles = pl.ntiles; P.kgroups = pl.kgroups;
    const uint32_t units = pl.ntiles * pl.kgroups;
    P.units_q = units / pl.grid; P.units_r = units % pl.grid;
    P.nraw = pl.nraw; P.nb = pl.nb; P.nxs = pl.nxs;
    P.off_xs = pl.off_xs; P.off_raw = pl.off_raw; P.off_bar = pl.off_bar;
    P.xs_row_bytes = pl.xs_row_bytes; P.xs_stage_bytes = pl.xs_stage_bytes;
    P.parts = reinterpret_cast<unsigned long long*>(ws);
    P.token = tc_next_token();
    P.err = device_error_word();
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    static std::atomic<uint32_t> attr_set[64];
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemv_tc_kernel<SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBudget));
        attr_set[dev].store(1);
    }
    rc = launch_pdl(gemv_tc_kernel<SCHEME>, dim3(pl.grid), dim3(kTcThreads), pl.smem_bytes, stream, P);
    if (rc) return rc;
    count_launch();
    return check_launch("gemv_tc_kernel");
}

int launch_gemv_tc(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf,
                   uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    switch (scheme) {
        case RLXQ_Q4_0: return launch_tc_t<RLXQ_Q4_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q8_0: return launch_tc_t<RLXQ_Q8_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        case RLXQ_Q4_K: return launch_tc_t<RLXQ_Q4_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes);
        default: return fail(RLXQ_E_SCHEME, "tensor-core GEMV: unsupported scheme %u", scheme);
    }
}

}  // namespace rlxq
