// Streaming decode GEMV for batch 1-8: integer dot products on raw block quants.
//
// The activations are quantised once to two int8 limbs per value, X = round(x / s_b) in
// [-16256, 16256] = 128*h + l, one f32 scale s_b per 32 values, with the integer block sums the
// formats' offsets need.  Weights are never converted: four 4-bit (or 8-, 6-bit) quants are masked
// into one register and multiplied against activations in int32, exactly; one int->float
// conversion and one FMA per 32-weight block apply d_block * s_block (f32 from there on).
// Two kinds of unit do the multiplying:
//  * dp4a units (batch 1-2, on request 3-4): one dp4a per four weights, limb and activation row;
//  * integer-MMA units (batch 2-8 for Q4_0, Q8_0, Q4_K, Q5_K, Q6_K; batch 1-8 for Q8_K, Q2_K, Q3_K, Q4_1, Q5_0,
//    Q5_1, which have no dp4a unit): one m16n8k32 MMA per 32-weight block of all 16 tile rows against four
//    activation rows x two limbs (m16n8k16 per 16-weight sub-block for Q6_K, Q2_K, Q3_K).  mma.sync with 8-bit integers runs at
//    one m16n8k32 per 8 cycles per sub-core here, far more than the stream needs; what the units
//    save is instruction issue, which is what bounds the dp4a units from batch 3 on.
//
// gemv_int_kernel (the streaming kernel).  Persistent CTAs, two per SM (one with the integer-MMA
// units or more than two rows).  All CTAs together walk one
// global list of work items, (16-row weight tile, 2048-weight chunk), split into equal contiguous
// ranges ("stream-K"), so every SM streams the same number of bytes whatever n and k are.  Per CTA
// a producer warp keeps a ring of shared-memory stages full, one 2-D TMA box (16 rows x one chunk)
// and one mbarrier per stage; the ring takes all the shared memory the CTA has.  Eight consumer
// warps take one 256-weight unit of the stage each (sixteen, half a unit each, with the integer-MMA
// units); a finisher warp adds their partial sums and
// writes the tile, so the consumers never wait on global memory.
//
// Two ways to run it:
//  * single-kernel mode (m*k <= 12288; k <= 4096 for three or four rows with the integer-MMA units; tiles shared by at most
//    two CTAs): the consumer warps
//    quantise the activations themselves into shared memory.  Two ring stages are requested before
//    the dependency wait (weights are immutable, so they overlap the previous kernel's tail), then
//    the activation loads, then the rest of the ring: a load issued behind a full ring of weight
//    requests waits for microseconds in the SM's memory queue.  A tile shared by two CTAs is
//    completed through a token exchange that needs no zeroed memory.
//  * two-kernel mode (everything else): quantise_x_kernel writes the quantised activations to the
//    workspace, clears the tile counters (and y for the two-contributor add mode); the streaming
//    kernel fetches them by bulk copy.
//
// All kernels use programmatic dependent launch: the streaming kernel is made resident while its
// predecessor drains and requests weight stages before griddepcontrol.wait.
//
// Error: the activation quantisation only; |y - y_exact| <= 2^-15 * sqrt(32) * |x| * |w_row|
// = 1.7e-4 * |x| * |w_row| in the worst case, about 1e-6 typically, plus f32 accumulation over
// blocks.
//
// Replaces, for m <= 8, the reference's dequantise-everything + cublasSgemm
// (rlx-cuda/src/gguf_gpu.rs:62-134).
#include <chrono>

#include "common.cuh"
#include "decode.cuh"
#include "kernels.h"
#include "staged_common.cuh"
#include "tensormap.cuh"
#include "tp_comm.cuh"

namespace rlxq {

constexpr uint32_t kIntWarps = 8;                      // consumer warps of the dp4a units
// Consumer warps: one per 256-weight unit of a stage for the dp4a units, two (four blocks of the unit each)
// for the integer-MMA units, whose chain load -> mask -> MMA -> convert -> FMA wants more warps to hide under.
constexpr uint32_t int_warps(bool mma) { return mma ? 16u : kIntWarps; }
constexpr uint32_t int_threads(bool mma) { return (int_warps(mma) + 2) * 32; }   // + one producer warp + one finisher warp
// lanes of a consumer warp that hand partial sums to the finisher
constexpr uint32_t int_red_lanes(bool mma) { return mma ? 16u : 32u; }
constexpr uint32_t kIntRB = 4;                         // ring of reduction buffers between consumers and finisher
// single-kernel mode: groups of 8 activations a consumer thread quantises (8 for the four-row kernel)
// integer-MMA units, single-kernel mode: log2 of the activation rows a warp quantises per round
__host__ __device__ constexpr uint32_t inline_rows_log2(uint32_t m_real) { return m_real >= 3 ? 2u : (m_real == 2 ? 1u : 0u); }
constexpr uint32_t inline_groups(int mm, bool mma = false) { return mma ? 4u : (mm > 2 ? 8u : 6u); }
constexpr uint32_t kIntCU = 8;                         // 256-weight units per stage = one per warp

// A stage is NB boxes of 16 rows x UB units, each box fetched by ONE 2-D TMA request (a request
// per row costs about 250 cycles of issue time each and caps the stream near 3 TB/s; one box per
// request does not).  A box row is UB units plus 16 bytes (32 for Q4_0, whose lane mapping wants a
// row pitch of 8 words mod 32), read from the next units or zero past the row end, so that rows do
// not all start on the same shared-memory bank; Q6_K's 1680-byte rows already do not.  TMA boxes
// are at most 256 eight-byte elements wide, hence two for Q8_0.
// (The integer-MMA unit of Q4_0 reads word t of rows g and g + 8, lane = 4 g + t: a pitch of 4 words mod 32.)
// (Q8_K: two boxes of four 292-byte units, 32 bytes of padding: a pitch of 12 words mod 32.  Q2_K: 8 x 84 + 16 bytes,
// also 12 mod 32.  Q3_K: 8 x 110 bytes, 28 mod 32, no padding.)
template <uint32_t SCHEME, bool MMA = false> struct IntBox {
    static constexpr uint32_t NB = (SCHEME == RLXQ_Q8_0 || SCHEME == RLXQ_Q8_K) ? 2u : 1u;
    static constexpr uint32_t UB = kIntCU / NB;                               // units per box
    static constexpr uint32_t ROW = UB * StagedTraits<SCHEME>::UNIT_B +
        ((SCHEME == RLXQ_Q6_K || SCHEME == RLXQ_Q3_K) ? 0u : ((SCHEME == RLXQ_Q4_0 && !MMA) || SCHEME == RLXQ_Q8_K) ? 32u : 16u);
    static constexpr uint32_t BOX_BYTES = 16 * ROW;
    static constexpr uint32_t STAGE_BYTES = NB * BOX_BYTES;
};

struct IntParams {
    CUtensorMap wmap;      // W as [n rows][row_bytes / 8] eight-byte elements, box = 16 rows x IntBox::ROW
    const uint8_t* w;
    void* y;
    const uint8_t* xq;     // workspace: per row [h: k][l: k][s_b: k/32 f32][sums: k/SUB i32]
    float* partial;        // [ntiles][slots][MM][16]
    uint32_t* counters;    // [ntiles] chunks finished per tile
    int* err;
    uint32_t k, n, y_bf16;
    uint32_t m_real;       // activation rows actually present (3 runs with the four-row kernel)
    uint32_t use_red;      // shared tiles have exactly two contributors: add them into zeroed f32 y
    uint32_t row_bytes, ntiles, nchunks, total_chunks, slots;
    uint32_t chunks_q, chunks_r;   // total_chunks = grid * chunks_q + chunks_r: the first chunks_r CTAs take one more
    uint32_t nstages;
    uint32_t xq_row_bytes; // bytes of one row of xq (integer-MMA units: of one of the equal pieces it is fetched in)
    uint32_t xq_pieces;    // bulk copies that fetch xq: one per activation row (integer-MMA units: 8)
    // Integer-MMA units when the fragments of all rows do not fit in shared memory: nothing of xq is resident;
    // every ring stage carries, behind its weights, the fragments and scale entries of its own 2048-weight
    // chunk (two bulk copies from the workspace, out of L2).  stage_stride: bytes from one ring stage to the next.
    uint32_t xstream, stage_stride;
    // Chain kernel only: CTAs that take part in this layer (the split chunks_q / chunks_r is over them), and
    // whether the layer's input is the SwiGLU product of the previous layer's [gate | up] output.
    uint32_t active, swiglu;
    // Tensor-parallel push (tp.world = 0: off).  The kernel is the row-parallel down projection of a sharded FFN:
    // a finished tile goes into this rank's slot of every rank's exchange buffer instead of y; after its last
    // tile a CTA counts itself in at every rank, waits until every rank's CTAs are all in, and writes its share
    // of y = sum over ranks, in rank order, out of its own rank's buffer.  The quantiser kernel in front advances
    // the step counter and the expected arrival count (tp_comm.cuh).
    TpPush tp;
    uint32_t off_stage, off_red, off_bar;
    // Single-kernel mode: the consumer warps quantise the activations themselves (no quantiser kernel in
    // front), and a tile shared by two CTAs is completed through a token exchange that needs no zeroed memory.
    uint32_t inline_q;
    const void* x;         // [MM][k] activations, f32 or bf16 (single-kernel mode)
    uint32_t x_bf16;
    unsigned long long* flags;   // [ntiles] rendezvous words of shared tiles (single-kernel mode)
    unsigned long long token;    // odd, unique to this call
    uint32_t early;              // single-kernel mode: stages requested before the dependency wait
    // Expert-indirect mode (MoE decode): W is a stack of [n, k] slabs and this launch multiplies by slab
    // *expert_sel read as the reference's `as usize` cast does (expert_of_row), on the device after the
    // dependency wait; an id of num_experts or more makes the kernel return at once (the caller has zeroed y).
    const float* expert_sel;
    uint32_t num_experts;
};

// Per-thread view for the integer kernel.  Everything is a 32-bit shared-memory byte address: the
// inner loops then run on 32-bit address arithmetic and ld.shared, never on generic 64-bit pointers.
struct QLane {
    uint32_t row;      // this thread's tile row inside the current stage
    uint32_t xh, xl;   // limb planes of activation row 0, already advanced to this thread's half (+128 * half)
    uint32_t sb;       // f32 scale per 32 activations, advanced by 16 * half
    uint32_t sx;       // i32 offset-premultiplied block sums, advanced to this thread's half
    uint32_t xstride;  // bytes between activation rows (all four arrays of a row move together)
    uint32_t half;     // which half of a 256-weight unit this thread handles
    uint32_t lane;
    uint32_t row_pitch; // bytes between tile rows inside a stage
};


__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float ldsf(uint32_t a) { return __uint_as_float(lds32(a)); }

// Sum over 4*NW weights of q * X for one activation row: q words against the two limb planes.
template <int NW>
__device__ __forceinline__ int dot_limbs(const uint32_t (&q)[NW], uint32_t xh, uint32_t xl, int init_low) {
    int ah = 0, al = init_low;
#pragma unroll
    for (int i = 0; i < NW; i += 4) {
        const uint4 h = lds128(xh + 4 * i), l = lds128(xl + 4 * i);
        ah = __dp4a((int)q[i], (int)h.x, ah);         al = __dp4a((int)q[i], (int)l.x, al);
        ah = __dp4a((int)q[i + 1], (int)h.y, ah);     al = __dp4a((int)q[i + 1], (int)l.y, al);
        ah = __dp4a((int)q[i + 2], (int)h.z, ah);     al = __dp4a((int)q[i + 2], (int)l.z, al);
        ah = __dp4a((int)q[i + 3], (int)h.w, ah);     al = __dp4a((int)q[i + 3], (int)l.w, al);
    }
    return ah * 128 + al;
}

template <uint32_t SCHEME, int MM> struct QUnit;

// In every run(): u = unit inside the box row, kb = index of the unit's first weight in the row.

// Defaults of the per-format mappings: a lane is (tile row = lane & 15, half of the unit = lane >> 4)
// and keeps one accumulator per activation row.
template <int MM> struct QUnitRowHalf {
    static constexpr int NT = 1;                                           // accumulators per activation row
    static constexpr int NACC = MM;
    static constexpr bool HALF_OFFSETS = true;                             // the activation views start at the lane's half
    static constexpr uint32_t STRIDE_ROWS = 1;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane & 15u; }
    __device__ static __forceinline__ void finalize(float (&)[MM], uint32_t) {}
};

// ---- Q4_0: unit = 8 blocks of 18 bytes.  Lane = (row group rq = lane & 3, block b = lane >> 2): it
// takes block b of the four tile rows rq, rq + 4, rq + 8, rq + 12.  The 32 activations of block b stay
// in registers for all four rows, so a weight costs a quarter of the shared-memory traffic a
// (row, half-unit) mapping pays for re-reading activations; with a row pitch of 8 words mod 32 the
// weight reads of a warp fall on 32 different banks, and the eight lanes that a 16-byte activation
// load is served for together want two addresses only.  The eight block sums of a row meet in finalize().
template <int MM> struct QUnit<RLXQ_Q4_0, MM> {
    static constexpr int NT = 4;
    static constexpr int NACC = 4 * MM;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane & 3u; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[NT * MM]) {
        const uint32_t b = L.lane >> 2, odd = b & 1u;
        const uint32_t sh = 16u + 16u * odd, dsh = 16u * odd;
        // an even block starts on a word (d, then the quants from byte 2); an odd one two bytes into a word
        const uint32_t p = L.row + u * 144 + 36 * (b >> 1) + 16 * odd;
        const uint32_t kx = kb + 32 * b;
        uint4 xh[MM][2], xl[MM][2];
        float sbv[MM];
        int sxv[MM];
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            const uint32_t o = m * L.xstride;
            xh[m][0] = lds128(L.xh + o + kx); xh[m][1] = lds128(L.xh + o + kx + 16);
            xl[m][0] = lds128(L.xl + o + kx); xl[m][1] = lds128(L.xl + o + kx + 16);
            sbv[m] = ldsf(L.sb + o + (kx >> 3));
            sxv[m] = (int)lds32(L.sx + o + (kx >> 3));   // -8 * sum(X): the format's offset
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t pr = p + 4 * i * L.row_pitch;
            uint32_t w[5];
#pragma unroll
            for (int j = 0; j < 5; ++j) w[j] = lds32(pr + 4 * j);
            const float d = f16_bits_to_f32((w[0] >> dsh) & 0xFFFFu);
            uint32_t lo[4], hi[4];                    // low nibbles: weights 0..15 of the block, high: 16..31
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t qs = __funnelshift_rc(w[j], w[j + 1], sh);
                lo[j] = qs & 0x0F0F0F0Fu;
                hi[j] = (qs >> 4) & 0x0F0F0F0Fu;
            }
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                int ah = 0, al = sxv[m];
                ah = __dp4a((int)lo[0], (int)xh[m][0].x, ah);  al = __dp4a((int)lo[0], (int)xl[m][0].x, al);
                ah = __dp4a((int)lo[1], (int)xh[m][0].y, ah);  al = __dp4a((int)lo[1], (int)xl[m][0].y, al);
                ah = __dp4a((int)lo[2], (int)xh[m][0].z, ah);  al = __dp4a((int)lo[2], (int)xl[m][0].z, al);
                ah = __dp4a((int)lo[3], (int)xh[m][0].w, ah);  al = __dp4a((int)lo[3], (int)xl[m][0].w, al);
                ah = __dp4a((int)hi[0], (int)xh[m][1].x, ah);  al = __dp4a((int)hi[0], (int)xl[m][1].x, al);
                ah = __dp4a((int)hi[1], (int)xh[m][1].y, ah);  al = __dp4a((int)hi[1], (int)xl[m][1].y, al);
                ah = __dp4a((int)hi[2], (int)xh[m][1].z, ah);  al = __dp4a((int)hi[2], (int)xl[m][1].z, al);
                ah = __dp4a((int)hi[3], (int)xh[m][1].w, ah);  al = __dp4a((int)hi[3], (int)xl[m][1].w, al);
                tot[i * MM + m] = fmaf(d * sbv[m], (float)(ah * 128 + al), tot[i * MM + m]);
            }
        }
    }
    // Adds the eight block lanes of every row (a fixed butterfly: the order never changes) and hands
    // lane l < 16 the total of tile row l in tot[0 .. MM); lanes 16..31 get zero.
    __device__ static __forceinline__ void finalize(float (&tot)[NT * MM], uint32_t lane) {
#pragma unroll
        for (int t = 0; t < NT * MM; ++t) {
            float v = tot[t];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            tot[t] = v;
        }
        // tile row l = rq + 4 i lives in the lanes rq = l & 3 (mod 4) as accumulator i = l >> 2
        float out[MM];
#pragma unroll
        for (int m = 0; m < MM; ++m) out[m] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                const float v = __shfl_sync(0xFFFFFFFFu, tot[i * MM + m], lane & 3u);
                if (lane < 16u && (lane >> 2) == (uint32_t)i) out[m] = v;
            }
#pragma unroll
        for (int m = 0; m < MM; ++m) tot[m] = out[m];
    }
};

// ---- Q8_0: unit = 8 blocks of 34 bytes; a thread takes 4 consecutive blocks (136 bytes) ----
template <int MM> struct QUnit<RLXQ_Q8_0, MM> : QUnitRowHalf<MM> {
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM]) {
        const uint32_t p = L.row + u * 272 + 136 * L.half;
        const uint32_t xh = L.xh + kb, xl = L.xl + kb, sb = L.sb + (kb >> 3);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {              // two blocks = 68 bytes = 17 words at a time
            uint32_t w[18];
#pragma unroll
            for (int i = 0; i < 9; ++i) { const uint2 v = lds64(p + 64 * jj + 8 * i); w[2 * i] = v.x; w[2 * i + 1] = v.y; }
            // jj = 0 reads bytes [0, 72): words 0..17 hold blocks 0 and 1 (17 words) plus one spare.
            // jj = 1 reads bytes [64, 136): block 2 starts at byte 68, i.e. at word 1 of this window.
            const int o = jj;                          // word offset of the block pair inside w[]
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t q[8], dbits;
                if (j == 0) {
                    dbits = w[o] & 0xFFFFu;
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[o + i], w[o + i + 1], 16);
                } else {
                    dbits = w[o + 8] >> 16;
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[i] = w[o + 9 + i];
                }
                const float d = f16_bits_to_f32(dbits);
                const int bj = 2 * jj + j;
#pragma unroll
                for (int m = 0; m < MM; ++m) {
                    const uint32_t ox = m * L.xstride;
                    const int c = dot_limbs<8>(q, xh + ox + 32 * bj, xl + ox + 32 * bj, 0);
                    tot[m] = fmaf(d * ldsf(sb + ox + 4 * bj), (float)c, tot[m]);
                }
            }
        }
    }
};

// ---- Q4_K: unit = one 144-byte super-block; a thread takes sub-blocks 4*half .. 4*half+3 ----
template <int MM> struct QUnit<RLXQ_Q4_K, MM> : QUnitRowHalf<MM> {
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM]) {
        const uint32_t p = L.row + u * 144;
        const uint4 hd = lds128(p);                   // d, dmin, 12 scale bytes
        const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
        uint32_t scb, mnb;                            // four 6-bit scales / mins, one per byte
        if (L.half == 0) {
            scb = hd.y & 0x3F3F3F3Fu;
            mnb = hd.z & 0x3F3F3F3Fu;
        } else {
            scb = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mnb = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
        }
        const uint32_t xh = L.xh + kb, xl = L.xl + kb, sb = L.sb + (kb >> 3), sx = L.sx + (kb >> 3);
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {              // a pair of sub-blocks shares 32 bytes
            const uint32_t qp = p + 16 + 64 * L.half + 32 * pp;
            const uint4 a = lds128(qp), b = lds128(qp + 16);
            const uint32_t raw[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                uint32_t q[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = (raw[i] >> (4 * nib)) & 0x0F0F0F0Fu;
                const int js = 2 * pp + nib;          // sub-block index within this half
                const float dsc = d * (float)((scb >> (8 * js)) & 0xFFu);
                const float dmn = dmin * (float)((mnb >> (8 * js)) & 0xFFu);
#pragma unroll
                for (int m = 0; m < MM; ++m) {
                    const uint32_t ox = m * L.xstride;
                    const int c = dot_limbs<8>(q, xh + ox + 32 * js, xl + ox + 32 * js, 0);
                    const float sbv = ldsf(sb + ox + 4 * js);
                    // sx holds sum(X) of the block: the min term is dmin * m * s_b * sum(X)
                    const float sxf = sbv * (float)(int)lds32(sx + ox + 4 * js);
                    tot[m] = fmaf(dsc * sbv, (float)c, fmaf(-dmn, sxf, tot[m]));
                }
            }
        }
    }
};

// ---- Q5_K: unit = one 176-byte super-block d | dmin | 12 scale bytes | qh[32] | qs[128]; as Q4_K, with bit
// j of qh[l] adding 16 to weight l of sub-block j (rlx-gguf/src/lib.rs:1019-1068) ----
template <int MM> struct QUnit<RLXQ_Q5_K, MM> : QUnitRowHalf<MM> {
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM]) {
        const uint32_t p = L.row + u * 176;
        const uint4 hd = lds128(p);                   // d, dmin, 12 scale bytes
        const float d = f16_bits_to_f32(hd.x & 0xFFFFu), dmin = f16_bits_to_f32(hd.x >> 16);
        uint32_t scb, mnb;                            // four 6-bit scales / mins, one per byte
        if (L.half == 0) {
            scb = hd.y & 0x3F3F3F3Fu;
            mnb = hd.z & 0x3F3F3F3Fu;
        } else {
            scb = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mnb = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
        }
        const uint4 ha = lds128(p + 16), hb = lds128(p + 32);
        // the four high bits this half needs, moved to bits 0..3 of every byte
        const uint32_t hs = 4 * L.half;
        const uint32_t qh[8] = {(ha.x >> hs) & 0x0F0F0F0Fu, (ha.y >> hs) & 0x0F0F0F0Fu, (ha.z >> hs) & 0x0F0F0F0Fu,
                                (ha.w >> hs) & 0x0F0F0F0Fu, (hb.x >> hs) & 0x0F0F0F0Fu, (hb.y >> hs) & 0x0F0F0F0Fu,
                                (hb.z >> hs) & 0x0F0F0F0Fu, (hb.w >> hs) & 0x0F0F0F0Fu};
        const uint32_t xh = L.xh + kb, xl = L.xl + kb, sb = L.sb + (kb >> 3), sx = L.sx + (kb >> 3);
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {              // a pair of sub-blocks shares 32 bytes
            const uint32_t qp = p + 48 + 64 * L.half + 32 * pp;
            const uint4 a = lds128(qp), b = lds128(qp + 16);
            const uint32_t raw[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int js = 2 * pp + nib;          // sub-block index within this half
                uint32_t q[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    q[i] = ((raw[i] >> (4 * nib)) & 0x0F0F0F0Fu) | (((qh[i] >> js) & 0x01010101u) << 4);
                const float dsc = d * (float)((scb >> (8 * js)) & 0xFFu);
                const float dmn = dmin * (float)((mnb >> (8 * js)) & 0xFFu);
#pragma unroll
                for (int m = 0; m < MM; ++m) {
                    const uint32_t ox = m * L.xstride;
                    const int c = dot_limbs<8>(q, xh + ox + 32 * js, xl + ox + 32 * js, 0);
                    const float sbv = ldsf(sb + ox + 4 * js);
                    const float sxf = sbv * (float)(int)lds32(sx + ox + 4 * js);
                    tot[m] = fmaf(dsc * sbv, (float)c, fmaf(-dmn, sxf, tot[m]));
                }
            }
        }
    }
};

// ---- Q6_K: unit = one 210-byte super-block (only 2-byte aligned); a thread takes one half ----
template <int MM> struct QUnit<RLXQ_Q6_K, MM> : QUnitRowHalf<MM> {
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM]) {
        // 210*u is 2 mod 4 for odd u: read aligned words from 2 bytes earlier and funnel-shift.
        const uint32_t odd = u & 1u, sh = odd * 16u;
        const uint32_t pa = L.row + u * 210 - 2 * odd;
        const uint32_t h = L.half;
        uint32_t ql[16], qh[8], scw[2];
        {
            uint32_t a[17];
#pragma unroll
            for (int i = 0; i < 17; ++i) a[i] = lds32(pa + 64 * h + 4 * i);
#pragma unroll
            for (int i = 0; i < 16; ++i) ql[i] = __funnelshift_r(a[i], a[i + 1], sh);
            uint32_t b[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) b[i] = lds32(pa + 128 + 32 * h + 4 * i);
#pragma unroll
            for (int i = 0; i < 8; ++i) qh[i] = __funnelshift_r(b[i], b[i + 1], sh);
            uint32_t c3[3];
#pragma unroll
            for (int i = 0; i < 3; ++i) c3[i] = lds32(pa + 192 + 8 * h + 4 * i);
            scw[0] = __funnelshift_r(c3[0], c3[1], sh);
            scw[1] = __funnelshift_r(c3[1], c3[2], sh);
        }
        const uint32_t dw = lds32(pa + 208);
        const float d = f16_bits_to_f32((dw >> sh) & 0xFFFFu);
        // here the sums are per 16 values: L.sx was advanced by 32 * half (8 sums of 4 bytes)
        const uint32_t xh = L.xh + kb, xl = L.xl + kb, sb = L.sb + (kb >> 3), sx = L.sx + (kb >> 2);
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {              // four interleaved 32-weight groups per half
            const int nib = g4 >> 1, ps = g4 & 1;
#pragma unroll
            for (int i = 0; i < 2; ++i) {             // 16-weight sub-blocks, each with its own scale
                uint32_t q[4];
#pragma unroll
                for (int wv = 0; wv < 4; ++wv) {
                    const uint32_t lo = (ql[8 * ps + 4 * i + wv] >> (4 * nib)) & 0x0F0F0F0Fu;
                    const uint32_t hv = qh[4 * i + wv];
                    const uint32_t hi = (g4 < 2 ? (hv << (4 - 2 * g4)) : (hv >> (2 * g4 - 4))) & 0x30303030u;
                    q[wv] = lo | hi;
                }
                const int si = 2 * g4 + i;            // scale index inside the half
                const float ds = d * (float)(int8_t)((scw[si >> 2] >> (8 * (si & 3))) & 0xFFu);
                const int ke = 32 * g4 + 16 * i;      // first weight of the sub-block inside this half
#pragma unroll
                for (int m = 0; m < MM; ++m) {
                    // sx holds -32 * sum(X) per 16 values
                    const uint32_t ox = m * L.xstride;
                    const int c = dot_limbs<4>(q, xh + ox + ke, xl + ox + ke, (int)lds32(sx + ox + 4 * si));
                    tot[m] = fmaf(ds * ldsf(sb + ox + 4 * g4), (float)c, tot[m]);
                }
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Integer-MMA units (batch 3-8).  A dp4a unit pays two instructions per four weights and activation
// row.  Here one integer MMA (m16n8k32, u8 x s8 -> s32; 8 cycles per sub-core on this GPU) multiplies
// a 32-weight block of all 16 tile rows by eight columns = four activation rows x two limbs.  The
// weights are still never converted (the nibbles are masked into the A fragment straight from the
// block), the products are exact in int32, and both limb sums of an (output row, activation row)
// pair land in one lane: for lane = 4 g + t, c0 = sum q h and c1 = sum q l of (tile row g, activation
// row t), c2 and c3 the same for tile row g + 8.  The activations sit in shared memory in fragment
// order: [block][group of four rows][lane]{b0, b1}, then [block][row]{scale, bias * block sum}.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    // c = a * b (a zero accumulator comes in as the zero register, not as four moves)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void imma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Bytes of the fragment-ordered activations of mmg groups of four rows, and where their scales start.
__host__ __device__ constexpr uint32_t frag_scale_offset(uint32_t k, uint32_t mmg) { return (k / 32) * mmg * 256; }
// A scale entry is {scale, bias * sum} (8 bytes) or, for formats whose offsets need the sums of 16 values,
// {scale, bias * sum of the first 16, bias * sum of the second 16, -} (16 bytes).
__host__ __device__ constexpr uint32_t frag_entry_bytes(uint32_t sub) { return sub == 16 ? 16u : 8u; }
__host__ __device__ constexpr uint32_t frag_total_bytes(uint32_t k, uint32_t mmg, uint32_t sub) {
    return (k / 32) * mmg * (256 + 4 * frag_entry_bytes(sub));
}

template <uint32_t SCHEME, int MM> struct QUnitMma;

// Hands lane l < 16 the totals of tile row l in tot[0 .. MM) (zero to lanes 16..31), from the MMA's
// accumulator layout: lane 4 g + t holds (tile row g, activation row 4 q + t) in tot[2 q] and
// (tile row g + 8, the same activation row) in tot[2 q + 1].
template <int MM>
__device__ __forceinline__ void mma_rows_to_lanes(float (&tot)[MM], uint32_t lane) {
    float out[MM];
#pragma unroll
    for (int c = 0; c < MM; ++c) {
        const uint32_t src = 4u * (lane & 7u) + (uint32_t)(c & 3);
        const float v0 = __shfl_sync(0xFFFFFFFFu, tot[2 * (c >> 2)], src);
        const float v1 = __shfl_sync(0xFFFFFFFFu, tot[2 * (c >> 2) + 1], src);
        out[c] = lane < 16u ? ((lane >> 3) ? v1 : v0) : 0.f;
    }
#pragma unroll
    for (int c = 0; c < MM; ++c) tot[c] = out[c];
}

// ---- Q4_0: quant word t of a block holds weights 4t .. 4t+3 in its low nibbles (the MMA's k = 4t ..)
// and weights 16+4t .. in its high nibbles (k = 16+4t ..): one load and three logic instructions per
// tile row and block.
template <int MM> struct QUnitMma<RLXQ_Q4_0, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    // part: which four blocks of the unit this warp takes (two warps share a unit)
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * 144 + 72 * part, p8 = p0 + 8 * L.row_pitch;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            // the word that holds d: an even block starts on a word (d, then the quants from byte 2), an
            // odd one two bytes into a word (d in its upper half, the quants aligned behind it)
            const uint32_t o = 36 * (b >> 1) + 16 * (b & 1);
            uint32_t q0, q8, dw0, dw8;
            if (b & 1) {
                dw0 = lds32(p0 + o) >> 16;
                dw8 = lds32(p8 + o) >> 16;
                q0 = lds32(p0 + o + 4 + 4 * t);
                q8 = lds32(p8 + o + 4 + 4 * t);
            } else {
                dw0 = lds32(p0 + o) & 0xFFFFu;
                dw8 = lds32(p8 + o) & 0xFFFFu;
                q0 = __funnelshift_r(lds32(p0 + o + 4 * t), lds32(p0 + o + 4 * t + 4), 16);
                q8 = __funnelshift_r(lds32(p8 + o + 4 * t), lds32(p8 + o + 4 * t + 4), 16);
            }
            const float d0 = f16_bits_to_f32(dw0), d8 = f16_bits_to_f32(dw8);
            const uint32_t a0 = q0 & 0x0F0F0F0Fu, a2 = (q0 >> 4) & 0x0F0F0F0Fu;
            const uint32_t a1 = q8 & 0x0F0F0F0Fu, a3 = (q8 >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int gq = 0; gq < MMG; ++gq) {
                const uint2 bb = lds64(fb + (b * MMG + gq) * 256);
                const uint2 sc = lds64(sb + (b * MMG + gq) * 32);
                int c[4];
                imma_u8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                const float s = __uint_as_float(sc.x);
                const int sx = (int)sc.y;                          // -8 * sum(X): the format's offset
                tot[2 * gq] = fmaf(d0 * s, (float)(c[0] * 128 + c[1] + sx), tot[2 * gq]);
                tot[2 * gq + 1] = fmaf(d8 * s, (float)(c[2] * 128 + c[3] + sx), tot[2 * gq + 1]);
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q4_1 / Q5_0 / Q5_1 (rlx-gguf/src/lib.rs:635-729): blocks of 32 weights, d (f16) [m (f16)] [qh (u32)] and 16
// nibble bytes laid out as Q4_0's (low nibbles weights 0..15, high nibbles 16..31); bit j (16 + j) of qh is the
// fifth bit of weight j (16 + j).  Q4_1, Q5_1: w = d q + m, the m term through the activation block sums as Q4_K's
// min; Q5_0: w = d (q - 16), the offset folded into the integer sum as Q4_0's.  BB = bytes per block.
__device__ __forceinline__ uint32_t spread4_bits(uint32_t x) { return ((x & 0xFu) * 0x00204081u) & 0x01010101u; }
template <int MM, int BB, bool HAS_M, bool HAS_H> struct QUnitMmaBlk32 {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    // the 32-bit word at byte offset o (even) behind p
    __device__ static __forceinline__ uint32_t word(uint32_t p, uint32_t o) {
        return (o & 2u) ? __funnelshift_r(lds32(p + o - 2), lds32(p + o + 2), 16) : lds32(p + o);
    }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * (8 * BB) + 4 * BB * part, p8 = p0 + 8 * L.row_pitch;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            constexpr int OQ = 2 + (HAS_M ? 2 : 0) + (HAS_H ? 4 : 0);
            const uint32_t o = BB * b;
            const uint32_t h0 = word(p0, o), h8 = word(p8, o);                   // d (and m) of rows r and r + 8
            const float d0 = f16_bits_to_f32(h0 & 0xFFFFu), d8 = f16_bits_to_f32(h8 & 0xFFFFu);
            const uint32_t q0 = word(p0, o + OQ + 4 * t), q8 = word(p8, o + OQ + 4 * t);
            uint32_t a0 = q0 & 0x0F0F0F0Fu, a2 = (q0 >> 4) & 0x0F0F0F0Fu;
            uint32_t a1 = q8 & 0x0F0F0F0Fu, a3 = (q8 >> 4) & 0x0F0F0F0Fu;
            if (HAS_H) {
                const uint32_t g0 = word(p0, o + OQ - 4), g8 = word(p8, o + OQ - 4);
                a0 |= spread4_bits(g0 >> (4 * t)) << 4; a2 |= spread4_bits(g0 >> (16 + 4 * t)) << 4;
                a1 |= spread4_bits(g8 >> (4 * t)) << 4; a3 |= spread4_bits(g8 >> (16 + 4 * t)) << 4;
            }
#pragma unroll
            for (int gq = 0; gq < MMG; ++gq) {
                const uint2 bb = lds64(fb + (b * MMG + gq) * 256);
                const uint2 sc = lds64(sb + (b * MMG + gq) * 32);
                int c[4];
                imma_u8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                const float s = __uint_as_float(sc.x);
                if (HAS_M) {
                    const float sxf = __uint_as_float(sc.y);                       // scale * sum(X)
                    const float m0 = f16_bits_to_f32(h0 >> 16), m8 = f16_bits_to_f32(h8 >> 16);
                    tot[2 * gq] = fmaf(d0 * s, (float)(c[0] * 128 + c[1]), fmaf(m0, sxf, tot[2 * gq]));
                    tot[2 * gq + 1] = fmaf(d8 * s, (float)(c[2] * 128 + c[3]), fmaf(m8, sxf, tot[2 * gq + 1]));
                } else {
                    const int sx = (int)sc.y;                                      // -16 * sum(X)
                    tot[2 * gq] = fmaf(d0 * s, (float)(c[0] * 128 + c[1] + sx), tot[2 * gq]);
                    tot[2 * gq + 1] = fmaf(d8 * s, (float)(c[2] * 128 + c[3] + sx), tot[2 * gq + 1]);
                }
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};
template <int MM> struct QUnitMma<RLXQ_Q4_1, MM> : QUnitMmaBlk32<MM, 20, true, false> {};
template <int MM> struct QUnitMma<RLXQ_Q5_0, MM> : QUnitMmaBlk32<MM, 22, false, true> {};
template <int MM> struct QUnitMma<RLXQ_Q5_1, MM> : QUnitMmaBlk32<MM, 24, true, true> {};

// ---- Q8_0: the quants are the A fragment as they are (s8 x s8).  Blocks are 34 bytes: an even block of
// the unit starts on a word (d, then the quants from byte 2: two words funnel-shifted per fragment
// register), an odd one two bytes into a word (quants aligned).
template <int MM> struct QUnitMma<RLXQ_Q8_0, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * 272 + 136 * part, p8 = p0 + 8 * L.row_pitch;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t o = 68 * (b >> 1) + 32 * (b & 1);       // the word that holds d
            uint32_t a0, a1, a2, a3, dw0, dw8;
            if (b & 1) {
                dw0 = lds32(p0 + o) >> 16;
                dw8 = lds32(p8 + o) >> 16;
                a0 = lds32(p0 + o + 4 + 4 * t);  a2 = lds32(p0 + o + 20 + 4 * t);
                a1 = lds32(p8 + o + 4 + 4 * t);  a3 = lds32(p8 + o + 20 + 4 * t);
            } else {
                dw0 = lds32(p0 + o) & 0xFFFFu;
                dw8 = lds32(p8 + o) & 0xFFFFu;
                a0 = __funnelshift_r(lds32(p0 + o + 4 * t), lds32(p0 + o + 4 * t + 4), 16);
                a2 = __funnelshift_r(lds32(p0 + o + 16 + 4 * t), lds32(p0 + o + 20 + 4 * t), 16);
                a1 = __funnelshift_r(lds32(p8 + o + 4 * t), lds32(p8 + o + 4 * t + 4), 16);
                a3 = __funnelshift_r(lds32(p8 + o + 16 + 4 * t), lds32(p8 + o + 20 + 4 * t), 16);
            }
            const float d0 = f16_bits_to_f32(dw0), d8 = f16_bits_to_f32(dw8);
#pragma unroll
            for (int gq = 0; gq < MMG; ++gq) {
                const uint2 bb = lds64(fb + (b * MMG + gq) * 256);
                const float s = ldsf(sb + (b * MMG + gq) * 32);
                int c[4];
                imma_s8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                tot[2 * gq] = fmaf(d0 * s, (float)(c[0] * 128 + c[1]), tot[2 * gq]);
                tot[2 * gq + 1] = fmaf(d8 * s, (float)(c[2] * 128 + c[3]), tot[2 * gq + 1]);
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q4_K: a pair of sub-blocks shares 32 bytes (low nibbles: the first, high: the second); words t and
// 4 + t of the pair are the two k-halves of lane t's fragment for both.  The warp's part of the unit is
// four sub-blocks = one word of 6-bit scales and one of mins per tile row.  The second entry of an
// activation block's pair is the float s_b * sum(X): the min term is dmin * m * that.
template <int MM> struct QUnitMma<RLXQ_Q4_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void header(uint32_t p, uint32_t part, float& d, float& dmin, uint32_t& scb, uint32_t& mnb) {
        const uint4 hd = lds128(p);                   // d, dmin, 12 scale bytes
        d = f16_bits_to_f32(hd.x & 0xFFFFu);
        dmin = f16_bits_to_f32(hd.x >> 16);
        if (part == 0) {
            scb = hd.y & 0x3F3F3F3Fu;
            mnb = hd.z & 0x3F3F3F3Fu;
        } else {
            scb = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mnb = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
        }
    }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * 144, p8 = p0 + 8 * L.row_pitch;
        float d0, m0, d8, m8;
        uint32_t sc0, mn0, sc8, mn8;
        header(p0, part, d0, m0, sc0, mn0);
        header(p8, part, d8, m8, sc8, mn8);
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
            const uint32_t qo = 16 + 64 * part + 32 * pp + 4 * t;
            const uint32_t w0 = lds32(p0 + qo), w0b = lds32(p0 + qo + 16);
            const uint32_t w8 = lds32(p8 + qo), w8b = lds32(p8 + qo + 16);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int js = 2 * pp + nib;          // sub-block inside the warp's part
                const uint32_t a0 = (w0 >> (4 * nib)) & 0x0F0F0F0Fu, a2 = (w0b >> (4 * nib)) & 0x0F0F0F0Fu;
                const uint32_t a1 = (w8 >> (4 * nib)) & 0x0F0F0F0Fu, a3 = (w8b >> (4 * nib)) & 0x0F0F0F0Fu;
                const float dsc0 = d0 * (float)((sc0 >> (8 * js)) & 0xFFu), dmn0 = m0 * (float)((mn0 >> (8 * js)) & 0xFFu);
                const float dsc8 = d8 * (float)((sc8 >> (8 * js)) & 0xFFu), dmn8 = m8 * (float)((mn8 >> (8 * js)) & 0xFFu);
#pragma unroll
                for (int gq = 0; gq < MMG; ++gq) {
                    const uint2 bb = lds64(fb + (js * MMG + gq) * 256);
                    const uint2 sc = lds64(sb + (js * MMG + gq) * 32);
                    int c[4];
                    imma_u8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                    const float s = __uint_as_float(sc.x), sxf = __uint_as_float(sc.y);
                    tot[2 * gq] = fmaf(dsc0 * s, (float)(c[0] * 128 + c[1]), fmaf(-dmn0, sxf, tot[2 * gq]));
                    tot[2 * gq + 1] = fmaf(dsc8 * s, (float)(c[2] * 128 + c[3]), fmaf(-dmn8, sxf, tot[2 * gq + 1]));
                }
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q5_K: Q4_K with a fifth bit: the unit is d | dmin | 12 scale bytes | qh[32] | qs[128], and bit j of qh[l]
// adds 16 to weight l of sub-block j.  Words t and 4 + t of qh hold lane t's bits for every sub-block.
template <int MM> struct QUnitMma<RLXQ_Q5_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * 176, p8 = p0 + 8 * L.row_pitch;
        float d0, m0, d8, m8;
        uint32_t sc0, mn0, sc8, mn8;
        QUnitMma<RLXQ_Q4_K, MM>::header(p0, part, d0, m0, sc0, mn0);
        QUnitMma<RLXQ_Q4_K, MM>::header(p8, part, d8, m8, sc8, mn8);
        // the four high bits this part needs, moved to bits 0..3 of every byte
        const uint32_t hs = 4 * part;
        const uint32_t h0 = (lds32(p0 + 16 + 4 * t) >> hs) & 0x0F0F0F0Fu, h0b = (lds32(p0 + 32 + 4 * t) >> hs) & 0x0F0F0F0Fu;
        const uint32_t h8 = (lds32(p8 + 16 + 4 * t) >> hs) & 0x0F0F0F0Fu, h8b = (lds32(p8 + 32 + 4 * t) >> hs) & 0x0F0F0F0Fu;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
            const uint32_t qo = 48 + 64 * part + 32 * pp + 4 * t;
            const uint32_t w0 = lds32(p0 + qo), w0b = lds32(p0 + qo + 16);
            const uint32_t w8 = lds32(p8 + qo), w8b = lds32(p8 + qo + 16);
#pragma unroll
            for (int nib = 0; nib < 2; ++nib) {
                const int js = 2 * pp + nib;          // sub-block inside the warp's part
                const uint32_t a0 = ((w0 >> (4 * nib)) & 0x0F0F0F0Fu) | (((h0 >> js) & 0x01010101u) << 4);
                const uint32_t a2 = ((w0b >> (4 * nib)) & 0x0F0F0F0Fu) | (((h0b >> js) & 0x01010101u) << 4);
                const uint32_t a1 = ((w8 >> (4 * nib)) & 0x0F0F0F0Fu) | (((h8 >> js) & 0x01010101u) << 4);
                const uint32_t a3 = ((w8b >> (4 * nib)) & 0x0F0F0F0Fu) | (((h8b >> js) & 0x01010101u) << 4);
                const float dsc0 = d0 * (float)((sc0 >> (8 * js)) & 0xFFu), dmn0 = m0 * (float)((mn0 >> (8 * js)) & 0xFFu);
                const float dsc8 = d8 * (float)((sc8 >> (8 * js)) & 0xFFu), dmn8 = m8 * (float)((mn8 >> (8 * js)) & 0xFFu);
#pragma unroll
                for (int gq = 0; gq < MMG; ++gq) {
                    const uint2 bb = lds64(fb + (js * MMG + gq) * 256);
                    const uint2 sc = lds64(sb + (js * MMG + gq) * 32);
                    int c[4];
                    imma_u8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                    const float s = __uint_as_float(sc.x), sxf = __uint_as_float(sc.y);
                    tot[2 * gq] = fmaf(dsc0 * s, (float)(c[0] * 128 + c[1]), fmaf(-dmn0, sxf, tot[2 * gq]));
                    tot[2 * gq + 1] = fmaf(dsc8 * s, (float)(c[2] * 128 + c[3]), fmaf(-dmn8, sxf, tot[2 * gq + 1]));
                }
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

__device__ __forceinline__ void imma16_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// ---- Q6_K: 16-weight sub-blocks with an int8 scale each, so the MMA is the k = 16 shape, two per 32-weight
// group (the B fragment's b0 and b1 serve one each).  The warp's part of the unit is one half of the super-block:
// ql words t, 4+t, 8+t, 12+t and qh words t, 4+t of the half hold lane t's bytes of all four groups (low / high
// nibble of ql[l] and ql[l+32], two bits of qh[l] each).  The six-bit quants go in unsigned; the -32 comes from
// the block sums of 16 activations.  Both sub-blocks of a group share d and the activation scale, so their int8
// scales are applied in integers (|sum| < 2^31) and one conversion and one FMA finish the group.  A unit starts
// 2 bytes off a word when its index is odd: words are read from the aligned address below and funnel-shifted.
template <int MM> struct QUnitMma<RLXQ_Q6_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    // word i (0 .. n-1, 4 bytes apart from byte offset `off` of the unit) for this lane's row
    template <int N>
    __device__ static __forceinline__ void words(uint32_t pa, uint32_t off, uint32_t stride, uint32_t sh, bool odd, uint32_t (&w)[N]) {
        if (odd) {
#pragma unroll
            for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(lds32(pa + off + stride * i), lds32(pa + off + stride * i + 4), sh);
        } else {
#pragma unroll
            for (int i = 0; i < N; ++i) w[i] = lds32(pa + off + stride * i);
        }
    }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const bool odd = u & 1u;
        const uint32_t sh = odd ? 16u : 0u;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 64) + t * 16;
        uint32_t ql[2][4], qh[2][2], scw[2][2];
        float d[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t pa = L.row + 8 * r * L.row_pitch + u * 210 - (odd ? 2u : 0u);
            words<4>(pa, 64 * part + 4 * t, 16, sh, odd, ql[r]);
            words<2>(pa, 128 + 32 * part + 4 * t, 16, sh, odd, qh[r]);
            words<2>(pa, 192 + 8 * part, 4, sh, odd, scw[r]);
            d[r] = f16_bits_to_f32((lds32(pa + 208) >> sh) & 0xFFFFu);
        }
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {               // the four 32-weight groups of the half
            uint32_t a[2][2];                          // [sub-block][row]
#pragma unroll
            for (int sbk = 0; sbk < 2; ++sbk)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t lo = (ql[r][2 * (gq & 1) + sbk] >> (4 * (gq >> 1))) & 0x0F0F0F0Fu;
                    const uint32_t hv = qh[r][sbk];
                    const uint32_t hi = (gq < 2 ? (hv << (4 - 2 * gq)) : (hv >> (2 * gq - 4))) & 0x30303030u;
                    a[sbk][r] = lo | hi;
                }
            int sc[2][2];                              // [sub-block][row]
#pragma unroll
            for (int sbk = 0; sbk < 2; ++sbk)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int si = 2 * gq + sbk;
                    sc[sbk][r] = (int)(int8_t)((scw[r][si >> 2] >> (8 * (si & 3))) & 0xFFu);
                }
#pragma unroll
            for (int g2 = 0; g2 < MMG; ++g2) {
                const uint2 bb = lds64(fb + (gq * MMG + g2) * 256);
                const uint4 se = lds128(sb + (gq * MMG + g2) * 64);      // scale, -32 * sum of 16, -32 * sum of the next 16
                int c0[4], c1[4];
                imma16_u8s8(c0, a[0][0], a[0][1], bb.x);
                imma16_u8s8(c1, a[1][0], a[1][1], bb.y);
                const float s = __uint_as_float(se.x);
                const int v0 = (c0[0] * 128 + c0[1] + (int)se.y) * sc[0][0] + (c1[0] * 128 + c1[1] + (int)se.z) * sc[1][0];
                const int v8 = (c0[2] * 128 + c0[3] + (int)se.y) * sc[0][1] + (c1[2] * 128 + c1[3] + (int)se.z) * sc[1][1];
                tot[2 * g2] = fmaf(d[0] * s, (float)v0, tot[2 * g2]);
                tot[2 * g2 + 1] = fmaf(d[1] * s, (float)v8, tot[2 * g2 + 1]);
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q8_K: f32 d, then 256 int8 quants in order (the 16 block sums behind them are not read): the quants are the
// A fragment as they are, word-aligned.
template <int MM> struct QUnitMma<RLXQ_Q8_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t p0 = L.row + u * 292, p8 = p0 + 8 * L.row_pitch;
        const float d0 = ldsf(p0), d8 = ldsf(p8);
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 32) + t * 8;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t o = 4 + 128 * part + 32 * b + 4 * t;
            const uint32_t a0 = lds32(p0 + o), a2 = lds32(p0 + o + 16), a1 = lds32(p8 + o), a3 = lds32(p8 + o + 16);
#pragma unroll
            for (int gq = 0; gq < MMG; ++gq) {
                const uint2 bb = lds64(fb + (b * MMG + gq) * 256);
                const float s = ldsf(sb + (b * MMG + gq) * 32);
                int c[4];
                imma_s8s8(c, a0, a1, a2, a3, bb.x, bb.y);
                tot[2 * gq] = fmaf(d0 * s, (float)(c[0] * 128 + c[1]), tot[2 * gq]);
                tot[2 * gq + 1] = fmaf(d8 * s, (float)(c[2] * 128 + c[3]), tot[2 * gq + 1]);
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q2_K as the reference reads it: d, dmin, 16 bytes of (scale | min << 4), 64 quant bytes.  A half of the
// super-block is 32 bytes holding four 2-bit planes of 32 weights; every 16 weights have their own 4-bit scale and
// min, so the MMA is the k = 16 shape.  Scales and mins multiply the integer sums (dot products, and the sums of
// 16 activations that come with the fragments); d and dmin times the activation scale finish a group of 32.
template <int MM> struct QUnitMma<RLXQ_Q2_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        const uint32_t t = L.lane & 3u;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 64) + t * 16;
        uint32_t q[2][2], scw[2][2];
        float d[2], dm[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t p = L.row + 8 * r * L.row_pitch + u * 84;
            const uint32_t hd = lds32(p);
            d[r] = f16_bits_to_f32(hd & 0xFFFFu);
            dm[r] = f16_bits_to_f32(hd >> 16);
            scw[r][0] = lds32(p + 4 + 8 * part);
            scw[r][1] = lds32(p + 8 + 8 * part);
            q[r][0] = lds32(p + 20 + 32 * part + 4 * t);
            q[r][1] = lds32(p + 36 + 32 * part + 4 * t);
        }
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {               // the four 2-bit planes of the half
            uint32_t a[2][2];                          // [sub-block][row]
            int sc[2][2], mn[2][2];
#pragma unroll
            for (int sbk = 0; sbk < 2; ++sbk)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    a[sbk][r] = (q[r][sbk] >> (2 * gq)) & 0x03030303u;
                    const int si = 2 * gq + sbk;
                    const uint32_t byte = (scw[r][si >> 2] >> (8 * (si & 3))) & 0xFFu;
                    sc[sbk][r] = (int)(byte & 0xFu);
                    mn[sbk][r] = (int)(byte >> 4);
                }
#pragma unroll
            for (int g2 = 0; g2 < MMG; ++g2) {
                const uint2 bb = lds64(fb + (gq * MMG + g2) * 256);
                const uint4 se = lds128(sb + (gq * MMG + g2) * 64);      // scale, sum of 16, sum of the next 16
                int c0[4], c1[4];
                imma16_u8s8(c0, a[0][0], a[0][1], bb.x);
                imma16_u8s8(c1, a[1][0], a[1][1], bb.y);
                const float s = __uint_as_float(se.x);
                const int v0 = (c0[0] * 128 + c0[1]) * sc[0][0] + (c1[0] * 128 + c1[1]) * sc[1][0];
                const int v8 = (c0[2] * 128 + c0[3]) * sc[0][1] + (c1[2] * 128 + c1[3]) * sc[1][1];
                const int m0 = (int)se.y * mn[0][0] + (int)se.z * mn[1][0];
                const int m8 = (int)se.y * mn[0][1] + (int)se.z * mn[1][1];
                tot[2 * g2] = fmaf(d[0] * s, (float)v0, fmaf(-dm[0] * s, (float)m0, tot[2 * g2]));
                tot[2 * g2 + 1] = fmaf(d[1] * s, (float)v8, fmaf(-dm[1] * s, (float)m8, tot[2 * g2 + 1]));
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// ---- Q3_K as the reference reads it: d, 12 bytes of sixteen 6-bit scales, 32 high-mask bytes, 64 quant bytes.  A
// weight is its 2-bit plane value, minus 4 unless its mask bit is set, times d * (scale - 32): the quants go in as
// 2 bits + 4 * mask bit (0 .. 7) and the -4 comes from the sums of 16 activations.  A unit starts 2 bytes off a
// word when its index is odd.
template <int MM> struct QUnitMma<RLXQ_Q3_K, MM> {
    static_assert(MM == 4 || MM == 8, "groups of four activation rows");
    static constexpr int NT = 1, NACC = MM, MMG = MM / 4;
    static constexpr bool HALF_OFFSETS = false;
    __device__ static __forceinline__ uint32_t first_row(uint32_t lane) { return lane >> 2; }
    __device__ static __forceinline__ void run(const QLane& L, uint32_t u, uint32_t kb, float (&tot)[MM], uint32_t part) {
        using W = QUnitMma<RLXQ_Q6_K, MM>;             // its word loader: aligned words, funnel-shifted for odd units
        const uint32_t t = L.lane & 3u;
        const bool odd = u & 1u;
        const uint32_t sh = odd ? 16u : 0u;
        const uint32_t fb = L.xh + ((kb >> 5) + 4 * part) * (MMG * 256) + L.lane * 8;
        const uint32_t sb = L.sb + ((kb >> 5) + 4 * part) * (MMG * 64) + t * 16;
        uint32_t q[2][2], hm[2][2], scw[2][2];
        float d[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t pa = L.row + 8 * r * L.row_pitch + u * 110 - (odd ? 2u : 0u);
            // bytes 0..15 of the unit: d, the 12 scale bytes, two mask bytes
            uint32_t hd[4];
            W::template words<4>(pa, 0, 4, sh, odd, hd);
            d[r] = f16_bits_to_f32(hd[0] & 0xFFFFu);
            const uint32_t aux0 = __funnelshift_r(hd[0], hd[1], 16), aux1 = __funnelshift_r(hd[1], hd[2], 16),
                           tmp = __funnelshift_r(hd[2], hd[3], 16);
            // the eight scales of this half, one per byte (rlx-gguf/src/lib.rs:897-911)
            if (part == 0) {
                scw[r][0] = (aux0 & 0x0F0F0F0Fu) | ((tmp & 0x03030303u) << 4);
                scw[r][1] = (aux1 & 0x0F0F0F0Fu) | (((tmp >> 2) & 0x03030303u) << 4);
            } else {
                scw[r][0] = ((aux0 >> 4) & 0x0F0F0F0Fu) | (((tmp >> 4) & 0x03030303u) << 4);
                scw[r][1] = ((aux1 >> 4) & 0x0F0F0F0Fu) | (((tmp >> 6) & 0x03030303u) << 4);
            }
            // the mask (byte 14) and the quants (byte 46) sit 2 mod 4 inside the unit: aligned in an odd unit,
            // funnel-shifted from the word below in an even one
            W::template words<2>(pa, (odd ? 16u : 12u) + 4 * t, 16, 16u, !odd, hm[r]);
            W::template words<2>(pa, (odd ? 48u : 44u) + 32 * part + 4 * t, 16, 16u, !odd, q[r]);
        }
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
            uint32_t a[2][2];
            int sc[2][2];
#pragma unroll
            for (int sbk = 0; sbk < 2; ++sbk)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t lo = (q[r][sbk] >> (2 * gq)) & 0x03030303u;
                    const uint32_t hb = (hm[r][sbk] >> (4 * part + gq)) & 0x01010101u;
                    a[sbk][r] = lo | (hb << 2);
                    const int si = 2 * gq + sbk;
                    sc[sbk][r] = (int)((scw[r][si >> 2] >> (8 * (si & 3))) & 0xFFu) - 32;
                }
#pragma unroll
            for (int g2 = 0; g2 < MMG; ++g2) {
                const uint2 bb = lds64(fb + (gq * MMG + g2) * 256);
                const uint4 se = lds128(sb + (gq * MMG + g2) * 64);      // scale, -4 * sum of 16, -4 * sum of the next 16
                int c0[4], c1[4];
                imma16_u8s8(c0, a[0][0], a[0][1], bb.x);
                imma16_u8s8(c1, a[1][0], a[1][1], bb.y);
                const float s = __uint_as_float(se.x);
                const int v0 = (c0[0] * 128 + c0[1] + (int)se.y) * sc[0][0] + (c1[0] * 128 + c1[1] + (int)se.z) * sc[1][0];
                const int v8 = (c0[2] * 128 + c0[3] + (int)se.y) * sc[0][1] + (c1[2] * 128 + c1[3] + (int)se.z) * sc[1][1];
                tot[2 * g2] = fmaf(d[0] * s, (float)v0, tot[2 * g2]);
                tot[2 * g2 + 1] = fmaf(d[1] * s, (float)v8, tot[2 * g2 + 1]);
            }
        }
    }
    __device__ static __forceinline__ void finalize(float (&tot)[MM], uint32_t lane) { mma_rows_to_lanes<MM>(tot, lane); }
};

// What the per-block integer sums are multiplied by before they are stored.
template <uint32_t SCHEME> struct SumBias;
template <> struct SumBias<RLXQ_Q4_0> { static constexpr int value = -8; };
template <> struct SumBias<RLXQ_Q8_0> { static constexpr int value = 0; };
template <> struct SumBias<RLXQ_Q4_K> { static constexpr int value = 1; };
template <> struct SumBias<RLXQ_Q5_K> { static constexpr int value = 1; };
template <> struct SumBias<RLXQ_Q6_K> { static constexpr int value = -32; };
template <> struct SumBias<RLXQ_Q8_K> { static constexpr int value = 0; };
template <> struct SumBias<RLXQ_Q2_K> { static constexpr int value = 1; };
template <> struct SumBias<RLXQ_Q3_K> { static constexpr int value = -4; };
template <> struct SumBias<RLXQ_Q4_1> { static constexpr int value = 1; };
template <> struct SumBias<RLXQ_Q5_0> { static constexpr int value = -16; };
template <> struct SumBias<RLXQ_Q5_1> { static constexpr int value = 1; };
// Whether the fragment-ordered activations carry the block sum as the float s_b * bias * sum(X) (formats
// with a min term) or as the integer bias * sum(X) (added to the dot product before it is converted).
constexpr bool frag_sum_is_float(uint32_t scheme) {
    return scheme == RLXQ_Q4_K || scheme == RLXQ_Q5_K || scheme == RLXQ_Q4_1 || scheme == RLXQ_Q5_1;
}

// ---------------------------------------------------------------------------------------------
// Kernel 1: activations -> two int8 limbs + per-32 scale + per-SUB integer sums (workspace).
// One thread per 8 values; the scale is local to a 32-value block (four lanes).
// ---------------------------------------------------------------------------------------------
// 16-byte global load that stays where it is written relative to the other asm statements (the
// single-kernel mode wants its activation loads in the memory queue ahead of the weight requests).
__device__ __forceinline__ uint4 ldg128_here(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// The raw 32 bytes (f32) or 16 bytes (bf16) of the eight activations x[r][c .. c+8).
__device__ __forceinline__ void load_raw8(const void* __restrict__ x, uint32_t x_bf16, uint32_t k, uint32_t r,
                                          uint32_t c, uint4 (&raw)[2]) {
    if (x_bf16) {
        raw[0] = ldg128_here(reinterpret_cast<const uint16_t*>(x) + (size_t)r * k + c);
    } else {
        const float* p = reinterpret_cast<const float*>(x) + (size_t)r * k + c;
        raw[0] = ldg128_here(p);
        raw[1] = ldg128_here(p + 4);
    }
}
__device__ __forceinline__ void raw8_to_f32(const uint4 (&raw)[2], uint32_t x_bf16, float (&f)[8]) {
    if (x_bf16) {
        const uint32_t wv[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            f[2 * q] = __uint_as_float(wv[q] << 16);
            f[2 * q + 1] = __uint_as_float(wv[q] & 0xFFFF0000u);
        }
    } else {
        f[0] = __uint_as_float(raw[0].x); f[1] = __uint_as_float(raw[0].y); f[2] = __uint_as_float(raw[0].z); f[3] = __uint_as_float(raw[0].w);
        f[4] = __uint_as_float(raw[1].x); f[5] = __uint_as_float(raw[1].y); f[6] = __uint_as_float(raw[1].z); f[7] = __uint_as_float(raw[1].w);
    }
}

// Reads the eight activations x[r][c .. c+8) (f32 or bf16) as f32.
__device__ __forceinline__ void load_group8(const void* __restrict__ x, uint32_t x_bf16, uint32_t k, uint32_t r,
                                            uint32_t c, float (&f)[8]) {
    if (x_bf16) {
        const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (size_t)r * k + c);
        const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            f[2 * q] = __uint_as_float(wv[q] << 16);
            f[2 * q + 1] = __uint_as_float(wv[q] & 0xFFFF0000u);
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)r * k + c);
        const float4 a = p[0], b = p[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
}

// The SwiGLU form: x is [m][2k] f32 = [gate | up] of an FFN and the activation is up * silu(gate)
// (rlx-cpu/src/naive.rs:54-56, rlx-cuda/src/unfuse.rs:254-293), formed here instead of in a kernel of its own.
__device__ __forceinline__ void load_group8_swiglu(const void* __restrict__ x, uint32_t k, uint32_t r, uint32_t c,
                                                   float (&f)[8]) {
    const float* row = reinterpret_cast<const float*>(x) + (size_t)r * 2 * k;
    const float4 g0 = *reinterpret_cast<const float4*>(row + c), g1 = *reinterpret_cast<const float4*>(row + c + 4);
    const float4 u0 = *reinterpret_cast<const float4*>(row + k + c), u1 = *reinterpret_cast<const float4*>(row + k + c + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
    for (int q = 0; q < 8; ++q) f[q] = u[q] * (g[q] / (1.0f + expf(-g[q])));
}

// Quantises eight activations (columns c .. c+8 of a row) into row_dst
// ([h: k][l: k][s_b: k/32 f32][sums: k/SUB i32]).  The four lanes 4j .. 4j+3 of a warp must hold the
// four groups of one 32-value block.
template <uint32_t SUB>
__device__ __forceinline__ void quantise_store8(const float (&f)[8], uint32_t k, int bias, uint32_t c,
                                                uint8_t* row_dst, uint32_t lane) {
    float amax = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const bool ok = amax > 0.f && amax < 3.0e38f;
    const float inv = ok ? 16256.0f / amax : 0.f;
    const float s = ok ? amax * (1.0f / 16256.0f) : 0.f;
    int sum = 0;
    uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int X = max(-16256, min(16256, __float2int_rn(f[q] * inv)));
        sum += X;
        const int hq = (X + 64) >> 7;             // in [-127, 127]
        const int lq = X - (hq << 7);             // in [-64, 63]
        hw[q >> 2] |= ((uint32_t)hq & 0xFFu) << (8 * (q & 3));
        lw[q >> 2] |= ((uint32_t)lq & 0xFFu) << (8 * (q & 3));
    }
    *reinterpret_cast<uint2*>(row_dst + c) = make_uint2(hw[0], hw[1]);
    *reinterpret_cast<uint2*>(row_dst + k + c) = make_uint2(lw[0], lw[1]);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if (SUB == 32) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    float* sb = reinterpret_cast<float*>(row_dst + 2 * (size_t)k);
    int* sx = reinterpret_cast<int*>(row_dst + 2 * (size_t)k + (size_t)(k / 32) * 4);
    if ((lane & 3u) == 0) sb[c / 32] = s;
    if ((lane & (SUB / 8 - 1)) == 0) sx[c / SUB] = bias * sum;
}

// The same quantisation, stored in the fragment order of the integer-MMA units: dst = [block][MMG groups
// of four rows][lane]{b0, b1} and, from byte frag_scale_offset(k, MMG) on, [block][row]{scale, bias * sum}.
// Column 2 (r & 3) + limb of the MMA's B operand is (activation row r, limb); lane 4 col + t holds k = 4t ..
// 4t+3 in b0 and k = 16+4t .. in b1.
template <int MMG, bool FSUM, uint32_t SUB>
__device__ __forceinline__ void quantise_store8_frag(const float (&f)[8], uint32_t k, int bias, uint32_t r, uint32_t c,
                                                     uint8_t* dst, uint32_t lane) {
    float amax = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) amax = fmaxf(amax, fabsf(f[q]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const bool ok = amax > 0.f && amax < 3.0e38f;
    const float inv = ok ? 16256.0f / amax : 0.f;
    const float s = ok ? amax * (1.0f / 16256.0f) : 0.f;
    int sum = 0;
    uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int X = max(-16256, min(16256, __float2int_rn(f[q] * inv)));
        sum += X;
        const int hq = (X + 64) >> 7;             // in [-127, 127]
        const int lq = X - (hq << 7);             // in [-64, 63]
        hw[q >> 2] |= ((uint32_t)hq & 0xFFu) << (8 * (q & 3));
        lw[q >> 2] |= ((uint32_t)lq & 0xFFu) << (8 * (q & 3));
    }
    const uint32_t blk = c >> 5, j = (c >> 3) & 3u;                  // the block, and which eight of its 32 values
    const uint32_t half = j >> 1, t0 = 2u * (j & 1u), col = 2u * (r & 3u);
    uint32_t* fr = reinterpret_cast<uint32_t*>(dst + ((size_t)blk * MMG + (r >> 2)) * 256) + half;
    fr[2 * (4 * col + t0)] = hw[0];
    fr[2 * (4 * col + t0 + 1)] = hw[1];
    fr[2 * (4 * (col + 1) + t0)] = lw[0];
    fr[2 * (4 * (col + 1) + t0 + 1)] = lw[1];
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if constexpr (SUB == 16) {
        // lanes 0 and 2 of the block's four hold the sums of its two halves
        uint32_t* e = reinterpret_cast<uint32_t*>(dst + frag_scale_offset(k, MMG) + ((size_t)blk * MMG * 4 + r) * 16);
        if ((lane & 3u) == 0) { e[0] = __float_as_uint(s); e[1] = (uint32_t)(bias * sum); }
        if ((lane & 3u) == 2) e[2] = (uint32_t)(bias * sum);
    } else {
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if ((lane & 3u) == 0)
            *reinterpret_cast<uint2*>(dst + frag_scale_offset(k, MMG) + ((size_t)blk * MMG * 4 + r) * 8) =
                make_uint2(__float_as_uint(s), FSUM ? __float_as_uint(s * (float)(bias * sum)) : (uint32_t)(bias * sum));
    }
}

template <uint32_t SUB, int MMG = 0, bool FSUM = false>
__global__ void __launch_bounds__(256) quantise_x_kernel(const void* __restrict__ x, uint32_t x_bf16, uint32_t m,
                                                         uint32_t k, int bias, uint8_t* __restrict__ xq,
                                                         uint32_t xq_row_bytes, uint32_t* __restrict__ counters,
                                                         uint32_t ntiles, float* __restrict__ y_zero, uint32_t y_count,
                                                         uint32_t swiglu_pair, unsigned long long* __restrict__ tp_header,
                                                         uint32_t tp_arrivals) {
    griddep_launch_dependents();   // the streaming kernel may become resident and prefetch weights
    const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31u;
    griddep_wait();                // x (and the counters) may still be in use by the previous kernel
    if (tp_header && gtid == 0) {  // tensor-parallel push: one more step, tp_arrivals more CTAs expected from every rank
        tp_header[kCommWordEpoch] += 1ull;
        tp_header[kCommWordExpected] += tp_arrivals;
    }
    for (uint32_t i = gtid; i < ntiles; i += gridDim.x * blockDim.x) counters[i] = 0u;
    for (uint32_t i = gtid; i < y_count; i += gridDim.x * blockDim.x) y_zero[i] = 0.f;   // two-contributor add mode
    const uint32_t groups_per_row = k / 8;
    const uint32_t total = groups_per_row * m;          // a multiple of 32
    if (gtid >= total) return;                          // whole warps leave together
    const uint32_t r = gtid / groups_per_row, c = (gtid - r * groups_per_row) * 8;
    float f[8];
    if (swiglu_pair) load_group8_swiglu(x, k, r, c, f);
    else load_group8(x, x_bf16, k, r, c, f);
    if constexpr (MMG > 0) quantise_store8_frag<MMG, FSUM, SUB>(f, k, bias, r, c, xq, lane);   // fragment order (integer-MMA units)
    else quantise_store8<SUB>(f, k, bias, c, xq + (size_t)r * xq_row_bytes, lane);
}

// ---------------------------------------------------------------------------------------------
// Work list ("stream-K").  All (tile, chunk) items form one list, chunk-major inside a tile; the T
// items are dealt to the G CTAs as contiguous ranges of T/G items, the first T mod G ranges one
// longer, so every CTA streams the same number of bytes (+-1 chunk) whatever n and k are.  A range cuts at most two tiles: its head and its tail.  Those
// two shared segments are processed FIRST, the whole tiles between them afterwards, so that the
// latency of finishing a shared tile (a fence, an atomic, a re-read) hides behind streaming.
// ---------------------------------------------------------------------------------------------
struct Segment { uint32_t tile, c0, c1; };

// A CTA's range: its cut head tile (chunks head_c0 .. nchunks of tile head_tile) if has_head, its cut
// tail tile (chunks 0 .. tail_c1 of tile tail_tile) if has_tail, and nwhole whole tiles from first_whole.
struct Range { uint32_t len, has_head, has_tail, head_tile, head_c0, head_c1, tail_tile, tail_c1, first_whole, nseg, nshared; };

__device__ __forceinline__ Range make_range(const IntParams& P, uint32_t me) {
    // CTA i takes chunks [i*q + min(i, r), ...): the first r CTAs one chunk more (q, r from the host)
    Range rg;
    const uint32_t nc = P.nchunks;
    const uint32_t beg = me * P.chunks_q + min(me, P.chunks_r);
    const uint32_t end = beg + P.chunks_q + (me < P.chunks_r ? 1u : 0u);
    rg.len = end - beg;
    const uint32_t bt = beg / nc, et = end / nc;
    const uint32_t bc = beg - bt * nc, ec = end - et * nc;
    // head: from beg to the next tile boundary (or to end, for a range inside one tile), if beg is inside a tile
    const uint32_t head_end = bc ? min(end, (bt + 1) * nc) : beg;
    rg.has_head = bc ? 1u : 0u;
    rg.head_tile = bt;
    rg.head_c0 = bc;
    rg.head_c1 = head_end - bt * nc;
    // tail: from the last tile boundary to end, if end is inside a tile and past the head
    rg.has_tail = (ec && et * nc >= head_end) ? 1u : 0u;
    rg.tail_tile = et;
    rg.tail_c1 = ec;
    rg.first_whole = bc ? bt + 1 : bt;
    const uint32_t nwhole = et > rg.first_whole ? et - rg.first_whole : 0u;
    rg.nshared = rg.has_head + rg.has_tail;
    rg.nseg = rg.nshared + nwhole;
    return rg;
}
// The CTA whose range holds chunk g (the inverse of the split in make_range).
__device__ __forceinline__ uint32_t owner_of(const IntParams& P, uint32_t g) {
    const uint32_t big = P.chunks_r * (P.chunks_q + 1);
    return g < big ? g / (P.chunks_q + 1) : P.chunks_r + (g - big) / P.chunks_q;
}
__device__ __forceinline__ Segment segment_at(const IntParams& P, const Range& rg, uint32_t idx) {
    Segment sg;
    if (rg.has_head && idx == 0) { sg.tile = rg.head_tile; sg.c0 = rg.head_c0; sg.c1 = rg.head_c1; }
    else if (rg.has_tail && idx == rg.has_head) { sg.tile = rg.tail_tile; sg.c0 = 0; sg.c1 = rg.tail_c1; }
    else { sg.tile = rg.first_whole + (idx - rg.nshared); sg.c0 = 0; sg.c1 = P.nchunks; }
    return sg;
}

// Tail of a pushing down projection (one warp): wait, bounded, until every rank has counted all its CTAs in, then
// write outputs e0 .. e1 as the sum over ranks, in rank order, out of this rank's own buffer.  Kept out of line: its
// registers (eight outputs x eight ranks in flight) must not weigh on the kernel that calls it.
static __device__ __noinline__ void tp_wait_and_sum(const TpPush& tp, unsigned long long tp_expected, size_t tp_parity,
                                                    uint32_t e0, uint32_t e1, void* y, uint32_t y_bf16, int* err, uint32_t lane) {
    bool ok = true;
    if (lane < tp.world) {
        const unsigned long long* arr = reinterpret_cast<const unsigned long long*>(tp.buf[tp.rank]) + kCommWordArrive + lane;
        ok = false;
        for (uint32_t it = 0; it < tp.spin_limit; ++it) {
            unsigned long long seen;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(arr) : "memory");
            if (seen >= tp_expected) { ok = true; break; }
            __nanosleep(32);
        }
        if (!ok) atomicExch(err, 40 + (int)lane);
    }
    if (!__all_sync(0xFFFFFFFFu, ok)) return;
    const float* slots = reinterpret_cast<const float*>(tp.buf[tp.rank] + comm_push_offset(tp.max_elems)) + tp_parity;
    for (uint32_t c0 = e0; c0 < e1; c0 += 256u) {
        float part[8][kCommMaxWorld];
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t e = c0 + j * 32 + lane;
#pragma unroll
            for (uint32_t pr = 0; pr < kCommMaxWorld; ++pr) {
                part[j][pr] = 0.f;
                if (pr < tp.world && e < e1)
                    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(part[j][pr]) : "l"(slots + (size_t)pr * tp.max_elems + e) : "memory");
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t e = c0 + j * 32 + lane;
            float acc = 0.f;
#pragma unroll
            for (uint32_t pr = 0; pr < kCommMaxWorld; ++pr)
                if (pr < tp.world) acc += part[j][pr];
            if (e < e1) {
                if (y_bf16) reinterpret_cast<uint16_t*>(y)[e] = (uint16_t)f32_to_bf16_bits(acc);
                else reinterpret_cast<float*>(y)[e] = acc;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel 2: the streaming kernel
// ---------------------------------------------------------------------------------------------
template <uint32_t SCHEME, int MM, bool MMA = false, bool TP = false>
__global__ void __launch_bounds__(int_threads(MMA), (MMA || MM > 2) ? 1 : 2) gemv_int_kernel(const __grid_constant__ IntParams P) {
    constexpr uint32_t CW = int_warps(MMA), WPU = CW / kIntCU, RL = int_red_lanes(MMA);
    using T = StagedTraits<SCHEME>;
    using B = IntBox<SCHEME, MMA>;
    using QU = std::conditional_t<MMA, QUnitMma<SCHEME, MM>, QUnit<SCHEME, MM>>;
    constexpr uint32_t STRIDE = B::ROW;
    constexpr uint32_t stage_bytes = B::STAGE_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    // activations first, in the workspace's layout, one row after the other
    uint8_t* xs = smem;
    uint8_t* stages = smem + P.off_stage;
    float* red = reinterpret_cast<float*>(smem + P.off_red);          // [RB][8 warps][32 lanes][MM]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P.off_bar);   // full[NS], empty[NS], xbar
    const uint32_t NS = P.nstages;
    uint64_t* rbars = bars + 2 * NS + 1;                                // rfull[RB], rempty[RB]
    uint32_t* misc = reinterpret_cast<uint32_t*>(rbars + 2 * kIntRB);
    volatile uint32_t* abort_flag = misc;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    griddep_launch_dependents();
    if (tid == 0) tma_prefetch_desc(&P.wmap);

    const uint32_t G = gridDim.x, me = blockIdx.x;
    const Range rg = make_range(P, me);
    const uint32_t nseg = rg.nseg;
    const uint32_t ku = P.k / 256;

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[NS + s]), CW);
        }
        mbar_init(smem_u32(&bars[2 * NS]), 1);
        for (uint32_t r = 0; r < kIntRB; ++r) {
            mbar_init(smem_u32(&rbars[r]), CW);
            mbar_init(smem_u32(&rbars[kIntRB + r]), 1);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The first fill of the ring is spread over the warps, one stage each: a TMA request occupies its
    // issuing thread for a few hundred cycles, and one thread issuing them all delays the stream's start.
    const uint32_t pre = P.xstream ? 0u : min(min(NS, CW), rg.len);

    // expert-indirect mode: every role learns the slab after the dependency wait (nothing is requested
    // before it) and leaves at once when the id is out of range
    auto resolve_expert = [&](uint32_t& row_off) -> bool {
        row_off = 0u;
        if (!P.expert_sel) return true;
        griddep_wait();
        uint32_t e;
        if (!expert_of_row(*P.expert_sel, P.num_experts, &e)) return false;
        row_off = e * P.n;
        return true;
    };

    if (warp == CW) {
        // ---------------- producer warp ----------------
        uint32_t row_off;
        if (!resolve_expert(row_off)) return;
        auto produce = [&](uint32_t tile, uint32_t chunk, uint32_t s) {
            // rows past n and bytes past the row end arrive as zeros (d = 0: they add nothing)
            const uint32_t full = smem_u32(&bars[s]);
            if (lane == 0) {
                uint32_t xb_frag = 0, xb_scale = 0;
                if constexpr (MMA) {
                    if (P.xstream) {                  // this chunk's blocks of 32 activations: fragments and scale entries
                        const uint32_t blocks = min(kIntCU, ku - chunk * kIntCU) * 8u;
                        xb_frag = blocks * (MM / 4) * 256u;
                        xb_scale = blocks * (MM / 4) * 4u * frag_entry_bytes(T::SUB);
                    }
                }
                mbar_arrive_expect_tx(full, stage_bytes + xb_frag + xb_scale);
#pragma unroll
                for (uint32_t b = 0; b < B::NB; ++b)
                    tma_load_2d(smem_u32(stages + s * P.stage_stride + b * B::BOX_BYTES), &P.wmap,
                                (int32_t)(((chunk * kIntCU + b * B::UB) * T::UNIT_B) / 8), (int32_t)(row_off + tile * 16), full);
                if constexpr (MMA) {
                    if (P.xstream) {
                        constexpr uint32_t FC = kIntCU * 8u * (MM / 4) * 256u, SC = kIntCU * 8u * (MM / 4) * 4u * frag_entry_bytes(T::SUB);
                        const uint32_t dst = smem_u32(stages + s * P.stage_stride + stage_bytes);
                        bulk_g2s(dst, P.xq + (size_t)chunk * FC, xb_frag, full);
                        bulk_g2s(dst + FC, P.xq + frag_scale_offset(P.k, MM / 4) + (size_t)chunk * SC, xb_scale, full);
                    }
                }
            }
        };
        uint32_t s = 0, ph = 1, issued = 0;   // ph: parity to wait for on empty[s] (1 passes on a fresh barrier)
        bool waited = false, dead = false;
        if (P.xstream) {     // every stage carries activations: nothing can be requested before they exist
            waited = true;
            griddep_wait();
        }
        for (uint32_t si = 0; si < nseg && !dead; ++si) {
            const Segment sg = segment_at(P, rg, si);
            for (uint32_t c = sg.c0; c < sg.c1; ++c, ++issued) {
                if (issued == NS && !waited) {
                    // the ring is full of (immutable) weights: only now wait for the previous kernel
                    waited = true;
                    griddep_wait();
                    const uint32_t xbar = smem_u32(&bars[2 * NS]);
                    if (lane == 0 && !P.inline_q && !P.xstream) mbar_arrive_expect_tx(xbar, P.xq_row_bytes * P.xq_pieces);
                    __syncwarp();
                    if (lane < P.xq_pieces && !P.inline_q && !P.xstream)
                        bulk_g2s(smem_u32(xs + lane * P.xq_row_bytes), P.xq + (size_t)lane * P.xq_row_bytes, P.xq_row_bytes, xbar);
                }
                if (issued >= NS) {
                    if (*abort_flag || !mbar_wait(smem_u32(&bars[NS + s]), ph)) {
                        if (lane == 0) { atomicExch(P.err, 3); *abort_flag = 1u; }
                        dead = true;
                        break;
                    }
                }
                if (issued >= pre) produce(sg.tile, c, s);   // the first `pre` stages were requested by the consumer warps
                if (++s == NS) { s = 0; ph ^= 1u; }
            }
        }
        if (!waited) {   // fewer chunks than stages: everything is in flight, now fetch the activations
            griddep_wait();
            const uint32_t xbar = smem_u32(&bars[2 * NS]);
            if (lane == 0 && !P.inline_q && !P.xstream) mbar_arrive_expect_tx(xbar, P.xq_row_bytes * P.xq_pieces);
            __syncwarp();
            if (lane < P.xq_pieces && !P.inline_q && !P.xstream)
                bulk_g2s(smem_u32(xs + lane * P.xq_row_bytes), P.xq + (size_t)lane * P.xq_row_bytes, P.xq_row_bytes, xbar);
        }
        return;
    }

    if (warp == CW + 1) {
        // ---------------- finisher warp ----------------
        { uint32_t ro; if (!resolve_expert(ro)) return; }
        // Adds the 16 partials of every output (2 halves x 8 warps, fixed order) and writes the tile,
        // or, for a tile shared with other CTAs, runs the publish / count / re-read sequence.  That
        // sequence is a chain of three global round trips; here it delays nobody, because the
        // consumer warps only hand over a reduction buffer and go on.
        griddep_wait();
        // tensor-parallel push: which set of slots this step uses, and where this rank's slot starts in a buffer
        size_t tp_slot = 0, tp_parity = 0;
        unsigned long long tp_expected = 0ull;
        if constexpr (TP) {
            const unsigned long long* hdr = reinterpret_cast<const unsigned long long*>(P.tp.buf[P.tp.rank]);
            tp_parity = (size_t)(hdr[kCommWordEpoch] & 1ull) * kCommMaxWorld * P.tp.max_elems;
            tp_slot = tp_parity + (size_t)P.tp.rank * P.tp.max_elems;
            tp_expected = hdr[kCommWordExpected];
        }
        // a lane finishes tile row rrow of activation rows col = 2 cp + (lane >> 4), cp = 0 .. NC-1
        constexpr int NC = (MM + 1) / 2;
        const uint32_t chalf = lane >> 4, rrow = lane & 15u;
        uint32_t r = 0, rph = 0;
        for (uint32_t si = 0; si < nseg; ++si) {
            const Segment sg = segment_at(P, rg, si);
            const uint32_t tile = sg.tile, mine = sg.c1 - sg.c0;
            if (*abort_flag || !mbar_wait(smem_u32(&rbars[r]), rph)) {
                if (lane == 0) { atomicExch(P.err, 6); *abort_flag = 1u; }
                break;
            }
            const float* rbuf = red + r * (CW * RL * MM);
            float v[NC];
#pragma unroll
            for (int cp = 0; cp < NC; ++cp) {
                const uint32_t col = 2 * cp + chalf;
                v[cp] = 0.f;
                if (col < (uint32_t)MM) {
#pragma unroll
                    for (uint32_t wv = 0; wv < CW; ++wv) {
                        v[cp] += rbuf[(wv * RL + rrow) * MM + col];
                        if (RL == 32) v[cp] += rbuf[(wv * RL + 16 + rrow) * MM + col];
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&rbars[kIntRB + r]));
            if (++r == kIntRB) { r = 0; rph ^= 1u; }
            const uint32_t orow = tile * 16 + rrow;
            bool store = mine == P.nchunks;
            if (!store && P.inline_q) {
                // Exactly two CTAs share this tile: the one holding its first chunks (role 0) and the one
                // holding its last (role 1).  Each publishes its part and swaps its token into the tile's
                // word; the one that finds the other's token there came second and completes the tile.
                // The word may hold anything on entry: a token is unique to (call, role), so stale
                // contents are never mistaken for it, and the word is left at zero for a replay of the
                // same captured launch.
                const uint32_t role = sg.c0 ? 1u : 0u;
                float* pt = P.partial + (size_t)tile * 2 * (MM * 16);
#pragma unroll
                for (int cp = 0; cp < NC; ++cp)
                    if (2 * cp + chalf < (uint32_t)MM) pt[(role * MM + 2 * cp + chalf) * 16 + rrow] = v[cp];
                __threadfence();
                __syncwarp();
                unsigned long long old = 0ull;
                if (lane == 0) old = atomicExch(&P.flags[tile], P.token + 2ull * role);
                old = __shfl_sync(0xFFFFFFFFu, old, 0);
                if (old == P.token + 2ull * (1u - role)) {
                    __threadfence();
#pragma unroll
                    for (int cp = 0; cp < NC; ++cp)
                        if (2 * cp + chalf < (uint32_t)MM) v[cp] += __ldcg(&pt[((1u - role) * MM + 2 * cp + chalf) * 16 + rrow]);
                    if (lane == 0) P.flags[tile] = 0ull;
                    store = true;
                }
            } else if (!store && P.use_red) {
                // exactly two CTAs share this tile and y starts at zero: 0 + a + b = 0 + b + a, so a
                // plain reduction to memory is deterministic and needs no fence, counter or re-read
#pragma unroll
                for (int cp = 0; cp < NC; ++cp) {
                    const uint32_t col = 2 * cp + chalf;
                    if (col < P.m_real && orow < P.n) atomicAdd(reinterpret_cast<float*>(P.y) + (size_t)col * P.n + orow, v[cp]);
                }
            } else if (!store) {
                // the tile is shared with neighbouring CTAs: publish this part in the slot given by the
                // CTA's position among the tile's contributors; whoever completes the tile adds the slots
                const uint32_t first_owner = owner_of(P, tile * P.nchunks), last_owner = owner_of(P, (tile + 1) * P.nchunks - 1);
                float* pt = P.partial + ((size_t)tile * P.slots) * (MM * 16);
#pragma unroll
                for (int cp = 0; cp < NC; ++cp)
                    if (2 * cp + chalf < (uint32_t)MM) pt[((me - first_owner) * MM + 2 * cp + chalf) * 16 + rrow] = v[cp];
                __threadfence();
                __syncwarp();
                uint32_t prev = 0;
                if (lane == 0) prev = atomicAdd(&P.counters[tile], mine);
                prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
                if (prev + mine == P.nchunks) {
                    __threadfence();
#pragma unroll
                    for (int cp = 0; cp < NC; ++cp) {
                        const uint32_t col = 2 * cp + chalf;
                        v[cp] = 0.f;
                        if (col < (uint32_t)MM)
                            for (uint32_t sl = 0; sl <= last_owner - first_owner; ++sl)
                                v[cp] += __ldcg(&pt[(sl * MM + col) * 16 + rrow]);
                    }
                    store = true;
                }
            }
            if (store) {
#pragma unroll
                for (int cp = 0; cp < NC; ++cp) {
                    const uint32_t col = 2 * cp + chalf;
                    if (col < P.m_real && orow < P.n) {
                        const size_t o = (size_t)col * P.n + orow;
                        if constexpr (TP) {
#pragma unroll
                            for (uint32_t pr = 0; pr < kCommMaxWorld; ++pr)
                                if (pr < P.tp.world)
                                    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(reinterpret_cast<float*>(P.tp.buf[pr] + comm_push_offset(P.tp.max_elems)) + tp_slot + o),
                                                 "f"(v[cp]) : "memory");
                        } else if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(v[cp]);
                        else reinterpret_cast<float*>(P.y)[o] = v[cp];
                    }
                }
            }
        }
        if constexpr (TP) {
            // Everything this CTA pushes is out (a tile it shares is pushed by whoever completes it, before that
            // CTA counts itself in).  CTAs count in on this rank's own word; the one that completes the count tells
            // every rank, behind all of this rank's pushes, with one addition each.  (Every CTA adding at every rank
            // would put grid x world same-address reductions on the links, which serialise at the far L2.)
            __threadfence_system();
            __syncwarp();
            unsigned long long prev = 0ull;
            if (lane == 0)
                prev = atomicAdd(reinterpret_cast<unsigned long long*>(P.tp.buf[P.tp.rank]) + kCommWordLocal, 1ull);
            prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
            if (prev + 1ull == tp_expected) {
                __threadfence_system();
                if (lane < P.tp.world)
                    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long*>(P.tp.buf[lane]) + kCommWordArrive + P.tp.rank),
                                 "l"((unsigned long long)G) : "memory");
            }
            // A few CTAs stay for the sum, 256 outputs each; the others leave now, so that the next kernel's CTAs can
            // become resident and fetch their first weights while the exchange completes.
            const uint32_t total = P.m_real * P.n, per = max(256u, ((total + G - 1) / G + 31u) & ~31u);
            const uint32_t e0 = me * per, e1 = min(total, e0 + per);
            if (e0 >= total) return;
            tp_wait_and_sum(P.tp, tp_expected, tp_parity, e0, e1, P.y, P.y_bf16, P.err, lane);
        }
        return;
    }

    // ---------------- consumer warps: lane = (tile row, half of the unit) ----------------
    uint32_t row_off;
    if (!resolve_expert(row_off)) return;
    auto request_first_stage = [&](uint32_t w0, uint32_t w1) {
        if (warp >= w0 && warp < min(w1, pre) && lane == 0) {
            uint32_t i = warp, si = 0;
            Segment sg = segment_at(P, rg, 0);
            while (i >= sg.c1 - sg.c0) { i -= sg.c1 - sg.c0; sg = segment_at(P, rg, ++si); }
            const uint32_t full = smem_u32(&bars[warp]);
            mbar_arrive_expect_tx(full, stage_bytes);
#pragma unroll
            for (uint32_t b = 0; b < B::NB; ++b)
                tma_load_2d(smem_u32(stages + warp * P.stage_stride + b * B::BOX_BYTES), &P.wmap,
                            (int32_t)((((sg.c0 + i) * kIntCU + b * B::UB) * T::UNIT_B) / 8), (int32_t)(row_off + sg.tile * 16), full);
        }
    };
    // Two-kernel mode: the weights are requested before the dependency wait (they are immutable).  In
    // single-kernel mode the activations have to come through the same memory path first: requests
    // behind tens of KB of weight traffic per SM wait for microseconds, so the weights go second.
    const uint32_t early = P.inline_q ? P.early : pre;   // stages requested before the dependency wait
    request_first_stage(0, early);
    griddep_wait();
    QLane L;
    L.half = lane >> 4;
    L.xstride = P.xq_row_bytes;
    L.lane = lane;
    L.row_pitch = STRIDE;
    // formats mapped (row, half) read from their half's offset on; Q4_0 indexes by block instead
    const uint32_t hoff = QU::HALF_OFFSETS ? L.half : 0u;
    L.xh = smem_u32(xs) + 128 * hoff;
    L.xl = L.xh + P.k;
    L.sb = smem_u32(xs) + 2 * P.k + 16 * hoff;
    L.sx = smem_u32(xs) + 2 * P.k + (P.k / 32) * 4 + (32 / T::SUB) * 16 * hoff;
    if constexpr (MMA) L.sb = smem_u32(xs) + frag_scale_offset(P.k, MM / 4);   // fragments at xh, {scale, sum} pairs here
    const uint32_t trow = QU::first_row(lane), stages_u32 = smem_u32(stages);
    bool dead = false;
    if (P.inline_q) {
        {
            // every load is issued before the first value is used: one trip to L2, not one per group
            const uint32_t gpr = P.k / 8, total = gpr * P.m_real;   // whole warps stay together: gpr % 32 == 0
            constexpr uint32_t kInlineGroups = inline_groups(MM, MMA);
            // the i-th group of eight activations of this thread: row r, first column c (false: none)
            auto group_of = [&](uint32_t i, uint32_t& r, uint32_t& c) -> bool {
                if constexpr (MMA) {
                    // A warp takes 1, 2 or 4 activation rows (m_real 1, 2, 3+) of 8, 4 or 2 blocks at a time,
                    // lane = (block, row, which eight values of the block): the same eight values of the next
                    // block lie 256 bytes further on in the fragment order, so blocks collide on a bank and
                    // rows do not.
                    const uint32_t lr = inline_rows_log2(P.m_real);
                    const uint32_t item = warp + i * CW;             // (group of 8 >> lr blocks, group of four rows)
                    if (item >= ((P.k / 256) << lr) * (MM / 4)) return false;
                    const uint32_t bg = item / (MM / 4), rg = item % (MM / 4);
                    r = 4 * rg + ((lane >> 2) & ((1u << lr) - 1u));
                    c = (bg * (8u >> lr) + (lane >> (2 + lr))) * 32 + 8 * (lane & 3u);
                    return true;
                } else {
                    const uint32_t g = tid + i * CW * 32;
                    if (g >= total) return false;
                    r = MM > 1 ? g / gpr : 0u;
                    c = (g - r * gpr) * 8;
                    return true;
                }
            };
            uint4 raw[kInlineGroups][2];
#pragma unroll
            for (uint32_t i = 0; i < kInlineGroups; ++i) {
                uint32_t r, c;
                raw[i][0] = raw[i][1] = make_uint4(0u, 0u, 0u, 0u);   // rows past m_real (integer-MMA units): zeros
                if (group_of(i, r, c) && r < P.m_real) load_raw8(P.x, P.x_bf16, P.k, r, c, raw[i]);
            }
            request_first_stage(early, pre);
#pragma unroll
            for (uint32_t i = 0; i < kInlineGroups; ++i) {
                uint32_t r, c;
                if (group_of(i, r, c)) {
                    float f[8];
                    raw8_to_f32(raw[i], P.x_bf16, f);
                    if constexpr (MMA)
                        quantise_store8_frag<MM / 4, frag_sum_is_float(SCHEME), T::SUB>(f, P.k, (int)SumBias<SCHEME>::value, r, c, xs, lane);
                    else
                        quantise_store8<T::SUB>(f, P.k, (int)SumBias<SCHEME>::value, c, xs + r * P.xq_row_bytes, lane);
                }
            }
        }
        consumer_bar_n<CW * 32>();
    } else if (!P.xstream && !mbar_wait(smem_u32(&bars[2 * NS]), 0)) {
        dead = true;
        if (lane == 0) { atomicExch(P.err, 5); *abort_flag = 1u; }
    }
    uint32_t s = 0, ph = 0, rr = 0, rrph = 1;   // rrph: a fresh 'empty' barrier passes a wait on parity 1
    for (uint32_t si = 0; si < nseg; ++si) {
        const Segment sg = segment_at(P, rg, si);
        float tot[QU::NACC];
#pragma unroll
        for (int m = 0; m < QU::NACC; ++m) tot[m] = 0.f;
        for (uint32_t chunk = sg.c0; chunk < sg.c1; ++chunk) {
            if (!dead && (*abort_flag || !mbar_wait(smem_u32(&bars[s]), ph))) {
                dead = true;
                if (lane == 0) { atomicExch(P.err, 4); *abort_flag = 1u; }
            }
            if (!dead) {
                const uint32_t cu = min(kIntCU, ku - chunk * kIntCU);
                const uint32_t uw = warp / WPU;                   // the unit of the stage this warp works on
                L.row = stages_u32 + s * P.stage_stride + (uw / B::UB) * B::BOX_BYTES + trow * STRIDE;
                uint32_t kb = (chunk * kIntCU + uw) * 256;
                if constexpr (MMA) {
                    if (P.xstream) {                  // the stage's own fragments and scale entries, indexed inside the chunk
                        L.xh = stages_u32 + s * P.stage_stride + stage_bytes;
                        L.sb = L.xh + kIntCU * 8u * (MM / 4) * 256u;
                        kb = uw * 256;
                    }
                }
                if (uw < cu) {
                    if constexpr (MMA) QU::run(L, uw % B::UB, kb, tot, warp % WPU);
                    else QU::run(L, uw % B::UB, kb, tot);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars[NS + s]));
            }
            if (++s == NS) { s = 0; ph ^= 1u; }
        }
        // hand the warp's partials to the finisher through the ring of reduction buffers
        if (!dead && (*abort_flag || !mbar_wait(smem_u32(&rbars[kIntRB + rr]), rrph))) {
            dead = true;
            if (lane == 0) { atomicExch(P.err, 7); *abort_flag = 1u; }
        }
        if (!dead) {
            float* rbuf = red + rr * (CW * RL * MM);
            QU::finalize(tot, lane);
            if (lane < RL) {
#pragma unroll
                for (int m = 0; m < MM; ++m) rbuf[(warp * RL + lane) * MM + m] = tot[m];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&rbars[rr]));
        }
        if (++rr == kIntRB) { rr = 0; rrph ^= 1u; }
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel 3: a chain of dependent GEMVs in one launch (batch 1-2, dp4a units)
// ---------------------------------------------------------------------------------------------
// A decode step is a chain of small GEMVs, each the input of the next (gate/up -> SwiGLU -> down), and at
// 25-50 MB per matrix a launch is mostly hand-over: the next kernel cannot be resident before this one
// leaves, its ring starts empty, its activations come from L2 behind its own weight requests.  Here one
// cooperative grid runs the whole chain.  The producer warps never stop: weights are immutable, so the ring
// refills with the next layer's stages while this layer is still being multiplied, and the only thing a
// layer waits for is its input: a grid-wide barrier between layers (every CTA's finisher arrives after its
// last store of the layer; the consumer warps poll, bounded), then the usual in-kernel quantisation.
// The barrier words need no zeroed memory and survive graph replay: a word counts arrivals under the
// call's tag ((tag << 32) | count; any other upper half reads as zero), and the CTA that arrives last at
// the exit word, when nobody polls any more, zeroes them all.
// Measured, it does not pay yet (Q4_0 4096 -> 11008 -> 4096 at batch 1: 24.3 us against 16.2 us for two
// launches; Q4_K 8192 -> 2 x 14336 -> 8192 with SwiGLU: 60 us against 41 us): behind every barrier each CTA
// loads and quantises the layer's whole input (1.5-3.5 us, three rounds of loads for k = 14336, the SwiGLU
// exponentials included) while its ring sits full and HBM idles, and programmatic dependent launch already
// hides most of a launch boundary.  It runs on request only (option "gemv_chain").
constexpr uint32_t kChainMaxLayers = 3;

struct ChainParams {
    IntParams layer[kChainMaxLayers];
    uint32_t nlayers;
    uint32_t tag;                   // odd: never the upper half of a zeroed word
    uint32_t spin_limit;            // polls of a barrier word before the kernel gives up (error 8)
    unsigned long long* sync;       // [nlayers]: barrier after layer i (i < nlayers - 1), then the exit word
};

// Counts this CTA in and returns the count including it.  Once the word carries the call's tag it only ever
// counts up until the last CTA out zeroes it, so a plain atomic add does (hundreds of CTAs retrying a
// compare-and-swap on one word would take one memory round trip per success); only the first arrivals, which
// find something else in the word, install the tag by compare-and-swap.
__device__ __forceinline__ uint32_t chain_arrive(unsigned long long* word, uint32_t tag) {
    unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(word);
    for (;;) {
        if ((uint32_t)(old >> 32) == tag) return (uint32_t)atomicAdd(word, 1ull) + 1u;
        const unsigned long long nw = ((unsigned long long)tag << 32) | 1ull;
        const unsigned long long prev = atomicCAS(word, old, nw);
        if (prev == old) return 1u;
        old = prev;
    }
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ldg128_cg(const void* p) {      // from L2: the line may be stale in this SM's L1
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// The raw bytes of eight activations x[r][c .. c+8) of a layer: f32 or bf16 input (raw[0..1]), or, for the SwiGLU
// product of the previous layer's [gate | up] output (P.swiglu: x is [m][2k] f32), gate in raw[0..1] and up in
// raw[2..3].  Loads only: the caller issues all of a round's loads before it touches a value.
__device__ __forceinline__ void chain_load_raw(const IntParams& P, uint32_t r, uint32_t c, uint4 (&raw)[4]) {
    if (P.swiglu) {
        const float* row = reinterpret_cast<const float*>(P.x) + (size_t)r * 2 * P.k;
        raw[0] = ldg128_cg(row + c); raw[1] = ldg128_cg(row + c + 4);
        raw[2] = ldg128_cg(row + P.k + c); raw[3] = ldg128_cg(row + P.k + c + 4);
    } else if (P.x_bf16) {
        raw[0] = ldg128_cg(reinterpret_cast<const uint16_t*>(P.x) + (size_t)r * P.k + c);
    } else {
        const float* q = reinterpret_cast<const float*>(P.x) + (size_t)r * P.k + c;
        raw[0] = ldg128_cg(q); raw[1] = ldg128_cg(q + 4);
    }
}
__device__ __forceinline__ void chain_raw_to_f32(const IntParams& P, const uint4 (&raw)[4], float (&f)[8]) {
    const uint4 a[2] = {raw[0], raw[1]};
    if (P.swiglu) {
        const uint4 b[2] = {raw[2], raw[3]};
        float gf[8], uf[8];
        raw8_to_f32(a, 0u, gf);
        raw8_to_f32(b, 0u, uf);
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] = uf[q] * (gf[q] / (1.0f + expf(-gf[q])));
    } else {
        raw8_to_f32(a, P.x_bf16, f);
    }
}

template <uint32_t SCHEME, int MM>
__global__ void __launch_bounds__(int_threads(false), 2) gemv_chain_kernel(const __grid_constant__ ChainParams A) {
    static_assert(MM == 1 || MM == 2, "the chain kernel carries one or two activation rows");
    constexpr uint32_t CW = kIntWarps;
    using T = StagedTraits<SCHEME>;
    using B = IntBox<SCHEME, false>;
    using QU = QUnit<SCHEME, MM>;
    constexpr uint32_t STRIDE = B::ROW;
    constexpr uint32_t stage_bytes = B::STAGE_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    // one layout for all layers (the host sizes the activation area for the longest k)
    const IntParams& P0 = A.layer[0];
    uint8_t* xs = smem;
    uint8_t* stages = smem + P0.off_stage;
    float* red = reinterpret_cast<float*>(smem + P0.off_red);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P0.off_bar);   // full[NS], empty[NS], "first loads issued"
    const uint32_t NS = P0.nstages;
    uint64_t* rbars = bars + 2 * NS + 1;
    uint32_t* misc = reinterpret_cast<uint32_t*>(rbars + 2 * kIntRB);
    volatile uint32_t* abort_flag = misc;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t G = gridDim.x, me = blockIdx.x;
    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[NS + s]), CW);
        }
        mbar_init(smem_u32(&bars[2 * NS]), CW);
        for (uint32_t r = 0; r < kIntRB; ++r) {
            mbar_init(smem_u32(&rbars[r]), CW);
            mbar_init(smem_u32(&rbars[kIntRB + r]), 1);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    griddep_launch_dependents();
    // a layer may use fewer CTAs than the grid has (chunks_q / chunks_r split its chunks over `active` CTAs);
    // the others have nothing to do in that layer
    auto range_of = [&](const IntParams& P) -> Range {
        if (me < P.active) return make_range(P, me);
        Range rg{};
        return rg;                                  // nseg = 0
    };

    if (warp == CW) {
        // ---------------- producer warp: the ring never drains between layers ----------------
        uint32_t s = 0, ph = 1, issued = 0;
        bool dead = false;
        for (uint32_t li = 0; li < A.nlayers && !dead; ++li) {
            const IntParams& P = A.layer[li];
            if (lane == 0) tma_prefetch_desc(&P.wmap);
            const Range rg = range_of(P);
            for (uint32_t si = 0; si < rg.nseg && !dead; ++si) {
                const Segment sg = segment_at(P, rg, si);
                for (uint32_t c = sg.c0; c < sg.c1; ++c, ++issued) {
                    if (issued == 2 && li == 0) {
                        // the first activation loads must not queue behind a ring of weight requests: two stages,
                        // then wait until the consumer warps have issued theirs
                        if (!mbar_wait(smem_u32(&bars[2 * NS]), 0)) {
                            if (lane == 0) { atomicExch(P.err, 5); *abort_flag = 1u; }
                            dead = true;
                            break;
                        }
                    }
                    if (issued >= NS) {
                        if (*abort_flag || !mbar_wait(smem_u32(&bars[NS + s]), ph)) {
                            if (lane == 0) { atomicExch(P.err, 3); *abort_flag = 1u; }
                            dead = true;
                            break;
                        }
                    }
                    if (lane == 0) {
                        const uint32_t full = smem_u32(&bars[s]);
                        mbar_arrive_expect_tx(full, stage_bytes);
#pragma unroll
                        for (uint32_t b = 0; b < B::NB; ++b)
                            tma_load_2d(smem_u32(stages + s * stage_bytes + b * B::BOX_BYTES), &P.wmap,
                                        (int32_t)(((c * kIntCU + b * B::UB) * T::UNIT_B) / 8), (int32_t)(sg.tile * 16), full);
                    }
                    if (++s == NS) { s = 0; ph ^= 1u; }
                }
            }
        }
        return;
    }

    if (warp == CW + 1) {
        // ---------------- finisher warp ----------------
        constexpr int NC = (MM + 1) / 2;
        const uint32_t chalf = lane >> 4, rrow = lane & 15u;
        uint32_t r = 0, rph = 0;
        bool dead = false;
        griddep_wait();      // the workspace (partial tiles, rendezvous and barrier words) may be the previous launch's
        for (uint32_t li = 0; li < A.nlayers; ++li) {
            const IntParams& P = A.layer[li];
            const Range rg = range_of(P);
            for (uint32_t si = 0; si < rg.nseg && !dead; ++si) {
                const Segment sg = segment_at(P, rg, si);
                const uint32_t tile = sg.tile, mine = sg.c1 - sg.c0;
                if (*abort_flag || !mbar_wait(smem_u32(&rbars[r]), rph)) {
                    if (lane == 0) { atomicExch(P.err, 6); *abort_flag = 1u; }
                    dead = true;
                    break;
                }
                const float* rbuf = red + r * (CW * 32 * MM);
                float v[NC];
#pragma unroll
                for (int cp = 0; cp < NC; ++cp) {
                    const uint32_t col = 2 * cp + chalf;
                    v[cp] = 0.f;
                    if (col < (uint32_t)MM) {
#pragma unroll
                        for (uint32_t wv = 0; wv < CW; ++wv) {
                            v[cp] += rbuf[(wv * 32 + rrow) * MM + col];
                            v[cp] += rbuf[(wv * 32 + 16 + rrow) * MM + col];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&rbars[kIntRB + r]));
                if (++r == kIntRB) { r = 0; rph ^= 1u; }
                const uint32_t orow = tile * 16 + rrow;
                bool store = mine == P.nchunks;
                if (!store) {
                    // a tile cut between two CTAs: token exchange as in gemv_int_kernel's single-kernel mode
                    const uint32_t role = sg.c0 ? 1u : 0u;
                    float* pt = P.partial + (size_t)tile * 2 * (MM * 16);
#pragma unroll
                    for (int cp = 0; cp < NC; ++cp)
                        if (2 * cp + chalf < (uint32_t)MM) pt[(role * MM + 2 * cp + chalf) * 16 + rrow] = v[cp];
                    __threadfence();
                    __syncwarp();
                    unsigned long long old = 0ull;
                    if (lane == 0) old = atomicExch(&P.flags[tile], P.token + 2ull * role);
                    old = __shfl_sync(0xFFFFFFFFu, old, 0);
                    if (old == P.token + 2ull * (1u - role)) {
                        __threadfence();
#pragma unroll
                        for (int cp = 0; cp < NC; ++cp)
                            if (2 * cp + chalf < (uint32_t)MM) v[cp] += __ldcg(&pt[((1u - role) * MM + 2 * cp + chalf) * 16 + rrow]);
                        if (lane == 0) P.flags[tile] = 0ull;
                        store = true;
                    }
                }
                if (store) {
#pragma unroll
                    for (int cp = 0; cp < NC; ++cp) {
                        const uint32_t col = 2 * cp + chalf;
                        if (col < P.m_real && orow < P.n) {
                            const size_t o = (size_t)col * P.n + orow;
                            if (P.y_bf16) reinterpret_cast<uint16_t*>(P.y)[o] = (uint16_t)f32_to_bf16_bits(v[cp]);
                            else reinterpret_cast<float*>(P.y)[o] = v[cp];
                        }
                    }
                }
            }
            // everything this CTA contributes to the layer is stored (or will be by the partner that completes a
            // shared tile before its own arrival): count in; a dead CTA counts in too, the error word tells
            __threadfence();
            __syncwarp();
            if (lane == 0 && li + 1 < A.nlayers) chain_arrive(A.sync + li, A.tag);
        }
        if (lane == 0) {
            // nobody polls after its last layer: the last CTA out leaves every word at zero for the next replay
            if (chain_arrive(A.sync + A.nlayers - 1, A.tag) == G)
                for (uint32_t i = 0; i < A.nlayers; ++i) A.sync[i] = 0ull;
        }
        return;
    }

    // ---------------- consumer warps ----------------
    QLane L;
    L.half = lane >> 4;
    L.lane = lane;
    L.row_pitch = STRIDE;
    const uint32_t hoff = QU::HALF_OFFSETS ? L.half : 0u;
    const uint32_t trow = QU::first_row(lane), stages_u32 = smem_u32(stages);
    bool dead = false;
    uint32_t s = 0, ph = 0, rr = 0, rrph = 1;
    for (uint32_t li = 0; li < A.nlayers; ++li) {
        const IntParams& P = A.layer[li];
        if (li > 0) {
            // the layer's input is the previous layer's output: every CTA must have stored its part
            if (tid == 0) {
                const unsigned long long want = ((unsigned long long)A.tag << 32) | G;
                uint32_t ok = 0;
                for (uint32_t i = 0; i < A.spin_limit && !*abort_flag; ++i) {
                    if (ld_acquire_u64(A.sync + li - 1) == want) { ok = 1; break; }
                    __nanosleep(40);
                }
                if (!ok) { atomicExch(P.err, 8); *abort_flag = 1u; }
            }
            consumer_bar_n<CW * 32>();
            if (*abort_flag) dead = true;
        }
        L.xstride = P.xq_row_bytes;
        L.xh = smem_u32(xs) + 128 * hoff;
        L.xl = L.xh + P.k;
        L.sb = smem_u32(xs) + 2 * P.k + 16 * hoff;
        L.sx = smem_u32(xs) + 2 * P.k + (P.k / 32) * 4 + (32 / T::SUB) * 16 * hoff;
        if (li == 0) griddep_wait();                                    // x may be the previous kernel's output
        if (!dead) {
            // quantise the layer's activations; a round's loads (three groups of eight per thread) are all issued
            // before the first value is used
            const uint32_t gpr = P.k / 8, total = gpr * P.m_real;       // gpr % 32 == 0: whole warps stay together
            constexpr uint32_t kInFlight = 3;
            bool told = li != 0;                                        // whether the producer has been told to go on
            for (uint32_t g0 = tid; g0 < total; g0 += kInFlight * CW * 32) {
                uint4 raw[kInFlight][4];
#pragma unroll
                for (uint32_t i = 0; i < kInFlight; ++i) {
                    const uint32_t g = g0 + i * CW * 32;
                    if (g < total) {
                        const uint32_t r = MM > 1 ? g / gpr : 0u;
                        chain_load_raw(P, r, (g - r * gpr) * 8, raw[i]);
                    }
                }
                if (!told) {                                            // the producer may go on filling the ring
                    told = true;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[2 * NS]));
                }
#pragma unroll
                for (uint32_t i = 0; i < kInFlight; ++i) {
                    const uint32_t g = g0 + i * CW * 32;
                    if (g < total) {
                        const uint32_t r = MM > 1 ? g / gpr : 0u;
                        float f[8];
                        chain_raw_to_f32(P, raw[i], f);
                        quantise_store8<T::SUB>(f, P.k, (int)SumBias<SCHEME>::value, (g - r * gpr) * 8,
                                                xs + r * P.xq_row_bytes, lane);
                    }
                }
            }
            if (!told && lane == 0) mbar_arrive(smem_u32(&bars[2 * NS]));   // a warp without a group to quantise
        } else if (li == 0 && lane == 0) {
            mbar_arrive(smem_u32(&bars[2 * NS]));
        }
        consumer_bar_n<CW * 32>();
        const Range rg = range_of(P);
        const uint32_t ku = P.k / 256;
        for (uint32_t si = 0; si < rg.nseg; ++si) {
            const Segment sg = segment_at(P, rg, si);
            float tot[QU::NACC];
#pragma unroll
            for (int m = 0; m < QU::NACC; ++m) tot[m] = 0.f;
            for (uint32_t chunk = sg.c0; chunk < sg.c1; ++chunk) {
                if (!dead && (*abort_flag || !mbar_wait(smem_u32(&bars[s]), ph))) {
                    dead = true;
                    if (lane == 0) { atomicExch(P.err, 4); *abort_flag = 1u; }
                }
                if (!dead) {
                    const uint32_t cu = min(kIntCU, ku - chunk * kIntCU);
                    L.row = stages_u32 + s * stage_bytes + (warp / B::UB) * B::BOX_BYTES + trow * STRIDE;
                    if (warp < cu) QU::run(L, warp % B::UB, (chunk * kIntCU + warp) * 256, tot);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[NS + s]));
                }
                if (++s == NS) { s = 0; ph ^= 1u; }
            }
            if (!dead && (*abort_flag || !mbar_wait(smem_u32(&rbars[kIntRB + rr]), rrph))) {
                dead = true;
                if (lane == 0) { atomicExch(P.err, 7); *abort_flag = 1u; }
            }
            if (!dead) {
                float* rbuf = red + rr * (CW * 32 * MM);
                QU::finalize(tot, lane);
#pragma unroll
                for (int m = 0; m < MM; ++m) rbuf[(warp * 32 + lane) * MM + m] = tot[m];
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&rbars[rr]));
            }
            if (++rr == kIntRB) { rr = 0; rrph ^= 1u; }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct IntPlan {
    bool ok;
    uint32_t grid, ntiles, nchunks, total_chunks, slots, nstages;
    bool two_way;
    uint32_t xq_row_bytes, xq_pieces, off_stage, off_red, off_bar, smem_bytes;
    uint32_t xstream, stage_stride;
    size_t ws_xq, ws_partial, ws_counters, ws_bytes;
};

// Formats that have a integer-MMA unit (QUnitMma).
constexpr bool int_has_mma(uint32_t scheme) {
    return scheme == RLXQ_Q4_0 || scheme == RLXQ_Q8_0 || scheme == RLXQ_Q4_K || scheme == RLXQ_Q5_K || scheme == RLXQ_Q6_K ||
           scheme == RLXQ_Q8_K || scheme == RLXQ_Q2_K || scheme == RLXQ_Q3_K || scheme == RLXQ_Q4_1 || scheme == RLXQ_Q5_0 ||
           scheme == RLXQ_Q5_1;
}
// Formats that have a dp4a unit (QUnit); the others run batch 1 on their integer-MMA unit as well.
// formats whose down projection also exists as a pushing kernel (tensor-parallel exchange inside the finisher)
constexpr bool int_has_push(uint32_t scheme) {
    return scheme == RLXQ_Q4_0 || scheme == RLXQ_Q8_0 || scheme == RLXQ_Q4_K || scheme == RLXQ_Q5_K || scheme == RLXQ_Q6_K;
}
constexpr bool int_has_dp4a(uint32_t scheme) {
    return scheme == RLXQ_Q4_0 || scheme == RLXQ_Q8_0 || scheme == RLXQ_Q4_K || scheme == RLXQ_Q5_K || scheme == RLXQ_Q6_K;
}

template <uint32_t SCHEME, bool MMA = false>
static IntPlan plan_int(uint32_t m, uint32_t k, uint32_t n) {
    using T = StagedTraits<SCHEME>;
    constexpr uint32_t stage_bytes = IntBox<SCHEME, MMA>::STAGE_BYTES;
    IntPlan pl{};
    pl.ok = false;
    if (m == 0 || m > (MMA ? 8u : 4u) || n == 0 || k == 0 || k % (256 * T::AG)) return pl;
    if (MMA && !int_has_mma(SCHEME)) return pl;
    const uint32_t mm = MMA ? (m > 4 ? 8u : 4u) : (m > 2 ? 4u : m);    // rows the kernel template carries
    const uint32_t sms = (uint32_t)sm_count();
    auto align = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    pl.ntiles = (n + 15) / 16;
    pl.nchunks = (k / 256 + kIntCU - 1) / kIntCU;
    if ((uint64_t)pl.ntiles * pl.nchunks > 0xFFFFFFFFull / 2) return pl;
    pl.xq_row_bytes = 2 * k + (k / 32) * 4 + (k / T::SUB) * 4;      // a multiple of 16: k % 256 == 0
    pl.xq_pieces = mm;
    uint32_t stage_stride = stage_bytes;
    if (MMA) {                                                       // fragment order, fetched in 8 equal pieces
        if ((uint64_t)k * (mm / 4) * 10 > 0x7FFFFFFFull) return pl;
        pl.xq_pieces = 8;
        pl.xq_row_bytes = frag_total_bytes(k, mm / 4, T::SUB) / 8;   // 9 (or 10) k MMG / 8: a multiple of 16
    }
    uint32_t fixed = (uint32_t)align((size_t)pl.xq_row_bytes * pl.xq_pieces, 128);
    const uint32_t red_bytes = kIntRB * int_warps(MMA) * int_red_lanes(MMA) * mm * 4;
    const uint32_t tail = red_bytes + 1024;                            // reduction buffers, barriers, flags
    if (MMA && (uint64_t)fixed + tail + 2 * stage_bytes > 226u * 1024u) {
        // the fragments of all rows do not fit beside a ring: none stay resident, every stage carries its chunk's
        pl.xstream = 1;
        fixed = 0;
        stage_stride = stage_bytes + kIntCU * 8u * (mm / 4) * (256u + 4u * frag_entry_bytes(T::SUB));
    }
    // two CTAs per SM when that still leaves each a ring of >= 4 stages, else one
    const uint32_t budget2 = 113u * 1024u, budget1 = 226u * 1024u;
    uint32_t per_sm = 2, budget = budget2;
    // the four-row kernel keeps 64 activation words in registers: one CTA per SM
    if (mm > 2 || fixed + tail + 4 * stage_stride > budget2) { per_sm = 1; budget = budget1; }
    if (fixed + tail + 2 * stage_stride > budget) return pl;         // activations do not fit: not this kernel
    pl.nstages = (budget - fixed - tail) / stage_stride;
    if (pl.nstages > 24) pl.nstages = 24;
    pl.stage_stride = stage_stride;
    pl.off_stage = fixed;
    pl.off_red = pl.off_stage + pl.nstages * stage_stride;
    pl.off_bar = pl.off_red + red_bytes;
    pl.smem_bytes = pl.off_bar + (2 * pl.nstages + 1 + 2 * kIntRB) * 8 + 64;
    pl.total_chunks = pl.ntiles * pl.nchunks;
    pl.grid = sms * per_sm;
    // Slightly fewer tiles than CTAs: one whole tile per CTA beats splitting tiles (no shared tiles).
    if (pl.ntiles < pl.grid && pl.ntiles * 10 >= pl.grid * 7) pl.grid = pl.ntiles;
    if (pl.grid > pl.total_chunks) pl.grid = pl.total_chunks;
    const uint32_t per_cta = pl.total_chunks / pl.grid;              // >= 1
    pl.two_way = per_cta >= pl.nchunks;                              // a tile is cut by at most one range boundary
    pl.slots = (pl.nchunks + per_cta - 1) / per_cta + 1;             // contributors a tile can have
    // (a streamed chunk is copied whole-sized entries at a time: 16 bytes of slack behind the last one)
    pl.ws_xq = align((size_t)pl.xq_row_bytes * pl.xq_pieces + 16, 256);
    pl.ws_partial = align((size_t)pl.ntiles * pl.slots * mm * 16 * 4, 256);
    pl.ws_counters = align((size_t)pl.ntiles * 4, 256);
    pl.ws_bytes = pl.ws_xq + pl.ws_partial + pl.ws_counters + align((size_t)pl.ntiles * 8, 256);   // + rendezvous words
    pl.ok = true;
    return pl;
}

// Odd 64-bit values, a different one (and one two above it) for every call of this process; the
// starting point differs from process to process.
static unsigned long long next_call_token() {
    static std::atomic<unsigned long long> epoch{
        ((unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9E3779B97F4A7C15ull) >> 2};
    return (epoch.fetch_add(1) << 2) | 1ull;
}

template <uint32_t SCHEME, int MM, bool MMA = false, bool TP = false>
static int launch_int_t(cudaStream_t stream, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf,
                        uint32_t k, uint32_t n, void* ws, size_t ws_bytes, const IntPlan& pl, int* err_word, bool pair,
                        const float* expert_sel = nullptr, uint32_t num_experts = 0, uint32_t m_real = (uint32_t)MM,
                        const TpPush* tp = nullptr) {
    using T = StagedTraits<SCHEME>;
    Geometry g;
    geometry(SCHEME, &g);
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(RLXQ_E_WORKSPACE, "integer GEMV needs %zu workspace bytes, got %zu", pl.ws_bytes, ws_bytes);
    if ((uintptr_t)ws & 15u) return fail(RLXQ_E_ALIGN, "workspace must be 16-byte aligned");
    IntParams P{};
    int rcm = encode_weight_map(&P.wmap, w, expert_sel ? (uint64_t)n * num_experts : n, (uint64_t)k / g.elems * g.bytes,
                                IntBox<SCHEME, MMA>::ROW / 8, 16);
    if (rcm) return rcm;
    P.w = w; P.y = y;
    P.xq = reinterpret_cast<const uint8_t*>(ws);
    P.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + pl.ws_xq);
    P.counters = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(ws) + pl.ws_xq + pl.ws_partial);
    P.k = k; P.n = n; P.y_bf16 = ybf; P.m_real = m_real;
    P.use_red = (pl.two_way && !ybf) ? 1u : 0u;
    P.row_bytes = k / g.elems * g.bytes;
    P.ntiles = pl.ntiles; P.nchunks = pl.nchunks; P.total_chunks = pl.total_chunks; P.slots = pl.slots;
    P.chunks_q = pl.total_chunks / pl.grid; P.chunks_r = pl.total_chunks % pl.grid;
    P.nstages = pl.nstages; P.xq_row_bytes = pl.xq_row_bytes; P.xq_pieces = pl.xq_pieces;
    P.xstream = pl.xstream; P.stage_stride = pl.stage_stride;
    P.off_stage = pl.off_stage; P.off_red = pl.off_red; P.off_bar = pl.off_bar;
    // One kernel instead of two when every shared tile has exactly two contributors and re-quantising
    // the activations in every CTA is cheap (they come from L2): the quantiser kernel in front costs a
    // dependent-launch hop and a copy on the critical path of a call that lasts only microseconds.
    const int64_t iq = options().gemv_inline_q.load();
    // what the consumer threads can quantise: groups of eight values each (integer-MMA units: a warp takes
    // eight blocks of one row, four of two or two of four per round)
    const bool fits_inline = MMA ? ((uint64_t)k * (MM / 4) << inline_rows_log2(m_real)) <= inline_groups(MM, true) * int_warps(true) * 256u
                                 : (uint64_t)k * m_real <= inline_groups(MM) * kIntWarps * 32u * 8u;
    P.inline_q = (!pair && !tp && pl.two_way && fits_inline && !pl.xstream && (iq == 2 || iq == 0)) ? 1u : 0u;
    if (P.inline_q) P.use_red = 0u;
    if (TP != (tp != nullptr)) return fail(RLXQ_E_SHAPE, "pushing and plain launches are different kernels");
    if (tp) {                        // tiles go to the exchange buffers with plain stores, the quantiser kernel advances the step
        if ((uint64_t)m_real * n > tp->max_elems) return fail(RLXQ_E_SHAPE, "the exchange buffers hold %u values, the output has %llu", tp->max_elems, (unsigned long long)m_real * n);
        P.tp = *tp;
        P.use_red = 0u;
    }
    P.expert_sel = expert_sel;
    P.num_experts = num_experts;
    if (expert_sel && !P.inline_q) return fail(RLXQ_E_SHAPE, "expert-indirect GEMV needs the single-kernel mode");
    P.x = x; P.x_bf16 = xbf ? 1u : 0u;
    P.flags = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(ws) + pl.ws_xq + pl.ws_partial + pl.ws_counters);
    P.token = next_call_token();
    P.early = expert_sel ? 0u : (uint32_t)options().gemv_early.load();   // an indirect launch cannot prefetch before it knows its slab
    P.err = err_word;
    if (!P.err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    static std::atomic<uint32_t> attr_set[64];
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && attr_set[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemv_int_kernel<SCHEME, MM, MMA, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev].store(1);
    }
    const uint32_t groups = (k / 8) * m_real;
    int rc = RLXQ_OK;
    const uint32_t qgrid = (groups + 255) / 256;
    if (!P.inline_q) rc = launch_pdl(quantise_x_kernel<T::SUB, MMA ? MM / 4 : 0, MMA && frag_sum_is_float(SCHEME)>, dim3(qgrid), dim3(256), 0, stream, x, (uint32_t)xbf,
                        m_real, k, (int)SumBias<SCHEME>::value, reinterpret_cast<uint8_t*>(ws), pl.xq_row_bytes,
                        P.counters, pl.ntiles, reinterpret_cast<float*>(y), P.use_red ? m_real * n : 0u,
                        (pair ? 1u : 0u), tp ? reinterpret_cast<unsigned long long*>(tp->buf[tp->rank]) : nullptr, tp ? pl.grid : 0u);
    if (rc) return rc;
    if (!P.inline_q) count_launch();
    rc = launch_pdl(gemv_int_kernel<SCHEME, MM, MMA, TP>, dim3(pl.grid), dim3(int_threads(MMA)), pl.smem_bytes, stream, P);
    if (rc) return rc;
    count_launch();
    return check_launch("gemv_int_kernel");
}

template <uint32_t SCHEME>
static int launch_int_s(cudaStream_t stream, const void* x, bool xbf, const uint8_t* w, void* y, bool ybf,
                        uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes, int* err_word, bool pair,
                        const float* expert_sel = nullptr, uint32_t num_experts = 0, bool mma = false, const TpPush* tp = nullptr) {
    if (mma) {
        if constexpr (int_has_mma(SCHEME)) {
            const IntPlan plm = plan_int<SCHEME, true>(m, k, n);
            if (!plm.ok) return fail(RLXQ_E_SHAPE, "integer-MMA GEMV does not support m=%u k=%u n=%u", m, k, n);
            if (tp) {
                if constexpr (int_has_push(SCHEME)) {
                    if (m <= 4) return launch_int_t<SCHEME, 4, true, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, plm, err_word, pair, nullptr, 0, m, tp);
                    return launch_int_t<SCHEME, 8, true, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, plm, err_word, pair, nullptr, 0, m, tp);
                } else {
                    return fail(RLXQ_E_SHAPE, "no pushing GEMV for scheme %u", (unsigned)SCHEME);
                }
            }
            if (m <= 4) return launch_int_t<SCHEME, 4, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, plm, err_word, pair, nullptr, 0, m);
            return launch_int_t<SCHEME, 8, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, plm, err_word, pair, nullptr, 0, m);
        } else {
            return fail(RLXQ_E_SHAPE, "no integer-MMA GEMV for scheme %u", (unsigned)SCHEME);
        }
    }
    if constexpr (int_has_dp4a(SCHEME)) {
        const IntPlan pl = plan_int<SCHEME>(m, k, n);
        if (!pl.ok) return fail(RLXQ_E_SHAPE, "integer GEMV does not support m=%u k=%u n=%u", m, k, n);
        if (tp) {
            if constexpr (int_has_push(SCHEME)) {
                if (m == 1) return launch_int_t<SCHEME, 1, false, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, pl, err_word, pair, nullptr, 0, 1, tp);
                if (m == 2) return launch_int_t<SCHEME, 2, false, true>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, pl, err_word, pair, nullptr, 0, 2, tp);
            }
            return fail(RLXQ_E_SHAPE, "no pushing dp4a GEMV for scheme %u at m=%u", (unsigned)SCHEME, m);
        }
        if (m == 1) return launch_int_t<SCHEME, 1>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, pl, err_word, pair, expert_sel, num_experts, 1);
        if (m == 2) return launch_int_t<SCHEME, 2>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, pl, err_word, pair, nullptr, 0, 2);
        return launch_int_t<SCHEME, 4>(stream, x, xbf, w, y, ybf, k, n, ws, ws_bytes, pl, err_word, pair, nullptr, 0, m);
    } else {
        return fail(RLXQ_E_SHAPE, "no dp4a unit for scheme %u", (unsigned)SCHEME);
    }
}

bool int_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x) {
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    switch (scheme) {
        case RLXQ_Q4_0: return plan_int<RLXQ_Q4_0>(m, k, n).ok;
        case RLXQ_Q8_0: return plan_int<RLXQ_Q8_0>(m, k, n).ok;
        case RLXQ_Q4_K: return plan_int<RLXQ_Q4_K>(m, k, n).ok;
        case RLXQ_Q5_K: return plan_int<RLXQ_Q5_K>(m, k, n).ok;
        case RLXQ_Q6_K: return plan_int<RLXQ_Q6_K>(m, k, n).ok;
        default: return false;
    }
}

size_t int_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n) {
    IntPlan pl{};
    switch (scheme) {
        case RLXQ_Q4_0: pl = plan_int<RLXQ_Q4_0>(m, k, n); break;
        case RLXQ_Q8_0: pl = plan_int<RLXQ_Q8_0>(m, k, n); break;
        case RLXQ_Q4_K: pl = plan_int<RLXQ_Q4_K>(m, k, n); break;
        case RLXQ_Q5_K: pl = plan_int<RLXQ_Q5_K>(m, k, n); break;
        case RLXQ_Q6_K: pl = plan_int<RLXQ_Q6_K>(m, k, n); break;
        default: break;
    }
    return pl.ok ? pl.ws_bytes : 0;
}

static int launch_gemv_int_err(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w,
                               void* y, bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes,
                               int* err_word, bool pair = false) {
    switch (scheme) {
        case RLXQ_Q4_0: return launch_int_s<RLXQ_Q4_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err_word, pair);
        case RLXQ_Q8_0: return launch_int_s<RLXQ_Q8_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err_word, pair);
        case RLXQ_Q4_K: return launch_int_s<RLXQ_Q4_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err_word, pair);
        case RLXQ_Q5_K: return launch_int_s<RLXQ_Q5_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err_word, pair);
        case RLXQ_Q6_K: return launch_int_s<RLXQ_Q6_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err_word, pair);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
}

int launch_gemv_int(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                    bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    return launch_gemv_int_err(stream, scheme, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, device_error_word());
}

// The same kernel with its integer-MMA units: batch 1-8 (carried as 4 or 8 rows); Q4_0, Q8_0, Q4_K.
bool int_mma_supported(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n, const void* w, const void* x) {
    if (((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    switch (scheme) {
        case RLXQ_Q4_0: return plan_int<RLXQ_Q4_0, true>(m, k, n).ok;
        case RLXQ_Q8_0: return plan_int<RLXQ_Q8_0, true>(m, k, n).ok;
        case RLXQ_Q4_K: return plan_int<RLXQ_Q4_K, true>(m, k, n).ok;
        case RLXQ_Q5_K: return plan_int<RLXQ_Q5_K, true>(m, k, n).ok;
        case RLXQ_Q6_K: return plan_int<RLXQ_Q6_K, true>(m, k, n).ok;
        case RLXQ_Q8_K: return plan_int<RLXQ_Q8_K, true>(m, k, n).ok;
        case RLXQ_Q2_K: return plan_int<RLXQ_Q2_K, true>(m, k, n).ok;
        case RLXQ_Q3_K: return plan_int<RLXQ_Q3_K, true>(m, k, n).ok;
        case RLXQ_Q4_1: return plan_int<RLXQ_Q4_1, true>(m, k, n).ok;
        case RLXQ_Q5_0: return plan_int<RLXQ_Q5_0, true>(m, k, n).ok;
        case RLXQ_Q5_1: return plan_int<RLXQ_Q5_1, true>(m, k, n).ok;
        default: return false;
    }
}

size_t int_mma_workspace_bytes(uint32_t scheme, uint32_t m, uint32_t k, uint32_t n) {
    IntPlan pl{};
    switch (scheme) {
        case RLXQ_Q4_0: pl = plan_int<RLXQ_Q4_0, true>(m, k, n); break;
        case RLXQ_Q8_0: pl = plan_int<RLXQ_Q8_0, true>(m, k, n); break;
        case RLXQ_Q4_K: pl = plan_int<RLXQ_Q4_K, true>(m, k, n); break;
        case RLXQ_Q5_K: pl = plan_int<RLXQ_Q5_K, true>(m, k, n); break;
        case RLXQ_Q6_K: pl = plan_int<RLXQ_Q6_K, true>(m, k, n); break;
        case RLXQ_Q8_K: pl = plan_int<RLXQ_Q8_K, true>(m, k, n); break;
        case RLXQ_Q2_K: pl = plan_int<RLXQ_Q2_K, true>(m, k, n); break;
        case RLXQ_Q3_K: pl = plan_int<RLXQ_Q3_K, true>(m, k, n); break;
        case RLXQ_Q4_1: pl = plan_int<RLXQ_Q4_1, true>(m, k, n); break;
        case RLXQ_Q5_0: pl = plan_int<RLXQ_Q5_0, true>(m, k, n); break;
        case RLXQ_Q5_1: pl = plan_int<RLXQ_Q5_1, true>(m, k, n); break;
        default: break;
    }
    return pl.ok ? pl.ws_bytes : 0;
}

int launch_gemv_int_mma(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w, void* y,
                        bool ybf, uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes) {
    int* err = device_error_word();
    switch (scheme) {
        case RLXQ_Q4_0: return launch_int_s<RLXQ_Q4_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q8_0: return launch_int_s<RLXQ_Q8_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q4_K: return launch_int_s<RLXQ_Q4_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q5_K: return launch_int_s<RLXQ_Q5_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q6_K: return launch_int_s<RLXQ_Q6_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q8_K: return launch_int_s<RLXQ_Q8_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q2_K: return launch_int_s<RLXQ_Q2_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q3_K: return launch_int_s<RLXQ_Q3_K>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q4_1: return launch_int_s<RLXQ_Q4_1>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q5_0: return launch_int_s<RLXQ_Q5_0>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        case RLXQ_Q5_1: return launch_int_s<RLXQ_Q5_1>(stream, x, xbf, w, y, ybf, m, k, n, ws, ws_bytes, err, false, nullptr, 0, true);
        default: return fail(RLXQ_E_SCHEME, "no integer-MMA GEMV for scheme %u", scheme);
    }
}

// One row of an MoE decode step: y[n] = x[k] . W_e^T where W is a stack of num_experts [n, k] slabs and
// e = (uint32_t)*expert_sel is read on the device.  Needs the single-kernel mode (k <= 12288, tiles shared
// by at most two CTAs); int_expert_supported tells.
bool int_expert_supported(uint32_t scheme, uint32_t k, uint32_t n, const void* w, const void* x) {
    if (!int_supported(scheme, 1, k, n, w, x)) return false;
    if ((uint64_t)k > inline_groups(1) * kIntWarps * 32u * 8u || options().gemv_inline_q.load() == 1) return false;
    switch (scheme) {
        case RLXQ_Q4_0: return plan_int<RLXQ_Q4_0>(1, k, n).two_way;
        case RLXQ_Q8_0: return plan_int<RLXQ_Q8_0>(1, k, n).two_way;
        case RLXQ_Q4_K: return plan_int<RLXQ_Q4_K>(1, k, n).two_way;
        case RLXQ_Q5_K: return plan_int<RLXQ_Q5_K>(1, k, n).two_way;
        case RLXQ_Q6_K: return plan_int<RLXQ_Q6_K>(1, k, n).two_way;
        default: return false;
    }
}

int launch_gemv_int_expert(cudaStream_t stream, uint32_t scheme, const void* x, bool xbf, const uint8_t* w_stack, void* y,
                           bool ybf, uint32_t k, uint32_t n, uint32_t num_experts, const float* expert_sel, void* ws,
                           size_t ws_bytes) {
    int* err = device_error_word();
    switch (scheme) {
        case RLXQ_Q4_0: return launch_int_s<RLXQ_Q4_0>(stream, x, xbf, w_stack, y, ybf, 1, k, n, ws, ws_bytes, err, false, expert_sel, num_experts);
        case RLXQ_Q8_0: return launch_int_s<RLXQ_Q8_0>(stream, x, xbf, w_stack, y, ybf, 1, k, n, ws, ws_bytes, err, false, expert_sel, num_experts);
        case RLXQ_Q4_K: return launch_int_s<RLXQ_Q4_K>(stream, x, xbf, w_stack, y, ybf, 1, k, n, ws, ws_bytes, err, false, expert_sel, num_experts);
        case RLXQ_Q5_K: return launch_int_s<RLXQ_Q5_K>(stream, x, xbf, w_stack, y, ybf, 1, k, n, ws, ws_bytes, err, false, expert_sel, num_experts);
        case RLXQ_Q6_K: return launch_int_s<RLXQ_Q6_K>(stream, x, xbf, w_stack, y, ybf, 1, k, n, ws, ws_bytes, err, false, expert_sel, num_experts);
        default: return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    }
}

// y = (up * silu(gate)) . W^T with gu = [gate | up] ([m][2k] f32): the SwiGLU product is formed by the
// activation quantiser, so the row-parallel down projection of an FFN needs no kernel in between.
bool int_push_supported(uint32_t scheme) { return int_has_push(scheme); }

int launch_gemv_int_swiglu(cudaStream_t stream, uint32_t scheme, const float* gu, const uint8_t* w, void* y, bool ybf,
                           uint32_t m, uint32_t k, uint32_t n, void* ws, size_t ws_bytes, const TpPush* tp) {
    int* err = device_error_word();
    const bool mma = m >= 2 && int_mma_supported(scheme, m, k, n, w, gu);     // batch 2-8: the integer-MMA units
    switch (scheme) {
        case RLXQ_Q4_0: return launch_int_s<RLXQ_Q4_0>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, mma, tp);
        case RLXQ_Q8_0: return launch_int_s<RLXQ_Q8_0>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, mma, tp);
        case RLXQ_Q4_K: return launch_int_s<RLXQ_Q4_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, mma, tp);
        case RLXQ_Q5_K: return launch_int_s<RLXQ_Q5_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, mma, tp);
        case RLXQ_Q6_K: return launch_int_s<RLXQ_Q6_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, mma, tp);
        case RLXQ_Q8_K: return launch_int_s<RLXQ_Q8_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        case RLXQ_Q2_K: return launch_int_s<RLXQ_Q2_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        case RLXQ_Q3_K: return launch_int_s<RLXQ_Q3_K>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        case RLXQ_Q4_1: return launch_int_s<RLXQ_Q4_1>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        case RLXQ_Q5_0: return launch_int_s<RLXQ_Q5_0>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        case RLXQ_Q5_1: return launch_int_s<RLXQ_Q5_1>(stream, gu, false, w, y, ybf, m, k, n, ws, ws_bytes, err, true, nullptr, 0, true, tp);
        default: return fail(RLXQ_E_SCHEME, "no integer GEMV for scheme %u", scheme);
    }
}

// ---------------------------------------------------------------------------------------------
// The chain kernel's host side
// ---------------------------------------------------------------------------------------------
struct ChainPlan {
    bool ok;
    uint32_t grid, nstages, off_stage, off_red, off_bar, smem_bytes;
    struct { uint32_t ntiles, nchunks, total_chunks, active, xq_row_bytes; size_t off_partial, off_flags, off_y; } l[kChainMaxLayers];
    size_t off_sync, ws_bytes;
};

template <uint32_t SCHEME>
static ChainPlan plan_chain(const ChainLayer* L, uint32_t nl, uint32_t m) {
    using T = StagedTraits<SCHEME>;
    constexpr uint32_t stage_bytes = IntBox<SCHEME, false>::STAGE_BYTES;
    ChainPlan pl{};
    if (nl < 2 || nl > kChainMaxLayers || m == 0 || m > 2) return pl;
    auto align = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    const uint32_t sms = (uint32_t)sm_count();
    pl.grid = 2 * sms;
    uint32_t xq_max = 0;
    size_t off = 0;
    for (uint32_t i = 0; i < nl; ++i) {
        const uint32_t k = L[i].k, n = L[i].n;
        if (n == 0 || k == 0 || k % (256 * T::AG)) return pl;
        // a layer's input is the previous layer's output, or the SwiGLU product of its [gate | up] halves
        if (i > 0 && L[i - 1].n != (L[i].swiglu ? 2 * k : k)) return pl;
        if (i == 0 && L[i].swiglu) return pl;
        auto& q = pl.l[i];
        q.ntiles = (n + 15) / 16;
        q.nchunks = (k / 256 + kIntCU - 1) / kIntCU;
        if ((uint64_t)q.ntiles * q.nchunks > 0xFFFFFFFFull / 2) return pl;
        q.total_chunks = q.ntiles * q.nchunks;
        q.active = pl.grid;
        if (q.ntiles < q.active && q.ntiles * 10 >= q.active * 7) q.active = q.ntiles;   // one whole tile per CTA
        if (q.active > q.total_chunks) q.active = q.total_chunks;
        if (q.total_chunks / q.active < q.nchunks) return pl;        // a tile would be cut more than once
        q.xq_row_bytes = 2 * k + (k / 32) * 4 + (k / T::SUB) * 4;
        xq_max = q.xq_row_bytes > xq_max ? q.xq_row_bytes : xq_max;
        q.off_partial = off; off += align((size_t)q.ntiles * 2 * m * 16 * 4, 256);
        q.off_flags = off;   off += align((size_t)q.ntiles * 8, 256);
        q.off_y = off;       if (i + 1 < nl) off += align((size_t)m * n * 4, 256);   // intermediate outputs (f32)
    }
    pl.off_sync = off; off += 256;
    pl.ws_bytes = off;
    const uint32_t fixed = (uint32_t)align((size_t)xq_max * m, 128);
    const uint32_t red_bytes = kIntRB * kIntWarps * 32 * m * 4;
    const uint32_t budget = 113u * 1024u;
    if (fixed + red_bytes + 1024 + 3 * stage_bytes > budget) return pl;   // too little ring left beside the activations
    pl.nstages = (budget - fixed - red_bytes - 1024) / stage_bytes;
    if (pl.nstages > 24) pl.nstages = 24;
    pl.off_stage = fixed;
    pl.off_red = pl.off_stage + pl.nstages * stage_bytes;
    pl.off_bar = pl.off_red + red_bytes;
    pl.smem_bytes = pl.off_bar + (2 * pl.nstages + 1 + 2 * kIntRB) * 8 + 64;
    pl.ok = true;
    return pl;
}

template <uint32_t SCHEME, int MM>
static int launch_chain_t(cudaStream_t stream, const ChainLayer* L, uint32_t nl, const void* x, bool xbf, void* y, bool ybf,
                          void* ws, size_t ws_bytes, const ChainPlan& pl) {
    Geometry g;
    geometry(SCHEME, &g);
    if (!ws || ws_bytes < pl.ws_bytes)
        return fail(RLXQ_E_WORKSPACE, "GEMV chain needs %zu workspace bytes, got %zu", pl.ws_bytes, ws_bytes);
    if ((uintptr_t)ws & 255u) return fail(RLXQ_E_ALIGN, "chain workspace must be 256-byte aligned");
    static std::atomic<int> coop_ok[64];        // 0 unknown, 1 usable, -1 not (the grid would not be co-resident)
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(RLXQ_E_CUDA, "device index out of range");
    if (coop_ok[dev].load() == 0) {
        RLXQ_CUDA_TRY(cudaFuncSetAttribute(gemv_chain_kernel<SCHEME, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        int coop = 0, per_sm = 0;
        RLXQ_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        RLXQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_chain_kernel<SCHEME, MM>, (int)int_threads(false),
                                                                    pl.smem_bytes));
        coop_ok[dev].store(coop && per_sm >= 2 ? 1 : -1);
    }
    if (coop_ok[dev].load() < 0) return fail(RLXQ_E_SHAPE, "the chain kernel's grid cannot be co-resident on this device");
    ChainParams A{};
    uint8_t* base = static_cast<uint8_t*>(ws);
    const unsigned long long token = next_call_token();
    int* err = device_error_word();
    if (!err) return fail(RLXQ_E_CUDA, "device error word unavailable");
    for (uint32_t i = 0; i < nl; ++i) {
        IntParams& P = A.layer[i];
        const auto& q = pl.l[i];
        int rc = encode_weight_map(&P.wmap, L[i].w, L[i].n, (uint64_t)L[i].k / g.elems * g.bytes, IntBox<SCHEME, false>::ROW / 8, 16);
        if (rc) return rc;
        P.w = L[i].w;
        P.y = i + 1 < nl ? static_cast<void*>(base + q.off_y) : y;
        P.y_bf16 = i + 1 < nl ? 0u : (ybf ? 1u : 0u);
        P.x = i == 0 ? x : A.layer[i - 1].y;
        P.x_bf16 = i == 0 && xbf ? 1u : 0u;
        P.k = L[i].k; P.n = L[i].n; P.m_real = MM;
        P.row_bytes = L[i].k / g.elems * g.bytes;
        P.ntiles = q.ntiles; P.nchunks = q.nchunks; P.total_chunks = q.total_chunks; P.slots = 2;
        P.active = q.active;
        P.chunks_q = q.total_chunks / q.active; P.chunks_r = q.total_chunks % q.active;
        P.nstages = pl.nstages; P.xq_row_bytes = q.xq_row_bytes; P.xq_pieces = MM;
        P.stage_stride = IntBox<SCHEME, false>::STAGE_BYTES;
        P.off_stage = pl.off_stage; P.off_red = pl.off_red; P.off_bar = pl.off_bar;
        P.inline_q = 1u;
        P.partial = reinterpret_cast<float*>(base + q.off_partial);
        P.flags = reinterpret_cast<unsigned long long*>(base + q.off_flags);
        P.token = token;
        P.swiglu = L[i].swiglu ? 1u : 0u;
        P.err = err;
    }
    A.nlayers = nl;
    A.tag = (uint32_t)(token >> 8) | 1u;
    A.spin_limit = 1u << 22;
    A.sync = reinterpret_cast<unsigned long long*>(base + pl.off_sync);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(int_threads(false));
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;      // the CTAs wait for one another: they must all be resident
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // with programmatic serialization the ring fills while the predecessor drains; where the driver does not take
    // both attributes together the launch is cooperative only
    static std::atomic<int> both_ok[64];             // 0 untried, 1 accepted, -1 refused
    cfg.numAttrs = (options().pdl.load() && both_ok[dev].load() >= 0) ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemv_chain_kernel<SCHEME, MM>, A);
    if (le != cudaSuccess && cfg.numAttrs == 2 && both_ok[dev].load() == 0) {
        (void)cudaGetLastError();
        both_ok[dev].store(-1);
        cfg.numAttrs = 1;
        le = cudaLaunchKernelEx(&cfg, gemv_chain_kernel<SCHEME, MM>, A);
    } else if (le == cudaSuccess && cfg.numAttrs == 2) {
        both_ok[dev].store(1);
    }
    RLXQ_CUDA_TRY(le);
    count_launch();
    return check_launch("gemv_chain_kernel");
}

template <uint32_t SCHEME>
static int launch_chain_s(cudaStream_t stream, const ChainLayer* L, uint32_t nl, const void* x, bool xbf, void* y, bool ybf,
                          uint32_t m, void* ws, size_t ws_bytes) {
    const ChainPlan pl = plan_chain<SCHEME>(L, nl, m);
    if (!pl.ok) return fail(RLXQ_E_SHAPE, "these layers cannot run as one chain kernel");
    if (m == 1) return launch_chain_t<SCHEME, 1>(stream, L, nl, x, xbf, y, ybf, ws, ws_bytes, pl);
    return launch_chain_t<SCHEME, 2>(stream, L, nl, x, xbf, y, ybf, ws, ws_bytes, pl);
}

// 0 when the layers cannot run as one chain kernel (then the caller runs them one by one).
size_t chain_workspace_bytes(uint32_t scheme, const ChainLayer* L, uint32_t nl, uint32_t m) {
    ChainPlan pl{};
    switch (scheme) {
        case RLXQ_Q4_0: pl = plan_chain<RLXQ_Q4_0>(L, nl, m); break;
        case RLXQ_Q8_0: pl = plan_chain<RLXQ_Q8_0>(L, nl, m); break;
        case RLXQ_Q4_K: pl = plan_chain<RLXQ_Q4_K>(L, nl, m); break;
        case RLXQ_Q5_K: pl = plan_chain<RLXQ_Q5_K>(L, nl, m); break;
        case RLXQ_Q6_K: pl = plan_chain<RLXQ_Q6_K>(L, nl, m); break;
        default: break;
    }
    return pl.ok ? pl.ws_bytes : 0;
}

int launch_gemv_chain(cudaStream_t stream, uint32_t scheme, const ChainLayer* L, uint32_t nl, const void* x, bool xbf, void* y,
                      bool ybf, uint32_t m, void* ws, size_t ws_bytes) {
    for (uint32_t i = 0; i < nl; ++i)
        if ((uintptr_t)L[i].w & 15u) return fail(RLXQ_E_ALIGN, "chain weights must be 16-byte aligned");
    if ((uintptr_t)x & 15u) return fail(RLXQ_E_ALIGN, "x must be 16-byte aligned");
    switch (scheme) {
        case RLXQ_Q4_0: return launch_chain_s<RLXQ_Q4_0>(stream, L, nl, x, xbf, y, ybf, m, ws, ws_bytes);
        case RLXQ_Q8_0: return launch_chain_s<RLXQ_Q8_0>(stream, L, nl, x, xbf, y, ybf, m, ws, ws_bytes);
        case RLXQ_Q4_K: return launch_chain_s<RLXQ_Q4_K>(stream, L, nl, x, xbf, y, ybf, m, ws, ws_bytes);
        case RLXQ_Q5_K: return launch_chain_s<RLXQ_Q5_K>(stream, L, nl, x, xbf, y, ybf, m, ws, ws_bytes);
        case RLXQ_Q6_K: return launch_chain_s<RLXQ_Q6_K>(stream, L, nl, x, xbf, y, ybf, m, ws, ws_bytes);
        default: return fail(RLXQ_E_SCHEME, "no chain kernel for scheme %u", scheme);
    }
}

// ---------------------------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory
// ---------------------------------------------------------------------------------------------
// Some hosts of this library run where cudaMalloc is off the table: inside a latency-critical
// decode loop whose memory was sized and pinned down at start-up, in a process that has handed its
// whole device budget to another allocator, or in code reviewed under a "no allocation after
// initialisation" rule.  rlxq_matmul needs a caller-provided workspace for the batch 1-2 GEMV
// (quantised activations, a few partial tiles, tile counters); such callers may have nowhere to
// take it from.  For them the same two kernels run with a workspace that lives in this library's
// own image: a file-scope device array of fixed size that every GPU loading the library carries
// until the process exits.
//
// In host code `g_static_scratch` is only a handle for the symbol, not an address the GPU can use;
// the device address is looked up once per device with cudaGetSymbolAddress (with that device
// current) and that pointer is what the kernels get.
constexpr size_t kStaticScratchBytes = 2u << 20;          // 2 MiB per GPU
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_error_word;                // used when the device has no error word yet

struct StaticScratch { uint8_t* scratch; int* err; };

// First call on a device: resolve the two symbols.  No allocation; must happen outside stream
// capture (symbol lookup may initialise the module on this device).
static std::atomic<uint8_t*> scratch_ptr[64];
static std::atomic<int*> err_ptr[64];

// The built-in error word of the current device if an allocation-free call has resolved it, else null.
int* static_error_word_if_resolved() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return err_ptr[dev].load();
}

static int static_scratch_for_current_device(StaticScratch* out) {
    int dev = 0;
    RLXQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(RLXQ_E_ARG, "device ordinal %d out of range", dev);
    uint8_t* sp = scratch_ptr[dev].load();
    int* ep = err_ptr[dev].load();
    if (!sp || !ep) {
        void* a = nullptr;
        void* b = nullptr;
        RLXQ_CUDA_TRY(cudaGetSymbolAddress(&a, g_static_scratch));
        RLXQ_CUDA_TRY(cudaGetSymbolAddress(&b, g_static_error_word));
        if (!a || !b) return fail(RLXQ_E_CUDA, "cudaGetSymbolAddress returned a null device address");
        sp = static_cast<uint8_t*>(a);
        ep = static_cast<int*>(b);
        scratch_ptr[dev].store(sp);
        err_ptr[dev].store(ep);
    }
    out->scratch = sp;
    out->err = ep;
    return RLXQ_OK;
}

}  // namespace rlxq

using namespace rlxq;


extern "C" int rlxq_matmul_static_scratch(rlxq_stream_t stream, uint32_t scheme, const void* x, uint32_t x_dtype,
                                          const void* w_blocks, void* y, uint32_t y_dtype, uint32_t m, uint32_t k,
                                          uint32_t n) {
    Geometry g;
    if (!geometry(scheme, &g)) return fail(RLXQ_E_SCHEME, "unknown scheme %u", scheme);
    if ((x_dtype != RLXQ_F32 && x_dtype != RLXQ_BF16) || (y_dtype != RLXQ_F32 && y_dtype != RLXQ_BF16))
        return fail(RLXQ_E_DTYPE, "unknown dtype");
    if (m == 0 || n == 0) return RLXQ_OK;
    if (m > 2) return fail(RLXQ_E_SHAPE, "the static-scratch entry point covers batch 1 and 2 only (m=%u)", m);
    if (k == 0 || k % g.elems) return fail(RLXQ_E_SHAPE, "k=%u is not a positive multiple of the block size %u", k, g.elems);
    if (!x || !w_blocks || !y) return fail(RLXQ_E_NULL, "null buffer");
    if (((uintptr_t)x & 15u) || ((uintptr_t)w_blocks & 15u)) return fail(RLXQ_E_ALIGN, "x and w_blocks must be 16-byte aligned");
    if ((uintptr_t)y & (y_dtype == RLXQ_BF16 ? 1u : 3u)) return fail(RLXQ_E_ALIGN, "y must be aligned to its element size");
    if (!int_supported(scheme, m, k, n, w_blocks, x))
        return fail(RLXQ_E_SHAPE, "the streaming GEMV needs k %% 256 == 0 (2048 for Q6_K) and activations that fit in shared memory");
    const size_t need = int_workspace_bytes(scheme, m, k, n);
    if (need > kStaticScratchBytes)
        return fail(RLXQ_E_LIMIT, "this shape needs %zu bytes of scratch; the built-in scratch holds %zu", need,
                    (size_t)kStaticScratchBytes);
    StaticScratch ss;
    int rc = static_scratch_for_current_device(&ss);
    if (rc) return rc;
    // Timeouts of bounded waits go to the device's regular error word when it already exists, otherwise
    // to a word in this library's image; rlxq_device_status reads both and allocates neither.
    int* err = device_error_word_if_ready();
    if (!err) err = ss.err;
    // Nothing an earlier call left in the scratch is ever consumed: partial tiles are written before
    // they are read; in two-kernel mode the quantiser rewrites the activations and zeroes the tile
    // counters (and y in the two-contributor add mode); in single-kernel mode the rendezvous words
    // are only ever compared with this call's own tokens.
    return launch_gemv_int_err((cudaStream_t)stream, scheme, x, x_dtype == RLXQ_BF16, (const uint8_t*)w_blocks, y,
                               y_dtype == RLXQ_BF16, m, k, n, ss.scratch, kStaticScratchBytes, err);
}
