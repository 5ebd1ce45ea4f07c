// Streaming dequant-fused matvec for block qtypes at HBM rate: one persistent CTA per SM walks a
// list of (matrix, 16-row tile) tasks, so one launch covers one large matrix or a batch of
// independent matrices with their own input vectors.
//
// Arithmetic. The weights enter the tensor cores as signed bytes (mma.sync.m16n8k32, s8 x s8 ->
// s32): IQ2_XXS +-{8,25,43}, Q4_K codes 0..15, Q8_0 its int8 quants, MXFP4 its levels + 16. The f32 activation row is
// quantised once per matrix to a 28-bit fixed-point number relative to a power of two above its
// largest magnitude and split into four balanced base-128 digits (planes of signed bytes), so
// products and the 32-term sums are exact integers and only the 2^-27 input quantisation and
// the final f32 arithmetic round. Every qtype here scales groups of 32 weights (IQ2_XXS
// sub-scale, Q4_K sub-block scale, Q8_0 block scale), and one MMA covers 32 k for 16 rows. The
// B operand is arranged so that the 8 MMA columns are (group, digit): quad lane t of a row
// owns one whole group, column 2t / 2t+1 carries the activation digits only at the k slots of
// lane t. The accumulator fragment of lane (row, t) is then the exact integer dot product of ITS
// group with two digit planes, and the group's scale - known to that lane, which decoded the
// group - is applied locally: no shuffles, no shared memory, nothing per MMA. Two MMAs (digit
// planes 3,2 and 1,0) share one decoded A fragment.
//
// Data movement. A tile is 16 (or 32) consecutive matrix rows = one contiguous byte range, fetched
// by ONE bulk copy (cp.async.bulk + mbarrier) into a ring of stages - or, for decoders whose loads would
// otherwise meet the 8 rows of an MMA fragment on the same shared-memory banks (row sizes that are
// multiples of 128 bytes), by one bulk copy per row into rows spaced row bytes + Dec::kRowPad apart; a control warp issues the
// copies, and afterwards adds the K-slice partial sums of each tile in a fixed order, applies
// additive / bf16 rounding and stores the results. Consumer warp w decodes K-slice w of the
// staged rows straight from shared memory.
//
// IQ2_XXS tables. Codebook and sign lookups return PRMT selectors; both tables are replicated per
// lane (entry i of lane l at byte 256*i + 4*l, signs 128 bytes further) so that a warp's 32
// random lookups never share a bank, and they sit on a 64 KiB boundary of the shared window so
// that ONE byte permute builds a lookup address from the raw index byte. The 64 KiB image is a
// constant of the module and arrives by one bulk copy while the first tiles are in flight.
#pragma once
#include <cstdlib>
#include <type_traits>

#include "moe_common.cuh"
#include "qtype_decode.cuh"
#include "tcgen05.cuh"

namespace yb {
namespace gs {

constexpr int kMaxDepth = 6, kMaxConsumers = 16, kTileRows = 16;
constexpr uint32_t kTableBytes = 64 * 1024;

template <bool kFirst>
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (kFirst) {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// ---- the IQ2_XXS lookup image (constant of the module) ------------------------------------------------
constexpr uint32_t kIq2NibblesHost[256] = {
#include "iq2xxs_grid_nibbles.inc"
};
struct Iq2StreamTable { uint32_t w[kTableBytes / 4]; };
constexpr Iq2StreamTable make_iq2_stream_table() {
    Iq2StreamTable t{};
    for (int i = 0; i < 256; ++i) {
        // 7 stored sign bits + their parity as bit 7 (src/gguf/quant_block.c:378-386), spread to bit 2 of
        // each selector nibble; entry i and entry i ^ 128 are equal, so the index byte may carry a stray top bit
        uint32_t low7 = (uint32_t)i & 127u, parity = 0, spread = 0;
        for (int b = 0; b < 7; ++b) parity ^= (low7 >> b) & 1u;
        const uint32_t signs = low7 | (parity << 7);
        for (int l = 0; l < 8; ++l) spread |= ((signs >> l) & 1u) << (4 * l + 2);
        for (int l = 0; l < 32; ++l) {
            t.w[i * 64 + l] = kIq2NibblesHost[i];
            t.w[i * 64 + 32 + l] = spread;
        }
    }
    return t;
}
__device__ const Iq2StreamTable kIq2StreamTable = make_iq2_stream_table();

// Loads by 32-bit shared-window address. Not volatile, so that the compiler may schedule them freely;
// every address they are given derives from a register that was redefined (an empty volatile asm)
// after the wait that made the data visible, which keeps them behind that wait.
__device__ __forceinline__ uint32_t lds32(uint32_t a) { uint32_t v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds16(uint32_t a) { uint16_t v; asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds8(uint32_t a) { uint32_t v; asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds64(uint32_t a) { uint2 v; asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// Byte permute as the hardware does it (the CUDA intrinsic first masks bit 3 of every selector nibble, one
// more instruction per call; the selectors used here never set it) and a right shift by a constant on the
// multiplier pipe instead of the half-rate integer pipe that the decode saturates.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <int kBits> __device__ __forceinline__ uint32_t shr_mul(uint32_t v) { return kBits ? __umulhi(v, 1u << (32 - kBits)) : v; }

__device__ __forceinline__ float ldsf(uint32_t a) { float v; asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a)); return v; }
// A block scale is acceptable when it is a finite, non-negative f16: as an unsigned pattern, anything above
// 65504.0f is larger than that, infinite, NaN or negative.
__device__ __forceinline__ bool scale_bad(float d) { return __float_as_uint(d) > 0x477fe000u; }

// ---- per-lane state shared by the decoders ---------------------------------------------------------------
struct Lane {
    int g, t;                         // MMA row (and row + 8) / quad lane = group within a half block
    uint32_t nib_base, sgn_base;      // IQ2_XXS: table address with the lane's bank in byte 0, index byte still 0
};

// The B operand of one 256-weight unit: bh[4h + j] / bl[4h + j] are this lane's fragments of digit planes
// (3,2) / (1,0) for half h, subgroup j - non-zero only in the lane that owns the column's group.
struct BUnit { uint2 bh[8], bl[8]; };

__device__ __forceinline__ float comb(int a_hi, int a_lo, int b_hi, int b_lo) {
    return fmaf((float)(a_hi * 128 + a_lo), 16384.0f, (float)(b_hi * 128 + b_lo));
}

// What a decoder provides:
//   kBlockBytes / kBlockK   bytes and weights of the unit a warp walks (IQ2_XXS, Q4_K: one 256-weight
//                           superblock; Q8_0: eight 32-weight blocks, so that every qtype has 8 groups per unit)
//   unit(...)               adds this lane's share of the dot products of rows g and g + 8 with the
//                           activation over one unit to acc[0] / acc[1] (in units of 2^-27 * x scale);
//                           bad bit 0 / 1: a malformed block scale in row g / g + 8
struct StreamIq2 {
    static constexpr unsigned kQtype = Q_IQ2_XXS;
    static constexpr int kBlockBytes = 66, kBlockK = 256;
    static constexpr bool kTables = true;
    static constexpr int kSumGroup = 0;                  // activation sums over this many values (0: none needed)
    static constexpr bool kInterleave = false;           // order of the activation digits within a group of 32 (see StreamMxfp4)
    static constexpr bool kParity = false;               // unit<1> for odd units of a row, unit<0> for even ones
    static constexpr int kRowPad = 0;                    // bytes between the rows of a stage (0: the tile arrives as one copy)

    __device__ __forceinline__ static void group(uint32_t a, uint32_t &grids, uint32_t &ss) {
        // a group starts on a 2-byte boundary: three aligned words, funnel-shifted when it sits mid-word
        const uint32_t sh = (a & 2u) * 8u, w = a & ~3u;
        const uint32_t w0 = lds32(w), w1 = lds32(w + 4), w2 = lds32(w + 8);
        grids = __funnelshift_r(w0, w1, sh);
        ss = __funnelshift_r(w1, w2, sh);
    }
    // One subgroup of 8 weights -> two registers of signed bytes.
    template <int J> __device__ __forceinline__ static void sub(uint32_t grids, uint32_t ss, const Lane &l, uint32_t &lo, uint32_t &hi) {
        constexpr uint32_t kPos = 8u | (25u << 8) | (43u << 16), kNeg = 0xf8u | (0xe7u << 8) | (0xd5u << 16);
        const uint32_t na = prmt(grids, l.nib_base, 0x7604u | ((uint32_t)J << 4));
        const uint32_t sa = prmt(shr_mul<7 * J>(ss), l.sgn_base, 0x7604u);
        uint32_t nib, sgn;
        // reads of a table that never changes once it has arrived: free to be scheduled anywhere after
        // the point where the lane's table base registers were (re)defined, i.e. after the arrival wait
        asm("ld.shared.u32 %0, [%1];" : "=r"(nib) : "r"(na));
        asm("ld.shared.u32 %0, [%1];" : "=r"(sgn) : "r"(sa));
        const uint32_t sel = nib | sgn;
        lo = prmt(kPos, kNeg, sel);
        hi = prmt(kPos, kNeg, shr_mul<16>(sel));
    }
    // Everything below is written out over compile-time (half, subgroup) indices: the table addresses, shift
    // counts and fragment registers are then all static.
    template <int H, int J> __device__ __forceinline__ static void step(uint32_t g0, uint32_t s0, uint32_t g1, uint32_t s1, const BUnit &b,
                                                                        const Lane &l, int (&ca)[4], int (&cb)[4]) {
        uint32_t a[4];
        sub<J>(g0, s0, l, a[0], a[2]);
        sub<J>(g1, s1, l, a[1], a[3]);
        mma_s8<J == 0>(ca, a, b.bh[4 * H + J].x, b.bh[4 * H + J].y);
        mma_s8<J == 0>(cb, a, b.bl[4 * H + J].x, b.bl[4 * H + J].y);
    }
    template <int H> __device__ __forceinline__ static void half(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, float &blk0,
                                                                 float &blk1) {
        uint32_t g0, s0, g1, s1;
        group(row0 + 2 + 8 * (4 * H + l.t), g0, s0);
        group(row1 + 2 + 8 * (4 * H + l.t), g1, s1);
        int ca[4], cb[4];
        step<H, 0>(g0, s0, g1, s1, b, l, ca, cb);
        step<H, 1>(g0, s0, g1, s1, b, l, ca, cb);
        step<H, 2>(g0, s0, g1, s1, b, l, ca, cb);
        step<H, 3>(g0, s0, g1, s1, b, l, ca, cb);
        blk0 = fmaf(comb(ca[0], ca[1], cb[0], cb[1]), (float)((s0 >> 27) | 1u), blk0);       // 2 * sub + 1
        blk1 = fmaf(comb(ca[2], ca[3], cb[2], cb[3]), (float)((s1 >> 27) | 1u), blk1);
    }
    template <int> __device__ __forceinline__ static void unit(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t,
                                                float (&acc)[2], int &bad) {
        float blk0 = 0.0f, blk1 = 0.0f;
        half<0>(row0, row1, b, l, blk0, blk1);
        half<1>(row0, row1, b, l, blk0, blk1);
        const float f0 = f16_bits_to_float((uint16_t)lds16(row0)), f1 = f16_bits_to_float((uint16_t)lds16(row1));
        bad |= (scale_bad(f0) ? 1 : 0) | (scale_bad(f1) ? 2 : 0);
        acc[0] = fmaf(blk0, 0.125f * f0, acc[0]);
        acc[1] = fmaf(blk1, 0.125f * f1, acc[1]);
    }
};

// Q4_K (extension; no reference decoder): 144 bytes = f16 d, f16 dmin, 12 bytes of 6-bit (scale, min)
// pairs, 128 bytes of 4-bit codes; chunk c (32 bytes) carries sub-block 2c in the low and 2c + 1 in
// the high nibbles. value = d * sc * code - dmin * m. Lane t of half h owns sub-block 4h + t.
struct StreamQ4k {
    static constexpr unsigned kQtype = Q_Q4_K;
    static constexpr int kBlockBytes = 144, kBlockK = 256;
    static constexpr bool kTables = false;
    static constexpr int kSumGroup = 32;
    static constexpr bool kInterleave = false, kParity = false;
    static constexpr int kRowPad = 0;                    // (64 measured: 2.3 KB row copies are slower than the conflicts they avoid)

    // 6-bit (scale, min) of sub-block j from the 12 packed bytes behind d and dmin (three aligned words)
    __device__ __forceinline__ static void scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int h, int t, uint32_t &sc, uint32_t &m) {
        if (h == 0) {                                   // sub-blocks 0..3: low six bits of bytes t and t + 4
            sc = (s0 >> (8 * t)) & 63u;
            m = (s1 >> (8 * t)) & 63u;
        } else {                                        // sub-blocks 4..7: nibbles of byte t + 8, top bits from bytes t and t + 4
            const uint32_t b = (s2 >> (8 * t)) & 255u;
            sc = (b & 15u) | (((s0 >> (8 * t + 6)) & 3u) << 4);
            m = (b >> 4) | (((s1 >> (8 * t + 6)) & 3u) << 4);
        }
    }
    template <int H, int J> __device__ __forceinline__ static void step(const uint32_t (&w0)[8], const uint32_t (&w1)[8], int shift,
                                                                        const BUnit &b, int (&ca)[4], int (&cb)[4]) {
        uint32_t a[4];
        a[0] = (w0[2 * J] >> shift) & 0x0f0f0f0fu; a[2] = (w0[2 * J + 1] >> shift) & 0x0f0f0f0fu;
        a[1] = (w1[2 * J] >> shift) & 0x0f0f0f0fu; a[3] = (w1[2 * J + 1] >> shift) & 0x0f0f0f0fu;
        mma_s8<J == 0>(ca, a, b.bh[4 * H + J].x, b.bh[4 * H + J].y);
        mma_s8<J == 0>(cb, a, b.bl[4 * H + J].x, b.bl[4 * H + J].y);
    }
    template <int H> __device__ __forceinline__ static void half(uint32_t row0, uint32_t row1, const uint4 &head0, const uint4 &head1,
                                                                 const BUnit &b, const Lane &l, uint32_t sums, float &blk0, float &blk1,
                                                                 float &min0, float &min1) {
        const int sb = 4 * H + l.t, shift = 4 * (sb & 1);
        const uint32_t c0 = row0 + 16 + 32 * (sb >> 1), c1 = row1 + 16 + 32 * (sb >> 1);
        const uint4 x0 = lds128(c0), x1 = lds128(c0 + 16), y0 = lds128(c1), y1 = lds128(c1 + 16);
        const uint32_t w0[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const uint32_t w1[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
        int ca[4], cb[4];
        step<H, 0>(w0, w1, shift, b, ca, cb);
        step<H, 1>(w0, w1, shift, b, ca, cb);
        step<H, 2>(w0, w1, shift, b, ca, cb);
        step<H, 3>(w0, w1, shift, b, ca, cb);
        uint32_t sc0, m0, sc1, m1;
        scale_min(head0.y, head0.z, head0.w, H, l.t, sc0, m0);
        scale_min(head1.y, head1.z, head1.w, H, l.t, sc1, m1);
        const float xs = ldsf(sums + 4 * sb);                    // sum of the activation over this sub-block, in the same units
        blk0 = fmaf(comb(ca[0], ca[1], cb[0], cb[1]), (float)sc0, blk0);
        blk1 = fmaf(comb(ca[2], ca[3], cb[2], cb[3]), (float)sc1, blk1);
        min0 = fmaf((float)m0, xs, min0);
        min1 = fmaf((float)m1, xs, min1);
    }
    template <int> __device__ __forceinline__ static void unit(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t sums,
                                                float (&acc)[2], int &bad) {
        float blk0 = 0.0f, blk1 = 0.0f, min0 = 0.0f, min1 = 0.0f;
        const uint4 head0 = lds128(row0), head1 = lds128(row1);          // d, dmin and the 12 scale bytes
        half<0>(row0, row1, head0, head1, b, l, sums, blk0, blk1, min0, min1);
        half<1>(row0, row1, head0, head1, b, l, sums, blk0, blk1, min0, min1);
        const float d0 = f16_bits_to_float((uint16_t)head0.x), n0 = f16_bits_to_float((uint16_t)(head0.x >> 16));
        const float d1 = f16_bits_to_float((uint16_t)head1.x), n1 = f16_bits_to_float((uint16_t)(head1.x >> 16));
        bad |= (scale_bad(d0) || scale_bad(n0) ? 1 : 0) | (scale_bad(d1) || scale_bad(n1) ? 2 : 0);
        acc[0] += fmaf(d0, blk0, -n0 * min0);
        acc[1] += fmaf(d1, blk1, -n1 * min1);
    }
};

// Q2_K (src/gguf/quant_block.c:769-817): 84 bytes = 16 bytes of (4-bit scale | 4-bit min << 4) per 16-weight
// sub-block, 64 bytes of 2-bit codes, f16 d, f16 dmin. Weight k = 128 h + 32 p + i (i < 32) is
// (q[32 h + i] >> 2 p) & 3 of sub-block 8 h + 2 p + (i >= 16): value = d * sc * code - dmin * m.
// Lane t of half h owns plane p = t, i.e. K indices 128 h + 32 t .. + 31: the same 32 code bytes for all four
// lanes, shifted by 2 t. Its two sub-blocks have different scales, so the codes are multiplied by their scale
// BEFORE the MMA (4 codes per word at once: 3 * 15 = 45 fits a byte); the group sum then needs no factor.
// Blocks are only 4-byte aligned, hence the word loads.
struct StreamQ2k {
    static constexpr unsigned kQtype = Q_Q2_K;
    static constexpr int kBlockBytes = 84, kBlockK = 256;
    static constexpr bool kTables = false;
    static constexpr int kSumGroup = 16;
    static constexpr bool kInterleave = false, kParity = false;
    static constexpr int kRowPad = 0;

    template <int H, int J> __device__ __forceinline__ static void step(const uint32_t (&w0)[8], const uint32_t (&w1)[8], int shift,
                                                                        uint32_t sc0, uint32_t sc1, const BUnit &b, int (&ca)[4],
                                                                        int (&cb)[4]) {
        uint32_t a[4];
        a[0] = ((w0[2 * J] >> shift) & 0x03030303u) * sc0; a[2] = ((w0[2 * J + 1] >> shift) & 0x03030303u) * sc0;
        a[1] = ((w1[2 * J] >> shift) & 0x03030303u) * sc1; a[3] = ((w1[2 * J + 1] >> shift) & 0x03030303u) * sc1;
        mma_s8<J == 0>(ca, a, b.bh[4 * H + J].x, b.bh[4 * H + J].y);
        mma_s8<J == 0>(cb, a, b.bl[4 * H + J].x, b.bl[4 * H + J].y);
    }
    template <int H> __device__ __forceinline__ static void half(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t sums,
                                                                 float &blk0, float &blk1, float &min0, float &min1) {
        uint32_t w0[8], w1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { w0[i] = lds32(row0 + 16 + 32 * H + 4 * i); w1[i] = lds32(row1 + 16 + 32 * H + 4 * i); }
        // scale bytes 8 H + 2 t and 8 H + 2 t + 1: a 16-bit field of word 2 H + (t >> 1)
        const uint32_t s0 = lds32(row0 + 8 * H + 4 * (l.t >> 1)) >> (16 * (l.t & 1)), s1 = lds32(row1 + 8 * H + 4 * (l.t >> 1)) >> (16 * (l.t & 1));
        const int shift = 2 * l.t;
        int ca[4], cb[4];
        step<H, 0>(w0, w1, shift, s0 & 15u, s1 & 15u, b, ca, cb);
        step<H, 1>(w0, w1, shift, s0 & 15u, s1 & 15u, b, ca, cb);
        step<H, 2>(w0, w1, shift, (s0 >> 8) & 15u, (s1 >> 8) & 15u, b, ca, cb);
        step<H, 3>(w0, w1, shift, (s0 >> 8) & 15u, (s1 >> 8) & 15u, b, ca, cb);
        const int sub = 8 * H + 2 * l.t;
        const float xa = ldsf(sums + 4 * sub), xb = ldsf(sums + 4 * sub + 4);       // activation sums over the two sub-blocks
        blk0 += comb(ca[0], ca[1], cb[0], cb[1]);
        blk1 += comb(ca[2], ca[3], cb[2], cb[3]);
        min0 = fmaf((float)((s0 >> 4) & 15u), xa, fmaf((float)((s0 >> 12) & 15u), xb, min0));
        min1 = fmaf((float)((s1 >> 4) & 15u), xa, fmaf((float)((s1 >> 12) & 15u), xb, min1));
    }
    template <int> __device__ __forceinline__ static void unit(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t sums,
                                                float (&acc)[2], int &bad) {
        float blk0 = 0.0f, blk1 = 0.0f, min0 = 0.0f, min1 = 0.0f;
        half<0>(row0, row1, b, l, sums, blk0, blk1, min0, min1);
        half<1>(row0, row1, b, l, sums, blk0, blk1, min0, min1);
        const uint32_t h0 = lds32(row0 + 80), h1 = lds32(row1 + 80);                 // d, dmin
        const float d0 = f16_bits_to_float((uint16_t)h0), n0 = f16_bits_to_float((uint16_t)(h0 >> 16));
        const float d1 = f16_bits_to_float((uint16_t)h1), n1 = f16_bits_to_float((uint16_t)(h1 >> 16));
        bad |= (scale_bad(d0) || scale_bad(n0) ? 1 : 0) | (scale_bad(d1) || scale_bad(n1) ? 2 : 0);
        acc[0] += fmaf(d0, blk0, -n0 * min0);
        acc[1] += fmaf(d1, blk1, -n1 * min1);
    }
};

// Q8_0 (src/gguf/quant_block.c:819-833): 34 bytes = f16 d + 32 int8. A unit is eight blocks (256 weights);
// lane t of half h owns block 4h + t, whose quants are the A operand as they are.
struct StreamQ80 {
    static constexpr unsigned kQtype = Q_Q8_0;
    static constexpr int kBlockBytes = 8 * 34, kBlockK = 256;
    static constexpr bool kTables = false;
    static constexpr int kSumGroup = 0;
    static constexpr bool kInterleave = false, kParity = false;
    static constexpr int kRowPad = 16;                   // word loads: eight rows on banks 4 apart meet two at a time instead of eight

    __device__ __forceinline__ static void block(uint32_t a, uint32_t (&q)[8], float &d, int &bad, int flag) {
        // the block starts on a 2-byte boundary: nine aligned words, funnel-shifted when it sits mid-word
        const uint32_t sh = (a & 2u) * 8u, w = a & ~3u;
        uint32_t v[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = lds32(w + 4 * i);
        const uint32_t head = __funnelshift_r(v[0], v[1], sh);
        d = f16_bits_to_float((uint16_t)head);
        bad |= scale_bad(d) ? flag : 0;
        // quants start 2 bytes into the block
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = sh ? v[i + 1] : __funnelshift_r(v[i], v[i + 1], 16);
    }
    template <int H, int J> __device__ __forceinline__ static void step(const uint32_t (&q0)[8], const uint32_t (&q1)[8], const BUnit &b,
                                                                        int (&ca)[4], int (&cb)[4]) {
        const uint32_t a[4] = {q0[2 * J], q1[2 * J], q0[2 * J + 1], q1[2 * J + 1]};
        mma_s8<J == 0>(ca, a, b.bh[4 * H + J].x, b.bh[4 * H + J].y);
        mma_s8<J == 0>(cb, a, b.bl[4 * H + J].x, b.bl[4 * H + J].y);
    }
    template <int H> __device__ __forceinline__ static void half(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, float (&acc)[2],
                                                                 int &bad) {
        uint32_t q0[8], q1[8];
        float d0, d1;
        block(row0 + 34 * (4 * H + l.t), q0, d0, bad, 1);
        block(row1 + 34 * (4 * H + l.t), q1, d1, bad, 2);
        int ca[4], cb[4];
        step<H, 0>(q0, q1, b, ca, cb);
        step<H, 1>(q0, q1, b, ca, cb);
        step<H, 2>(q0, q1, b, ca, cb);
        step<H, 3>(q0, q1, b, ca, cb);
        acc[0] = fmaf(comb(ca[0], ca[1], cb[0], cb[1]), d0, acc[0]);
        acc[1] = fmaf(comb(ca[2], ca[3], cb[2], cb[3]), d1, acc[1]);
    }
    template <int> __device__ __forceinline__ static void unit(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t,
                                                float (&acc)[2], int &bad) {
        half<0>(row0, row1, b, l, acc, bad);
        half<1>(row0, row1, b, l, acc, bad);
    }
};

// MXFP4 (src/backend/cuda/kernel_primitives.h:100-111): 17 bytes = an E8M0 scale byte e, then 16 bytes whose low
// nibbles are weights 0..15 and high nibbles weights 16..31; value = level(code) * 2^(e - 128), levels
// {0,1,2,3,4,6,8,12} with bit 3 of the code as the sign. A unit is eight blocks (136 bytes); lane t of half h owns
// block 4h + t.
//   Decode. A byte permute is a lookup of four 3-bit indices in an 8-byte pool, and an index nibble whose bit 3 is
// set returns the pool byte's sign bit replicated - zero for a pool of small positive bytes. So the raw data word
// as the selector looks up the non-negative codes (and yields 0 for the others), the word with every bit 3
// flipped looks up the negative ones in a second pool, and the OR of the two is the weight. The pools hold
// level + 16 and 16 - level, i.e. bytes 4..28, so both are positive; the 16 comes off again as 16 x the sum of the
// group's activation digits (the same sums the Q4_K minimum term uses).
//   Order. The low 16 bits of a data word select for output bytes (w_i, w_16+i, w_i+1, w_17+i): nibble order, not
// weight order. Rather than sort the bytes, the activation digits of a group are stored in that order
// (kInterleave): position 8 j + 2 i + hi <- weight 16 hi + 4 j + i.
//   Alignment. A row is a multiple of 272 bytes (an even number of units, checked by the host), so a unit starts
// 0 or 8 bytes past a 16-byte boundary, the same for every row of a stage: unit<0> / unit<1>. Block b starts b
// bytes into the 16-byte chunk at 16 b (0 mod 16 units) and its 17 bytes end within 24: one 16-byte and one
// 8-byte load, in the order the alignment allows, give six words of which five are used from word h on.
struct StreamMxfp4 {
    static constexpr unsigned kQtype = Q_MXFP4;
    static constexpr int kBlockBytes = 8 * 17, kBlockK = 256;
    static constexpr bool kTables = false;
    static constexpr int kSumGroup = 32;
    static constexpr bool kInterleave = true, kParity = true;
    static constexpr int kRowPad = 0;

    template <int H, int kOdd> __device__ __forceinline__ static void block(uint32_t unit, int t, uint32_t (&x)[4], float &scale, int &bad,
                                                                            int flag) {
        const uint32_t at = unit + 16u * (uint32_t)(4 * H + t);
        uint32_t w[6];
        if (kOdd) {
            const uint2 lo = lds64(at);
            const uint4 hi = lds128(at + 8);
            w[0] = lo.x; w[1] = lo.y; w[2] = hi.x; w[3] = hi.y; w[4] = hi.z; w[5] = hi.w;
        } else {
            const uint4 lo = lds128(at);
            const uint2 hi = lds64(at + 16);
            w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w; w[4] = hi.x; w[5] = hi.y;
        }
        const uint32_t e = (w[H] >> (8 * t)) & 255u;
        bad |= e == 255u ? flag : 0;
        scale = __uint_as_float(e ? e << 23 : 0x00400000u) * 0.5f;
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = __funnelshift_rc(w[H + i], w[H + i + 1], 8 * (t + 1));
    }
    // eight codes of one data word -> two registers of bytes level + 16
    __device__ __forceinline__ static void codes(uint32_t x, uint32_t &lo, uint32_t &hi) {
        constexpr uint32_t kP0 = 0x13121110u, kP1 = 0x1c181614u;        // 16 + {0,1,2,3}, 16 + {4,6,8,12}
        constexpr uint32_t kN0 = 0x0d0e0f10u, kN1 = 0x04080a0cu;        // 16 - the same
        const uint32_t xf = x ^ 0x88888888u;
        lo = prmt(kP0, kP1, x) | prmt(kN0, kN1, xf);
        hi = prmt(kP0, kP1, x >> 16) | prmt(kN0, kN1, xf >> 16);
    }
    template <int H, int J> __device__ __forceinline__ static void step(const uint32_t (&x0)[4], const uint32_t (&x1)[4], const BUnit &b,
                                                                        int (&ca)[4], int (&cb)[4]) {
        uint32_t a[4];
        codes(x0[J], a[0], a[2]);
        codes(x1[J], a[1], a[3]);
        mma_s8<J == 0>(ca, a, b.bh[4 * H + J].x, b.bh[4 * H + J].y);
        mma_s8<J == 0>(cb, a, b.bl[4 * H + J].x, b.bl[4 * H + J].y);
    }
    template <int H, int kOdd> __device__ __forceinline__ static void half(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l,
                                                                           uint32_t sums, float (&acc)[2], int &bad) {
        uint32_t x0[4], x1[4];
        float s0, s1;
        block<H, kOdd>(row0, l.t, x0, s0, bad, 1);
        block<H, kOdd>(row1, l.t, x1, s1, bad, 2);
        int ca[4], cb[4];
        step<H, 0>(x0, x1, b, ca, cb);
        step<H, 1>(x0, x1, b, ca, cb);
        step<H, 2>(x0, x1, b, ca, cb);
        step<H, 3>(x0, x1, b, ca, cb);
        const float off = 16.0f * ldsf(sums + 4 * (4 * H + l.t));        // 16 x the sum of the activation over this block
        acc[0] = fmaf(comb(ca[0], ca[1], cb[0], cb[1]) - off, s0, acc[0]);
        acc[1] = fmaf(comb(ca[2], ca[3], cb[2], cb[3]) - off, s1, acc[1]);
    }
    template <int kOdd> __device__ __forceinline__ static void unit(uint32_t row0, uint32_t row1, const BUnit &b, const Lane &l, uint32_t sums,
                                                                    float (&acc)[2], int &bad) {
        half<0, kOdd>(row0, row1, b, l, sums, acc, bad);
        half<1, kOdd>(row0, row1, b, l, sums, acc, bad);
    }
};

// ---- kernel ------------------------------------------------------------------------------------------------
struct StreamParams {
    const uint8_t *enc;
    uint64_t matrix_stride;             // bytes from one matrix to the next
    uint32_t count;                     // matrices
    // optional device tables for matrices that are not evenly spaced (the experts a router picked):
    // matrix m starts at matrix_ptrs[m] (16-byte aligned, or the launch reports status 2) and reads
    // input row x_rows[m]; consecutive matrices with the same input row share one activation preparation
    const uint8_t *const *matrix_ptrs;
    const uint32_t *x_rows;
    uint64_t rows, row_bytes;
    uint32_t pitch;                     // bytes from one row of a stage to the next (row_bytes, or more when the rows are copied one by one)
    int K, slices, units_per_slice, row_warps, depth;      // consumer warps = slices x row_warps
    uint32_t stage_bytes, smem_bytes;
    const float *x;                     // input vector of matrix m at x + m * x_stride
    uint64_t x_stride;
    // optional: the input of matrix m is bf16(SwiGLU(x row, x_up row) * x_weight[m]) with the clamp x_limit
    // (src/graph/moe.c:605-613), x_up rows spaced like the x rows; formed while the planes are prepared
    const float *x_up;
    const float *x_weight;
    float x_limit;
    const float *additive;              // optional, laid out like out
    float *out;                         // result of matrix m at out + m * out_stride
    uint64_t out_stride;
    int round_bf16;
    int *status;
};

constexpr int kMaxGroupsPerWarp = 2;    // 16-row groups one consumer warp decodes per stage (independent work in flight)

struct StreamCtl {
    uint64_t full[kMaxDepth], empty[kMaxDepth], red_full[kMaxDepth + 1], tab_full;
    uint32_t stage[kMaxDepth];          // shared-window addresses
    uint32_t planes, zeros, sums, red, table;
    float xscale[8], warp_max[kMaxConsumers];
    int abort, layout_bad;
};

__host__ __device__ inline uint32_t stream_small_bytes(int K, int consumers, int depth, int units_per_slice, int groups) {
    return (uint32_t)(4 * K + 256 * units_per_slice + 128 + (K / 16) * 4 + 128 + (depth + 1) * consumers * groups * kTileRows * 4 + 256);
}

// The task list of one CTA, walked without divisions: tile `tile` of matrix `m`.
struct TaskCursor {
    uint32_t m;
    uint64_t tile, tiles_m;
    __device__ __forceinline__ void init(uint64_t q, uint64_t per_matrix) { tiles_m = per_matrix; m = (uint32_t)(q / per_matrix); tile = q - (uint64_t)m * per_matrix; }
    __device__ __forceinline__ void next() { if (++tile == tiles_m) { tile = 0; ++m; } }
};

// kBReg: the warp's whole K-slice is one unit, so its B fragments live in registers from one matrix change to the next.
// kGroupsPerWarp: 16-row groups a consumer warp decodes per stage.
template <class Dec, bool kBReg, int kGroupsPerWarp>
__global__ void __launch_bounds__(32 * (kMaxConsumers + 1), 1) gemv_stream_kernel(const StreamParams p) {
    using namespace sm100;
    extern __shared__ __align__(128) uint8_t dyn[];
    __shared__ StreamCtl ctl;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int consumers = p.slices * p.row_warps;
    const int D = p.depth;
    const uint32_t warp_rows = (uint32_t)(kTileRows * kGroupsPerWarp), tile_rows = warp_rows * (uint32_t)p.row_warps;
    const uint64_t tiles_m = (p.rows + tile_rows - 1) / tile_rows, Q = (uint64_t)p.count * tiles_m;
    const uint64_t q0 = Q * blockIdx.x / gridDim.x, q1 = Q * (blockIdx.x + 1) / gridDim.x;
    const uint32_t n_local = (uint32_t)(q1 - q0);
    // Launched with programmatic stream serialization: this CTA may start while the kernel before it on the stream still
    // runs. Everything up to pdl_wait() (shared-memory layout, barriers, the table image, which is a constant) touches
    // nothing that kernel could write; the kernel after this one may be scheduled as soon as SMs come free.
    pdl_trigger();

    if (threadIdx.x == 0) {
        // placement: a bump allocator over the dynamic window that steps over the 64 KiB-aligned table window
        const uint32_t base = smem_u32(dyn), end = base + p.smem_bytes;
        const uint32_t tab = Dec::kTables ? (base + 0xffffu) & ~0xffffu : end;
        uint32_t cur = base;
        auto take = [&](uint32_t bytes) {
            cur = (cur + 127u) & ~127u;
            if (Dec::kTables && cur < tab + kTableBytes && cur + bytes > tab) cur = tab + kTableBytes;
            const uint32_t at = cur;
            cur += bytes;
            return at;
        };
        for (int i = 0; i < D; ++i) ctl.stage[i] = take(p.stage_bytes + 16);
        ctl.planes = take((uint32_t)(4 * p.K));
        ctl.zeros = take((uint32_t)(256 * p.units_per_slice + 16));
        ctl.sums = take((uint32_t)(p.K / 16) * 4u);
        ctl.red = take((uint32_t)((D + 1) * consumers * kGroupsPerWarp * kTileRows) * 4u);
        ctl.table = tab;
        ctl.layout_bad = cur > end || (Dec::kTables && tab + kTableBytes > end);
        ctl.abort = 0;
        for (int i = 0; i < D; ++i) { mbar_init(&ctl.full[i], 1); mbar_init(&ctl.empty[i], (uint32_t)consumers); }
        for (int i = 0; i <= D; ++i) mbar_init(&ctl.red_full[i], (uint32_t)consumers);
        mbar_init(&ctl.tab_full, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (ctl.layout_bad) {                                    // uniform: nothing is in flight yet
        if (threadIdx.x == 0) raise(p.status, YVEX_B200_STATUS_ARGUMENT);
        return;
    }
    auto generic = [&](uint32_t shared_addr) { return dyn + (shared_addr - smem_u32(dyn)); };
    auto rows_of = [&](const TaskCursor &c, uint64_t &row0) {
        row0 = c.tile * tile_rows;
        return (uint32_t)(p.rows - row0 < tile_rows ? p.rows - row0 : tile_rows);
    };

    if (warp == consumers) {
        // ---------------- control warp: copies in, results out ----------------
        if (Dec::kTables && lane == 0 && n_local) {
            mbar_expect_tx(&ctl.tab_full, kTableBytes);
            bulk_load(generic(ctl.table), &kIq2StreamTable, kTableBytes, &ctl.tab_full);
        }
        pdl_wait();                                          // matrix tables, weights and inputs may come from the kernel before
        TaskCursor ci, cj;                                   // next tile to fetch / next tile to publish
        ci.init(q0, tiles_m);
        cj.init(q0, tiles_m);
        uint32_t issued = 0, i_slot = 0, i_phase = 0, j_buf = 0, j_phase = 0;      // i_phase = (issued / D) & 1, j_phase = (j / (D + 1)) & 1
        bool ok = true;
        const int per_tile = consumers * kGroupsPerWarp * kTileRows;
        for (uint32_t j = 0; j < n_local && ok; ++j, cj.next()) {
            while (issued < n_local && issued < j + (uint32_t)D && ok) {
                const uint32_t slot = i_slot;               // issued % D; its previous use was one ring turn ago
                if (issued >= (uint32_t)D) ok = mbar_wait_warp<kTryWaitHintNs>(&ctl.empty[slot], i_phase ^ 1u, &ctl.abort);
                if (!ok) break;
                uint64_t row0;
                const uint32_t nrows = rows_of(ci, row0);
                const uint8_t *mat = p.matrix_ptrs ? p.matrix_ptrs[ci.m] : p.enc + (uint64_t)ci.m * p.matrix_stride;
                if (reinterpret_cast<uintptr_t>(mat) & 15u) {            // a bulk copy from there would fault: refuse instead
                    if (lane == 0) { raise(p.status, YVEX_B200_STATUS_ARGUMENT); ctl.abort = 1; }
                    ok = false;
                    break;
                }
                const uint8_t *src = mat + row0 * p.row_bytes;
                uint8_t *dst = generic(ctl.stage[slot]);
                if (p.pitch != (uint32_t)p.row_bytes) {
                    // one copy per row (rows are multiples of 16 bytes here), all counted by the same barrier
                    if (lane == 0) mbar_expect_tx(&ctl.full[slot], (uint32_t)(nrows * p.row_bytes));
                    __syncwarp();
                    for (uint32_t r = (uint32_t)lane; r < nrows; r += 32)
                        bulk_load(dst + (size_t)r * p.pitch, src + (uint64_t)r * p.row_bytes, (uint32_t)p.row_bytes, &ctl.full[slot]);
                } else {
                    const uint32_t bytes = (uint32_t)(nrows * p.row_bytes), bulk = bytes & ~15u;
                    if (lane < (int)(bytes - bulk)) dst[bulk + lane] = __ldg(src + bulk + lane);      // the last < 16 bytes of a ragged tile
                    __syncwarp();
                    if (lane == 0) {
                        mbar_expect_tx(&ctl.full[slot], bulk);
                        if (bulk) bulk_load(dst, src, bulk, &ctl.full[slot]);
                    }
                }
                ++issued;
                if (++i_slot == (uint32_t)D) { i_slot = 0; i_phase ^= 1u; }
                ci.next();
            }
            if (!ok) break;
            const uint32_t buf = j_buf;
            ok = mbar_wait_warp<kTryWaitHintNs>(&ctl.red_full[buf], j_phase, &ctl.abort);
            if (++j_buf == (uint32_t)(D + 1)) { j_buf = 0; j_phase ^= 1u; }
            if (!ok) break;
            uint64_t row0;
            const uint32_t nrows = rows_of(cj, row0);
            // partial sums of the tile: [row warp][slice][group][16 rows]
            const float *red = reinterpret_cast<const float *>(generic(ctl.red)) + (size_t)buf * per_tile;
            const float scale = ctl.xscale[cj.m & 7u];
            for (uint32_t r = lane; r < nrows; r += 32) {
                const uint32_t rw = r / warp_rows, in_warp = r % warp_rows;
                float sum = 0.0f;
                for (int s = 0; s < p.slices; ++s) sum += red[((size_t)rw * p.slices + s) * warp_rows + in_warp];        // fixed order
                sum *= scale;
                const uint64_t at = (uint64_t)cj.m * p.out_stride + row0 + r;
                if (p.additive) sum += p.additive[at];
                if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                p.out[at] = p.round_bf16 ? bf16_round(sum) : sum;
            }
        }
        if (!ok && lane == 0) {
            // copies still in flight land in this CTA's shared memory: give them a bounded time to finish
            int ignore = 0;
            if (Dec::kTables) mbar_wait<kTryWaitHintNs>(&ctl.tab_full, 0u, &ignore);
            raise(p.status, YVEX_B200_STATUS_TIMEOUT);
        }
        return;
    }
    if (warp > consumers) return;

    // ---------------- consumer warps ----------------
    pdl_wait();
    Lane l;
    l.g = lane >> 2; l.t = lane & 3;
    const int sl = warp % p.slices, rw = warp / p.slices;
    const int unit0 = sl * p.units_per_slice, nunits_total = p.K / Dec::kBlockK;
    const int my_units = min(p.units_per_slice, nunits_total - unit0);
    const bool b_active = (lane & 3) == (lane >> 3);                        // column n = lane >> 2 belongs to group n >> 1
    // column 2t' carries the higher plane of a pair, column 2t' + 1 the lower one
    const int col_plane = (lane >> 2) & 1;
    uint32_t b_hi = b_active ? ctl.planes + (uint32_t)((0 + col_plane) * p.K + unit0 * Dec::kBlockK + 32 * (lane >> 3)) : ctl.zeros;
    uint32_t b_lo = b_active ? ctl.planes + (uint32_t)((2 + col_plane) * p.K + unit0 * Dec::kBlockK + 32 * (lane >> 3)) : ctl.zeros;
    l.nib_base = (ctl.table & 0xffff0000u) | (uint32_t)(lane * 4);
    l.sgn_base = l.nib_base + 128u;
    constexpr int kSumsPerUnit = Dec::kSumGroup ? Dec::kBlockK / Dec::kSumGroup : 0;
    uint32_t sums = ctl.sums + (uint32_t)(unit0 * kSumsPerUnit * 4);
    const uint32_t row_bytes = p.pitch;                                    // stage rows, as the consumers see them
    float *red_all = reinterpret_cast<float *>(generic(ctl.red));
    const int cthreads = consumers * 32;
    if (threadIdx.x < 64 * p.units_per_slice + 4) reinterpret_cast<uint32_t *>(generic(ctl.zeros))[threadIdx.x] = 0u;
    auto load_b = [&](BUnit &b, int u) {
#pragma unroll
        for (int hj = 0; hj < 8; ++hj) {
            const uint32_t k = (uint32_t)(u * Dec::kBlockK + 128 * (hj >> 2) + 8 * (hj & 3));
            b.bh[hj] = lds64(b_hi + k);
            b.bl[hj] = lds64(b_lo + k);
        }
    };

    // A warp whose wait ran out keeps walking the task list without touching data, so that it still
    // meets the other consumers at the named barriers of every matrix change and nobody waits for it.
    bool dead = false;
    if (Dec::kTables && n_local) {
        if (!mbar_wait_warp<kTryWaitHintNs>(&ctl.tab_full, 0u, &ctl.abort)) dead = true;
        asm volatile("" : "+r"(l.nib_base), "+r"(l.sgn_base));      // table reads may not move above this point
    }
    BUnit breg;
    uint32_t cur_m = 0xffffffffu, cur_x = 0xffffffffu;
    TaskCursor c;
    c.init(q0, tiles_m);
    uint32_t c_slot = 0, c_buf = 0, c_phase = 0;
    for (uint32_t i = 0; i < n_local; ++i, c.next()) {
        uint64_t row0;
        const uint32_t nrows = rows_of(c, row0);
        if (c.m != cur_m && cur_m != 0xffffffffu && p.x_rows && __ldg(p.x_rows + c.m) == cur_x) {
            // the next matrix reads the same input row: the planes, sums and B registers stand as they are
            if (threadIdx.x == 0) ctl.xscale[c.m & 7u] = ctl.xscale[cur_m & 7u];
            cur_m = c.m;
        }
        if (c.m != cur_m) {
            // a new matrix: its activation row becomes four planes of signed base-128 digits. Every
            // consumer has finished the previous matrix once it is past this barrier.
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            cur_x = p.x_rows ? __ldg(p.x_rows + c.m) : c.m;
            const float *x = p.x + (uint64_t)cur_x * p.x_stride;
            float mx = 0.0f;
            bool badx = false;
            const float *xu = p.x_up ? p.x_up + (uint64_t)cur_x * p.x_stride : nullptr;
            const float xw = p.x_up ? __ldg(p.x_weight + c.m) : 1.0f;
            for (int k = threadIdx.x; k < p.K; k += cthreads) {
                float v = __ldg(x + k);
                if (xu) v = swiglu_mid(v, __ldg(xu + k), xw, p.x_limit, p.status);
                badx |= !isfinite(v);
                mx = fmaxf(mx, fabsf(v));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0) ctl.warp_max[warp] = mx;
            if (badx) raise(p.status, YVEX_B200_STATUS_NUMERIC);
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            mx = 0.0f;
            for (int w = 0; w < consumers; ++w) mx = fmaxf(mx, ctl.warp_max[w]);
            // S = the power of two above the largest magnitude; q = rint(x / S * 2^27), |q| <= 2^27
            int e = 0;
            if (mx > 0.0f && isfinite(mx)) frexpf(mx, &e);
            const float to_q = ldexpf(1.0f, 27 - e);
            if (threadIdx.x == 0) ctl.xscale[c.m & 7u] = ldexpf(1.0f, e - 27);
            int8_t *pl = reinterpret_cast<int8_t *>(generic(ctl.planes));
            float *sm = reinterpret_cast<float *>(generic(ctl.sums));
            for (int k8 = threadIdx.x; k8 < p.K / 8; k8 += cthreads) {
                uint32_t d[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};
                float s = 0.0f;
                const float4 xa = __ldg(reinterpret_cast<const float4 *>(x + 8 * k8)), xb = __ldg(reinterpret_cast<const float4 *>(x + 8 * k8) + 1);
                float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                if (xu) {
                    const float4 ua = __ldg(reinterpret_cast<const float4 *>(xu + 8 * k8)), ub = __ldg(reinterpret_cast<const float4 *>(xu + 8 * k8) + 1);
                    const float uv[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
                    for (int i8 = 0; i8 < 8; ++i8) xv[i8] = swiglu_mid(xv[i8], uv[i8], xw, p.x_limit, p.status);
                }
#pragma unroll
                for (int i8 = 0; i8 < 8; ++i8) {
                    int q = isfinite(xv[i8]) ? __float2int_rn(xv[i8] * to_q) : 0;
                    s += (float)q;
                    // balanced digits: d0..d2 in [-64, 63], the top digit takes what is left (|d3| <= 64)
                    const int d0 = ((q + 64) & 127) - 64; q = (q - d0) >> 7;
                    const int d1 = ((q + 64) & 127) - 64; q = (q - d1) >> 7;
                    const int d2 = ((q + 64) & 127) - 64; q = (q - d2) >> 7;
                    const int dig[4] = {q, d2, d1, d0};                     // plane 0 is the most significant
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi) d[pi][i8 >> 2] |= (uint32_t)(dig[pi] & 0xff) << (8 * (i8 & 3));
                }
                if (Dec::kInterleave) {
                    // lanes s and s + 2 of a quad hold weights 8 s .. and 16 + 8 s ..: lane s builds the 8-byte chunk 2 s
                    // (its own first word and the partner's, bytes alternating), lane s + 2 chunk 2 s + 1 (the second words)
                    const int sub = k8 & 3;
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi) {
                        const uint32_t got = __shfl_xor_sync(0xffffffffu, sub < 2 ? d[pi][1] : d[pi][0], 2);
                        const uint32_t lo = sub < 2 ? d[pi][0] : got, hi = sub < 2 ? got : d[pi][1];
                        const int chunk = sub < 2 ? 2 * sub : 2 * (sub - 2) + 1;
                        *reinterpret_cast<uint2 *>(pl + (size_t)pi * p.K + 32 * (k8 >> 2) + 8 * chunk) =
                            make_uint2(prmt(lo, hi, 0x5140u), prmt(lo, hi, 0x7362u));
                    }
                } else {
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi)
                        *reinterpret_cast<uint2 *>(pl + (size_t)pi * p.K + 8 * k8) = make_uint2(d[pi][0], d[pi][1]);
                }
                if (Dec::kSumGroup == 32) {
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if ((threadIdx.x & 3) == 0) sm[k8 >> 2] = s;
                } else if (Dec::kSumGroup == 16) {
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    if ((threadIdx.x & 1) == 0) sm[k8 >> 1] = s;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            asm volatile("" : "+r"(b_hi), "+r"(b_lo), "+r"(sums));      // reads of the new planes stay behind the barrier
            if (kBReg) load_b(breg, 0);
            cur_m = c.m;
        }
        // stage i % D with phase (i / D) & 1 and result buffer i % (D + 1), kept as counters (no divisions in this loop)
        const uint32_t slot = c_slot, buf = c_buf;
        if (!dead && !mbar_wait_warp<kTryWaitHintNs>(&ctl.full[slot], c_phase, &ctl.abort)) dead = true;
        if (++c_slot == (uint32_t)D) { c_slot = 0; c_phase ^= 1u; }
        if (++c_buf == (uint32_t)(D + 1)) c_buf = 0;
        float acc[kGroupsPerWarp][2];
        int bad[kGroupsPerWarp];
#pragma unroll
        for (int gi = 0; gi < kGroupsPerWarp; ++gi) { acc[gi][0] = acc[gi][1] = 0.0f; bad[gi] = 0; }
        const uint32_t first = warp_rows * (uint32_t)rw;                     // this warp's first row within the tile
        if (!dead && first < nrows) {
            uint32_t base = ctl.stage[slot] + (first + (uint32_t)l.g) * row_bytes + (uint32_t)(unit0 * Dec::kBlockBytes);
            asm volatile("" : "+r"(base));                              // reads of the stage stay behind the wait above
            for (int u = 0; u < my_units; ++u) {
                BUnit bmem;
                if (!kBReg) load_b(bmem, u);
                const BUnit &b = kBReg ? breg : bmem;
                auto groups = [&](auto odd) {
#pragma unroll
                    for (int gi = 0; gi < kGroupsPerWarp; ++gi) {
                        // groups past a ragged tile's last row decode stale bytes; their results are never stored
                        const uint32_t r0 = base + (uint32_t)(kTileRows * gi) * row_bytes + (uint32_t)(u * Dec::kBlockBytes);
                        Dec::template unit<decltype(odd)::value>(r0, r0 + 8 * row_bytes, b, l, sums + (uint32_t)(u * kSumsPerUnit * 4), acc[gi],
                                                                 bad[gi]);
                    }
                };
                if (Dec::kParity && ((unit0 + u) & 1)) groups(std::integral_constant<int, 1>{});
                else groups(std::integral_constant<int, 0>{});
            }
        }
        // this warp is done with the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.empty[slot]);
        float *red = red_all + ((size_t)buf * consumers + warp) * warp_rows;
#pragma unroll
        for (int gi = 0; gi < kGroupsPerWarp; ++gi) {
            float a0 = acc[gi][0], a1 = acc[gi][1];
            a0 += __shfl_xor_sync(0xffffffffu, a0, 1); a0 += __shfl_xor_sync(0xffffffffu, a0, 2);
            a1 += __shfl_xor_sync(0xffffffffu, a1, 1); a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
            if (l.t == 0) { red[kTileRows * gi + l.g] = a0; red[kTileRows * gi + l.g + 8] = a1; }
            // a malformed block scale only counts for rows that exist
            const uint32_t r_lo = first + (uint32_t)(kTileRows * gi + l.g), r_hi = r_lo + 8;
            if (((bad[gi] & 1) && r_lo < nrows) || ((bad[gi] & 2) && r_hi < nrows)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.red_full[buf]);
    }
}

// ---- host side -----------------------------------------------------------------------------------------------
struct StreamShape { int slices, units_per_slice, row_warps, consumers, depth, groups; uint32_t stage_bytes, smem_bytes, pitch; };

// K-slices (consumer warps along K), units per slice, warps along the rows of a stage and the deepest ring that fits.
inline bool stream_shape(unsigned q, uint64_t width, uint64_t row_bytes, StreamShape &sh) {
    const bool tables = q == Q_IQ2_XXS;
    const int units = (int)(width / 256);
    if (!units || width % 256 || width > 8192) return false;
    if (q == Q_MXFP4 && units % 2) return false;           // its loads want rows that are multiples of 16 bytes
    sh.units_per_slice = (units + kMaxConsumers - 1) / kMaxConsumers;
    sh.slices = (units + sh.units_per_slice - 1) / sh.units_per_slice;
    sh.row_warps = sh.slices <= kMaxConsumers / 2 ? 2 : 1;
    sh.consumers = sh.slices * sh.row_warps;
    {
        const int pad = q == Q_Q4_K ? StreamQ4k::kRowPad : q == Q_Q8_0 ? StreamQ80::kRowPad : q == Q_MXFP4 ? StreamMxfp4::kRowPad : 0;
        // Padded rows help where the row size is a multiple of 128 bytes (every row of a fragment on the same banks) and a
        // row is large: an SM completes about 8.5 M bulk copies a second, so rows of 4352 bytes still stream at 5.5 TB/s
        // over the device while rows of 2304 bytes would be held to 2.9 TB/s.
        sh.pitch = (uint32_t)row_bytes + (pad && row_bytes % 128 == 0 && row_bytes >= 4096 ? (uint32_t)pad : 0u);
    }
    const uint32_t limit = 226u * 1024u;                   // the kernel also has a few hundred bytes of static shared memory
    // two row groups per warp when at least three such stages fit, else one
    for (sh.groups = kMaxGroupsPerWarp; sh.groups >= 1; --sh.groups) {
        sh.stage_bytes = (uint32_t)(kTileRows * sh.groups * sh.row_warps * sh.pitch);
        for (sh.depth = kMaxDepth; sh.depth >= (sh.groups > 1 ? 3 : 2); --sh.depth) {
            // every piece is rounded up to 128 bytes; with tables one piece may have to step over the table window,
            // which starts at most 64 KiB - 1 into the allocation (what lies before it stays usable)
            const uint32_t pieces = (uint32_t)sh.depth * (sh.stage_bytes + 16 + 128) +
                                    stream_small_bytes((int)width, sh.consumers, sh.depth, sh.units_per_slice, sh.groups) + 5 * 128;
            sh.smem_bytes = tables ? pieces + kTableBytes + sh.stage_bytes + 16 + 128 : pieces;
            if (tables && sh.smem_bytes < 2 * kTableBytes) sh.smem_bytes = 2 * kTableBytes;
            if (sh.smem_bytes <= limit) return true;
        }
    }
    return false;
}

inline bool stream_qtype(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q8_0 || q == Q_Q2_K || q == Q_MXFP4; }

inline bool stream_eligible(unsigned q, uint64_t rows, uint64_t width, uint64_t row_bytes, const void *enc, uint64_t matrix_stride,
                            uint64_t count, const float *x, uint64_t x_stride) {
    StreamShape sh;
    return stream_qtype(q) && rows && count && count <= 0xffffffffull && (reinterpret_cast<uintptr_t>(enc) & 15u) == 0 &&
           matrix_stride % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && x_stride % 4 == 0 &&
           stream_shape(q, width, row_bytes, sh);
}

template <class Dec, bool kBReg, int kG>
inline int stream_launch_v(StreamParams &p, const StreamShape &sh, cudaStream_t stream) {
    static SmemOptIn opt_in;
    if (opt_in.ensure(gemv_stream_kernel<Dec, kBReg, kG>, 226 * 1024) != OK) return ERR_BACKEND;
    const uint64_t tile_rows = (uint64_t)kTileRows * kG * sh.row_warps;
    const uint64_t tasks = (uint64_t)p.count * ((p.rows + tile_rows - 1) / tile_rows);
    const unsigned grid = (unsigned)(tasks < (uint64_t)kSmCount ? tasks : (uint64_t)kSmCount);
    if (launch_pdl(gemv_stream_kernel<Dec, kBReg, kG>, dim3(grid), dim3(32 * (sh.consumers + 1)), sh.smem_bytes, stream, p) != cudaSuccess)
        return ERR_BACKEND;
    return launch_status(1);
}

template <class Dec>
inline int stream_launch_t(StreamParams &p, const StreamShape &sh, cudaStream_t stream) {
    const bool breg = sh.units_per_slice == 1;
    if (sh.groups == 2) return breg ? stream_launch_v<Dec, true, 2>(p, sh, stream) : stream_launch_v<Dec, false, 2>(p, sh, stream);
    return breg ? stream_launch_v<Dec, true, 1>(p, sh, stream) : stream_launch_v<Dec, false, 1>(p, sh, stream);
}

struct StreamActivation { const float *up; const float *weight; float limit; };

inline int stream_launch(unsigned q, const uint8_t *enc, uint64_t matrix_stride, uint64_t count, uint64_t rows, uint64_t width,
                         uint64_t row_bytes, const float *x, uint64_t x_stride, const float *additive, float *out,
                         uint64_t out_stride, int round_bf16, int *status, cudaStream_t stream,
                         const uint8_t *const *matrix_ptrs = nullptr, const uint32_t *x_rows = nullptr,
                         const StreamActivation *act = nullptr) {
    StreamShape sh;
    if (!stream_shape(q, width, row_bytes, sh)) return ERR_BOUNDS;
    StreamParams p{};
    p.matrix_ptrs = matrix_ptrs; p.x_rows = x_rows;
    if (act) {
        if (x_rows || (reinterpret_cast<uintptr_t>(act->up) & 15u)) return ERR_INVALID_ARG;
        p.x_up = act->up; p.x_weight = act->weight; p.x_limit = act->limit;
    }
    p.enc = enc; p.matrix_stride = matrix_stride; p.count = (uint32_t)count; p.rows = rows; p.row_bytes = row_bytes;
    p.K = (int)width; p.slices = sh.slices; p.units_per_slice = sh.units_per_slice; p.row_warps = sh.row_warps; p.depth = sh.depth;
    p.stage_bytes = sh.stage_bytes; p.smem_bytes = sh.smem_bytes; p.pitch = sh.pitch;
    p.x = x; p.x_stride = x_stride; p.additive = additive; p.out = out; p.out_stride = out_stride;
    p.round_bf16 = round_bf16; p.status = status;
    switch (q) {
    case Q_IQ2_XXS: return stream_launch_t<StreamIq2>(p, sh, stream);
    case Q_Q4_K: return stream_launch_t<StreamQ4k>(p, sh, stream);
    case Q_Q8_0: return stream_launch_t<StreamQ80>(p, sh, stream);
    case Q_Q2_K: return stream_launch_t<StreamQ2k>(p, sh, stream);
    case Q_MXFP4: return stream_launch_t<StreamMxfp4>(p, sh, stream);
    default: return ERR_UNSUPPORTED;
    }
}

}  // namespace gs
}  // namespace yb
