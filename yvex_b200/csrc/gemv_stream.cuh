// Streaming dequant-fused matvec for block qtypes at HBM rate: one persistent CTA per SM walks a
// list of (matrix, 16-row tile) tasks, so one launch covers one large matrix or a batch of
// independent matrices with their own input vectors.
//
// Arithmetic. The weights enter the tensor cores as signed bytes (mma.sync.m16n8k32, s8 x s8 ->
// s32): IQ2_XXS +-{8,25,43}, Q4_K codes 0..15, Q8_0 its int8 quants. The f32 activation row is
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
// by ONE bulk copy (cp.async.bulk + mbarrier) into a ring of stages; a control warp issues the
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
#include "qtype_decode.cuh"
#include "tcgen05.cuh"

namespace yb {
namespace gs {

constexpr int kMaxDepth = 6, kMaxConsumers = 16, kTileRows = 16;
constexpr uint32_t kTableBytes = 64 * 1024;

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, bool first) {
    if (first) {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
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

// ---- per-lane state shared by the decoders ---------------------------------------------------------------
struct Lane {
    int g, t;                         // MMA row (and row + 8) / quad lane = group within a half block
    const uint8_t *b_hi, *b_lo;       // this lane's B source for digit planes (3,2) / (1,0) at k = 0 of its K-slice
    uint32_t nib_base, sgn_base;      // IQ2_XXS: table address with the lane's bank in byte 0, index byte still 0
};

// What a decoder provides:
//   kBlockBytes / kBlockK   bytes and weights of the unit a warp walks (IQ2_XXS, Q4_K: one 256-weight
//                           superblock; Q8_0: eight 32-weight blocks, so that every qtype has 8 groups per unit)
//   unit(...)               adds this lane's share of the dot products of rows g and g + 8 with the
//                           activation over one unit to acc[0] / acc[1] (in units of 2^-27 * x scale)
struct StreamIq2 {
    static constexpr unsigned kQtype = Q_IQ2_XXS;
    static constexpr int kBlockBytes = 66, kBlockK = 256;
    static constexpr bool kTables = true, kSums = false;

    __device__ __forceinline__ static void group(const uint8_t *p, uint32_t &grids, uint32_t &ss) {
        // a group starts on a 2-byte boundary: three aligned words, funnel-shifted when it sits mid-word
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t sh = (uint32_t)(a & 2u) * 8u;
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
        grids = __funnelshift_r(w0, w1, sh);
        ss = __funnelshift_r(w1, w2, sh);
    }
    // One subgroup of 8 weights -> two registers of signed bytes.
    template <int J> __device__ __forceinline__ static void sub(uint32_t grids, uint32_t ss, const Lane &l, uint32_t &lo, uint32_t &hi) {
        constexpr uint32_t kPos = 8u | (25u << 8) | (43u << 16), kNeg = 0xf8u | (0xe7u << 8) | (0xd5u << 16);
        const uint32_t na = __byte_perm(grids, l.nib_base, 0x7604u | ((uint32_t)J << 4));
        const uint32_t sa = __byte_perm(J ? ss >> (7 * J) : ss, l.sgn_base, 0x7604u);
        uint32_t nib, sgn;
        // reads of a table that never changes once it has arrived: free to be scheduled anywhere after
        // the point where the lane's table base registers were (re)defined, i.e. after the arrival wait
        asm("ld.shared.u32 %0, [%1];" : "=r"(nib) : "r"(na));
        asm("ld.shared.u32 %0, [%1];" : "=r"(sgn) : "r"(sa));
        const uint32_t sel = nib | sgn;
        lo = __byte_perm(kPos, kNeg, sel);
        hi = __byte_perm(kPos, kNeg, sel >> 16);
    }
    __device__ __forceinline__ static float comb(int a_hi, int a_lo, int b_hi, int b_lo) {
        return fmaf((float)(a_hi * 128 + a_lo), 16384.0f, (float)(b_hi * 128 + b_lo));
    }
    __device__ __forceinline__ static void unit(const uint8_t *row0, const uint8_t *row1, int kofs, const Lane &l, const float *,
                                                float (&acc)[2], int &bad) {
        float blk0 = 0.0f, blk1 = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t g0, s0, g1, s1;
            group(row0 + 2 + 8 * (4 * h + l.t), g0, s0);
            group(row1 + 2 + 8 * (4 * h + l.t), g1, s1);
            int ca[4], cb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a[4];
                switch (j) {
                case 0: sub<0>(g0, s0, l, a[0], a[2]); sub<0>(g1, s1, l, a[1], a[3]); break;
                case 1: sub<1>(g0, s0, l, a[0], a[2]); sub<1>(g1, s1, l, a[1], a[3]); break;
                case 2: sub<2>(g0, s0, l, a[0], a[2]); sub<2>(g1, s1, l, a[1], a[3]); break;
                default: sub<3>(g0, s0, l, a[0], a[2]); sub<3>(g1, s1, l, a[1], a[3]); break;
                }
                const int k = kofs + 128 * h + 8 * j;
                const uint2 bh = *reinterpret_cast<const uint2 *>(l.b_hi + k), bl = *reinterpret_cast<const uint2 *>(l.b_lo + k);
                mma_s8(ca, a, bh.x, bh.y, j == 0);
                mma_s8(cb, a, bl.x, bl.y, j == 0);
            }
            blk0 = fmaf(comb(ca[0], ca[1], cb[0], cb[1]), (float)((s0 >> 27) | 1u), blk0);       // 2 * sub + 1
            blk1 = fmaf(comb(ca[2], ca[3], cb[2], cb[3]), (float)((s1 >> 27) | 1u), blk1);
        }
        const float f0 = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(row0));
        const float f1 = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(row1));
        bad |= !(f0 >= 0.0f && f0 <= 65504.0f) ? 1 : 0;
        bad |= !(f1 >= 0.0f && f1 <= 65504.0f) ? 2 : 0;
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
    static constexpr bool kTables = false, kSums = true;

    __device__ __forceinline__ static void scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &m) {
        if (j < 4) { sc = s[j] & 63u; m = s[j + 4] & 63u; }
        else { sc = (s[j + 4] & 15u) | ((s[j - 4] >> 6) << 4); m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
    }
    __device__ __forceinline__ static void unit(const uint8_t *row0, const uint8_t *row1, int kofs, const Lane &l, const float *sums,
                                                float (&acc)[2], int &bad) {
        float blk0 = 0.0f, blk1 = 0.0f, min0 = 0.0f, min1 = 0.0f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int sb = 4 * h + l.t, shift = 4 * (sb & 1);
            const uint4 *q0 = reinterpret_cast<const uint4 *>(row0 + 16 + 32 * (sb >> 1));
            const uint4 *q1 = reinterpret_cast<const uint4 *>(row1 + 16 + 32 * (sb >> 1));
            const uint4 x0 = q0[0], x1 = q0[1], y0 = q1[0], y1 = q1[1];
            const uint32_t w0[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const uint32_t w1[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
            int ca[4], cb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a[4];
                a[0] = (w0[2 * j] >> shift) & 0x0f0f0f0fu; a[2] = (w0[2 * j + 1] >> shift) & 0x0f0f0f0fu;
                a[1] = (w1[2 * j] >> shift) & 0x0f0f0f0fu; a[3] = (w1[2 * j + 1] >> shift) & 0x0f0f0f0fu;
                const int k = kofs + 128 * h + 8 * j;
                const uint2 bh = *reinterpret_cast<const uint2 *>(l.b_hi + k), bl = *reinterpret_cast<const uint2 *>(l.b_lo + k);
                mma_s8(ca, a, bh.x, bh.y, j == 0);
                mma_s8(cb, a, bl.x, bl.y, j == 0);
            }
            uint32_t sc0, m0, sc1, m1;
            scale_min(row0 + 4, sb, sc0, m0);
            scale_min(row1 + 4, sb, sc1, m1);
            const float xs = sums[(kofs >> 5) + sb];                 // sum of the activation over this sub-block, in the same units
            blk0 = fmaf(StreamIq2::comb(ca[0], ca[1], cb[0], cb[1]), (float)sc0, blk0);
            blk1 = fmaf(StreamIq2::comb(ca[2], ca[3], cb[2], cb[3]), (float)sc1, blk1);
            min0 = fmaf((float)m0, xs, min0);
            min1 = fmaf((float)m1, xs, min1);
        }
        const uint32_t dd0 = *reinterpret_cast<const uint32_t *>(row0), dd1 = *reinterpret_cast<const uint32_t *>(row1);
        const float d0 = f16_bits_to_float((uint16_t)dd0), n0 = f16_bits_to_float((uint16_t)(dd0 >> 16));
        const float d1 = f16_bits_to_float((uint16_t)dd1), n1 = f16_bits_to_float((uint16_t)(dd1 >> 16));
        bad |= !(d0 >= 0.0f && d0 <= 65504.0f && n0 >= 0.0f && n0 <= 65504.0f) ? 1 : 0;
        bad |= !(d1 >= 0.0f && d1 <= 65504.0f && n1 >= 0.0f && n1 <= 65504.0f) ? 2 : 0;
        acc[0] += fmaf(d0, blk0, -n0 * min0);
        acc[1] += fmaf(d1, blk1, -n1 * min1);
    }
};

// Q8_0 (src/gguf/quant_block.c:819-833): 34 bytes = f16 d + 32 int8. A unit is eight blocks (256 weights);
// lane t of half h owns block 4h + t, whose quants are the A operand as they are.
struct StreamQ80 {
    static constexpr unsigned kQtype = Q_Q8_0;
    static constexpr int kBlockBytes = 8 * 34, kBlockK = 256;
    static constexpr bool kTables = false, kSums = false;

    __device__ __forceinline__ static void block(const uint8_t *p, uint32_t (&q)[8], float &d, int &bad, int flag) {
        // the block starts on a 2-byte boundary: nine aligned words, funnel-shifted when it sits mid-word
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t sh = (uint32_t)(a & 2u) * 8u;
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        uint32_t v[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = w[i];
        const uint32_t head = __funnelshift_r(v[0], v[1], sh);
        d = f16_bits_to_float((uint16_t)head);
        bad |= !(d >= 0.0f && d <= 65504.0f) ? flag : 0;
        // quants start 2 bytes into the block
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = sh ? v[i + 1] : __funnelshift_r(v[i], v[i + 1], 16);
    }
    __device__ __forceinline__ static void unit(const uint8_t *row0, const uint8_t *row1, int kofs, const Lane &l, const float *,
                                                float (&acc)[2], int &bad) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t q0[8], q1[8];
            float d0, d1;
            block(row0 + 34 * (4 * h + l.t), q0, d0, bad, 1);
            block(row1 + 34 * (4 * h + l.t), q1, d1, bad, 2);
            int ca[4], cb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a[4] = {q0[2 * j], q1[2 * j], q0[2 * j + 1], q1[2 * j + 1]};
                const int k = kofs + 128 * h + 8 * j;
                const uint2 bh = *reinterpret_cast<const uint2 *>(l.b_hi + k), bl = *reinterpret_cast<const uint2 *>(l.b_lo + k);
                mma_s8(ca, a, bh.x, bh.y, j == 0);
                mma_s8(cb, a, bl.x, bl.y, j == 0);
            }
            acc[0] = fmaf(StreamIq2::comb(ca[0], ca[1], cb[0], cb[1]), d0, acc[0]);
            acc[1] = fmaf(StreamIq2::comb(ca[2], ca[3], cb[2], cb[3]), d1, acc[1]);
        }
    }
};

// ---- kernel ------------------------------------------------------------------------------------------------
struct StreamParams {
    const uint8_t *enc;
    uint64_t matrix_stride;             // bytes from one matrix to the next
    uint32_t count;                     // matrices
    uint64_t rows, row_bytes;
    int K, slices, units_per_slice, row_groups, depth;
    uint32_t stage_bytes, smem_bytes;
    const float *x;                     // input vector of matrix m at x + m * x_stride
    uint64_t x_stride;
    const float *additive;              // optional, laid out like out
    float *out;                         // result of matrix m at out + m * out_stride
    uint64_t out_stride;
    int round_bf16;
    int *status;
};

struct StreamCtl {
    uint64_t full[kMaxDepth], empty[kMaxDepth], red_full[kMaxDepth + 1], tab_full;
    uint32_t stage[kMaxDepth];          // shared-window addresses
    uint32_t planes, zeros, sums, red, table;
    float xscale[8], warp_max[kMaxConsumers];
    int abort, layout_bad;
};

// Bytes of dynamic shared memory the kernel needs in the worst placement of the 64 KiB table window.
__host__ __device__ inline uint32_t stream_small_bytes(int K, int consumers, int depth, int units_per_slice) {
    return (uint32_t)(4 * K + 256 * units_per_slice + 128 + (K / 32) * 4 + 128 + (depth + 1) * consumers * kTileRows * 4 + 256);
}

template <class Dec>
__global__ void __launch_bounds__(32 * (kMaxConsumers + 1), 1) gemv_stream_kernel(const StreamParams p) {
    using namespace sm100;
    extern __shared__ __align__(128) uint8_t dyn[];
    __shared__ StreamCtl ctl;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int consumers = p.slices * p.row_groups;
    const int D = p.depth;
    const uint32_t tile_rows = (uint32_t)(kTileRows * p.row_groups);
    const uint64_t tiles_m = (p.rows + tile_rows - 1) / tile_rows, Q = (uint64_t)p.count * tiles_m;
    const uint64_t q0 = Q * blockIdx.x / gridDim.x, q1 = Q * (blockIdx.x + 1) / gridDim.x;
    const uint32_t n_local = (uint32_t)(q1 - q0);

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
        ctl.sums = take((uint32_t)(p.K / 32) * 4u);
        ctl.red = take((uint32_t)((D + 1) * consumers * kTileRows) * 4u);
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
    auto task = [&](uint32_t i, uint32_t &m, uint64_t &row0, uint32_t &nrows) {
        const uint64_t q = q0 + i;
        m = (uint32_t)(q / tiles_m);
        row0 = (q - (uint64_t)m * tiles_m) * tile_rows;
        nrows = (uint32_t)(p.rows - row0 < tile_rows ? p.rows - row0 : tile_rows);
    };

    if (warp == consumers) {
        // ---------------- control warp: copies in, results out ----------------
        if (Dec::kTables && lane == 0 && n_local) {
            mbar_expect_tx(&ctl.tab_full, kTableBytes);
            bulk_load(generic(ctl.table), &kIq2StreamTable, kTableBytes, &ctl.tab_full);
        }
        uint32_t issued = 0;
        bool ok = true;
        for (uint32_t j = 0; j < n_local && ok; ++j) {
            while (issued < n_local && issued < j + (uint32_t)D && ok) {
                const uint32_t slot = issued % D;
                if (issued >= (uint32_t)D) ok = mbar_wait_warp(&ctl.empty[slot], ((issued / D) - 1u) & 1u, &ctl.abort);
                if (!ok) break;
                uint32_t m; uint64_t row0; uint32_t nrows;
                task(issued, m, row0, nrows);
                const uint8_t *src = p.enc + (uint64_t)m * p.matrix_stride + row0 * p.row_bytes;
                const uint32_t bytes = (uint32_t)(nrows * p.row_bytes), bulk = bytes & ~15u;
                uint8_t *dst = generic(ctl.stage[slot]);
                if (lane < (int)(bytes - bulk)) dst[bulk + lane] = __ldg(src + bulk + lane);      // the last < 16 bytes of a ragged tile
                __syncwarp();
                if (lane == 0) {
                    mbar_expect_tx(&ctl.full[slot], bulk);
                    if (bulk) bulk_load(dst, src, bulk, &ctl.full[slot]);
                }
                ++issued;
            }
            if (!ok) break;
            const uint32_t buf = j % (uint32_t)(D + 1);
            ok = mbar_wait_warp(&ctl.red_full[buf], (j / (uint32_t)(D + 1)) & 1u, &ctl.abort);
            if (!ok) break;
            uint32_t m; uint64_t row0; uint32_t nrows;
            task(j, m, row0, nrows);
            const float *red = reinterpret_cast<const float *>(generic(ctl.red)) + (size_t)buf * consumers * kTileRows;
            const float scale = ctl.xscale[m & 7u];
            if ((uint32_t)lane < nrows) {
                const int rg = lane / kTileRows, r = lane % kTileRows;
                float sum = 0.0f;
                for (int s = 0; s < p.slices; ++s) sum += red[(rg * p.slices + s) * kTileRows + r];        // fixed order
                sum *= scale;
                const uint64_t at = (uint64_t)m * p.out_stride + row0 + lane;
                if (p.additive) sum += p.additive[at];
                if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                p.out[at] = p.round_bf16 ? bf16_round(sum) : sum;
            }
        }
        if (!ok && lane == 0) {
            // copies still in flight land in this CTA's shared memory: give them a bounded time to finish
            int ignore = 0;
            if (Dec::kTables) mbar_wait(&ctl.tab_full, 0u, &ignore);
            raise(p.status, YVEX_B200_STATUS_TIMEOUT);
        }
        return;
    }
    if (warp > consumers) return;

    // ---------------- consumer warps ----------------
    Lane l;
    l.g = lane >> 2; l.t = lane & 3;
    const int sl = warp % p.slices, rg = warp / p.slices;
    const int unit0 = sl * p.units_per_slice, nunits_total = p.K / Dec::kBlockK;
    const int my_units = min(p.units_per_slice, nunits_total - unit0);
    const bool b_active = (lane & 3) == (lane >> 3);                        // column n = lane >> 2 belongs to group n >> 1
    const uint8_t *planes = generic(ctl.planes), *zeros = generic(ctl.zeros);
    // column 2t' carries the higher plane of a pair, column 2t' + 1 the lower one
    const int col_plane = (lane >> 2) & 1;
    l.b_hi = b_active ? planes + (size_t)(0 + col_plane) * p.K + unit0 * Dec::kBlockK + 32 * (lane >> 3) : zeros;
    l.b_lo = b_active ? planes + (size_t)(2 + col_plane) * p.K + unit0 * Dec::kBlockK + 32 * (lane >> 3) : zeros;
    l.nib_base = (ctl.table & 0xffff0000u) | (uint32_t)(lane * 4);
    l.sgn_base = l.nib_base + 128u;
    const float *sums = reinterpret_cast<const float *>(generic(ctl.sums)) + unit0 * (Dec::kBlockK / 32);
    float *red_all = reinterpret_cast<float *>(generic(ctl.red));
    const int cthreads = consumers * 32;
    if (threadIdx.x < 64 * p.units_per_slice + 4) reinterpret_cast<uint32_t *>(generic(ctl.zeros))[threadIdx.x] = 0u;

    uint32_t cur_m = 0xffffffffu;
    // A warp whose wait ran out keeps walking the task list without touching data, so that it still
    // meets the other consumers at the named barriers of every matrix change and nobody waits for it.
    bool dead = false;
    if (Dec::kTables && n_local) {
        if (!mbar_wait_warp(&ctl.tab_full, 0u, &ctl.abort)) dead = true;
        asm volatile("" : "+r"(l.nib_base), "+r"(l.sgn_base));      // table reads may not move above this point
    }
    for (uint32_t i = 0; i < n_local; ++i) {
        uint32_t m; uint64_t row0; uint32_t nrows;
        task(i, m, row0, nrows);
        if (m != cur_m) {
            // a new matrix: its activation row becomes four planes of signed base-128 digits. Every
            // consumer has finished the previous matrix once it is past this barrier.
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            const float *x = p.x + (uint64_t)m * p.x_stride;
            float mx = 0.0f;
            bool badx = false;
            for (int k = threadIdx.x; k < p.K; k += cthreads) {
                const float v = __ldg(x + k);
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
            if (threadIdx.x == 0) ctl.xscale[m & 7u] = ldexpf(1.0f, e - 27);
            int8_t *pl = reinterpret_cast<int8_t *>(generic(ctl.planes));
            float *sm = reinterpret_cast<float *>(generic(ctl.sums));
            for (int k8 = threadIdx.x; k8 < p.K / 8; k8 += cthreads) {
                uint32_t d[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};
                float s = 0.0f;
#pragma unroll
                for (int i8 = 0; i8 < 8; ++i8) {
                    const float v = __ldg(x + 8 * k8 + i8);
                    int q = isfinite(v) ? __float2int_rn(v * to_q) : 0;
                    s += (float)q;
                    // balanced digits: d0..d2 in [-64, 63], the top digit takes what is left (|d3| <= 64)
                    const int d0 = ((q + 64) & 127) - 64; q = (q - d0) >> 7;
                    const int d1 = ((q + 64) & 127) - 64; q = (q - d1) >> 7;
                    const int d2 = ((q + 64) & 127) - 64; q = (q - d2) >> 7;
                    const int dig[4] = {q, d2, d1, d0};                     // plane 0 is the most significant
#pragma unroll
                    for (int pi = 0; pi < 4; ++pi) d[pi][i8 >> 2] |= (uint32_t)(dig[pi] & 0xff) << (8 * (i8 & 3));
                }
#pragma unroll
                for (int pi = 0; pi < 4; ++pi)
                    *reinterpret_cast<uint2 *>(pl + (size_t)pi * p.K + 8 * k8) = make_uint2(d[pi][0], d[pi][1]);
                if (Dec::kSums) {
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if ((threadIdx.x & 3) == 0) sm[k8 >> 2] = s;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(cthreads) : "memory");
            cur_m = m;
        }
        const uint32_t slot = i % D, buf = i % (uint32_t)(D + 1);
        if (!dead && !mbar_wait_warp(&ctl.full[slot], (i / D) & 1u, &ctl.abort)) dead = true;
        float acc[2] = {0.0f, 0.0f};
        int bad = 0;
        if (!dead && (uint32_t)(kTileRows * rg) < nrows) {
            const uint8_t *stage = generic(ctl.stage[slot]);
            const uint8_t *row0p = stage + (size_t)(kTileRows * rg + l.g) * p.row_bytes + (size_t)unit0 * Dec::kBlockBytes;
            const uint8_t *row1p = row0p + 8 * p.row_bytes;
            for (int u = 0; u < my_units; ++u)
                Dec::unit(row0p + (size_t)u * Dec::kBlockBytes, row1p + (size_t)u * Dec::kBlockBytes, u * Dec::kBlockK, l, sums, acc, bad);
        }
        // this warp is done with the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.empty[slot]);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 1);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 2);
        float *red = red_all + ((size_t)buf * consumers + warp) * kTileRows;
        if (l.t == 0) { red[l.g] = acc[0]; red[l.g + 8] = acc[1]; }
        // a malformed block scale only counts for rows that exist (rows past a ragged tile hold stale bytes)
        const uint32_t r_lo = (uint32_t)(kTileRows * rg + l.g), r_hi = r_lo + 8;
        if (((bad & 1) && r_lo < nrows) || ((bad & 2) && r_hi < nrows)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.red_full[buf]);
    }
}

// ---- host side -----------------------------------------------------------------------------------------------
struct StreamShape { int slices, units_per_slice, row_groups, consumers, depth; uint32_t stage_bytes, smem_bytes; };

// K-slices (consumer warps along K), units per slice, row groups per stage and the deepest ring that fits.
inline bool stream_shape(uint64_t width, uint64_t row_bytes, bool tables, StreamShape &sh) {
    const int units = (int)(width / 256);
    if (!units || width % 256 || width > 8192) return false;
    sh.units_per_slice = (units + kMaxConsumers - 1) / kMaxConsumers;
    sh.slices = (units + sh.units_per_slice - 1) / sh.units_per_slice;
    sh.row_groups = sh.slices <= kMaxConsumers / 2 ? 2 : 1;
    sh.consumers = sh.slices * sh.row_groups;
    sh.stage_bytes = (uint32_t)(kTileRows * sh.row_groups * row_bytes);
    const uint32_t limit = 227u * 1024u - 1024u;
    for (sh.depth = kMaxDepth; sh.depth >= 2; --sh.depth) {
        // every piece is rounded up to 128 bytes; one piece may have to step over the table window
        const uint32_t pieces = (uint32_t)sh.depth * (sh.stage_bytes + 16 + 128) + stream_small_bytes((int)width, sh.consumers, sh.depth, sh.units_per_slice) + 5 * 128;
        sh.smem_bytes = pieces + (tables ? 2 * kTableBytes : 0u);
        // with tables: the window starts at most 64 KiB - 1 into the allocation and whatever lies before it stays
        // usable, so the worst case is one stage of slack, not a second 64 KiB
        if (tables) sh.smem_bytes = pieces + kTableBytes + sh.stage_bytes + 16 + 128;
        if (tables && sh.smem_bytes < 2 * kTableBytes) sh.smem_bytes = 2 * kTableBytes;
        if (sh.smem_bytes <= limit) return true;
    }
    return false;
}

inline bool stream_qtype(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q8_0; }

inline bool stream_eligible(unsigned q, uint64_t rows, uint64_t width, uint64_t row_bytes, const void *enc, uint64_t matrix_stride,
                            uint64_t count) {
    StreamShape sh;
    return stream_qtype(q) && rows && count && count <= 0xffffffffull && (reinterpret_cast<uintptr_t>(enc) & 15u) == 0 &&
           matrix_stride % 16 == 0 && stream_shape(width, row_bytes, q == Q_IQ2_XXS, sh);
}

template <class Dec>
inline int stream_launch_t(StreamParams &p, const StreamShape &sh, cudaStream_t stream) {
    static SmemOptIn opt_in;
    if (opt_in.ensure(gemv_stream_kernel<Dec>, 227 * 1024) != OK) return ERR_BACKEND;
    const uint64_t tile_rows = (uint64_t)kTileRows * sh.row_groups;
    const uint64_t tasks = (uint64_t)p.count * ((p.rows + tile_rows - 1) / tile_rows);
    const unsigned grid = (unsigned)(tasks < (uint64_t)kSmCount ? tasks : (uint64_t)kSmCount);
    gemv_stream_kernel<Dec><<<grid, 32 * (sh.consumers + 1), sh.smem_bytes, stream>>>(p);
    return launch_status(1);
}

inline int stream_launch(unsigned q, const uint8_t *enc, uint64_t matrix_stride, uint64_t count, uint64_t rows, uint64_t width,
                         uint64_t row_bytes, const float *x, uint64_t x_stride, const float *additive, float *out,
                         uint64_t out_stride, int round_bf16, int *status, cudaStream_t stream) {
    StreamShape sh;
    if (!stream_shape(width, row_bytes, q == Q_IQ2_XXS, sh)) return ERR_BOUNDS;
    StreamParams p{};
    p.enc = enc; p.matrix_stride = matrix_stride; p.count = (uint32_t)count; p.rows = rows; p.row_bytes = row_bytes;
    p.K = (int)width; p.slices = sh.slices; p.units_per_slice = sh.units_per_slice; p.row_groups = sh.row_groups; p.depth = sh.depth;
    p.stage_bytes = sh.stage_bytes; p.smem_bytes = sh.smem_bytes;
    p.x = x; p.x_stride = x_stride; p.additive = additive; p.out = out; p.out_stride = out_stride;
    p.round_bf16 = round_bf16; p.status = status;
    switch (q) {
    case Q_IQ2_XXS: return stream_launch_t<StreamIq2>(p, sh, stream);
    case Q_Q4_K: return stream_launch_t<StreamQ4k>(p, sh, stream);
    case Q_Q8_0: return stream_launch_t<StreamQ80>(p, sh, stream);
    default: return ERR_UNSUPPORTED;
    }
}

}  // namespace gs
}  // namespace yb
