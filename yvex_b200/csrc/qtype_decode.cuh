// Qtype geometry, the fail-closed registry, and the per-element reference-exact decoders.
// Layouts: src/gguf/qtype.c:15-104; arithmetic: src/gguf/quant_block.c:715-767, :819-833.
#pragma once
#include "common.cuh"

namespace yb {

struct Geometry { unsigned elems, bytes; };

// Block geometry for every id the reference knows (0..42); {0,0} = removed id.
__host__ __device__ inline Geometry geometry_of(unsigned q) {
    constexpr uint16_t e[43] = {1, 1, 32, 32, 0, 0, 32, 32, 32, 32, 256, 256, 256, 256, 256, 256,
                                256, 256, 256, 256, 32, 256, 256, 256, 1, 1, 1, 1, 1, 256, 1, 0,
                                0, 0, 256, 256, 0, 0, 0, 32, 64, 128, 64};
    constexpr uint16_t b[43] = {4, 2, 18, 20, 0, 0, 22, 24, 34, 36, 84, 110, 144, 176, 210, 292,
                                66, 74, 98, 50, 18, 110, 82, 136, 1, 2, 4, 8, 8, 56, 2, 0,
                                0, 0, 54, 66, 0, 0, 0, 17, 36, 18, 18};
    if (q > 42u) return Geometry{0u, 0u};
    return Geometry{e[q], b[q]};
}

// The only qtypes any kernel here will touch. Everything else is refused before a launch.
__host__ __device__ inline bool qtype_supported(unsigned q) {
    return q == Q_F32 || q == Q_F16 || q == Q_BF16 || q == Q_Q8_0 || q == Q_Q2_K ||
           q == Q_Q4_K || q == Q_IQ2_XXS || q == Q_MXFP4;
}

// Returns 0 when (rows, width, row_bytes) is a consistent canonical layout for q.
inline int check_rows(unsigned q, uint64_t rows, uint64_t width, uint64_t row_bytes) {
    if (!qtype_supported(q)) return ERR_UNSUPPORTED;
    Geometry g = geometry_of(q);
    if (!rows || !width) return ERR_INVALID_ARG;
    if (width % g.elems) return ERR_BOUNDS;
    if (row_bytes != width / g.elems * g.bytes) return ERR_BOUNDS;
    return OK;
}

// IQ2_XXS codebook, one nibble per lane: digit 0/1/2 = magnitude 8/25/43.
__device__ const uint32_t kIq2Nibbles[256] = {
#include "iq2xxs_grid_nibbles.inc"
};

__device__ __forceinline__ uint32_t ld_u32_unaligned2(const uint8_t *p) {  // p is 2-byte aligned
    return static_cast<uint32_t>(ldg_u16(p)) | (static_cast<uint32_t>(ldg_u16(p + 2)) << 16);
}

// 8-bit sign mask of an IQ2_XXS subgroup: 7 stored bits + their parity as bit 7
// (src/gguf/quant_block.c:378-386).
__device__ __forceinline__ uint32_t iq2_signs(uint32_t low7) {
    return low7 | ((__popc(low7) & 1u) << 7);
}

__device__ __forceinline__ float iq2_level(uint32_t digit) {
    return digit == 0u ? 8.0f : digit == 1u ? 25.0f : 43.0f;
}

// One element of one block, with the reference decoder's exact f32 association. `status` gets
// 1 for the scale faults the reference refuses (negative / non-finite block scales).
__device__ inline float decode_element(unsigned q, const uint8_t *blk, unsigned i, int *status) {
    switch (q) {
    case Q_F32: return __uint_as_float(ld_u32_unaligned2(blk));
    case Q_F16: return f16_bits_to_float(ldg_u16(blk));
    case Q_BF16: return __uint_as_float(static_cast<uint32_t>(ldg_u16(blk)) << 16);
    case Q_Q8_0: {
        float d = f16_bits_to_float(ldg_u16(blk));
        if (!isfinite(d) || d < 0.0f) raise(status, YVEX_B200_STATUS_NUMERIC);
        return __fmul_rn(d, static_cast<float>(static_cast<int8_t>(__ldg(blk + 2 + i))));
    }
    case Q_MXFP4: {
        // 17 bytes: an E8M0 scale, then 16 bytes whose low nibbles are elements 0..15 and high nibbles 16..31;
        // value = level(code) * (2^(e - 127) / 2), levels {0,1,2,3,4,6,8,12} with bit 3 as the sign
        // (src/backend/cuda/kernel_primitives.h:100-111; golden block tests/unit/quant_numeric.c:529-540)
        const unsigned e = __ldg(blk);
        if (e == 0xffu) raise(status, YVEX_B200_STATUS_NUMERIC);
        const float scale = __fmul_rn(__uint_as_float(e ? e << 23 : 0x00400000u), 0.5f);
        const unsigned byte = __ldg(blk + 1 + (i & 15u)), code = i < 16u ? byte & 15u : byte >> 4;
        unsigned mag = code & 7u;
        mag += (mag & 3u) * (mag >> 2);
        mag += mag == 10u ? 2u : 0u;
        return __fmul_rn(__uint_as_float(__float_as_uint(static_cast<float>(mag)) | ((code & 8u) << 28)), scale);
    }
    case Q_Q2_K: {
        float d = f16_bits_to_float(ldg_u16(blk + 80)), dmin = f16_bits_to_float(ldg_u16(blk + 82));
        if (!isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f)
            raise(status, YVEX_B200_STATUS_NUMERIC);
        unsigned sub = i >> 4, lane = i & 15u;
        unsigned half = sub >> 3, plane = (sub >> 1) & 3u, pair = sub & 1u;
        unsigned sb = __ldg(blk + sub);
        unsigned code = (__ldg(blk + 16 + 32 * half + 16 * pair + lane) >> (2 * plane)) & 3u;
        float scale = __fmul_rn(d, static_cast<float>(sb & 15u));
        float minimum = __fmul_rn(dmin, static_cast<float>(sb >> 4));
        return __fsub_rn(__fmul_rn(scale, static_cast<float>(code)), minimum);
    }
    case Q_Q4_K: {  // extension: no reference decoder exists for this qtype
        float d = f16_bits_to_float(ldg_u16(blk)), dmin = f16_bits_to_float(ldg_u16(blk + 2));
        if (!isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f)
            raise(status, YVEX_B200_STATUS_NUMERIC);
        unsigned j = i >> 5, lane = i & 31u, sc, m;
        const uint8_t *s = blk + 4;
        if (j < 4) { sc = __ldg(s + j) & 63u; m = __ldg(s + j + 4) & 63u; }
        else {
            sc = (__ldg(s + j + 4) & 15u) | ((__ldg(s + j - 4) >> 6) << 4);
            m = (__ldg(s + j + 4) >> 4) | ((__ldg(s + j) >> 6) << 4);
        }
        unsigned byte = __ldg(blk + 16 + 32 * (j >> 1) + lane);
        unsigned code = (j & 1u) ? byte >> 4 : byte & 15u;
        float scale = __fmul_rn(d, static_cast<float>(sc));
        float minimum = __fmul_rn(dmin, static_cast<float>(m));
        return __fsub_rn(__fmul_rn(scale, static_cast<float>(code)), minimum);
    }
    case Q_IQ2_XXS: {
        float d = f16_bits_to_float(ldg_u16(blk));
        if (!isfinite(d) || d < 0.0f) raise(status, YVEX_B200_STATUS_NUMERIC);
        unsigned g = i >> 5, s = (i >> 3) & 3u, lane = i & 7u;
        uint32_t grids = ld_u32_unaligned2(blk + 2 + 8 * g);
        uint32_t ss = ld_u32_unaligned2(blk + 6 + 8 * g);
        float gs = __fmul_rn(__fmul_rn(d, 0.5f + static_cast<float>(ss >> 28)), 0.25f);
        uint32_t digit = (kIq2Nibbles[(grids >> (8 * s)) & 255u] >> (4 * lane)) & 3u;
        uint32_t signs = iq2_signs((ss >> (7 * s)) & 127u);
        return __fmul_rn(__fmul_rn(gs, iq2_level(digit)), (signs >> lane) & 1u ? -1.0f : 1.0f);
    }
    default:
        raise(status, YVEX_B200_STATUS_ARGUMENT);
        return 0.0f;
    }
}

}  // namespace yb
