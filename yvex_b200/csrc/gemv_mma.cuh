// Streaming dequant-fused matvec engine for 256-element superblock qtypes.
//
// Why tensor cores for a matvec: at 0.26 bytes per IQ2_XXS weight the HBM stream delivers ~80
// weights per SM per clock, and a scalar multiply-add per weight alone would fill most of the
// FP32 pipe. Here a warp owns 8 matrix rows x a 512-weight K-slice; every thread decodes eight
// weights at a time into four packed-fp16 registers holding EXACT small integers (code x integer
// sub-scale, sign included) and feeds them to mma.sync.m16n8k16 as the A fragment. The 16 MMA
// rows are 8 matrix rows x 2 halves of those eight weights; the B fragment carries the
// activation in columns 0-2 for the first halves and 4-6 for the second halves - either an f32
// row split into three fp16 pieces (x = hi + mid*2^-11 + lo*2^-22, ~33 bits) or, when the caller
// knows the row is bf16-exact (MoE ingress rows and SwiGLU intermediates are, by contract), its
// single fp16 image. Products are therefore exact and only the f32 accumulation rounds. The
// per-superblock f16 scale multiplies the drained accumulator once per 256 weights; affine
// qtypes (Q4_K, Q2_K) subtract dmin * sum(m_sub * sum_x(sub)) with precomputed per-sub-block
// activation sums. Because a dot product does not care about the order of k, a decoder may hand
// any 8 weights of its block to any MMA slot as long as the B fragment uses the same
// permutation (Decoder::k_of); that is what keeps the per-weight instruction count low.
//
// Data movement: every warp owns a private ring of staging slots in shared memory. A unit is 8
// rows x up to 4 superblocks; the warp copies it with 16-byte cp.async chunks (lanes 4 wide along
// a row, 8 rows per instruction), keeps two units in flight while it decodes a third, and needs
// only __syncwarp between copy and use. Chunks that would cross the ends of the tensor are copied
// with guarded 2-byte loads, so no byte outside [encoded, encoded + rows*row_bytes) is ever read.
// The activation (B operand) lives in shared memory once per CTA - the fp16 image of a bf16-exact
// row, or the three fp16 pieces of an f32 row - and each MMA fetches its fragment from there.
// K is split over the warps of a CTA when a matrix has too few rows to occupy the device
// otherwise; the partial dots meet in shared memory once per 8*RG rows.
#pragma once
#include "qtype_decode.cuh"

namespace yb {

constexpr int kChunkBlocks = 4;                    // superblocks per staged unit (1024 weights x 8 rows)
constexpr int kRingDepth = 2;                      // staged units per warp: one in use, one in flight (many warps per SM)
constexpr int kMaxK = 8192;                        // widest row on this path

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The activation fragment source of one lane: `p` points at this lane's fp16 piece array at the
// first k of the current superblock and moves on by `stride` halves per superblock; lanes that
// own a zero column of B point at a block of zeros and stand still (stride 0), so the fetch needs
// no branch. `hi` selects the second half of each 8-weight group.
struct BLane {
    const __half *p;
    int stride, t, hi;
    template <class Dec> __device__ __forceinline__ uint2 get(int half, int j) const {
        return *reinterpret_cast<const uint2 *>(p + Dec::k_of(half, t, j, hi));
    }
};
constexpr int kZeroHalves = 256;                   // zeros every k_of() offset of one superblock can index

// Lookup tables every decoder shares, resident in shared memory for the life of the CTA.
struct MmaTables {
    uint32_t nib[256];    // IQ2_XXS codebook, one nibble per lane
    uint32_t sign[128];   // 7 stored sign bits -> 8 sign bits (parity) spread to bit 2 of each nibble
    uint2 scale[64];      // integer scale s -> {half2(s,s), half2(-bias*s)}; bias depends on qtype
};

__device__ __forceinline__ void load_tables(MmaTables *t, float bias) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) t->nib[i] = kIq2Nibbles[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) {
        uint32_t s = iq2_signs(i), spread = 0;
        for (int l = 0; l < 8; ++l) spread |= ((s >> l) & 1u) << (4 * l + 2);
        t->sign[i] = spread;
    }
    for (int i = threadIdx.x; i < 64; i += blockDim.x) {
        __half2 s = __float2half2_rn(static_cast<float>(i));
        __half2 nb = __float2half2_rn(-bias * static_cast<float>(i));
        t->scale[i] = make_uint2(*reinterpret_cast<uint32_t *>(&s), *reinterpret_cast<uint32_t *>(&nb));
    }
}

// Four code bytes -> two half2 registers holding code*scale exactly: fp16(0x6400 | b) = 1024 + b,
// then one fused multiply-add removes the bias (single rounding of an exactly representable value).
__device__ __forceinline__ void bytes_to_scaled_half2(uint32_t bytes, __half2 sc2, __half2 nb2, uint32_t &h01,
                                                      uint32_t &h23) {
    uint32_t a = __byte_perm(bytes, 0x64646464u, 0x4140), b = __byte_perm(bytes, 0x64646464u, 0x4342);
    __half2 va = __hfma2(*reinterpret_cast<__half2 *>(&a), sc2, nb2);
    __half2 vb = __hfma2(*reinterpret_cast<__half2 *>(&b), sc2, nb2);
    h01 = *reinterpret_cast<uint32_t *>(&va);
    h23 = *reinterpret_cast<uint32_t *>(&vb);
}

// ---- IQ2_XXS ---------------------------------------------------------------------------------------
// 66 bytes: f16 d, then eight 8-byte groups {4 codebook indices, 4x7 sign bits + 4-bit sub-scale}.
// value = d/8 * (2*sub+1) * (+-{8,25,43})  ==  the reference's d*(0.5+sub)*0.25*level*sign, every
// factor but d being a small integer (src/gguf/quant_block.c:745-767). Quad thread t decodes
// group 4*half+t; MMA j takes its subgroup j.
struct Iq2Decoder {
    static constexpr unsigned kQtype = Q_IQ2_XXS;
    static constexpr int kBlockBytes = 66, kSumGroup = 0, kAlign = 2;
    // when the next kernel on the stream may move in (programmatic dependent launch): at the start of this
    // one, or when its rows are done. Measured on 4096 x 4096: the early trigger gives Q4_K +18 % and
    // costs the instruction-bound IQ2_XXS decode 15 %.
    static constexpr bool kEarlyDependents = false;
    static constexpr float kBias = 1152.0f;        // fp16(0x6400 | (b + 128)) = 1152 + b

    __device__ static int k_of(int half, int t, int j, int hi) { return 128 * half + 32 * t + 8 * j + 4 * hi; }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const BLane &b, float (&d)[4], float &, const float *) {
        const uint8_t *p = blk + 2 + 8 * (4 * half + t);
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        const uint32_t sh = (a & 2u) * 8u;
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
        const uint32_t grids = __funnelshift_r(w0, w1, sh), ss = __funnelshift_r(w1, w2, sh);
        const uint2 sc = tab->scale[2u * (ss >> 28) + 1u];
        const __half2 sc2 = *reinterpret_cast<const __half2 *>(&sc.x);
        const __half2 nb2 = *reinterpret_cast<const __half2 *>(&sc.y);
        constexpr uint32_t kLo = (8u + 128u) | ((25u + 128u) << 8) | ((43u + 128u) << 16);
        constexpr uint32_t kHi = (128u - 8u) | ((128u - 25u) << 8) | ((128u - 43u) << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t sel = tab->nib[(grids >> (8 * j)) & 255u] | tab->sign[(ss >> (7 * j)) & 127u];
            const uint32_t u_lo = __byte_perm(kLo, kHi, sel), u_hi = __byte_perm(kLo, kHi, sel >> 16);
            uint32_t afrag[4];
            bytes_to_scaled_half2(u_lo, sc2, nb2, afrag[0], afrag[2]);
            bytes_to_scaled_half2(u_hi, sc2, nb2, afrag[1], afrag[3]);
            const uint2 bf = b.get<Iq2Decoder>(half, j);
            mma_f16(d, afrag, bf.x, bf.y);
        }
    }

    __device__ static float finish(const uint8_t *blk, float val, float, bool &bad) {
        float d = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk));
        bad = !isfinite(d) || d < 0.0f;
        return d * 0.125f * val;
    }
};

// ---- Q4_K (extension; no reference decoder) ---------------------------------------------------------
// 144 bytes: f16 d, f16 dmin, 12 bytes of 6-bit (scale, min) pairs for eight 32-element sub-blocks,
// 128 bytes of 4-bit codes; chunk c (32 bytes) holds sub-block 2c in the low and 2c+1 in the high
// nibbles. value = d*sc*code - dmin*m. Quad thread t of half h reads the 16 code bytes
// 16*(t&1).. of chunk c = 2h + (t>>1); MMA j takes word j: low nibbles = first half, high = second.
struct Q4kDecoder {
    static constexpr unsigned kQtype = Q_Q4_K;
    static constexpr int kBlockBytes = 144, kSumGroup = 32, kAlign = 16;
    static constexpr bool kEarlyDependents = true;
    static constexpr float kBias = 1024.0f;

    __device__ static int k_of(int half, int t, int j, int hi) {
        return 64 * (2 * half + (t >> 1)) + 32 * hi + 16 * (t & 1) + 4 * j;
    }

    __device__ static void scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &m) {
        if (j < 4) { sc = s[j] & 63u; m = s[j + 4] & 63u; }
        else { sc = (s[j + 4] & 15u) | ((s[j - 4] >> 6) << 4); m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
    }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const BLane &b, float (&d)[4], float &minacc, const float *sums) {
        const int c = 2 * half + (t >> 1);
        uint32_t sc0, m0, sc1, m1;
        scale_min(blk + 4, 2 * c, sc0, m0);
        scale_min(blk + 4, 2 * c + 1, sc1, m1);
        const uint2 s0 = tab->scale[sc0], s1 = tab->scale[sc1];
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c + 16 * (t & 1));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t afrag[4];
            bytes_to_scaled_half2(w[j] & 0x0f0f0f0fu, *reinterpret_cast<const __half2 *>(&s0.x),
                                  *reinterpret_cast<const __half2 *>(&s0.y), afrag[0], afrag[2]);
            bytes_to_scaled_half2((w[j] >> 4) & 0x0f0f0f0fu, *reinterpret_cast<const __half2 *>(&s1.x),
                                  *reinterpret_cast<const __half2 *>(&s1.y), afrag[1], afrag[3]);
            const uint2 bf = b.get<Q4kDecoder>(half, j);
            mma_f16(d, afrag, bf.x, bf.y);
        }
        // one quad thread per sub-block carries its min term: even t -> 2c, odd t -> 2c+1
        minacc = fmaf(static_cast<float>((t & 1) ? m1 : m0), sums[2 * c + (t & 1)], minacc);
    }

    __device__ static float finish(const uint8_t *blk, float val, float minacc, bool &bad) {
        float d = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk));
        float dmin = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 2));
        bad = !isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f;
        return fmaf(d, val, -dmin * minacc);
    }
};

// ---- Q2_K --------------------------------------------------------------------------------------------
// 84 bytes: 16 bytes of (4-bit scale | 4-bit min << 4) for sixteen 16-element sub-blocks, 64 bytes of
// 2-bit codes, f16 d, f16 dmin (src/gguf/quant_block.c:715-743). Byte l of half hf carries planes
// 0..3 = elements 128*hf + 32*plane + l. Quad thread t of half hf reads bytes 8t..8t+7; MMA j takes
// word j>>1 and plane pair j&1: plane 2*(j&1) = first half, plane 2*(j&1)+1 = second half.
struct Q2kDecoder {
    static constexpr unsigned kQtype = Q_Q2_K;
    static constexpr int kBlockBytes = 84, kSumGroup = 16, kAlign = 4;
    static constexpr bool kEarlyDependents = true;
    static constexpr float kBias = 1024.0f;

    __device__ static int k_of(int half, int t, int j, int hi) {
        return 128 * half + 32 * (2 * (j & 1) + hi) + 8 * t + 4 * (j >> 1);
    }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const BLane &b, float (&d)[4], float &minacc, const float *sums) {
        const uint32_t *q = reinterpret_cast<const uint32_t *>(blk + 16 + 32 * half + 8 * t);   // 4-byte aligned
        const uint32_t w[2] = {q[0], q[1]};
        uint32_t sb[4];                     // scale bytes of planes 0..3: sub-block 8*half + 2*plane + (t>>1)
#pragma unroll
        for (int pl = 0; pl < 4; ++pl) sb[pl] = blk[8 * half + 2 * pl + (t >> 1)];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p0 = 2 * (j & 1);
            const uint2 s0 = tab->scale[sb[p0] & 15u], s1 = tab->scale[sb[p0 + 1] & 15u];
            const uint32_t word = w[j >> 1];
            uint32_t afrag[4];
            bytes_to_scaled_half2((word >> (2 * p0)) & 0x03030303u, *reinterpret_cast<const __half2 *>(&s0.x),
                                  *reinterpret_cast<const __half2 *>(&s0.y), afrag[0], afrag[2]);
            bytes_to_scaled_half2((word >> (2 * p0 + 2)) & 0x03030303u, *reinterpret_cast<const __half2 *>(&s1.x),
                                  *reinterpret_cast<const __half2 *>(&s1.y), afrag[1], afrag[3]);
            const uint2 bf = b.get<Q2kDecoder>(half, j);
            mma_f16(d, afrag, bf.x, bf.y);
        }
        // min terms: even t carries planes 0,1, odd t planes 2,3 of sub-block column (t>>1)
        const int pb = 2 * (t & 1);
        minacc = fmaf(static_cast<float>(sb[pb] >> 4), sums[8 * half + 2 * pb + (t >> 1)], minacc);
        minacc = fmaf(static_cast<float>(sb[pb + 1] >> 4), sums[8 * half + 2 * (pb + 1) + (t >> 1)], minacc);
    }

    __device__ static float finish(const uint8_t *blk, float val, float minacc, bool &bad) {
        float d = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 80));
        float dmin = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 82));
        bad = !isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f;
        return fmaf(d, val, -dmin * minacc);
    }
};

// ---- activation vectors in shared memory ---------------------------------------------------------------
// Both helpers give each thread 16 consecutive elements per pass, issue all of its global loads
// before touching the data, and also produce the per-sub-block sums the affine qtypes need
// (G = 16 or 32 elements per sum, 0 = none). All threads of the CTA take part, every lane runs
// the same number of passes, the caller synchronises.

// f32 row -> three fp16 piece arrays pieces[0..3K): x = hi + mid*2^-11 + lo*2^-22 (~33 bits).
template <int G>
__device__ __forceinline__ void prepare_row_f32(__half *pieces, float *sums, const float *x, int K, int *status) {
    const int per_pass = 16 * blockDim.x;
    bool bad = false;
    for (int base = 0; base < K; base += per_pass) {
        const int k0 = base + 16 * threadIdx.x;
        const bool active = k0 < K;
        float4 v4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            v4[i] = active ? __ldg(reinterpret_cast<const float4 *>(x + k0) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float *v = reinterpret_cast<const float *>(v4);
        __align__(16) __half h[3][16];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __half hi = __float2half_rn(v[i]);
            bad |= !isfinite(v[i]) || __hisinf(hi);
            const float r1 = (v[i] - __half2float(hi)) * 2048.0f;
            const __half mid = __float2half_rn(r1);
            const float r2 = (r1 - __half2float(mid)) * 2048.0f;
            h[0][i] = hi; h[1][i] = mid; h[2][i] = __float2half_rn(r2);
            s += v[i];
        }
        if (active) {
#pragma unroll
            for (int pc = 0; pc < 3; ++pc) {
                *reinterpret_cast<uint4 *>(pieces + pc * K + k0) = *reinterpret_cast<const uint4 *>(&h[pc][0]);
                *reinterpret_cast<uint4 *>(pieces + pc * K + k0 + 8) = *reinterpret_cast<const uint4 *>(&h[pc][8]);
            }
        }
        if (G == 16 && active) sums[k0 / 16] = s;
        if (G == 32) {
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if (active && !(threadIdx.x & 1)) sums[k0 / 32] = s;
        }
    }
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
}

// fp16 rows (16-byte aligned, `halves` a multiple of 16, bf16-exact values) -> shared memory.
template <int G>
__device__ __forceinline__ void prepare_row_half(__half *dst, float *sums, const __half *src, int halves) {
    const int per_pass = 16 * blockDim.x;
    for (int base = 0; base < halves; base += per_pass) {
        const int k0 = base + 16 * threadIdx.x;
        const bool active = k0 < halves;
        uint4 raw[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
            raw[i] = active ? __ldg(reinterpret_cast<const uint4 *>(src + k0) + i) : make_uint4(0u, 0u, 0u, 0u);
        if (active) {
            *reinterpret_cast<uint4 *>(dst + k0) = raw[0];
            *reinterpret_cast<uint4 *>(dst + k0 + 8) = raw[1];
        }
        if (G != 0) {
            const __half2 *h2 = reinterpret_cast<const __half2 *>(raw);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = __half22float2(h2[i]);
                s += f.x + f.y;
            }
            if (G == 16 && active) sums[k0 / 16] = s;
            if (G == 32) {
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                if (active && !(threadIdx.x & 1)) sums[k0 / 32] = s;
            }
        }
    }
}

// This lane's B source. f32 rows: columns 0-2 / 4-6 carry the three pieces, 3 and 7 are zero.
// bf16-exact rows: only columns 0 and 4 are non-zero. `zeros`: kZeroHalves zero halves.
template <bool kHalfB> __device__ __forceinline__ BLane lane_b(const __half *vec, const __half *zeros, int K, int g, int t) {
    BLane b;
    b.t = t;
    b.hi = g >> 2;
    const bool active = kHalfB ? (g & 3) == 0 : (g & 3) != 3;
    b.p = !active ? zeros : kHalfB ? vec : vec + (g & 3) * K;
    b.stride = active ? 256 : 0;
    return b;
}

// This thread's share of its matrix row's block dot product, from the drained accumulator.
template <bool kHalfB> __device__ __forceinline__ float drain(const float (&d)[4], int t) {
    if (kHalfB) return t == 0 ? d[0] : t == 2 ? d[2] : 0.0f;
    constexpr float k11 = 1.0f / 2048.0f, k22 = 1.0f / 4194304.0f;
    return t == 0 ? d[0] + d[1] * k11 : t == 1 ? d[0] * k22 : t == 2 ? d[2] + d[3] * k11 : d[2] * k22;
}

// ---- per-warp staging ring ---------------------------------------------------------------------------
template <class Dec> struct UnitGeom {
    static constexpr int kSlot = (15 + kChunkBlocks * Dec::kBlockBytes + 15) & ~15;   // one row: misalignment + 4 blocks
    static constexpr int kUnitBytes = 8 * kSlot;
    static constexpr int kRingBytes = kRingDepth * kUnitBytes;
    static constexpr int kSumsPerBlock = Dec::kSumGroup ? 256 / Dec::kSumGroup : 0;
};

// One unit of work of a warp: rows src, src + row_bytes, ... (nrows <= 8 of them are real),
// nblocks <= kChunkBlocks superblocks each; [lo, hi) bounds the tensor the rows belong to.
struct Unit {
    const uint8_t *src, *lo, *hi;
    uint64_t row_bytes;
    int nrows, nblocks;
};

// Copies the unit into `slot`; the byte at address a of row r lands at slot + r*kSlot + (a - a16)
// where a16 is the row start rounded down to 16. The caller commits the cp.async group.
template <class Dec>
__device__ __forceinline__ void stage_unit(uint8_t *slot, const Unit &u, int lane) {
    const int r = lane >> 2;
    if (r < u.nrows) {
        const uint8_t *s = u.src + (uint64_t)r * u.row_bytes;
        const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(s) & 15u);
        const uint8_t *first = s - mis;
        const int chunks = (int)((mis + (uint32_t)u.nblocks * Dec::kBlockBytes + 15u) >> 4);
        uint8_t *d = slot + r * UnitGeom<Dec>::kSlot;
        for (int c = lane & 3; c < chunks; c += 4) {
            const uint8_t *gp = first + 16 * c;
            if (gp >= u.lo && gp + 16 <= u.hi) {
                cp_async16(d + 16 * c, gp);
            } else {
#pragma unroll
                for (int b = 0; b < 16; b += 2)
                    if (gp + b >= u.lo && gp + b + 2 <= u.hi)
                        *reinterpret_cast<uint16_t *>(d + 16 * c + b) = ldg_u16(gp + b);
            }
        }
    }
}

// Partial dot products of the unit's 8 rows with the activation: the return value is this
// thread's share of row g (sum the four threads of a quad). `b` and `sums` point at the unit's
// first superblock.
template <class Dec, bool kHalfB>
__device__ __forceinline__ float unit_dot(const uint8_t *slot, const Unit &u, const MmaTables *tab, BLane b,
                                          const float *sums, int g, int t, int *status) {
    const uint8_t *row = slot + g * UnitGeom<Dec>::kSlot +
                         (reinterpret_cast<uintptr_t>(u.src + (uint64_t)g * u.row_bytes) & 15u);
    float acc = 0.0f;
#pragma unroll
    for (int bl = 0; bl < kChunkBlocks; ++bl) {
        if (bl < u.nblocks) {
            const uint8_t *blk = row + bl * Dec::kBlockBytes;
            float d[4] = {0.f, 0.f, 0.f, 0.f}, minacc = 0.0f;
            Dec::half_block(blk, 0, t, tab, b, d, minacc, sums);
            Dec::half_block(blk, 1, t, tab, b, d, minacc, sums);
            bool bad;
            acc += Dec::finish(blk, drain<kHalfB>(d, t), minacc, bad);
            if (bad && g < u.nrows) raise(status, YVEX_B200_STATUS_NUMERIC);
            b.p += b.stride;
            sums += UnitGeom<Dec>::kSumsPerBlock;
        }
    }
    return acc;
}

// The ring itself: issue() stages the next unit (or nothing) and commits one group; front() waits
// until the oldest staged unit has landed; pop() lets its slot be reused.
template <class Dec> struct WarpRing {
    uint8_t *base;
    int head, tail, lane;
    __device__ __forceinline__ void init(uint8_t *b, int l) { base = b; head = tail = 0; lane = l; }
    __device__ __forceinline__ void issue(const Unit *u) {
        if (u) stage_unit<Dec>(base + head * UnitGeom<Dec>::kUnitBytes, *u, lane);
        cp_async_commit();
        head = head + 1 == kRingDepth ? 0 : head + 1;
    }
    __device__ __forceinline__ const uint8_t *front() {
        cp_async_wait<kRingDepth - 1>();
        __syncwarp();
        return base + tail * UnitGeom<Dec>::kUnitBytes;
    }
    __device__ __forceinline__ void pop() {
        __syncwarp();
        tail = tail + 1 == kRingDepth ? 0 : tail + 1;
    }
};

// ---- plain matvec ------------------------------------------------------------------------------------
struct GemvMmaParams {
    const uint8_t *enc;
    uint64_t rows, row_bytes;
    int K, slices, slice_blocks, row_groups;
    const float *x, *additive;          // blockIdx.y selects the input row: x + y*K, additive/out + y*rows
    float *out;
    int round_bf16;
    int *status;
};

// Shared memory: tables | zeros | activation pieces [3][K] fp16 | sums [K/16] f32 | red [2][warps*8] f32 | rings
__host__ __device__ inline size_t gemv_smem_fixed(int K, int warps) {
    return sizeof(MmaTables) + kZeroHalves * 2 + (size_t)3 * K * 2 + (size_t)(K / 16) * 4 + (size_t)2 * warps * 8 * 4;
}

template <class Dec>
__global__ void __launch_bounds__(512, 2) gemv_mma_kernel(GemvMmaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    MmaTables *tab = reinterpret_cast<MmaTables *>(smem);
    __half *zeros = reinterpret_cast<__half *>(smem + sizeof(MmaTables));
    __half *pieces = zeros + kZeroHalves;
    float *sums = reinterpret_cast<float *>(pieces + 3 * p.K);
    const int warps = blockDim.x >> 5;
    float *red = sums + p.K / 16;
    uint8_t *rings = reinterpret_cast<uint8_t *>(red + 2 * warps * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int sl = warp % p.slices, rg = warp / p.slices;
    const int nblk = p.K / 256;
    const int my_first = sl * p.slice_blocks;
    const int my_blocks = min(p.slice_blocks, nblk - my_first);
    const int nu = (my_blocks + kChunkBlocks - 1) / kChunkBlocks;             // units per task for this warp
    const uint64_t octets = (p.rows + 7) / 8, ctasks = (octets + p.row_groups - 1) / p.row_groups;
    const float *x = p.x + (uint64_t)blockIdx.y * p.K;
    const float *additive = p.additive ? p.additive + (uint64_t)blockIdx.y * p.rows : nullptr;
    float *out = p.out + (uint64_t)blockIdx.y * p.rows;
    const uint8_t *lo = p.enc, *hi = p.enc + p.rows * p.row_bytes;

    auto unit_at = [&](uint64_t ct, int ui, Unit &u) {
        const uint64_t r0 = (ct * p.row_groups + rg) * 8;
        if (ct >= ctasks || r0 >= p.rows) return false;
        u.nrows = (int)(p.rows - r0 < 8 ? p.rows - r0 : 8);
        u.nblocks = min(kChunkBlocks, my_blocks - ui * kChunkBlocks);
        u.row_bytes = p.row_bytes;
        u.src = p.enc + r0 * p.row_bytes + (uint64_t)(my_first + ui * kChunkBlocks) * Dec::kBlockBytes;
        u.lo = lo; u.hi = hi;
        return true;
    };
    // Programmatic dependent launch: this kernel reads its activation and writes its results only after
    // griddepcontrol.wait, i.e. after the kernel before it on the stream has completed, and lets the
    // kernel after it start once its own rows are done (below), so that launch latency and the next
    // kernel's weight prefetch overlap this kernel's tail. What is read before the wait - the encoded
    // weights - must not be produced by the kernel before.
    if (Dec::kEarlyDependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // weight bytes first: the staging ring fills while the tables and the activation are prepared
    WarpRing<Dec> ring;
    ring.init(rings + (size_t)warp * UnitGeom<Dec>::kRingBytes, lane);
    uint64_t ict = blockIdx.x;
    int iui = 0;
    auto issue_next = [&]() {
        Unit u;
        const bool any = nu > 0 && unit_at(ict, iui, u);
        ring.issue(any ? &u : nullptr);
        if (++iui >= nu) { iui = 0; ict += gridDim.x; }
    };
#pragma unroll
    for (int d = 0; d < kRingDepth - 1; ++d) issue_next();
    load_tables(tab, Dec::kBias);
    for (int i = threadIdx.x; i < kZeroHalves / 2; i += blockDim.x) reinterpret_cast<uint32_t *>(zeros)[i] = 0u;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    prepare_row_f32<Dec::kSumGroup>(pieces, sums, x, p.K, p.status);
    __syncthreads();
    const BLane b0 = lane_b<false>(pieces, zeros, p.K, g, t);

    int par = 0;
    for (uint64_t ct = blockIdx.x; ct < ctasks; ct += gridDim.x, par ^= 1) {
        float acc = 0.0f;
        for (int ui = 0; ui < nu; ++ui) {
            issue_next();
            const uint8_t *slot = ring.front();
            Unit u;
            if (unit_at(ct, ui, u)) {
                BLane b = b0;
                const int kb = my_first + ui * kChunkBlocks;
                b.p += b.stride * kb;
                acc += unit_dot<Dec, false>(slot, u, tab, b, sums + kb * UnitGeom<Dec>::kSumsPerBlock, g, t, p.status);
            }
            ring.pop();
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (t == 0) red[(par * warps + warp) * 8 + g] = acc;
        __syncthreads();
        if (threadIdx.x < 8 * p.row_groups) {
            const int rrg = threadIdx.x >> 3, rgi = threadIdx.x & 7;
            const uint64_t orow = (ct * p.row_groups + rrg) * 8 + rgi;
            if (orow < p.rows) {
                float sum = 0.0f;
                for (int s = 0; s < p.slices; ++s) sum += red[(par * warps + rrg * p.slices + s) * 8 + rgi];
                if (additive) sum += additive[orow];
                if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                out[orow] = p.round_bf16 ? bf16_round(sum) : sum;
            }
        }
    }
    if (!Dec::kEarlyDependents) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cp_async_wait<0>();
}

// K-slices (warps along K), superblocks per slice and row groups (8-row sets per CTA task).
inline void mma_shape(uint64_t width, int &slices, int &slice_blocks, int &row_groups) {
    const int nblk = (int)(width / 256);
    slice_blocks = kChunkBlocks;
    slices = (nblk + slice_blocks - 1) / slice_blocks;
    slice_blocks = (nblk + slices - 1) / slices;            // even the slices out (6 blocks -> 3 + 3)
    row_groups = slices >= 8 ? 1 : slices >= 4 ? 2 : slices >= 2 ? 4 : 8;
}

inline bool mma_decoder_for(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q2_K; }

inline bool gemv_mma_eligible(unsigned q, uint64_t rows, uint64_t width, const uint8_t *enc) {
    (void)rows;
    const uintptr_t align = q == Q_Q4_K ? 15u : q == Q_Q2_K ? 3u : 1u;
    return mma_decoder_for(q) && width % 256 == 0 && width <= (uint64_t)kMaxK &&
           (reinterpret_cast<uintptr_t>(enc) & align) == 0;
}

// Resident CTAs per SM the launch should count on: shared memory and the 64-registers-per-thread
// budget of these kernels (65536 / (64 * threads)) bound it.
inline int ctas_per_sm(size_t smem, int threads) {
    int by_smem = (int)((size_t)(227 * 1024) / (smem + 1024));
    int by_regs = 65536 / (64 * threads);
    int n = by_smem < by_regs ? by_smem : by_regs;
    return n < 1 ? 1 : n > 4 ? 4 : n;
}


template <class Dec>
inline int gemv_mma_launch_t(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes,
                             const float *x, uint64_t input_rows, const float *additive, float *out, int round_bf16,
                             int *status, cudaStream_t stream) {
    GemvMmaParams p{};
    p.enc = enc; p.rows = rows; p.row_bytes = row_bytes; p.K = (int)width;
    mma_shape(width, p.slices, p.slice_blocks, p.row_groups);
    p.x = x; p.additive = additive; p.out = out; p.round_bf16 = round_bf16; p.status = status;
    const int warps = p.slices * p.row_groups;
    const size_t smem = ((gemv_smem_fixed(p.K, warps) + 15) & ~(size_t)15) + (size_t)warps * UnitGeom<Dec>::kRingBytes;
    static SmemOptIn opt_in;
    if (opt_in.ensure(gemv_mma_kernel<Dec>, 200 * 1024) != OK) return ERR_BACKEND;
    if (smem > 200 * 1024 || warps > 16 || input_rows > 65535) return ERR_BOUNDS;
    const uint64_t ctasks = ((rows + 7) / 8 + p.row_groups - 1) / p.row_groups;
    const uint64_t cap = (uint64_t)kSmCount * ctas_per_sm(smem, 32 * warps);
    dim3 grid((unsigned)(ctasks < cap ? ctasks : cap), (unsigned)input_rows);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(32 * warps); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemv_mma_kernel<Dec>, p) != cudaSuccess) return ERR_BACKEND;
    return launch_status();
}

inline int gemv_mma_launch(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width,
                           uint64_t row_bytes, const float *x, uint64_t input_rows, const float *additive, float *out,
                           int round_bf16, int *status, cudaStream_t stream) {
    switch (q) {
    case Q_IQ2_XXS:
        return gemv_mma_launch_t<Iq2Decoder>(enc, rows, width, row_bytes, x, input_rows, additive, out, round_bf16, status, stream);
    case Q_Q4_K:
        return gemv_mma_launch_t<Q4kDecoder>(enc, rows, width, row_bytes, x, input_rows, additive, out, round_bf16, status, stream);
    case Q_Q2_K:
        return gemv_mma_launch_t<Q2kDecoder>(enc, rows, width, row_bytes, x, input_rows, additive, out, round_bf16, status, stream);
    default:
        return ERR_UNSUPPORTED;
    }
}

}  // namespace yb
