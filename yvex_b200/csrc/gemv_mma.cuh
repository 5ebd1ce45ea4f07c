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
// Data movement: a CTA walks tiles of 8*RG contiguous rows, copies each tile into shared memory
// with 16-byte cp.async chunks through a ring of stages and decodes from there; chunks that
// would cross the ends of the tensor are copied with guarded 2-byte loads, so no byte outside
// [encoded, encoded + rows*row_bytes) is ever read.
#pragma once
#include "qtype_decode.cuh"

namespace yb {

constexpr int kGemvStages = 4;
constexpr int kSliceBlocks = 2;                    // 512 weights per warp K-slice
constexpr int kMaxSlices = 16;                     // K <= 8192 on this path
constexpr int kMaxSums = 8192 / 16;

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

// Copies global bytes [src, src+bytes) so that byte `src` lands at dst + (src & 15); only bytes
// inside [lo, hi) are dereferenced. All threads of the CTA take part; the caller commits.
__device__ __forceinline__ void stage_span(uint8_t *dst, const uint8_t *src, uint64_t bytes,
                                           const uint8_t *lo, const uint8_t *hi) {
    const uint8_t *first = src - (reinterpret_cast<uintptr_t>(src) & 15u);
    const uint64_t chunks = (static_cast<uint64_t>(src - first) + bytes + 15u) >> 4;
    for (uint64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
        const uint8_t *g = first + (c << 4);
        uint8_t *s = dst + (c << 4);
        if (g >= lo && g + 16 <= hi) {
            cp_async16(s, g);
        } else {
#pragma unroll
            for (int b = 0; b < 16; b += 2)
                if (g + b >= lo && g + b + 2 <= hi)
                    *reinterpret_cast<uint16_t *>(s + b) = ldg_u16(g + b);
        }
    }
}

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
    static constexpr float kBias = 1152.0f;        // fp16(0x6400 | (b + 128)) = 1152 + b

    __device__ static int k_of(int half, int t, int j, int hi) { return 128 * half + 32 * t + 8 * j + 4 * hi; }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const uint32_t (*bfrag)[2], float (&d)[4], float &, const float *) {
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
            mma_f16(d, afrag, bfrag[4 * half + j][0], bfrag[4 * half + j][1]);
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
    static constexpr float kBias = 1024.0f;

    __device__ static int k_of(int half, int t, int j, int hi) {
        return 64 * (2 * half + (t >> 1)) + 32 * hi + 16 * (t & 1) + 4 * j;
    }

    __device__ static void scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &m) {
        if (j < 4) { sc = s[j] & 63u; m = s[j + 4] & 63u; }
        else { sc = (s[j + 4] & 15u) | ((s[j - 4] >> 6) << 4); m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
    }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const uint32_t (*bfrag)[2], float (&d)[4], float &minacc, const float *sums) {
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
            mma_f16(d, afrag, bfrag[4 * half + j][0], bfrag[4 * half + j][1]);
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
    static constexpr float kBias = 1024.0f;

    __device__ static int k_of(int half, int t, int j, int hi) {
        return 128 * half + 32 * (2 * (j & 1) + hi) + 8 * t + 4 * (j >> 1);
    }

    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const uint32_t (*bfrag)[2], float (&d)[4], float &minacc, const float *sums) {
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
            mma_f16(d, afrag, bfrag[4 * half + j][0], bfrag[4 * half + j][1]);
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

// ---- B fragments -----------------------------------------------------------------------------------
// kHalfB = false: x is an f32 row, each thread builds the fp16 piece of its column (3-way split).
// kHalfB = true : xh is the fp16 image of a bf16-exact row; only columns 0 and 4 are non-zero.
template <class Dec, bool kHalfB>
__device__ __forceinline__ void build_bfrag(uint32_t (&bfrag)[8 * kSliceBlocks][2], const float *x, const __half *xh,
                                            int kbase, int K, int g, int t, int *status) {
#pragma unroll
    for (int bl = 0; bl < kSliceBlocks; ++bl)
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = kbase + 256 * bl + Dec::k_of(half, t, j, g >> 2);
                uint32_t r0 = 0u, r1 = 0u;
                if (kHalfB) {
                    if ((g & 3) == 0 && k + 3 < K) {
                        uint2 v = __ldg(reinterpret_cast<const uint2 *>(xh + k));
                        r0 = v.x; r1 = v.y;
                    }
                } else if ((g & 3) != 3 && k + 3 < K) {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(x + k));
                    const float v[4] = {f.x, f.y, f.z, f.w};
                    __half h[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half hi = __float2half_rn(v[i]);
                        if (!isfinite(v[i]) || __hisinf(hi)) raise(status, YVEX_B200_STATUS_NUMERIC);
                        float r1f = (v[i] - __half2float(hi)) * 2048.0f;
                        __half mid = __float2half_rn(r1f);
                        float r2f = (r1f - __half2float(mid)) * 2048.0f;
                        h[i] = (g & 3) == 0 ? hi : (g & 3) == 1 ? mid : __float2half_rn(r2f);
                    }
                    r0 = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
                    r1 = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
                }
                bfrag[8 * bl + 4 * half + j][0] = r0;
                bfrag[8 * bl + 4 * half + j][1] = r1;
            }
}

// This thread's share of its matrix row's block dot product, from the drained accumulator.
template <bool kHalfB> __device__ __forceinline__ float drain(const float (&d)[4], int t) {
    if (kHalfB) return t == 0 ? d[0] : t == 2 ? d[2] : 0.0f;
    constexpr float k11 = 1.0f / 2048.0f, k22 = 1.0f / 4194304.0f;
    return t == 0 ? d[0] + d[1] * k11 : t == 1 ? d[0] * k22 : t == 2 ? d[2] + d[3] * k11 : d[2] * k22;
}

// Per-sub-block sums of an activation row into shared memory (all warps of the CTA cooperate;
// the caller synchronises before use). G = 32 or 16 elements per sum.
template <int G> __device__ __forceinline__ void build_sums(float *sums, const float *x, int K) {
    if (G == 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    constexpr int GG = G == 0 ? 32 : G;
    for (int i = warp; i < K / GG; i += nw) {
        float v = lane < GG ? x[i * GG + lane] : 0.0f;
        v = warp_sum(v);
        if (lane == 0) sums[i] = v;
    }
}

// One warp: partial dots of its 8 rows over its K-slice, read from the staged tile. `sums` points
// at the activation sums of the slice's first block.
template <class Dec, bool kHalfB>
__device__ __forceinline__ float warp_slice_dot(const uint8_t *row, int blocks, const MmaTables *tab,
                                                const uint32_t (&bfrag)[8 * kSliceBlocks][2], const float *sums,
                                                int t, bool row_valid, int *status) {
    constexpr int kSumsPerBlock = Dec::kSumGroup ? 256 / Dec::kSumGroup : 0;
    float acc = 0.0f;
#pragma unroll
    for (int bl = 0; bl < kSliceBlocks; ++bl) {
        if (bl < blocks) {
            const uint8_t *blk = row + bl * Dec::kBlockBytes;
            float d[4] = {0.f, 0.f, 0.f, 0.f}, minacc = 0.0f;
            Dec::half_block(blk, 0, t, tab, &bfrag[8 * bl], d, minacc, sums + bl * kSumsPerBlock);
            Dec::half_block(blk, 1, t, tab, &bfrag[8 * bl], d, minacc, sums + bl * kSumsPerBlock);
            bool bad;
            acc += Dec::finish(blk, drain<kHalfB>(d, t), minacc, bad);
            if (bad && row_valid) raise(status, YVEX_B200_STATUS_NUMERIC);
        }
    }
    return acc;
}

struct GemvMmaParams {
    const uint8_t *enc;
    uint64_t rows, row_bytes;
    int K, slices, row_groups;
    const float *x, *additive;
    float *out;
    int round_bf16;
    int *status;
    uint32_t stage_bytes;
};

// Shared-memory carve-up common to the kernels built on this engine.
struct MmaSmem {
    MmaTables tab;
    float red[8 * kMaxSlices * 4];     // [row_groups][slices][8] partial dots
    float sums[kMaxSums];              // activation sums per sub-block (affine qtypes)
};

template <class Dec>
__global__ void __launch_bounds__(512) gemv_mma_kernel(GemvMmaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    MmaSmem *sm = reinterpret_cast<MmaSmem *>(smem);
    uint8_t *stages = smem + sizeof(MmaSmem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int slice = warp % p.slices, rg = warp / p.slices;
    const int tile_rows = 8 * p.row_groups;
    const uint64_t tiles = (p.rows + tile_rows - 1) / tile_rows;
    const uint8_t *lo = p.enc, *hi = p.enc + p.rows * p.row_bytes;
    load_tables(&sm->tab, Dec::kBias);
    build_sums<Dec::kSumGroup>(sm->sums, p.x, p.K);
    uint32_t bfrag[8 * kSliceBlocks][2];
    build_bfrag<Dec, false>(bfrag, p.x, nullptr, slice * 256 * kSliceBlocks, p.K, g, t, p.status);
    const int nblocks = p.K / 256;
    const int my_blocks = min(kSliceBlocks, nblocks - slice * kSliceBlocks);
    constexpr int kSumsPerBlock = Dec::kSumGroup ? 256 / Dec::kSumGroup : 0;

    auto issue = [&](uint64_t tile, int stage) {
        if (tile < tiles) {
            uint64_t r0 = tile * tile_rows;
            uint64_t n = p.rows - r0 < (uint64_t)tile_rows ? p.rows - r0 : (uint64_t)tile_rows;
            stage_span(stages + (size_t)stage * p.stage_bytes, p.enc + r0 * p.row_bytes, n * p.row_bytes, lo, hi);
        }
        cp_async_commit();
    };
    uint64_t tile = blockIdx.x;
#pragma unroll
    for (int s = 0; s < kGemvStages - 1; ++s) issue(tile + (uint64_t)s * gridDim.x, s);
    for (int it = 0; tile < tiles; tile += gridDim.x, ++it) {
        issue(tile + (uint64_t)(kGemvStages - 1) * gridDim.x, (it + kGemvStages - 1) % kGemvStages);
        cp_async_wait<kGemvStages - 1>();
        __syncthreads();
        const uint64_t r0 = tile * tile_rows;
        const uint8_t *src = p.enc + r0 * p.row_bytes;
        const uint8_t *base = stages + (size_t)(it % kGemvStages) * p.stage_bytes +
                              (reinterpret_cast<uintptr_t>(src) & 15u);
        const uint64_t row = r0 + 8 * rg + g;
        const bool valid = row < p.rows;
        const uint8_t *rowp = base + (size_t)(8 * rg + g) * p.row_bytes +
                              (size_t)slice * kSliceBlocks * Dec::kBlockBytes;
        float part = warp_slice_dot<Dec, false>(rowp, my_blocks, &sm->tab, bfrag,
                                                sm->sums + slice * kSliceBlocks * kSumsPerBlock, t, valid, p.status);
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        if (t == 0) sm->red[(rg * p.slices + slice) * 8 + g] = part;
        __syncthreads();
        if (threadIdx.x < tile_rows) {
            const int rrg = threadIdx.x >> 3, rgi = threadIdx.x & 7;
            const uint64_t orow = r0 + threadIdx.x;
            if (orow < p.rows) {
                float sum = 0.0f;
                for (int s = 0; s < p.slices; ++s) sum += sm->red[(rrg * p.slices + s) * 8 + rgi];
                if (p.additive) sum += p.additive[orow];
                if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                p.out[orow] = p.round_bf16 ? bf16_round(sum) : sum;
            }
        }
    }
    cp_async_wait<0>();
}

// K-slices (warps along K) and row groups (8-row sets per CTA) for a row width.
inline void mma_shape(uint64_t width, int &slices, int &row_groups) {
    slices = (int)((width / 256 + kSliceBlocks - 1) / kSliceBlocks);
    row_groups = slices >= 8 ? 1 : slices >= 4 ? 2 : 4;
}

inline bool mma_decoder_for(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q2_K; }

inline bool gemv_mma_eligible(unsigned q, uint64_t rows, uint64_t width, const uint8_t *enc) {
    (void)rows;
    const uintptr_t align = q == Q_Q4_K ? 15u : q == Q_Q2_K ? 3u : 1u;
    return mma_decoder_for(q) && width % 256 == 0 && width / 256 <= kMaxSlices * kSliceBlocks &&
           (reinterpret_cast<uintptr_t>(enc) & align) == 0;   // callers also need a 16-byte aligned x
}

template <class Kernel> inline int mma_opt_in(Kernel kernel) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess
               ? OK : ERR_BACKEND;
}

template <class Dec>
inline int gemv_mma_launch_t(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes,
                             const float *x, const float *additive, float *out, int round_bf16,
                             int *status, cudaStream_t stream) {
    GemvMmaParams p{};
    p.enc = enc; p.rows = rows; p.row_bytes = row_bytes; p.K = (int)width;
    mma_shape(width, p.slices, p.row_groups);
    p.x = x; p.additive = additive; p.out = out; p.round_bf16 = round_bf16; p.status = status;
    const int tile_rows = 8 * p.row_groups;
    p.stage_bytes = (uint32_t)(((uint64_t)tile_rows * row_bytes + 16 + 15) & ~15ull);
    size_t smem = sizeof(MmaSmem) + (size_t)kGemvStages * p.stage_bytes;
    static bool configured = false;
    if (!configured) {
        if (mma_opt_in(gemv_mma_kernel<Dec>) != OK) return ERR_BACKEND;
        configured = true;
    }
    if (smem > 200 * 1024) return ERR_BOUNDS;
    uint64_t tiles = (rows + tile_rows - 1) / tile_rows;
    int grid = (int)(tiles < (uint64_t)kSmCount * 2 ? tiles : (uint64_t)kSmCount * 2);
    gemv_mma_kernel<Dec><<<grid, 32 * p.slices * p.row_groups, smem, stream>>>(p);
    return launch_status();
}

inline int gemv_mma_launch(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width,
                           uint64_t row_bytes, const float *x, const float *additive, float *out,
                           int round_bf16, int *status, cudaStream_t stream) {
    switch (q) {
    case Q_IQ2_XXS:
        return gemv_mma_launch_t<Iq2Decoder>(enc, rows, width, row_bytes, x, additive, out, round_bf16, status, stream);
    case Q_Q4_K:
        return gemv_mma_launch_t<Q4kDecoder>(enc, rows, width, row_bytes, x, additive, out, round_bf16, status, stream);
    case Q_Q2_K:
        return gemv_mma_launch_t<Q2kDecoder>(enc, rows, width, row_bytes, x, additive, out, round_bf16, status, stream);
    default:
        return ERR_UNSUPPORTED;
    }
}

}  // namespace yb
