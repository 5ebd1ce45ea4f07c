// Streaming dequant-fused matvec engine for 256-element superblock qtypes.
//
// Why tensor cores for a matvec: at 0.26 bytes per IQ2_XXS weight the HBM stream delivers ~80
// weights per SM per clock, and a scalar multiply-add per weight alone would fill most of the
// FP32 pipe. Here a warp owns 8 matrix rows x a 512-weight K-slice; every thread decodes the
// eight weights of one codebook entry into four packed-fp16 registers holding EXACT small
// integers (magnitude x sign x integer sub-scale) and feeds them to mma.sync.m16n8k16 as the A
// fragment. The 16 MMA rows are 8 matrix rows x 2 halves of the entry; the B fragment carries
// the f32 activation split into three fp16 pieces (x = hi + mid*2^-11 + lo*2^-22, ~33 bits) in
// columns 0-2 for the first halves and 4-6 for the second halves, so the products are exact and
// only the f32 accumulation rounds. The per-superblock f16 scale multiplies the drained
// accumulator once per 256 weights. Because a dot product does not care about the order of k,
// the decoder is free to hand any 8 weights of its K-slice to any MMA slot as long as the B
// fragment is built with the same permutation; that is what makes the mapping cheap.
//
// Data movement: a CTA walks 8*RG-row tiles (rows are contiguous in the canonical layout), copies
// each tile into shared memory with 16-byte cp.async chunks through a kStages-deep ring, and
// decodes from there; chunks that would cross the ends of the tensor are copied with guarded
// 2-byte loads, so no byte outside [encoded, encoded + rows*row_bytes) is ever read.
#pragma once
#include "qtype_decode.cuh"

namespace yb {

constexpr int kGemvStages = 4;
constexpr int kSliceBlocks = 2;                    // 512 weights per warp K-slice
constexpr int kMaxSlices = 16;                     // K <= 8192 on this path

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

// Splits four consecutive activations into the fp16 piece this thread's B column carries.
__device__ __forceinline__ void split_piece(const float (&x)[4], int piece, uint32_t &r0,
                                            uint32_t &r1, int *status) {
    __half h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half hi = __float2half_rn(x[i]);
        if (!isfinite(x[i]) || __hisinf(hi)) raise(status, YVEX_B200_STATUS_NUMERIC);
        float r1f = (x[i] - __half2float(hi)) * 2048.0f;
        __half mid = __float2half_rn(r1f);
        float r2f = (r1f - __half2float(mid)) * 2048.0f;
        h[i] = piece == 0 ? hi : piece == 1 ? mid : piece == 2 ? __float2half_rn(r2f)
                                                                : __float2half_rn(0.0f);
    }
    r0 = static_cast<uint32_t>(__half_as_ushort(h[0])) | (static_cast<uint32_t>(__half_as_ushort(h[1])) << 16);
    r1 = static_cast<uint32_t>(__half_as_ushort(h[2])) | (static_cast<uint32_t>(__half_as_ushort(h[3])) << 16);
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

// ---- IQ2_XXS decoder ---------------------------------------------------------------------------
// A superblock is 66 bytes: f16 d, then eight 8-byte groups {4 codebook indices, 4x7 sign bits +
// 4-bit sub-scale}. value = d/8 * (2*sub+1) * (+-{8,25,43})  ==  the reference's
// d*(0.5+sub)*0.25*level*sign, every factor but d being a small integer
// (src/gguf/quant_block.c:745-767). Thread t of a quad decodes subgroup j of group 4*half+t.
struct Iq2Decoder {
    static constexpr unsigned kQtype = Q_IQ2_XXS;
    static constexpr int kBlockBytes = 66;
    static constexpr float kBias = 1152.0f;        // fp16(0x6400 | (b + 128)) = 1152 + b
    static constexpr float kBlockScale = 0.125f;

    // K index (within the block) of the first of the 4 consecutive weights that MMA j of
    // half-block `half` takes from quad thread t for the first (hi=0) / second (hi=1) half.
    __device__ static int k_of(int half, int t, int j, int hi) { return 128 * half + 32 * t + 8 * j + 4 * hi; }

    __device__ static float block_scale(const uint8_t *blk, bool &bad) {
        float d = f16_bits_to_float(*reinterpret_cast<const uint16_t *>(blk));
        bad = !isfinite(d) || d < 0.0f;
        return d * kBlockScale;
    }

    // Decodes the 32 weights of group (4*half + t) and issues the four MMAs.
    __device__ static void half_block(const uint8_t *blk, int half, int t, const MmaTables *tab,
                                      const uint32_t (*bfrag)[2], float (&d)[4], float &) {
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
            uint32_t h[4] = {__byte_perm(u_lo, 0x64646464u, 0x4140), __byte_perm(u_lo, 0x64646464u, 0x4342),
                             __byte_perm(u_hi, 0x64646464u, 0x4140), __byte_perm(u_hi, 0x64646464u, 0x4342)};
            uint32_t afrag[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 v = __hfma2(*reinterpret_cast<__half2 *>(&h[i]), sc2, nb2);
                h[i] = *reinterpret_cast<uint32_t *>(&v);
            }
            afrag[0] = h[0]; afrag[1] = h[2]; afrag[2] = h[1]; afrag[3] = h[3];
            mma_f16(d, afrag, bfrag[4 * half + j][0], bfrag[4 * half + j][1]);
        }
    }
};

// Folds a drained accumulator into this thread's share of its matrix row's dot product.
__device__ __forceinline__ float drain(const float (&d)[4], int t) {
    constexpr float k11 = 1.0f / 2048.0f, k22 = 1.0f / 4194304.0f;
    return t == 0 ? d[0] + d[1] * k11 : t == 1 ? d[0] * k22 : t == 2 ? d[2] + d[3] * k11 : d[2] * k22;
}

// Builds the B fragments of one warp's K-slice for activation row x (K floats).
template <class Dec>
__device__ __forceinline__ void build_bfrag(uint32_t (&bfrag)[8 * kSliceBlocks][2], const float *x,
                                            int kbase, int K, int g, int t, int *status) {
#pragma unroll
    for (int bl = 0; bl < kSliceBlocks; ++bl)
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int k = kbase + 256 * bl + Dec::k_of(half, t, j, g >> 2);
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (k + 3 < K) {
                    float4 f = __ldg(reinterpret_cast<const float4 *>(x + k));
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                }
                split_piece(v, g & 3, bfrag[8 * bl + 4 * half + j][0], bfrag[8 * bl + 4 * half + j][1], status);
            }
}

// One warp: partial dots of its 8 rows over its K-slice, read from the staged tile.
template <class Dec>
__device__ __forceinline__ float warp_slice_dot(const uint8_t *row, int blocks, const MmaTables *tab,
                                                const uint32_t (&bfrag)[8 * kSliceBlocks][2], int t,
                                                bool row_valid, int *status) {
    float acc = 0.0f, extra = 0.0f;
    for (int bl = 0; bl < blocks; ++bl) {
        const uint8_t *blk = row + bl * Dec::kBlockBytes;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        Dec::half_block(blk, 0, t, tab, &bfrag[8 * bl], d, extra);
        Dec::half_block(blk, 1, t, tab, &bfrag[8 * bl], d, extra);
        bool bad;
        float scale = Dec::block_scale(blk, bad);
        if (bad && row_valid) raise(status, YVEX_B200_STATUS_NUMERIC);
        acc = fmaf(scale, drain(d, t), acc);
    }
    return acc + extra;
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

template <class Dec>
__global__ void __launch_bounds__(512) gemv_mma_kernel(GemvMmaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    MmaTables *tab = reinterpret_cast<MmaTables *>(smem);
    float *red = reinterpret_cast<float *>(smem + sizeof(MmaTables));      // [row_groups][slices][8]
    uint8_t *stages = smem + sizeof(MmaTables) + sizeof(float) * 8 * kMaxSlices * 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int slice = warp % p.slices, rg = warp / p.slices;
    const int tile_rows = 8 * p.row_groups;
    const uint64_t tiles = (p.rows + tile_rows - 1) / tile_rows;
    const uint8_t *lo = p.enc, *hi = p.enc + p.rows * p.row_bytes;
    load_tables(tab, Dec::kBias);
    uint32_t bfrag[8 * kSliceBlocks][2];
    build_bfrag<Dec>(bfrag, p.x, slice * 256 * kSliceBlocks, p.K, g, t, p.status);
    const int nblocks = p.K / 256;
    const int my_blocks = min(kSliceBlocks, nblocks - slice * kSliceBlocks);

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
        float part = warp_slice_dot<Dec>(rowp, my_blocks, tab, bfrag, t, valid, p.status);
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        if (t == 0) red[(rg * p.slices + slice) * 8 + g] = part;
        __syncthreads();
        if (threadIdx.x < tile_rows) {
            const int rrg = threadIdx.x >> 3, rgi = threadIdx.x & 7;
            const uint64_t orow = r0 + threadIdx.x;
            if (orow < p.rows) {
                float sum = 0.0f;
                for (int s = 0; s < p.slices; ++s) sum += red[(rrg * p.slices + s) * 8 + rgi];
                if (p.additive) sum += p.additive[orow];
                if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                p.out[orow] = p.round_bf16 ? bf16_round(sum) : sum;
            }
        }
    }
    cp_async_wait<0>();
}

inline bool gemv_mma_eligible(unsigned q, uint64_t rows, uint64_t width, const uint8_t *enc) {
    (void)rows;
    return q == Q_IQ2_XXS && width % 256 == 0 && width / 256 <= kMaxSlices * kSliceBlocks &&
           (reinterpret_cast<uintptr_t>(enc) & 1u) == 0;   // callers also need a 16-byte aligned x
}

template <class Dec>
inline int gemv_mma_launch_t(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes,
                             const float *x, const float *additive, float *out, int round_bf16,
                             int *status, cudaStream_t stream) {
    GemvMmaParams p{};
    p.enc = enc; p.rows = rows; p.row_bytes = row_bytes; p.K = (int)width;
    p.slices = (int)((width / 256 + kSliceBlocks - 1) / kSliceBlocks);
    p.row_groups = p.slices >= 8 ? 1 : p.slices >= 4 ? 2 : 4;
    p.x = x; p.additive = additive; p.out = out; p.round_bf16 = round_bf16; p.status = status;
    const int tile_rows = 8 * p.row_groups;
    p.stage_bytes = (uint32_t)(((uint64_t)tile_rows * row_bytes + 16 + 15) & ~15ull);
    size_t smem = sizeof(MmaTables) + sizeof(float) * 8 * kMaxSlices * 4 + (size_t)kGemvStages * p.stage_bytes;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemv_mma_kernel<Dec>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024) != cudaSuccess)
            return ERR_BACKEND;
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
        return gemv_mma_launch_t<Iq2Decoder>(enc, rows, width, row_bytes, x, additive, out, round_bf16,
                                             status, stream);
    default:
        return ERR_UNSUPPORTED;
    }
}

}  // namespace yb
