// Grouped dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the wide MoE path.
//
// Problem: for every expert group g with n_g token rows, OUT[row][m] = sum_k W_g[m][k] * X[row][k],
// W_g stored as GGUF superblocks. Weights sit on the MMA M side (128-row tiles), tokens on N
// (<=128 per tile, ragged tails padded to 16), so a small group wastes at most 15 columns.
//
// Exactness: the A operand carries EXACT small integers in fp16 (IQ2_XXS: +-{8,25,43}*(2*sub+1);
// Q4_K / Q2_K: code * sub-scale), the B operand the fp16 image of bf16-exact activations, so
// every product is exact and only the f32 accumulation in TMEM rounds. The per-superblock f16
// scale d cannot ride inside the MMA; the accumulator is therefore drained once per 256 K by the
// epilogue warps (acc[row][n] += d[row][block] * tmem[row][n]) while the MMA warp fills the other
// TMEM buffer. Affine qtypes add one more K=16/32 MMA per superblock: A' = integer mins,
// B' = per-sub-block activation sums (hi/lo fp16 split), drained as acc -= dmin * tmem'.
//
// CTA = 20 warps, persistent over a device-built tile list:
//   warp 0      TMA producer: activation tiles [N x 64] fp16, 128-byte swizzle, mbarrier tx
//   warp 1      MMA issuer (one elected lane): 4 x tcgen05.mma (K=16) per 64-K chunk
//   warps 2-3   min-term tiles (A' from the packed scale bytes, B' from the sums array)
//   warps 4-11  dequant producers: thread = (weight row, half of a 64-K chunk); decode 32 weights
//               to fp16 and store four 16-byte chunks into the swizzled A tile
//   warps 12-19 epilogue: TMEM -> registers (tcgen05.ld), scale, accumulate, final store
// Every mbarrier wait is bounded; on expiry the CTA sets status 3, unwinds and frees its TMEM.
#pragma once
#include "gemv_mma.cuh"
#include "moe_common.cuh"
#include "tcgen05.cuh"

namespace yb {

constexpr int kGemmThreads = 640;
constexpr int kTileM = 128, kTileN = 128, kChunkK = 64;
constexpr int kStages = 4;                                  // ring of {A, B} 64-K chunks
constexpr uint32_t kTileBytes = kTileM * kChunkK * 2;        // 16 KiB, both A and B chunks
constexpr uint32_t kTmemCols = 512;

struct ColBlock { int row0, ncols, expert, pad; };          // expert < 0: the shared expert

struct GemmParams {
    const uint8_t *w_routed[2], *w_shared[2];   // packs; 2 matrices (gate, up) or 1 (down)
    uint64_t row_bytes;
    int M, K, nmat;
    const ColBlock *colblocks;
    const int *num_colblocks;
    float *out_f32[2];                          // [rows][M] f32 (gate/up results) ...
    uint16_t *out_bf16;                         // ... or [rows][M] bf16 bits (down results)
    const __half *sums;                         // [rows][K/256][32] hi/lo sub-block sums (affine qtypes)
    int *status;
};

struct GemmSmem {
    uint64_t full_a[kStages], full_b[kStages], empty[kStages];
    uint64_t acc_full[2], acc_empty[2], min_full[2], min_empty[2];
    uint32_t tmem_base;
    int abort;
};

// ---- per-qtype chunk decoders: 32 weights (row, k = 64*c + 32*h ..) -> four 16-byte fp16 chunks ----
__device__ __forceinline__ void store_scaled8(uint8_t *tile, uint32_t row, uint32_t chunk, uint32_t bytes_lo,
                                              uint32_t bytes_hi, __half2 sc2, __half2 nb2) {
    uint32_t a = __byte_perm(bytes_lo, 0x64646464u, 0x4140), b = __byte_perm(bytes_lo, 0x64646464u, 0x4342);
    uint32_t c = __byte_perm(bytes_hi, 0x64646464u, 0x4140), d = __byte_perm(bytes_hi, 0x64646464u, 0x4342);
    __half2 va = __hfma2(*reinterpret_cast<__half2 *>(&a), sc2, nb2), vb = __hfma2(*reinterpret_cast<__half2 *>(&b), sc2, nb2);
    __half2 vc = __hfma2(*reinterpret_cast<__half2 *>(&c), sc2, nb2), vd = __hfma2(*reinterpret_cast<__half2 *>(&d), sc2, nb2);
    uint4 v = make_uint4(*reinterpret_cast<uint32_t *>(&va), *reinterpret_cast<uint32_t *>(&vb),
                         *reinterpret_cast<uint32_t *>(&vc), *reinterpret_cast<uint32_t *>(&vd));
    *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, chunk)) = v;
}

__device__ __forceinline__ __half2 half2_of(float v) { return __float2half2_rn(v); }

struct GemmIq2 {
    static constexpr int kBlockBytes = 66, kMinSlots = 0;
    static constexpr float kBias = 1152.0f;
    // blk: the row's superblock in global memory (2-byte aligned)
    __device__ static void chunk(const uint8_t *blk, int c, int h, uint8_t *tile, uint32_t row, const MmaTables *tab) {
        const uint8_t *p = blk + 2 + 8 * (2 * c + h);
        const uint32_t grids = ld_u32_unaligned2(p), ss = ld_u32_unaligned2(p + 4);
        const uint2 sc = tab->scale[2u * (ss >> 28) + 1u];
        const __half2 sc2 = *reinterpret_cast<const __half2 *>(&sc.x), nb2 = *reinterpret_cast<const __half2 *>(&sc.y);
        constexpr uint32_t kLo = (8u + 128u) | ((25u + 128u) << 8) | ((43u + 128u) << 16);
        constexpr uint32_t kHi = (128u - 8u) | ((128u - 25u) << 8) | ((128u - 43u) << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t sel = tab->nib[(grids >> (8 * j)) & 255u] | tab->sign[(ss >> (7 * j)) & 127u];
            store_scaled8(tile, row, 4 * h + j, __byte_perm(kLo, kHi, sel), __byte_perm(kLo, kHi, sel >> 16), sc2, nb2);
        }
    }
    __device__ static float scale(const uint8_t *blk, float &dmin, bool &bad) {
        float d = f16_bits_to_float(ldg_u16(blk));
        bad = !isfinite(d) || d < 0.0f;
        dmin = 0.0f;
        return d * 0.125f;
    }
    __device__ static void mins(const uint8_t *, int, uint8_t *, uint32_t) {}
};

struct GemmQ4k {
    static constexpr int kBlockBytes = 144, kMinSlots = 16;       // 8 mins x (hi, lo)
    static constexpr float kBias = 1024.0f;
    __device__ static void scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &m) {
        if (j < 4) { sc = __ldg(s + j) & 63u; m = __ldg(s + j + 4) & 63u; }
        else { sc = (__ldg(s + j + 4) & 15u) | ((__ldg(s + j - 4) >> 6) << 4); m = (__ldg(s + j + 4) >> 4) | ((__ldg(s + j) >> 6) << 4); }
    }
    __device__ static void chunk(const uint8_t *blk, int c, int h, uint8_t *tile, uint32_t row, const MmaTables *tab) {
        uint32_t sc, m;
        scale_min(blk + 4, 2 * c + h, sc, m);
        const uint2 s = tab->scale[sc];
        const __half2 sc2 = *reinterpret_cast<const __half2 *>(&s.x), nb2 = *reinterpret_cast<const __half2 *>(&s.y);
        const uint4 *q = reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
        const uint4 q0 = __ldg(q), q1 = __ldg(q + 1);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t a = h ? (w[2 * j] >> 4) & 0x0f0f0f0fu : w[2 * j] & 0x0f0f0f0fu;
            const uint32_t b = h ? (w[2 * j + 1] >> 4) & 0x0f0f0f0fu : w[2 * j + 1] & 0x0f0f0f0fu;
            store_scaled8(tile, row, 4 * h + j, a, b, sc2, nb2);
        }
    }
    __device__ static float scale(const uint8_t *blk, float &dmin, bool &bad) {
        float d = f16_bits_to_float(ldg_u16(blk));
        dmin = f16_bits_to_float(ldg_u16(blk + 2));
        bad = !isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f;
        return d;
    }
    // A' row: slots 0..7 = mins (paired with the hi sums), 8..15 = the same mins (lo sums).
    __device__ static void mins(const uint8_t *blk, int part, uint8_t *tile, uint32_t row) {
        __half v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t sc, m;
            scale_min(blk + 4, j, sc, m);
            v[j] = __float2half_rn(static_cast<float>(m));
        }
        *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, part)) = *reinterpret_cast<uint4 *>(v);
    }
};

struct GemmQ2k {
    static constexpr int kBlockBytes = 84, kMinSlots = 32;        // 16 mins x (hi, lo)
    static constexpr float kBias = 1024.0f;
    __device__ static void chunk(const uint8_t *blk, int c, int h, uint8_t *tile, uint32_t row, const MmaTables *tab) {
        const int hf = c >> 1, plane = 2 * (c & 1) + h;
        const uint2 s0 = tab->scale[__ldg(blk + 8 * hf + 2 * plane) & 15u], s1 = tab->scale[__ldg(blk + 8 * hf + 2 * plane + 1) & 15u];
        const uint32_t *q = reinterpret_cast<const uint32_t *>(blk + 16 + 32 * hf);     // 4-byte aligned
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint2 s = j < 2 ? s0 : s1;                                            // bytes 0..15 / 16..31
            const uint32_t a = (__ldg(q + 2 * j) >> (2 * plane)) & 0x03030303u, b = (__ldg(q + 2 * j + 1) >> (2 * plane)) & 0x03030303u;
            store_scaled8(tile, row, 4 * h + j, a, b, *reinterpret_cast<const __half2 *>(&s.x), *reinterpret_cast<const __half2 *>(&s.y));
        }
    }
    __device__ static float scale(const uint8_t *blk, float &dmin, bool &bad) {
        float d = f16_bits_to_float(ldg_u16(blk + 80));
        dmin = f16_bits_to_float(ldg_u16(blk + 82));
        bad = !isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f;
        return d;
    }
    // A' row: slots 0..15 = mins (hi sums), 16..31 = the same mins (lo sums); `part` = 16-byte chunk 0..3.
    __device__ static void mins(const uint8_t *blk, int part, uint8_t *tile, uint32_t row) {
        __half v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __float2half_rn(static_cast<float>(__ldg(blk + 8 * (part & 1) + j) >> 4));
        *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, part)) = *reinterpret_cast<uint4 *>(v);
    }
};

template <class Dec>
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap act_map, GemmParams p) {
    using namespace sm100;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte aligned tiles first, bookkeeping after them
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t *a_tiles = tiles;                                   // [kStages][16 KiB]
    uint8_t *b_tiles = tiles + kStages * kTileBytes;            // [kStages][16 KiB]
    uint8_t *amin_tiles = b_tiles + kStages * kTileBytes;       // [2][16 KiB]
    uint8_t *bmin_tiles = amin_tiles + 2 * kTileBytes;          // [2][16 KiB]
    MmaTables *tab = reinterpret_cast<MmaTables *>(bmin_tiles + 2 * kTileBytes);
    GemmSmem *sm = reinterpret_cast<GemmSmem *>(reinterpret_cast<uint8_t *>(tab) + sizeof(MmaTables));
    constexpr bool kHasMin = Dec::kMinSlots > 0;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full_a[s], 8); mbar_init(&sm->full_b[s], 1); mbar_init(&sm->empty[s], 1); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm->acc_full[b], 1); mbar_init(&sm->acc_empty[b], 8);
            mbar_init(&sm->min_full[b], 2); mbar_init(&sm->min_empty[b], 1);
        }
        sm->abort = 0;
        fence_barrier_init();
    }
    load_tables(tab, Dec::kBias);
    if (warp == 0) tmem_alloc(&sm->tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    volatile int *abort = &sm->abort;

    const int ncb = *p.num_colblocks;
    const int mtiles = p.M / kTileM, nsb = p.K / 256;
    const long long tiles_total = (long long)ncb * mtiles * p.nmat;

    // Every role walks the same tile sequence: tile -> (column block, matrix, m tile), m fastest.
    auto tile_of = [&](long long t, ColBlock &cb, int &mat, int &mt) {
        const int per_cb = mtiles * p.nmat;
        cb = p.colblocks[t / per_cb];
        const int r = (int)(t % per_cb);
        mat = r / mtiles;
        mt = r % mtiles;
    };
    auto weights_of = [&](const ColBlock &cb, int mat, int mt) {
        const uint8_t *base = cb.expert < 0 ? p.w_shared[mat] : p.w_routed[mat] + (uint64_t)cb.expert * p.M * p.row_bytes;
        return base + (uint64_t)mt * kTileM * p.row_bytes;
    };

    if (warp == 0) {
        // ---------------- TMA producer: activation tiles ----------------
        if (lane == 0) {
            prefetch_tensormap(&act_map);
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                for (int kc = 0; kc < p.K / kChunkK; ++kc, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait(&sm->empty[s], ph ^ 1u, abort)) break;
                    mbar_expect_tx(&sm->full_b[s], kTileBytes);
                    tma_load_2d(b_tiles + s * kTileBytes, &act_map, kc * kChunkK, cb.row0, &sm->full_b[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, sb_it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                const uint32_t n = (uint32_t)((cb.ncols + 15) & ~15);
                const uint32_t idesc = idesc_f16(n);
                for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                    const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                    if (!mbar_wait(&sm->acc_empty[buf], bph ^ 1u, abort)) break;
                    tc_fence_after();
                    for (int c = 0; c < 4; ++c, ++it) {
                        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                        if (!mbar_wait(&sm->full_a[s], ph, abort) || !mbar_wait(&sm->full_b[s], ph, abort)) break;
                        tc_fence_after();
                        const uint32_t a0 = smem_u32(a_tiles + s * kTileBytes), b0 = smem_u32(b_tiles + s * kTileBytes);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f16(tmem + buf * kTileN, smem_desc_sw128(a0 + 32 * k), smem_desc_sw128(b0 + 32 * k), idesc,
                                     (c | k) ? 1u : 0u);
                        umma_commit(&sm->empty[s]);
                    }
                    if (kHasMin) {
                        if (!mbar_wait(&sm->min_full[buf], bph, abort)) break;
                        tc_fence_after();
                        const uint32_t a0 = smem_u32(amin_tiles + buf * kTileBytes), b0 = smem_u32(bmin_tiles + buf * kTileBytes);
#pragma unroll
                        for (int k = 0; k < Dec::kMinSlots / 16; ++k)
                            umma_f16(tmem + 256 + buf * kTileN, smem_desc_sw128(a0 + 32 * k), smem_desc_sw128(b0 + 32 * k), idesc,
                                     k ? 1u : 0u);
                        umma_commit(&sm->min_empty[buf]);
                    }
                    umma_commit(&sm->acc_full[buf]);
                }
            }
        }
    } else if (warp < 4) {
        // ---------------- min-term tiles (affine qtypes only) ----------------
        if (kHasMin) {
            const int tid = threadIdx.x - 64;                   // 0..63: two weight rows / two token rows each
            uint32_t sb_it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                const uint8_t *wbase = weights_of(cb, mat, mt);
                for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                    const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                    if (!mbar_wait(&sm->min_empty[buf], bph ^ 1u, abort)) break;
                    uint8_t *at = amin_tiles + buf * kTileBytes, *bt = bmin_tiles + buf * kTileBytes;
                    for (int r = tid; r < kTileM; r += 64) {
                        const uint8_t *blk = wbase + (uint64_t)r * p.row_bytes + (uint64_t)sb * Dec::kBlockBytes;
#pragma unroll
                        for (int part = 0; part < Dec::kMinSlots / 8; ++part) Dec::mins(blk, part, at, r);
                        // B': this token row's sums for the superblock (zero rows past the block's tail)
                        const uint4 *src = reinterpret_cast<const uint4 *>(p.sums + ((uint64_t)(cb.row0 + r) * nsb + sb) * 32);
#pragma unroll
                        for (int part = 0; part < Dec::kMinSlots / 8; ++part) {
                            uint4 v = r < cb.ncols ? __ldg(src + part) : make_uint4(0, 0, 0, 0);
                            *reinterpret_cast<uint4 *>(bt + sw128_offset(r, part)) = v;
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->min_full[buf]);
                }
            }
        }
    } else if (warp < 12) {
        // ---------------- dequant producers ----------------
        const int tid = threadIdx.x - 128, row = tid & 127, h = tid >> 7;
        uint32_t it = 0;
        for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
            ColBlock cb; int mat, mt;
            tile_of(t, cb, mat, mt);
            const uint8_t *wrow = weights_of(cb, mat, mt) + (uint64_t)row * p.row_bytes;
            for (int sb = 0; sb < nsb; ++sb) {
                const uint8_t *blk = wrow + (uint64_t)sb * Dec::kBlockBytes;
                for (int c = 0; c < 4; ++c, ++it) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!mbar_wait(&sm->empty[s], ph ^ 1u, abort)) goto done;
                    Dec::chunk(blk, c, h, a_tiles + s * kTileBytes, row, tab);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->full_a[s]);
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int ew = warp - 12, quarter = warp & 3, colhalf = ew >> 2;     // TMEM lanes 32*quarter.., columns 64*colhalf..
        const int row = 32 * quarter + lane;
        const uint32_t lane_addr = (uint32_t)(32 * quarter) << 16;
        uint32_t sb_it = 0;
        for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
            ColBlock cb; int mat, mt;
            tile_of(t, cb, mat, mt);
            const uint8_t *wrow = weights_of(cb, mat, mt) + (uint64_t)row * p.row_bytes;
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
            const int ncols_here = cb.ncols - 64 * colhalf;       // columns this warp owns that are real
            for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                float dmin;
                bool bad;
                const float d = Dec::scale(wrow + (uint64_t)sb * Dec::kBlockBytes, dmin, bad);
                if (bad) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                if (!mbar_wait(&sm->acc_full[buf], bph, abort)) goto done;
                tc_fence_after();
                if (ncols_here > 0) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t v[16];
                        tmem_ld16(tmem + lane_addr + buf * kTileN + 64 * colhalf + 16 * q, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[16 * q + i] = fmaf(d, __uint_as_float(v[i]), acc[16 * q + i]);
                        if (kHasMin) {
                            tmem_ld16(tmem + lane_addr + 256 + buf * kTileN + 64 * colhalf + 16 * q, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[16 * q + i] = fmaf(-dmin, __uint_as_float(v[i]), acc[16 * q + i]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->acc_empty[buf]);
            }
            // store: out[(row0 + n)][mt*128 + row]
            const uint64_t m = (uint64_t)mt * kTileM + row;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                if (i < ncols_here) {
                    const uint64_t orow = (uint64_t)cb.row0 + 64 * colhalf + i;
                    float v = acc[i];
                    if (!isfinite(v)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                    if (p.out_bf16) p.out_bf16[orow * p.M + m] = bf16_bits(v);
                    else p.out_f32[mat][orow * p.M + m] = v;
                }
            }
        }
    }
done:
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sm->abort) raise(p.status, YVEX_B200_STATUS_TIMEOUT);
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace yb
