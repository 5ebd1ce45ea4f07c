// Grouped dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the wide MoE path.
//
// Problem: for every expert group g with n_g token rows, OUT[row][m] = sum_k W_g[m][k] * X[row][k],
// W_g stored as GGUF superblocks. Weights sit on the MMA M side (128-row tiles), tokens on N
// (<=256 per tile for qtypes without a min term, <=128 for the affine ones whose second
// accumulator needs the other half of TMEM; ragged tails padded to 16), so a small group wastes
// at most 15 columns. A wider N halves the shared-memory traffic per flop of everything on the
// weight side (decode stores, table lookups, A operand reads), which is what bounds this kernel.
//
// Exactness: the A operand carries EXACT small integers in fp16 (IQ2_XXS: +-{8,25,43}*(2*sub+1);
// Q4_K / Q2_K: code * sub-scale), the B operand the fp16 image of bf16-exact activations, so
// every product is exact and only the f32 accumulation in TMEM rounds. The per-superblock f16
// scale d cannot ride inside the MMA; the accumulator is therefore drained once per 256 K by the
// epilogue warps (acc[row][n] += d[row][block] * tmem[row][n]) while the other TMEM buffer is
// being filled. Affine qtypes add one more K=16/32 MMA per superblock: A' = integer mins,
// B' = per-sub-block activation sums (hi/lo fp16 split), drained as acc -= dmin * tmem'.
//
// CTA = 28 warps, persistent over a device-built tile list:
//   warp 0      TMA producer: activation tiles [N x 64] fp16, 128-byte swizzle, mbarrier tx; and the raw
//               weight superblocks of the tile's 128 rows (u8 boxes, three superblocks in flight)
//   warps 1-2   MMA issuers (one elected lane each, alternating superblocks / TMEM buffers):
//               4 x tcgen05.mma (K=16) per 64-K chunk
//   warp 3      B' tiles of the min term (copies the activation sums into the swizzled tile)
//   warps 4-11  dequant producers. Each warp owns 16 weight rows of the tile; thread = (row, half of a
//               64-K chunk) decodes 32 weights of the staged superblock to fp16 and stores 16-byte
//               chunks into the swizzled A tile. The same warps write the A' rows and the
//               per-row block scales for the epilogue. (Staging the raw bytes through these warps'
//               registers cost them about as many instructions as the decode itself.)
//   warps 12-27 epilogue, one warp per (32 TMEM lanes, 64 or 32 columns): TMEM -> registers
//               (tcgen05.ld), scale, accumulate, final store
// Every mbarrier wait is bounded; on expiry the CTA sets status 3, unwinds and frees its TMEM.
//
// Two forms. The plain one multiplies by ONE matrix and stores bf16 rows (down projection). The
// fused one computes gate and up together: a tile's 128 A rows are 64 gate rows and the 64 up rows
// of the same intermediates, interleaved (A row 2i = gate row i, 2i + 1 = up row i; the producers
// are free to choose which weight row feeds which tile row). Gate and up of an intermediate then
// sit in neighbouring TMEM lanes, i.e. in neighbouring threads of an epilogue warp, which pairs
// them with one shuffle, applies the clamps, SiLU, the route weight and the single bf16 rounding
// (src/graph/moe.c:605-613) and stores the fp16 image the down GEMM reads. Neither projection is
// ever written to memory.
#pragma once
#include <type_traits>

#include "gemv_mma.cuh"
#include "moe_common.cuh"
#include "tcgen05.cuh"

namespace yb {

constexpr int kTileM = 128, kBoxN = 128, kMaxTileN = 256, kChunkK = 64;
constexpr int kStages = 4;                                  // {A, B} 64-K chunk stages: two rings of two
constexpr uint32_t kTileBytes = kTileM * kChunkK * 2;        // 16 KiB: an A chunk, or one 128-row box of a B chunk
constexpr uint32_t kTmemCols = 512;
constexpr int kScaleRing = 4;                               // superblocks of per-row scales kept for the epilogue
constexpr int kRawStages = 3;                               // raw weight superblocks in flight

// <= kTileN token rows of one expert (expert < 0: the shared expert). Column blocks of the same expert
// form groups of consecutive entries [first, first + count) covering <= kGroupRows rows: the tiles of a
// group are walked weight tile by weight tile, so the CTAs running side by side share one weight
// tile (read from DRAM once) while the group's activation rows stay in L2.
struct ColBlock { int row0, ncols, expert, first, count, pad; };
constexpr int kGroupRows = 1024;

// Tensor maps of one launch. A weight pack is described as u8 [rows / fuse][fuse * row_bytes] with
// `fuse` consecutive rows joined into one tensor row, so that the row pitch is a multiple of 16
// bytes whatever the block size (66-byte IQ2_XXS blocks give pitches that are only multiples of 2).
struct GemmMaps {
    CUtensorMap act;
    CUtensorMap w_routed[2], w_shared[2];
};

struct GemmParams {
    uint32_t row_bytes;
    int fuse;                                   // rows per tensor row of the weight maps: 1, 2, 4 or 8
    int M, K, nmat;
    const ColBlock *colblocks;
    const int *num_colblocks;
    uint16_t *out_bf16;                         // [rows][M] bf16 bits (plain kernel: down results) ...
    const int *out_rows;                        // optional: result row of sorted row r is out_rows[r]
    // optional: sorted row r is stored at this byte address instead, which may lie in ANOTHER GPU's memory
    // (plain peer stores over NVLink: an expert-parallel rank returns a pair's row straight to its home
    // rank from the epilogue, so no separate exchange carries it back); 0 = the row is dropped
    const unsigned long long *out_addr;
    __half *mid;                                // ... or [rows][M] SwiGLU intermediates as fp16 (fused gate/up kernel)
    const float *col_weight;                    // route weight of sorted row r (fused kernel)
    float limit;                                // SwiGLU clamp (fused kernel)
    const __half *sums;                         // [rows][K/256][32] hi/lo sub-block sums (affine qtypes)
    int *status;
};

struct GemmSmem {
    uint64_t full[kStages], empty[kStages];
    uint64_t raw_full[kRawStages], raw_empty[kRawStages];
    uint64_t acc_full[2], acc_empty[2], min_full[2], min_empty[2];
    uint32_t tmem_base;
    int abort;
};

// Chunk `it` (four per superblock, counted over the CTA's whole tile sequence) -> stage and phase.
// Even superblocks cycle through stages 0-1, odd ones through stages 2-3, so each MMA issuer
// only ever waits on stages whose fills it consumes itself, in order. (With one shared ring an
// issuer that skips the other's superblock could test a barrier that is still a whole phase
// behind, and a parity wait cannot tell "one phase behind" from "done".)
__device__ __forceinline__ uint32_t stage_of(uint32_t it) { return ((it >> 1) & 2u) | (it & 1u); }
__device__ __forceinline__ uint32_t phase_of(uint32_t it) { return (it >> 1) & 1u; }     // fills per stage: 2 per own superblock

// ---- per-qtype decoders -----------------------------------------------------------------------------
// A decoder sees one superblock of one weight row as 32-bit words in shared memory, starting at the
// 4-byte aligned address at or below the block (`mis` = bytes skipped, 0 or 2). kBoxBytes is the
// width of the TMA box that fetches it: the block plus the most its start can lie above a 16-byte
// boundary (block sizes are multiples of 2, 4 or 16 bytes), rounded up to 16.
//   kParts     threads per row: each decodes 64 / kParts weights of a 64-K chunk
//   store      weights k = 64*c + (64/kParts)*part .. -> 16-byte fp16 chunks of the A tile row
//   scales     {d, dmin} of the block, and whether they are acceptable
//   mins       this thread's share of the A' row (affine qtypes)
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

// Four bytes (each < 1024) -> four exact fp16 values: 0x6400 | b is 1024 + b, minus 1024.
__device__ __forceinline__ uint2 bytes_to_half4(uint32_t b4) {
    uint32_t lo = __byte_perm(b4, 0x64646464u, 0x4140), hi = __byte_perm(b4, 0x64646464u, 0x4342);
    const __half2 k = __floats2half2_rn(1024.0f, 1024.0f);
    const __half2 a = __hsub2(*reinterpret_cast<__half2 *>(&lo), k), b = __hsub2(*reinterpret_cast<__half2 *>(&hi), k);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
}

__device__ __forceinline__ float2 checked_scales(uint32_t d_bits, uint32_t dmin_bits, float d_mul, bool &bad) {
    const float d = f16_bits_to_float((uint16_t)d_bits), dmin = f16_bits_to_float((uint16_t)dmin_bits);
    bad = !isfinite(d) || !isfinite(dmin) || d < 0.0f || dmin < 0.0f;
    return make_float2(d * d_mul, dmin);
}

// prmt.b32 with a run-time selector. (__byte_perm masks the selector with 0x7777 first; the decoders'
// selectors never have bit 3 of a nibble set, and the instruction reads only the low 16 bits.)
__device__ __forceinline__ uint32_t prmt_raw(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

struct GemmIq2 {
    static constexpr int kBlockBytes = 66, kMinSlots = 0, kBoxBytes = 80;     // 66 bytes from a 2-byte aligned start
    static constexpr int kParts = 2;
    static constexpr float kBias = 1152.0f;
    __device__ static void store(const uint32_t *raw, uint32_t mis, int c, int h, uint8_t *tile, uint32_t row,
                                 const MmaTables *tab) {
        const uint32_t o = mis + 2u + 8u * (2 * c + h), sh = 8u * (o & 3u);
        const uint32_t *w = raw + (o >> 2);
        const uint32_t w1 = w[1];
        const uint32_t grids = __funnelshift_r(w[0], w1, sh), ss = __funnelshift_r(w1, w[2], sh);
        const uint2 sc = tab->scale[2u * (ss >> 28) + 1u];
        const __half2 sc2 = *reinterpret_cast<const __half2 *>(&sc.x), nb2 = *reinterpret_cast<const __half2 *>(&sc.y);
        constexpr uint32_t kLo = (8u + 128u) | ((25u + 128u) << 8) | ((43u + 128u) << 16);
        constexpr uint32_t kHi = (128u - 8u) | ((128u - 25u) << 8) | ((128u - 43u) << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t sel = tab->nib[(grids >> (8 * j)) & 255u] | tab->sign[(ss >> (7 * j)) & 127u];
            store_scaled8(tile, row, 4 * h + j, prmt_raw(kLo, kHi, sel), prmt_raw(kLo, kHi, sel >> 16), sc2, nb2);
        }
    }
    __device__ static float2 scales(const uint32_t *raw, uint32_t mis, bool &bad) {
        return checked_scales(raw[0] >> (8u * mis), 0u, 0.125f, bad);
    }
    __device__ static void mins(const uint32_t *, int, uint8_t *, uint32_t) {}
};

struct GemmQ4k {
    static constexpr int kBlockBytes = 144, kMinSlots = 16, kBoxBytes = 144;   // 8 mins x (hi, lo); blocks are 16-byte aligned
    static constexpr int kParts = 4;
    static constexpr float kBias = 1024.0f;
    // 6-bit (scale, min) of sub-block j from the 12 packed bytes held as three little-endian words
    __device__ static void scale_min_words(uint32_t s0, uint32_t s1, uint32_t s2, int j, uint32_t &sc, uint32_t &m) {
        const uint32_t w[3] = {s0, s1, s2};
        auto byte = [&](int i) { return (w[i >> 2] >> (8 * (i & 3))) & 255u; };
        if (j < 4) { sc = byte(j) & 63u; m = byte(j + 4) & 63u; }
        else { sc = (byte(j + 4) & 15u) | ((byte(j - 4) >> 6) << 4); m = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4); }
    }
    // part = 2 * h + half: sub-block 2c + h (low or high nibbles of the chunk's 32 bytes), bytes 16*half .. +15
    __device__ static void store(const uint32_t *raw, uint32_t, int c, int part, uint8_t *tile, uint32_t row, const MmaTables *tab) {
        const int h = part >> 1;
        uint32_t sc, m;
        scale_min_words(raw[1], raw[2], raw[3], 2 * c + h, sc, m);
        const uint2 s = tab->scale[sc];
        const __half2 sc2 = *reinterpret_cast<const __half2 *>(&s.x), nb2 = *reinterpret_cast<const __half2 *>(&s.y);
        const uint4 q = *reinterpret_cast<const uint4 *>(raw + 4 + 8 * c + 4 * (part & 1));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t a = h ? (w[2 * j] >> 4) & 0x0f0f0f0fu : w[2 * j] & 0x0f0f0f0fu;
            const uint32_t b = h ? (w[2 * j + 1] >> 4) & 0x0f0f0f0fu : w[2 * j + 1] & 0x0f0f0f0fu;
            store_scaled8(tile, row, 2 * part + j, a, b, sc2, nb2);
        }
    }
    __device__ static float2 scales(const uint32_t *raw, uint32_t, bool &bad) {
        return checked_scales(raw[0], raw[0] >> 16, 1.0f, bad);
    }
    // A' row: slots 0..7 = the eight mins (paired with the hi sums), 8..15 = the same mins (lo sums);
    // thread h writes 16-byte part h.
    // (the eight 6-bit mins, four bytes at a time: mins 0..3 are bytes 4..7 & 63, mins 4..7 the high
    // nibbles of bytes 8..11 with the top two bits of bytes 4..7 above them)
    __device__ static void mins(const uint32_t *raw, int h, uint8_t *tile, uint32_t row) {
        const uint32_t s1 = raw[2], s2 = raw[3];
        const uint2 a = bytes_to_half4(s1 & 0x3f3f3f3fu);
        const uint2 b = bytes_to_half4(((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4));
        *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, h)) = make_uint4(a.x, a.y, b.x, b.y);
    }
};

struct GemmQ2k {
    static constexpr int kBlockBytes = 84, kMinSlots = 32, kBoxBytes = 96;     // 16 mins x (hi, lo); 4-byte aligned start
    static constexpr int kParts = 4;
    static constexpr float kBias = 1024.0f;
    // part = 2 * h + half: 2-bit plane 2*(c&1) + h of the 32 bytes, bytes 16*half .. +15 (one 16-weight sub-block)
    __device__ static void store(const uint32_t *raw, uint32_t, int c, int part, uint8_t *tile, uint32_t row, const MmaTables *tab) {
        const int hf = c >> 1, plane = 2 * (c & 1) + (part >> 1), half = part & 1;
        const uint32_t *q = raw + 4 + 8 * hf + 4 * half;
        const uint32_t sbytes = raw[2 * hf + (plane >> 1)] >> (16 * (plane & 1) + 8 * half);   // scale byte 8*hf + 2*plane + half
        const uint2 s = tab->scale[sbytes & 15u];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t a = (q[2 * j] >> (2 * plane)) & 0x03030303u, b = (q[2 * j + 1] >> (2 * plane)) & 0x03030303u;
            store_scaled8(tile, row, 2 * part + j, a, b, *reinterpret_cast<const __half2 *>(&s.x), *reinterpret_cast<const __half2 *>(&s.y));
        }
    }
    __device__ static float2 scales(const uint32_t *raw, uint32_t, bool &bad) {
        return checked_scales(raw[20], raw[20] >> 16, 1.0f, bad);
    }
    // A' row: slots 0..15 = the sixteen mins (hi sums), 16..31 = the same mins (lo sums); thread h
    // converts mins 8h..8h+7 and writes them to parts h and h + 2.
    __device__ static void mins(const uint32_t *raw, int h, uint8_t *tile, uint32_t row) {
        const uint2 a = bytes_to_half4((raw[2 * h] >> 4) & 0x0f0f0f0fu), b = bytes_to_half4((raw[2 * h + 1] >> 4) & 0x0f0f0f0fu);
        const uint4 v = make_uint4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, h)) = v;
        *reinterpret_cast<uint4 *>(tile + sm100::sw128_offset(row, h + 2)) = v;
    }
};

// ---- shared-memory plan -----------------------------------------------------------------------------
// tiles (1024-byte aligned; the kernel refuses to run if the dynamic shared memory does not start on
// such a boundary): A ring, B ring, [min tiles: A' in 16-byte parts 0..3 of each row, B' in parts
// 4..7], then the raw superblock ring (kRawStages x 128 rows x kBoxBytes, plus a pad: the decoders'
// funnel reads run one word over), the scale ring, the decode tables and the barriers.
template <class Dec> struct GemmPlan {
    static constexpr bool kHasMin = Dec::kMinSlots > 0;
    static constexpr int kTileN = kHasMin ? 128 : 256;                              // columns per tile
    // 8 producer and 16 epilogue warps: an epilogue warp owns 32 TMEM lanes x kColsPerWarp columns
    // (64 with 256-column tiles, 32 with 128-column ones, where the shorter tile-end store matters
    // more than more producers: with K of 1536..2048 a tile ends every six to eight superblocks)
    static constexpr int kEpilogueWarps = 16, kColsPerWarp = kTileN / (kEpilogueWarps / 4);
    static constexpr int kProducerWarps = 8, kRowsPerWarp = kTileM / kProducerWarps;
    static constexpr int kPartsPerThread = Dec::kParts / (32 / kRowsPerWarp);       // chunk parts a producer thread decodes
    static constexpr int kThreads = 32 * (4 + kProducerWarps + kEpilogueWarps);
    // registers per thread of each role (setmaxnreg); the B' warp of the affine qtypes holds a tile of sums
    static constexpr int kCtlRegs = kHasMin ? 72 : 48;                               // the B' warp holds eight uint4
    static constexpr int kProdRegs = kHasMin ? 56 : 48, kEpiRegs = kHasMin ? 80 : 88;
    static constexpr uint32_t kBTileBytes = (kTileN / kBoxN) * kTileBytes;
    static constexpr uint32_t kRawStageBytes = kTileM * Dec::kBoxBytes;
    using Scale = typename std::conditional<kHasMin, float2, float>::type;          // {d, dmin} or d per row and superblock
    static constexpr size_t kTilesBytes = (size_t)kStages * (kTileBytes + kBTileBytes) + (kHasMin ? 2 : 0) * (size_t)kTileBytes;
    static constexpr size_t kRawBytes = (size_t)kRawStages * kRawStageBytes + 128;
    static constexpr size_t kScaleBytes = (size_t)kScaleRing * kTileM * sizeof(Scale);
    static constexpr size_t kBytes = kTilesBytes + kRawBytes + kScaleBytes + sizeof(MmaTables) + sizeof(GemmSmem);
    static_assert(kBytes <= 227 * 1024, "shared memory plan exceeds the 227 KiB a CTA can have");
    static_assert(kRawStageBytes % 128 == 0 && (kTileM / 16) * Dec::kBoxBytes % 128 == 0,
                  "TMA destinations are 128-byte aligned (boxes of 64 rows, up to 8 rows fused)");
};

// Sets this warpgroup's registers per thread to N, given the count the kernel was launched with. An
// increase waits until other warpgroups of the CTA have handed enough registers back.
template <int N, int kLaunched> __device__ __forceinline__ void set_registers() {
    if constexpr (N > kLaunched) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
    else if constexpr (N < kLaunched) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <class Dec, bool kFused>
__global__ void __launch_bounds__(GemmPlan<Dec>::kThreads, 1)
moe_grouped_gemm_kernel(const __grid_constant__ GemmMaps maps, GemmParams p) {
    using namespace sm100;
    using Plan = GemmPlan<Dec>;
    constexpr bool kHasMin = Plan::kHasMin;
    constexpr int kTileN = Plan::kTileN;
    constexpr uint32_t kBTileBytes = Plan::kBTileBytes;
    constexpr int kProducerWarps = Plan::kProducerWarps, kRowsPerWarp = Plan::kRowsPerWarp;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    if (smem_u32(smem_raw) & 1023u) {                           // uniform: nothing has been set up yet
        if (threadIdx.x == 0) raise(p.status, YVEX_B200_STATUS_TIMEOUT);
        return;
    }
    uint8_t *tiles = smem_raw;
    uint8_t *a_tiles = tiles;                                   // [kStages][16 KiB]
    uint8_t *b_tiles = tiles + kStages * kTileBytes;            // [kStages][16 or 32 KiB]
    uint8_t *min_tiles = b_tiles + kStages * kBTileBytes;       // [2][16 KiB] when the qtype has mins
    uint8_t *raw_stage = tiles + Plan::kTilesBytes;             // [kRawStages][fuse][128 / fuse rows][kBoxBytes]
    typename Plan::Scale *dscale = reinterpret_cast<typename Plan::Scale *>(raw_stage + Plan::kRawBytes);
    MmaTables *tab = reinterpret_cast<MmaTables *>(reinterpret_cast<uint8_t *>(dscale) + Plan::kScaleBytes);
    GemmSmem *sm = reinterpret_cast<GemmSmem *>(reinterpret_cast<uint8_t *>(tab) + sizeof(MmaTables));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        // full[s]: 8 producer warps + the TMA thread's expect_tx arrival (and its bytes) complete a stage,
        // so an MMA issuer pays for one wait per 64-K chunk, not two.
        for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full[s], kProducerWarps + 1); mbar_init(&sm->empty[s], 1); }
        for (int s = 0; s < kRawStages; ++s) { mbar_init(&sm->raw_full[s], 1); mbar_init(&sm->raw_empty[s], kProducerWarps); }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm->acc_full[b], 1); mbar_init(&sm->acc_empty[b], Plan::kEpilogueWarps);
            mbar_init(&sm->min_full[b], kProducerWarps + 1); mbar_init(&sm->min_empty[b], 1);
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
    constexpr int kRowsPerMat = kFused ? kTileM / 2 : kTileM;      // weight rows of one matrix in a tile
    const int mtiles = p.M / kRowsPerMat, nsb = p.K / 256;
    const long long tiles_total = (long long)ncb * mtiles * p.nmat;

    // Every role walks the same tile sequence: group of column blocks -> (matrix, m tile) -> column block.
    auto tile_of = [&](long long t, ColBlock &cb, int &mat, int &mt) {
        const int per_cb = mtiles * p.nmat;
        const ColBlock g0 = p.colblocks[t / per_cb];            // any block of the group names the group
        const int local = (int)(t - (long long)g0.first * per_cb);
        const int r = local / g0.count;
        cb = p.colblocks[g0.first + local % g0.count];
        mat = r / mtiles;
        mt = r % mtiles;
    };
    // Weight map and first tensor row of a tile. (Selects, not maps.w_routed[mat]: a dynamically
    // indexed parameter array makes the compiler copy the parameter block to local memory.)
    auto weights_of = [&](const ColBlock &cb, int mat, int mt, int &y) {
        const CUtensorMap *shared = mat ? &maps.w_shared[1] : &maps.w_shared[0], *routed = mat ? &maps.w_routed[1] : &maps.w_routed[0];
        y = ((cb.expert < 0 ? 0 : cb.expert * p.M) + mt * kRowsPerMat) / p.fuse;
        return cb.expert < 0 ? shared : routed;
    };

    // Register budget per role (256-column tiles only: 28 warps leave 72 registers per thread, and the
    // epilogue's 64 partial sums per thread do not fit in that): the control warps hand registers back
    // and the epilogue warpgroups take them. Warps 0-3, 4-11 and 12+ are whole warpgroups.
    {
        static_assert(4 * Plan::kCtlRegs + kProducerWarps * Plan::kProdRegs + Plan::kEpilogueWarps * Plan::kEpiRegs <=
                                           ((65536 / Plan::kThreads) & ~7) * (Plan::kThreads / 32),
                      "the role budgets must fit in the registers the CTA was launched with, or the increase never returns");
        constexpr int kLaunched = (65536 / Plan::kThreads) & ~7;
        if (warp < 4) set_registers<Plan::kCtlRegs, kLaunched>();
        else if (warp < 4 + kProducerWarps) set_registers<Plan::kProdRegs, kLaunched>();
        else set_registers<Plan::kEpiRegs, kLaunched>();
    }
    if (warp == 0) {
        // ---------------- TMA producer: activation tiles ----------------
        if (lane == 0) {
            prefetch_tensormap(&maps.act);
            // Raw weight superblocks run kRawStages - 1 ahead of the producers: one box per fused row
            // r, [128 / fuse tensor rows] x [kBoxBytes from the 16-byte boundary at or below the block].
            // (the fused form: the same from each of the two matrices, 64 / fuse tensor rows per box)
            struct { long long t; int sb, y; uint32_t n; const CUtensorMap *map, *map2; } raw{(long long)blockIdx.x, 0, 0, 0u, nullptr, nullptr};
            auto issue_raw = [&]() -> bool {
                if (raw.t >= tiles_total) return true;
                if (raw.sb == 0) {
                    ColBlock cb; int mat, mt;
                    tile_of(raw.t, cb, mat, mt);
                    raw.map = weights_of(cb, mat, mt, raw.y);
                    if constexpr (kFused) raw.map2 = weights_of(cb, 1, mt, raw.y);
                }
                const uint32_t s = raw.n % kRawStages, ph = (raw.n / kRawStages) & 1u;
                if (!mbar_wait(&sm->raw_empty[s], ph ^ 1u, abort)) return false;
                mbar_expect_tx(&sm->raw_full[s], Plan::kRawStageBytes);
                const int rows = kRowsPerMat / p.fuse;
                for (int r = 0; r < p.fuse; ++r) {
                    const int x = (int)(r * p.row_bytes + raw.sb * Dec::kBlockBytes) & ~15;
                    uint8_t *dst = raw_stage + s * Plan::kRawStageBytes + r * rows * Dec::kBoxBytes;
                    tma_load_2d(dst, raw.map, x, raw.y, &sm->raw_full[s]);
                    if constexpr (kFused) tma_load_2d(dst + kRowsPerMat * Dec::kBoxBytes, raw.map2, x, raw.y, &sm->raw_full[s]);
                }
                ++raw.n;
                if (++raw.sb == nsb) { raw.sb = 0; raw.t += gridDim.x; }
                return true;
            };
            bool ok = true;
            for (int i = 0; i < kRawStages - 1 && ok; ++i) ok = issue_raw();
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort && ok; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                const bool two = cb.ncols > kBoxN;             // a second 128-row box (only when kTileN = 256)
                for (int kc = 0; kc < p.K / kChunkK; ++kc, ++it) {
                    const uint32_t s = stage_of(it), ph = phase_of(it);
                    if (!mbar_wait(&sm->empty[s], ph ^ 1u, abort)) { ok = false; break; }
                    mbar_expect_tx(&sm->full[s], two ? 2 * kTileBytes : kTileBytes);
                    tma_load_2d(b_tiles + s * kBTileBytes, &maps.act, kc * kChunkK, cb.row0, &sm->full[s]);
                    if (two) tma_load_2d(b_tiles + s * kBTileBytes + kTileBytes, &maps.act, kc * kChunkK, cb.row0 + kBoxN, &sm->full[s]);
                    // after the second chunk of a superblock: by then the producers have finished the
                    // superblock before it, whose stage the next raw load reuses, so this wait is short
                    if ((kc & 3) == 1 && !issue_raw()) { ok = false; break; }
                }
            }
        }
    } else if (warp < 3) {
        // ---------------- MMA issuers ----------------
        // Issuing is latency-bound in the issuing thread (barrier wait + four tcgen05.mma + commit cost
        // more cycles than the MMAs execute), so two threads alternate superblocks: warp 1 fills TMEM
        // buffer 0 with the even ones, warp 2 buffer 1 with the odd ones. The buffers are independent
        // accumulators, so no ordering between the two instruction streams is needed.
        if (lane == 0) {
            const uint32_t mine = (uint32_t)(warp - 1);
            const uint64_t adesc0 = smem_desc_sw128(smem_u32(a_tiles)), bdesc0 = smem_desc_sw128(smem_u32(b_tiles));
            const uint64_t amin0 = smem_desc_sw128(smem_u32(min_tiles + mine * kTileBytes));
            const uint64_t bmin0 = amin0 + 4;                  // parts 4..7 of the same rows (64 bytes along K)
            uint32_t sb_it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                const uint32_t n = (uint32_t)((cb.ncols + 15) & ~15);
                const uint32_t idesc = idesc_f16(n);
                for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                    if ((sb_it & 1u) != mine) continue;
                    const uint32_t bph = (sb_it >> 1) & 1u;
                    if (!mbar_wait(&sm->acc_empty[mine], bph ^ 1u, abort)) break;
                    tc_fence_after();
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t it = 4u * sb_it + c, s = stage_of(it), ph = phase_of(it);
                        if (!mbar_wait(&sm->full[s], ph, abort)) break;
                        tc_fence_after();
                        // descriptors differ from the stage-0 ones only in the start-address field (16-byte units)
                        const uint64_t ad = adesc0 + (uint64_t)(s * (kTileBytes >> 4)), bd = bdesc0 + (uint64_t)(s * (kBTileBytes >> 4));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f16(tmem + mine * kTileN, ad + 2 * k, bd + 2 * k, idesc, (c | k) ? 1u : 0u);
                        umma_commit(&sm->empty[s]);
                    }
                    if (kHasMin) {
                        if (!mbar_wait(&sm->min_full[mine], bph, abort)) break;
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < Dec::kMinSlots / 16; ++k)
                            umma_f16(tmem + 2 * kTileN + mine * kTileN, amin0 + 2 * k, bmin0 + 2 * k, idesc, k ? 1u : 0u);
                        umma_commit(&sm->min_empty[mine]);
                    }
                    umma_commit(&sm->acc_full[mine]);
                }
            }
        }
    } else if (warp < 4) {
        // ---------------- B' tiles of the min term (affine qtypes only) ----------------
        if (kHasMin) {
            constexpr int kParts = kHasMin ? Dec::kMinSlots / 8 : 1, kRowsPerPass = 32 / kParts;
            const int part = lane % kParts, rsub = lane / kParts;
            uint32_t sb_it = 0;
            for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
                ColBlock cb; int mat, mt;
                tile_of(t, cb, mat, mt);
                for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                    const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                    // this token row's sums for the superblock (zero rows past the block's tail), eight rows
                    // per lane in flight together; the first eight are loaded before the wait for the tile
                    constexpr int kPasses = kTileM / kRowsPerPass, kBatch = 8;
                    uint8_t *tile = min_tiles + buf * kTileBytes;
#pragma unroll
                    for (int base = 0; base < kPasses; base += kBatch) {
                        uint4 v[kBatch];
#pragma unroll
                        for (int i = 0; i < kBatch; ++i) {
                            const int r = rsub + (base + i) * kRowsPerPass;
                            const uint4 *src = reinterpret_cast<const uint4 *>(p.sums + ((uint64_t)(cb.row0 + r) * nsb + sb) * 32);
                            v[i] = r < cb.ncols ? __ldg(src + part) : make_uint4(0, 0, 0, 0);
                        }
                        if (base == 0 && !mbar_wait_warp(&sm->min_empty[buf], bph ^ 1u, abort)) goto done;
#pragma unroll
                        for (int i = 0; i < kBatch; ++i)
                            *reinterpret_cast<uint4 *>(tile + sw128_offset(rsub + (base + i) * kRowsPerPass, 4 + part)) = v[i];
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->min_full[buf]);
                }
            }
        }
    } else if (warp < 4 + kProducerWarps) {
        // ---------------- dequant producers ----------------
        const int pw = warp - 4, rl = lane % kRowsPerWarp, h = lane / kRowsPerWarp;     // h: this thread's part of a chunk
        const uint32_t row = (uint32_t)(kRowsPerWarp * pw + rl);
        // where the row's bytes land in a raw stage, and where its superblock 0 starts in the tensor row
        // (fused form: tile row 2i is row i of the first matrix, 2i + 1 row i of the second, whose boxes follow)
        const uint32_t wrow = kFused ? row >> 1 : row, wmat = kFused ? row & 1u : 0u;
        const uint32_t sub = wrow % (uint32_t)p.fuse;
        const uint32_t slot = ((wmat * (uint32_t)p.fuse + sub) * (uint32_t)(kRowsPerMat / p.fuse) + wrow / (uint32_t)p.fuse) * Dec::kBoxBytes;
        const uint32_t x_row = sub * p.row_bytes;
        const long long my_tiles = tiles_total > blockIdx.x ? (tiles_total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        uint32_t sb_it = 0;
        for (long long tile = 0; tile < my_tiles && !*abort; ++tile) {
            for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                const uint32_t rs = sb_it % kRawStages, rph = (sb_it / kRawStages) & 1u;
                if (!mbar_wait_warp(&sm->raw_full[rs], rph, abort)) goto done;
                const uint32_t off = (x_row + (uint32_t)sb * Dec::kBlockBytes) & 15u, mis = off & 3u;
                const uint32_t *raw = reinterpret_cast<const uint32_t *>(raw_stage + rs * Plan::kRawStageBytes + slot + (off & ~3u));
                if (h == 0) {
                    bool bad;
                    const float2 dd = Dec::scales(raw, mis, bad);
                    if constexpr (kHasMin) dscale[(sb_it % kScaleRing) * kTileM + row] = dd;
                    else dscale[(sb_it % kScaleRing) * kTileM + row] = dd.x;
                    if (bad) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t it = 4u * sb_it + c, s = stage_of(it), ph = phase_of(it);
                    if (!mbar_wait_warp(&sm->empty[s], ph ^ 1u, abort)) goto done;
#pragma unroll
                    for (int q = 0; q < Plan::kPartsPerThread; ++q)
                        Dec::store(raw, mis, c, h * Plan::kPartsPerThread + q, a_tiles + s * kTileBytes, row, tab);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->full[s]);
                }
                if (kHasMin) {
                    const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                    if (!mbar_wait_warp(&sm->min_empty[buf], bph ^ 1u, abort)) goto done;
                    if (h < 2) Dec::mins(raw, h, min_tiles + buf * kTileBytes, row);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->min_full[buf]);
                }
                __syncwarp();                                   // every lane is done reading the stage
                if (lane == 0) mbar_arrive(&sm->raw_empty[rs]);
            }
        }
    } else {
        // ---------------- epilogue ----------------
        constexpr int kCols = Plan::kColsPerWarp;
        const int ew = warp - (4 + kProducerWarps), quarter = warp & 3, colhalf = ew >> 2;     // TMEM lanes 32*quarter.., columns kCols*colhalf..
        const int row = 32 * quarter + lane;
        const uint32_t lane_addr = (uint32_t)(32 * quarter) << 16;
        uint32_t sb_it = 0;
        for (long long t = blockIdx.x; t < tiles_total && !*abort; t += gridDim.x) {
            ColBlock cb; int mat, mt;
            tile_of(t, cb, mat, mt);
            float acc[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) acc[i] = 0.0f;
            const int ncols_here = cb.ncols - kCols * colhalf;    // columns this warp owns that are real
            // fused form: the route weights of this warp's columns, lane l holding those of columns l and
            // 32 + l; loaded here so that their latency is long gone when the tile ends
            float w_lo = 0.0f, w_hi = 0.0f;
            if constexpr (kFused) {
                const float *wcol = p.col_weight + cb.row0 + kCols * colhalf;
                if (lane < ncols_here) w_lo = __ldg(wcol + lane);
                if (kCols > 32 && 32 + lane < ncols_here) w_hi = __ldg(wcol + 32 + lane);
            }
            for (int sb = 0; sb < nsb; ++sb, ++sb_it) {
                const uint32_t buf = sb_it & 1u, bph = (sb_it >> 1) & 1u;
                if (!mbar_wait_warp(&sm->acc_full[buf], bph, abort)) goto done;
                tc_fence_after();
                // written by the row's producer before its last chunk of this superblock was published
                float d, dmin = 0.0f;
                if constexpr (kHasMin) { const float2 dd = dscale[(sb_it % kScaleRing) * kTileM + row]; d = dd.x; dmin = dd.y; }
                else d = dscale[(sb_it % kScaleRing) * kTileM + row];
                {
                    // (16-column groups without a real column are skipped: their sums stay zero, and the
                    // columns of a ragged group hold sums over neighbouring real rows, so every sum is
                    // finite unless real data is not)
#pragma unroll
                    for (int q = 0; q < kCols / 16; ++q) {
                        if (16 * q >= ncols_here) break;
                        uint32_t v[16];
                        tmem_ld16(tmem + lane_addr + buf * kTileN + kCols * colhalf + 16 * q, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[16 * q + i] = fmaf(d, __uint_as_float(v[i]), acc[16 * q + i]);
                        if (kHasMin) {
                            tmem_ld16(tmem + lane_addr + 2 * kTileN + buf * kTileN + kCols * colhalf + 16 * q, v);
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
            // non-finite sums are refused: x * 0 is zero for finite x and NaN otherwise
            float poison = 0.0f;
#pragma unroll
            for (int i = 0; i < kCols; ++i) poison = fmaf(acc[i], 0.0f, poison);
            if (poison != poison) raise(p.status, YVEX_B200_STATUS_NUMERIC);
            if constexpr (kFused) {
                // Even lanes hold the gate row of intermediate i = row / 2, odd lanes its up row. A pair of
                // lanes swaps every other column, so the even lane ends up with gate and up of the even
                // columns, the odd lane of the odd ones, and each evaluates half of the pair's SwiGLUs.
                // Then the four lanes of equal parity in every aligned group of eight transpose 4 x 4
                // blocks (intermediates x columns) with shuffles: lane (a, r, parity) ends up with
                // intermediates 4a..4a+3 of column 8b + 2r + parity, multiplies by that column's route
                // weight and stores them as one 8-byte vector.
                // Shuffles share the shared-memory pipe with the producers' table lookups and tile stores,
                // which keep it busy, so a shuffle takes long to come back. The tile end is therefore
                // written in ROUNDS of independent shuffles (all swaps; all first transpose steps; all
                // second steps) rather than block by block with three dependent shuffles each.
                const bool odd = lane & 1, o2 = lane & 2, o4 = lane & 4;
                const int rr = (lane >> 1) & 3;
                const uint64_t m0 = (uint64_t)mt * kRowsPerMat + 16 * quarter + 4 * (lane >> 3);
#pragma unroll
                for (int m = 0; m < kCols / 2; ++m) {               // acc[2m] = gate, acc[2m + 1] = up of column 2m + parity
                    const float keep = odd ? acc[2 * m + 1] : acc[2 * m];
                    const float got = __shfl_xor_sync(0xffffffffu, odd ? acc[2 * m] : acc[2 * m + 1], 1);
                    acc[2 * m] = odd ? got : keep;
                    acc[2 * m + 1] = odd ? keep : got;
                }
#pragma unroll
                for (int m = 0; m < kCols / 2; ++m)                 // acc[m] = silu(gate) * up
                    acc[m] = swiglu_product(acc[2 * m], acc[2 * m + 1], 1.0f, p.limit);
                float wv[kCols / 8];                                // route weight of column 8b + 2rr + parity
#pragma unroll
                for (int b = 0; b < kCols / 8; ++b) wv[b] = __shfl_sync(0xffffffffu, b < 4 ? w_lo : w_hi, (8 * b + 2 * rr + (odd ? 1 : 0)) & 31);
#pragma unroll
                for (int b0 = 0; b0 < kCols / 8; b0 += 4) {           // four blocks (eight shuffles) per round
#pragma unroll
                    for (int b = b0; b < b0 + 4; ++b) {
                        float *r = acc + 4 * b;
                        const float s0 = __shfl_xor_sync(0xffffffffu, o2 ? r[0] : r[1], 2), s1 = __shfl_xor_sync(0xffffffffu, o2 ? r[2] : r[3], 2);
                        if (o2) { r[0] = s0; r[2] = s1; } else { r[1] = s0; r[3] = s1; }
                    }
#pragma unroll
                    for (int b = b0; b < b0 + 4; ++b) {
                        float *r = acc + 4 * b;
                        const float s0 = __shfl_xor_sync(0xffffffffu, o4 ? r[0] : r[2], 4), s1 = __shfl_xor_sync(0xffffffffu, o4 ? r[1] : r[3], 4);
                        if (o4) { r[0] = s0; r[1] = s1; } else { r[2] = s0; r[3] = s1; }
                    }
                }
                bool bad = false;
#pragma unroll
                for (int b = 0; b < kCols / 8; ++b) {
                    const int col = 8 * b + 2 * rr + (odd ? 1 : 0);
                    if (col < ncols_here) {
                        const uint64_t srow = (uint64_t)cb.row0 + kCols * colhalf + col;
                        const float r0 = acc[4 * b] * wv[b], r1 = acc[4 * b + 1] * wv[b], r2 = acc[4 * b + 2] * wv[b], r3 = acc[4 * b + 3] * wv[b];
                        bad |= !isfinite(r0) || !isfinite(r1) || !isfinite(r2) || !isfinite(r3);
                        // f32 -> bf16 (round to nearest even; the product is finite or the launch is refused) -> the same values as fp16
                        const __nv_bfloat162 b01 = __floats2bfloat162_rn(r0, r1), b23 = __floats2bfloat162_rn(r2, r3);
                        const __half2 h01 = __float22half2_rn(__bfloat1622float2(b01)), h23 = __float22half2_rn(__bfloat1622float2(b23));
                        *reinterpret_cast<uint2 *>(p.mid + srow * p.M + m0) =
                            make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
                    }
                }
                if (bad) raise(p.status, YVEX_B200_STATUS_NUMERIC);
            } else {
                // store: out[(row0 + n)][mt*128 + row]. A thread holds 64 token columns of ONE weight row, so a
                // direct store is one instruction per column and 2 bytes per lane. Instead every aligned
                // group of four lanes transposes 4 x 4 blocks with shuffles: lane 4a+j ends up with weight
                // rows 4a..4a+3 of token column 4b+j and stores them as one 8-byte vector (a quarter of
                // the store instructions). Two rounds of independent shuffles, as above.
                const bool odd = lane & 1, hi = lane & 2;
                const int j4 = lane & 3;
                const uint64_t m0 = (uint64_t)mt * kTileM + 32 * quarter + (lane & ~3);
#pragma unroll
                for (int b0 = 0; b0 < kCols / 4; b0 += 4) {           // four blocks (eight shuffles) per round
#pragma unroll
                    for (int b = b0; b < b0 + 4; ++b) {
                        float *r = acc + 4 * b;
                        const float s0 = __shfl_xor_sync(0xffffffffu, odd ? r[0] : r[1], 1), s1 = __shfl_xor_sync(0xffffffffu, odd ? r[2] : r[3], 1);
                        if (odd) { r[0] = s0; r[2] = s1; } else { r[1] = s0; r[3] = s1; }
                    }
#pragma unroll
                    for (int b = b0; b < b0 + 4; ++b) {
                        float *r = acc + 4 * b;
                        const float s0 = __shfl_xor_sync(0xffffffffu, hi ? r[0] : r[2], 2), s1 = __shfl_xor_sync(0xffffffffu, hi ? r[1] : r[3], 2);
                        if (hi) { r[0] = s0; r[1] = s1; } else { r[2] = s0; r[3] = s1; }
                    }
                }
#pragma unroll
                for (int b = 0; b < kCols / 4; ++b) {
                    const int col = 4 * b + j4;
                    if (col < ncols_here) {
                        const uint64_t srow = (uint64_t)cb.row0 + kCols * colhalf + col;
                        uint16_t *dst;
                        if (p.out_addr) dst = reinterpret_cast<uint16_t *>(__ldg(p.out_addr + srow));
                        else dst = p.out_bf16 + (p.out_rows ? (uint64_t)__ldg(p.out_rows + srow) : srow) * p.M;
                        // streaming stores: the results are not read again by this kernel and must not push the
                        // activation tiles and weight rows that other CTAs are about to reuse out of L2
                        const uint2 v = make_uint2(bf16_bits(acc[4 * b]) | ((uint32_t)bf16_bits(acc[4 * b + 1]) << 16),
                                                   bf16_bits(acc[4 * b + 2]) | ((uint32_t)bf16_bits(acc[4 * b + 3]) << 16));
                        if (dst) __stcs(reinterpret_cast<uint2 *>(dst + m0), v);
                    }
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
