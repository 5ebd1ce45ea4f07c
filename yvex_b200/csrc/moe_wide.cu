// Wide-batch (prefill / expert-parallel shard) MoE execution.
//
// The unit of work is a PAIR LIST: pair p = (source row src[p], expert e[p], route weight w[p]),
// e[p] == experts meaning the shared expert. The pipeline is
//   expert-major stable counting sort (the reference's worklist order, src/graph/worklist.c:369-441)
//   -> gather source rows to expert-major fp16
//   -> grouped dequant GEMM gate & up (tcgen05) with SwiGLU * route weight -> bf16 in its epilogue
//   (-> sub-block sums of the intermediates for affine down qtypes)
//   -> grouped dequant GEMM down -> one bf16 row per pair.
// yvex_b200_moe_wide builds the list from its own router output (T*k routed pairs + T shared
// pairs) and finishes with the rank-ordered unpermute: routed rows summed in rank order in f32,
// + shared, -> bf16 (src/runtime/moe.c:619-632). yvex_b200_moe_expert_rows runs a caller-made
// list (an expert-parallel rank's received rows) and returns the per-pair rows in list order;
// yvex_b200_moe_combine is the unpermute on its own.
#include <cudaTypedefs.h>

#include <atomic>
#include <type_traits>

#include "moe_gemm.cuh"

namespace yb {

// ---- pair list of the single-device layer ----------------------------------------------------------
__global__ void wide_pairs_kernel(const int32_t *selected, const float *weights, uint64_t tokens, uint64_t topk, int experts,
                                  int *expert_of_pair, int *src_of_pair, float *weight_of_pair) {
    const uint64_t routed = tokens * topk, total = routed + tokens;
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < total; p += (uint64_t)gridDim.x * blockDim.x) {
        const bool r = p < routed;
        expert_of_pair[p] = r ? selected[p] : experts;
        src_of_pair[p] = (int)(r ? p / topk : p - routed);
        weight_of_pair[p] = r ? weights[p] : 1.0f;
    }
}

// Pair list handed in by the caller: pair p reads source row p; a negative id is the shared expert.
__global__ void wide_list_kernel(const int32_t *ids, const float *weights, uint64_t pairs, int experts, int *expert_of_pair,
                                 int *src_of_pair, float *weight_of_pair) {
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < pairs; p += (uint64_t)gridDim.x * blockDim.x) {
        expert_of_pair[p] = ids[p] < 0 ? experts : ids[p];      // ids >= experts are refused by the count kernel
        src_of_pair[p] = (int)p;
        weight_of_pair[p] = weights[p];
    }
}

// ---- permute ---------------------------------------------------------------------------------------
__global__ void wide_count_kernel(const int *expert_of_pair, uint64_t pairs, int bins, int *counts, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < pairs; i += (uint64_t)gridDim.x * blockDim.x) {
        const int e = expert_of_pair[i];
        if (e < 0 || e >= bins) raise(status, YVEX_B200_STATUS_ARGUMENT);
        else atomicAdd(&counts[e], 1);
    }
}

// One warp per list: exclusive scan of the group sizes and the column-block list in expert order
// (bin `experts` is the shared expert, published as expert -1). Block 0 builds the list of the
// gate/up GEMM (and the offsets), block 1 the list of the down GEMM, whose tiles may be narrower.
// Lanes take 32 consecutive bins at a time; shuffle scans give each bin its first row and block.
__global__ void wide_plan_kernel(const int *counts, int experts, uint64_t pairs, int *offsets, ColBlock *blocks_gu,
                                 ColBlock *blocks_down, int *num_blocks, int max_blocks, int tile_gu, int tile_down, int *status) {
    ColBlock *blocks = blockIdx.x ? blocks_down : blocks_gu;
    const int tile_n = blockIdx.x ? tile_down : tile_gu, lane = threadIdx.x;
    const int per_group = kGroupRows / tile_n;                              // groups of <= kGroupRows token rows
    num_blocks += blockIdx.x;
    int off = 0, nb = 0;                                                     // running totals, the same in every lane
    for (int base = 0; base <= experts; base += 32) {
        const int e = base + lane;
        const int count = e <= experts ? counts[e] : 0;
        const int nblocks = (count + tile_n - 1) / tile_n;
        int row_end = count, blk_end = nblocks;                              // inclusive scans over the 32 bins
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, row_end, d), b = __shfl_up_sync(0xffffffffu, blk_end, d);
            if (lane >= d) { row_end += r; blk_end += b; }
        }
        const int row0 = off + row_end - count, blk0 = nb + blk_end - nblocks;
        if (e <= experts) {
            if (blockIdx.x == 0) offsets[e] = row0;
            for (int b = 0; b < nblocks; ++b) {
                const int first = blk0 + b - b % per_group;
                const int in_group = min(per_group, nblocks - (b - b % per_group));
                if (blk0 + b < max_blocks)
                    blocks[blk0 + b] = ColBlock{row0 + b * tile_n, min(tile_n, count - b * tile_n), e < experts ? e : -1, first, in_group, 0};
            }
        }
        off += __shfl_sync(0xffffffffu, row_end, 31);
        nb += __shfl_sync(0xffffffffu, blk_end, 31);
    }
    if (lane) return;
    if (blockIdx.x == 0) offsets[experts + 1] = off;
    if ((uint64_t)off != pairs) raise(status, YVEX_B200_STATUS_ARGUMENT);
    if (nb > max_blocks) { raise(status, YVEX_B200_STATUS_ARGUMENT); nb = max_blocks; }
    *num_blocks = nb;
}

// One CTA per bin: stable compaction of the pairs routed to it (ascending pair index).
__global__ void wide_scatter_kernel(const int *expert_of_pair, uint64_t pairs, const int *offsets, int *perm, int *pos_of_pair) {
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __shared__ int warp_count[32];
    __shared__ int base;
    if (threadIdx.x == 0) base = offsets[e];
    __syncthreads();
    if (offsets[e + 1] == offsets[e]) return;          // empty bin (uniform across the CTA)
    for (uint64_t start = 0; start < pairs; start += blockDim.x) {
        const uint64_t i = start + threadIdx.x;
        const bool hit = i < pairs && expert_of_pair[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < nw; ++w) { if (w < warp) before += warp_count[w]; total += warp_count[w]; }
        if (hit) {
            const int pos = base + before + __popc(ballot & ((1u << lane) - 1u));
            perm[pos] = (int)i;
            pos_of_pair[i] = pos;
        }
        __syncthreads();
        if (threadIdx.x == 0) base += total;
        __syncthreads();
    }
}

// act_h[pos] = fp16 source row of the pair sorted to position pos. Source rows are `src_pitch` bytes apart
// (a multiple of 16; rows that travelled between ranks carry a trailer behind their hidden values).
// weight_sorted[pos] = its route weight (refused unless finite). group != 0 (affine gate/up qtypes: 32
// for Q4_K, 16 for Q2_K): also the hi/lo fp16 sums over `group` consecutive values of the row, the
// B' operand of the gate/up GEMM's min term.
__global__ void wide_gather_kernel(const __half *rows_h, const int *perm, const int *src_of_pair, const float *weight_of_pair,
                                   uint64_t pairs, uint64_t hidden, __half *act_h, float *weight_sorted, uint64_t src_pitch,
                                   int group, __half *act_sums, int *status) {
    const uint32_t chunks = (uint32_t)(hidden / 8);           // 16-byte chunks per row
    for (uint64_t row = blockIdx.x; row < pairs; row += gridDim.x) {          // a CTA copies whole rows
        const int pair = perm[row];
        if (weight_of_pair && threadIdx.x == 0) {               // (a plain row gather passes no weights)
            const float w = weight_of_pair[pair];
            if (!isfinite(w)) raise(status, YVEX_B200_STATUS_NUMERIC);
            weight_sorted[row] = w;
        }
        const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(rows_h) +
                                                           (uint64_t)src_of_pair[pair] * src_pitch);
        uint4 *dst = reinterpret_cast<uint4 *>(act_h) + row * chunks;
        for (uint32_t c = threadIdx.x; c < chunks; c += blockDim.x) {      // chunks is a multiple of 32: whole warps
            const uint4 v = __ldg(src + c);
            dst[c] = v;
            if (group) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
                const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&v.z)), f = __half22float2(*reinterpret_cast<const __half2 *>(&v.w));
                float sum = ((a.x + a.y) + (b.x + b.y)) + ((e.x + e.y) + (f.x + f.y));
                for (int o = group / 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);     // group / 8 lanes per sum
                if ((c & (uint32_t)(group / 8 - 1)) == 0) {
                    const __half hi = __float2half_rn(sum), lo = __float2half_rn(sum - __half2float(hi));
                    const uint32_t k = 8 * c, sb = k / 256, sub = (k % 256) / group, per = 256 / group;
                    __half *out = act_sums + (row * (hidden / 256) + sb) * 32;
                    out[sub] = hi;
                    out[per + sub] = lo;
                }
            }
        }
    }
}

// Trailer of a row that travels between expert-parallel ranks: behind its hidden fp16 values.
struct EpTrailer { int32_t local_expert; float weight; int32_t home_pair; int32_t home_rank; };

// Where the result of the pair sorted to position pos goes: its home rank's buffer, row home_pair.
__global__ void wide_dest_kernel(const uint8_t *payload, uint64_t pitch, uint64_t hidden, const int *perm, uint64_t pairs,
                                 const unsigned long long *home_bases, int home_world, uint64_t home_pairs,
                                 unsigned long long *dest, int *status) {
    for (uint64_t pos = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; pos < pairs; pos += (uint64_t)gridDim.x * blockDim.x) {
        const EpTrailer t = *reinterpret_cast<const EpTrailer *>(payload + (uint64_t)perm[pos] * pitch + hidden * 2);
        if (t.home_rank < 0 || t.home_rank >= home_world || t.home_pair < 0 || (uint64_t)t.home_pair >= home_pairs) {
            raise(status, YVEX_B200_STATUS_ARGUMENT);
            dest[pos] = 0ull;                                   // the row is dropped, never stored through a bad address
        } else {
            dest[pos] = home_bases[t.home_rank] + (unsigned long long)t.home_pair * hidden * 2ull;
        }
    }
}

// Pair list from the trailers of received rows: pair p reads source row p.
__global__ void wide_list_payload_kernel(const uint8_t *payload, uint64_t pitch, uint64_t hidden, uint64_t pairs, int experts,
                                         int *expert_of_pair, int *src_of_pair, float *weight_of_pair) {
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < pairs; p += (uint64_t)gridDim.x * blockDim.x) {
        const EpTrailer t = *reinterpret_cast<const EpTrailer *>(payload + p * pitch + hidden * 2);
        expert_of_pair[p] = t.local_expert < 0 ? experts : t.local_expert;
        src_of_pair[p] = (int)p;
        weight_of_pair[p] = t.weight;
    }
}

// hi/lo fp16 sums over `group` consecutive intermediates of a row (32 for Q4_K, 16 for Q2_K) for the
// down GEMM's min term: sums[(row, superblock)][sub] = hi, [256 / group + sub] = lo. A thread adds the
// eight values of a 16-byte chunk as a balanced tree and group / 8 neighbouring lanes finish the tree
// (inter is a multiple of 256, so rows start on warp boundaries of the flattened chunk index).
__global__ void __launch_bounds__(256)
wide_mid_sums_kernel(const __half *mid_h, uint64_t rows, uint64_t inter, int group, __half *sums) {
    const uint64_t chunks = rows * (inter / 8), stride = (uint64_t)gridDim.x * blockDim.x;
    const uint32_t per_row = (uint32_t)(inter / 8);
    constexpr int kUnroll = 4;
    for (uint64_t base = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; base < chunks; base += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            const uint64_t c = base + i * stride;
            v[i] = c < chunks ? __ldcs(reinterpret_cast<const uint4 *>(mid_h) + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            const uint64_t c = base + i * stride;                  // (chunks and stride are multiples of 32: whole warps)
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v[i].x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&v[i].y));
            const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&v[i].z)), f = __half22float2(*reinterpret_cast<const __half2 *>(&v[i].w));
            float sum = ((a.x + a.y) + (b.x + b.y)) + ((e.x + e.y) + (f.x + f.y));
            for (int o = 1; o < group / 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (c < chunks && (c & (uint64_t)(group / 8 - 1)) == 0) {
                const __half hi = __float2half_rn(sum), lo = __float2half_rn(sum - __half2float(hi));
                const uint64_t row = c / per_row;
                const uint32_t k = 8 * (uint32_t)(c - row * per_row), sb = k / 256, sub = (k % 256) / group, per = 256 / group;
                __half *dst = sums + (row * (inter / 256) + sb) * 32;
                dst[sub] = hi;
                dst[per + sub] = lo;
            }
        }
    }
}

// out[t] = bf16( sum_{rank} y[row(t, rank)] (rank order, f32) + y_shared[row(t)] ); `pos` maps a
// pair index to its row in y (nullptr = identity). Threads take 8 columns (one 16-byte load per
// source row); blockIdx.y strides the tokens.
__global__ void __launch_bounds__(128)
wide_combine_kernel(const uint16_t *y, const uint16_t *y_shared, const int *pos, const int *pos_shared,
                    uint64_t tokens, uint64_t topk, uint64_t hidden, float *out, float *routed_out = nullptr,
                    float *shared_out = nullptr) {
    const uint32_t chunks = (uint32_t)(hidden / 8), c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    for (uint64_t t = blockIdx.y; t < tokens; t += gridDim.y) {
        float routed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) routed[i] = 0.0f;
        for (uint64_t r = 0; r < topk; ++r) {
            const uint64_t row = pos ? (uint64_t)pos[t * topk + r] : t * topk + r;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(y + row * hidden) + c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                routed[2 * i] += __uint_as_float(w[i] << 16);
                routed[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
        const uint64_t srow = pos_shared ? (uint64_t)pos_shared[t] : t;
        const uint4 sv = __ldg(reinterpret_cast<const uint4 *>(y_shared + srow * hidden) + c);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        float4 o0, o1;
        o0.x = bf16_round(routed[0] + __uint_as_float(sw[0] << 16));
        o0.y = bf16_round(routed[1] + __uint_as_float(sw[0] & 0xffff0000u));
        o0.z = bf16_round(routed[2] + __uint_as_float(sw[1] << 16));
        o0.w = bf16_round(routed[3] + __uint_as_float(sw[1] & 0xffff0000u));
        o1.x = bf16_round(routed[4] + __uint_as_float(sw[2] << 16));
        o1.y = bf16_round(routed[5] + __uint_as_float(sw[2] & 0xffff0000u));
        o1.z = bf16_round(routed[6] + __uint_as_float(sw[3] << 16));
        o1.w = bf16_round(routed[7] + __uint_as_float(sw[3] & 0xffff0000u));
        float4 *dst = reinterpret_cast<float4 *>(out + t * hidden) + 2 * c;
        dst[0] = o0;
        dst[1] = o1;
        if (routed_out) {                       // the parts of the sum, unrounded routed total and the shared row
            float4 *r = reinterpret_cast<float4 *>(routed_out + t * hidden) + 2 * c;
            r[0] = make_float4(routed[0], routed[1], routed[2], routed[3]);
            r[1] = make_float4(routed[4], routed[5], routed[6], routed[7]);
        }
        if (shared_out) {
            float4 *sh = reinterpret_cast<float4 *>(shared_out + t * hidden) + 2 * c;
            sh[0] = make_float4(__uint_as_float(sw[0] << 16), __uint_as_float(sw[0] & 0xffff0000u), __uint_as_float(sw[1] << 16),
                                __uint_as_float(sw[1] & 0xffff0000u));
            sh[1] = make_float4(__uint_as_float(sw[2] << 16), __uint_as_float(sw[2] & 0xffff0000u), __uint_as_float(sw[3] << 16),
                                __uint_as_float(sw[3] & 0xffff0000u));
        }
    }
}

// ---- workspace -------------------------------------------------------------------------------------
struct PairWorkspace {
    int *counts, *offsets, *perm, *pos_of_pair, *num_blocks, *expert_of_pair, *src_of_pair;
    float *weight_of_pair, *weight_sorted;
    ColBlock *blocks, *blocks_down;         // column-block lists of the gate/up and the down GEMM (num_blocks[0], [1])
    __half *act_h, *mid_h, *sums, *act_sums;
    unsigned long long *dest;               // byte address of each sorted row's result (results returned to their home ranks)
    uint16_t *y;
    int max_blocks;
    void rebase(void *base) {
        auto fix = [&](auto *&ptr) { ptr = reinterpret_cast<std::remove_reference_t<decltype(ptr)>>(
                                         reinterpret_cast<uintptr_t>(base) + reinterpret_cast<uintptr_t>(ptr)); };
        fix(counts); fix(offsets); fix(perm); fix(pos_of_pair); fix(num_blocks); fix(expert_of_pair); fix(src_of_pair);
        fix(weight_of_pair); fix(weight_sorted); fix(blocks); fix(blocks_down); fix(act_h); fix(mid_h); fix(sums); fix(act_sums); fix(dest); fix(y);
    }
};

// Offsets of the pair pipeline's scratch for `pairs` pairs, starting at base_off.
static uint64_t pair_layout(const MoeGeom &g, uint64_t pairs, uint64_t base_off, PairWorkspace *ws) {
    uint64_t off = base_off;
    auto take = [&](uint64_t bytes) { uint64_t at = off; off = (off + bytes + 255) & ~255ull; return at; };
    PairWorkspace l{};
    l.max_blocks = (int)(pairs / kBoxN + g.experts + 2);
    l.counts = reinterpret_cast<int *>(take((g.experts + 2) * 4));
    l.offsets = reinterpret_cast<int *>(take((g.experts + 3) * 4));
    l.num_blocks = reinterpret_cast<int *>(take(8));
    l.perm = reinterpret_cast<int *>(take(pairs * 4));
    l.pos_of_pair = reinterpret_cast<int *>(take(pairs * 4));
    l.expert_of_pair = reinterpret_cast<int *>(take(pairs * 4));
    l.src_of_pair = reinterpret_cast<int *>(take(pairs * 4));
    l.weight_of_pair = reinterpret_cast<float *>(take(pairs * 4));
    l.weight_sorted = reinterpret_cast<float *>(take(pairs * 4));
    l.blocks = reinterpret_cast<ColBlock *>(take((uint64_t)l.max_blocks * sizeof(ColBlock)));
    l.blocks_down = reinterpret_cast<ColBlock *>(take((uint64_t)l.max_blocks * sizeof(ColBlock)));
    l.act_h = reinterpret_cast<__half *>(take(pairs * g.hidden * 2));
    l.mid_h = reinterpret_cast<__half *>(take(pairs * g.inter * 2));
    l.sums = reinterpret_cast<__half *>(take(pairs * (g.inter / 256) * 64));
    l.act_sums = reinterpret_cast<__half *>(take(pairs * (g.hidden / 256) * 64));
    l.dest = reinterpret_cast<unsigned long long *>(take(pairs * 8));
    l.y = reinterpret_cast<uint16_t *>(take(pairs * g.hidden * 2));
    if (ws) *ws = l;
    return off;
}

uint64_t moe_wide_workspace_bytes(const MoeGeom &g, uint64_t rows) {
    return pair_layout(g, rows * (g.topk + 1), moe_workspace_layout(g, rows, nullptr), nullptr);
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult q;
        void *p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
    return fn;
}

// Row-major fp16 [rows][width] -> boxes of [kBoxN rows][64 columns], 128-byte swizzle, zero fill.
// (pitch_bytes: distance between rows when they are not packed, a multiple of 16; 0 = packed)
static int make_act_map(CUtensorMap *map, const __half *base, uint64_t rows, uint64_t width, uint64_t pitch_bytes = 0) {
    auto fn = encode_fn();
    if (!fn) return ERR_BACKEND;
    cuuint64_t dims[2] = {width, rows}, strides[1] = {pitch_bytes ? pitch_bytes : width * 2};
    cuuint32_t box[2] = {kChunkK, kBoxN}, estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? OK : ERR_BACKEND;
}

// A weight pack of `rows` rows as u8 [rows / fuse][fuse * row_bytes], boxes of [128 / fuse][box_bytes].
// (box_rows: 128, or 64 for the fused gate/up kernel, which takes half of a tile's rows from each matrix)
static int make_weight_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t row_bytes, int fuse, uint32_t box_bytes,
                           int box_rows) {
    auto fn = encode_fn();
    if (!fn) return ERR_BACKEND;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return ERR_INVALID_ARG;        // weight packs must start on a 16-byte boundary
    cuuint64_t dims[2] = {fuse * row_bytes, rows / fuse}, strides[1] = {fuse * row_bytes};
    cuuint32_t box[2] = {box_bytes, (cuuint32_t)(box_rows / fuse)}, estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? OK : ERR_BACKEND;
}

// Rows fused into one tensor row so that its pitch is a multiple of 16 bytes (block sizes are even).
static int fuse_of(uint64_t row_bytes) {
    int fuse = 1;
    while ((fuse * row_bytes) % 16) fuse *= 2;
    return fuse;
}

// CTAs of the persistent grouped GEMM. One per SM by default; an expert-parallel caller that runs its
// exchange beside the GEMM leaves a few SMs to the communication kernels.
static std::atomic<int> g_gemm_ctas{kSmCount};

template <class Dec, bool kFused>
static int launch_gemm(const GemmMaps &map, const GemmParams &p, cudaStream_t s) {
    const size_t smem = GemmPlan<Dec>::kBytes;
    static SmemOptIn opt_in;
    if (opt_in.ensure(moe_grouped_gemm_kernel<Dec, kFused>, (int)smem) != OK) return ERR_BACKEND;
    moe_grouped_gemm_kernel<Dec, kFused><<<g_gemm_ctas.load(std::memory_order_relaxed), GemmPlan<Dec>::kThreads, smem, s>>>(map, p);
    return launch_status(1);
}

static uint32_t gemm_box_bytes(unsigned qtype) {
    return qtype == Q_IQ2_XXS ? GemmIq2::kBoxBytes : qtype == Q_Q4_K ? GemmQ4k::kBoxBytes : GemmQ2k::kBoxBytes;
}

// The weight maps of one GEMM: routed and shared packs of its one or two matrices.
static int make_weight_maps(GemmMaps *maps, unsigned qtype, const void *const routed[2], const void *const shared[2], int nmat,
                            uint64_t routed_rows, uint64_t shared_rows, const GemmParams &p) {
    for (int m = 0; m < 2; ++m) {
        const int src = m < nmat ? m : 0;              // unused slots repeat matrix 0 so every map is valid
        const int box_rows = nmat == 2 ? kTileM / 2 : kTileM;
        int rc = make_weight_map(&maps->w_routed[m], routed[src], routed_rows, p.row_bytes, p.fuse, gemm_box_bytes(qtype), box_rows);
        if (rc != OK) return rc;
        rc = make_weight_map(&maps->w_shared[m], shared[src] ? shared[src] : routed[src], shared[src] ? shared_rows : routed_rows,
                             p.row_bytes, p.fuse, gemm_box_bytes(qtype), box_rows);
        if (rc != OK) return rc;
    }
    return OK;
}

// fused: the gate/up form (two matrices, SwiGLU epilogue); otherwise the one-matrix bf16 form.
static int run_gemm(unsigned qtype, bool fused, const GemmMaps &map, const GemmParams &p, cudaStream_t s) {
    switch (qtype) {
    case Q_IQ2_XXS: return fused ? launch_gemm<GemmIq2, true>(map, p, s) : launch_gemm<GemmIq2, false>(map, p, s);
    case Q_Q4_K: return fused ? launch_gemm<GemmQ4k, true>(map, p, s) : launch_gemm<GemmQ4k, false>(map, p, s);
    case Q_Q2_K: return fused ? launch_gemm<GemmQ2k, true>(map, p, s) : launch_gemm<GemmQ2k, false>(map, p, s);
    default: return ERR_UNSUPPORTED;
    }
}

static bool gemm_qtype(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q2_K; }
// Token columns per GEMM tile: 256 unless the qtype's min term needs the second accumulator.
static int gemm_tile_n(unsigned q) { return q == Q_IQ2_XXS ? GemmPlan<GemmIq2>::kTileN : q == Q_Q4_K ? GemmPlan<GemmQ4k>::kTileN : GemmPlan<GemmQ2k>::kTileN; }

bool moe_wide_gemm_eligible(const MoeGeom &g, const MoeWeights &w) {
    const uintptr_t ptrs = (uintptr_t)w.gate | (uintptr_t)w.up | (uintptr_t)w.down | (uintptr_t)w.shared_gate |
                           (uintptr_t)w.shared_up | (uintptr_t)w.shared_down;
    return g.gate_qtype == g.up_qtype && gemm_qtype(g.gate_qtype) && gemm_qtype(g.down_qtype) &&
           g.inter == g.shared_inter && g.hidden % 256 == 0 && g.inter % 256 == 0 && g.inter % kTileM == 0 &&
           g.hidden % kTileM == 0 && (ptrs & 15u) == 0;
}

// Runs the pair list already stored in pw.{expert,src,weight}_of_pair; leaves one bf16 row per
// pair in pw.y at row pw.pos_of_pair[pair] or, when y_list is given, in y_list at row `pair` (the
// down GEMM's epilogue then stores through the permutation, so no separate unsort pass is needed).
// rows_h: the fp16 source rows the list indexes.
static int run_sorted_gemms(const MoeGeom &g, const MoeWeights &w, const PairWorkspace &pw, const __half *act, uint64_t act_pitch,
                            uint64_t pairs, int *status, cudaStream_t s, uint16_t *y, const int *out_rows,
                            const unsigned long long *out_addr);

// home_bases (optional, device array of `home_world` addresses; rows_h then are payload rows with trailers):
// the row of a pair is stored at home_bases[trailer.home_rank] + trailer.home_pair * hidden * 2 instead.
static int run_pair_list(const MoeGeom &g, const MoeWeights &w, const PairWorkspace &pw, const __half *rows_h, uint64_t pairs,
                         int *status, cudaStream_t s, uint16_t *y_list = nullptr, uint64_t src_pitch = 0,
                         const unsigned long long *home_bases = nullptr, int home_world = 0, uint64_t home_pairs = 0) {
    if (!src_pitch) src_pitch = g.hidden * 2;
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
    const int bins = (int)g.experts + 1;
    cudaMemsetAsync(pw.counts, 0, (g.experts + 2) * 4, s);
    wide_count_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(pw.expert_of_pair, pairs, bins, pw.counts, status);
    wide_plan_kernel<<<2, 32, 0, s>>>(pw.counts, (int)g.experts, pairs, pw.offsets, pw.blocks, pw.blocks_down, pw.num_blocks,
                                      pw.max_blocks, gemm_tile_n(g.gate_qtype), gemm_tile_n(g.down_qtype), status);
    wide_scatter_kernel<<<(unsigned)bins, 512, 0, s>>>(pw.expert_of_pair, pairs, pw.offsets, pw.perm, pw.pos_of_pair);
    const auto sum_group = [](unsigned q) { return q == Q_Q4_K ? 32 : q == Q_Q2_K ? 16 : 0; };
    wide_gather_kernel<<<grid_for(pairs, 1, 16), 128, 0, s>>>(rows_h, pw.perm, pw.src_of_pair, pw.weight_of_pair, pairs, g.hidden,
                                                              pw.act_h, pw.weight_sorted, src_pitch, sum_group(g.gate_qtype),
                                                              pw.act_sums, status);
    if (home_bases)
        wide_dest_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(reinterpret_cast<const uint8_t *>(rows_h), src_pitch, g.hidden, pw.perm,
                                                               pairs, home_bases, home_world, home_pairs, pw.dest, status);
    int rc = launch_status(4);
    if (rc != OK) return rc;
    mark_phase(2, s);
    return run_sorted_gemms(g, w, pw, pw.act_h, 0, pairs, status, s, y_list ? y_list : pw.y, y_list ? pw.perm : nullptr,
                            home_bases ? pw.dest : nullptr);
}

// The two grouped GEMMs over rows that already stand in expert-major order (`act`, `act_pitch` bytes apart,
// 0 = packed), with pw.blocks / pw.blocks_down / pw.num_blocks / pw.weight_sorted (and pw.act_sums for an
// affine gate/up qtype) prepared. Results: bf16 rows into y (through out_rows when given), or at out_addr.
static int run_sorted_gemms(const MoeGeom &g, const MoeWeights &w, const PairWorkspace &pw, const __half *act, uint64_t act_pitch,
                            uint64_t pairs, int *status, cudaStream_t s, uint16_t *y, const int *out_rows,
                            const unsigned long long *out_addr) {
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
    const auto sum_group = [](unsigned q) { return q == Q_Q4_K ? 32 : q == Q_Q2_K ? 16 : 0; };
    int rc;
    GemmMaps gu_maps, dn_maps;
    if (make_act_map(&gu_maps.act, act, pairs, g.hidden, act_pitch) != OK || make_act_map(&dn_maps.act, pw.mid_h, pairs, g.inter) != OK)
        return ERR_BACKEND;
    GemmParams gu{};
    gu.row_bytes = (uint32_t)(g.hidden / gg.elems * gg.bytes);
    gu.fuse = fuse_of(gu.row_bytes);
    gu.M = (int)g.inter; gu.K = (int)g.hidden; gu.nmat = 1;              // one fused pass over both matrices
    {
        const void *routed[2] = {w.gate, w.up}, *shared[2] = {w.shared_gate, w.shared_up};
        rc = make_weight_maps(&gu_maps, g.gate_qtype, routed, shared, 2, (uint64_t)g.experts * g.inter, g.inter, gu);
        if (rc != OK) return rc;
    }
    gu.colblocks = pw.blocks; gu.num_colblocks = pw.num_blocks;
    gu.mid = pw.mid_h; gu.col_weight = pw.weight_sorted; gu.limit = (float)g.limit; gu.out_bf16 = nullptr; gu.sums = pw.act_sums;
    gu.status = status;
    rc = run_gemm(g.gate_qtype, true, gu_maps, gu, s);
    if (rc != OK) return rc;
    mark_phase(3, s);

    const int group = sum_group(g.down_qtype);
    if (group)
        wide_mid_sums_kernel<<<grid_for(pairs * (g.inter / 8), 256, 8), 256, 0, s>>>(pw.mid_h, pairs, g.inter, group, pw.sums);
    mark_phase(6, s);                                   // sums done (an extra probe point, outside the 0..5 sequence)
    GemmParams dn{};
    dn.row_bytes = (uint32_t)(g.inter / dg.elems * dg.bytes);
    dn.fuse = fuse_of(dn.row_bytes);
    dn.M = (int)g.hidden; dn.K = (int)g.inter; dn.nmat = 1;
    {
        const void *routed[2] = {w.down, nullptr}, *shared[2] = {w.shared_down, nullptr};
        rc = make_weight_maps(&dn_maps, g.down_qtype, routed, shared, 1, (uint64_t)g.experts * g.hidden, g.hidden, dn);
        if (rc != OK) return rc;
    }
    dn.colblocks = pw.blocks_down; dn.num_colblocks = pw.num_blocks + 1;
    dn.out_bf16 = y; dn.out_rows = out_rows; dn.sums = pw.sums; dn.status = status;
    dn.out_addr = out_addr;
    rc = run_gemm(g.down_qtype, false, dn_maps, dn, s);
    if (rc != OK) return rc;
    mark_phase(4, s);
    return launch_status(1);
}

}  // namespace yb

using namespace yb;

extern "C" int yvex_b200_moe_wide(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                  const float *x, const float *logits, const uint32_t *token_ids,
                                  uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                                  void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    return yvex_b200_moe_wide_parts(geom, w, x, logits, token_ids, rows, out, nullptr, nullptr, selected_out, weights_out, workspace,
                                    workspace_bytes, status, stream);
}

extern "C" int yvex_b200_moe_wide_parts(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                        const float *x, const float *logits, const uint32_t *token_ids,
                                        uint64_t rows, float *out, float *routed_out, float *shared_out,
                                        int32_t *selected_out, float *weights_out,
                                        void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!x || !out || !status || !rows) return ERR_INVALID_ARG;
    if (rows * (geom->topk + 1) > 0x7fffff00ull / 2) return ERR_BOUNDS;       // 32-bit row indices
    MoeGeom g = *geom;
    MoeWorkspace ws;
    const bool gemm = moe_wide_gemm_eligible(g, *w);
    const uint64_t base = moe_workspace_layout(g, rows, &ws);
    const uint64_t need = gemm ? moe_wide_workspace_bytes(g, rows) : base;
    if (!workspace || workspace_bytes < need) return ERR_NOMEM;
    ws.rebase(workspace);
    ws.routed_out = routed_out;
    ws.shared_out = shared_out;
    cudaStream_t s = as_stream(stream);
    mark_phase(0, s);
    rc = moe_ingress_and_route(g, *w, ws, x, logits, token_ids, rows, status, s);
    if (rc != OK) return rc;
    mark_phase(1, s);
    if (gemm) {
        PairWorkspace pw;
        const uint64_t pairs = rows * (g.topk + 1), routed = rows * g.topk;
        pair_layout(g, pairs, base, &pw);
        pw.rebase(workspace);
        wide_pairs_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(ws.selected, ws.weights, rows, g.topk, (int)g.experts,
                                                                pw.expert_of_pair, pw.src_of_pair, pw.weight_of_pair);
        rc = run_pair_list(g, *w, pw, ws.xr_h, pairs, status, s);
        if (rc != OK) return rc;
        wide_combine_kernel<<<dim3((unsigned)((g.hidden / 8 + 127) / 128), (unsigned)grid_for(rows, 1, 16)), 128, 0, s>>>(
            pw.y, pw.y, pw.pos_of_pair, pw.pos_of_pair + routed, rows, g.topk, g.hidden, out, routed_out, shared_out);
        mark_phase(5, s);
        rc = launch_status(2);
    } else {
        rc = moe_experts_rows(g, *w, ws, rows, out, status, s);
    }
    if (rc != OK) return rc;
    if (selected_out) cudaMemcpyAsync(selected_out, ws.selected, rows * g.topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, s);
    if (weights_out) cudaMemcpyAsync(weights_out, ws.weights, rows * g.topk * sizeof(float), cudaMemcpyDeviceToDevice, s);
    return launch_status(0);
}

extern "C" int yvex_b200_moe_wide_uses_gemm(const yvex_b200_moe_geometry *g, const yvex_b200_moe_weights *w) {
    return g && w && moe_check_geometry(g, w) == OK && moe_wide_gemm_eligible(*g, *w) ? 1 : 0;
}

extern "C" uint64_t yvex_b200_moe_wide_tile_columns(unsigned int qtype) { return gemm_qtype(qtype) ? (uint64_t)gemm_tile_n(qtype) : 0; }

extern "C" uint64_t yvex_b200_moe_wide_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t rows) {
    return g ? moe_wide_workspace_bytes(*g, rows) : 0;
}

extern "C" uint64_t yvex_b200_moe_expert_rows_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t pairs) {
    return g ? pair_layout(*g, pairs, 0, nullptr) : 0;
}

extern "C" int yvex_b200_moe_expert_rows(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                         const void *rows_f16, const int32_t *expert_ids, const float *route_weights,
                                         uint64_t pairs, void *y_bf16, void *workspace, uint64_t workspace_bytes,
                                         int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!pairs) return OK;
    if (!rows_f16 || !expert_ids || !route_weights || !y_bf16 || !status) return ERR_INVALID_ARG;
    if (pairs > 0x7fffff00ull / 2 || (reinterpret_cast<uintptr_t>(rows_f16) & 15u) || (reinterpret_cast<uintptr_t>(y_bf16) & 15u))
        return ERR_BOUNDS;
    MoeGeom g = *geom;
    if (!moe_wide_gemm_eligible(g, *w)) return ERR_UNSUPPORTED;
    PairWorkspace pw;
    if (!workspace || workspace_bytes < pair_layout(g, pairs, 0, &pw)) return ERR_NOMEM;
    pw.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    // the caller's list: source row of pair p is row p; a negative id names the shared expert
    mark_phase(0, s);
    wide_list_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(expert_ids, route_weights, pairs, (int)g.experts,
                                                           pw.expert_of_pair, pw.src_of_pair, pw.weight_of_pair);
    mark_phase(1, s);
    rc = run_pair_list(g, *w, pw, static_cast<const __half *>(rows_f16), pairs, status, s, static_cast<uint16_t *>(y_bf16));
    if (rc != OK) return rc;
    mark_phase(5, s);
    return launch_status(1);
}

// ---- expert worklist as a result of its own (src/graph/worklist.c:369-441) ------------------------------
// Compact bucket list and the pointer-free observation from the per-expert counts and first rows
// (one thread: at most 256 experts). Same arithmetic as yvex_expert_worklist_build and the summary
// of its device twin (src/backend/cuda/moe_kernels.cu:294-397).
__global__ void worklist_observe_kernel(const int *counts, const int *offsets, int experts, uint64_t pairs, uint64_t rows,
                                        uint64_t tc_min, uint64_t width, unsigned provenance, yvex_b200_worklist_observation *obs,
                                        int32_t *expert_ids, int32_t *bucket_offsets, int32_t *bucket_populations, int *status) {
    if (threadIdx.x || blockIdx.x) return;
    yvex_b200_worklist_observation o;
    memset(&o, 0, sizeof(o));
    o.schema_version = 1u;
    o.worklist_count = 1ull;
    o.pair_count = pairs;
    o.width_histogram[rows < YVEX_B200_WORKLIST_HISTOGRAM_CAP ? rows : YVEX_B200_WORKLIST_HISTOGRAM_CAP - 1u] = 1ull;
    o.provenance_counts[provenance] = 1ull;
    uint64_t emitted = 0, unique = 0;
    for (int e = 0; e < experts; ++e) {
        const uint64_t n = (uint64_t)counts[e];
        if (!n) continue;
        if (expert_ids) expert_ids[unique] = e;
        if (bucket_offsets) bucket_offsets[unique] = offsets[e];
        if (bucket_populations) bucket_populations[unique] = (int32_t)n;
        if (n > o.maximum_bucket_population) o.maximum_bucket_population = n;
        o.population_histogram[n < YVEX_B200_WORKLIST_HISTOGRAM_CAP ? n : YVEX_B200_WORKLIST_HISTOGRAM_CAP - 1u]++;
        if (tc_min && n >= tc_min) {
            o.tensor_core_eligible_pairs += n;
            if (n % width) o.tail_rows += width - n % width;
        } else {
            o.narrow_pairs += n;
        }
        emitted += n;
        ++unique;
    }
    if (bucket_offsets) bucket_offsets[unique] = (int32_t)emitted;
    o.bucket_count = unique;
    if (emitted != pairs) raise(status, YVEX_B200_STATUS_ARGUMENT);
    if (obs) *obs = o;
}

__global__ void worklist_rows_kernel(const int *order, uint64_t pairs, uint64_t topk, int32_t *source_rows, int32_t *destination_rows) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < pairs; i += (uint64_t)gridDim.x * blockDim.x) {
        const int p = order[i];
        if (source_rows) source_rows[i] = (int32_t)(p / topk);
        if (destination_rows) destination_rows[i] = p;
    }
}

// The whole worklist of a narrow batch in one CTA (pairs <= kSmallWorklistPairs): shared-memory
// counts, a serial scan over the experts, and the reference's stable emission (thread e walks
// the pairs in order and emits those of expert e).
constexpr int kSmallWorklistPairs = 2048;
__global__ void __launch_bounds__(256)
worklist_small_kernel(const int32_t *selected, uint64_t rows, uint64_t topk, int experts, uint64_t tc_min, uint64_t width,
                      unsigned provenance, int32_t *order, int32_t *source_rows, int32_t *destination_rows, int32_t *expert_ids,
                      int32_t *bucket_offsets, int32_t *bucket_populations, yvex_b200_worklist_observation *obs, int *status) {
    __shared__ int counts[257], offsets[257], bad;
    const int pairs = (int)(rows * topk);
    for (int e = threadIdx.x; e <= 256; e += blockDim.x) counts[e] = 0;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = selected[p];
        if (e < 0 || e >= experts) bad = 1; else atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (bad) { if (threadIdx.x == 0) raise(status, YVEX_B200_STATUS_ARGUMENT); return; }
    if (threadIdx.x == 0) {
        int off = 0;
        for (int e = 0; e < experts; ++e) { offsets[e] = off; off += counts[e]; }
        offsets[experts] = off;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        yvex_b200_worklist_observation o;
        memset(&o, 0, sizeof(o));
        o.schema_version = 1u; o.worklist_count = 1ull; o.pair_count = (uint64_t)pairs;
        o.width_histogram[rows < YVEX_B200_WORKLIST_HISTOGRAM_CAP ? rows : YVEX_B200_WORKLIST_HISTOGRAM_CAP - 1u] = 1ull;
        o.provenance_counts[provenance] = 1ull;
        uint64_t unique = 0;
        for (int e = 0; e < experts; ++e) {
            const uint64_t n = (uint64_t)counts[e];
            if (!n) continue;
            if (expert_ids) expert_ids[unique] = e;
            if (bucket_offsets) bucket_offsets[unique] = offsets[e];
            if (bucket_populations) bucket_populations[unique] = (int32_t)n;
            if (n > o.maximum_bucket_population) o.maximum_bucket_population = n;
            o.population_histogram[n < YVEX_B200_WORKLIST_HISTOGRAM_CAP ? n : YVEX_B200_WORKLIST_HISTOGRAM_CAP - 1u]++;
            if (tc_min && n >= tc_min) {
                o.tensor_core_eligible_pairs += n;
                if (n % width) o.tail_rows += width - n % width;
            } else {
                o.narrow_pairs += n;
            }
            ++unique;
        }
        if (bucket_offsets) bucket_offsets[unique] = offsets[experts];
        o.bucket_count = unique;
        if (obs) *obs = o;
    }
    if (!order && !source_rows && !destination_rows) return;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int cursor = offsets[e];
        if (!counts[e]) continue;
        for (int p = 0; p < pairs; ++p)
            if (selected[p] == e) {
                if (order) order[cursor] = p;
                if (source_rows) source_rows[cursor] = (int32_t)(p / (int)topk);
                if (destination_rows) destination_rows[cursor] = p;
                ++cursor;
            }
    }
}

// ---- expert-parallel dispatch plan -----------------------------------------------------------------
// dest rank and source token of every (token, rank) pair, and the pairs per destination
__global__ void ep_dest_kernel(const int32_t *selected, uint64_t pairs, uint64_t topk, int per_rank, int world, int *dest,
                               int *src_token, int *counts, int *status) {
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < pairs; p += (uint64_t)gridDim.x * blockDim.x) {
        const int e = selected[p];
        int d = e >= 0 ? e / per_rank : world;
        src_token[p] = (int)(p / topk);
        // an id outside the ranks' experts raises the status; the pair still gets a bin, so that the
        // counts, the send order and everything indexed through them stay consistent and in range
        if (d >= world) { raise(status, YVEX_B200_STATUS_ARGUMENT); d = 0; }
        dest[p] = d;
        atomicAdd(&counts[d], 1);
    }
}

__global__ void ep_offsets_kernel(const int *counts, int world, int *offsets, long long *counts_out) {
    if (threadIdx.x || blockIdx.x) return;
    int off = 0;
    for (int r = 0; r < world; ++r) { offsets[r] = off; off += counts[r]; counts_out[r] = counts[r]; }
    offsets[world] = off;
}

// metadata of the pairs in send order: (expert id local to its rank, route weight bits)
__global__ void ep_meta_kernel(const int32_t *selected, const float *weights, const int *order, uint64_t pairs, int per_rank,
                               int32_t *meta) {
    for (uint64_t pos = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; pos < pairs; pos += (uint64_t)gridDim.x * blockDim.x) {
        const int p = order[pos];
        meta[2 * pos] = selected[p] % per_rank;
        meta[2 * pos + 1] = __float_as_int(weights[p]);
    }
}

extern "C" uint64_t yvex_b200_ep_dispatch_workspace_bytes(uint64_t pairs, uint64_t world) {
    // bin of pair, source token, send order; counts and offsets per bin; the pushed dispatch's write offsets
    return (3 * pairs + 2 * world + 8) * sizeof(int) + 256 + 8 * world + 64;
}

extern "C" int yvex_b200_ep_dispatch(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens,
                                     uint64_t topk, uint64_t hidden, uint64_t experts_per_rank, uint64_t world,
                                     void *send_rows_f16, int32_t *meta, int32_t *inverse, long long *send_counts,
                                     void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    if (!selected || !weights || !rows_f16 || !send_rows_f16 || !meta || !inverse || !send_counts || !status || !workspace)
        return ERR_INVALID_ARG;
    if (!tokens || !topk || !experts_per_rank || !world || world > 1024 || hidden % 8) return ERR_INVALID_ARG;
    const uint64_t pairs = tokens * topk;
    if (pairs > 0x7fffff00ull || ((reinterpret_cast<uintptr_t>(rows_f16) | reinterpret_cast<uintptr_t>(send_rows_f16)) & 15u))
        return ERR_BOUNDS;
    if (workspace_bytes < yvex_b200_ep_dispatch_workspace_bytes(pairs, world)) return ERR_NOMEM;
    int *dest = static_cast<int *>(workspace), *src = dest + pairs, *order = src + pairs;
    int *counts = order + pairs, *offsets = counts + world + 1;
    cudaStream_t s = as_stream(stream);
    cudaMemsetAsync(counts, 0, (world + 1) * sizeof(int), s);
    ep_dest_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(selected, pairs, topk, (int)experts_per_rank, (int)world, dest, src, counts,
                                                          status);
    ep_offsets_kernel<<<1, 32, 0, s>>>(counts, (int)world, offsets, send_counts);
    wide_scatter_kernel<<<(unsigned)world, 512, 0, s>>>(dest, pairs, offsets, order, inverse);
    ep_meta_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(selected, weights, order, pairs, (int)experts_per_rank, meta);
    wide_gather_kernel<<<grid_for(pairs, 1, 16), 128, 0, s>>>(static_cast<const __half *>(rows_f16), order, src, nullptr, pairs, hidden,
                                                              static_cast<__half *>(send_rows_f16), nullptr, hidden * 2, 0, nullptr,
                                                              status);
    return launch_status(5);
}

// Segmented dispatch: pairs grouped by (segment of the destination's local experts, destination rank), each
// row sent with its trailer. bin = segment * world + rank, so one segment's rows for all ranks are contiguous.
__global__ void ep_bin_kernel(const int32_t *selected, uint64_t pairs, uint64_t topk, int per_rank, int world, int segments, int *bin_of,
                              int *src_token, int *counts, int *status) {
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; p < pairs; p += (uint64_t)gridDim.x * blockDim.x) {
        const int e = selected[p];
        int d = e >= 0 ? e / per_rank : world, local = e >= 0 ? e % per_rank : 0;
        src_token[p] = (int)(p / topk);
        if (d >= world) { raise(status, YVEX_B200_STATUS_ARGUMENT); d = 0; local = 0; }      // keeps counts and order consistent
        const int bin = (int)((int64_t)local * segments / per_rank) * world + d;
        bin_of[p] = bin;
        atomicAdd(&counts[bin], 1);
    }
}

__global__ void ep_payload_kernel(const __half *rows_h, const int32_t *selected, const float *weights, const int *order,
                                  const int *src_token, uint64_t pairs, uint64_t hidden, int per_rank, int home_rank, uint8_t *payload,
                                  uint64_t pitch) {
    const uint32_t chunks = (uint32_t)(hidden / 8);
    for (uint64_t pos = blockIdx.x; pos < pairs; pos += gridDim.x) {
        const int p = order[pos];
        const uint4 *src = reinterpret_cast<const uint4 *>(rows_h) + (uint64_t)src_token[p] * chunks;
        uint4 *dst = reinterpret_cast<uint4 *>(payload + pos * pitch);
        for (uint32_t c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = __ldg(src + c);
        if (threadIdx.x == 0) {
            const int e = selected[p];
            const EpTrailer t{e >= 0 ? e % per_rank : 0, weights[p], p, home_rank};
            *reinterpret_cast<EpTrailer *>(payload + pos * pitch + hidden * 2) = t;
        }
    }
}

extern "C" uint64_t yvex_b200_ep_payload_pitch(uint64_t hidden) { return hidden * 2 + sizeof(EpTrailer); }

// ---- dispatch by peer stores ----------------------------------------------------------------------------
// Every rank knows how many rows every rank sends into every bin (counts_all[src][bin], all-gathered).
// A bin's rows land in the destination rank's receive buffer grouped by source rank, ascending: this
// rank writes behind the rows of the ranks below it.
// expert_major (bins = local expert * world + destination, one receive buffer per destination): the bins of
// one destination follow each other in its buffer in local-expert order, so that the rows arrive already
// sorted the way the grouped GEMM walks them.
__global__ void ep_push_offsets_kernel(const long long *counts_all, int bins, int world, int rank, int expert_major,
                                       long long *row_base) {
    for (int b = threadIdx.x; b < bins; b += blockDim.x) {
        long long off = 0;
        for (int r = 0; r < rank; ++r) off += counts_all[(size_t)r * bins + b];
        if (expert_major)
            for (int b2 = b % world; b2 < b; b2 += world)
                for (int r = 0; r < world; ++r) off += counts_all[(size_t)r * bins + b2];
        row_base[b] = off;
    }
}

// Receiver of an expert-major push: rows of local expert l = what every rank sent into bin l * world + rank.
__global__ void ep_sorted_counts_kernel(const long long *counts_all, int world, int rank, int per_rank, uint64_t pairs, int *counts,
                                        int *status) {
    __shared__ long long total;
    if (threadIdx.x == 0) total = 0;
    __syncthreads();
    const int bins = per_rank * world;
    for (int l = threadIdx.x; l <= per_rank; l += blockDim.x) {
        long long n = 0;
        if (l < per_rank)
            for (int r = 0; r < world; ++r) n += counts_all[(size_t)r * bins + (size_t)l * world + rank];
        counts[l] = (int)n;                                  // bin per_rank is the shared expert: none here
        atomicAdd(reinterpret_cast<unsigned long long *>(&total), (unsigned long long)n);
    }
    __syncthreads();
    if (threadIdx.x == 0 && (uint64_t)total != pairs) raise(status, YVEX_B200_STATUS_ARGUMENT);
}

// Sorted rows' route weights and result addresses from their trailers; a trailer that names another expert
// than the group its row stands in, a rank or a pair out of range sets status 2 and its row is dropped.
__global__ void wide_trailer_kernel(const uint8_t *payload, uint64_t pitch, uint64_t hidden, uint64_t pairs, const int *offsets,
                                    int experts, const unsigned long long *home_bases, int home_world, uint64_t home_pairs,
                                    float *weight_sorted, unsigned long long *dest, int *status) {
    for (uint64_t pos = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; pos < pairs; pos += (uint64_t)gridDim.x * blockDim.x) {
        const EpTrailer t = *reinterpret_cast<const EpTrailer *>(payload + pos * pitch + hidden * 2);
        int lo = 0, hi = experts;                            // group of pos: offsets[lo] <= pos < offsets[lo + 1]
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if ((uint64_t)offsets[mid] <= pos) lo = mid; else hi = mid; }
        const bool ok = t.local_expert == lo && t.home_rank >= 0 && t.home_rank < home_world && t.home_pair >= 0 &&
                        (uint64_t)t.home_pair < home_pairs && isfinite(t.weight);
        if (!ok) raise(status, YVEX_B200_STATUS_ARGUMENT);
        weight_sorted[pos] = ok ? t.weight : 0.0f;
        dest[pos] = ok ? home_bases[t.home_rank] + (unsigned long long)t.home_pair * hidden * 2ull : 0ull;
    }
}

// The payload row of send position pos goes straight to recv_bases[bin] + (row_base[bin] + its index in the bin) * pitch,
// an address in the destination rank's memory (plain 16-byte stores; the own rank's bins are local stores).
__global__ void ep_push_kernel(const __half *rows_h, const int32_t *selected, const float *weights, const int *order, const int *bin_of,
                               const int *src_token, const int *bin_start, const long long *row_base,
                               const unsigned long long *recv_bases, uint64_t capacity_rows, uint64_t pairs, uint64_t hidden,
                               int per_rank, int home_rank, uint64_t pitch, int *status) {
    const uint32_t chunks = (uint32_t)(hidden / 8);
    for (uint64_t pos = blockIdx.x; pos < pairs; pos += gridDim.x) {
        const int p = order[pos], b = bin_of[p];
        const uint64_t at = (uint64_t)row_base[b] + (pos - (uint64_t)bin_start[b]);
        if (at >= capacity_rows) {                       // never a store past the receiver's buffer
            if (threadIdx.x == 0) raise(status, YVEX_B200_STATUS_ARGUMENT);
            continue;
        }
        uint8_t *row = reinterpret_cast<uint8_t *>(recv_bases[b]) + at * pitch;
        const uint4 *src = reinterpret_cast<const uint4 *>(rows_h) + (uint64_t)src_token[p] * chunks;
        uint4 *dst = reinterpret_cast<uint4 *>(row);
        for (uint32_t c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = __ldg(src + c);
        if (threadIdx.x == 0) {
            const int e = selected[p];
            const EpTrailer t{e >= 0 ? e % per_rank : 0, weights[p], p, home_rank};
            *reinterpret_cast<EpTrailer *>(row + hidden * 2) = t;
        }
    }
}

extern "C" int yvex_b200_ep_dispatch_payload(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens,
                                             uint64_t topk, uint64_t hidden, uint64_t experts_per_rank, uint64_t world,
                                             uint64_t rank, uint64_t segments, void *payload, int32_t *inverse, long long *send_counts,
                                             void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    if (!selected || !weights || !rows_f16 || !payload || !inverse || !send_counts || !status || !workspace) return ERR_INVALID_ARG;
    if (!tokens || !topk || !experts_per_rank || !world || rank >= world || !segments || world * segments > 1024 ||
        segments > experts_per_rank || hidden % 8)
        return ERR_INVALID_ARG;
    const uint64_t pairs = tokens * topk, bins = world * segments;
    if (pairs > 0x7fffff00ull || ((reinterpret_cast<uintptr_t>(rows_f16) | reinterpret_cast<uintptr_t>(payload)) & 15u)) return ERR_BOUNDS;
    if (workspace_bytes < yvex_b200_ep_dispatch_workspace_bytes(pairs, bins)) return ERR_NOMEM;
    int *bin_of = static_cast<int *>(workspace), *src = bin_of + pairs, *order = src + pairs;
    int *counts = order + pairs, *offsets = counts + bins + 1;
    cudaStream_t s = as_stream(stream);
    cudaMemsetAsync(counts, 0, (bins + 1) * sizeof(int), s);
    ep_bin_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(selected, pairs, topk, (int)experts_per_rank, (int)world, (int)segments, bin_of,
                                                         src, counts, status);
    ep_offsets_kernel<<<1, 32, 0, s>>>(counts, (int)bins, offsets, send_counts);
    wide_scatter_kernel<<<(unsigned)bins, 512, 0, s>>>(bin_of, pairs, offsets, order, inverse);
    ep_payload_kernel<<<grid_for(pairs, 1, 16), 128, 0, s>>>(static_cast<const __half *>(rows_f16), selected, weights, order, src, pairs,
                                                             hidden, (int)experts_per_rank, (int)rank, static_cast<uint8_t *>(payload),
                                                             yvex_b200_ep_payload_pitch(hidden));
    return launch_status(4);
}

extern "C" int yvex_b200_ep_dispatch_plan(const int32_t *selected, uint64_t tokens, uint64_t topk, uint64_t experts_per_rank,
                                          uint64_t world, uint64_t segments, int32_t *inverse, long long *send_counts, void *workspace,
                                          uint64_t workspace_bytes, int *status, void *stream) {
    if (!selected || !inverse || !send_counts || !status || !workspace) return ERR_INVALID_ARG;
    if (!tokens || !topk || !experts_per_rank || !world || !segments || world * segments > 1024 || segments > experts_per_rank)
        return ERR_INVALID_ARG;
    const uint64_t pairs = tokens * topk, bins = world * segments;
    if (pairs > 0x7fffff00ull) return ERR_BOUNDS;
    if (workspace_bytes < yvex_b200_ep_dispatch_workspace_bytes(pairs, bins)) return ERR_NOMEM;
    int *bin_of = static_cast<int *>(workspace), *src = bin_of + pairs, *order = src + pairs;
    int *counts = order + pairs, *offsets = counts + bins + 1;
    cudaStream_t s = as_stream(stream);
    cudaMemsetAsync(counts, 0, (bins + 1) * sizeof(int), s);
    ep_bin_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(selected, pairs, topk, (int)experts_per_rank, (int)world, (int)segments, bin_of,
                                                         src, counts, status);
    ep_offsets_kernel<<<1, 32, 0, s>>>(counts, (int)bins, offsets, send_counts);
    wide_scatter_kernel<<<(unsigned)bins, 512, 0, s>>>(bin_of, pairs, offsets, order, inverse);
    return launch_status(3);
}

extern "C" int yvex_b200_ep_dispatch_push(const int32_t *selected, const float *weights, const void *rows_f16, uint64_t tokens,
                                          uint64_t topk, uint64_t hidden, uint64_t experts_per_rank, uint64_t world, uint64_t rank,
                                          uint64_t segments, const long long *counts_all, const unsigned long long *recv_bases,
                                          uint64_t capacity_rows, int expert_major, void *workspace, uint64_t workspace_bytes,
                                          int *status, void *stream) {
    if (!selected || !weights || !rows_f16 || !counts_all || !recv_bases || !status || !workspace) return ERR_INVALID_ARG;
    if (!tokens || !topk || !experts_per_rank || !world || rank >= world || !segments || world * segments > 1024 ||
        segments > experts_per_rank || hidden % 8 || !capacity_rows)
        return ERR_INVALID_ARG;
    const uint64_t pairs = tokens * topk, bins = world * segments;
    if (pairs > 0x7fffff00ull || (reinterpret_cast<uintptr_t>(rows_f16) & 15u)) return ERR_BOUNDS;
    if (workspace_bytes < yvex_b200_ep_dispatch_workspace_bytes(pairs, bins)) return ERR_NOMEM;
    // the plan of yvex_b200_ep_dispatch_plan, left in the same workspace; the write offsets go behind it
    int *bin_of = static_cast<int *>(workspace), *src = bin_of + pairs, *order = src + pairs;
    int *counts = order + pairs, *offsets = counts + bins + 1;
    long long *row_base = reinterpret_cast<long long *>((reinterpret_cast<uintptr_t>(offsets + bins + 2) + 7u) & ~uintptr_t(7));
    cudaStream_t s = as_stream(stream);
    if (expert_major && segments != experts_per_rank) return ERR_INVALID_ARG;
    ep_push_offsets_kernel<<<1, 256, 0, s>>>(counts_all, (int)bins, (int)world, (int)rank, expert_major, row_base);
    ep_push_kernel<<<grid_for(pairs, 1, 16), 128, 0, s>>>(static_cast<const __half *>(rows_f16), selected, weights, order, bin_of, src,
                                                          offsets, row_base, recv_bases, capacity_rows, pairs, hidden,
                                                          (int)experts_per_rank, (int)rank, yvex_b200_ep_payload_pitch(hidden), status);
    return launch_status(2);
}

extern "C" int yvex_b200_moe_expert_rows_payload(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                                 const void *payload, uint64_t pairs, void *y_bf16, void *workspace,
                                                 uint64_t workspace_bytes, int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!pairs) return OK;
    if (!payload || !y_bf16 || !status) return ERR_INVALID_ARG;
    if (pairs > 0x7fffff00ull / 2 || (reinterpret_cast<uintptr_t>(payload) & 15u) || (reinterpret_cast<uintptr_t>(y_bf16) & 15u))
        return ERR_BOUNDS;
    MoeGeom g = *geom;
    if (!moe_wide_gemm_eligible(g, *w)) return ERR_UNSUPPORTED;
    PairWorkspace pw;
    if (!workspace || workspace_bytes < pair_layout(g, pairs, 0, &pw)) return ERR_NOMEM;
    pw.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    const uint64_t pitch = yvex_b200_ep_payload_pitch(g.hidden);
    mark_phase(0, s);
    wide_list_payload_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(static_cast<const uint8_t *>(payload), pitch, g.hidden, pairs,
                                                                   (int)g.experts, pw.expert_of_pair, pw.src_of_pair, pw.weight_of_pair);
    mark_phase(1, s);
    rc = run_pair_list(g, *w, pw, static_cast<const __half *>(payload), pairs, status, s, static_cast<uint16_t *>(y_bf16), pitch);
    if (rc != OK) return rc;
    mark_phase(5, s);
    return launch_status(1);
}

extern "C" int yvex_b200_moe_expert_rows_scatter(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                                 const void *payload, uint64_t pairs, const unsigned long long *home_bases,
                                                 uint64_t world, uint64_t home_pairs, void *workspace, uint64_t workspace_bytes,
                                                 int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!pairs) return OK;
    if (!payload || !home_bases || !status || !world || world > 1024 || !home_pairs) return ERR_INVALID_ARG;
    if (pairs > 0x7fffff00ull / 2 || home_pairs > 0x7fffff00ull || (reinterpret_cast<uintptr_t>(payload) & 15u)) return ERR_BOUNDS;
    MoeGeom g = *geom;
    if (!moe_wide_gemm_eligible(g, *w)) return ERR_UNSUPPORTED;
    PairWorkspace pw;
    if (!workspace || workspace_bytes < pair_layout(g, pairs, 0, &pw)) return ERR_NOMEM;
    pw.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    const uint64_t pitch = yvex_b200_ep_payload_pitch(g.hidden);
    mark_phase(0, s);
    wide_list_payload_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(static_cast<const uint8_t *>(payload), pitch, g.hidden, pairs,
                                                                   (int)g.experts, pw.expert_of_pair, pw.src_of_pair, pw.weight_of_pair);
    mark_phase(1, s);
    rc = run_pair_list(g, *w, pw, static_cast<const __half *>(payload), pairs, status, s, nullptr, pitch, home_bases, (int)world,
                       home_pairs);
    if (rc != OK) return rc;
    mark_phase(5, s);
    return launch_status(1);
}

extern "C" int yvex_b200_moe_expert_rows_sorted(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                                const void *payload, uint64_t pairs, const long long *counts_all, uint64_t world,
                                                uint64_t rank, const unsigned long long *home_bases, uint64_t home_pairs,
                                                void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!pairs) return OK;
    if (!payload || !counts_all || !home_bases || !status || !world || world > 1024 || rank >= world || !home_pairs) return ERR_INVALID_ARG;
    if (pairs > 0x7fffff00ull / 2 || home_pairs > 0x7fffff00ull || (reinterpret_cast<uintptr_t>(payload) & 15u)) return ERR_BOUNDS;
    MoeGeom g = *geom;
    // the activation sums an affine gate/up qtype needs are made by the gather this path does without
    if (!moe_wide_gemm_eligible(g, *w) || g.gate_qtype == Q_Q4_K || g.gate_qtype == Q_Q2_K) return ERR_UNSUPPORTED;
    PairWorkspace pw;
    if (!workspace || workspace_bytes < pair_layout(g, pairs, 0, &pw)) return ERR_NOMEM;
    pw.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    const uint64_t pitch = yvex_b200_ep_payload_pitch(g.hidden);
    mark_phase(0, s);
    ep_sorted_counts_kernel<<<1, 256, 0, s>>>(counts_all, (int)world, (int)rank, (int)g.experts, pairs, pw.counts, status);
    wide_plan_kernel<<<2, 32, 0, s>>>(pw.counts, (int)g.experts, pairs, pw.offsets, pw.blocks, pw.blocks_down, pw.num_blocks,
                                      pw.max_blocks, gemm_tile_n(g.gate_qtype), gemm_tile_n(g.down_qtype), status);
    wide_trailer_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(static_cast<const uint8_t *>(payload), pitch, g.hidden, pairs, pw.offsets,
                                                              (int)g.experts, home_bases, (int)world, home_pairs, pw.weight_sorted,
                                                              pw.dest, status);
    rc = launch_status(3);
    if (rc != OK) return rc;
    mark_phase(1, s);
    mark_phase(2, s);
    rc = run_sorted_gemms(g, *w, pw, static_cast<const __half *>(payload), pitch, pairs, status, s, nullptr, nullptr, pw.dest);
    if (rc != OK) return rc;
    mark_phase(5, s);
    return launch_status(1);
}

extern "C" int yvex_b200_moe_wide_set_cta_limit(int ctas) {
    if (ctas < 1 || ctas > kSmCount) return ERR_INVALID_ARG;
    g_gemm_ctas.store(ctas, std::memory_order_relaxed);
    return OK;
}

extern "C" uint64_t yvex_b200_expert_worklist_workspace_bytes(uint64_t pairs, uint64_t experts) {
    const uint64_t blocks = pairs / 128 + experts + 2;
    return 256 * 8 + (2 * experts + 8) * 4 + 2 * pairs * 4 + 2 * blocks * sizeof(ColBlock) + 64;
}

extern "C" int yvex_b200_expert_worklist(const int32_t *selected, uint64_t rows, uint64_t topk, uint64_t experts,
                                         uint64_t tensor_core_minimum, uint64_t admitted_width, unsigned int provenance,
                                         int32_t *source_pairs, int32_t *source_rows, int32_t *destination_rows,
                                         int32_t *expert_ids, int32_t *bucket_offsets, int32_t *bucket_populations,
                                         yvex_b200_worklist_observation *observation, void *workspace,
                                         uint64_t workspace_bytes, int *status, void *stream) {
    if (!selected || !status || !rows || !topk || !experts || experts > 256 || topk > experts || !admitted_width ||
        provenance >= YVEX_B200_WORKLIST_PROVENANCE_COUNT)
        return ERR_INVALID_ARG;
    if (rows > 0x7fffff00ull / topk) return ERR_BOUNDS;
    const uint64_t pairs = rows * topk;
    cudaStream_t s = as_stream(stream);
    if (pairs <= (uint64_t)kSmallWorklistPairs) {
        worklist_small_kernel<<<1, 256, 0, s>>>(selected, rows, topk, (int)experts, tensor_core_minimum, admitted_width, provenance,
                                                source_pairs, source_rows, destination_rows, expert_ids, bucket_offsets,
                                                bucket_populations, observation, status);
        return launch_status(1);
    }
    if (!workspace || workspace_bytes < yvex_b200_expert_worklist_workspace_bytes(pairs, experts)) return ERR_NOMEM;
    // the sort of the wide path itself: count, plan (offsets), stable scatter
    uint8_t *base = static_cast<uint8_t *>(workspace);
    auto take = [&](uint64_t bytes) { uint8_t *at = base; base += (bytes + 255) & ~255ull; return at; };
    const int max_blocks = (int)(pairs / 128 + experts + 2);
    int *counts = reinterpret_cast<int *>(take((experts + 2) * 4)), *offsets = reinterpret_cast<int *>(take((experts + 3) * 4));
    int *num_blocks = reinterpret_cast<int *>(take(8));
    int *order = source_pairs ? source_pairs : reinterpret_cast<int *>(take(pairs * 4));
    int *pos = reinterpret_cast<int *>(take(pairs * 4));
    ColBlock *b0 = reinterpret_cast<ColBlock *>(take((uint64_t)max_blocks * sizeof(ColBlock)));
    ColBlock *b1 = reinterpret_cast<ColBlock *>(take((uint64_t)max_blocks * sizeof(ColBlock)));
    cudaMemsetAsync(counts, 0, (experts + 2) * 4, s);
    wide_count_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(selected, pairs, (int)experts + 1, counts, status);
    wide_plan_kernel<<<2, 32, 0, s>>>(counts, (int)experts, pairs, offsets, b0, b1, num_blocks, max_blocks, 256, 128, status);
    worklist_observe_kernel<<<1, 32, 0, s>>>(counts, offsets, (int)experts, pairs, rows, tensor_core_minimum, admitted_width, provenance,
                                             observation, expert_ids, bucket_offsets, bucket_populations, status);
    int launches = 3;
    if (source_pairs || source_rows || destination_rows) {
        wide_scatter_kernel<<<(unsigned)experts + 1, 512, 0, s>>>(selected, pairs, offsets, order, pos);
        worklist_rows_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(order, pairs, topk, source_rows, destination_rows);
        launches += 2;
    }
    return launch_status(launches);
}

extern "C" int yvex_b200_moe_combine_indexed(const void *y_routed_bf16, const int32_t *routed_rows, const void *y_shared_bf16,
                                             const int32_t *shared_rows, uint64_t tokens, uint64_t topk, uint64_t hidden,
                                             float *out, int *status, void *stream) {
    if (!y_routed_bf16 || !y_shared_bf16 || !out || !status || !tokens || !topk || !hidden) return ERR_INVALID_ARG;
    if (hidden % 8 || ((reinterpret_cast<uintptr_t>(y_routed_bf16) | reinterpret_cast<uintptr_t>(y_shared_bf16) |
                        reinterpret_cast<uintptr_t>(out)) & 15u))
        return ERR_INVALID_ARG;
    wide_combine_kernel<<<dim3((unsigned)((hidden / 8 + 127) / 128), (unsigned)grid_for(tokens, 1, 16)), 128, 0, as_stream(stream)>>>(
        static_cast<const uint16_t *>(y_routed_bf16), static_cast<const uint16_t *>(y_shared_bf16), routed_rows, shared_rows, tokens,
        topk, hidden, out);
    return launch_status(1);
}

extern "C" int yvex_b200_moe_combine(const void *y_routed_bf16, const void *y_shared_bf16, uint64_t tokens, uint64_t topk,
                                     uint64_t hidden, float *out, int *status, void *stream) {
    return yvex_b200_moe_combine_indexed(y_routed_bf16, nullptr, y_shared_bf16, nullptr, tokens, topk, hidden, out, status, stream);
}
