// Wide-batch (prefill / expert-parallel shard) MoE layer:
//   ingress + route  ->  expert-major stable counting sort (the reference's worklist order,
//   src/graph/worklist.c:369-441)  ->  gather rows to expert-major fp16  ->  grouped dequant GEMM
//   gate & up (tcgen05)  ->  SwiGLU * route weight -> bf16 (+ sub-block sums for affine down
//   qtypes)  ->  grouped dequant GEMM down -> bf16 per pair  ->  unpermute: routed rows summed in
//   rank order in f32, + shared, -> bf16 (src/runtime/moe.c:619-632).
// The shared expert is one more group holding every token in token order.
#include <cudaTypedefs.h>

#include <type_traits>

#include "moe_gemm.cuh"

namespace yb {

// ---- permute ---------------------------------------------------------------------------------------
__global__ void wide_count_kernel(const int32_t *selected, uint64_t pairs, int experts, int *counts, int *status) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < pairs; i += (uint64_t)gridDim.x * blockDim.x) {
        const int e = selected[i];
        if (e < 0 || e >= experts) raise(status, YVEX_B200_STATUS_ARGUMENT);
        else atomicAdd(&counts[e], 1);
    }
}

// One thread: exclusive scan of the group sizes and the column-block list (routed groups in
// expert order, then the shared expert's token blocks).
__global__ void wide_plan_kernel(const int *counts, int experts, uint64_t tokens, uint64_t pairs, int *offsets,
                                 ColBlock *blocks, int *num_blocks, int max_blocks, int *status) {
    if (threadIdx.x || blockIdx.x) return;
    int off = 0, nb = 0;
    for (int e = 0; e < experts; ++e) {
        offsets[e] = off;
        for (int c = 0; c < counts[e]; c += kTileN) {
            if (nb < max_blocks) blocks[nb] = ColBlock{off + c, min(kTileN, counts[e] - c), e, 0};
            ++nb;
        }
        off += counts[e];
    }
    offsets[experts] = off;
    if ((uint64_t)off != pairs) raise(status, YVEX_B200_STATUS_ARGUMENT);
    for (uint64_t c = 0; c < tokens; c += kTileN) {
        if (nb < max_blocks) blocks[nb] = ColBlock{(int)(pairs + c), (int)min((uint64_t)kTileN, tokens - c), -1, 0};
        ++nb;
    }
    if (nb > max_blocks) { raise(status, YVEX_B200_STATUS_ARGUMENT); nb = max_blocks; }
    *num_blocks = nb;
}

// One CTA per expert: stable compaction of the pairs routed to it (ascending pair index).
__global__ void wide_scatter_kernel(const int32_t *selected, uint64_t pairs, const int *offsets, int *perm, int *pos_of_pair) {
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __shared__ int warp_count[32];
    __shared__ int base;
    if (threadIdx.x == 0) base = offsets[e];
    __syncthreads();
    for (uint64_t start = 0; start < pairs; start += blockDim.x) {
        const uint64_t i = start + threadIdx.x;
        const bool hit = i < pairs && selected[i] == e;
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

// act_h[pos] = fp16 row of the pair's token (routed, expert-major) and of every token (shared).
__global__ void wide_gather_kernel(const __half *xr_h, const int *perm, uint64_t pairs, uint64_t tokens, uint64_t topk,
                                   uint64_t hidden, __half *act_h) {
    const uint64_t chunks = hidden / 8;           // 16-byte chunks per row
    const uint64_t total = (pairs + tokens) * chunks;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / chunks, c = i % chunks;
        const uint64_t tok = row < pairs ? (uint64_t)perm[row] / topk : row - pairs;
        reinterpret_cast<uint4 *>(act_h)[row * chunks + c] = __ldg(reinterpret_cast<const uint4 *>(xr_h) + tok * chunks + c);
    }
}

// mid = bf16(silu(min(g,L)) * clamp(u,+-L) * w) as fp16, plus hi/lo fp16 sums over `group`
// consecutive intermediates (32 for Q4_K, 16 for Q2_K, 0 = none) for the down GEMM's min term.
__global__ void wide_swiglu_kernel(const float *gate, const float *up, const int *perm, const float *weights, uint64_t pairs,
                                   uint64_t rows, uint64_t inter, float limit, int group, __half *mid_h, __half *sums,
                                   int *status) {
    const int lane = threadIdx.x & 31;
    const uint64_t total = rows * inter;          // inter is a multiple of 256, so warps never straddle rows
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / inter, col = i % inter;
        const float w = row < pairs ? weights[perm[row]] : 1.0f;
        const float v = swiglu_mid(gate[i], up[i], w, limit, status);
        mid_h[i] = __float2half_rn(v);
        if (group) {
            float s = v;
            for (int o = group / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if ((lane & (group - 1)) == 0) {
                const __half hi = __float2half_rn(s), lo = __float2half_rn(s - __half2float(hi));
                const uint64_t sb = col / 256, sub = (col % 256) / group, per = 256 / group;
                __half *dst = sums + (row * (inter / 256) + sb) * 32;
                dst[sub] = hi;
                dst[per + sub] = lo;
            }
        }
    }
}

// out[t] = bf16( sum_{rank} y[pos(t, rank)] (rank order, f32) + y[pairs + t] )
__global__ void wide_combine_kernel(const uint16_t *y, const int *pos_of_pair, uint64_t tokens, uint64_t topk, uint64_t pairs,
                                    uint64_t hidden, float *out) {
    const uint64_t total = tokens * hidden;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t t = i / hidden, h = i % hidden;
        float routed = 0.0f;
        for (uint64_t r = 0; r < topk; ++r)
            routed += __uint_as_float((uint32_t)y[(uint64_t)pos_of_pair[t * topk + r] * hidden + h] << 16);
        const float shared = __uint_as_float((uint32_t)y[(pairs + t) * hidden + h] << 16);
        out[i] = bf16_round(routed + shared);
    }
}

// ---- workspace -------------------------------------------------------------------------------------
struct WideWorkspace {
    int *counts, *offsets, *perm, *pos_of_pair, *num_blocks;
    ColBlock *blocks;
    __half *act_h, *mid_h, *sums;
    float *gate, *up;
    uint16_t *y;
    int max_blocks;
};

static uint64_t wide_layout(const MoeGeom &g, uint64_t rows, uint64_t base_off, WideWorkspace *ws) {
    uint64_t off = base_off;
    auto take = [&](uint64_t bytes) { uint64_t at = off; off = (off + bytes + 255) & ~255ull; return at; };
    const uint64_t pairs = rows * g.topk, all = pairs + rows;
    WideWorkspace l{};
    l.max_blocks = (int)(pairs / kTileN + g.experts + rows / kTileN + 2);
    l.counts = reinterpret_cast<int *>(take((g.experts + 1) * 4));
    l.offsets = reinterpret_cast<int *>(take((g.experts + 2) * 4));
    l.num_blocks = reinterpret_cast<int *>(take(4));
    l.perm = reinterpret_cast<int *>(take(pairs * 4));
    l.pos_of_pair = reinterpret_cast<int *>(take(pairs * 4));
    l.blocks = reinterpret_cast<ColBlock *>(take((uint64_t)l.max_blocks * sizeof(ColBlock)));
    l.act_h = reinterpret_cast<__half *>(take((all + kTileN) * g.hidden * 2));
    l.mid_h = reinterpret_cast<__half *>(take((all + kTileN) * g.inter * 2));
    l.sums = reinterpret_cast<__half *>(take((all + kTileN) * (g.inter / 256) * 64));
    l.gate = reinterpret_cast<float *>(take(all * g.inter * 4));
    l.up = reinterpret_cast<float *>(take(all * g.inter * 4));
    l.y = reinterpret_cast<uint16_t *>(take(all * g.hidden * 2));
    if (ws) *ws = l;
    return off;
}

uint64_t moe_wide_workspace_bytes(const MoeGeom &g, uint64_t rows) {
    return wide_layout(g, rows, moe_workspace_layout(g, rows, nullptr), nullptr);
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

// Row-major fp16 [rows][width] -> tiles of [kTileN rows][64 columns], 128-byte swizzle, zero fill.
static int make_act_map(CUtensorMap *map, const __half *base, uint64_t rows, uint64_t width) {
    auto fn = encode_fn();
    if (!fn) return ERR_BACKEND;
    cuuint64_t dims[2] = {width, rows}, strides[1] = {width * 2};
    cuuint32_t box[2] = {kChunkK, kTileN}, estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? OK : ERR_BACKEND;
}

template <class Dec>
static int launch_gemm(const CUtensorMap &map, const GemmParams &p, cudaStream_t s) {
    const size_t smem = (size_t)(2 * kStages + 4) * kTileBytes + sizeof(MmaTables) + sizeof(GemmSmem) + 1024 + 64;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(moe_grouped_gemm_kernel<Dec>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return ERR_BACKEND;
        configured = true;
    }
    moe_grouped_gemm_kernel<Dec><<<kSmCount, kGemmThreads, smem, s>>>(map, p);
    return launch_status(1);
}

static int run_gemm(unsigned qtype, const CUtensorMap &map, const GemmParams &p, cudaStream_t s) {
    switch (qtype) {
    case Q_IQ2_XXS: return launch_gemm<GemmIq2>(map, p, s);
    case Q_Q4_K: return launch_gemm<GemmQ4k>(map, p, s);
    case Q_Q2_K: return launch_gemm<GemmQ2k>(map, p, s);
    default: return ERR_UNSUPPORTED;
    }
}

static bool gemm_qtype(unsigned q) { return q == Q_IQ2_XXS || q == Q_Q4_K || q == Q_Q2_K; }

bool moe_wide_gemm_eligible(const MoeGeom &g, const MoeWeights &w) {
    const uintptr_t ptrs = (uintptr_t)w.gate | (uintptr_t)w.up | (uintptr_t)w.down | (uintptr_t)w.shared_gate |
                           (uintptr_t)w.shared_up | (uintptr_t)w.shared_down;
    return g.gate_qtype == g.up_qtype && gemm_qtype(g.gate_qtype) && gemm_qtype(g.down_qtype) &&
           g.inter == g.shared_inter && g.hidden % 256 == 0 && g.inter % 256 == 0 && (ptrs & 15u) == 0;
}

int moe_experts_wide(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, void *workspace, uint64_t rows,
                     float *out, int *status, cudaStream_t s) {
    WideWorkspace ww;
    wide_layout(g, rows, moe_workspace_layout(g, rows, nullptr), &ww);
    auto rebase = [&](auto *&ptr) { ptr = reinterpret_cast<std::remove_reference_t<decltype(ptr)>>(
                                        reinterpret_cast<uintptr_t>(workspace) + reinterpret_cast<uintptr_t>(ptr)); };
    rebase(ww.counts); rebase(ww.offsets); rebase(ww.perm); rebase(ww.pos_of_pair); rebase(ww.num_blocks);
    rebase(ww.blocks); rebase(ww.act_h); rebase(ww.mid_h); rebase(ww.sums); rebase(ww.gate); rebase(ww.up); rebase(ww.y);
    const uint64_t pairs = rows * g.topk, all = pairs + rows;
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);

    cudaMemsetAsync(ww.counts, 0, (g.experts + 1) * 4, s);
    wide_count_kernel<<<grid_for(pairs, 256, 4), 256, 0, s>>>(ws.selected, pairs, (int)g.experts, ww.counts, status);
    wide_plan_kernel<<<1, 32, 0, s>>>(ww.counts, (int)g.experts, rows, pairs, ww.offsets, ww.blocks, ww.num_blocks,
                                      ww.max_blocks, status);
    wide_scatter_kernel<<<(unsigned)g.experts, 512, 0, s>>>(ws.selected, pairs, ww.offsets, ww.perm, ww.pos_of_pair);
    wide_gather_kernel<<<grid_for(all * (g.hidden / 8), 256, 16), 256, 0, s>>>(ws.xr_h, ww.perm, pairs, rows, g.topk, g.hidden,
                                                                               ww.act_h);
    int rc = launch_status(4);
    if (rc != OK) return rc;
    mark_phase(2, s);

    CUtensorMap act_map, mid_map;
    if (make_act_map(&act_map, ww.act_h, all, g.hidden) != OK || make_act_map(&mid_map, ww.mid_h, all, g.inter) != OK)
        return ERR_BACKEND;
    GemmParams gu{};
    gu.w_routed[0] = (const uint8_t *)w.gate; gu.w_routed[1] = (const uint8_t *)w.up;
    gu.w_shared[0] = (const uint8_t *)w.shared_gate; gu.w_shared[1] = (const uint8_t *)w.shared_up;
    gu.row_bytes = g.hidden / gg.elems * gg.bytes;
    gu.M = (int)g.inter; gu.K = (int)g.hidden; gu.nmat = 2;
    gu.colblocks = ww.blocks; gu.num_colblocks = ww.num_blocks;
    gu.out_f32[0] = ww.gate; gu.out_f32[1] = ww.up; gu.out_bf16 = nullptr; gu.sums = nullptr; gu.status = status;
    if (g.inter % kTileM || g.hidden % kTileM) return ERR_BOUNDS;
    rc = run_gemm(g.gate_qtype, act_map, gu, s);
    if (rc != OK) return rc;
    mark_phase(3, s);

    const int group = g.down_qtype == Q_Q4_K ? 32 : g.down_qtype == Q_Q2_K ? 16 : 0;
    wide_swiglu_kernel<<<grid_for(all * g.inter, 256, 16), 256, 0, s>>>(ww.gate, ww.up, ww.perm, ws.weights, pairs, all, g.inter,
                                                                       (float)g.limit, group, ww.mid_h, ww.sums, status);
    GemmParams dn{};
    dn.w_routed[0] = (const uint8_t *)w.down; dn.w_shared[0] = (const uint8_t *)w.shared_down;
    dn.row_bytes = g.inter / dg.elems * dg.bytes;
    dn.M = (int)g.hidden; dn.K = (int)g.inter; dn.nmat = 1;
    dn.colblocks = ww.blocks; dn.num_colblocks = ww.num_blocks;
    dn.out_bf16 = ww.y; dn.sums = ww.sums; dn.status = status;
    rc = run_gemm(g.down_qtype, mid_map, dn, s);
    if (rc != OK) return rc;
    mark_phase(4, s);
    wide_combine_kernel<<<grid_for(rows * g.hidden, 256, 16), 256, 0, s>>>(ww.y, ww.pos_of_pair, rows, g.topk, pairs, g.hidden, out);
    return launch_status(2);
}

}  // namespace yb

using namespace yb;

extern "C" int yvex_b200_moe_wide(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                  const float *x, const float *logits, const uint32_t *token_ids,
                                  uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                                  void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!x || !out || !status || !rows) return ERR_INVALID_ARG;
    if (rows * (geom->topk + 1) > 0x7fffff00ull / 2) return ERR_BOUNDS;       // 32-bit row indices
    MoeGeom g = *geom;
    MoeWorkspace ws;
    const bool gemm = moe_wide_gemm_eligible(g, *w);
    const uint64_t need = gemm ? moe_wide_workspace_bytes(g, rows) : moe_workspace_layout(g, rows, nullptr);
    moe_workspace_layout(g, rows, &ws);
    if (!workspace || workspace_bytes < need) return ERR_NOMEM;
    ws.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    mark_phase(0, s);
    rc = moe_ingress_and_route(g, *w, ws, x, logits, token_ids, rows, status, s);
    if (rc != OK) return rc;
    mark_phase(1, s);
    rc = gemm ? moe_experts_wide(g, *w, ws, workspace, rows, out, status, s) : moe_experts_rows(g, *w, ws, rows, out, status, s);
    if (rc != OK) return rc;
    if (selected_out) cudaMemcpyAsync(selected_out, ws.selected, rows * g.topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, s);
    if (weights_out) cudaMemcpyAsync(weights_out, ws.weights, rows * g.topk * sizeof(float), cudaMemcpyDeviceToDevice, s);
    return launch_status(0);
}

extern "C" uint64_t yvex_b200_moe_wide_workspace_bytes(const yvex_b200_moe_geometry *g, uint64_t rows) {
    return g ? moe_wide_workspace_bytes(*g, rows) : 0;
}
