// Narrow-batch (decode) expert execution on the streaming tensor-core matvec engine.
//
//   gate_up kernel: a tile is 8 rows of the gate matrix and the same 8 rows of the up matrix of
//     one (token, expert) pair; the two row sets are the CTA's two row groups, so the SwiGLU *
//     route weight -> bf16 epilogue (src/graph/moe.c:605-613) runs in the kernel that produced
//     both dot products. The expert id comes from the router's device output: no host round trip.
//   down kernel: a tile is 8*RG output rows of one token; the CTA walks the token's k routed
//     experts in rank order and then the shared expert, rounds each expert's row to bf16, sums
//     the routed rows in rank order in f32 and publishes bf16(routed + shared)
//     (src/graph/moe.c:616-620, src/runtime/moe.c:619-632). No atomics: the order is fixed.
// Both kernels are persistent over their tile list with the cp.async ring of gemv_mma.cuh.
#include "gemv_mma.cuh"
#include "moe_common.cuh"

namespace yb {

struct NarrowParams {
    MoeGeom g;
    MoeWeights w;
    MoeWorkspace ws;
    uint64_t rows;
    float *out;
    int *status;
    int slices, row_groups;
    uint32_t stage_bytes;      // one row set (gate or up / one down tile), 16-byte multiple
    uint64_t gate_row_bytes, down_row_bytes;
};

template <class Dec>
__global__ void __launch_bounds__(512) moe_gate_up_mma_kernel(NarrowParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    MmaSmem *sm = reinterpret_cast<MmaSmem *>(smem);
    uint8_t *stages = smem + sizeof(MmaSmem);
    const MoeGeom &g = p.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gi = lane >> 2, t = lane & 3;
    const int slice = warp % p.slices, rg = warp / p.slices;       // rg 0 = gate rows, 1 = up rows
    const uint64_t ppr = g.topk + 1, imax = g.inter > g.shared_inter ? g.inter : g.shared_inter;
    const uint64_t itiles = (imax + 7) / 8, tiles = p.rows * ppr * itiles;
    const uint64_t rb = p.gate_row_bytes;
    constexpr int kSumsPerBlock = Dec::kSumGroup ? 256 / Dec::kSumGroup : 0;
    const int K = (int)g.hidden, nblocks = K / 256;
    const int my_blocks = min(kSliceBlocks, nblocks - slice * kSliceBlocks);
    load_tables(&sm->tab, Dec::kBias);

    struct Tile { const uint8_t *gate, *up, *lo_g, *hi_g, *lo_u, *hi_u; uint64_t pair, i0, width; float rw; };
    auto locate = [&](uint64_t tile) {
        Tile tl;
        tl.pair = tile / itiles;
        tl.i0 = (tile % itiles) * 8;
        const uint64_t r = tl.pair / ppr, pp = tl.pair % ppr;
        if (pp == g.topk) {
            tl.width = g.shared_inter; tl.rw = 1.0f;
            tl.lo_g = (const uint8_t *)p.w.shared_gate; tl.lo_u = (const uint8_t *)p.w.shared_up;
            tl.hi_g = tl.lo_g + g.shared_inter * rb; tl.hi_u = tl.lo_u + g.shared_inter * rb;
            tl.gate = tl.lo_g + tl.i0 * rb; tl.up = tl.lo_u + tl.i0 * rb;
        } else {
            const uint64_t e = (uint64_t)p.ws.selected[r * g.topk + pp];
            tl.width = g.inter; tl.rw = p.ws.weights[r * g.topk + pp];
            tl.lo_g = (const uint8_t *)p.w.gate; tl.lo_u = (const uint8_t *)p.w.up;
            tl.hi_g = tl.lo_g + g.experts * g.inter * rb; tl.hi_u = tl.lo_u + g.experts * g.inter * rb;
            tl.gate = tl.lo_g + (e * g.inter + tl.i0) * rb; tl.up = tl.lo_u + (e * g.inter + tl.i0) * rb;
        }
        return tl;
    };
    auto issue = [&](uint64_t tile, int stage) {
        if (tile < tiles) {
            Tile tl = locate(tile);
            if (tl.i0 < tl.width) {
                const uint64_t n = tl.width - tl.i0 < 8 ? tl.width - tl.i0 : 8;
                uint8_t *st = stages + (size_t)stage * 2 * p.stage_bytes;
                stage_span(st, tl.gate, n * rb, tl.lo_g, tl.hi_g);
                stage_span(st + p.stage_bytes, tl.up, n * rb, tl.lo_u, tl.hi_u);
            }
        }
        cp_async_commit();
    };
    uint32_t bfrag[8 * kSliceBlocks][2];
    uint64_t cur_row = ~0ull;
    uint64_t tile = blockIdx.x;
#pragma unroll
    for (int s = 0; s < kGemvStages - 1; ++s) issue(tile + (uint64_t)s * gridDim.x, s);
    for (int it = 0; tile < tiles; tile += gridDim.x, ++it) {
        issue(tile + (uint64_t)(kGemvStages - 1) * gridDim.x, (it + kGemvStages - 1) % kGemvStages);
        const Tile tl = locate(tile);
        const uint64_t r = tl.pair / ppr;
        if (r != cur_row) {          // uniform across the CTA: every thread walks the same tile list
            build_bfrag<Dec, true>(bfrag, nullptr, p.ws.xr_h + r * g.hidden, slice * 256 * kSliceBlocks, K, gi, t, p.status);
            build_sums<Dec::kSumGroup>(sm->sums, p.ws.xr + r * g.hidden, K);
            cur_row = r;
        }
        cp_async_wait<kGemvStages - 1>();
        __syncthreads();
        if (tl.i0 < tl.width) {
            const uint8_t *src = rg == 0 ? tl.gate : tl.up;
            const uint8_t *base = stages + (size_t)(it % kGemvStages) * 2 * p.stage_bytes + (size_t)rg * p.stage_bytes +
                                  (reinterpret_cast<uintptr_t>(src) & 15u);
            const bool valid = tl.i0 + gi < tl.width;
            const uint8_t *rowp = base + (size_t)gi * rb + (size_t)slice * kSliceBlocks * Dec::kBlockBytes;
            float part = warp_slice_dot<Dec, true>(rowp, my_blocks, &sm->tab, bfrag,
                                                   sm->sums + slice * kSliceBlocks * kSumsPerBlock, t, valid, p.status);
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            if (t == 0) sm->red[(rg * p.slices + slice) * 8 + gi] = part;
        }
        __syncthreads();
        if (threadIdx.x < 8 && tl.i0 + threadIdx.x < tl.width) {
            float gs = 0.0f, us = 0.0f;
            for (int s = 0; s < p.slices; ++s) {
                gs += sm->red[s * 8 + threadIdx.x];
                us += sm->red[(p.slices + s) * 8 + threadIdx.x];
            }
            const float v = swiglu_mid(gs, us, tl.rw, (float)g.limit, p.status);
            p.ws.mid[tl.pair * imax + tl.i0 + threadIdx.x] = v;
            p.ws.mid_h[tl.pair * imax + tl.i0 + threadIdx.x] = __float2half_rn(v);
        }
    }
    cp_async_wait<0>();
}

template <class Dec>
__global__ void __launch_bounds__(512) moe_down_mma_kernel(NarrowParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    MmaSmem *sm = reinterpret_cast<MmaSmem *>(smem);
    uint8_t *stages = smem + sizeof(MmaSmem);
    const MoeGeom &g = p.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gi = lane >> 2, t = lane & 3;
    const int slice = warp % p.slices, rg = warp / p.slices;
    const int tile_rows = 8 * p.row_groups;
    const uint64_t ppr = g.topk + 1, imax = g.inter;            // inter == shared_inter on this path
    const uint64_t htiles = (g.hidden + tile_rows - 1) / tile_rows, tiles = p.rows * htiles, steps = tiles * ppr;
    const uint64_t rb = p.down_row_bytes;
    constexpr int kSumsPerBlock = Dec::kSumGroup ? 256 / Dec::kSumGroup : 0;
    const int K = (int)g.inter, nblocks = K / 256;
    const int my_blocks = min(kSliceBlocks, nblocks - slice * kSliceBlocks);
    load_tables(&sm->tab, Dec::kBias);

    struct Step { const uint8_t *src, *lo, *hi; uint64_t r, h0, pp; };
    // local step ls of this CTA -> (tile = blockIdx.x + (ls / ppr) * gridDim.x, pair rank ls % ppr)
    auto locate = [&](uint64_t ls, Step &st) {
        const uint64_t tile = blockIdx.x + (ls / ppr) * gridDim.x;
        if (tile >= tiles) return false;
        st.pp = ls % ppr;
        st.r = tile / htiles;
        st.h0 = (tile % htiles) * tile_rows;
        if (st.pp == g.topk) {
            st.lo = (const uint8_t *)p.w.shared_down;
            st.hi = st.lo + g.hidden * rb;
            st.src = st.lo + st.h0 * rb;
        } else {
            const uint64_t e = (uint64_t)p.ws.selected[st.r * g.topk + st.pp];
            st.lo = (const uint8_t *)p.w.down;
            st.hi = st.lo + g.experts * g.hidden * rb;
            st.src = st.lo + (e * g.hidden + st.h0) * rb;
        }
        return true;
    };
    auto issue = [&](uint64_t ls, int stage) {
        Step st;
        if (locate(ls, st)) {
            const uint64_t n = g.hidden - st.h0 < (uint64_t)tile_rows ? g.hidden - st.h0 : (uint64_t)tile_rows;
            stage_span(stages + (size_t)stage * p.stage_bytes, st.src, n * rb, st.lo, st.hi);
        }
        cp_async_commit();
    };
    (void)steps;
    uint32_t bfrag[8 * kSliceBlocks][2];
    float routed = 0.0f;
#pragma unroll
    for (int s = 0; s < kGemvStages - 1; ++s) issue(s, s);
    Step st;
    for (uint64_t ls = 0; locate(ls, st); ++ls) {
        issue(ls + kGemvStages - 1, (int)((ls + kGemvStages - 1) % kGemvStages));
        const uint64_t pair = st.r * ppr + st.pp;
        build_bfrag<Dec, true>(bfrag, nullptr, p.ws.mid_h + pair * imax, slice * 256 * kSliceBlocks, K, gi, t, p.status);
        build_sums<Dec::kSumGroup>(sm->sums, p.ws.mid + pair * imax, K);
        cp_async_wait<kGemvStages - 1>();
        __syncthreads();
        const uint8_t *base = stages + (size_t)(ls % kGemvStages) * p.stage_bytes + (reinterpret_cast<uintptr_t>(st.src) & 15u);
        const bool valid = st.h0 + 8 * rg + gi < g.hidden;
        const uint8_t *rowp = base + (size_t)(8 * rg + gi) * rb + (size_t)slice * kSliceBlocks * Dec::kBlockBytes;
        float part = warp_slice_dot<Dec, true>(rowp, my_blocks, &sm->tab, bfrag,
                                               sm->sums + slice * kSliceBlocks * kSumsPerBlock, t, valid, p.status);
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        if (t == 0) sm->red[(rg * p.slices + slice) * 8 + gi] = part;
        __syncthreads();
        if (threadIdx.x < tile_rows && st.h0 + threadIdx.x < g.hidden) {
            const int rrg = threadIdx.x >> 3, rgi = threadIdx.x & 7;
            float sum = 0.0f;
            for (int s = 0; s < p.slices; ++s) sum += sm->red[(rrg * p.slices + s) * 8 + rgi];
            if (!isfinite(sum)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
            sum = bf16_round(sum);
            if (st.pp == g.topk) {
                p.out[st.r * g.hidden + st.h0 + threadIdx.x] = bf16_round(routed + sum);
                routed = 0.0f;
            } else {
                routed += sum;
            }
        }
    }
    cp_async_wait<0>();
}

template <class Dec>
static int launch_gate_up(NarrowParams &p, cudaStream_t s) {
    int rgs;
    mma_shape(p.g.hidden, p.slices, rgs);
    p.row_groups = 2;
    p.stage_bytes = (uint32_t)((8 * p.gate_row_bytes + 16 + 15) & ~15ull);
    const size_t smem = sizeof(MmaSmem) + (size_t)kGemvStages * 2 * p.stage_bytes;
    static bool configured = false;
    if (!configured) {
        if (mma_opt_in(moe_gate_up_mma_kernel<Dec>) != OK) return ERR_BACKEND;
        configured = true;
    }
    if (smem > 200 * 1024 || p.slices * 2 > 16) return ERR_BOUNDS;
    const uint64_t imax = p.g.inter > p.g.shared_inter ? p.g.inter : p.g.shared_inter;
    const uint64_t tiles = p.rows * (p.g.topk + 1) * ((imax + 7) / 8);
    moe_gate_up_mma_kernel<Dec><<<grid_for(tiles, 1, 2), 64 * p.slices, smem, s>>>(p);
    return launch_status(1);
}

template <class Dec>
static int launch_down(NarrowParams &p, cudaStream_t s) {
    mma_shape(p.g.inter, p.slices, p.row_groups);
    if (p.row_groups > 2) p.row_groups = 2;
    p.stage_bytes = (uint32_t)((8ull * p.row_groups * p.down_row_bytes + 16 + 15) & ~15ull);
    const size_t smem = sizeof(MmaSmem) + (size_t)kGemvStages * p.stage_bytes;
    static bool configured = false;
    if (!configured) {
        if (mma_opt_in(moe_down_mma_kernel<Dec>) != OK) return ERR_BACKEND;
        configured = true;
    }
    if (smem > 200 * 1024) return ERR_BOUNDS;
    const uint64_t tiles = p.rows * ((p.g.hidden + 8 * p.row_groups - 1) / (8 * p.row_groups));
    moe_down_mma_kernel<Dec><<<grid_for(tiles, 1, 3), 32 * p.slices * p.row_groups, smem, s>>>(p);
    return launch_status(1);
}

static bool aligned_for(unsigned q, const void *ptr) {
    const uintptr_t a = q == Q_Q4_K ? 15u : q == Q_Q2_K ? 3u : 1u;
    return (reinterpret_cast<uintptr_t>(ptr) & a) == 0;
}

int moe_experts_narrow(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows,
                       float *out, int *status, cudaStream_t s) {
    NarrowParams p{};
    p.g = g; p.w = w; p.ws = ws; p.rows = rows; p.out = out; p.status = status;
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
    p.gate_row_bytes = g.hidden / gg.elems * gg.bytes;
    p.down_row_bytes = g.inter / dg.elems * dg.bytes;
    int rc;
    const bool up_mma = g.gate_qtype == g.up_qtype && mma_decoder_for(g.gate_qtype) && g.hidden % 256 == 0 &&
                        (g.hidden / 256 + kSliceBlocks - 1) / kSliceBlocks <= 8 &&     // 2 row sets x slices <= 16 warps
                        aligned_for(g.gate_qtype, w.gate) && aligned_for(g.gate_qtype, w.up) &&
                        aligned_for(g.gate_qtype, w.shared_gate) && aligned_for(g.gate_qtype, w.shared_up);
    if (up_mma) {
        rc = g.gate_qtype == Q_IQ2_XXS ? launch_gate_up<Iq2Decoder>(p, s)
             : g.gate_qtype == Q_Q4_K  ? launch_gate_up<Q4kDecoder>(p, s)
                                       : launch_gate_up<Q2kDecoder>(p, s);
    } else {
        rc = moe_up_rows(g, w, ws, rows, status, s);
    }
    if (rc != OK) return rc;
    mark_phase(2, s);
    const bool down_mma = mma_decoder_for(g.down_qtype) && g.inter == g.shared_inter && g.inter % 256 == 0 &&
                          g.inter / 256 <= kMaxSlices * kSliceBlocks && aligned_for(g.down_qtype, w.down) &&
                          aligned_for(g.down_qtype, w.shared_down);
    if (down_mma) {
        rc = g.down_qtype == Q_IQ2_XXS ? launch_down<Iq2Decoder>(p, s)
             : g.down_qtype == Q_Q4_K  ? launch_down<Q4kDecoder>(p, s)
                                       : launch_down<Q2kDecoder>(p, s);
    } else {
        rc = moe_down_rows(g, w, ws, rows, out, status, s);
    }
    mark_phase(3, s);
    return rc;
}

}  // namespace yb
