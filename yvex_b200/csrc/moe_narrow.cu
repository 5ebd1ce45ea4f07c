// Narrow-batch (decode) expert execution on the streaming tensor-core matvec engine.
//
// One CTA column (blockIdx.y) per token row, so the row's activation sits in shared memory once.
//   gate_up kernel: a CTA task is 8 rows of the gate matrix and the same 8 rows of the up matrix of
//     one (token, expert) pair; warps are (gate | up) x K-slices, the partial dots meet in shared
//     memory and the SwiGLU * route weight -> bf16 epilogue (src/graph/moe.c:605-613) runs in the
//     kernel that produced both dot products. The expert ids come from the router's device
//     output: no host round trip.
//   down kernel: a CTA task is 8 output rows of the token; warp w multiplies them with the
//     SwiGLU row of pair w (rank order, then the shared expert), each expert's row is rounded to
//     bf16, the routed rows are summed in rank order in f32 and bf16(routed + shared) is published
//     (src/graph/moe.c:616-620, src/runtime/moe.c:619-632). No atomics: the order is fixed.
// Both kernels are persistent over their task list; every warp streams its rows through its own
// cp.async ring (gemv_mma.cuh).
#include "gemv_mma.cuh"
#include "moe_common.cuh"

namespace yb {

constexpr int kMaxPairs = 17;           // topk <= 16 plus the shared expert

struct NarrowParams {
    MoeGeom g;
    MoeWeights w;
    MoeWorkspace ws;
    uint64_t rows;
    float *out;
    int *status;
    int slices, slice_blocks;           // gate/up: K-slices per row set and superblocks per slice
    int down_warps;                     // down: pairs handled concurrently
    uint64_t gate_row_bytes, down_row_bytes;
};

struct RouteSmem {
    int sel[kMaxPairs + 3];
    float weight[kMaxPairs + 3];
};

// Shared memory: tables | zeros | activation fp16 [vec_halves] | sums [sum_floats] | route | red [2][red_rows*8] | rings
__host__ __device__ inline size_t narrow_smem_fixed(size_t vec_halves, size_t sum_floats, int red_rows) {
    return (sizeof(MmaTables) + kZeroHalves * 2 + vec_halves * 2 + sum_floats * 4 + sizeof(RouteSmem) + (size_t)2 * red_rows * 8 * 4 + 15) &
           ~(size_t)15;
}

template <class Dec>
__global__ void __launch_bounds__(512, 2) moe_gate_up_mma_kernel(NarrowParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const MoeGeom &g = p.g;
    const int K = (int)g.hidden, nblk = K / 256, warps = blockDim.x >> 5;
    MmaTables *tab = reinterpret_cast<MmaTables *>(smem);
    __half *zeros = reinterpret_cast<__half *>(smem + sizeof(MmaTables));
    __half *xh = zeros + kZeroHalves;
    float *sums = reinterpret_cast<float *>(xh + K);
    RouteSmem *route = reinterpret_cast<RouteSmem *>(sums + K / 16);
    float *red = reinterpret_cast<float *>(route + 1);
    uint8_t *rings = smem + narrow_smem_fixed(K, K / 16, warps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gi = lane >> 2, t = lane & 3;
    const int sl = warp % p.slices, rg = warp / p.slices;          // rg 0 = gate rows, 1 = up rows
    const int my_first = sl * p.slice_blocks, my_blocks = min(p.slice_blocks, nblk - my_first);
    const int nu = (my_blocks + kChunkBlocks - 1) / kChunkBlocks;
    const uint32_t r = blockIdx.y, topk = (uint32_t)g.topk, ppr = topk + 1;
    const uint32_t imax = (uint32_t)(g.inter > g.shared_inter ? g.inter : g.shared_inter);
    const uint32_t itiles = (imax + 7) / 8, ctasks = ppr * itiles;
    const uint64_t rb = p.gate_row_bytes;

    // The routing kernel runs right before this one: nothing of this row can be read earlier.
    pdl_wait();
    if (threadIdx.x < topk) {
        route->sel[threadIdx.x] = p.ws.selected[r * topk + threadIdx.x];
        route->weight[threadIdx.x] = p.ws.weights[r * topk + threadIdx.x];
    }
    __syncthreads();

    auto unit_at = [&](uint32_t ct, int ui, Unit &u) {
        if (ct >= ctasks) return false;
        const uint32_t pair = ct / itiles, i0 = (ct - pair * itiles) * 8;
        const uint32_t width = (uint32_t)(pair == topk ? g.shared_inter : g.inter);
        if (i0 >= width) return false;
        const uint8_t *pack;
        uint64_t first_row, pack_rows;
        if (pair == topk) {
            pack = static_cast<const uint8_t *>(rg == 0 ? p.w.shared_gate : p.w.shared_up);
            first_row = i0; pack_rows = g.shared_inter;
        } else {
            pack = static_cast<const uint8_t *>(rg == 0 ? p.w.gate : p.w.up);
            first_row = (uint64_t)route->sel[pair] * g.inter + i0; pack_rows = g.experts * g.inter;
        }
        u.lo = pack; u.hi = pack + pack_rows * rb;
        u.row_bytes = rb;
        u.nrows = (int)(width - i0 < 8 ? width - i0 : 8);
        u.nblocks = min(kChunkBlocks, my_blocks - ui * kChunkBlocks);
        u.src = pack + first_row * rb + (uint64_t)(my_first + ui * kChunkBlocks) * Dec::kBlockBytes;
        return true;
    };
    WarpRing<Dec> ring;
    ring.init(rings + (size_t)warp * UnitGeom<Dec>::kRingBytes, lane);
    uint32_t ict = blockIdx.x;
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
    prepare_row_half<Dec::kSumGroup>(xh, sums, p.ws.xr_h + (uint64_t)r * g.hidden, K);
    __syncthreads();
    const BLane b0 = lane_b<true>(xh, zeros, K, gi, t);

    int par = 0;
    for (uint32_t ct = blockIdx.x; ct < ctasks; ct += gridDim.x, par ^= 1) {
        float acc = 0.0f;
        for (int ui = 0; ui < nu; ++ui) {
            issue_next();
            const uint8_t *slot = ring.front();
            Unit u;
            if (unit_at(ct, ui, u)) {
                BLane b = b0;
                const int kb = my_first + ui * kChunkBlocks;
                b.p += b.stride * kb;
                acc += unit_dot<Dec, true>(slot, u, tab, b, sums + kb * UnitGeom<Dec>::kSumsPerBlock, gi, t, p.status);
            }
            ring.pop();
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (t == 0) red[(par * warps + warp) * 8 + gi] = acc;
        __syncthreads();
        if (threadIdx.x < 8) {
            const uint32_t pair = ct / itiles, i = (ct - pair * itiles) * 8 + threadIdx.x;
            const uint32_t width = (uint32_t)(pair == topk ? g.shared_inter : g.inter);
            if (i < width) {
                float gs = 0.0f, us = 0.0f;
                for (int s = 0; s < p.slices; ++s) {
                    gs += red[(par * warps + s) * 8 + threadIdx.x];
                    us += red[(par * warps + p.slices + s) * 8 + threadIdx.x];
                }
                const float v = swiglu_mid(gs, us, pair == topk ? 1.0f : route->weight[pair], (float)g.limit, p.status);
                const uint64_t at = ((uint64_t)r * ppr + pair) * imax + i;
                p.ws.mid[at] = v;
                p.ws.mid_h[at] = __float2half_rn(v);
            }
        }
    }
    // The down kernel may move in now: it reads the selection (complete before this kernel started) and
    // prefetches its experts' rows, and touches the SwiGLU rows only after this kernel has completed.
    pdl_trigger();
    cp_async_wait<0>();
}

template <class Dec>
__global__ void __launch_bounds__(512, 2) moe_down_mma_kernel(NarrowParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const MoeGeom &g = p.g;
    const int K = (int)g.inter, nblk = K / 256, warps = blockDim.x >> 5;      // inter == shared_inter on this path
    const uint32_t r = blockIdx.y, topk = (uint32_t)g.topk, ppr = topk + 1;
    MmaTables *tab = reinterpret_cast<MmaTables *>(smem);
    __half *zeros = reinterpret_cast<__half *>(smem + sizeof(MmaTables));
    __half *mids = zeros + kZeroHalves;                                         // [ppr][K]
    float *sums = reinterpret_cast<float *>(mids + (size_t)ppr * K);           // [ppr][K / sum group], packed
    const int kSumsPerRow = Dec::kSumGroup ? K / Dec::kSumGroup : 0;
    RouteSmem *route = reinterpret_cast<RouteSmem *>(sums + (size_t)ppr * (K / 16));
    float *red = reinterpret_cast<float *>(route + 1);                          // [2][kMaxPairs + 3][8]
    uint8_t *rings = smem + narrow_smem_fixed((size_t)ppr * K, (size_t)ppr * (K / 16), kMaxPairs + 3);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gi = lane >> 2, t = lane & 3;
    const int nu = (nblk + kChunkBlocks - 1) / kChunkBlocks;
    const uint32_t passes = (ppr + warps - 1) / warps;
    const uint32_t ctasks = (uint32_t)((g.hidden + 7) / 8);
    const uint64_t rb = p.down_row_bytes;

    // Read before pdl_wait(): the selection was written two kernels back, and the gate/up kernel before
    // this one lets its successor start only after it has itself waited for the routing kernel.
    if (threadIdx.x < topk) route->sel[threadIdx.x] = p.ws.selected[r * topk + threadIdx.x];
    __syncthreads();

    auto unit_at = [&](uint32_t ct, uint32_t pass, int ui, Unit &u) {
        const uint32_t pair = pass * warps + warp;
        if (ct >= ctasks || pair >= ppr) return false;
        const uint64_t h0 = (uint64_t)ct * 8;
        const uint8_t *pack;
        uint64_t first_row, pack_rows;
        if (pair == topk) {
            pack = static_cast<const uint8_t *>(p.w.shared_down);
            first_row = h0; pack_rows = g.hidden;
        } else {
            pack = static_cast<const uint8_t *>(p.w.down);
            first_row = (uint64_t)route->sel[pair] * g.hidden + h0; pack_rows = g.experts * g.hidden;
        }
        u.lo = pack; u.hi = pack + pack_rows * rb;
        u.row_bytes = rb;
        u.nrows = (int)(g.hidden - h0 < 8 ? g.hidden - h0 : 8);
        u.nblocks = min(kChunkBlocks, nblk - ui * kChunkBlocks);
        u.src = pack + first_row * rb + (uint64_t)(ui * kChunkBlocks) * Dec::kBlockBytes;
        return true;
    };
    WarpRing<Dec> ring;
    ring.init(rings + (size_t)warp * UnitGeom<Dec>::kRingBytes, lane);
    uint32_t ict = blockIdx.x, ipass = 0;
    int iui = 0;
    auto issue_next = [&]() {
        Unit u;
        const bool any = unit_at(ict, ipass, iui, u);
        ring.issue(any ? &u : nullptr);
        if (++iui >= nu) {
            iui = 0;
            if (++ipass >= passes) { ipass = 0; ict += gridDim.x; }
        }
    };
#pragma unroll
    for (int d = 0; d < kRingDepth - 1; ++d) issue_next();
    load_tables(tab, Dec::kBias);
    for (int i = threadIdx.x; i < kZeroHalves / 2; i += blockDim.x) reinterpret_cast<uint32_t *>(zeros)[i] = 0u;
    pdl_wait();                                         // the SwiGLU rows are the gate/up kernel's output
    pdl_trigger();
    // all pairs' SwiGLU rows are contiguous; with K a multiple of 256 no sum straddles two pairs
    prepare_row_half<Dec::kSumGroup>(mids, sums, p.ws.mid_h + (uint64_t)r * ppr * K, (int)(ppr * K));
    __syncthreads();

    int par = 0;
    for (uint32_t ct = blockIdx.x; ct < ctasks; ct += gridDim.x, par ^= 1) {
        for (uint32_t pass = 0; pass < passes; ++pass) {
            const uint32_t pair = pass * warps + warp;
            float acc = 0.0f;
            for (int ui = 0; ui < nu; ++ui) {
                issue_next();
                const uint8_t *slot = ring.front();
                Unit u;
                if (unit_at(ct, pass, ui, u)) {
                    BLane b = lane_b<true>(mids + (size_t)pair * K, zeros, K, gi, t);
                    b.p += b.stride * ui * kChunkBlocks;
                    acc += unit_dot<Dec, true>(slot, u, tab, b,
                                               sums + pair * kSumsPerRow + ui * kChunkBlocks * UnitGeom<Dec>::kSumsPerBlock, gi, t,
                                               p.status);
                }
                ring.pop();
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (t == 0 && pair < ppr) red[(par * (kMaxPairs + 3) + pair) * 8 + gi] = acc;
        }
        __syncthreads();
        if (threadIdx.x < 8 && (uint64_t)ct * 8 + threadIdx.x < g.hidden) {
            float routed = 0.0f;
            for (uint32_t pp = 0; pp < topk; ++pp) {
                const float y = red[(par * (kMaxPairs + 3) + pp) * 8 + threadIdx.x];
                if (!isfinite(y)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
                routed += bf16_round(y);
            }
            const float ys = red[(par * (kMaxPairs + 3) + topk) * 8 + threadIdx.x];
            if (!isfinite(ys)) raise(p.status, YVEX_B200_STATUS_NUMERIC);
            const uint64_t at = (uint64_t)r * g.hidden + (uint64_t)ct * 8 + threadIdx.x;
            p.out[at] = bf16_round(routed + bf16_round(ys));
            if (p.ws.routed_out) p.ws.routed_out[at] = routed;
            if (p.ws.shared_out) p.ws.shared_out[at] = bf16_round(ys);
        }
    }
    cp_async_wait<0>();
}

static int ctas_per_row(uint64_t rows, uint64_t tasks, int per_sm) {
    uint64_t want = ((uint64_t)kSmCount * per_sm + rows - 1) / rows;
    if (want > tasks) want = tasks;
    return (int)(want < 1 ? 1 : want);
}

template <class Dec>
static int launch_gate_up(NarrowParams &p, cudaStream_t s) {
    int rgs;
    mma_shape(p.g.hidden, p.slices, p.slice_blocks, rgs);
    const int warps = 2 * p.slices;
    const int K = (int)p.g.hidden;
    const size_t smem = narrow_smem_fixed(K, K / 16, warps) + (size_t)warps * UnitGeom<Dec>::kRingBytes;
    static SmemOptIn opt_in;
    if (opt_in.ensure(moe_gate_up_mma_kernel<Dec>, 200 * 1024) != OK) return ERR_BACKEND;
    if (smem > 200 * 1024 || warps > 16 || p.rows > 65535) return ERR_BOUNDS;
    const uint64_t imax = p.g.inter > p.g.shared_inter ? p.g.inter : p.g.shared_inter;
    const uint64_t tasks = (p.g.topk + 1) * ((imax + 7) / 8);
    dim3 grid((unsigned)ctas_per_row(p.rows, tasks, ctas_per_sm(smem, 32 * warps)), (unsigned)p.rows);
    if (launch_pdl(moe_gate_up_mma_kernel<Dec>, grid, dim3(32 * warps), smem, s, p) != cudaSuccess) return ERR_BACKEND;
    return launch_status(1);
}

template <class Dec>
static size_t down_smem(const NarrowParams &p, int warps) {
    const size_t ppr = p.g.topk + 1, K = p.g.inter;
    return narrow_smem_fixed(ppr * K, ppr * (K / 16), kMaxPairs + 3) + (size_t)warps * UnitGeom<Dec>::kRingBytes;
}

template <class Dec>
static int launch_down(NarrowParams &p, cudaStream_t s) {
    const int ppr = (int)p.g.topk + 1;
    int warps = ppr < 8 ? ppr : 8;
    while (warps > 1 && down_smem<Dec>(p, warps) > 200 * 1024) --warps;
    const size_t smem = down_smem<Dec>(p, warps);
    static SmemOptIn opt_in;
    if (opt_in.ensure(moe_down_mma_kernel<Dec>, 200 * 1024) != OK) return ERR_BACKEND;
    if (smem > 200 * 1024 || p.rows > 65535) return ERR_BOUNDS;
    p.down_warps = warps;
    const uint64_t tasks = (p.g.hidden + 7) / 8;
    dim3 grid((unsigned)ctas_per_row(p.rows, tasks, ctas_per_sm(smem, 32 * warps)), (unsigned)p.rows);
    if (launch_pdl(moe_down_mma_kernel<Dec>, grid, dim3(32 * warps), smem, s, p) != cudaSuccess) return ERR_BACKEND;
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
                        g.hidden <= (uint64_t)kMaxK && g.topk + 1 <= (uint64_t)kMaxPairs &&
                        aligned_for(g.gate_qtype, w.gate) && aligned_for(g.gate_qtype, w.up) &&
                        aligned_for(g.gate_qtype, w.shared_gate) && aligned_for(g.gate_qtype, w.shared_up);
    if (up_mma) {
        rc = g.gate_qtype == Q_IQ2_XXS ? launch_gate_up<Iq2Decoder>(p, s)
             : g.gate_qtype == Q_Q4_K  ? launch_gate_up<Q4kDecoder>(p, s)
                                       : launch_gate_up<Q2kDecoder>(p, s);
        if (rc == ERR_BOUNDS) rc = moe_up_rows(g, w, ws, rows, status, s);
    } else {
        rc = moe_up_rows(g, w, ws, rows, status, s);
    }
    if (rc != OK) return rc;
    mark_phase(2, s);
    const bool down_mma = mma_decoder_for(g.down_qtype) && g.inter == g.shared_inter && g.inter % 256 == 0 &&
                          g.inter <= (uint64_t)kMaxK && g.topk + 1 <= (uint64_t)kMaxPairs &&
                          aligned_for(g.down_qtype, w.down) && aligned_for(g.down_qtype, w.shared_down);
    if (down_mma) {
        rc = g.down_qtype == Q_IQ2_XXS ? launch_down<Iq2Decoder>(p, s)
             : g.down_qtype == Q_Q4_K  ? launch_down<Q4kDecoder>(p, s)
                                       : launch_down<Q2kDecoder>(p, s);
        if (rc == ERR_BOUNDS) rc = moe_down_rows(g, w, ws, rows, out, status, s);
    } else {
        rc = moe_down_rows(g, w, ws, rows, out, status, s);
    }
    mark_phase(3, s);
    return rc;
}

}  // namespace yb
