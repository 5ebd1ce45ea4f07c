// Decode-time expert execution on the streaming matvec: the (k + 1) experts of every row are run as
// TWO batched launches of gemv_stream_kernel (gate and up of every active expert, then down), each a
// persistent kernel that streams the selected experts' weight rows through shared memory once, found
// through a device table of matrix addresses built from the router's selection (by the router's top-k
// kernel itself at decode width, else by decode_tables_kernel). SwiGLU * route weight -> bf16
// (src/graph/moe.c:605-613) is applied by the down launch while it prepares its input rows; one small
// kernel sums the per-pair bf16 rows in rank order, adds the shared expert's and rounds
// (src/runtime/moe.c:606-637).
#include "gemv_stream.cuh"
#include "moe_common.cuh"

namespace yb {

// Scratch behind the MoE workspace's fixed part (narrow batches only).
uint64_t moe_decode_stream_layout(const MoeGeom &g, uint64_t rows, uint64_t base, DecodeStreamScratch *out) {
    uint64_t off = base;
    auto take = [&](uint64_t bytes) { uint64_t at = off; off = (off + bytes + 255) & ~255ull; return at; };
    const uint64_t pairs = rows * (g.topk + 1), imax = g.inter > g.shared_inter ? g.inter : g.shared_inter;
    DecodeStreamScratch l;
    l.gu_ptrs = reinterpret_cast<const uint8_t **>(take(pairs * 2 * sizeof(void *)));
    l.down_ptrs = reinterpret_cast<const uint8_t **>(take(pairs * sizeof(void *)));
    l.gu_rows = reinterpret_cast<uint32_t *>(take(pairs * 2 * sizeof(uint32_t)));
    l.gu = reinterpret_cast<float *>(take(pairs * 2 * imax * 4));
    l.y = reinterpret_cast<float *>(take(pairs * g.hidden * 4));
    l.pair_weight = reinterpret_cast<float *>(take(pairs * 4));
    if (out) *out = l;
    return off;
}

bool moe_decode_stream_eligible(const MoeGeom &g, const MoeWeights &w) {
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
    if (g.gate_qtype != g.up_qtype || !gs::stream_qtype(g.gate_qtype) || !gs::stream_qtype(g.down_qtype)) return false;
    if (g.inter != g.shared_inter || g.hidden % 256 || g.inter % 256) return false;
    const uint64_t grb = g.hidden / gg.elems * gg.bytes, drb = g.inter / dg.elems * dg.bytes;
    gs::StreamShape sh;
    if (!gs::stream_shape(g.gate_qtype, g.hidden, grb, sh) || !gs::stream_shape(g.down_qtype, g.inter, drb, sh))
        return false;
    const uintptr_t ptrs = (uintptr_t)w.gate | (uintptr_t)w.up | (uintptr_t)w.down | (uintptr_t)w.shared_gate |
                           (uintptr_t)w.shared_up | (uintptr_t)w.shared_down;
    // every expert's matrix starts on a 16-byte boundary
    return (ptrs & 15u) == 0 && (g.inter * grb) % 16 == 0 && (g.hidden * drb) % 16 == 0;
}

// pair q = row * (k + 1) + p: p < k the routed expert selected[row][p], p == k the shared expert
__global__ void decode_tables_kernel(MoeGeom g, RouteTables rt, const int32_t *selected, const float *weights, uint64_t rows, int *status) {
    const uint64_t ppr = g.topk + 1, pairs = rows * ppr;
    for (uint64_t q = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; q < pairs; q += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = q / ppr, p = q % ppr;
        const bool shared = p == g.topk;
        int64_t e = shared ? 0 : selected[r * g.topk + p];
        if (e < 0 || (uint64_t)e >= g.experts) { raise(status, YVEX_B200_STATUS_ARGUMENT); e = 0; }
        write_pair_tables(rt, q, (uint32_t)r, shared, e, shared ? 1.0f : weights[r * g.topk + p]);
    }
}

__global__ void decode_combine_kernel(MoeGeom g, const float *y, uint64_t rows, float *out, float *routed_out, float *shared_out) {
    const uint64_t ppr = g.topk + 1, total = rows * g.hidden;
    pdl_wait();                                              // y comes from the launch before
    pdl_trigger();
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / g.hidden, h = i % g.hidden;
        float routed = 0.0f;
        for (uint64_t p = 0; p < g.topk; ++p) routed += y[(r * ppr + p) * g.hidden + h];          // rank order
        const float shared = y[(r * ppr + g.topk) * g.hidden + h];
        out[i] = bf16_round(routed + shared);
        if (routed_out) routed_out[i] = routed;
        if (shared_out) shared_out[i] = shared;
    }
}

int moe_experts_stream(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, const DecodeStreamScratch &t, bool tables_ready,
                       uint64_t rows, float *out, int *status, cudaStream_t s) {
    const Geometry gg = geometry_of(g.gate_qtype), dg = geometry_of(g.down_qtype);
    const uint64_t grb = g.hidden / gg.elems * gg.bytes, drb = g.inter / dg.elems * dg.bytes;
    const uint64_t pairs = rows * (g.topk + 1), imax = g.inter;
    int rc;
    if (!tables_ready) {
        RouteTables rt{};
        rt.w = w; rt.gate_bytes = g.inter * grb; rt.down_bytes = g.hidden * drb; rt.t = t; rt.enabled = 1;
        decode_tables_kernel<<<grid_for(pairs, 128, 1), 128, 0, s>>>(g, rt, ws.selected, ws.weights, rows, status);
        rc = launch_status(1);
        if (rc != OK) return rc;
    }
    rc = gs::stream_launch(g.gate_qtype, nullptr, 0, pairs * 2, g.inter, g.hidden, grb, ws.xr, g.hidden, nullptr, t.gu, imax, 0, status, s,
                           t.gu_ptrs, t.gu_rows);
    if (rc != OK) return rc;
    mark_phase(2, s);
    // input row of pair q = bf16(SwiGLU(gate row, up row) * route weight), formed while the launch prepares its activation planes
    gs::StreamActivation act{t.gu + imax, t.pair_weight, (float)g.limit};
    rc = gs::stream_launch(g.down_qtype, nullptr, 0, pairs, g.hidden, g.inter, drb, t.gu, 2 * imax, nullptr, t.y, g.hidden, 1, status, s,
                           t.down_ptrs, nullptr, &act);
    if (rc != OK) return rc;
    if (launch_pdl(decode_combine_kernel, dim3(grid_for(rows * g.hidden, 256, 8)), dim3(256), 0, s, g, (const float *)t.y, rows, out, ws.routed_out,
                   ws.shared_out) != cudaSuccess)
        return ERR_BACKEND;
    mark_phase(3, s);
    return launch_status(1);
}

}  // namespace yb
