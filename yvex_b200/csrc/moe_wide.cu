// Wide-batch (prefill / expert-parallel shard) MoE layer.
#include "moe_common.cuh"

using namespace yb;

extern "C" int yvex_b200_moe_wide(const yvex_b200_moe_geometry *geom, const yvex_b200_moe_weights *w,
                                  const float *x, const float *logits, const uint32_t *token_ids,
                                  uint64_t rows, float *out, int32_t *selected_out, float *weights_out,
                                  void *workspace, uint64_t workspace_bytes, int *status, void *stream) {
    int rc = moe_check_geometry(geom, w);
    if (rc != OK) return rc;
    if (!x || !out || !status || !rows) return ERR_INVALID_ARG;
    MoeGeom g = *geom;
    MoeWorkspace ws;
    if (!workspace || workspace_bytes < moe_workspace_layout(g, rows, &ws)) return ERR_NOMEM;
    ws.rebase(workspace);
    cudaStream_t s = as_stream(stream);
    mark_phase(0, s);
    rc = moe_ingress_and_route(g, *w, ws, x, logits, token_ids, rows, status, s);
    if (rc != OK) return rc;
    mark_phase(1, s);
    rc = moe_experts_rows(g, *w, ws, rows, out, status, s);
    if (rc != OK) return rc;
    if (selected_out) cudaMemcpyAsync(selected_out, ws.selected, rows * g.topk * sizeof(int32_t), cudaMemcpyDeviceToDevice, s);
    if (weights_out) cudaMemcpyAsync(weights_out, ws.weights, rows * g.topk * sizeof(float), cudaMemcpyDeviceToDevice, s);
    return launch_status(0);
}
