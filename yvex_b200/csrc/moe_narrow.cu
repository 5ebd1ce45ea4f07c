// Narrow-batch (decode) expert execution: dispatch between the streaming tensor-core matvec
// kernels and the reference-shaped per-row kernels.
#include "moe_common.cuh"

namespace yb {

int moe_experts_narrow(const MoeGeom &g, const MoeWeights &w, const MoeWorkspace &ws, uint64_t rows,
                       float *out, int *status, cudaStream_t s) {
    return moe_experts_rows(g, w, ws, rows, out, status, s);
}

}  // namespace yb
