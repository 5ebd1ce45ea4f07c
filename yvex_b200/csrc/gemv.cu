// Dequant kernels for encoded rows: the bit-exact row decoder and the dequant-fused matvec.
//
// Two matvec paths:
//   * gemv_rows_kernel  - any supported qtype, one warp per output row, f32 FMA. Used for the
//     scalar qtypes (router weights are F32) and as the reference-shaped fallback.
//   * gemv_mma_kernel   - the streaming path for block qtypes (gemv_mma.cuh): every warp stages
//     its rows into shared memory with 16-byte cp.async copies, decodes them to exact
//     small-integer fp16 fragments and multiplies them on the tensor cores against a 3-way fp16
//     split of the f32 activation, with the per-superblock f16 scale applied to the drained
//     accumulator.
#include "gemv_mma.cuh"
#include "qtype_decode.cuh"

namespace yb {

// ---- elementwise decode (reference: yvex_encoded_row_decode, src/backend/cuda/kernels.cu:784) ----
__global__ void dequant_rows_kernel(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width,
                                    uint64_t row_bytes, float *out, int *status) {
    const Geometry g = geometry_of(q);
    const uint64_t total = rows * width;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = i / width, c = i % width;
        const uint8_t *blk = enc + r * row_bytes + (c / g.elems) * g.bytes;
        float v = decode_element(q, blk, static_cast<unsigned>(c % g.elems), status);
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[i] = v;
    }
}

// ---- generic matvec: warp per (input row, output row) ----------------------------------------
__global__ void gemv_rows_kernel(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width,
                                 uint64_t row_bytes, const float *input, uint64_t input_rows,
                                 const float *additive, float *out, int round_bf16, int *status) {
    const Geometry g = geometry_of(q);
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t job = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
         job < rows * input_rows; job += warps) {
        const uint64_t r = job % rows, in = job / rows;
        const uint8_t *row = enc + r * row_bytes;
        const float *x = input + in * width;
        float acc = 0.0f;
        for (uint64_t c = lane; c < width; c += 32) {
            float w = decode_element(q, row + (c / g.elems) * g.bytes,
                                     static_cast<unsigned>(c % g.elems), status);
            acc = fmaf(w, __ldg(x + c), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (additive) acc += additive[job];
            if (!isfinite(acc)) raise(status, YVEX_B200_STATUS_NUMERIC);
            out[job] = round_bf16 ? bf16_round(acc) : acc;
        }
    }
}

}  // namespace yb

using namespace yb;

extern "C" int yvex_b200_dequant_rows(unsigned int qtype, const void *encoded, uint64_t rows,
                                      uint64_t width, uint64_t row_bytes, float *out, int *status,
                                      void *stream) {
    if (!encoded || !out || !status) return ERR_INVALID_ARG;
    int rc = check_rows(qtype, rows, width, row_bytes);
    if (rc != OK) return rc;
    uint64_t total = rows * width;
    int grid = (int)((total + 255) / 256 < (uint64_t)kSmCount * 16 ? (total + 255) / 256
                                                                     : (uint64_t)kSmCount * 16);
    dequant_rows_kernel<<<grid, 256, 0, as_stream(stream)>>>(
        qtype, static_cast<const uint8_t *>(encoded), rows, width, row_bytes, out, status);
    return launch_status();
}

extern "C" int yvex_b200_gemv(unsigned int qtype, const void *encoded, uint64_t rows,
                              uint64_t width, uint64_t row_bytes, const float *input,
                              uint64_t input_rows, const float *additive, float *out,
                              int round_bf16, int *status, void *stream) {
    if (!encoded || !input || !out || !status || !input_rows) return ERR_INVALID_ARG;
    int rc = check_rows(qtype, rows, width, row_bytes);
    if (rc != OK) return rc;
    const uint8_t *enc = static_cast<const uint8_t *>(encoded);
    if (gemv_mma_eligible(qtype, rows, width, enc) &&
        (reinterpret_cast<uintptr_t>(input) & 15u) == 0) {
        return gemv_mma_launch(qtype, enc, rows, width, row_bytes, input, input_rows, additive, out, round_bf16, status,
                               as_stream(stream));
    }
    uint64_t jobs = rows * input_rows;
    int grid = (int)((jobs + 7) / 8 < (uint64_t)kSmCount * 8 ? (jobs + 7) / 8
                                                              : (uint64_t)kSmCount * 8);
    gemv_rows_kernel<<<grid, 256, 0, as_stream(stream)>>>(qtype, enc, rows, width, row_bytes, input,
                                                          input_rows, additive, out, round_bf16,
                                                          status);
    return launch_status();
}
