// Dequant kernels for encoded rows: the bit-exact row decoder and the dequant-fused matvec.
//
// Three matvec paths:
//   * gemv_rows_kernel  - any supported qtype, one warp per output row, f32 FMA. Used for the
//     scalar qtypes (router weights are F32) and for shapes the other two do not take.
//   * gemv_q8_0_kernel  - Q8_0 rows streamed through shared memory by bulk copies, f32 FMA.
//   * gemv_mma_kernel   - the streaming path for block qtypes (gemv_mma.cuh): every warp stages
//     its rows into shared memory with 16-byte cp.async copies, decodes them to exact
//     small-integer fp16 fragments and multiplies them on the tensor cores against a 3-way fp16
//     split of the f32 activation, with the per-superblock f16 scale applied to the drained
//     accumulator.
#include "gemv_mma.cuh"
#include "gemv_stream.cuh"
#include "qtype_decode.cuh"
#include "tcgen05.cuh"

namespace yb {

// ---- elementwise decode (reference: yvex_encoded_row_decode, src/backend/cuda/kernels.cu:784) ----
// row_ids (optional): output row r decodes matrix row row_ids[r] (yvex_qtype_gather, the decode of selected
// rows behind yvex_backend_cuda_encoded_gather, src/backend/cuda/qtype.c:404-520); `matrix_rows` bounds the ids.
__global__ void dequant_rows_kernel(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width,
                                    uint64_t row_bytes, const uint32_t *row_ids, uint64_t matrix_rows, float *out, int *status) {
    const Geometry g = geometry_of(q);
    const uint64_t total = rows * width;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t r = i / width, c = i % width;
        if (row_ids) {
            r = row_ids[r];
            if (r >= matrix_rows) { raise(status, YVEX_B200_STATUS_ARGUMENT); continue; }
        }
        const uint8_t *blk = enc + r * row_bytes + (c / g.elems) * g.bytes;
        float v = decode_element(q, blk, static_cast<unsigned>(c % g.elems), status);
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[i] = v;
    }
}

// ---- activation preparation ---------------------------------------------------------------------
// Q8_K round trip of an activation row, one warp per 256-value block: the element of largest magnitude
// (the first of equals) sets inverse = -127 / value, every element becomes rint(inverse * x) clamped to
// [-128, 127] and is published as that integer / inverse. These are the values the reference's Q8_K
// activation path multiplies the weights by (quantiser src/backend/cuda/kernels.cu:436-489; the
// definition its own test restates, tests/unit/cuda/quant_qtype.c:161-186).
__global__ void __launch_bounds__(256) q8k_round_trip_kernel(const float *x, uint64_t blocks, float *out, int *status) {
    const int lane = threadIdx.x & 31;
    for (uint64_t b = blockIdx.x * (uint64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); b < blocks; b += (uint64_t)gridDim.x * (blockDim.x >> 5)) {
        const float4 lo = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + 2 * lane), hi = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + 2 * lane + 1);
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float best = 0.0f, best_signed = 0.0f;
        int best_at = 0;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            bad |= !isfinite(v[i]);
            if (fabsf(v[i]) > best) { best = fabsf(v[i]); best_signed = v[i]; best_at = 8 * lane + i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, best_signed, o);
            const int oa = __shfl_xor_sync(0xffffffffu, best_at, o);
            if (ob > best || (ob == best && oa < best_at)) { best = ob; best_signed = os; best_at = oa; }
        }
        if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
        const float inverse = best == 0.0f ? 0.0f : -127.0f / best_signed;
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = inverse == 0.0f ? 0 : __float2int_rn(inverse * v[i]);
            q = q > 127 ? 127 : q < -128 ? -128 : q;
            r[i] = inverse == 0.0f ? 0.0f : (float)q / inverse;
        }
        float4 *dst = reinterpret_cast<float4 *>(out + b * 256) + 2 * lane;
        dst[0] = make_float4(r[0], r[1], r[2], r[3]);
        dst[1] = make_float4(r[4], r[5], r[6], r[7]);
    }
}

// A row given in two parts (head_width values, then the rest) as one bf16-rounded row: what the
// reference's split-input matvec multiplies by (yvex_qtype_split_matvec, src/backend/cuda/kernels.cu:736-781).
__global__ void concat_bf16_kernel(const float *head, const float *tail, uint64_t head_width, uint64_t width, uint64_t rows,
                                   float *out, int *status) {
    const uint64_t total = rows * width, tail_width = width - head_width;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = i / width, c = i % width;
        const float v = c < head_width ? head[r * head_width + c] : tail[r * tail_width + (c - head_width)];
        if (!isfinite(v)) raise(status, YVEX_B200_STATUS_NUMERIC);
        out[i] = bf16_round(v);
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

// ---- scalar-qtype matvec: F32 / F16 / BF16 rows streamed with 16-byte loads ---------------------------
// The output-head projection of the reference model is such a matrix (BF16 rows, about 1 GB per call,
// src/runtime/logits.c:644-649): pure streaming, one warp per row, the activation row in shared
// memory, every lane four independent 16-byte loads ahead of its multiply-adds.
template <unsigned kQ> __device__ __forceinline__ void dense_chunk(const uint4 v, const float *xs, float &acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (kQ == Q_F32) {
        const float4 xv = *reinterpret_cast<const float4 *>(xs);
        acc = fmaf(__uint_as_float(w[0]), xv.x, acc); acc = fmaf(__uint_as_float(w[1]), xv.y, acc);
        acc = fmaf(__uint_as_float(w[2]), xv.z, acc); acc = fmaf(__uint_as_float(w[3]), xv.w, acc);
    } else {
        const float4 x0 = reinterpret_cast<const float4 *>(xs)[0], x1 = reinterpret_cast<const float4 *>(xs)[1];
        const float xe[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            if (kQ == Q_BF16) { lo = __uint_as_float(w[i] << 16); hi = __uint_as_float(w[i] & 0xffff0000u); }
            else { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i])); lo = f.x; hi = f.y; }
            acc = fmaf(lo, xe[2 * i], acc);
            acc = fmaf(hi, xe[2 * i + 1], acc);
        }
    }
}

template <unsigned kQ>
__global__ void __launch_bounds__(512) gemv_dense_kernel(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes,
                                                         const float *input, const float *additive, float *out, int round_bf16,
                                                         int *status) {
    extern __shared__ __align__(16) float dense_x[];
    constexpr int kPer = kQ == Q_F32 ? 4 : 8;                               // elements per 16-byte chunk
    const float *x = input + (uint64_t)blockIdx.y * width;
    bool bad = false;
    for (uint32_t i = threadIdx.x; i < (uint32_t)width; i += blockDim.x) { const float v = __ldg(x + i); bad |= !isfinite(v); dense_x[i] = v; }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const uint32_t chunks = (uint32_t)(row_bytes / 16);
    for (uint64_t r = (uint64_t)blockIdx.x * warps + warp; r < rows; r += (uint64_t)gridDim.x * warps) {
        const uint4 *rp = reinterpret_cast<const uint4 *>(enc + r * row_bytes);
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        uint32_t c = lane;
        for (; c + 96 < chunks; c += 128) {
            const uint4 v0 = __ldcs(rp + c), v1 = __ldcs(rp + c + 32), v2 = __ldcs(rp + c + 64), v3 = __ldcs(rp + c + 96);
            dense_chunk<kQ>(v0, dense_x + (size_t)c * kPer, a0);
            dense_chunk<kQ>(v1, dense_x + (size_t)(c + 32) * kPer, a1);
            dense_chunk<kQ>(v2, dense_x + (size_t)(c + 64) * kPer, a2);
            dense_chunk<kQ>(v3, dense_x + (size_t)(c + 96) * kPer, a3);
        }
        for (; c < chunks; c += 32) dense_chunk<kQ>(__ldcs(rp + c), dense_x + (size_t)c * kPer, a0);
        float acc = warp_sum((a0 + a1) + (a2 + a3));
        if (lane == 0) {
            const uint64_t job = (uint64_t)blockIdx.y * rows + r;
            if (additive) acc += additive[job];
            if (!isfinite(acc)) bad = true;
            out[job] = round_bf16 ? bf16_round(acc) : acc;
        }
    }
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
}

static bool gemv_dense_eligible(unsigned q, uint64_t width, uint64_t row_bytes, const uint8_t *enc, const float *input, uint64_t input_rows) {
    return (q == Q_F32 || q == Q_F16 || q == Q_BF16) && row_bytes % 16 == 0 && width * 4 <= 48 * 1024 && input_rows <= 65535 &&
           ((reinterpret_cast<uintptr_t>(enc) | reinterpret_cast<uintptr_t>(input)) & 15u) == 0 && (width * 4) % 16 == 0;
}

static int gemv_dense_launch(unsigned q, const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes, const float *input,
                             uint64_t input_rows, const float *additive, float *out, int round_bf16, int *status, cudaStream_t s) {
    const uint64_t want = (rows + 15) / 16, cap = (uint64_t)kSmCount * 4;
    const dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)input_rows);
    const size_t smem = width * 4;
    if (q == Q_F32) gemv_dense_kernel<Q_F32><<<grid, 512, smem, s>>>(enc, rows, width, row_bytes, input, additive, out, round_bf16, status);
    else if (q == Q_F16) gemv_dense_kernel<Q_F16><<<grid, 512, smem, s>>>(enc, rows, width, row_bytes, input, additive, out, round_bf16, status);
    else gemv_dense_kernel<Q_BF16><<<grid, 512, smem, s>>>(enc, rows, width, row_bytes, input, additive, out, round_bf16, status);
    return launch_status();
}

// ---- Q8_0 streaming matvec ------------------------------------------------------------------------
// A Q8_0 row is a run of 34-byte blocks (f16 d, 32 int8), so neither the blocks nor the quants are
// 4-byte aligned and a thread-per-block global load touches 17 cache lines per instruction. A CTA
// therefore streams groups of eight consecutive rows (two warps per row, alternating 32-block
// segments; the pair meets on a named barrier and adds its two partial sums) through a two-stage ring in
// shared memory, each stage filled by ONE bulk copy that completes on an mbarrier (many small
// copies are bound by the copy engine's per-copy cost, not by bytes); lane b of a warp decodes
// block 32*s + b of its row from shared memory (nine 4-byte reads, a 16-bit funnel shift for the
// even blocks) and multiplies it with its 32 activations, which sit in shared memory as
// [element / 4][block] float4 so that the lanes read consecutive 16-byte slots. int8 -> f32 goes
// through the 2^23 trick (XOR 0x80, PRMT into the mantissa, subtract 2^23 + 128): exact, and on
// the ALU and FMA pipes instead of the conversion unit. d multiplies the block's f32 sum once.
constexpr int kQ8Rows = 8, kQ8Split = 2, kQ8Warps = kQ8Rows * kQ8Split, kQ8Depth = 2;

struct Q8Ctl { uint64_t full[kQ8Depth], empty[kQ8Depth]; int abort; int pad[3]; float part[2][kQ8Rows][kQ8Split]; };

__global__ void __launch_bounds__(32 * kQ8Warps)
gemv_q8_0_kernel(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes, const float *input,
                 const float *additive, float *out, int round_bf16, int *status) {
    using namespace sm100;
    extern __shared__ __align__(128) uint8_t q8_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nblk = (uint32_t)(width / 32), nseg = (nblk + 31) / 32;
    const uint32_t stage_bytes = (uint32_t)(kQ8Rows * row_bytes);
    const int rw = warp / kQ8Split, half = warp % kQ8Split;                  // row of the group, share of its segments
    uint8_t *ring = q8_smem;                                                  // [kQ8Depth][8 rows][row_bytes]
    Q8Ctl *ctl = reinterpret_cast<Q8Ctl *>(q8_smem + (size_t)kQ8Depth * stage_bytes);
    float4 *xs = reinterpret_cast<float4 *>(ctl + 1);                        // [8][nblk]
    const float *x = input + (uint64_t)blockIdx.y * width;
    const uint64_t groups = (rows + kQ8Rows - 1) / kQ8Rows;
    const uint64_t mine = groups > blockIdx.x ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    auto issue = [&](uint64_t n) {                                           // thread 0 only: group n of this CTA
        const uint64_t row0 = (blockIdx.x + n * gridDim.x) * kQ8Rows;
        const uint32_t bytes = (uint32_t)(min((uint64_t)kQ8Rows, rows - row0) * row_bytes);
        mbar_expect_tx(&ctl->full[n % kQ8Depth], bytes);
        bulk_load(ring + (n % kQ8Depth) * stage_bytes, enc + row0 * row_bytes, bytes, &ctl->full[n % kQ8Depth]);
    };
    uint64_t issued = 0, done = 0;                                         // thread 0: stages requested / consumed
    // programmatic dependent launch, as in gemv_mma_kernel: only the encoded rows are touched before the wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        for (int i = 0; i < kQ8Depth; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], kQ8Warps); }
        ctl->abort = 0;
        fence_barrier_init();
        for (uint64_t n = 0; n < mine && n < (uint64_t)kQ8Depth; ++n) { issue(n); issued = n + 1; }
    }
    // the activation row goes to shared memory while the first stages are in flight
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t i = threadIdx.x; i < (uint32_t)width; i += blockDim.x) {
        const uint32_t b = i >> 5, e = i & 31u;
        reinterpret_cast<float *>(xs + (e >> 2) * nblk + b)[e & 3u] = __ldg(x + i);
    }
    __syncthreads();
    bool bad = false;
    for (uint64_t n = 0; n < mine; ++n) {
        const uint32_t slot = (uint32_t)(n % kQ8Depth), ph = (uint32_t)((n / kQ8Depth) & 1u);
        // Every thread of the CTA takes the same way out: a warp that left alone would leave its row
        // partner at the pair barrier below, and lanes that left alone would break the warp shuffles.
        const bool landed = mbar_wait<kTryWaitHintNs>(&ctl->full[slot], ph, &ctl->abort) && !ctl->abort;
        if (!__syncthreads_and(landed)) break;
        const uint64_t r = (blockIdx.x + n * gridDim.x) * kQ8Rows + rw;
        if (r < rows) {                                                       // uniform over the row's warp pair
            const uint32_t *row = reinterpret_cast<const uint32_t *>(ring + slot * stage_bytes + rw * row_bytes);
            const bool odd = lane & 1;
            float acc = 0.0f;
            for (uint32_t sgm = half; sgm < nseg; sgm += kQ8Split) {
                const uint32_t blk = 32u * sgm + lane;
                if (blk < nblk) {
                    // block `blk` starts at byte 34*blk: word 17m for block 2m, the upper half of word 17m + 8 for 2m + 1
                    const uint32_t *wp = row + ((34u * blk) >> 2);
                    uint32_t w[9];
#pragma unroll
                    for (int k = 0; k < 9; ++k) w[k] = wp[k];
                    const float d = f16_bits_to_float((uint16_t)(odd ? w[0] >> 16 : w[0]));
                    bad |= !isfinite(d);
                    const float4 *xb = xs + blk;
                    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;          // four chains instead of one of 32 FMAs
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t q = __funnelshift_r(odd ? w[k + 1] : w[k], w[k + 1], odd ? 0u : 16u) ^ 0x80808080u;
                        const float4 xv = xb[k * nblk];
                        constexpr float kBias = 8388608.0f + 128.0f;
                        s0 = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7540)) - kBias, xv.x, s0);
                        s1 = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7541)) - kBias, xv.y, s1);
                        s2 = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7542)) - kBias, xv.z, s2);
                        s3 = fmaf(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7543)) - kBias, xv.w, s3);
                    }
                    acc = fmaf(d, (s0 + s1) + (s2 + s3), acc);
                }
            }
            acc = warp_sum(acc);
            if (lane == 0) ctl->part[n & 1][rw][half] = acc;
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rw), "r"(32 * kQ8Split) : "memory");     // the row's warps
            if (lane == 0 && half == 0) {
                float total = 0.0f;
#pragma unroll
                for (int h = 0; h < kQ8Split; ++h) total += ctl->part[n & 1][rw][h];     // fixed order
                const uint64_t job = (uint64_t)blockIdx.y * rows + r;
                if (additive) total += additive[job];
                if (!isfinite(total)) bad = true;
                out[job] = round_bf16 ? bf16_round(total) : total;
            }
        }
        // the stage is refilled by the async proxy: order this warp's reads before that write
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->empty[slot]);
        if (threadIdx.x == 0 && n + kQ8Depth < mine) {
            // every warp is done with the stage; when this wait runs out the abort flag is up and the
            // whole CTA leaves together at the top of the next iteration
            if (mbar_wait<kTryWaitHintNs>(&ctl->empty[slot], ph, &ctl->abort)) { issue(n + kQ8Depth); issued = n + kQ8Depth + 1; }
        }
        done = n + 1;
    }
    if (threadIdx.x == 0 && ctl->abort) {
        // copies still in flight land in this CTA's shared memory: give them a bounded time to finish
        int ignore = 0;
        for (uint64_t m = done; m < issued; ++m) mbar_wait<kTryWaitHintNs>(&ctl->full[m % kQ8Depth], (uint32_t)((m / kQ8Depth) & 1u), &ignore);
    }
    if (bad) raise(status, YVEX_B200_STATUS_NUMERIC);
    if (lane == 0 && ctl->abort) raise(status, YVEX_B200_STATUS_TIMEOUT);
}

static size_t q8_smem_bytes(uint64_t width, uint64_t row_bytes) {
    return (size_t)kQ8Depth * kQ8Warps * row_bytes + sizeof(Q8Ctl) + (size_t)width * 4;
}

// The streaming kernel wants 16-byte aligned rows (width a multiple of 256 gives that) and two
// stages of eight rows plus the activation row in shared memory.
static bool gemv_q8_0_eligible(unsigned q, uint64_t width, uint64_t row_bytes, const uint8_t *enc) {
    return q == Q_Q8_0 && width % 256 == 0 && row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(enc) & 15u) == 0 &&
           q8_smem_bytes(width, row_bytes) <= 200 * 1024;
}

static int gemv_q8_0_launch(const uint8_t *enc, uint64_t rows, uint64_t width, uint64_t row_bytes, const float *input,
                            uint64_t input_rows, const float *additive, float *out, int round_bf16, int *status,
                            cudaStream_t s) {
    const size_t smem = q8_smem_bytes(width, row_bytes);
    static SmemOptIn opt_in;
    if (opt_in.ensure(gemv_q8_0_kernel, 200 * 1024) != OK) return ERR_BACKEND;
    const uint64_t groups = (rows + kQ8Warps - 1) / kQ8Warps, per_sm = (227 * 1024) / (smem + 1024);
    const uint64_t cap = (uint64_t)kSmCount * (per_sm < 1 ? 1 : per_sm > 2 ? 2 : per_sm);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(groups < cap ? groups : cap), (unsigned)input_rows);
    cfg.blockDim = dim3(32 * kQ8Warps); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, gemv_q8_0_kernel, enc, rows, width, row_bytes, input, additive, out, round_bf16, status) != cudaSuccess)
        return ERR_BACKEND;
    return launch_status();
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
        qtype, static_cast<const uint8_t *>(encoded), rows, width, row_bytes, nullptr, rows, out, status);
    return launch_status();
}

extern "C" int yvex_b200_dequant_gather(unsigned int qtype, const void *encoded, uint64_t rows, uint64_t width, uint64_t row_bytes,
                                        const uint32_t *row_ids, uint64_t selected_rows, float *out, int *status, void *stream) {
    if (!encoded || !out || !status || !row_ids || !selected_rows) return ERR_INVALID_ARG;
    int rc = check_rows(qtype, rows, width, row_bytes);
    if (rc != OK) return rc;
    dequant_rows_kernel<<<grid_for(selected_rows * width, 256, 16), 256, 0, as_stream(stream)>>>(
        qtype, static_cast<const uint8_t *>(encoded), selected_rows, width, row_bytes, row_ids, rows, out, status);
    return launch_status();
}

extern "C" int yvex_b200_q8k_round_trip(const float *x, uint64_t rows, uint64_t width, float *out, int *status, void *stream) {
    if (!x || !out || !status || !rows || !width) return ERR_INVALID_ARG;
    if (width % 256 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u)) return ERR_BOUNDS;
    const uint64_t blocks = rows * (width / 256);
    q8k_round_trip_kernel<<<grid_for(blocks, 8, 16), 256, 0, as_stream(stream)>>>(x, blocks, out, status);
    return launch_status();
}

extern "C" int yvex_b200_concat_bf16(const float *head, const float *tail, uint64_t head_width, uint64_t width, uint64_t rows,
                                     float *out, int *status, void *stream) {
    if (!head || !tail || !out || !status || !rows) return ERR_INVALID_ARG;
    if (!head_width || head_width >= width) return ERR_BOUNDS;
    concat_bf16_kernel<<<grid_for(rows * width, 256, 16), 256, 0, as_stream(stream)>>>(head, tail, head_width, width, rows, out, status);
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
    // input rows are a batch that shares one matrix
    if (gs::stream_eligible(qtype, rows, width, row_bytes, enc, 0, input_rows, input, width))
        return gs::stream_launch(qtype, enc, 0, input_rows, rows, width, row_bytes, input, width, additive, out, rows, round_bf16, status,
                                 as_stream(stream));
    if (gemv_mma_eligible(qtype, rows, width, enc) &&
        (reinterpret_cast<uintptr_t>(input) & 15u) == 0) {
        return gemv_mma_launch(qtype, enc, rows, width, row_bytes, input, input_rows, additive, out, round_bf16, status,
                               as_stream(stream));
    }
    if (gemv_dense_eligible(qtype, width, row_bytes, enc, input, input_rows))
        return gemv_dense_launch(qtype, enc, rows, width, row_bytes, input, input_rows, additive, out, round_bf16, status, as_stream(stream));
    if (gemv_q8_0_eligible(qtype, width, row_bytes, enc) && input_rows <= 65535)
        return gemv_q8_0_launch(enc, rows, width, row_bytes, input, input_rows, additive, out, round_bf16, status, as_stream(stream));
    uint64_t jobs = rows * input_rows;
    int grid = (int)((jobs + 7) / 8 < (uint64_t)kSmCount * 8 ? (jobs + 7) / 8
                                                              : (uint64_t)kSmCount * 8);
    gemv_rows_kernel<<<grid, 256, 0, as_stream(stream)>>>(qtype, enc, rows, width, row_bytes, input,
                                                          input_rows, additive, out, round_bf16,
                                                          status);
    return launch_status();
}

extern "C" int yvex_b200_gemv_batch(unsigned int qtype, const void *encoded, uint64_t matrix_stride, uint64_t count,
                                    uint64_t rows, uint64_t width, uint64_t row_bytes, const float *input,
                                    uint64_t input_stride, const float *additive, float *out, uint64_t out_stride,
                                    int round_bf16, int *status, void *stream) {
    if (!encoded || !input || !out || !status || !count) return ERR_INVALID_ARG;
    int rc = check_rows(qtype, rows, width, row_bytes);
    if (rc != OK) return rc;
    if (input_stride < width || out_stride < rows || (count > 1 && matrix_stride < rows * row_bytes)) return ERR_BOUNDS;
    const uint8_t *enc = static_cast<const uint8_t *>(encoded);
    if (gs::stream_eligible(qtype, rows, width, row_bytes, enc, matrix_stride, count, input, input_stride))
        return gs::stream_launch(qtype, enc, matrix_stride, count, rows, width, row_bytes, input, input_stride, additive, out, out_stride,
                                 round_bf16, status, as_stream(stream));
    // shapes and qtypes the streaming kernel does not take: one matvec per matrix
    for (uint64_t m = 0; m < count; ++m) {
        rc = yvex_b200_gemv(qtype, enc + m * matrix_stride, rows, width, row_bytes, input + m * input_stride, 1,
                            additive ? additive + m * out_stride : nullptr, out + m * out_stride, round_bf16, status, stream);
        if (rc != OK) return rc;
    }
    return OK;
}
