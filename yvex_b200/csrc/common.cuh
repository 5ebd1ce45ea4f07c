// Shared device helpers: status word, scalar codecs, warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/yvex_b200_kernels.h"

namespace yb {

enum : int { OK = 0, ERR = -1, ERR_NOMEM = -2, ERR_FORMAT = -4, ERR_UNSUPPORTED = -5,
             ERR_BACKEND = -6, ERR_BOUNDS = -7, ERR_STATE = -8, ERR_INVALID_ARG = -10 };

enum : unsigned { Q_F32 = 0, Q_F16 = 1, Q_Q8_0 = 8, Q_Q2_K = 10, Q_Q4_K = 12, Q_IQ2_XXS = 16,
                  Q_BF16 = 30, Q_MXFP4 = 39 };

constexpr int kSmCount = 148;

// First fault wins, like the reference kernels' atomicCAS(status, 0, code).
__device__ __forceinline__ void raise(int *status, int code) {
    if (status) atomicCAS(status, 0, code);
}
__device__ __forceinline__ bool faulted(const int *status) {
    return status && *reinterpret_cast<const volatile int *>(status) != 0;
}

// f32 -> bf16 -> f32, round-to-nearest-even, NaN quieted: src/gguf/quant_scalar.c:130-143.
__device__ __forceinline__ float bf16_round(float v) {
    uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu))
        return __uint_as_float((bits | 0x00400000u) & 0xffff0000u);
    uint32_t lower = bits & 0xffffu, upper = bits >> 16;
    if (lower > 0x8000u || (lower == 0x8000u && (upper & 1u))) ++upper;
    return __uint_as_float(upper << 16);
}
__device__ __forceinline__ uint16_t bf16_bits(float v) {
    return static_cast<uint16_t>(__float_as_uint(bf16_round(v)) >> 16);
}

// IEEE binary16 -> f32 including subnormals: src/gguf/quant_scalar.c:40-68.
__device__ __forceinline__ float f16_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint16_t ldg_u16(const uint8_t *p) {
    return __ldg(reinterpret_cast<const uint16_t *>(p));
}

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }
// Grid size for `jobs` units at `per_block` units per CTA, capped at `waves` CTAs per SM.
inline unsigned grid_for(uint64_t jobs, uint64_t per_block, uint64_t waves) {
    uint64_t need = (jobs + per_block - 1) / per_block, cap = (uint64_t)kSmCount * waves;
    return (unsigned)(need < 1 ? 1 : need < cap ? need : cap);
}
// Programmatic dependent launch (device side). A kernel launched with launch_pdl may begin before
// the kernel before it on the stream has finished; pdl_wait() returns once that kernel has completed
// and its writes are visible, pdl_trigger() lets the kernel after this one begin. Both are no-ops
// for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with programmatic stream serialization allowed.
template <class... Params, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// A kernel's opt-in to more than 48 KiB of dynamic shared memory is a per-DEVICE attribute of the
// function. One of these sits beside each such kernel's launch code and remembers, per device
// ordinal, that the attribute has been set; devices beyond the table set it on every launch.
struct SmemOptIn {
    static constexpr int kDevices = 64;
    std::atomic<int> bytes[kDevices];
    template <class Kernel> int ensure(Kernel kernel, int want) {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return ERR_BACKEND;
        if (dev < kDevices && bytes[dev].load(std::memory_order_acquire) >= want) return OK;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, want) != cudaSuccess) return ERR_BACKEND;
        if (dev < kDevices) bytes[dev].store(want, std::memory_order_release);
        return OK;
    }
};

// Adds `launches` to the library's kernel-launch counter and reports a failed enqueue.
int launch_status(int launches = 1);
// Records the caller-registered phase event `phase` on `s` (no-op when none is registered).
void mark_phase(int phase, cudaStream_t s);

}  // namespace yb
