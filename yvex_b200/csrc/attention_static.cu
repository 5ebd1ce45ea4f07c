// GQA decode attention for callers that can hand over no scratch memory and must not trigger an
// allocation: the split-KV partials live in a fixed device array that is part of the loaded module
// image, so a call performs no device-memory allocation or release, directly or through a library.
//
// Who needs this: a host runtime that has planned every device byte up front and treats an
// allocator call in the middle of a decode step as an accounting error (it cannot grow its
// workspace there), and code on a latency-critical path whose rules forbid entering the device
// allocator because an allocation may synchronise the whole device.
// Such callers cannot use the ordinary entry point unless they reserved its workspace earlier.
//
// Limits and rules:
//   * the partials must fit kStaticScratchBytes (8 MiB); larger problems are refused with
//     YVEX_B200_ERR_BOUNDS before any launch (the ordinary entry point has no such limit);
//   * the FIRST call on each device looks up the array's device address (cudaGetSymbolAddress,
//     with that device current). Make that first call once per device during start-up, before
//     any stream capture begins; later calls only launch kernels;
//   * nothing in the array has to start at zero: every (session, kv head, split) slot is written
//     by the first kernel of a call before the merge kernel of the same call reads it;
//   * the array used is that of the device that is CURRENT in the calling thread; `stream` must be a
//     stream of that same device (the call does not check the pairing);
//   * there is ONE array per device. Two calls that overlap in time on the same device (different
//     streams, threads or processes sharing the context) race on it; callers serialise them.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "yvex_b200_kernels.h"

namespace {

constexpr uint64_t kStaticScratchBytes = 8ull << 20;
constexpr int kMaxDevices = 64;

__device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal, filled on first use on that device.
std::atomic<void *> g_scratch_address[kMaxDevices];

// YVEX status codes used here (include/yvex_b200_backend.h: yvex_status).
constexpr int kErrBackend = -6, kErrBounds = -7, kErrInvalidArg = -10;

int scratch_for_current_device(void **out) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return kErrBackend;
    void *p = g_scratch_address[device].load(std::memory_order_acquire);
    if (!p) {
        // one-time set-up for this device: no allocation, only a symbol lookup in the module
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return kErrBackend;
        g_scratch_address[device].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

}  // namespace

extern "C" uint64_t yvex_b200_attention_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int yvex_b200_attention_gqa_decode_static(const void *q, const void *k, const void *v, uint64_t sessions,
                                                     uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                                                     uint64_t context, uint64_t position, float scale, float *out,
                                                     int *status, void *stream) {
    if (!kv_heads || !sessions || !q_heads || !context) return kErrInvalidArg;
    if (position >= context) return kErrBounds;
    // Size by the visible prefix exactly as the ordinary entry point does for this position.
    const uint64_t need = yvex_b200_attention_workspace_bytes(sessions, q_heads, kv_heads, head_dim, position + 1);
    if (need > kStaticScratchBytes) return kErrBounds;          // problem too large for the fixed array
    void *scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    return yvex_b200_attention_gqa_decode(q, k, v, sessions, q_heads, kv_heads, head_dim, context, position, scale,
                                          out, scratch, kStaticScratchBytes, status, stream);
}
