// Library identity, the registry queries of the C-ABI, and the two pieces of process-wide
// bookkeeping: the kernel-launch counter and the optional phase events used for per-kernel timing.
#include <atomic>

#include "qtype_decode.cuh"
#include "tcgen05.cuh"

namespace yb {

static std::atomic<unsigned long long> g_launches{0};
static void **g_phase_events = nullptr;
static int g_phase_count = 0;

int launch_status(int launches) {
    g_launches.fetch_add((unsigned long long)launches, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? OK : ERR_BACKEND;
}

void mark_phase(int phase, cudaStream_t s) {
    if (g_phase_events && phase < g_phase_count && g_phase_events[phase])
        cudaEventRecord(static_cast<cudaEvent_t>(g_phase_events[phase]), s);
}

// One warp; lane 0 waits for a phase that never completes.
__global__ void selftest_wait_kernel(uint64_t limit_ns, uint64_t *elapsed_ns, int *status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncwarp();
    const uint64_t t0 = sm100::global_ns();
    const bool done = sm100::mbar_wait_warp(&bar, 0u, &abort_flag, limit_ns);
    if (threadIdx.x == 0) {
        if (elapsed_ns) *elapsed_ns = sm100::global_ns() - t0;
        if (!done) raise(status, YVEX_B200_STATUS_TIMEOUT);
    }
}

}  // namespace yb

using namespace yb;

extern "C" const char *yvex_b200_version(void) { return "yvex-b200 0.1 (sm_100a)"; }

extern "C" int yvex_b200_qtype_supported(unsigned int qtype) { return qtype_supported(qtype) ? 1 : 0; }

extern "C" int yvex_b200_qtype_geometry(unsigned int qtype, unsigned int *block_elements,
                                        unsigned int *block_bytes) {
    Geometry g = geometry_of(qtype);
    if (qtype > 42u) return 0;
    if (block_elements) *block_elements = g.elems;
    if (block_bytes) *block_bytes = g.bytes;
    return 1;
}

extern "C" unsigned long long yvex_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int yvex_b200_phase_events(void **events, int count) {
    if (count < 0 || (count > 0 && !events)) return ERR_INVALID_ARG;
    g_phase_events = count ? events : nullptr;
    g_phase_count = count;
    return OK;
}

extern "C" int yvex_b200_selftest_bounded_wait(uint64_t limit_ns, uint64_t *elapsed_ns, int *status, void *stream) {
    if (!status || !limit_ns || limit_ns > 5000000000ull) return ERR_INVALID_ARG;
    selftest_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(limit_ns, elapsed_ns, status);
    return launch_status(1);
}
