// Library identity, the registry queries of the C-ABI, and the two pieces of process-wide
// bookkeeping: the kernel-launch counter and the optional phase events used for per-kernel timing.
#include <atomic>

#include "qtype_decode.cuh"

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
