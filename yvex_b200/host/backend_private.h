/* Private state of the host boundary (counterpart of src/backend/private.h:66-93). */
#ifndef YVEX_B200_BACKEND_PRIVATE_H
#define YVEX_B200_BACKEND_PRIVATE_H
#include <cuda_runtime_api.h>
#include <stdatomic.h>
#include <stdint.h>

#include "yvex_b200_backend.h"
#include "yvex_b200_kernels.h"

#define YVEX_MOE_MAX_CHUNKS 4
#define YVEX_HOST_SCRATCH_BYTES (1u << 20)   /* pinned: status read-back and router selections of narrow batches */

/* Launch graphs of the narrow MoE entry (counterpart of yvex_cuda_graph_execute, src/backend/cuda/moe.c:1645-1681): the kernel
 * sequence of one (layer, row count, buffers) combination, captured the second time the combination is seen. */
#define YVEX_MOE_GRAPH_SLOTS 8
#define YVEX_MOE_GRAPH_KEY_WORDS 56
typedef struct {
    unsigned long long key[YVEX_MOE_GRAPH_KEY_WORDS];
    int seen;                         /* 0 free, 1 seen once (ran eagerly), 2 captured, -1 capture failed: stays eager */
    cudaGraphExec_t exec;
    unsigned long long launches, stamp;
} yvex_moe_graph_slot;

struct yvex_backend {
    yvex_backend_kind kind;
    _Atomic int status;
    int device, closing;
    cudaStream_t stream;
    yvex_backend_memory_stats stats;
    unsigned long long next_owner_id;
    const unsigned char *resident_host_base;
    unsigned long long resident_host_bytes, resident_device_address, resident_generation;
    yvex_device_tensor *workspace;
    int *status_word;                 /* device: first fault of the enqueued kernels */
    unsigned char *host_scratch;      /* pinned */
    yvex_moe_device_completion_slot *pending_slot;   /* deferred completion in flight */
    unsigned long long last_pipeline_chunks;         /* row ranges of the last wide call's copy pipeline */
    unsigned char *act_scratch;                      /* prepared activation rows / row ids of the encoded matvec family */
    unsigned long long act_scratch_bytes;            /* (grown on demand, freed at close) */
    /* copy pipeline of the wide entry: host rows go in on copy_in and come back on copy_out while the
     * compute stream works on another chunk of rows */
    yvex_moe_graph_slot moe_graphs[YVEX_MOE_GRAPH_SLOTS];
    unsigned long long moe_graph_stamp;
    cudaStream_t copy_in, copy_out;
    cudaEvent_t ev_begin, ev_end, ev_in[YVEX_MOE_MAX_CHUNKS], ev_done[YVEX_MOE_MAX_CHUNKS];
};
#define YVEX_DEVICE_OBSERVATION_OFFSET 256   /* the worklist summary lives behind the status word */
#define YVEX_DEVICE_STATE_BYTES 1024
#define YVEX_HOST_DEFERRED_STATUS_OFFSET 128   /* in the pinned host scratch: the status word of a deferred completion */

int yvex_refuse(yvex_error *err, yvex_status code, const char *where, const char *message);
int yvex_backend_admit(const yvex_backend *backend, const char *where, yvex_error *err);
int yvex_backend_fail(yvex_backend *backend, const char *where, yvex_error *err);
int yvex_tensor_owned(const yvex_backend *backend, const yvex_device_tensor *t);
unsigned char *yvex_workspace_take(yvex_backend *backend, unsigned long long *cursor, unsigned long long bytes);
int yvex_backend_take_status(yvex_backend *backend, int *code);
/* Test seam of the reference (src/backend/cuda/qtype.c:625-661): 1 if the environment variable `name` is set to `value`. */
int yvex_test_seam(const char *name, const char *value);
void yvex_moe_graphs_release(yvex_backend *backend);
int yvex_moe_plan_geometry(const yvex_moe_layer_plan *layer, const yvex_moe_layer_job *job, yvex_b200_moe_geometry *g);
int yvex_moe_resolve_view(const yvex_backend *backend, const yvex_moe_weight_view *v, int required, const void **out);
int yvex_moe_view_consistent(const yvex_moe_weight_view *v, unsigned long long rows, unsigned long long width);
int yvex_moe_status_error(int code, yvex_error *err);
#endif
