/*
 * Expert-parallel MoE layer over the ranks of one box, orchestrated from C11 with NCCL point-to-point calls
 * (no reference counterpart: the reference is single-device, as its own README.md:184 states; per-pair meaning
 * src/graph/moe.c:587-622, combination src/runtime/moe.c:596-645).
 *
 * One process per GPU. Every rank owns the tokens it is given (its home rows) and a contiguous shard of
 * routed_experts / world experts, plus a copy of the shared expert. One call runs one layer for the rank's rows:
 *
 *   ingress rounding, router, top-k                                   (device layer, this rank's rows)
 *   dispatch   pairs grouped by destination rank into payload records (yvex_b200_ep_dispatch_payload)
 *   counts     one all-to-all of the split sizes: ncclSend/ncclRecv of one int64 per peer in one group;
 *              the step's only host read
 *   exchange   all-to-all-v of the records: ncclGroupStart; ncclSend/ncclRecv x world; ncclGroupEnd
 *   shared     the shared expert on the rank's own rows (covers the exchange on the device timeline)
 *   experts    the received records as a pair list on the local shard (yvex_b200_moe_expert_rows_payload)
 *   return     the reverse all-to-all-v of the bf16 result rows
 *   combine    rank-ordered f32 sum + shared row, bf16 (yvex_b200_moe_combine_indexed)
 *
 * NCCL is found at run time (dlopen of libnccl.so.2, or the path in YVEX_B200_NCCL_LIBRARY), so the library has
 * no link-time dependency on it and every other entry point works without it. Every wait for a peer is bounded:
 * after a group has been enqueued the host polls the stream and ncclCommGetAsyncError until the work is done or
 * the deadline given at open has passed; then the communicator is aborted, the call returns YVEX_ERR_TIMEOUT and
 * every later call on the handle returns YVEX_ERR_STATE.
 */
#define _POSIX_C_SOURCE 200809L
#include "backend_private.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* the part of NCCL's C ABI used here (nccl.h: ncclUniqueId is 128 opaque bytes, ncclComm_t a pointer, results and
 * data types plain enums) */
typedef struct { char internal[128]; } ep_unique_id;
typedef void *ep_comm;
enum { EP_NCCL_SUCCESS = 0, EP_NCCL_IN_PROGRESS = 7 };
enum { EP_NCCL_UINT8 = 1, EP_NCCL_INT64 = 4 };

typedef struct {
    void *handle;
    int (*get_unique_id)(ep_unique_id *);
    int (*comm_init_rank)(ep_comm *, int, ep_unique_id, int);
    int (*comm_destroy)(ep_comm);
    int (*comm_abort)(ep_comm);
    int (*comm_get_async_error)(ep_comm, int *);
    int (*group_start)(void);
    int (*group_end)(void);
    int (*send)(const void *, size_t, int, int, ep_comm, cudaStream_t);
    int (*recv)(void *, size_t, int, int, ep_comm, cudaStream_t);
} ep_nccl;

struct yvex_moe_ep {
    yvex_backend *backend;
    ep_nccl nccl;
    ep_comm comm;
    unsigned int world, rank;
    unsigned long long deadline_ms;
    long long *host_counts;            /* pinned: send counts [world], receive counts [world] */
    int failed;
};

static unsigned long long now_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (unsigned long long)ts.tv_sec * 1000ull + (unsigned long long)ts.tv_nsec / 1000000ull;
}

static int nccl_load(ep_nccl *n, yvex_error *err) {
    const char *path = getenv("YVEX_B200_NCCL_LIBRARY");
    memset(n, 0, sizeof(*n));
    n->handle = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!n->handle) return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "moe.ep", "NCCL (libnccl.so.2) could not be loaded");
#define EP_SYM(field_, name_) do { *(void **)(&n->field_) = dlsym(n->handle, name_); if (!n->field_) goto missing; } while (0)
    EP_SYM(get_unique_id, "ncclGetUniqueId");
    EP_SYM(comm_init_rank, "ncclCommInitRank");
    EP_SYM(comm_destroy, "ncclCommDestroy");
    EP_SYM(comm_abort, "ncclCommAbort");
    EP_SYM(comm_get_async_error, "ncclCommGetAsyncError");
    EP_SYM(group_start, "ncclGroupStart");
    EP_SYM(group_end, "ncclGroupEnd");
    EP_SYM(send, "ncclSend");
    EP_SYM(recv, "ncclRecv");
#undef EP_SYM
    return YVEX_OK;
missing:
    dlclose(n->handle);
    memset(n, 0, sizeof(*n));
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "moe.ep", "the NCCL library lacks a required entry point");
}

int yvex_moe_ep_unique_id(unsigned char id[YVEX_MOE_EP_ID_BYTES], yvex_error *err) {
    ep_nccl n;
    ep_unique_id u;
    int rc;
    if (!id) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "moe.ep.unique_id", "an identifier buffer is required");
    rc = nccl_load(&n, err);
    if (rc != YVEX_OK) return rc;
    rc = n.get_unique_id(&u);
    dlclose(n.handle);
    if (rc != EP_NCCL_SUCCESS) return yvex_refuse(err, YVEX_ERR_BACKEND, "moe.ep.unique_id", "ncclGetUniqueId failed");
    memcpy(id, u.internal, YVEX_MOE_EP_ID_BYTES);
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_moe_ep_open(yvex_moe_ep **out, yvex_backend *backend, const unsigned char id[YVEX_MOE_EP_ID_BYTES], unsigned int world,
                     unsigned int rank, unsigned long long deadline_ms, yvex_error *err) {
    yvex_moe_ep *ep;
    ep_unique_id u;
    int rc;
    if (out) *out = NULL;
    if (!out || !backend || !id || !world || rank >= world || !deadline_ms)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "moe.ep.open", "backend, identifier, world size, rank and deadline are required");
    rc = yvex_backend_admit(backend, "moe.ep.open", err);
    if (rc != YVEX_OK) return rc;
    ep = (yvex_moe_ep *)calloc(1u, sizeof(*ep));
    if (!ep) return yvex_refuse(err, YVEX_ERR_NOMEM, "moe.ep.open", "owner allocation failed");
    ep->backend = backend; ep->world = world; ep->rank = rank; ep->deadline_ms = deadline_ms;
    rc = nccl_load(&ep->nccl, err);
    if (rc != YVEX_OK) { free(ep); return rc; }
    if (cudaSetDevice(backend->device) != cudaSuccess || cudaMallocHost((void **)&ep->host_counts, 2u * world * sizeof(long long)) != cudaSuccess) {
        cudaGetLastError();
        dlclose(ep->nccl.handle);
        free(ep);
        return yvex_refuse(err, YVEX_ERR_NOMEM, "moe.ep.open", "no page-locked memory for the split sizes");
    }
    memcpy(u.internal, id, sizeof(u.internal));
    if (ep->nccl.comm_init_rank(&ep->comm, (int)world, u, (int)rank) != EP_NCCL_SUCCESS) {
        cudaFreeHost(ep->host_counts);
        dlclose(ep->nccl.handle);
        free(ep);
        return yvex_refuse(err, YVEX_ERR_BACKEND, "moe.ep.open", "ncclCommInitRank failed");
    }
    *out = ep;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_moe_ep_close(yvex_moe_ep **ep, yvex_error *err) {
    if (ep && *ep) {
        yvex_moe_ep *e = *ep;
        if (e->comm) { if (e->failed) e->nccl.comm_abort(e->comm); else e->nccl.comm_destroy(e->comm); }
        if (e->host_counts) cudaFreeHost(e->host_counts);
        if (e->nccl.handle) dlclose(e->nccl.handle);
        free(e);
        *ep = NULL;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

/* Waits until everything enqueued on the backend's stream has run, a communicator error shows, or the deadline passes. */
static int ep_wait(yvex_moe_ep *ep, const char *where, yvex_error *err) {
    const unsigned long long until = now_ms() + ep->deadline_ms;
    for (;;) {
        const cudaError_t q = cudaStreamQuery(ep->backend->stream);
        int async = EP_NCCL_SUCCESS;
        if (q == cudaSuccess) return YVEX_OK;
        if (q != cudaErrorNotReady) { ep->failed = 1; return yvex_backend_fail(ep->backend, where, err); }
        if (ep->nccl.comm_get_async_error(ep->comm, &async) != EP_NCCL_SUCCESS || (async != EP_NCCL_SUCCESS && async != EP_NCCL_IN_PROGRESS)) {
            ep->failed = 1;
            ep->nccl.comm_abort(ep->comm);
            ep->comm = NULL;
            return yvex_refuse(err, YVEX_ERR_BACKEND, where, "the communicator reported an asynchronous error");
        }
        if (now_ms() >= until) {
            ep->failed = 1;
            ep->nccl.comm_abort(ep->comm);              /* stops the collective kernels that wait for the missing peer */
            ep->comm = NULL;
            cudaStreamSynchronize(ep->backend->stream);
            cudaGetLastError();
            return yvex_refuse(err, YVEX_ERR_TIMEOUT, where, "a peer did not take part before the deadline");
        }
        {
            const struct timespec nap = {0, 50000};
            nanosleep(&nap, NULL);
        }
    }
}

/* all-to-all-v of byte rows: send_counts / recv_counts rows of `pitch` bytes per peer, packed in rank order */
static int ep_exchange(yvex_moe_ep *ep, const unsigned char *send, const long long *send_counts, unsigned char *recv,
                       const long long *recv_counts, unsigned long long pitch) {
    unsigned long long so = 0, ro = 0;
    int ok = ep->nccl.group_start() == EP_NCCL_SUCCESS;
    for (unsigned int r = 0; r < ep->world && ok; ++r) {
        const size_t sb = (size_t)((unsigned long long)send_counts[r] * pitch), rb = (size_t)((unsigned long long)recv_counts[r] * pitch);
        if (sb) ok = ep->nccl.send(send + so, sb, EP_NCCL_UINT8, (int)r, ep->comm, ep->backend->stream) == EP_NCCL_SUCCESS;
        if (ok && rb) ok = ep->nccl.recv(recv + ro, rb, EP_NCCL_UINT8, (int)r, ep->comm, ep->backend->stream) == EP_NCCL_SUCCESS;
        so += sb;
        ro += rb;
    }
    return (ep->nccl.group_end() == EP_NCCL_SUCCESS) && ok;
}

static unsigned long long al256(unsigned long long v) { return (v + 255ull) & ~255ull; }

static unsigned long long ep_fixed_bytes(const yvex_b200_moe_geometry *g, unsigned long long rows, unsigned int world) {
    const unsigned long long pairs = rows * g->topk, pitch = yvex_b200_ep_payload_pitch(g->hidden);
    return al256(rows * g->hidden * 4ull) * 3ull /* rows in, rounded rows, rows out */ + al256(rows * g->hidden * 2ull) * 2ull /* fp16 rows, shared result */ +
           al256(rows * g->experts * 4ull) + al256(pairs * 4ull) * 3ull + al256(rows * 4ull) * 3ull + al256(world * 8ull) * 2ull +
           al256(pairs * pitch) + al256(pairs * g->hidden * 2ull) + al256(yvex_b200_ep_dispatch_workspace_bytes(pairs, world)) + 4096ull;
}

int yvex_moe_ep_workspace_required(const yvex_moe_layer_plan *layer, unsigned long long rows, unsigned int world, unsigned long long *bytes,
                                   yvex_error *err) {
    yvex_b200_moe_geometry g, gl;
    unsigned long long cap, kernel, shared;
    if (bytes) *bytes = 0;
    if (!layer || !rows || !world || !bytes || layer->routed_experts % world)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "moe.ep.workspace_required", "layer, rows, a world size that divides the experts and a result are required");
    yvex_moe_plan_geometry(layer, NULL, &g);
    gl = g;
    gl.experts = g.experts / world;
    cap = rows * g.topk * world;                                       /* every rank's pairs, were they all routed here */
    kernel = yvex_b200_moe_expert_rows_workspace_bytes(&gl, cap);
    shared = yvex_b200_moe_expert_rows_workspace_bytes(&gl, rows);
    *bytes = ep_fixed_bytes(&g, rows, world) + al256(cap * yvex_b200_ep_payload_pitch(g.hidden)) + al256(cap * g.hidden * 2ull) +
             al256(kernel > shared ? kernel : shared);
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_moe_ep_execute_rows(yvex_moe_ep *ep, const yvex_moe_layer_job *job, const yvex_moe_row_batch *batch,
                             const yvex_moe_row_batch_output *output, yvex_moe_row_batch_result *result, yvex_error *err) {
    const char *where = "moe.ep.execute_rows";
    const yvex_moe_layer_plan *layer = job ? job->layer : NULL;
    yvex_backend *backend = ep ? ep->backend : NULL;
    yvex_b200_moe_geometry g, gl;
    yvex_b200_moe_weights w;
    const float *host_logits = NULL;
    const void *addr[YVEX_MOE_WEIGHT_COUNT];
    static const int required[YVEX_MOE_WEIGHT_COUNT] = {0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1};
    unsigned long long rows, pairs, pitch, cursor = 0, launches0, n_recv = 0, ws_bytes, e_loc;
    unsigned char *x_in, *xr, *x_out, *xh, *y_shared, *lg, *sel, *wts, *inverse, *ids, *sh_ids, *sh_w, *cnt_send, *cnt_recv, *payload, *y_back,
        *plan_ws, *recv, *y_recv, *kernel_ws;
    int rc, code, slot;

    if (result) memset(result, 0, sizeof(*result));
    if (!ep || !job || !layer || !batch || !result || !output || !output->combined_rows)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "handle, job, layer, batch, host output and result are required");
    if (ep->failed || !ep->comm) return yvex_refuse(err, YVEX_ERR_STATE, where, "the communicator was aborted by an earlier failure");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (backend->pending_slot) return yvex_refuse(err, YVEX_ERR_STATE, where, "a deferred MoE completion is still pending");
    if (batch->schema_version == YVEX_MOE_ROW_BATCH_SCHEMA_B200_LOGITS) host_logits = ((const yvex_moe_row_batch_logits *)batch)->router_logits;
    else if (batch->schema_version != YVEX_MOE_ROW_BATCH_SCHEMA_V1) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "row batch schema is not one this backend reads");
    rows = batch->row_count;
    if (!rows || !batch->expanded_rows || batch->device_rows) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "host rows are required");
    if (layer->residual_streams > 1ull) return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "the expert-parallel entry runs the layer without the mHC envelope");
    if (batch->row_width != layer->hidden_width || (batch->row_stride && batch->row_stride != batch->row_width))
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "row batch geometry does not match the layer's row width");
    if (layer->routed_experts % ep->world) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "the world size must divide the routed experts");
    yvex_moe_plan_geometry(layer, job, &g);
    gl = g;
    e_loc = g.experts / ep->world;
    gl.experts = e_loc;
    for (slot = YVEX_MOE_WEIGHT_ROUTED_GATE; slot < YVEX_MOE_WEIGHT_COUNT; ++slot)
        if (!yvex_b200_qtype_supported(job->weights[slot].qtype))
            return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "expert qtype has no device decoder in this backend");
    /* the routed packs hold this rank's shard: experts [rank * e_loc, (rank + 1) * e_loc) */
    if (!yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_GATE], e_loc * g.inter, g.hidden) ||
        !yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_UP], e_loc * g.inter, g.hidden) ||
        !yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_ROUTED_DOWN], e_loc * g.hidden, g.inter) ||
        !yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_GATE], g.shared_inter, g.hidden) ||
        !yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_UP], g.shared_inter, g.hidden) ||
        !yvex_moe_view_consistent(&job->weights[YVEX_MOE_WEIGHT_SHARED_DOWN], g.hidden, g.shared_inter))
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "expert weight views are inconsistent with the rank's shard of the layer");
    for (slot = 0; slot < YVEX_MOE_WEIGHT_COUNT; ++slot)
        if (!yvex_moe_resolve_view(backend, &job->weights[slot], required[slot], &addr[slot]))
            return yvex_refuse(err, YVEX_ERR_STATE, where, "MoE weights are not resident on this backend");
    memset(&w, 0, sizeof(w));
    w.router = (const float *)addr[YVEX_MOE_WEIGHT_ROUTER];
    w.bias = (const float *)addr[YVEX_MOE_WEIGHT_ROUTER_BIAS];
    w.hash_table = (const int32_t *)addr[YVEX_MOE_WEIGHT_ROUTER_TABLE];
    w.gate = addr[YVEX_MOE_WEIGHT_ROUTED_GATE]; w.up = addr[YVEX_MOE_WEIGHT_ROUTED_UP]; w.down = addr[YVEX_MOE_WEIGHT_ROUTED_DOWN];
    w.shared_gate = addr[YVEX_MOE_WEIGHT_SHARED_GATE]; w.shared_up = addr[YVEX_MOE_WEIGHT_SHARED_UP];
    w.shared_down = addr[YVEX_MOE_WEIGHT_SHARED_DOWN];
    if (w.router && (job->weights[YVEX_MOE_WEIGHT_ROUTER].qtype != 0u || job->weights[YVEX_MOE_WEIGHT_ROUTER].encoded_bytes != g.experts * g.hidden * 4ull))
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "router weights must be F32 [experts x hidden]");
    if (!w.router && !host_logits) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "either resident router weights or router logits are required");
    if (g.router_class == 0 && (!batch->token_ids_present || !batch->token_ids)) return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "MoE hash router requires token IDs");
    if (output->combined_capacity < rows * g.hidden) return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "combined output capacity is too small");

    pairs = rows * g.topk;
    pitch = yvex_b200_ep_payload_pitch(g.hidden);
#define EP_TAKE(var_, bytes_) do { (var_) = yvex_workspace_take(backend, &cursor, (bytes_)); if (!(var_)) \
        return yvex_refuse(err, YVEX_ERR_NOMEM, where, "attached device workspace is smaller than yvex_moe_ep_workspace_required"); } while (0)
    EP_TAKE(x_in, rows * g.hidden * 4ull); EP_TAKE(xr, rows * g.hidden * 4ull); EP_TAKE(x_out, rows * g.hidden * 4ull);
    EP_TAKE(xh, rows * g.hidden * 2ull); EP_TAKE(y_shared, rows * g.hidden * 2ull);
    EP_TAKE(lg, rows * g.experts * 4ull); EP_TAKE(sel, pairs * 4ull); EP_TAKE(wts, pairs * 4ull); EP_TAKE(inverse, pairs * 4ull);
    EP_TAKE(ids, rows * 4ull); EP_TAKE(sh_ids, rows * 4ull); EP_TAKE(sh_w, rows * 4ull);
    EP_TAKE(cnt_send, ep->world * 8ull); EP_TAKE(cnt_recv, ep->world * 8ull);
    EP_TAKE(payload, pairs * pitch); EP_TAKE(y_back, pairs * g.hidden * 2ull);
    EP_TAKE(plan_ws, yvex_b200_ep_dispatch_workspace_bytes(pairs, ep->world));
#define EP_CUDA(call_) do { if ((call_) != cudaSuccess) return yvex_backend_fail(backend, where, err); } while (0)
#define EP_DEVICE(call_, message_) do { rc = (call_); if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err); \
        if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, (message_)); } while (0)
    launches0 = yvex_b200_launch_count();
    EP_CUDA(cudaMemcpyAsync(x_in, batch->expanded_rows, rows * g.hidden * 4ull, cudaMemcpyHostToDevice, backend->stream));
    result->h2d_bytes += rows * g.hidden * 4ull;
    result->upload_count++;
    if (host_logits) {
        EP_CUDA(cudaMemcpyAsync(lg, host_logits, rows * g.experts * 4ull, cudaMemcpyHostToDevice, backend->stream));
        result->h2d_bytes += rows * g.experts * 4ull;
        result->upload_count++;
    }
    if (batch->token_ids_present && batch->token_ids) {
        EP_CUDA(cudaMemcpyAsync(ids, batch->token_ids, rows * 4ull, cudaMemcpyHostToDevice, backend->stream));
        result->h2d_bytes += rows * 4ull;
    }
    EP_CUDA(cudaMemsetAsync(sh_ids, 0xff, rows * 4ull, backend->stream));                    /* expert id -1: the shared expert */
    EP_DEVICE(yvex_b200_moe_ingress((const float *)x_in, rows * g.hidden, (float *)xr, xh, backend->status_word, backend->stream),
              "device layer refused the ingress rows");
    EP_DEVICE(yvex_b200_moe_route(&g, &w, (const float *)xr, host_logits ? (const float *)lg : NULL,
                                  batch->token_ids_present && batch->token_ids ? (const uint32_t *)ids : NULL, rows, (int32_t *)sel, (float *)wts,
                                  host_logits ? NULL : (float *)lg, NULL, 0ull, backend->status_word, backend->stream),
              "device layer refused the router geometry");
    EP_DEVICE(yvex_b200_ep_dispatch_payload((const int32_t *)sel, (const float *)wts, xh, rows, g.topk, g.hidden, e_loc, ep->world, ep->rank, 1ull,
                                            payload, (int32_t *)inverse, (long long *)cnt_send, plan_ws,
                                            yvex_b200_ep_dispatch_workspace_bytes(pairs, ep->world), backend->status_word, backend->stream),
              "device layer refused the dispatch geometry");
    /* the split sizes: one int64 to and from every peer, then the step's only host read */
    {
        int ok = ep->nccl.group_start() == EP_NCCL_SUCCESS;
        for (unsigned int r = 0; r < ep->world && ok; ++r)
            ok = ep->nccl.send(cnt_send + 8ull * r, 1u, EP_NCCL_INT64, (int)r, ep->comm, backend->stream) == EP_NCCL_SUCCESS &&
                 ep->nccl.recv(cnt_recv + 8ull * r, 1u, EP_NCCL_INT64, (int)r, ep->comm, backend->stream) == EP_NCCL_SUCCESS;
        if (ep->nccl.group_end() != EP_NCCL_SUCCESS || !ok) { ep->failed = 1; return yvex_backend_fail(backend, where, err); }
    }
    EP_CUDA(cudaMemcpyAsync(ep->host_counts, cnt_send, ep->world * 8ull, cudaMemcpyDeviceToHost, backend->stream));
    EP_CUDA(cudaMemcpyAsync(ep->host_counts + ep->world, cnt_recv, ep->world * 8ull, cudaMemcpyDeviceToHost, backend->stream));
    result->d2h_bytes += 2ull * ep->world * 8ull;
    rc = ep_wait(ep, where, err);
    if (rc != YVEX_OK) return rc;
    result->stream_synchronizations++;
    for (unsigned int r = 0; r < ep->world; ++r) {
        if (ep->host_counts[r] < 0 || ep->host_counts[ep->world + r] < 0) return yvex_refuse(err, YVEX_ERR_STATE, where, "a split size is negative");
        n_recv += (unsigned long long)ep->host_counts[ep->world + r];
    }
    EP_TAKE(recv, (n_recv ? n_recv : 1ull) * pitch);
    EP_TAKE(y_recv, (n_recv ? n_recv : 1ull) * g.hidden * 2ull);
    {
        const unsigned long long a = yvex_b200_moe_expert_rows_workspace_bytes(&gl, n_recv ? n_recv : 1ull),
                                 b = yvex_b200_moe_expert_rows_workspace_bytes(&gl, rows);
        ws_bytes = a > b ? a : b;
    }
    EP_TAKE(kernel_ws, ws_bytes);
    if (!ep_exchange(ep, payload, ep->host_counts, recv, ep->host_counts + ep->world, pitch)) { ep->failed = 1; return yvex_backend_fail(backend, where, err); }
    /* route weight 1 of the shared expert's pairs: written after the sizes are known, before anything reads it */
    {
        float *ones = (float *)(backend->host_scratch + 4096);
        const unsigned long long chunk = (YVEX_HOST_SCRATCH_BYTES - 4096u) / 4u;
        for (unsigned long long i = 0; i < (rows < chunk ? rows : chunk); ++i) ones[i] = 1.0f;
        for (unsigned long long at = 0; at < rows; at += chunk) {
            const unsigned long long n = rows - at < chunk ? rows - at : chunk;
            EP_CUDA(cudaMemcpyAsync(sh_w + at * 4ull, ones, n * 4ull, cudaMemcpyHostToDevice, backend->stream));
        }
    }
    EP_DEVICE(yvex_b200_moe_expert_rows(&gl, &w, xh, (const int32_t *)sh_ids, (const float *)sh_w, rows, y_shared, kernel_ws, ws_bytes,
                                        backend->status_word, backend->stream), "device layer refused the shared expert's rows");
    if (n_recv)
        EP_DEVICE(yvex_b200_moe_expert_rows_payload(&gl, &w, recv, n_recv, y_recv, kernel_ws, ws_bytes, backend->status_word, backend->stream),
                  "device layer refused the received pair list");
    /* results go home over the reverse splits */
    if (!ep_exchange(ep, y_recv, ep->host_counts + ep->world, y_back, ep->host_counts, g.hidden * 2ull)) { ep->failed = 1; return yvex_backend_fail(backend, where, err); }
    EP_DEVICE(yvex_b200_moe_combine_indexed(y_back, (const int32_t *)inverse, y_shared, NULL, rows, g.topk, g.hidden, (float *)x_out,
                                            backend->status_word, backend->stream), "device layer refused the combination");
    EP_CUDA(cudaMemcpyAsync(output->combined_rows, x_out, rows * g.hidden * 4ull, cudaMemcpyDeviceToHost, backend->stream));
    result->d2h_bytes += rows * g.hidden * 4ull;
    result->download_count++;
    if (output->selected_weights && output->selection_capacity >= pairs) {
        EP_CUDA(cudaMemcpyAsync(output->selected_weights, wts, pairs * 4ull, cudaMemcpyDeviceToHost, backend->stream));
        result->d2h_bytes += pairs * 4ull;
    }
    if (output->selected_experts && output->selection_capacity >= pairs) {
        EP_CUDA(cudaMemcpyAsync((int32_t *)output->selected_experts + pairs, sel, pairs * 4ull, cudaMemcpyDeviceToHost, backend->stream));
        result->d2h_bytes += pairs * 4ull;
    }
    rc = ep_wait(ep, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, where, err);
    result->stream_synchronizations += 2ull;
    if (code) { memset(result, 0, sizeof(*result)); return yvex_moe_status_error(code, err); }
    if (output->selected_experts && output->selection_capacity >= pairs) {
        const int32_t *src = (const int32_t *)output->selected_experts + pairs;
        for (unsigned long long i = 0; i < pairs; ++i) output->selected_experts[i] = (unsigned long long)src[i];
    }
    result->schema_version = YVEX_MOE_ROW_BATCH_RESULT_SCHEMA_V4;
    result->execution_class = YVEX_EXECUTION_CLASS_DEVICE_NATIVE;
    result->row_count = rows;
    result->row_expert_pairs = pairs;
    result->grouped_expert_operations = n_recv;          /* pairs this rank's shard executed */
    result->shared_expert_operations = rows;
    result->expert_subviews_accessed = n_recv * 3ull;
    result->kernel_launches = yvex_b200_launch_count() - launches0;
    result->d2d_bytes = (pairs + n_recv) * (pitch + g.hidden * 2ull);      /* bytes this rank sent and received over NVLink */
    result->completed = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}
