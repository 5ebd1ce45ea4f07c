/*
 * Backend object, tensors, resident arena, workspace, capability and the non-MoE operators of the
 * host boundary (include/yvex_b200_backend.h). C11 over the CUDA runtime's C API; all compute is
 * delegated to the device layer (include/yvex_b200_kernels.h). There is no CPU path: a process
 * without a CUDA device cannot open a backend.
 */
#include "backend_private.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

void yvex_error_clear(yvex_error *err) {
    if (err) { err->code = YVEX_OK; err->where[0] = 0; err->message[0] = 0; }
}

void yvex_error_set(yvex_error *err, yvex_status code, const char *where, const char *message) {
    if (!err) return;
    err->code = code;
    snprintf(err->where, sizeof(err->where), "%s", where ? where : "");
    snprintf(err->message, sizeof(err->message), "%s", message ? message : "");
}

const char *yvex_status_name(yvex_status status) {
    switch (status) {
    case YVEX_OK: return "ok";
    case YVEX_ERR: return "error";
    case YVEX_ERR_NOMEM: return "nomem";
    case YVEX_ERR_IO: return "io";
    case YVEX_ERR_FORMAT: return "format";
    case YVEX_ERR_UNSUPPORTED: return "unsupported";
    case YVEX_ERR_BACKEND: return "backend";
    case YVEX_ERR_BOUNDS: return "bounds";
    case YVEX_ERR_STATE: return "state";
    case YVEX_ERR_CANCELLED: return "cancelled";
    case YVEX_ERR_INVALID_ARG: return "invalid-arg";
    case YVEX_ERR_TIMEOUT: return "timeout";
    }
    return "unknown";
}

int yvex_refuse(yvex_error *err, yvex_status code, const char *where, const char *message) {
    yvex_error_set(err, code, where, message);
    return code;
}

/* Dispatch guard of the reference (src/backend/private.h:105-115): closing or failed backends refuse. */
int yvex_backend_admit(const yvex_backend *backend, const char *where, yvex_error *err) {
    if (!backend) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "backend is required");
    if (backend->closing || atomic_load(&((yvex_backend *)backend)->status) == YVEX_BACKEND_STATUS_FAILED)
        return yvex_refuse(err, YVEX_ERR_STATE, where, "backend is closing or failed");
    if (cudaSetDevice(backend->device) != cudaSuccess)
        return yvex_refuse(err, YVEX_ERR_BACKEND, where, "CUDA device cannot be made current");
    return YVEX_OK;
}

/* Sticky fail-closed: a failed launch or copy demotes the backend (src/backend/cuda/capability.c:611-667). */
int yvex_backend_fail(yvex_backend *backend, const char *where, yvex_error *err) {
    atomic_store(&backend->status, YVEX_BACKEND_STATUS_FAILED);
    cudaGetLastError();
    return yvex_refuse(err, YVEX_ERR_BACKEND, where, "CUDA call failed; backend demoted to FAILED");
}

int yvex_test_seam(const char *name, const char *value) {
    const char *v = getenv(name);
    return v && !strcmp(v, value);
}

/* Creates (or destroys) the events of the copy pipeline; 1 on success. */
static int backend_events(yvex_backend *b, int create) {
    cudaEvent_t *all[2 + 2 * YVEX_MOE_MAX_CHUNKS];
    int n = 0, ok = 1;
    all[n++] = &b->ev_begin; all[n++] = &b->ev_end;
    for (int i = 0; i < YVEX_MOE_MAX_CHUNKS; ++i) { all[n++] = &b->ev_in[i]; all[n++] = &b->ev_done[i]; }
    for (int i = 0; i < n; ++i) {
        if (create) ok &= cudaEventCreateWithFlags(all[i], cudaEventDisableTiming) == cudaSuccess;
        else if (*all[i]) { ok &= cudaEventDestroy(*all[i]) == cudaSuccess; *all[i] = NULL; }
    }
    return ok;
}

int yvex_backend_open(yvex_backend **out, const yvex_backend_options *options, yvex_error *err) {
    int device = 0, count = 0;
    yvex_backend *b;
    if (out) *out = NULL;
    if (!out || !options) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_open", "out and options are required");
    if (options->kind != YVEX_BACKEND_KIND_CUDA)
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "yvex_backend_open",
                           "only the CUDA backend kind exists in this library; no cross-backend fallback");
    if (options->device && sscanf(options->device, "cuda:%d", &device) != 1 && strcmp(options->device, "cuda") != 0)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_open", "device must be \"cuda\" or \"cuda:N\"");
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return yvex_refuse(err, YVEX_ERR_BACKEND, "yvex_backend_open", "CUDA device is unavailable");
    }
    b = (yvex_backend *)calloc(1, sizeof(*b));
    if (!b) return yvex_refuse(err, YVEX_ERR_NOMEM, "yvex_backend_open", "backend allocation failed");
    b->kind = YVEX_BACKEND_KIND_CUDA;
    b->device = device;
    b->stats.memory_limit_bytes = options->memory_limit_bytes;
    b->next_owner_id = 1;
    atomic_init(&b->status, YVEX_BACKEND_STATUS_READY);
    if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&b->copy_in, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&b->copy_out, cudaStreamNonBlocking) != cudaSuccess || !backend_events(b, 1) ||
        cudaMalloc((void **)&b->status_word, YVEX_DEVICE_STATE_BYTES) != cudaSuccess ||
        cudaMallocHost((void **)&b->host_scratch, YVEX_HOST_SCRATCH_BYTES) != cudaSuccess ||
        cudaMemsetAsync(b->status_word, 0, YVEX_DEVICE_STATE_BYTES, b->stream) != cudaSuccess) {
        cudaGetLastError();
        yvex_backend_close(b);
        return yvex_refuse(err, YVEX_ERR_BACKEND, "yvex_backend_open", "CUDA context, stream or status word unavailable");
    }
    *out = b;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_close_checked(yvex_backend **backend, yvex_error *err) {
    yvex_backend *b = backend ? *backend : NULL;
    int ok = 1;
    if (!b) { yvex_error_clear(err); return YVEX_OK; }
    b->closing = 1;
    cudaSetDevice(b->device);
    if (b->stream) ok &= cudaStreamSynchronize(b->stream) == cudaSuccess;
    if (b->stats.allocation_count) {
        /* owned tensors must be released first: the owner is retained for retry (include/yvex/backend.h:142-152) */
        b->closing = 0;
        return yvex_refuse(err, YVEX_ERR_STATE, "yvex_backend_close_checked", "backend still owns tensors");
    }
    yvex_moe_graphs_release(b);
    if (b->status_word) ok &= cudaFree(b->status_word) == cudaSuccess;
    if (b->act_scratch) ok &= cudaFree(b->act_scratch) == cudaSuccess;
    if (b->host_scratch) ok &= cudaFreeHost(b->host_scratch) == cudaSuccess;
    ok &= backend_events(b, 0);
    if (b->copy_in) ok &= cudaStreamDestroy(b->copy_in) == cudaSuccess;
    if (b->copy_out) ok &= cudaStreamDestroy(b->copy_out) == cudaSuccess;
    if (b->stream) ok &= cudaStreamDestroy(b->stream) == cudaSuccess;
    free(b);
    *backend = NULL;
    if (!ok) { cudaGetLastError(); return yvex_refuse(err, YVEX_ERR_BACKEND, "yvex_backend_close_checked", "cleanup failed"); }
    yvex_error_clear(err);
    return YVEX_OK;
}

void yvex_backend_close(yvex_backend *backend) {
    if (!backend) return;
    cudaSetDevice(backend->device);
    if (backend->stream) cudaStreamSynchronize(backend->stream);
    yvex_moe_graphs_release(backend);
    backend_events(backend, 0);
    if (backend->copy_in) { cudaStreamSynchronize(backend->copy_in); cudaStreamDestroy(backend->copy_in); }
    if (backend->copy_out) { cudaStreamSynchronize(backend->copy_out); cudaStreamDestroy(backend->copy_out); }
    if (backend->stream) cudaStreamDestroy(backend->stream);
    if (backend->status_word) cudaFree(backend->status_word);
    if (backend->act_scratch) cudaFree(backend->act_scratch);
    if (backend->host_scratch) cudaFreeHost(backend->host_scratch);
    cudaGetLastError();
    free(backend);
}

yvex_backend_kind yvex_backend_kind_of(const yvex_backend *backend) { return backend ? backend->kind : YVEX_BACKEND_KIND_CPU; }

yvex_backend_status yvex_backend_status_of(const yvex_backend *backend) {
    return backend ? (yvex_backend_status)atomic_load(&((yvex_backend *)backend)->status) : YVEX_BACKEND_STATUS_UNSUPPORTED;
}

void *yvex_backend_stream(const yvex_backend *backend) { return backend ? (void *)backend->stream : NULL; }

int yvex_backend_get_memory_stats(const yvex_backend *backend, yvex_backend_memory_stats *out, yvex_error *err) {
    if (!backend || !out) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_get_memory_stats", "arguments are required");
    *out = backend->stats;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_sync(yvex_backend *backend, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_sync", err);
    if (rc != YVEX_OK) return rc;
    if (cudaStreamSynchronize(backend->stream) != cudaSuccess) return yvex_backend_fail(backend, "yvex_backend_sync", err);
    yvex_error_clear(err);
    return YVEX_OK;
}

/* ---- tensors ---------------------------------------------------------------------------------- */

int yvex_tensor_owned(const yvex_backend *backend, const yvex_device_tensor *t) {
    return t && t->owner == backend && t->owner_id != 0;           /* src/backend/private.h:153-157 */
}

static int tensor_new(yvex_backend *backend, const yvex_backend_tensor_desc *desc, int pinned_host, yvex_device_tensor **out,
                      yvex_error *err, const char *where) {
    yvex_device_tensor *t;
    int rc = yvex_backend_admit(backend, where, err);
    if (out) *out = NULL;
    if (rc != YVEX_OK) return rc;
    if (!desc || !out || !desc->bytes || desc->rank > YVEX_TENSOR_MAX_DIMS)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "tensor descriptor is invalid");
    if (backend->stats.memory_limit_bytes && backend->stats.allocated_bytes + desc->bytes > backend->stats.memory_limit_bytes)
        return yvex_refuse(err, YVEX_ERR_NOMEM, where, "allocation exceeds the backend memory limit");
    t = (yvex_device_tensor *)calloc(1, sizeof(*t));
    if (!t) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "tensor record allocation failed");
    if (cudaMalloc((void **)&t->data, desc->bytes) != cudaSuccess ||
        (pinned_host && cudaMallocHost((void **)&t->host_data, desc->bytes) != cudaSuccess)) {
        cudaGetLastError();
        if (t->data) cudaFree(t->data);
        free(t);
        return yvex_refuse(err, YVEX_ERR_NOMEM, where, "device or pinned host memory is exhausted");
    }
    t->owner = backend;
    t->owner_id = backend->next_owner_id++;
    t->dtype = desc->dtype;
    t->rank = desc->rank;
    memcpy(t->dims, desc->dims, sizeof(t->dims));
    t->bytes = desc->bytes;
    backend->stats.allocated_bytes += desc->bytes;
    backend->stats.allocation_count++;
    backend->stats.allocation_events++;
    if (backend->stats.allocated_bytes > backend->stats.peak_allocated_bytes)
        backend->stats.peak_allocated_bytes = backend->stats.allocated_bytes;
    *out = t;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_tensor_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc, yvex_device_tensor **out, yvex_error *err) {
    return tensor_new(backend, desc, 0, out, err, "yvex_backend_tensor_alloc");
}

void yvex_backend_tensor_free(yvex_backend *backend, yvex_device_tensor *tensor) {
    if (!backend || !yvex_tensor_owned(backend, tensor)) return;
    cudaSetDevice(backend->device);
    cudaStreamSynchronize(backend->stream);
    if (backend->workspace == tensor) backend->workspace = NULL;
    cudaFree(tensor->data);
    if (tensor->host_data) cudaFreeHost(tensor->host_data);
    backend->stats.allocated_bytes -= tensor->bytes;
    backend->stats.allocation_count--;
    backend->stats.release_events++;
    tensor->owner_id = 0;
    free(tensor);
}

int yvex_backend_tensor_write(yvex_backend *backend, yvex_device_tensor *tensor, const void *src, unsigned long long len, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_tensor_write", err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_tensor_owned(backend, tensor) || !src) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_tensor_write", "tensor must belong to this backend");
    if (len > tensor->bytes) return yvex_refuse(err, YVEX_ERR_BOUNDS, "yvex_backend_tensor_write", "write exceeds the tensor");
    if (cudaMemcpyAsync(tensor->data, src, len, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess ||
        cudaStreamSynchronize(backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, "yvex_backend_tensor_write", err);
    backend->stats.h2d_bytes += len;
    tensor->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_tensor_read(yvex_backend *backend, const yvex_device_tensor *tensor, void *dst, unsigned long long len, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_tensor_read", err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_tensor_owned(backend, tensor) || !dst) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_tensor_read", "tensor must belong to this backend");
    if (len > tensor->bytes) return yvex_refuse(err, YVEX_ERR_BOUNDS, "yvex_backend_tensor_read", "read exceeds the tensor");
    if (!tensor->is_written) return yvex_refuse(err, YVEX_ERR_STATE, "yvex_backend_tensor_read", "tensor has not been written");
    if (cudaMemcpyAsync(dst, tensor->data, len, cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess ||
        cudaStreamSynchronize(backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, "yvex_backend_tensor_read", err);
    backend->stats.d2h_bytes += len;
    yvex_error_clear(err);
    return YVEX_OK;
}

unsigned long long yvex_device_tensor_bytes(const yvex_device_tensor *tensor) { return tensor ? tensor->bytes : 0ull; }
int yvex_device_tensor_is_written(const yvex_device_tensor *tensor) { return tensor ? tensor->is_written : 0; }

/* ---- resident arena and workspace -------------------------------------------------------------- */

int yvex_backend_resident_alloc(yvex_backend *backend, const yvex_backend_tensor_desc *desc, yvex_device_tensor **out,
                                unsigned char **host, yvex_error *err) {
    int rc = tensor_new(backend, desc, 1, out, err, "yvex_backend_resident_alloc");
    if (host) *host = rc == YVEX_OK ? (*out)->host_data : NULL;
    return rc;
}

int yvex_backend_resident_prefetch(yvex_backend *backend, yvex_device_tensor *tensor, unsigned long long *prefetched_bytes, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_resident_prefetch", err);
    if (prefetched_bytes) *prefetched_bytes = 0;
    if (rc != YVEX_OK) return rc;
    if (!yvex_tensor_owned(backend, tensor) || !tensor->host_data)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_resident_prefetch", "tensor is not a resident arena of this backend");
    if (cudaMemcpyAsync(tensor->data, tensor->host_data, tensor->bytes, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess ||
        cudaStreamSynchronize(backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, "yvex_backend_resident_prefetch", err);
    backend->stats.h2d_bytes += tensor->bytes;
    tensor->is_written = 1;
    if (prefetched_bytes) *prefetched_bytes = tensor->bytes;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_resident_attach(yvex_backend *backend, const unsigned char *host_base, unsigned long long bytes,
                                 const yvex_device_tensor *device_tensor, unsigned long long generation, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_resident_attach", err);
    if (rc != YVEX_OK) return rc;
    if (!host_base || !bytes || !generation || !yvex_tensor_owned(backend, device_tensor) ||
        device_tensor->host_data != host_base || device_tensor->bytes < bytes)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_resident_attach",
                           "resident range must be the host side of a tensor this backend owns");
    backend->resident_host_base = host_base;
    backend->resident_host_bytes = bytes;
    backend->resident_device_address = (unsigned long long)(uintptr_t)device_tensor->data;
    backend->resident_generation = generation;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_resident_detach(yvex_backend *backend, yvex_error *err) {
    if (backend) {
        backend->resident_host_base = NULL;
        backend->resident_host_bytes = backend->resident_device_address = backend->resident_generation = 0ull;
    }
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_resident_resolve(const yvex_backend *backend, const unsigned char *host, unsigned long long bytes,
                                  unsigned long long *device_address) {
    unsigned long long offset;
    if (device_address) *device_address = 0ull;
    if (!backend || backend->closing || atomic_load(&((yvex_backend *)backend)->status) == YVEX_BACKEND_STATUS_FAILED || !host ||
        !bytes || !device_address || !backend->resident_host_base)
        return YVEX_BACKEND_RESIDENT_MISS;
    if ((uintptr_t)host < (uintptr_t)backend->resident_host_base) return YVEX_BACKEND_RESIDENT_MISS;
    offset = (unsigned long long)((uintptr_t)host - (uintptr_t)backend->resident_host_base);
    if (offset > backend->resident_host_bytes || bytes > backend->resident_host_bytes - offset) return YVEX_BACKEND_RESIDENT_MISS;
    if (backend->resident_device_address > UINT64_MAX - offset) return YVEX_BACKEND_RESIDENT_INVALID;
    *device_address = backend->resident_device_address + offset;
    return YVEX_BACKEND_RESIDENT_HIT;
}

int yvex_backend_workspace_attach(yvex_backend *backend, yvex_device_tensor *workspace, yvex_error *err) {
    int rc = yvex_backend_admit(backend, "yvex_backend_workspace_attach", err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_tensor_owned(backend, workspace)) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_workspace_attach", "workspace must belong to this backend");
    backend->workspace = workspace;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_workspace_detach(yvex_backend *backend, yvex_error *err) {
    if (backend) backend->workspace = NULL;
    yvex_error_clear(err);
    return YVEX_OK;
}

/* 256-byte aligned bump range inside the attached workspace (src/backend/cuda/moe.c:78-88). */
unsigned char *yvex_workspace_take(yvex_backend *backend, unsigned long long *cursor, unsigned long long bytes) {
    unsigned long long at = (*cursor + 255ull) & ~255ull;
    if (!backend->workspace || at + bytes > backend->workspace->bytes) return NULL;
    *cursor = at + bytes;
    return backend->workspace->data + at;
}

/* ---- capability ----------------------------------------------------------------------------------- */

int yvex_backend_qtype_supported(const yvex_backend *backend, unsigned int qtype) {
    return backend && yvex_b200_qtype_supported(qtype);
}

int yvex_backend_query_capability(const yvex_backend *backend, int variant, yvex_backend_capability_result *out, yvex_error *err) {
    if (!backend || !out || variant < 0 || variant >= YVEX_BACKEND_VARIANT_COUNT)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "yvex_backend_query_capability", "arguments are invalid");
    memset(out, 0, sizeof(*out));
    out->backend_kind = backend->kind;
    out->variant = variant;
    out->context_available = 1;
    if (atomic_load(&((yvex_backend *)backend)->status) == YVEX_BACKEND_STATUS_FAILED) out->state = YVEX_BACKEND_CAPABILITY_FAILED;
    else if (variant >= YVEX_BACKEND_VARIANT_ATTENTION_CAUSAL_F32) { out->state = YVEX_BACKEND_CAPABILITY_SUPPORTED; out->function_available = 1; }
    else out->state = YVEX_BACKEND_CAPABILITY_UNSUPPORTED;       /* embed / norm / rope / dense matmul / mlp: not on this path */
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_op_embed(yvex_backend *backend, const yvex_device_tensor *embedding, const unsigned int *token_ids,
                          unsigned long long token_count, yvex_device_tensor *out, yvex_error *err) {
    (void)backend; (void)embedding; (void)token_ids; (void)token_count; (void)out;
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "yvex_backend_op_embed", "operation is outside the quantized MoE path of this backend");
}

int yvex_backend_op_rms_norm(yvex_backend *backend, const yvex_device_tensor *input, const yvex_device_tensor *weight, float epsilon,
                             yvex_device_tensor *out, yvex_error *err) {
    (void)backend; (void)input; (void)weight; (void)epsilon; (void)out;
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "yvex_backend_op_rms_norm", "operation is outside the quantized MoE path of this backend");
}

int yvex_backend_op_matmul(yvex_backend *backend, const yvex_device_tensor *input, const yvex_device_tensor *weight,
                           yvex_device_tensor *out, yvex_error *err) {
    (void)backend; (void)input; (void)weight; (void)out;
    return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, "yvex_backend_op_matmul", "operation is outside the quantized MoE path of this backend");
}

/* ---- status word --------------------------------------------------------------------------------- */

/* Reads and clears the device status word (stream is synchronised). 0 ok, else the kernel's code. */
int yvex_backend_take_status(yvex_backend *backend, int *code) {
    int *host = (int *)backend->host_scratch;
    *code = 0;
    if (cudaMemcpyAsync(host, backend->status_word, sizeof(int), cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess ||
        cudaStreamSynchronize(backend->stream) != cudaSuccess)
        return 0;
    *code = *host;
    if (*code && cudaMemsetAsync(backend->status_word, 0, sizeof(int), backend->stream) != cudaSuccess) return 0;
    return 1;
}

int yvex_backend_selftest_bounded_wait(yvex_backend *backend, unsigned long long limit_ns, unsigned long long *elapsed_ns,
                                       yvex_error *err) {
    const char *where = "cuda.selftest.bounded-wait";
    unsigned long long *dev_elapsed, *host_elapsed;
    int rc = yvex_backend_admit(backend, where, err), code;
    if (elapsed_ns) *elapsed_ns = 0ull;
    if (rc != YVEX_OK) return rc;
    dev_elapsed = (unsigned long long *)((unsigned char *)backend->status_word + 64);
    host_elapsed = (unsigned long long *)(backend->host_scratch + 64);
    rc = yvex_b200_selftest_bounded_wait(limit_ns, (uint64_t *)dev_elapsed, backend->status_word, backend->stream);
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "limit must be between 1 ns and 5 s");
    if (cudaMemcpyAsync(host_elapsed, dev_elapsed, sizeof(*host_elapsed), cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess ||
        !yvex_backend_take_status(backend, &code))
        return yvex_backend_fail(backend, where, err);
    if (elapsed_ns) *elapsed_ns = *host_elapsed;
    if (code == YVEX_B200_STATUS_TIMEOUT) return yvex_refuse(err, YVEX_ERR_TIMEOUT, where, "a bounded device wait expired");
    return yvex_refuse(err, YVEX_ERR_BACKEND, where, "the wait did not expire or reported another status");
}

/* ---- encoded matvec -------------------------------------------------------------------------------- */

/* Backend-owned device scratch of at least `bytes` (prepared activation rows, row ids); grown on demand. */
static unsigned char *act_scratch(yvex_backend *backend, unsigned long long bytes) {
    if (backend->act_scratch_bytes < bytes) {
        void *fresh = NULL;
        if (cudaStreamSynchronize(backend->stream) != cudaSuccess) return NULL;
        if (backend->act_scratch && cudaFree(backend->act_scratch) != cudaSuccess) return NULL;
        backend->act_scratch = NULL;
        backend->act_scratch_bytes = 0ull;
        if (cudaMalloc(&fresh, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return NULL; }
        backend->act_scratch = (unsigned char *)fresh;
        backend->act_scratch_bytes = bytes;
    }
    return backend->act_scratch;
}

/* The qtypes whose rows the reference multiplies by Q8_K activations (src/backend/cuda/kernel_primitives.h:556-564). */
static int q8_activation_eligible(unsigned int qtype) { return qtype == 16u || qtype == 10u || qtype == 8u || qtype == 39u; }

int yvex_backend_cuda_encoded_matvec(yvex_backend *backend, const unsigned char *resident_encoded,
    unsigned long long encoded_bytes, unsigned int qtype, unsigned long long row_count,
    unsigned long long row_width, unsigned long long row_bytes, unsigned long long input_rows,
    const yvex_device_tensor *input, const yvex_device_tensor *input_tail, unsigned long long input_head_width,
    const yvex_device_tensor *additive, yvex_device_tensor *output, int activation_q8,
    yvex_backend_cuda_operation_facts *facts, yvex_error *err) {
    const char *where = "cuda.encoded-matvec";
    unsigned long long device_address = 0ull, launches0, temporary = sizeof(int);
    const int split = input_tail != NULL;
    const float *rows_in;
    int rc, code, q8_path;
    if (facts) memset(facts, 0, sizeof(*facts));
    if (activation_q8 != 0 && activation_q8 != 1)
        return yvex_refuse(err, YVEX_ERR_INVALID_ARG, "cuda.encoded-matvec.activation",
                           "activation Q8 policy must be explicitly disabled or enabled");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_b200_qtype_supported(qtype))
        return yvex_refuse(err, YVEX_ERR_UNSUPPORTED, where, "qtype has no device decoder in this backend");
    q8_path = activation_q8 && !split && row_width % 256ull == 0ull && q8_activation_eligible(qtype);
    if (!resident_encoded || !encoded_bytes || !row_count || !input_rows || !row_width || !row_bytes || !facts ||
        split != (input_head_width != 0ull) || (split && input_head_width >= row_width) ||
        row_count > UINT64_MAX / row_bytes || row_count * row_bytes != encoded_bytes ||
        !yvex_tensor_owned(backend, input) || !input->is_written || input->dtype != YVEX_DTYPE_F32 ||
        input->bytes < input_rows * (split ? input_head_width : row_width) * 4ull ||
        (split && (!yvex_tensor_owned(backend, input_tail) || !input_tail->is_written || input_tail->dtype != YVEX_DTYPE_F32 ||
                   input_tail->bytes < input_rows * (row_width - input_head_width) * 4ull || input_tail == output)) ||
        !yvex_tensor_owned(backend, output) || output->dtype != YVEX_DTYPE_F32 ||
        output->bytes < input_rows * row_count * 4ull ||
        (additive && (!yvex_tensor_owned(backend, additive) || additive->dtype != YVEX_DTYPE_F32 || !additive->is_written ||
                      additive->bytes < input_rows * row_count * 4ull || additive == output)) ||
        yvex_backend_resident_resolve(backend, resident_encoded, encoded_bytes, &device_address) != YVEX_BACKEND_RESIDENT_HIT)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "resident encoded matvec geometry or ownership is incompatible");
    output->is_written = 0;
    /* host-side fault seams, as the reference has them in front of its copies and its launch
     * (src/backend/cuda/qtype.c:625-661): a refused copy fails the call and the backend recovers,
     * a failed launch demotes the backend for good */
    if (yvex_test_seam("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "input"))
        return yvex_refuse(err, YVEX_ERR_BACKEND, "cuda.encoded-matvec.copy_input", "injected CUDA qtype input copy failure");
    if (yvex_test_seam("YVEX_TEST_CUDA_LAUNCH_FAILURE", "encoded-matvec")) return yvex_backend_fail(backend, "cuda.encoded-matvec.launch", err);
    launches0 = yvex_b200_launch_count();
    rows_in = (const float *)input->data;
    if (q8_path || split) {
        /* the variant's view of the input rows, written once to backend-owned scratch */
        float *prepared = (float *)act_scratch(backend, input_rows * row_width * 4ull);
        if (!prepared) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "no device memory for the prepared activation rows");
        rc = q8_path ? yvex_b200_q8k_round_trip(rows_in, input_rows, row_width, prepared, backend->status_word, backend->stream)
                     : yvex_b200_concat_bf16(rows_in, (const float *)input_tail->data, input_head_width, row_width, input_rows, prepared,
                                             backend->status_word, backend->stream);
        if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
        if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the activation rows");
        rows_in = prepared;
        temporary += input_rows * row_width * 4ull;
    }
    rc = yvex_b200_gemv(qtype, (const void *)(uintptr_t)device_address, row_count, row_width, row_bytes, rows_in,
                        input_rows, additive ? (const float *)additive->data : NULL, (float *)output->data, 0, backend->status_word,
                        backend->stream);
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the matvec geometry");
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, "cuda.encoded-matvec.sync", err);
    if (code) return yvex_refuse(err, code == 3 ? YVEX_ERR_TIMEOUT : YVEX_ERR_FORMAT, where, "encoded CUDA projection produced invalid numerics");
    if (yvex_test_seam("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "output"))
        return yvex_refuse(err, YVEX_ERR_BACKEND, "cuda.encoded-matvec.copy_output", "injected CUDA qtype output copy failure");
    output->is_written = 1;
    facts->kernel_launches = yvex_b200_launch_count() - launches0;
    facts->tensor_core_launches = facts->kernel_launches;
    facts->stream_synchronizations = 1;
    facts->d2h_bytes = sizeof(int);
    facts->download_count = 1;
    facts->active_weight_bytes = encoded_bytes;
    facts->activation_bytes = input_rows * row_width * 4ull + input_rows * row_count * 4ull * (additive ? 2ull : 1ull);
    facts->temporary_bytes = temporary;
    facts->compulsory_memory_facts_available = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_cuda_encoded_gather(yvex_backend *backend, const unsigned char *resident_encoded,
    unsigned long long encoded_bytes, unsigned int qtype, unsigned long long row_count, unsigned long long row_width,
    unsigned long long row_bytes, const unsigned int *row_ids, unsigned long long selected_rows, yvex_device_tensor *output,
    yvex_backend_cuda_operation_facts *facts, yvex_error *err) {
    const char *where = "cuda.encoded-gather";
    unsigned long long device_address = 0ull, i;
    unsigned int be = 0, bb = 0;
    unsigned char *ids;
    int rc, code;
    if (facts) memset(facts, 0, sizeof(*facts));
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_b200_qtype_supported(qtype) || !yvex_b200_qtype_geometry(qtype, &be, &bb) || !be)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "resident encoded gather geometry or ownership is incompatible");
    if (!resident_encoded || !encoded_bytes || !row_count || !row_width || !row_bytes || !row_ids || !selected_rows || !facts ||
        row_width % be || row_width / be * bb != row_bytes || row_count > UINT64_MAX / row_bytes || row_count * row_bytes != encoded_bytes ||
        selected_rows > UINT64_MAX / (row_width * 4ull) || !yvex_tensor_owned(backend, output) || output->dtype != YVEX_DTYPE_F32 ||
        output->bytes < selected_rows * row_width * 4ull ||
        yvex_backend_resident_resolve(backend, resident_encoded, encoded_bytes, &device_address) != YVEX_BACKEND_RESIDENT_HIT)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "resident encoded gather geometry or ownership is incompatible");
    output->is_written = 0;
    for (i = 0; i < selected_rows; ++i)
        if ((unsigned long long)row_ids[i] >= row_count)
            return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "encoded gather row identifier exceeds the resident matrix");
    ids = act_scratch(backend, selected_rows * 4ull);
    if (!ids) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "no device memory for the row identifiers");
    /* the ids are copied from pageable memory: the call returns only after the stream is idle, so the source stays valid */
    if (cudaMemcpyAsync(ids, row_ids, (size_t)(selected_rows * 4ull), cudaMemcpyHostToDevice, backend->stream) != cudaSuccess)
        return yvex_backend_fail(backend, where, err);
    rc = yvex_b200_dequant_gather(qtype, (const void *)(uintptr_t)device_address, row_count, row_width, row_bytes, (const uint32_t *)ids,
                                  selected_rows, (float *)output->data, backend->status_word, backend->stream);
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the gather geometry");
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, "cuda.encoded-gather.sync", err);
    if (code) return yvex_refuse(err, YVEX_ERR_FORMAT, where, "encoded CUDA gather produced invalid numerics");
    output->is_written = 1;
    facts->h2d_bytes = selected_rows * 4ull;
    facts->d2h_bytes = sizeof(int);
    facts->kernel_launches = 1ull;
    facts->upload_count = 1ull;
    facts->download_count = 1ull;
    facts->stream_synchronizations = 1ull;
    facts->active_weight_bytes = selected_rows * row_bytes;
    facts->activation_bytes = selected_rows * row_width * 4ull;
    facts->temporary_bytes = selected_rows * 4ull + sizeof(int);
    facts->compulsory_memory_facts_available = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

/* One encoded row against one f32 vector, both in HOST memory (src/backend/cuda/qtype.c:527-700): the row and the
 * vector go up, a one-row dequant matvec runs, the f32 result comes back. Every refusal fills `failure` the way
 * cuda_quant_fail does (src/backend/cuda/qtype.c:81-103) besides the error. */
static int row_dot_fail(yvex_quant_failure *failure, int code, unsigned int qtype, unsigned long long expected, unsigned long long actual,
                        yvex_error *err, int status, const char *message) {
    if (failure) {
        memset(failure, 0, sizeof(*failure));
        failure->code = code;
        failure->terminal_ordinal = failure->source_index = failure->block_index = ~0ull;
        failure->expected = expected;
        failure->actual = actual;
        failure->qtype = qtype;
        failure->operation = YVEX_TRANSFORM_OP_COUNT;
    }
    return yvex_refuse(err, (yvex_status)status, "cuda.quant.row_dot", message);
}

int yvex_cuda_quant_row_dot(yvex_backend *backend, unsigned int qtype, const unsigned char *encoded, size_t encoded_bytes,
                            const float *vector, unsigned long long elements, float *out, yvex_quant_failure *failure, yvex_error *err) {
    const char *where = "cuda.quant.row_dot";
    unsigned int be = 0, bb = 0;
    unsigned long long row_bytes, vector_bytes, enc_room;
    unsigned char *scratch;
    float *host_out;
    int rc, code;
    if (failure) memset(failure, 0, sizeof(*failure));
    yvex_error_clear(err);
    if (!backend || !encoded || !vector || !out || !elements || ((uintptr_t)vector % 4u) != 0u || ((uintptr_t)out % 4u) != 0u ||
        ((qtype == 0u || qtype == 26u) && ((uintptr_t)encoded % 4u) != 0u) || ((qtype == 1u || qtype == 30u) && ((uintptr_t)encoded % 2u) != 0u))
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_INVALID_ARGUMENT, qtype, 1ull, 0ull, err, YVEX_ERR_INVALID_ARG,
                            "CUDA encoded row, aligned vector/result, and backend are required");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_b200_qtype_supported(qtype) || !yvex_b200_qtype_geometry(qtype, &be, &bb) || !be)
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_CUDA_COMPUTE_UNAVAILABLE, qtype, 1ull, 0ull, err, YVEX_ERR_UNSUPPORTED,
                            "qtype has no dedicated CUDA numeric contract");
    if (elements % be)
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_ROW_DIVISIBILITY, qtype, be, elements, err, YVEX_ERR_BOUNDS,
                            "CUDA qtype row does not satisfy canonical block geometry");
    row_bytes = elements / be * bb;
    if (row_bytes != (unsigned long long)encoded_bytes || elements > SIZE_MAX / sizeof(float))
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_BYTE_OVERFLOW, qtype, row_bytes, encoded_bytes, err, YVEX_ERR_BOUNDS,
                            "CUDA encoded row byte geometry is inconsistent");
    vector_bytes = elements * 4ull;
    enc_room = (row_bytes + 255ull) & ~255ull;
    scratch = act_scratch(backend, enc_room + vector_bytes + 256ull);
    if (!scratch) return row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, err, YVEX_ERR_NOMEM, "no device memory for the row and the vector");
    if (yvex_test_seam("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "input"))
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, err, YVEX_ERR_BACKEND, "injected CUDA qtype input copy failure");
    /* pageable sources: the call returns only after the stream is idle, so they stay valid */
    if (cudaMemcpyAsync(scratch, encoded, (size_t)row_bytes, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess ||
        cudaMemcpyAsync(scratch + enc_room, vector, (size_t)vector_bytes, cudaMemcpyHostToDevice, backend->stream) != cudaSuccess) {
        row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, NULL, YVEX_ERR_BACKEND, "");
        return yvex_backend_fail(backend, where, err);
    }
    rc = yvex_b200_gemv(qtype, scratch, 1ull, elements, row_bytes, (const float *)(scratch + enc_room), 1ull, NULL,
                        (float *)(scratch + enc_room + vector_bytes), 0, backend->status_word, backend->stream);
    if (rc == YVEX_ERR_BACKEND) {
        row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, NULL, YVEX_ERR_BACKEND, "");
        return yvex_backend_fail(backend, where, err);
    }
    if (rc != YVEX_OK) return row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, err, rc, "CUDA qtype encoded-row execution failed");
    host_out = (float *)(backend->host_scratch + 1024);
    if (cudaMemcpyAsync(host_out, scratch + enc_room + vector_bytes, sizeof(float), cudaMemcpyDeviceToHost, backend->stream) != cudaSuccess ||
        !yvex_backend_take_status(backend, &code)) {
        row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, NULL, YVEX_ERR_BACKEND, "");
        return yvex_backend_fail(backend, where, err);
    }
    if (code) return row_dot_fail(failure, YVEX_QUANT_FAILURE_NONFINITE, qtype, 1ull, 0ull, err, YVEX_ERR_FORMAT,
                                  "CUDA qtype row held a malformed block or produced a non-finite sum");
    if (yvex_test_seam("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "output"))
        return row_dot_fail(failure, YVEX_QUANT_FAILURE_WORKER, qtype, 1ull, 0ull, err, YVEX_ERR_BACKEND, "injected CUDA qtype output copy failure");
    *out = *host_out;
    if (failure) memset(failure, 0, sizeof(*failure));
    yvex_error_clear(err);
    return YVEX_OK;
}

/* ---- attention ---------------------------------------------------------------------------------------- */

int yvex_backend_op_attention(yvex_backend *backend, const yvex_device_tensor *query, const yvex_device_tensor *keys,
                              const yvex_device_tensor *values, unsigned long long seq_len, unsigned long long position,
                              float scale, int causal, yvex_device_tensor *score_scratch,
                              yvex_device_tensor *probability_scratch, yvex_device_tensor *out, yvex_error *err) {
    const char *where = "yvex_backend_op_attention";
    const yvex_device_tensor *all[6] = {query, keys, values, score_scratch, probability_scratch, out};
    unsigned long long head_dim;
    int rc, code, i;
    if (!(scale > 0.0f) || scale > 3.0e38f) return yvex_refuse(err, YVEX_ERR_INVALID_ARG, where, "scale must be finite and positive");
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    for (i = 0; i < 6; ++i)
        if (!yvex_tensor_owned(backend, all[i]) || all[i]->dtype != YVEX_DTYPE_F32)
            return yvex_refuse(err, YVEX_ERR_FORMAT, where, "attention primitive supports F32 Q/K/V, scratches, and output of this backend");
    if (!seq_len || query->rank != 1 || !query->dims[0])
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, seq_len ? "attention query must be rank 1 with non-zero head_dim" : "attention-seq-len-zero");
    if (position >= seq_len) return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "position-out-of-range");
    head_dim = query->dims[0];
    if (keys->rank != 2 || keys->dims[0] != seq_len || keys->dims[1] != head_dim || values->rank != 2 ||
        values->dims[0] != seq_len || values->dims[1] != head_dim)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "attention keys and values must have dims [seq_len, head_dim]");
    if (score_scratch->dims[0] != seq_len || probability_scratch->dims[0] != seq_len || out->dims[0] != head_dim)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "attention scratches must have dims [seq_len], output [head_dim]");
    if (query->bytes < head_dim * 4 || keys->bytes < seq_len * head_dim * 4 || values->bytes < seq_len * head_dim * 4 ||
        score_scratch->bytes < seq_len * 4 || probability_scratch->bytes < seq_len * 4 || out->bytes < head_dim * 4)
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "attention tensor bytes must match F32 shape accounting");
    rc = yvex_b200_attention_f32((const float *)query->data, (const float *)keys->data, (const float *)values->data, seq_len, head_dim,
                                 position, scale, causal, (float *)score_scratch->data, (float *)probability_scratch->data,
                                 (float *)out->data, backend->status_word, backend->stream);
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the attention geometry");
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, where, err);
    if (code) return yvex_refuse(err, YVEX_ERR_STATE, where, "attention softmax sum is zero");
    score_scratch->is_written = probability_scratch->is_written = out->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}

int yvex_backend_attention_gqa_decode(yvex_backend *backend, const yvex_device_tensor *query, const yvex_device_tensor *keys,
                                      const yvex_device_tensor *values, unsigned long long sessions, unsigned long long q_heads,
                                      unsigned long long kv_heads, unsigned long long head_dim, unsigned long long context,
                                      unsigned long long position, float scale, yvex_device_tensor *out, yvex_error *err) {
    const char *where = "yvex_backend_attention_gqa_decode";
    unsigned long long need, cursor = 0;
    unsigned char *scratch;
    int rc, code;
    rc = yvex_backend_admit(backend, where, err);
    if (rc != YVEX_OK) return rc;
    if (!yvex_tensor_owned(backend, query) || !yvex_tensor_owned(backend, keys) || !yvex_tensor_owned(backend, values) ||
        !yvex_tensor_owned(backend, out) || query->dtype != YVEX_DTYPE_BF16 || keys->dtype != YVEX_DTYPE_BF16 ||
        values->dtype != YVEX_DTYPE_BF16 || out->dtype != YVEX_DTYPE_F32 || !query->is_written || !keys->is_written || !values->is_written)
        return yvex_refuse(err, YVEX_ERR_FORMAT, where, "GQA decode takes written BF16 Q/K/V and an F32 output of this backend");
    if (!sessions || !q_heads || !kv_heads || !head_dim || !context || query->bytes < sessions * q_heads * head_dim * 2 ||
        keys->bytes < sessions * kv_heads * context * head_dim * 2 || values->bytes < sessions * kv_heads * context * head_dim * 2 || out->bytes < sessions * q_heads * head_dim * 4)
        return yvex_refuse(err, YVEX_ERR_BOUNDS, where, "tensor bytes do not cover the stated geometry");
    need = yvex_b200_attention_workspace_bytes(sessions, q_heads, kv_heads, head_dim, context);
    scratch = yvex_workspace_take(backend, &cursor, need);
    if (!scratch) return yvex_refuse(err, YVEX_ERR_NOMEM, where, "attached workspace is too small for the split-KV partials");
    out->is_written = 0;
    rc = yvex_b200_attention_gqa_decode(query->data, keys->data, values->data, sessions, q_heads, kv_heads, head_dim, context, position,
                                        scale, (float *)out->data, scratch, need, backend->status_word, backend->stream);
    if (rc == YVEX_ERR_BACKEND) return yvex_backend_fail(backend, where, err);
    if (rc != YVEX_OK) return yvex_refuse(err, (yvex_status)rc, where, "device layer refused the attention geometry");
    if (!yvex_backend_take_status(backend, &code)) return yvex_backend_fail(backend, where, err);
    if (code) return yvex_refuse(err, YVEX_ERR_BACKEND, where, "attention kernel reported invalid numerics");
    out->is_written = 1;
    yvex_error_clear(err);
    return YVEX_OK;
}
