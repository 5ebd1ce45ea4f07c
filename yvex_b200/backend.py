"""ctypes mirror of the C11 host boundary (include/yvex_b200_backend.h) for the tests and the
end-to-end leg of the benchmark. Every call goes through the shared library; nothing here computes."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .lib import lib as _lib

ull, vp = C.c_ulonglong, C.c_void_p
OK, NOMEM, FORMAT, UNSUPPORTED, BACKEND, BOUNDS, STATE, CANCELLED, INVALID_ARG, TIMEOUT = 0, -2, -4, -5, -6, -7, -8, -9, -10, -11
KIND_CPU, KIND_CUDA, KIND_METAL = 0, 1, 2
F32, F16, BF16, I32, U8 = 1, 2, 3, 4, 5
(W_FFN_NORM, W_MHC_FUNCTION, W_MHC_BASE, W_MHC_SCALE, W_ROUTER, W_ROUTER_TABLE, W_ROUTER_BIAS, W_GATE, W_UP, W_DOWN,
 W_SHARED_GATE, W_SHARED_UP, W_SHARED_DOWN, W_COUNT) = range(14)


class Error(C.Structure):
    _fields_ = [("code", C.c_int), ("where", C.c_char * 96), ("message", C.c_char * 256)]


class Options(C.Structure):
    _fields_ = [("kind", C.c_int), ("device", C.c_char_p), ("memory_limit_bytes", ull)]


class TensorDesc(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int), ("rank", C.c_uint), ("dims", ull * 4), ("bytes", ull)]


class DeviceTensor(C.Structure):
    _fields_ = [("owner", vp), ("owner_id", ull), ("dtype", C.c_int), ("rank", C.c_uint), ("dims", ull * 4), ("bytes", ull),
                ("data", vp), ("host_data", vp), ("is_written", C.c_int)]


class Facts(C.Structure):
    _fields_ = [(n, ull) for n in ("h2d_bytes", "d2h_bytes", "d2d_bytes", "kernel_launches", "upload_count", "download_count",
                                   "stream_synchronizations", "device_synchronizations", "active_weight_bytes", "state_bytes",
                                   "activation_bytes", "temporary_bytes", "tensor_core_launches")] + [("available", C.c_int)]


HEX = C.c_char * 65
ROW_BATCH_SCHEMA_V1, ROW_BATCH_SCHEMA_LOGITS, ROW_BATCH_RESULT_SCHEMA_V4 = 1, 0x42320001, 4
EXECUTION_CLASS_DEVICE_NATIVE = 1


class MemoryFacts(C.Structure):
    """yvex_execution_memory_facts (include/yvex/internal/execution.h:329-333)."""
    _fields_ = [(n, ull) for n in ("active_weight_bytes", "state_bytes", "activation_bytes", "temporary_bytes",
                                   "measured_operations", "missing_operations")] + [("complete", C.c_int)]


class WeightView(C.Structure):
    """yvex_moe_weight_view, field for field (include/yvex/internal/moe.h:54-64)."""
    _fields_ = [("tensor_id", ull), ("expert_index", ull), ("role", C.c_int), ("qtype", C.c_uint), ("layout", C.c_int),
                ("activation", C.c_int), ("kernel_family", C.c_char_p), ("encoded", vp), ("encoded_bytes", C.c_size_t),
                ("storage_bytes", C.c_size_t), ("row_bytes", ull), ("row_width", ull), ("row_count", ull), ("device_address", ull)]


class LayerPlan(C.Structure):
    """yvex_moe_layer_plan (include/yvex/internal/moe.h:65-84)."""
    _fields_ = [("schema_version", C.c_uint), ("ordinal", ull), ("layer_index", ull), ("predictor_index", ull),
                ("tensor_scope", C.c_int), ("router_class", C.c_int), ("scoring", C.c_int), ("topk_policy", C.c_int),
                ("activation", C.c_int),
                ("hidden_width", ull), ("residual_streams", ull), ("expanded_width", ull),
                ("mhc_mixing_rows", ull), ("mhc_sinkhorn_iterations", ull),
                ("routed_experts", ull), ("shared_experts", ull), ("experts_per_token", ull),
                ("expert_intermediate_width", ull), ("shared_intermediate_width", ull), ("hash_table_rows", ull),
                ("hash_table_columns", ull), ("correction_bias_width", ull),
                ("rms_epsilon", C.c_double), ("mhc_epsilon", C.c_double), ("mhc_post_multiplier", C.c_double),
                ("routed_scaling_factor", C.c_double), ("activation_limit", C.c_double),
                ("requires_token_ids", C.c_int), ("requires_correction_bias", C.c_int), ("normalize_topk_probabilities", C.c_int),
                ("tensor_ids", ull * W_COUNT), ("qtypes", C.c_uint * W_COUNT), ("layer_identity", HEX)]


class WorklistObservation(C.Structure):
    """yvex_expert_worklist_observation (include/yvex/internal/execution_batch.h:126-137)."""
    _fields_ = [("schema_version", C.c_uint), ("worklist_count", ull), ("pair_count", ull), ("bucket_count", ull),
                ("maximum_bucket_population", ull), ("tensor_core_eligible_pairs", ull), ("tensor_core_executed_pairs", ull),
                ("narrow_pairs", ull), ("tail_rows", ull), ("width_histogram", ull * 17), ("population_histogram", ull * 17),
                ("provenance_counts", ull * 5)]


class CompletionSlot(C.Structure):
    """yvex_moe_device_completion_slot (include/yvex/internal/moe.h:182-189)."""
    _fields_ = [("row_count", ull), ("row_expert_pairs", ull), ("worklist", WorklistObservation),
                ("tensor_core_executed_pairs", ull), ("routed_experts", ull), ("active_base_bytes", ull),
                ("active_per_expert_bytes", ull), ("activation_bytes", ull), ("temporary_bytes", ull),
                ("status", C.c_int), ("pending", C.c_int)]


class Completion(C.Structure):
    _fields_ = [("defer", C.c_int), ("host", C.POINTER(CompletionSlot))]


CANCEL_FN = C.CFUNCTYPE(C.c_int, vp)


class LayerJob(C.Structure):
    """yvex_moe_layer_job (include/yvex/internal/moe.h:194-209)."""
    _fields_ = [("layer", C.POINTER(LayerPlan)), ("weights", WeightView * W_COUNT), ("expanded_input", vp),
                ("device_input", C.POINTER(DeviceTensor)), ("device_output", C.POINTER(DeviceTensor)),
                ("token_id", C.c_uint), ("token_id_present", C.c_int), ("cancel_requested", CANCEL_FN),
                ("cancel_context", vp), ("evidence_level", C.c_int), ("eager_execution", C.c_int),
                ("device_completion", C.POINTER(Completion)), ("execution_batch", vp), ("worklist_policy", vp)]


class RowBatch(C.Structure):
    """yvex_moe_row_batch (include/yvex/internal/moe.h:232-247)."""
    _fields_ = [("schema_version", C.c_uint), ("row_count", ull), ("row_width", ull), ("row_stride", ull),
                ("expanded_rows", vp), ("device_rows", C.POINTER(DeviceTensor)), ("device_outputs", C.POINTER(DeviceTensor)),
                ("token_ids", vp), ("token_ids_present", C.c_int), ("provenance", C.c_int), ("phase", C.c_uint),
                ("execution_class", C.c_int), ("execution_profile_identity", C.c_char_p), ("execution_sources", vp),
                ("execution_rows", vp), ("execution_source_count", ull), ("complete_after_operation", C.c_int)]


class RowBatchLogits(C.Structure):
    """The extension that carries caller-supplied router logits behind a reference-shaped batch."""
    _fields_ = [("base", RowBatch), ("router_logits", vp), ("device_router_logits", C.POINTER(DeviceTensor))]


def row_batch(rows, width, host_rows=None, device_rows=None, device_outputs=None, router_logits=None,
              device_router_logits=None, token_ids=None, provenance=None):
    """A row batch; with logits the extended struct (pass it to the table by reference like a plain batch)."""
    base = RowBatch(ROW_BATCH_SCHEMA_V1, rows, width, width, host_rows, device_rows, device_outputs, token_ids,
                    1 if token_ids else 0, (0 if rows == 1 else 2) if provenance is None else provenance, 0,
                    EXECUTION_CLASS_DEVICE_NATIVE, None, None, None, 0, 0)
    if router_logits is None and device_router_logits is None:
        return base
    base.schema_version = ROW_BATCH_SCHEMA_LOGITS
    return RowBatchLogits(base, router_logits, device_router_logits)


class RowBatchOutput(C.Structure):
    """yvex_moe_row_batch_output (include/yvex/internal/moe.h:249-256)."""
    _fields_ = [("combined_rows", vp), ("routed_rows", vp), ("shared_rows", vp), ("post_rows", vp), ("combination_rows", vp),
                ("combined_capacity", ull), ("routed_capacity", ull), ("shared_capacity", ull), ("post_capacity", ull),
                ("combination_capacity", ull), ("selected_experts", vp), ("selected_weights", vp), ("selection_capacity", ull)]


def row_output(combined=None, combined_capacity=0, selected_experts=None, selected_weights=None, selection_capacity=0,
               routed=None, shared=None, post=None, combination=None, routed_capacity=0, shared_capacity=0, post_capacity=0,
               combination_capacity=0):
    return RowBatchOutput(combined, routed, shared, post, combination, combined_capacity, routed_capacity, shared_capacity,
                          post_capacity, combination_capacity, selected_experts, selected_weights, selection_capacity)


class RowBatchResult(C.Structure):
    """yvex_moe_row_batch_result (include/yvex/internal/moe.h:258-281)."""
    _fields_ = [("schema_version", C.c_uint), ("completed", C.c_int), ("execution_profile_available", C.c_int),
                ("device_completion_pending", C.c_int), ("execution_class", C.c_int)] + [
        (n, ull) for n in ("row_count", "row_expert_pairs", "unique_experts")] + [("worklists", WorklistObservation)] + [
        (n, ull) for n in ("grouped_expert_operations", "shared_expert_operations", "expert_subviews_accessed", "encoded_bytes_read",
                           "h2d_bytes", "d2h_bytes", "d2d_bytes", "kernel_launches", "tensor_core_launches", "graph_launches",
                           "graph_captures", "graph_replays", "upload_count", "download_count", "cache_hits", "cache_misses",
                           "stream_synchronizations", "device_synchronizations", "active_weight_base_bytes",
                           "active_weight_per_unique_expert_bytes")] + [("memory", MemoryFacts), ("total_ns", ull),
                                                                        ("synchronization_ns", ull)] + [
        (n, HEX) for n in ("execution_profile_identity", "execution_batch_identity", "worklist_policy_identity",
                           "expert_worklist_identity", "routing_digest", "execution_identity")]


class RouterResult(C.Structure):
    """yvex_moe_router_result (include/yvex/internal/moe.h:160-166)."""
    _fields_ = [("selected_count", ull), ("selected_experts", ull * 16), ("router_logits", C.c_float * 256),
                ("router_scores", C.c_float * 256), ("selected_weights", C.c_float * 16)]


class LayerResult(C.Structure):
    """yvex_moe_layer_result (include/yvex/internal/moe.h:198-214): the token-local transaction's outputs and counters."""
    _fields_ = [("combined_output", vp), ("post", vp), ("combination", vp)] + [
        (n, ull) for n in ("combined_capacity", "post_capacity", "combination_capacity")] + [("routed_output", vp), ("shared_output", vp)] + [
        (n, ull) for n in ("routed_capacity", "shared_capacity")] + [("router", RouterResult)] + [
        (n, ull) for n in ("expert_subviews_accessed", "encoded_bytes_read", "host_to_device_bytes", "device_to_host_bytes",
                           "kernel_launches", "cache_hits", "cache_misses", "upload_count", "download_count",
                           "stream_synchronizations", "device_synchronizations", "device_to_device_bytes")] + [
        ("memory", MemoryFacts)] + [(n, ull) for n in ("ingress_ns", "routing_ns", "routed_ns", "shared_ns", "post_ns", "total_ns",
                                                       "synchronization_ns")] + [("qtype_counts", ull * 43)] + [
        (n, HEX) for n in ("routed_digest", "shared_digest", "combined_digest", "routing_digest")]


_EXEC = C.CFUNCTYPE(C.c_int, vp, C.POINTER(LayerJob), vp, C.POINTER(RowBatchOutput), C.POINTER(RowBatchResult),
                    C.POINTER(Error))          # the batch by address: a RowBatch or a RowBatchLogits
_WSREQ = C.CFUNCTYPE(C.c_int, C.POINTER(LayerPlan), ull, C.POINTER(ull), C.POINTER(Error))


class MoeOperations(C.Structure):
    _fields_ = [("derived_layout_plan", C.CFUNCTYPE(C.c_int, vp, C.POINTER(ull), C.POINTER(Error))),
                ("derived_layout_build", C.CFUNCTYPE(C.c_int, vp, vp, ull, vp, ull, C.POINTER(Error))),
                ("workspace_required", _WSREQ), ("execute_rows", _EXEC),
                ("complete_rows", C.CFUNCTYPE(C.c_int, vp, C.c_int, C.POINTER(RowBatchResult), C.POINTER(Error))),
                ("workspace_required_wide", _WSREQ), ("execute_rows_wide", _EXEC)]


_lib.yvex_backend_moe_operations_get.restype = C.POINTER(MoeOperations)
_lib.yvex_backend_moe_operations_get.argtypes = [vp]
_lib.yvex_backend_moe_begin.argtypes = [C.POINTER(vp), vp, C.POINTER(LayerJob), C.POINTER(LayerResult), C.POINTER(Error)]
_lib.yvex_backend_moe_add_expert.argtypes = [vp, C.POINTER(WeightView), C.POINTER(WeightView), C.POINTER(WeightView), C.c_float, C.c_int,
                                             C.POINTER(Error)]
_lib.yvex_backend_moe_finish.argtypes = [vp, C.POINTER(LayerResult), C.POINTER(Error)]
_lib.yvex_backend_moe_close.argtypes = [C.POINTER(vp), C.POINTER(Error)]
class QuantFailure(C.Structure):
    """yvex_quant_failure (include/yvex/internal/quant_numeric.h:83-93)."""
    _fields_ = [("code", C.c_int)] + [(n, ull) for n in ("terminal_ordinal", "source_index", "row_index", "block_index", "expected", "actual")] + [
        ("qtype", C.c_uint), ("operation", C.c_int)]


_lib.yvex_cuda_quant_row_dot.argtypes = [vp, C.c_uint, vp, C.c_size_t, vp, ull, C.POINTER(C.c_float), C.POINTER(QuantFailure), C.POINTER(Error)]
_lib.yvex_moe_ep_unique_id.argtypes = [vp, C.POINTER(Error)]
_lib.yvex_moe_ep_open.argtypes = [C.POINTER(vp), vp, vp, C.c_uint, C.c_uint, ull, C.POINTER(Error)]
_lib.yvex_moe_ep_workspace_required.argtypes = [C.POINTER(LayerPlan), ull, C.c_uint, C.POINTER(ull), C.POINTER(Error)]
_lib.yvex_moe_ep_execute_rows.argtypes = [vp, C.POINTER(LayerJob), vp, C.POINTER(RowBatchOutput), C.POINTER(RowBatchResult), C.POINTER(Error)]
_lib.yvex_moe_ep_close.argtypes = [C.POINTER(vp), C.POINTER(Error)]
_lib.yvex_backend_open.argtypes = [C.POINTER(vp), C.POINTER(Options), C.POINTER(Error)]
_lib.yvex_backend_close_checked.argtypes = [C.POINTER(vp), C.POINTER(Error)]
_lib.yvex_backend_close.argtypes = [vp]
_lib.yvex_backend_tensor_alloc.argtypes = [vp, C.POINTER(TensorDesc), C.POINTER(C.POINTER(DeviceTensor)), C.POINTER(Error)]
_lib.yvex_backend_resident_alloc.argtypes = [vp, C.POINTER(TensorDesc), C.POINTER(C.POINTER(DeviceTensor)), C.POINTER(vp),
                                             C.POINTER(Error)]
_lib.yvex_backend_tensor_free.argtypes = [vp, C.POINTER(DeviceTensor)]
_lib.yvex_backend_tensor_write.argtypes = [vp, C.POINTER(DeviceTensor), vp, ull, C.POINTER(Error)]
_lib.yvex_backend_tensor_read.argtypes = [vp, C.POINTER(DeviceTensor), vp, ull, C.POINTER(Error)]
_lib.yvex_backend_resident_prefetch.argtypes = [vp, C.POINTER(DeviceTensor), C.POINTER(ull), C.POINTER(Error)]
_lib.yvex_backend_resident_attach.argtypes = [vp, vp, ull, C.POINTER(DeviceTensor), ull, C.POINTER(Error)]
_lib.yvex_backend_resident_detach.argtypes = [vp, C.POINTER(Error)]
_lib.yvex_backend_resident_resolve.argtypes = [vp, vp, ull, C.POINTER(ull)]
_lib.yvex_backend_workspace_attach.argtypes = [vp, C.POINTER(DeviceTensor), C.POINTER(Error)]
_lib.yvex_backend_workspace_detach.argtypes = [vp, C.POINTER(Error)]
_lib.yvex_backend_sync.argtypes = [vp, C.POINTER(Error)]
_lib.yvex_backend_status_of.argtypes = [vp]
_lib.yvex_backend_kind_of.argtypes = [vp]
_lib.yvex_backend_qtype_supported.argtypes = [vp, C.c_uint]
_lib.yvex_backend_cuda_encoded_matvec.argtypes = [vp, vp, ull, C.c_uint, ull, ull, ull, ull, C.POINTER(DeviceTensor),
                                                  C.POINTER(DeviceTensor), ull, C.POINTER(DeviceTensor), C.POINTER(DeviceTensor),
                                                  C.c_int, C.POINTER(Facts), C.POINTER(Error)]
_lib.yvex_backend_cuda_encoded_gather.argtypes = [vp, vp, ull, C.c_uint, ull, ull, ull, vp, ull, C.POINTER(DeviceTensor),
                                                  C.POINTER(Facts), C.POINTER(Error)]
_lib.yvex_backend_op_attention.argtypes = [vp] + [C.POINTER(DeviceTensor)] * 3 + [ull, ull, C.c_float, C.c_int] + \
    [C.POINTER(DeviceTensor)] * 3 + [C.POINTER(Error)]
_lib.yvex_backend_attention_gqa_decode.argtypes = [vp] + [C.POINTER(DeviceTensor)] * 3 + [ull] * 6 + [C.c_float,
                                                                                                    C.POINTER(DeviceTensor),
                                                                                                    C.POINTER(Error)]
_lib.yvex_backend_op_matmul.argtypes = [vp] + [C.POINTER(DeviceTensor)] * 3 + [C.POINTER(Error)]
class MoeInputSummary(C.Structure):
    _fields_ = [("schema_version", C.c_uint), ("token_start", ull), ("token_count", ull), ("layer_count", ull),
                ("activation_payload_bytes", ull), ("token_id_payload_bytes", ull)] + [
        (n, C.c_char * 65) for n in ("logical_model_identity", "runtime_numeric_identity", "runtime_descriptor_identity",
                                     "moe_plan_identity", "activation_payload_digest", "token_id_payload_digest", "input_identity")]


class MoeInputRecord(C.Structure):
    _fields_ = [(n, ull) for n in ("ordinal", "layer_index", "width", "stride", "payload_offset", "payload_bytes")] + [
        ("layer_identity", C.c_char * 65)]


class MoeInputLimits(C.Structure):
    _fields_ = [("maximum_file_bytes", ull)]


_lib.yvex_moe_input_open_file.argtypes = [C.POINTER(vp), C.c_char_p, C.POINTER(MoeInputLimits), C.POINTER(Error)]
_lib.yvex_moe_input_open_image.argtypes = [C.POINTER(vp), vp, ull, C.POINTER(Error)]
_lib.yvex_moe_input_summary_get.restype = C.POINTER(MoeInputSummary)
_lib.yvex_moe_input_summary_get.argtypes = [vp]
_lib.yvex_moe_input_layer_record_at.restype = C.POINTER(MoeInputRecord)
_lib.yvex_moe_input_layer_record_at.argtypes = [vp, ull]
_lib.yvex_moe_input_layer_view.argtypes = [vp, ull, C.POINTER(C.POINTER(C.c_float)), C.POINTER(ull), C.POINTER(Error)]
_lib.yvex_moe_input_token_ids.restype = C.POINTER(C.c_uint)
_lib.yvex_moe_input_token_ids.argtypes = [vp]
_lib.yvex_moe_input_close.argtypes = [C.POINTER(vp)]
_lib.yvex_moe_input_row_batch.argtypes = [vp, ull, C.POINTER(RowBatch), C.POINTER(Error)]
_lib.yvex_backend_moe_last_pipeline_chunks.restype = ull
_lib.yvex_backend_moe_last_pipeline_chunks.argtypes = [vp]
_lib.yvex_backend_abi_layout.restype = C.c_char_p
_lib.yvex_backend_selftest_bounded_wait.argtypes = [vp, ull, C.POINTER(ull), C.POINTER(Error)]
_lib.yvex_status_name.restype = C.c_char_p


class Backend:
    """Owns one yvex_backend; helpers return raw status codes so tests can assert refusals."""

    def __init__(self, kind=KIND_CUDA, device=b"cuda:0", memory_limit=0):
        self.handle, self.err = vp(), Error()
        opts = Options(kind, device, memory_limit)
        self.rc = _lib.yvex_backend_open(C.byref(self.handle), C.byref(opts), C.byref(self.err))
        self.tensors = []

    @property
    def h(self):
        return self.handle

    def message(self):
        return self.err.message.decode()

    def tensor(self, nbytes, dtype=U8, dims=None, resident=False):
        dims = list(dims or [nbytes])
        desc = TensorDesc(b"t", dtype, len(dims), (ull * 4)(*(dims + [0] * (4 - len(dims)))), nbytes)
        t, host = C.POINTER(DeviceTensor)(), vp()
        if resident:
            rc = _lib.yvex_backend_resident_alloc(self.h, C.byref(desc), C.byref(t), C.byref(host), C.byref(self.err))
        else:
            rc = _lib.yvex_backend_tensor_alloc(self.h, C.byref(desc), C.byref(t), C.byref(self.err))
        if rc != OK:
            return rc, None, None
        self.tensors.append(t)
        return rc, t, host.value

    def write(self, t, array):
        a = np.ascontiguousarray(array)
        return _lib.yvex_backend_tensor_write(self.h, t, a.ctypes.data_as(vp), a.nbytes, C.byref(self.err))

    def read(self, t, dtype, count):
        out = np.empty(count, dtype)
        rc = _lib.yvex_backend_tensor_read(self.h, t, out.ctypes.data_as(vp), out.nbytes, C.byref(self.err))
        return rc, out

    def from_array(self, array, dtype, dims=None):
        a = np.ascontiguousarray(array)
        rc, t, _ = self.tensor(a.nbytes, dtype, dims or list(a.shape))
        assert rc == OK, self.message()
        assert self.write(t, a) == OK, self.message()
        return t

    def free(self, t):
        _lib.yvex_backend_tensor_free(self.h, t)
        self.tensors = [x for x in self.tensors if C.addressof(x.contents) != C.addressof(t.contents)]

    def close(self):
        for t in list(self.tensors):
            _lib.yvex_backend_tensor_free(self.h, t)
        self.tensors = []
        return _lib.yvex_backend_close_checked(C.byref(self.handle), C.byref(self.err))


class ResidentArena:
    """Packs named host arrays into one resident arena (pinned host side + HBM side) and attaches it."""

    def __init__(self, backend, arrays, generation=1):
        self.backend = backend
        self.offsets, off = {}, 0
        for name, a in arrays.items():
            self.offsets[name] = off
            off = (off + a.nbytes + 255) & ~255
        rc, self.tensor, self.host = backend.tensor(max(off, 256), U8, resident=True)
        assert rc == OK, backend.message()
        self.bytes = max(off, 256)
        view = (C.c_ubyte * self.bytes).from_address(self.host)
        self.view = np.frombuffer(view, dtype=np.uint8)
        self.sizes = {}
        for name, a in arrays.items():
            flat = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
            self.view[self.offsets[name]:self.offsets[name] + flat.size] = flat
            self.sizes[name] = flat.size
        moved = ull()
        assert _lib.yvex_backend_resident_prefetch(backend.h, self.tensor, C.byref(moved), C.byref(backend.err)) == OK
        assert _lib.yvex_backend_resident_attach(backend.h, self.host, self.bytes, self.tensor, generation,
                                                 C.byref(backend.err)) == OK, backend.message()

    def host_ptr(self, name):
        return self.host + self.offsets[name]


def moe_job(arena, spec, router=True, router_class=1, hash_rows=0, family=None, residual_streams=1, envelope_policy=None):
    """LayerPlan + LayerJob whose weight views point (by host address) into `arena`."""
    from . import synth
    S = max(residual_streams, 1)
    policy = dict(sinkhorn_iterations=20, rms_epsilon=1e-6, mhc_epsilon=1e-6, post_multiplier=2.0)
    policy.update(envelope_policy or {})
    plan = LayerPlan(schema_version=1, router_class=router_class, hidden_width=spec.hidden, residual_streams=residual_streams,
                     expanded_width=spec.hidden * S, mhc_mixing_rows=(S + 2) * S if residual_streams > 1 else 0,
                     mhc_sinkhorn_iterations=policy["sinkhorn_iterations"] if residual_streams > 1 else 0,
                     routed_experts=spec.experts, shared_experts=1, experts_per_token=spec.topk,
                     expert_intermediate_width=spec.inter, shared_intermediate_width=spec.shared_inter, hash_table_rows=hash_rows,
                     hash_table_columns=spec.topk if hash_rows else 0, rms_epsilon=policy["rms_epsilon"],
                     mhc_epsilon=policy["mhc_epsilon"], mhc_post_multiplier=policy["post_multiplier"],
                     routed_scaling_factor=spec.scaling, activation_limit=spec.limit,
                     requires_token_ids=1 if router_class == 0 else 0, normalize_topk_probabilities=spec.normalize)
    job = LayerJob()
    job.layer = C.pointer(plan)

    def view(slot, name, qtype, rows, width):
        if name not in arena.offsets:
            return
        v = job.weights[slot]
        v.qtype, v.kernel_family, v.encoded = qtype, family, arena.host_ptr(name)
        v.encoded_bytes, v.row_width, v.row_count = arena.sizes[name], width, rows
        v.row_bytes = synth.row_bytes(qtype, width)

    E, H, I, Is = spec.experts, spec.hidden, spec.inter, spec.shared_inter
    view(W_FFN_NORM, "ffn_norm", synth.F32, 1, H)
    view(W_MHC_FUNCTION, "mhc_fn", synth.F32, (S + 2) * S, S * H)
    view(W_MHC_BASE, "mhc_base", synth.F32, 1, (S + 2) * S)
    view(W_MHC_SCALE, "mhc_scale", synth.F32, 1, 3)
    if router:
        view(W_ROUTER, "router", synth.F32, E, H)
    view(W_ROUTER_BIAS, "bias", synth.F32, 1, E)
    view(W_ROUTER_TABLE, "hash_table", synth.I32, hash_rows or 1, spec.topk)
    view(W_GATE, "gate", spec.gate_qtype, E * I, H)
    view(W_UP, "up", spec.up_qtype, E * I, H)
    view(W_DOWN, "down", spec.down_qtype, E * H, I)
    view(W_SHARED_GATE, "shared_gate", spec.gate_qtype, Is, H)
    view(W_SHARED_UP, "shared_up", spec.up_qtype, Is, H)
    view(W_SHARED_DOWN, "shared_down", spec.down_qtype, H, Is)
    job._plan = plan
    return job


def expert_view(job, slot, expert, rows_per_expert):
    """The weight view of one expert of a routed pack (what runtime_moe_load_expert of src/runtime/moe.c hands to add_expert)."""
    pack = job.weights[slot]
    v = WeightView()
    C.memmove(C.byref(v), C.byref(pack), C.sizeof(WeightView))
    offset = expert * rows_per_expert * pack.row_bytes
    v.expert_index, v.row_count = expert, rows_per_expert
    v.encoded_bytes = v.storage_bytes = rows_per_expert * pack.row_bytes
    v.encoded = pack.encoded + offset
    if pack.device_address:
        v.device_address = pack.device_address + offset
    return v


def moe_ops(backend):
    p = _lib.yvex_backend_moe_operations_get(backend.h)
    return p.contents if p else None
