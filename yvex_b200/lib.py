"""ctypes loader and torch-tensor front-end for libyvex_b200.so (device layer C-ABI,
include/yvex_b200_kernels.h). PyTorch is used only for device memory and streams."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libyvex_b200.so")

u64, u32, vp = C.c_uint64, C.c_uint32, C.c_void_p

STATUS_NAMES = {0: "ok", -1: "error", -2: "nomem", -4: "format", -5: "unsupported", -6: "backend",
                -7: "bounds", -8: "state", -9: "cancelled", -10: "invalid-arg", -11: "timeout"}


class YvexError(RuntimeError):
    def __init__(self, code, where):
        super().__init__(f"{where}: {STATUS_NAMES.get(code, code)} ({code})")
        self.code = code


class MoeGeometry(C.Structure):
    _fields_ = [("hidden", u64), ("experts", u64), ("topk", u64), ("inter", u64), ("shared_inter", u64),
                ("scaling", C.c_double), ("limit", C.c_double), ("normalize", C.c_int),
                ("router_class", C.c_int), ("gate_qtype", C.c_uint), ("up_qtype", C.c_uint),
                ("down_qtype", C.c_uint), ("hash_rows", u64), ("hash_stored_rows", u64)]


class MoeWeights(C.Structure):
    _fields_ = [("router", vp), ("bias", vp), ("hash_table", vp), ("gate", vp), ("up", vp), ("down", vp),
                ("shared_gate", vp), ("shared_up", vp), ("shared_down", vp)]


class WorklistObservation(C.Structure):
    _fields_ = [("schema_version", C.c_uint), ("worklist_count", C.c_ulonglong), ("pair_count", C.c_ulonglong),
                ("bucket_count", C.c_ulonglong), ("maximum_bucket_population", C.c_ulonglong),
                ("tensor_core_eligible_pairs", C.c_ulonglong), ("tensor_core_executed_pairs", C.c_ulonglong),
                ("narrow_pairs", C.c_ulonglong), ("tail_rows", C.c_ulonglong), ("width_histogram", C.c_ulonglong * 17),
                ("population_histogram", C.c_ulonglong * 17), ("provenance_counts", C.c_ulonglong * 5)]


class Mhc(C.Structure):
    _fields_ = [("hidden", u64), ("streams", u64), ("sinkhorn_iterations", u64), ("rms_epsilon", C.c_double),
                ("mhc_epsilon", C.c_double), ("post_multiplier", C.c_double), ("mhc_fn", vp), ("scale", vp),
                ("base", vp), ("norm", vp)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m yvex_b200.build` (there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    lib.yvex_b200_version.restype = C.c_char_p
    lib.yvex_b200_moe_workspace_bytes.restype = u64
    lib.yvex_b200_moe_workspace_bytes.argtypes = [C.POINTER(MoeGeometry), u64]
    lib.yvex_b200_moe_wide_workspace_bytes.restype = u64
    lib.yvex_b200_moe_wide_workspace_bytes.argtypes = [C.POINTER(MoeGeometry), u64]
    lib.yvex_b200_launch_count.restype = C.c_ulonglong
    lib.yvex_b200_moe_expert_rows_workspace_bytes.restype = u64
    lib.yvex_b200_moe_expert_rows_workspace_bytes.argtypes = [C.POINTER(MoeGeometry), u64]
    lib.yvex_b200_moe_expert_rows.argtypes = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights), vp, vp, vp, u64, vp,
                                              vp, u64, vp, vp]
    lib.yvex_b200_moe_combine.argtypes = [vp, vp, u64, u64, u64, vp, vp, vp]
    lib.yvex_b200_moe_combine_indexed.argtypes = [vp, vp, vp, vp, u64, u64, u64, vp, vp, vp]
    lib.yvex_b200_ep_dispatch_workspace_bytes.restype = u64
    lib.yvex_b200_ep_dispatch_workspace_bytes.argtypes = [u64, u64]
    lib.yvex_b200_ep_dispatch.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, vp, vp, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_ep_payload_pitch.restype = u64
    lib.yvex_b200_ep_payload_pitch.argtypes = [u64]
    lib.yvex_b200_ep_dispatch_payload.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, u64, u64, vp, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_ep_dispatch_plan.argtypes = [vp, u64, u64, u64, u64, u64, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_ep_dispatch_push.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, u64, u64, vp, vp, u64, C.c_int, vp, u64, vp, vp]
    lib.yvex_b200_moe_expert_rows_sorted.argtypes = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights), vp, u64, vp, u64, u64, vp, u64,
                                                     vp, u64, vp, vp]
    lib.yvex_b200_moe_expert_rows_scatter.argtypes = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights), vp, u64, vp, u64, u64, vp, u64,
                                                      vp, vp]
    lib.yvex_b200_moe_expert_rows_payload.argtypes = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights), vp, u64, vp, vp, u64, vp, vp]
    lib.yvex_b200_moe_wide_set_cta_limit.argtypes = [C.c_int]
    lib.yvex_b200_attention_workspace_bytes.restype = u64
    lib.yvex_b200_attention_workspace_bytes.argtypes = [u64] * 5
    lib.yvex_b200_dequant_rows.argtypes = [C.c_uint, vp, u64, u64, u64, vp, vp, vp]
    lib.yvex_b200_gemv.argtypes = [C.c_uint, vp, u64, u64, u64, vp, u64, vp, vp, C.c_int, vp, vp]
    lib.yvex_b200_gemv_batch.argtypes = [C.c_uint, vp, u64, u64, u64, u64, u64, vp, u64, vp, vp, u64, C.c_int, vp, vp]
    moe_args = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights), vp, vp, vp, u64, vp, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_moe_route.argtypes = moe_args
    lib.yvex_b200_moe_decode.argtypes = moe_args
    lib.yvex_b200_moe_wide.argtypes = moe_args
    lib.yvex_b200_attention_gqa_decode.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, u64, C.c_float,
                                                   vp, vp, u64, vp, vp]
    lib.yvex_b200_attention_f32.argtypes = [vp, vp, vp, u64, u64, u64, C.c_float, C.c_int, vp, vp, vp, vp, vp]
    lib.yvex_b200_attention_sink.argtypes = [vp, vp, vp, u64, u64, u64, C.c_double, C.c_int, vp, vp, vp]
    lib.yvex_b200_mhc_workspace_bytes.restype = u64
    lib.yvex_b200_mhc_workspace_bytes.argtypes = [u64, u64]
    lib.yvex_b200_mhc_prepare.argtypes = [vp, vp, u64, vp, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_mhc_post.argtypes = [vp, vp, vp, vp, vp, u64, vp, vp, vp]
    lib.yvex_b200_expert_worklist_workspace_bytes.restype = u64
    lib.yvex_b200_expert_worklist_workspace_bytes.argtypes = [u64, u64]
    lib.yvex_b200_expert_worklist.argtypes = [vp, u64, u64, u64, u64, u64, C.c_uint, vp, vp, vp, vp, vp, vp, vp, vp, u64, vp, vp]
    lib.yvex_b200_selftest_bounded_wait.argtypes = [u64, vp, vp, vp]
    lib.yvex_b200_moe_wide_uses_gemm.argtypes = [C.POINTER(MoeGeometry), C.POINTER(MoeWeights)]
    lib.yvex_b200_moe_wide_tile_columns.restype = u64
    lib.yvex_b200_moe_wide_tile_columns.argtypes = [C.c_uint]
    lib.yvex_b200_attention_static_scratch_bytes.restype = u64
    lib.yvex_b200_attention_static_scratch_bytes.argtypes = []
    lib.yvex_b200_attention_gqa_decode_static.argtypes = [vp, vp, vp, u64, u64, u64, u64, u64, u64, C.c_float,
                                                          vp, vp, vp]
    return lib


lib = _load()

EXPORTS = ["yvex_b200_version", "yvex_b200_qtype_supported", "yvex_b200_qtype_geometry",
           "yvex_b200_dequant_rows", "yvex_b200_gemv", "yvex_b200_gemv_batch", "yvex_b200_moe_workspace_bytes",
           "yvex_b200_moe_route", "yvex_b200_moe_decode", "yvex_b200_moe_wide",
           "yvex_b200_moe_wide_workspace_bytes", "yvex_b200_launch_count", "yvex_b200_phase_events",
           "yvex_b200_moe_expert_rows_workspace_bytes", "yvex_b200_moe_expert_rows", "yvex_b200_moe_combine",
           "yvex_b200_moe_combine_indexed", "yvex_b200_ep_dispatch_workspace_bytes", "yvex_b200_ep_dispatch",
           "yvex_b200_attention_workspace_bytes", "yvex_b200_attention_gqa_decode",
           "yvex_b200_attention_f32", "yvex_b200_attention_sink", "yvex_b200_attention_static_scratch_bytes",
           "yvex_b200_attention_gqa_decode_static", "yvex_b200_mhc_workspace_bytes", "yvex_b200_mhc_prepare",
           "yvex_b200_mhc_post", "yvex_b200_expert_worklist_workspace_bytes", "yvex_b200_expert_worklist",
           "yvex_b200_selftest_bounded_wait", "yvex_b200_moe_wide_uses_gemm", "yvex_b200_moe_wide_tile_columns",
           "yvex_b200_ep_payload_pitch", "yvex_b200_ep_dispatch_payload", "yvex_b200_moe_expert_rows_payload",
           "yvex_b200_moe_wide_set_cta_limit", "yvex_b200_moe_decode_parts", "yvex_b200_moe_wide_parts",
           "yvex_b200_dequant_gather", "yvex_b200_q8k_round_trip", "yvex_b200_concat_bf16",
           "yvex_b200_moe_expert_rows_scatter", "yvex_b200_ep_dispatch_plan", "yvex_b200_ep_dispatch_push",
           "yvex_b200_moe_expert_rows_sorted"]


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("yvex_b200 compute entry points need a CUDA device; there is no CPU fallback")
    return torch


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _check(rc, where):
    if rc != 0:
        raise YvexError(rc, where)


class Status:
    """Device status word (0 ok / 1 numerics / 2 arguments / 3 timeout) with a host read-out."""

    def __init__(self, device="cuda"):
        torch = _torch()
        self.word = torch.zeros(1, dtype=torch.int32, device=device)

    def read(self):
        return int(self.word.item())

    def reset(self):
        self.word.zero_()


def geometry_of(spec, router_class=1, hash_rows=0, hash_stored_rows=0):
    g = MoeGeometry()
    g.hidden, g.experts, g.topk, g.inter, g.shared_inter = (spec.hidden, spec.experts, spec.topk, spec.inter,
                                                           spec.shared_inter)
    g.scaling, g.limit, g.normalize, g.router_class = spec.scaling, spec.limit, spec.normalize, router_class
    g.gate_qtype, g.up_qtype, g.down_qtype = spec.gate_qtype, spec.up_qtype, spec.down_qtype
    g.hash_rows, g.hash_stored_rows = hash_rows, hash_stored_rows
    return g


def weights_of(tensors):
    """tensors: dict name -> device torch tensor (router/bias/hash_table optional)."""
    w = MoeWeights()
    for name, _ in MoeWeights._fields_:
        setattr(w, name, _p(tensors.get(name)))
    w._keep = tensors
    return w


def dequant_rows(qtype, enc, rows, width, status):
    torch = _torch()
    out = torch.empty((rows, width), dtype=torch.float32, device=enc.device)
    row_bytes = enc.numel() // rows
    _check(lib.yvex_b200_dequant_rows(qtype, _p(enc), rows, width, row_bytes, _p(out), _p(status.word), _stream()),
           "dequant_rows")
    return out


def gemv(qtype, enc, rows, width, x, status, additive=None, round_bf16=False, out=None, row_bytes=None):
    torch = _torch()
    x2 = x.reshape(-1, width)
    if out is None:
        out = torch.empty((x2.shape[0], rows), dtype=torch.float32, device=x.device)
    rb = row_bytes if row_bytes is not None else enc.numel() // rows
    _check(lib.yvex_b200_gemv(qtype, _p(enc), rows, width, rb, _p(x2), x2.shape[0], _p(additive), _p(out),
                              int(round_bf16), _p(status.word), _stream()), "gemv")
    return out


def gemv_batch(qtype, enc, count, rows, width, xs, status, additive=None, round_bf16=False, out=None, row_bytes=None,
               matrix_stride=None):
    """`count` matrices of one shape stored back to back in `enc` (matrix_stride bytes apart), one input row each
    (xs [count, width] f32) -> out [count, rows] f32, one launch."""
    torch = _torch()
    rb = row_bytes if row_bytes is not None else enc.numel() // (rows * count)
    stride = matrix_stride if matrix_stride is not None else rows * rb
    if out is None:
        out = torch.empty((count, rows), dtype=torch.float32, device=xs.device)
    _check(lib.yvex_b200_gemv_batch(qtype, _p(enc), stride, count, rows, width, rb, _p(xs), width, _p(additive), _p(out), rows,
                                    int(round_bf16), _p(status.word), _stream()), "gemv_batch")
    return out


def moe_workspace_bytes(geom, rows, wide=False):
    fn = lib.yvex_b200_moe_wide_workspace_bytes if wide else lib.yvex_b200_moe_workspace_bytes
    return int(fn(C.byref(geom), rows))


def _moe_call(fn, name, geom, weights, x, logits, token_ids, rows, out, selected, wts, workspace, status):
    _check(fn(C.byref(geom), C.byref(weights), _p(x), _p(logits), _p(token_ids), rows, _p(out), _p(selected),
              _p(wts), _p(workspace), workspace.numel() if workspace is not None else 0, _p(status.word),
              _stream()), name)


def moe_layer(geom, weights, x, status, logits=None, token_ids=None, wide=False, workspace=None,
              out=None, selected=None, wts=None):
    """One MoE FFN layer on device rows x [rows, hidden] f32 -> out [rows, hidden] f32."""
    torch = _torch()
    rows = x.shape[0]
    if workspace is None:
        workspace = torch.empty(moe_workspace_bytes(geom, rows, wide), dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty_like(x)
    if selected is None:
        selected = torch.empty((rows, geom.topk), dtype=torch.int32, device=x.device)
    if wts is None:
        wts = torch.empty((rows, geom.topk), dtype=torch.float32, device=x.device)
    fn = lib.yvex_b200_moe_wide if wide else lib.yvex_b200_moe_decode
    _moe_call(fn, "moe_wide" if wide else "moe_decode", geom, weights, x, logits, token_ids, rows, out,
              selected, wts, workspace, status)
    return out, selected, wts


def moe_expert_rows(geom, weights, rows_f16, expert_ids, route_weights, status, workspace=None, out=None):
    """Pair list on this device's expert shard: rows_f16 [P, hidden] fp16, expert_ids [P] int32
    (negative = shared expert), route_weights [P] f32 -> bf16 rows [P, hidden]."""
    torch = _torch()
    pairs = rows_f16.shape[0]
    if out is None:
        out = torch.empty((pairs, geom.hidden), dtype=torch.bfloat16, device=rows_f16.device)
    if pairs == 0:
        return out
    if workspace is None:
        workspace = torch.empty(int(lib.yvex_b200_moe_expert_rows_workspace_bytes(C.byref(geom), pairs)),
                                dtype=torch.uint8, device=rows_f16.device)
    _check(lib.yvex_b200_moe_expert_rows(C.byref(geom), C.byref(weights), _p(rows_f16), _p(expert_ids),
                                         _p(route_weights), pairs, _p(out), _p(workspace), workspace.numel(),
                                         _p(status.word), _stream()), "moe_expert_rows")
    return out


def moe_combine(y_routed, y_shared, topk, status, out=None, routed_rows=None, shared_rows=None):
    """y_routed [T*topk, hidden] bf16 in (token, rank) order, y_shared [T, hidden] bf16 -> f32 [T, hidden].
    With routed_rows [T*topk] / shared_rows [T] (int32) the rows are taken from those positions instead."""
    torch = _torch()
    hidden = y_shared.shape[1]
    tokens = y_shared.shape[0] if shared_rows is None else shared_rows.shape[0]
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=y_shared.device)
    _check(lib.yvex_b200_moe_combine_indexed(_p(y_routed), _p(routed_rows), _p(y_shared), _p(shared_rows), tokens, topk,
                                             hidden, _p(out), _p(status.word), _stream()), "moe_combine")
    return out


def ep_dispatch(rows_f16, selected, route_weights, experts_per_rank, world, status):
    """Sending side of the expert-parallel dispatch: rows_f16 [T, hidden] fp16, selected / route_weights [T, k]
    -> (send_rows [T*k, hidden] fp16 grouped by destination rank, meta [T*k, 2] int32, inverse [T*k] int32,
    send_counts [world] int64)."""
    torch = _torch()
    tokens, hidden = rows_f16.shape
    topk = selected.shape[1]
    pairs, dev = tokens * topk, rows_f16.device
    send_rows = torch.empty((pairs, hidden), dtype=rows_f16.dtype, device=dev)
    meta = torch.empty((pairs, 2), dtype=torch.int32, device=dev)
    inverse = torch.empty(pairs, dtype=torch.int32, device=dev)
    counts = torch.empty(world, dtype=torch.int64, device=dev)
    ws = torch.empty(int(lib.yvex_b200_ep_dispatch_workspace_bytes(pairs, world)), dtype=torch.uint8, device=dev)
    _check(lib.yvex_b200_ep_dispatch(_p(selected), _p(route_weights), _p(rows_f16), tokens, topk, hidden, experts_per_rank,
                                     world, _p(send_rows), _p(meta), _p(inverse), _p(counts), _p(ws), ws.numel(),
                                     _p(status.word), _stream()), "ep_dispatch")
    return send_rows, meta, inverse, counts


def expert_worklist(selected, experts, status, tensor_core_minimum=0, admitted_width=1, provenance=3):
    """selected [rows, topk] int32 -> dict of the device-built worklist (order, source_rows, destination_rows,
    expert_ids, bucket_offsets, bucket_populations as CPU numpy arrays) and its observation struct."""
    torch = _torch()
    rows, topk = selected.shape
    pairs, dev = rows * topk, selected.device
    i32 = lambda n: torch.full((n,), -1, dtype=torch.int32, device=dev)
    order, src, dst = i32(pairs), i32(pairs), i32(pairs)
    ids, offs, pops = i32(experts), i32(experts + 1), i32(experts)
    obs = torch.zeros(C.sizeof(WorklistObservation), dtype=torch.uint8, device=dev)
    ws = torch.empty(int(lib.yvex_b200_expert_worklist_workspace_bytes(pairs, experts)), dtype=torch.uint8, device=dev)
    _check(lib.yvex_b200_expert_worklist(_p(selected.contiguous()), rows, topk, experts, tensor_core_minimum, admitted_width,
                                         provenance, _p(order), _p(src), _p(dst), _p(ids), _p(offs), _p(pops), _p(obs), _p(ws),
                                         ws.numel(), _p(status.word), _stream()), "expert_worklist")
    o = WorklistObservation.from_buffer_copy(obs.cpu().numpy().tobytes())
    n = int(o.bucket_count)
    return dict(order=order.cpu().numpy(), source_rows=src.cpu().numpy(), destination_rows=dst.cpu().numpy(),
                expert_ids=ids.cpu().numpy()[:n], bucket_offsets=offs.cpu().numpy()[:n + 1],
                bucket_populations=pops.cpu().numpy()[:n], observation=o)


def ep_dispatch_payload(rows_f16, selected, route_weights, experts_per_rank, world, segments, status, payload=None, inverse=None,
                        counts=None, workspace=None, rank=0):
    """Segmented sending side: rows_f16 [T, hidden] fp16, selected / route_weights [T, k] -> (payload [T*k, 2*hidden + 16] uint8
    in send order (segment, destination rank), inverse [T*k] int32, counts [segments * world] int64)."""
    torch = _torch()
    tokens, hidden = rows_f16.shape
    pairs, dev, bins = tokens * selected.shape[1], rows_f16.device, world * segments
    pitch = int(lib.yvex_b200_ep_payload_pitch(hidden))
    if payload is None:
        payload = torch.empty((pairs, pitch), dtype=torch.uint8, device=dev)
    if inverse is None:
        inverse = torch.empty(pairs, dtype=torch.int32, device=dev)
    if counts is None:
        counts = torch.empty(bins, dtype=torch.int64, device=dev)
    if workspace is None:
        workspace = torch.empty(int(lib.yvex_b200_ep_dispatch_workspace_bytes(pairs, bins)), dtype=torch.uint8, device=dev)
    _check(lib.yvex_b200_ep_dispatch_payload(_p(selected), _p(route_weights), _p(rows_f16), tokens, selected.shape[1], hidden,
                                             experts_per_rank, world, rank, segments, _p(payload), _p(inverse), _p(counts), _p(workspace),
                                             workspace.numel(), _p(status.word), _stream()), "ep_dispatch_payload")
    return payload, inverse, counts


def ep_dispatch_plan(selected, experts_per_rank, world, segments, status, inverse, counts, workspace):
    """Groups the pairs by (segment, destination rank): inverse [T*k] int32, counts [segments * world] int64; the plan stays in
    `workspace` for ep_dispatch_push."""
    tokens, topk = selected.shape
    _check(lib.yvex_b200_ep_dispatch_plan(_p(selected), tokens, topk, experts_per_rank, world, segments, _p(inverse), _p(counts),
                                          _p(workspace), workspace.numel(), _p(status.word), _stream()), "ep_dispatch_plan")
    return inverse, counts


def ep_dispatch_push(rows_f16, selected, route_weights, experts_per_rank, world, rank, segments, counts_all, recv_bases,
                     capacity_rows, status, workspace, expert_major=False):
    """Writes every payload row straight into its destination rank's receive buffer (recv_bases: int64 device tensor, one
    byte address per bin; counts_all: int64 device tensor [world, segments * world]). expert_major (segments ==
    experts_per_rank, one buffer per destination): the rows land sorted by local expert."""
    tokens, hidden = rows_f16.shape
    _check(lib.yvex_b200_ep_dispatch_push(_p(selected), _p(route_weights), _p(rows_f16), tokens, selected.shape[1], hidden,
                                          experts_per_rank, world, rank, segments, _p(counts_all), _p(recv_bases), capacity_rows,
                                          1 if expert_major else 0, _p(workspace), workspace.numel(), _p(status.word), _stream()),
           "ep_dispatch_push")


def moe_expert_rows_sorted(geom, weights, payload, counts_all, world, rank, home_bases, home_pairs, status, workspace):
    """Grouped GEMMs on records that an expert-major push left sorted by local expert; results stored at their home ranks."""
    pairs = payload.shape[0]
    if pairs == 0:
        return
    _check(lib.yvex_b200_moe_expert_rows_sorted(C.byref(geom), C.byref(weights), _p(payload), pairs, _p(counts_all), world, rank,
                                                _p(home_bases), home_pairs, _p(workspace), workspace.numel(), _p(status.word),
                                                _stream()), "moe_expert_rows_sorted")


def moe_expert_rows_scatter(geom, weights, payload, home_bases, home_pairs, status, workspace=None):
    """The same GEMMs with every pair's bf16 row stored straight into its home rank's buffer (home_bases: int64 device
    tensor of one byte address per rank; peers' buffers mapped into this process). Returns nothing: the rows are elsewhere."""
    torch = _torch()
    pairs = payload.shape[0]
    if pairs == 0:
        return
    if workspace is None:
        workspace = torch.empty(int(lib.yvex_b200_moe_expert_rows_workspace_bytes(C.byref(geom), pairs)),
                                dtype=torch.uint8, device=payload.device)
    _check(lib.yvex_b200_moe_expert_rows_scatter(C.byref(geom), C.byref(weights), _p(payload), pairs, _p(home_bases), home_bases.numel(),
                                                 home_pairs, _p(workspace), workspace.numel(), _p(status.word), _stream()),
           "moe_expert_rows_scatter")


def moe_expert_rows_payload(geom, weights, payload, status, workspace=None, out=None):
    """Received records (hidden fp16 values + trailer per row) on this device's expert shard -> bf16 rows [P, hidden]."""
    torch = _torch()
    pairs = payload.shape[0]
    if out is None:
        out = torch.empty((pairs, geom.hidden), dtype=torch.bfloat16, device=payload.device)
    if pairs == 0:
        return out
    if workspace is None:
        workspace = torch.empty(int(lib.yvex_b200_moe_expert_rows_workspace_bytes(C.byref(geom), pairs)),
                                dtype=torch.uint8, device=payload.device)
    _check(lib.yvex_b200_moe_expert_rows_payload(C.byref(geom), C.byref(weights), _p(payload), pairs, _p(out), _p(workspace),
                                                 workspace.numel(), _p(status.word), _stream()), "moe_expert_rows_payload")
    return out


def moe_route(geom, weights, status, rows_f32=None, logits=None, token_ids=None):
    torch = _torch()
    ref = rows_f32 if rows_f32 is not None else logits
    rows = ref.shape[0]
    selected = torch.empty((rows, geom.topk), dtype=torch.int32, device=ref.device)
    wts = torch.empty((rows, geom.topk), dtype=torch.float32, device=ref.device)
    lg = torch.empty((rows, geom.experts), dtype=torch.float32, device=ref.device)
    _check(lib.yvex_b200_moe_route(C.byref(geom), C.byref(weights), _p(rows_f32), _p(logits), _p(token_ids), rows,
                                   _p(selected), _p(wts), _p(lg), None, 0, _p(status.word), _stream()), "moe_route")
    return selected, wts, lg


def mhc_of(hidden, streams, mhc_fn, scale, base, norm, sinkhorn_iterations=20, rms_epsilon=1e-6, mhc_epsilon=1e-6,
           post_multiplier=2.0):
    """Envelope description over device F32 tensors (kept alive by the returned struct)."""
    m = Mhc(hidden, streams, sinkhorn_iterations, rms_epsilon, mhc_epsilon, post_multiplier, _p(mhc_fn), _p(scale),
            _p(base), _p(norm))
    m._keep = (mhc_fn, scale, base, norm)
    return m


def mhc_prepare(m, expanded, status):
    """expanded [rows, streams*hidden] f32 -> (normalized [rows, hidden], post [rows, streams], combination [rows, S*S])."""
    torch = _torch()
    rows, S, H = expanded.shape[0], m.streams, m.hidden
    normalized = torch.empty((rows, H), dtype=torch.float32, device=expanded.device)
    post = torch.empty((rows, S), dtype=torch.float32, device=expanded.device)
    comb = torch.empty((rows, S * S), dtype=torch.float32, device=expanded.device)
    ws = torch.empty(int(lib.yvex_b200_mhc_workspace_bytes(S, rows)), dtype=torch.uint8, device=expanded.device)
    _check(lib.yvex_b200_mhc_prepare(C.byref(m), _p(expanded), rows, _p(normalized), _p(post), _p(comb), _p(ws), ws.numel(),
                                     _p(status.word), _stream()), "mhc_prepare")
    return normalized, post, comb


def mhc_post(m, core, expanded, post, comb, status):
    torch = _torch()
    out = torch.empty_like(expanded)
    _check(lib.yvex_b200_mhc_post(C.byref(m), _p(core), _p(expanded), _p(post), _p(comb), expanded.shape[0], _p(out),
                                  _p(status.word), _stream()), "mhc_post")
    return out


def attention_gqa_decode(q, k, v, position, scale, status, workspace=None, out=None):
    """q [S,Hq,D] bf16, k/v [S,Hkv,ctx,D] bf16 -> out [S,Hq,D] f32."""
    torch = _torch()
    S, Hq, D = q.shape
    _, Hkv, ctx, _ = k.shape
    if workspace is None:
        workspace = torch.empty(int(lib.yvex_b200_attention_workspace_bytes(S, Hq, Hkv, D, ctx)),
                                dtype=torch.uint8, device=q.device)
    if out is None:
        out = torch.empty((S, Hq, D), dtype=torch.float32, device=q.device)
    _check(lib.yvex_b200_attention_gqa_decode(_p(q), _p(k), _p(v), S, Hq, Hkv, D, ctx, position, scale, _p(out),
                                              _p(workspace), workspace.numel(), _p(status.word), _stream()),
           "attention_gqa_decode")
    return out


def attention_sink(query, rows, sinks, scale, status, round_bf16=True):
    """query [heads, D], rows [n, D], sinks [heads] f32 device tensors -> out [heads, D]."""
    torch = _torch()
    heads, D = query.shape
    out = torch.zeros((heads, D), dtype=torch.float32, device=query.device)
    _check(lib.yvex_b200_attention_sink(_p(query), _p(rows), _p(sinks), heads, rows.shape[0], D, C.c_double(scale), int(round_bf16),
                                        _p(out), _p(status.word), _stream()), "attention_sink")
    return out


def attention_f32(q, keys, values, position, scale, causal, status):
    torch = _torch()
    seq, D = keys.shape
    scores = torch.zeros(seq, dtype=torch.float32, device=q.device)
    probs = torch.zeros(seq, dtype=torch.float32, device=q.device)
    out = torch.zeros(D, dtype=torch.float32, device=q.device)
    _check(lib.yvex_b200_attention_f32(_p(q), _p(keys), _p(values), seq, D, position, scale, int(causal),
                                       _p(scores), _p(probs), _p(out), _p(status.word), _stream()), "attention_f32")
    return out, scores, probs
