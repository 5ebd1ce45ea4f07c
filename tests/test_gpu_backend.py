"""The C11 host boundary on a B200: the calls the reference runtime makes on its backend for this
path (resident weights named by host pointers, workspace attach, execute_rows / complete_rows,
encoded matvec, op_attention), their outputs against the CPU oracle, and their refusals
(src/backend/cuda/moe.c:1826-1923, src/backend/cuda/qtype.c:220-405, src/backend/core.c:990-1036)."""
import ctypes as C

import numpy as np
import pytest

from golden_cases import CASES, ENVELOPE_POLICY, attention_inputs, envelope_inputs, layer_inputs, moe_input_image
from yvex_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def B():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from yvex_b200 import backend
    return backend


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def layer_setup(B, name, down=synth.Q2_K, **job_kw):
    spec, weights, router, x, logits = layer_inputs(name, down_qtype=down)
    be = B.Backend()
    assert be.rc == B.OK, be.message()
    arrays = dict(weights)
    if router is not None:
        arrays["router"] = router
    arena = B.ResidentArena(be, arrays)
    job = B.moe_job(arena, spec, router=router is not None, **job_kw)
    return be, arena, job, spec, x, logits


def attach_workspace(B, be, job, rows, wide=False, shrink=0):
    ops = B.moe_ops(be)
    need = B.ull()
    fn = ops.workspace_required_wide if wide else ops.workspace_required
    assert fn(job.layer, rows, C.byref(need), C.byref(be.err)) == B.OK
    rc, ws, _ = be.tensor(need.value - shrink)
    assert rc == B.OK
    assert B._lib.yvex_backend_workspace_attach(be.h, ws, C.byref(be.err)) == B.OK
    return ops, ws


def run_rows(B, be, ops, job, x, logits, wide=False, selection=True):
    rows, H = x.shape
    k = job._plan.experts_per_token
    out = np.zeros((rows, H), np.float32)
    sel = np.zeros((rows, k), np.uint64)
    wts = np.zeros((rows, k), np.float32)
    batch = B.row_batch(rows, H, host_rows=x.ctypes.data_as(B.vp),
                        router_logits=None if logits is None else logits.ctypes.data_as(B.vp))
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, sel.ctypes.data_as(B.vp) if selection else None,
                     wts.ctypes.data_as(B.vp) if selection else None, sel.size)
    res = B.RowBatchResult()
    fn = ops.execute_rows_wide if wide else ops.execute_rows
    rc = fn(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err))
    return rc, out, sel, wts, res


@pytest.mark.parametrize("name", ["small_router", "small_logits", "c2_shape"])
def test_execute_rows_host_buffers_vs_frozen_reference(B, golden, name):
    be, arena, job, spec, x, logits = layer_setup(B, name)
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    rc, out, sel, wts, res = run_rows(B, be, ops, job, x, logits)
    assert rc == B.OK, be.message()
    assert (sel == golden[f"layer_{name}_sel"]).all()
    assert np.abs(wts - golden[f"layer_{name}_w"].view(np.float32)).max() <= 2e-7
    assert rel_l2(out, golden[f"layer_{name}_out"].view(np.float32)) <= 1e-3
    assert res.completed == 1 and res.row_count == x.shape[0] and res.row_expert_pairs == x.shape[0] * spec.topk
    assert res.kernel_launches >= 3 and res.h2d_bytes >= x.nbytes and res.d2h_bytes >= out.nbytes
    assert res.active_weight_per_unique_expert_bytes == spec.weight_bytes_per_expert()
    assert be.close() == B.OK


def test_execute_rows_device_tensors_and_deferred_completion(B, golden):
    be, arena, job, spec, x, logits = layer_setup(B, "small_router")
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    rows, H = x.shape
    tin = be.from_array(x, B.F32)
    rc, tout, _ = be.tensor(x.nbytes, B.F32, [rows, H])
    slot = B.CompletionSlot()
    comp = B.Completion(1, C.pointer(slot))
    job.device_completion = C.pointer(comp)
    batch = B.row_batch(rows, H, device_rows=tin, device_outputs=tout)
    res = B.RowBatchResult()
    rc = ops.execute_rows(be.h, C.byref(job), C.byref(batch), None, C.byref(res), C.byref(be.err))
    assert rc == B.OK and res.device_completion_pending == 1 and res.completed == 0
    # a second layer may not start on this backend until the first is completed
    assert ops.execute_rows(be.h, C.byref(job), C.byref(batch), None, C.byref(B.RowBatchResult()), C.byref(be.err)) == B.STATE
    assert ops.complete_rows(be.h, 0, C.byref(res), C.byref(be.err)) == B.OK
    assert res.completed == 1 and slot.pending == 0 and slot.status == 0
    assert ops.complete_rows(be.h, 0, C.byref(res), C.byref(be.err)) == B.STATE
    rc, out = be.read(tout, np.float32, rows * H)
    assert rc == B.OK and rel_l2(out.reshape(rows, H), golden["layer_small_router_out"].view(np.float32)) <= 1e-3
    assert be.close() == B.OK


@pytest.mark.parametrize("wide", [False, True])
def test_partial_outputs_routed_shared_post_combination(B, golden, wide):
    """routed_rows / shared_rows (and with the envelope post_rows / combination_rows) are published when the
    caller gives room for them: the f32 rank-ordered routed sum and the shared expert's row, whose bf16-rounded
    sum is the combined row bit for bit (src/runtime/moe.c:606-637, :1501-1508)."""
    be, arena, job, spec, x, logits = layer_setup(B, "small_logits")
    rows, H = x.shape
    ops, _ = attach_workspace(B, be, job, rows, wide=wide)
    out, routed, shared = (np.zeros((rows, H), np.float32) for _ in range(3))
    batch = B.row_batch(rows, H, host_rows=x.ctypes.data_as(B.vp), router_logits=logits.ctypes.data_as(B.vp))
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, routed=routed.ctypes.data_as(B.vp), shared=shared.ctypes.data_as(B.vp),
                     routed_capacity=routed.size, shared_capacity=shared.size)
    res = B.RowBatchResult()
    fn = ops.execute_rows_wide if wide else ops.execute_rows
    assert fn(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.OK, be.message()
    assert rel_l2(out, golden["layer_small_logits_out"].view(np.float32)) <= 1e-3
    assert (synth.bf16_round(routed + shared).view(np.uint32) == out.view(np.uint32)).all()
    assert (synth.bf16_round(shared).view(np.uint32) == shared.view(np.uint32)).all() and np.abs(routed).max() > 0
    assert res.schema_version == 4 and res.execution_class == B.EXECUTION_CLASS_DEVICE_NATIVE and res.memory.complete == 1
    # too small a capacity is refused before anything runs
    o.routed_capacity = routed.size - 1
    assert fn(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.BOUNDS
    # a batch of an unknown schema, and a full-evidence job, are refused like the reference's width-N entry
    o.routed_capacity = routed.size
    batch.base.schema_version = 7
    assert fn(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.INVALID_ARG
    batch.base.schema_version = B.ROW_BATCH_SCHEMA_LOGITS
    job.evidence_level = 3
    assert fn(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.INVALID_ARG
    job.evidence_level = 0
    # a weight view that names its device address directly needs no arena lookup
    addr = B.ull()
    v = job.weights[B.W_DOWN]
    assert B._lib.yvex_backend_resident_resolve(be.h, v.encoded, v.encoded_bytes, C.byref(addr)) == 1
    v.device_address, keep = addr.value, v.encoded
    v.encoded = None
    out2 = np.zeros_like(out)
    o2 = B.row_output(out2.ctypes.data_as(B.vp), out2.size)
    assert fn(be.h, C.byref(job), C.byref(batch), C.byref(o2), C.byref(res), C.byref(be.err)) == B.OK, be.message()
    assert (out2.view(np.uint32) == out.view(np.uint32)).all()
    v.encoded, v.device_address = keep, 0
    assert be.close() == B.OK


def test_envelope_publishes_post_and_combination_rows(B, golden):
    H, S, T, seed = CASES["envelope"]["small"]
    fn_, scale, base, norm, expanded = envelope_inputs("small")
    spec, weights, router, _, _ = layer_inputs("small_router")
    be = B.Backend()
    arena = B.ResidentArena(be, dict(weights, router=router, ffn_norm=norm, mhc_fn=fn_, mhc_base=base, mhc_scale=scale))
    job = B.moe_job(arena, spec, residual_streams=S, envelope_policy=ENVELOPE_POLICY)
    ops, _ = attach_workspace(B, be, job, T)
    out = np.zeros((T, S * H), np.float32)
    post, comb = np.zeros((T, S), np.float32), np.zeros((T, S, S), np.float32)
    batch = B.row_batch(T, S * H, host_rows=expanded.ctypes.data_as(B.vp))
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, post=post.ctypes.data_as(B.vp), combination=comb.ctypes.data_as(B.vp),
                     post_capacity=post.size, combination_capacity=comb.size)
    res = B.RowBatchResult()
    assert ops.execute_rows(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.OK, be.message()
    assert rel_l2(out, golden["envelope_small_out"].view(np.float32)) <= 1e-3
    # post gates are multiplier * sigmoid(.) in (0, multiplier); Sinkhorn leaves every combination matrix doubly stochastic
    assert (post > 0).all() and (post < ENVELOPE_POLICY["post_multiplier"]).all()
    assert np.abs(comb.sum(axis=2) - 1.0).max() < 1e-3 and np.abs(comb.sum(axis=1) - 1.0).max() < 1e-3
    assert be.close() == B.OK


def test_execute_rows_refusals(B):
    be, arena, job, spec, x, logits = layer_setup(B, "small_logits")
    ops = B.moe_ops(be)
    # no workspace attached / too small -> NOMEM
    assert run_rows(B, be, ops, job, x, logits)[0] == B.NOMEM
    ops, ws = attach_workspace(B, be, job, x.shape[0], shrink=4096)
    assert run_rows(B, be, ops, job, x, logits)[0] == B.NOMEM
    be.free(ws)
    ops, ws = attach_workspace(B, be, job, x.shape[0])
    assert run_rows(B, be, ops, job, x, logits)[0] == B.OK
    # 63 rows is outside the narrow contract
    big = np.zeros((63, spec.hidden), np.float32)
    assert run_rows(B, be, ops, job, big, np.zeros((63, spec.experts), np.float32))[0] == B.UNSUPPORTED
    need = B.ull()
    assert ops.workspace_required(job.layer, 63, C.byref(need), C.byref(be.err)) == B.UNSUPPORTED
    # unknown kernel family
    job.weights[B.W_GATE].kernel_family = b"sm121-int8-tensorcore-expert"
    assert run_rows(B, be, ops, job, x, logits)[0] == B.UNSUPPORTED
    job.weights[B.W_GATE].kernel_family = b"sm100-dequant-gemv"
    assert run_rows(B, be, ops, job, x, logits)[0] == B.OK
    # a qtype without a decoder (Q3_K) never reaches the device
    job.weights[B.W_DOWN].qtype = 11
    assert run_rows(B, be, ops, job, x, logits)[0] == B.UNSUPPORTED
    job.weights[B.W_DOWN].qtype = spec.down_qtype
    # a plan that asks for the mHC envelope without its geometry is refused, never run without it
    job._plan.residual_streams = 4
    assert run_rows(B, be, ops, job, x, logits)[0] == B.FORMAT
    job._plan.residual_streams = 1
    # cancellation callback
    job.cancel_requested = B.CANCEL_FN(lambda ctx: 1)
    assert run_rows(B, be, ops, job, x, logits)[0] == B.CANCELLED
    job.cancel_requested = B.CANCEL_FN(0)
    # weights outside the resident arena -> STATE
    stray = np.zeros(job.weights[B.W_UP].encoded_bytes, np.uint8)
    keep = job.weights[B.W_UP].encoded
    job.weights[B.W_UP].encoded = stray.ctypes.data
    assert run_rows(B, be, ops, job, x, logits)[0] == B.STATE
    job.weights[B.W_UP].encoded = keep
    # non-finite input surfaces as a backend error and publishes nothing
    bad = x.copy()
    bad[0, 0] = np.nan
    rc, out, _, _, res = run_rows(B, be, ops, job, bad, logits)
    assert rc == B.BACKEND and res.completed == 0
    assert run_rows(B, be, ops, job, x, logits)[0] == B.OK            # the status word was cleared
    # derived layouts are not offered
    assert ops.derived_layout_plan(None, C.byref(need), C.byref(be.err)) == B.UNSUPPORTED
    assert be.close() == B.OK


def test_execute_rows_with_mhc_envelope_vs_frozen_reference(B, golden):
    """Expanded rows in, expanded rows out (4 residual streams around the small_router layer)."""
    H, S, T, seed = CASES["envelope"]["small"]
    fn, scale, base, norm, expanded = envelope_inputs("small")
    spec, weights, router, _, _ = layer_inputs("small_router")
    be = B.Backend()
    arrays = dict(weights, router=router, ffn_norm=norm, mhc_fn=fn, mhc_base=base, mhc_scale=scale)
    arena = B.ResidentArena(be, arrays)
    job = B.moe_job(arena, spec, residual_streams=S, envelope_policy=ENVELOPE_POLICY)
    ops, _ = attach_workspace(B, be, job, T)
    rc, out, sel, wts, res = run_rows(B, be, ops, job, expanded, None)
    assert rc == B.OK, be.message()
    assert (sel == golden["envelope_small_sel"]).all()
    assert out.shape == (T, S * H) and rel_l2(out, golden["envelope_small_out"].view(np.float32)) <= 1e-3
    assert res.completed == 1 and res.kernel_launches >= 6
    # supplied logits bypass the router the envelope feeds: refused
    lg = np.zeros((T, spec.experts), np.float32)
    assert run_rows(B, be, ops, job, expanded, lg)[0] == B.UNSUPPORTED
    # coefficients must be F32 and resident
    job.weights[B.W_MHC_BASE].qtype = synth.BF16
    assert run_rows(B, be, ops, job, expanded, None)[0] == B.UNSUPPORTED
    job.weights[B.W_MHC_BASE].qtype = synth.F32
    keep = job.weights[B.W_FFN_NORM].encoded
    job.weights[B.W_FFN_NORM].encoded = None
    assert run_rows(B, be, ops, job, expanded, None)[0] == B.STATE
    job.weights[B.W_FFN_NORM].encoded = keep
    # rows of the hidden width are no longer this layer's row shape
    assert run_rows(B, be, ops, job, expanded[:, :H].copy(), None)[0] == B.FORMAT
    assert run_rows(B, be, ops, job, expanded, None)[0] == B.OK
    assert be.close() == B.OK


def test_execute_rows_envelope_with_bf16_coefficients_vs_oracle(B, port):
    """BF16 coefficient tensors (the other flat format the reference decodes, src/graph/moe.c:416-419)."""
    H, S, T, seed = CASES["envelope"]["small"]
    fn, scale, base, norm, expanded = envelope_inputs("small")
    spec, weights, router, _, _ = layer_inputs("small_router")
    coeff = {"ffn_norm": norm, "mhc_fn": fn, "mhc_base": base, "mhc_scale": scale}
    rounded = {k: synth.bf16_round(v) for k, v in coeff.items()}
    be = B.Backend()
    arena = B.ResidentArena(be, dict(weights, router=router, **{k: synth.bf16_bits(v).reshape(v.shape) for k, v in coeff.items()}))
    job = B.moe_job(arena, spec, residual_streams=S, envelope_policy=ENVELOPE_POLICY)
    for slot in (B.W_FFN_NORM, B.W_MHC_FUNCTION, B.W_MHC_BASE, B.W_MHC_SCALE):
        job.weights[slot].qtype = synth.BF16
    ops, _ = attach_workspace(B, be, job, T)
    rc, out, sel, _, _ = run_rows(B, be, ops, job, expanded, None)
    assert rc == B.OK, be.message()
    M = port.mhc(H, S, rounded["mhc_fn"], rounded["mhc_scale"], rounded["mhc_base"], rounded["ffn_norm"], **ENVELOPE_POLICY)
    prep = [port.mhc_prepare(M, expanded[t]) for t in range(T)]
    normalized = np.stack([p[1] for p in prep])
    rcp, core, sel0, _ = port.moe_tokens(port.layer(spec, weights, router=router), normalized, threads=4)
    want = np.stack([port.mhc_post(M, core[t], expanded[t], prep[t][2], prep[t][3])[1] for t in range(T)])
    assert rcp == 0 and (sel == sel0).all() and rel_l2(out, want) <= 1e-3
    assert be.close() == B.OK


def test_execute_rows_wide_vs_oracle(B, port):
    H, E, k, I, T = 512, 8, 2, 256, 150
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q4_K)
    rng = np.random.default_rng(77)
    x, logits = rng.standard_normal((T, H)).astype(np.float32), rng.standard_normal((T, E)).astype(np.float32)
    weights = synth.moe_weights(spec, 78)
    be = B.Backend()
    arena = B.ResidentArena(be, weights)
    job = B.moe_job(arena, spec, router=False, family=b"sm100-f16-tcgen05-expert")
    ops, _ = attach_workspace(B, be, job, T, wide=True)
    rc, out, sel, wts, res = run_rows(B, be, ops, job, x, logits, wide=True)
    assert rc == B.OK, be.message()
    rcp, want, sel0, _ = port.moe_tokens(port.layer(spec, weights, allow_q4k=True), x, logits=logits, threads=8)
    assert rcp == 0 and (sel == sel0).all() and rel_l2(out, want) <= 1e-3
    assert be.close() == B.OK


def test_encoded_matvec_resident_pointer_contract(B, port):
    rows, width = 300, 4096
    w = synth.random_blocks(synth.IQ2_XXS, rows, width, 5)
    x = np.random.default_rng(6).standard_normal((2, width)).astype(np.float32)
    be = B.Backend()
    arena = B.ResidentArena(be, {"w": w})
    tin = be.from_array(x, B.F32)
    rc, tout, _ = be.tensor(2 * rows * 4, B.F32, [2, rows])
    facts = B.Facts()
    args = (arena.host_ptr("w"), w.size, synth.IQ2_XXS, rows, width, w.shape[1], 2, tin, None, 0, None, tout, 0, C.byref(facts),
            C.byref(be.err))
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *args) == B.OK, be.message()
    rc, y = be.read(tout, np.float32, 2 * rows)
    for i in range(2):
        _, want = port.matvec(synth.IQ2_XXS, w, rows, width, x[i], threads=4)
        assert rel_l2(y.reshape(2, rows)[i], want) <= 1e-5
    assert facts.kernel_launches == 1 and facts.active_weight_bytes == w.size and facts.stream_synchronizations == 1
    # refusals: Q4_0 has no codec anywhere; a pointer outside the arena
    bad = list(args)
    bad[2] = 2
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *bad) == B.UNSUPPORTED
    bad = list(args)
    bad[12] = 2
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *bad) == B.INVALID_ARG
    bad = list(args)
    bad[0] = w.ctypes.data
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *bad) == B.FORMAT
    unwritten = be.tensor(x.nbytes, B.F32, [2, width])[1]
    bad = list(args)
    bad[7] = unwritten
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *bad) == B.FORMAT
    assert be.close() == B.OK


@pytest.mark.parametrize("qtype", [synth.IQ2_XXS, synth.Q2_K, synth.Q8_0, synth.MXFP4, synth.Q4_K])
def test_encoded_matvec_with_q8k_activations(B, port, qtype):
    """activation_q8 = 1: the rows of the four qtypes the reference admits are multiplied by the Q8_K round trip
    of the input (5 x 4096 weights, 3 input rows, as tests/unit/cuda/quant_qtype.c:273-396 runs it), within its
    bound against the CPU codec on those values and its looser bound against the exact product; Q4_K is not
    one of the four and takes the plain path."""
    from oracle.oracle_lib import q8k_round_trip
    rows, width, inputs = 5, 4096, 3
    w = synth.random_blocks(qtype, rows, width, 21)
    idx = np.arange(width)
    x = np.stack([((idx + 5 * i) % 29 - 14).astype(np.float32) / np.float32(13 + i) for i in range(inputs)])
    be = B.Backend()
    arena = B.ResidentArena(be, {"w": w})
    tin = be.from_array(x, B.F32)
    rc, tout, _ = be.tensor(inputs * rows * 4, B.F32, [inputs, rows])
    facts = B.Facts()
    args = (arena.host_ptr("w"), w.size, qtype, rows, width, w.shape[1], inputs, tin, None, 0, None, tout, 1, C.byref(facts),
            C.byref(be.err))
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *args) == B.OK, be.message()
    rc, y = be.read(tout, np.float32, inputs * rows)
    y = y.reshape(inputs, rows)
    eligible = qtype != synth.Q4_K
    xq = q8k_round_trip(x) if eligible else x
    assert eligible == (not np.array_equal(xq, x))
    for i in range(inputs):
        _, want = port.matvec(qtype, w, rows, width, xq[i], threads=2, allow_q4k=True)
        _, exact = port.matvec(qtype, w, rows, width, x[i], threads=2, allow_q4k=True)
        assert (np.abs(y[i] - want) <= 1e-5 * (1 + np.abs(want))).all(), np.abs(y[i] - want).max()
        assert (np.abs(y[i] - exact) <= 0.1 * (1 + np.abs(exact))).all()
    assert facts.kernel_launches == (2 if eligible else 1)
    assert facts.temporary_bytes == 4 + (inputs * width * 4 if eligible else 0)
    assert be.close() == B.OK


def test_encoded_matvec_with_split_input(B, port):
    """input_tail: the row is head ++ tail rounded to bf16 (173 + 3923 values, tests/unit/cuda/quant_qtype.c:275,306-311)."""
    rows, width, head = 5, 4096, 173
    w = synth.random_blocks(synth.IQ2_XXS, rows, width, 22)
    x = np.random.default_rng(23).standard_normal((2, width)).astype(np.float32)
    be = B.Backend()
    arena = B.ResidentArena(be, {"w": w})
    thead, ttail = be.from_array(np.ascontiguousarray(x[:, :head]), B.F32), be.from_array(np.ascontiguousarray(x[:, head:]), B.F32)
    rc, tout, _ = be.tensor(2 * rows * 4, B.F32, [2, rows])
    facts = B.Facts()
    args = [arena.host_ptr("w"), w.size, synth.IQ2_XXS, rows, width, w.shape[1], 2, thead, ttail, head, None, tout, 0, C.byref(facts),
            C.byref(be.err)]
    assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *args) == B.OK, be.message()
    rc, y = be.read(tout, np.float32, 2 * rows)
    for i in range(2):
        _, want = port.matvec(synth.IQ2_XXS, w, rows, width, synth.bf16_round(x[i]), threads=2)
        assert (np.abs(y.reshape(2, rows)[i] - want) <= 1e-5 * (1 + np.abs(want))).all()
    # a head width without a tail (or the reverse), or a head as wide as the row, is refused
    for tail, hw in ((None, head), (ttail, 0), (ttail, width)):
        bad = list(args)
        bad[8], bad[9] = tail, hw
        assert B._lib.yvex_backend_cuda_encoded_matvec(be.h, *bad) == B.FORMAT
    assert be.close() == B.OK


@pytest.mark.parametrize("qtype", [synth.IQ2_XXS, synth.Q8_0, synth.Q2_K])
def test_encoded_gather_decodes_selected_rows_bit_exactly(B, port, qtype):
    rows, width = 40, 512
    w = synth.random_blocks(qtype, rows, width, 31)
    ids = np.array([7, 0, 39, 7, 12], np.uint32)
    be = B.Backend()
    arena = B.ResidentArena(be, {"w": w})
    rc, tout, _ = be.tensor(ids.size * width * 4, B.F32, [ids.size, width])
    facts = B.Facts()
    args = [arena.host_ptr("w"), w.size, qtype, rows, width, w.shape[1], ids.ctypes.data_as(B.vp), ids.size, tout, C.byref(facts),
            C.byref(be.err)]
    assert B._lib.yvex_backend_cuda_encoded_gather(be.h, *args) == B.OK, be.message()
    rc, got = be.read(tout, np.float32, ids.size * width)
    _, full = port.decode_rows(qtype, w, rows, width)
    assert (got.reshape(ids.size, width).view(np.uint32) == full.reshape(rows, width)[ids].view(np.uint32)).all()
    assert facts.kernel_launches == 1 and facts.active_weight_bytes == ids.size * w.shape[1] and facts.h2d_bytes == ids.nbytes
    far = np.array([3, rows], np.uint32)
    bad = list(args)
    bad[6], bad[7] = far.ctypes.data_as(B.vp), far.size
    assert B._lib.yvex_backend_cuda_encoded_gather(be.h, *bad) == B.BOUNDS
    assert be.close() == B.OK


def test_op_attention_and_gqa_decode(B, port, golden):
    be = B.Backend()
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal(s).astype(np.float32) for s in ((64,), (90, 64), (90, 64)))
    tq, tk, tv = be.from_array(q, B.F32), be.from_array(k, B.F32), be.from_array(v, B.F32)
    ts, tp, to = (be.tensor(n * 4, B.F32, [n])[1] for n in (90, 90, 64))
    A = B._lib.yvex_backend_op_attention
    assert A(be.h, tq, tk, tv, 90, 40, 0.125, 1, ts, tp, to, C.byref(be.err)) == B.OK, be.message()
    rc, out = be.read(to, np.float32, 64)
    _, want = port.attention_head(q, k, v, 40, 0.125, 1)
    assert rel_l2(out, want) <= 1e-5
    assert A(be.h, tq, tk, tv, 90, 90, 0.125, 1, ts, tp, to, C.byref(be.err)) == B.BOUNDS       # position-out-of-range
    assert A(be.h, tq, tk, tv, 90, 40, -1.0, 1, ts, tp, to, C.byref(be.err)) == B.INVALID_ARG
    assert A(be.h, tq, tk, tv, 91, 40, 0.125, 1, ts, tp, to, C.byref(be.err)) == B.FORMAT       # dims mismatch
    # GQA decode through the boundary
    import torch
    qf, kf, vf, pos, scale = attention_inputs("small")
    bits = lambda a: synth.bf16_bits(a).reshape(a.shape)
    gq, gk, gv = (be.from_array(bits(a), B.BF16) for a in (qf, kf, vf))
    S, Hq, D = qf.shape
    gout = be.tensor(qf.size * 4, B.F32, list(qf.shape))[1]
    G = B._lib.yvex_backend_attention_gqa_decode
    args = (gq, gk, gv, S, Hq, kf.shape[1], D, kf.shape[2], pos, scale, gout, C.byref(be.err))
    assert G(be.h, *args) == B.NOMEM                                  # no workspace attached yet
    ws = be.tensor(1 << 22)[1]
    assert B._lib.yvex_backend_workspace_attach(be.h, ws, C.byref(be.err)) == B.OK
    assert G(be.h, *args) == B.OK, be.message()
    rc, o = be.read(gout, np.float32, qf.size)
    assert rel_l2(o.reshape(qf.shape), golden["attention_small"].view(np.float32)) <= 1e-4
    # ops outside the path fail closed
    assert B._lib.yvex_backend_op_matmul(be.h, tq, tk, to, C.byref(be.err)) == B.UNSUPPORTED
    assert torch.cuda.is_available() and be.close() == B.OK


def test_backend_lifecycle_and_ownership(B):
    be = B.Backend()
    other = B.Backend()
    rc, t, _ = be.tensor(1024)
    assert other.write(t, np.zeros(16, np.uint8)) == B.INVALID_ARG           # foreign tensor
    assert be.read(t, np.uint8, 16)[0] == B.STATE                            # never written
    assert B._lib.yvex_backend_close_checked(C.byref(be.handle), C.byref(be.err)) == B.STATE   # still owns a tensor
    assert be.handle.value                                                   # owner retained for retry
    assert be.close() == B.OK and other.close() == B.OK
    limited = B.Backend(memory_limit=4096)
    assert limited.tensor(8192)[0] == B.NOMEM and limited.close() == B.OK


def test_execute_rows_result_counters_match_the_reference_contract(B):
    """The counters a caller asserts (src/runtime/moe.c:1457-1475; filled as in src/backend/cuda/moe.c:1757-1786,
    :1905-1915): one grouped operation per pair, one shared operation per row, the populated experts
    and the worklist summary built on the device, active bytes = replicated tensors + the experts in use."""
    be, arena, job, spec, x, logits = layer_setup(B, "small_logits")
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    rc, out, sel, wts, res = run_rows(B, be, ops, job, x, logits)
    assert rc == B.OK, be.message()
    rows, pairs = x.shape[0], x.shape[0] * spec.topk
    counts = np.bincount(sel.reshape(-1).astype(np.int64), minlength=spec.experts)
    unique = int((counts > 0).sum())
    assert res.grouped_expert_operations == pairs and res.shared_expert_operations == rows
    assert res.unique_experts == unique and res.tensor_core_launches == 2
    w = res.worklists
    assert (w.schema_version, w.worklist_count, w.pair_count, w.bucket_count) == (1, 1, pairs, unique)
    assert w.maximum_bucket_population == counts.max() and w.narrow_pairs == pairs and w.tensor_core_eligible_pairs == 0
    hist = np.bincount(np.minimum(counts[counts > 0], 16), minlength=17)
    assert list(w.population_histogram) == hist.tolist()
    assert list(w.width_histogram) == [1 if i == min(rows, 16) else 0 for i in range(17)]
    base = sum(job.weights[s].encoded_bytes for s in (B.W_SHARED_GATE, B.W_SHARED_UP, B.W_SHARED_DOWN, B.W_ROUTER))
    assert res.active_weight_base_bytes == base
    assert res.encoded_bytes_read == base + unique * spec.weight_bytes_per_expert() == res.memory.active_weight_bytes
    assert be.close() == B.OK


def test_execute_rows_wide_copy_pipeline_is_bit_identical(B):
    """Host rows in, host rows out on the wide entry run as row ranges whose copies overlap compute
    (rows are independent). The result must equal the same batch given as device rows, which runs in
    one piece, bit for bit."""
    H, E, k, I, T = 512, 8, 2, 256, 2600                    # 650 pairs per expert: four row ranges
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q2_K)
    rng = np.random.default_rng(91)
    x, logits = rng.standard_normal((T, H)).astype(np.float32), rng.standard_normal((T, E)).astype(np.float32)
    be = B.Backend()
    arena = B.ResidentArena(be, synth.moe_weights(spec, 92))
    job = B.moe_job(arena, spec, router=False)
    ops, _ = attach_workspace(B, be, job, T, wide=True)
    rc, out, sel, wts, res = run_rows(B, be, ops, job, x, logits, wide=True)
    assert rc == B.OK, be.message()
    assert B._lib.yvex_backend_moe_last_pipeline_chunks(be.h) == 4 and res.tensor_core_launches == 8 and res.completed == 1
    tin, tlg = be.from_array(x, B.F32), be.from_array(logits, B.F32)
    tout = be.tensor(x.nbytes, B.F32, [T, H])[1]
    sel2, wts2 = np.zeros((T, k), np.uint64), np.zeros((T, k), np.float32)
    batch = B.row_batch(T, H, device_rows=tin, device_outputs=tout, device_router_logits=tlg)
    o = B.row_output(None, 0, sel2.ctypes.data_as(B.vp), wts2.ctypes.data_as(B.vp), sel2.size)
    res2 = B.RowBatchResult()
    assert ops.execute_rows_wide(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res2), C.byref(be.err)) == B.OK, be.message()
    rc, whole = be.read(tout, np.float32, T * H)
    assert B._lib.yvex_backend_moe_last_pipeline_chunks(be.h) == 0 and res2.tensor_core_launches == 2
    assert (sel == sel2).all() and (wts.view(np.uint32) == wts2.view(np.uint32)).all()
    assert (out.view(np.uint32) == whole.reshape(T, H).view(np.uint32)).all()
    assert res.unique_experts == res2.unique_experts == E
    assert res.worklists.tensor_core_eligible_pairs == T * k and res.worklists.narrow_pairs == 0
    assert be.close() == B.OK


def test_bounded_device_wait_runs_out_and_maps_to_timeout(B):
    """A device wait that nothing satisfies gives up after its limit, the kernel returns status 3, the
    boundary reports YVEX_ERR_TIMEOUT and the backend stays usable (no trap, no hang, nothing demoted)."""
    import time
    be, arena, job, spec, x, logits = layer_setup(B, "small_logits")
    elapsed = B.ull()
    t0 = time.perf_counter()
    rc = B._lib.yvex_backend_selftest_bounded_wait(be.h, 20_000_000, C.byref(elapsed), C.byref(be.err))
    wall = time.perf_counter() - t0
    assert rc == B.TIMEOUT and b"bounded device wait" in be.err.message
    assert 20_000_000 <= elapsed.value < 1_000_000_000 and wall < 5.0, (elapsed.value, wall)
    assert B._lib.yvex_backend_status_of(be.h) == 0                          # still READY
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    assert run_rows(B, be, ops, job, x, logits)[0] == B.OK                   # the status word was cleared
    assert B._lib.yvex_backend_selftest_bounded_wait(be.h, 0, None, C.byref(be.err)) == B.INVALID_ARG
    assert be.close() == B.OK


def test_host_fault_seams_fail_closed(B, monkeypatch):
    """The reference's test seams (src/backend/cuda/qtype.c:625-661, tests/unit/cuda/quant_qtype.c:1749-1811):
    a refused copy fails the call and the backend recovers; a failed launch demotes the backend, which
    then refuses everything with a state error until it is closed. Nothing faults on the device."""
    rows, width = 64, 1024
    w = synth.random_blocks(synth.Q8_0, rows, width, 5)
    x = np.random.default_rng(6).standard_normal((1, width)).astype(np.float32)
    be = B.Backend()
    arena = B.ResidentArena(be, {"w": w})
    tin = be.from_array(x, B.F32)
    tout = be.tensor(rows * 4, B.F32, [1, rows])[1]
    facts = B.Facts()
    args = (arena.host_ptr("w"), w.size, synth.Q8_0, rows, width, w.shape[1], 1, tin, None, 0, None, tout, 0, C.byref(facts),
            C.byref(be.err))
    call = lambda: B._lib.yvex_backend_cuda_encoded_matvec(be.h, *args)
    for where in ("input", "output"):
        monkeypatch.setenv("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", where)
        assert call() == B.BACKEND and tout.contents.is_written == 0
        monkeypatch.delenv("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE")
        assert call() == B.OK and tout.contents.is_written == 1           # recovers after a copy refusal
    monkeypatch.setenv("YVEX_TEST_CUDA_LAUNCH_FAILURE", "encoded-matvec")
    assert call() == B.BACKEND
    monkeypatch.delenv("YVEX_TEST_CUDA_LAUNCH_FAILURE")
    assert B._lib.yvex_backend_status_of(be.h) == 3                          # FAILED, for good
    assert call() == B.STATE and B.moe_ops(be) is None
    assert be.read(tout, np.float32, rows)[0] == B.STATE
    be.close()
    # the MoE table has the same seam
    be, arena, job, spec, x, logits = layer_setup(B, "small_logits")
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    monkeypatch.setenv("YVEX_TEST_CUDA_LAUNCH_FAILURE", "moe-rows")
    rc, _, _, _, res = run_rows(B, be, ops, job, x, logits)
    monkeypatch.delenv("YVEX_TEST_CUDA_LAUNCH_FAILURE")
    assert rc == B.BACKEND and res.completed == 0 and B._lib.yvex_backend_status_of(be.h) == 3
    assert run_rows(B, be, ops, job, x, logits)[0] == B.STATE
    be.close()


def test_two_backends_on_two_devices(B):
    """Kernels that opt in to more than 48 KiB of shared memory do so per device: a second backend on
    another ordinal must run the same layer."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    spec, weights, router, x, logits = layer_inputs("small_logits")
    outs = []
    for dev in (b"cuda:0", b"cuda:1"):
        be = B.Backend(device=dev)
        assert be.rc == B.OK, be.message()
        arena = B.ResidentArena(be, weights)
        job = B.moe_job(arena, spec, router=False)
        ops, _ = attach_workspace(B, be, job, x.shape[0])
        rc, out, _, _, _ = run_rows(B, be, ops, job, x, logits)
        assert rc == B.OK, be.message()
        outs.append(out)
        assert be.close() == B.OK
    assert (outs[0].view(np.uint32) == outs[1].view(np.uint32)).all()


def test_fixture_file_drives_execute_rows(B, golden, tmp_path):
    """An external MoE input fixture (*.yvex-moe-input: activations of two layers + token ids) is opened by the
    library's reader and its rows run through execute_rows unchanged, like the reference's `graph execute moe`."""
    be, arena, job, spec, x, logits = layer_setup(B, "small_router")
    other = np.random.default_rng(5).standard_normal(x.shape).astype(np.float32)
    image = moe_input_image(0, [spec.hidden, spec.hidden], np.concatenate([other.reshape(-1), x.reshape(-1)]),
                            np.arange(x.shape[0], dtype=np.uint32), layer_indices=[0, 1])
    path = tmp_path / "layer.yvex-moe-input"
    path.write_bytes(image)
    handle = B.vp()
    limits = B.MoeInputLimits(1 << 20)
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(path).encode(), C.byref(limits), C.byref(be.err)) == B.OK, be.message()
    batch = B.RowBatch()
    assert B._lib.yvex_moe_input_row_batch(handle, 1, C.byref(batch), C.byref(be.err)) == B.OK
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    rows, H, k = x.shape[0], spec.hidden, spec.topk
    out, sel, wts = np.zeros((rows, H), np.float32), np.zeros((rows, k), np.uint64), np.zeros((rows, k), np.float32)
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, sel.ctypes.data_as(B.vp), wts.ctypes.data_as(B.vp), sel.size)
    res = B.RowBatchResult()
    assert ops.execute_rows(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err)) == B.OK, be.message()
    assert (sel == golden["layer_small_router_sel"]).all()
    assert rel_l2(out, golden["layer_small_router_out"].view(np.float32)) <= 1e-3
    B._lib.yvex_moe_input_close(C.byref(handle))
    assert be.close() == B.OK


# ---- token-local transaction: begin / add_expert / finish / close (src/backend/cuda/moe.c:504-848) ----------

def token_result(B, H, S=1):
    """A yvex_moe_layer_result with host room for every publication, and the arrays behind it."""
    a = dict(combined=np.zeros(H, np.float32), routed=np.zeros(H, np.float32), shared=np.zeros(H, np.float32),
             post=np.zeros(max(S, 1), np.float32), comb=np.zeros(max(S, 1) ** 2, np.float32))
    r = B.LayerResult()
    r.combined_output, r.combined_capacity = a["combined"].ctypes.data, H
    r.routed_output, r.routed_capacity = a["routed"].ctypes.data, H
    r.shared_output, r.shared_capacity = a["shared"].ctypes.data, H
    r.post, r.post_capacity = a["post"].ctypes.data, a["post"].size
    r.combination, r.combination_capacity = a["comb"].ctypes.data, a["comb"].size
    return r, a


def run_token(B, be, job, spec, row, add_routed=True, shared_first=False):
    """The call sequence of runtime_moe_layer_cuda (src/runtime/moe.c:647-694) for one token."""
    H = spec.hidden
    res, arrays = token_result(B, H, int(job._plan.residual_streams))
    keep = np.ascontiguousarray(row, np.float32)
    job.expanded_input = keep.ctypes.data if not job.device_input else None
    ex = B.vp()
    rc = B._lib.yvex_backend_moe_begin(C.byref(ex), be.h, C.byref(job), C.byref(res), C.byref(be.err))
    if rc != B.OK:
        return rc, res, arrays
    shared = [B.WeightView() for _ in range(3)]
    for v, slot in zip(shared, (B.W_SHARED_GATE, B.W_SHARED_UP, B.W_SHARED_DOWN)):
        C.memmove(C.byref(v), C.byref(job.weights[slot]), C.sizeof(B.WeightView))
    if shared_first:
        rc = B._lib.yvex_backend_moe_add_expert(ex, shared[0], shared[1], shared[2], 1.0, 1, C.byref(be.err))
    for rank in range(int(res.router.selected_count) if add_routed else 0):
        e = int(res.router.selected_experts[rank])
        views = [B.expert_view(job, B.W_GATE, e, spec.inter), B.expert_view(job, B.W_UP, e, spec.inter),
                 B.expert_view(job, B.W_DOWN, e, spec.hidden)]
        if rc == B.OK:
            rc = B._lib.yvex_backend_moe_add_expert(ex, views[0], views[1], views[2], res.router.selected_weights[rank], 0, C.byref(be.err))
    if rc == B.OK and not shared_first:
        rc = B._lib.yvex_backend_moe_add_expert(ex, shared[0], shared[1], shared[2], 1.0, 1, C.byref(be.err))
    if rc == B.OK:
        rc = B._lib.yvex_backend_moe_finish(ex, C.byref(res), C.byref(be.err))
        # a finished transaction takes no more experts and finishes only once
        assert B._lib.yvex_backend_moe_add_expert(ex, shared[0], shared[1], shared[2], 1.0, 1, C.byref(be.err)) == B.INVALID_ARG
        assert B._lib.yvex_backend_moe_finish(ex, C.byref(res), C.byref(be.err)) == B.INVALID_ARG
    assert B._lib.yvex_backend_moe_close(C.byref(ex), C.byref(be.err)) == B.OK and not ex.value
    return rc, res, arrays


@pytest.mark.parametrize("name", ["small_router", "c2_shape"])
def test_token_transaction_vs_frozen_reference(B, golden, name):
    """One token at a time, one expert per call: selection, weights and the combined row against the frozen
    outputs of the reference's CPU layer; bf16(routed + shared) is the combined row bit for bit."""
    be, arena, job, spec, x, _ = layer_setup(B, name)
    attach_workspace(B, be, job, 1)
    want = golden[f"layer_{name}_out"].view(np.float32).reshape(x.shape)
    for t in range(x.shape[0]):
        rc, res, a = run_token(B, be, job, spec, x[t])
        assert rc == B.OK, be.message()
        assert res.router.selected_count == spec.topk
        assert (np.array(res.router.selected_experts[:spec.topk], np.uint64) == golden[f"layer_{name}_sel"].reshape(x.shape[0], -1)[t]).all()
        assert np.abs(np.array(res.router.selected_weights[:spec.topk], np.float32) -
                      golden[f"layer_{name}_w"].view(np.float32).reshape(x.shape[0], -1)[t]).max() <= 2e-7
        assert rel_l2(a["combined"], want[t]) <= 1e-3
        assert (synth.bf16_round(a["routed"] + a["shared"]).view(np.uint32) == a["combined"].view(np.uint32)).all()
        scores = np.array(res.router.router_scores[:spec.experts], np.float64)
        logits = np.array(res.router.router_logits[:spec.experts], np.float64)
        assert np.abs(scores - np.sqrt(np.logaddexp(0.0, logits))).max() <= 1e-6
        assert res.expert_subviews_accessed == 3 * spec.topk and res.kernel_launches >= 5 * (spec.topk + 1)
        assert res.host_to_device_bytes >= x[t].nbytes and res.device_to_host_bytes >= 3 * x[t].nbytes and res.stream_synchronizations == 2
    # the aggregates are f32 sums in call order: the shared expert first changes nothing (it has its own aggregate)
    rc, _, b = run_token(B, be, job, spec, x[0], shared_first=True)
    rc2, _, c = run_token(B, be, job, spec, x[0])
    assert rc == B.OK and rc2 == B.OK and (b["combined"].view(np.uint32) == c["combined"].view(np.uint32)).all()
    assert be.close() == B.OK


def test_token_transaction_device_views_add_the_selected_experts_in_begin(B, golden):
    """With a device input and output, evidence below FULL and device addresses on the routed packs, begin runs the
    selected experts itself (src/runtime/moe.c:654-664 then skips its loop) and finish writes the device output."""
    be, arena, job, spec, x, _ = layer_setup(B, "small_router")
    attach_workspace(B, be, job, 1)
    H = spec.hidden
    rc, res0, host = run_token(B, be, job, spec, x[1])
    assert rc == B.OK
    tin = be.from_array(x[1:2], B.F32)
    rc, tout, _ = be.tensor(H * 4, B.F32, [1, H])
    job.device_input, job.device_output = tin, tout
    for slot in (B.W_GATE, B.W_UP, B.W_DOWN):
        addr = B.ull()
        v = job.weights[slot]
        assert B._lib.yvex_backend_resident_resolve(be.h, v.encoded, v.encoded_bytes, C.byref(addr)) == 1
        v.device_address = addr.value
    rc, res, a = run_token(B, be, job, spec, x[1], add_routed=False)
    assert rc == B.OK, be.message()
    rc, out = be.read(tout, np.float32, H)
    assert rc == B.OK and (out.view(np.uint32) == host["combined"].view(np.uint32)).all()
    assert not a["combined"].any()                       # nothing but the selection is downloaded in this mode
    assert list(res.router.selected_experts[:spec.topk]) == list(res0.router.selected_experts[:spec.topk])
    assert res.expert_subviews_accessed == 3 * spec.topk and res.memory.activation_bytes == 2 * H * 4
    # at FULL evidence the caller adds the experts and everything is published to the host as well
    job.evidence_level = 3
    rc, res, a = run_token(B, be, job, spec, x[1])
    assert rc == B.OK and (a["combined"].view(np.uint32) == host["combined"].view(np.uint32)).all()
    assert be.close() == B.OK


def test_token_transaction_with_envelope_matches_execute_rows(B, golden):
    H, S, T, seed = CASES["envelope"]["small"]
    fn, scale, base, norm, expanded = envelope_inputs("small")
    spec, weights, router, _, _ = layer_inputs("small_router")
    be = B.Backend()
    arena = B.ResidentArena(be, dict(weights, router=router, ffn_norm=norm, mhc_fn=fn, mhc_base=base, mhc_scale=scale))
    job = B.moe_job(arena, spec, residual_streams=S, envelope_policy=ENVELOPE_POLICY)
    ops, _ = attach_workspace(B, be, job, T)
    out = np.zeros((T, S * H), np.float32)
    post, comb, routed, shared = np.zeros((T, S), np.float32), np.zeros((T, S * S), np.float32), np.zeros((T, H), np.float32), np.zeros((T, H), np.float32)
    batch = B.row_batch(T, S * H, host_rows=expanded.ctypes.data_as(B.vp))
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, post=post.ctypes.data_as(B.vp), combination=comb.ctypes.data_as(B.vp),
                     post_capacity=post.size, combination_capacity=comb.size, routed=routed.ctypes.data_as(B.vp),
                     shared=shared.ctypes.data_as(B.vp), routed_capacity=routed.size, shared_capacity=shared.size)
    assert ops.execute_rows(be.h, C.byref(job), C.byref(batch), C.byref(o), C.byref(B.RowBatchResult()), C.byref(be.err)) == B.OK
    for t in range(T):
        rc, res, a = run_token(B, be, job, spec, expanded[t])
        assert rc == B.OK, be.message()
        assert (np.array(res.router.selected_experts[:spec.topk], np.uint64) == golden["envelope_small_sel"].reshape(T, -1)[t]).all()
        assert (a["post"].view(np.uint32) == post[t].view(np.uint32)).all() and (a["comb"].view(np.uint32) == comb[t].view(np.uint32)).all()
        assert rel_l2(a["combined"], synth.bf16_round(routed[t] + shared[t])) <= 1e-3
    # the post step into a device output equals the row batch's expanded output row
    tin = be.from_array(expanded[0:1], B.F32)
    rc, tout, _ = be.tensor(S * H * 4, B.F32, [1, S * H])
    job.device_input, job.device_output, job.evidence_level = tin, tout, 3
    rc, res, a = run_token(B, be, job, spec, expanded[0])
    assert rc == B.OK, be.message()
    rc, got = be.read(tout, np.float32, S * H)
    assert rc == B.OK and rel_l2(got, out[0]) <= 1e-3
    assert be.close() == B.OK


def test_token_transaction_refusals(B):
    be, arena, job, spec, x, _ = layer_setup(B, "small_router")
    H = spec.hidden
    res, arrays = token_result(B, H)
    ex = B.vp()
    row = np.ascontiguousarray(x[0])
    job.expanded_input = row.ctypes.data
    begin = lambda: B._lib.yvex_backend_moe_begin(C.byref(ex), be.h, C.byref(job), C.byref(res), C.byref(be.err))
    assert begin() == B.NOMEM and not ex.value                       # no workspace attached
    attach_workspace(B, be, job, 1)
    res.combined_capacity = H - 1
    assert begin() == B.INVALID_ARG
    res.combined_capacity = H
    keep = job.weights[B.W_ROUTER].encoded
    job.weights[B.W_ROUTER].encoded = None
    assert begin() == B.STATE                                        # the router is not resident
    job.weights[B.W_ROUTER].encoded = keep
    job.weights[B.W_ROUTER].qtype = 11                               # Q3_K: storage only, no decoder
    assert begin() == B.UNSUPPORTED
    job.weights[B.W_ROUTER].qtype = synth.F32
    assert begin() == B.OK and ex.value
    gate, up, down = (B.expert_view(job, B.W_GATE, 1, spec.inter), B.expert_view(job, B.W_UP, 1, spec.inter),
                      B.expert_view(job, B.W_DOWN, 1, spec.hidden))
    add = lambda g, u, d: B._lib.yvex_backend_moe_add_expert(ex, g, u, d, 0.5, 0, C.byref(be.err))
    assert add(gate, up, None) == B.INVALID_ARG
    bad = B.expert_view(job, B.W_GATE, 1, spec.inter - 32)
    assert add(bad, up, down) == B.INVALID_ARG                       # gate and up disagree
    bad = B.expert_view(job, B.W_DOWN, 1, spec.hidden)
    bad.qtype = 13                                                   # Q5_K
    assert add(gate, up, bad) == B.UNSUPPORTED
    bad = B.expert_view(job, B.W_DOWN, 1, spec.hidden)
    bad.row_bytes += 2
    assert add(gate, up, bad) == B.FORMAT
    bad = B.expert_view(job, B.W_DOWN, 1, spec.hidden)
    bad.encoded = 0x10                                               # not in the resident arena
    assert add(gate, up, bad) == B.STATE
    assert add(gate, up, down) == B.OK
    res.routed_capacity = H - 1
    assert B._lib.yvex_backend_moe_finish(ex, C.byref(res), C.byref(be.err)) == B.INVALID_ARG
    res.routed_capacity = H
    assert B._lib.yvex_backend_moe_finish(ex, C.byref(res), C.byref(be.err)) == B.OK
    assert B._lib.yvex_backend_moe_close(C.byref(ex), C.byref(be.err)) == B.OK
    assert B._lib.yvex_backend_moe_close(C.byref(ex), C.byref(be.err)) == B.OK       # closing nothing is fine
    assert be.close() == B.OK


@pytest.mark.parametrize("qtype", [synth.IQ2_XXS, synth.Q2_K, synth.Q8_0, synth.MXFP4, synth.Q4_K, synth.F32])
def test_quant_row_dot_host_row_and_vector(B, port, qtype, monkeypatch):
    """yvex_cuda_quant_row_dot: one encoded row and one vector from host memory (src/backend/cuda/qtype.c:527-700),
    the result against the CPU row dot, and the failure record of each refusal."""
    width = 1024
    if qtype == synth.F32:
        row = np.random.default_rng(3).standard_normal(width).astype(np.float32).view(np.uint8).reshape(1, -1)
    else:
        row = synth.random_blocks(qtype, 1, width, 90 + qtype)
    x = np.random.default_rng(4).standard_normal(width).astype(np.float32)
    rc, want = port.matvec(qtype, row, 1, width, x, allow_q4k=True)
    assert rc == 0
    be = B.Backend()
    out, fail = C.c_float(), B.QuantFailure()
    dot = lambda q, r, nbytes, v, n: B._lib.yvex_cuda_quant_row_dot(be.h, q, r.ctypes.data if r is not None else None, nbytes,
                                                                   v.ctypes.data, n, C.byref(out), C.byref(fail), C.byref(be.err))
    assert dot(qtype, row, row.nbytes, x, width) == B.OK, be.message()
    assert abs(out.value - want[0]) <= 1e-5 * (1 + abs(want[0])) + 2e-6 * np.abs(x).sum() * 4 and fail.code == 0
    assert dot(qtype, None, row.nbytes, x, width) == B.INVALID_ARG and fail.code == 1 and fail.qtype == qtype and fail.operation == 9
    assert dot(11, row, row.nbytes, x, width) == B.UNSUPPORTED and fail.code == 21 and fail.terminal_ordinal == 2 ** 64 - 1
    assert dot(qtype, row, row.nbytes - 1, x, width) == B.BOUNDS and fail.code == 30 and (fail.expected, fail.actual) == (row.nbytes, row.nbytes - 1)
    if qtype not in (synth.F32,):
        elems = synth.BLOCKS[qtype][0]
        assert dot(qtype, row, row.nbytes, x, width - 1) == B.BOUNDS and fail.code == 28 and (fail.expected, fail.actual) == (elems, width - 1)
    monkeypatch.setenv("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "input")
    assert dot(qtype, row, row.nbytes, x, width) == B.BACKEND and fail.code == 45
    monkeypatch.setenv("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE", "output")
    assert dot(qtype, row, row.nbytes, x, width) == B.BACKEND and fail.code == 45
    monkeypatch.delenv("YVEX_TEST_CUDA_QTYPE_COPY_FAILURE")
    assert dot(qtype, row, row.nbytes, x, width) == B.OK and fail.code == 0      # a refused copy does not demote the backend
    if qtype == synth.IQ2_XXS:
        bad = row.copy()
        bad[0, 0:2] = [0x00, 0xFC]                                               # d = -inf
        assert dot(qtype, bad, bad.nbytes, x, width) == B.FORMAT and fail.code == 37
        assert dot(qtype, row, row.nbytes, x, width) == B.OK
    assert be.close() == B.OK


@pytest.mark.parametrize("case", ["small_router", "envelope"])
def test_execute_rows_replays_a_launch_graph_from_the_third_call(B, golden, case, monkeypatch):
    """The narrow entry runs a (layer, row count, buffers) combination eagerly the first time, captures its kernel
    sequence into a launch graph the second time and replays it afterwards (src/backend/cuda/moe.c:1645-1681);
    the rows are the same bit for bit and the result reports launches / captures / replays like the reference."""
    if case == "envelope":
        H, S, T, seed = CASES["envelope"]["small"]
        fn, scale, base, norm, x = envelope_inputs("small")
        spec, weights, router, _, _ = layer_inputs("small_router")
        be = B.Backend()
        arena = B.ResidentArena(be, dict(weights, router=router, ffn_norm=norm, mhc_fn=fn, mhc_base=base, mhc_scale=scale))
        job = B.moe_job(arena, spec, residual_streams=S, envelope_policy=ENVELOPE_POLICY)
        want, logits = golden["envelope_small_out"].view(np.float32), None
    else:
        be, arena, job, spec, x, logits = layer_setup(B, case)
        want = golden[f"layer_{case}_out"].view(np.float32)
    ops, _ = attach_workspace(B, be, job, x.shape[0])
    runs = [run_rows(B, be, ops, job, x, logits) for _ in range(4)]
    assert all(r[0] == B.OK for r in runs), be.message()
    assert rel_l2(runs[0][1], want) <= 1e-3
    for rc, out, sel, wts, res in runs[1:]:
        assert (out.view(np.uint32) == runs[0][1].view(np.uint32)).all() and (sel == runs[0][2]).all()
        assert res.completed == 1 and res.unique_experts == runs[0][4].unique_experts
    counters = [(r[4].graph_launches, r[4].graph_captures, r[4].graph_replays) for r in runs]
    assert counters == [(0, 0, 0), (1, 1, 1), (1, 0, 1), (1, 0, 1)]
    assert runs[0][4].kernel_launches == runs[1][4].kernel_launches == runs[3][4].kernel_launches >= 3
    # another row count is another combination: eager again
    fewer = run_rows(B, be, ops, job, x[:1].copy(), None if logits is None else logits[:1].copy())
    assert fewer[0] == B.OK and fewer[4].graph_launches == 0
    assert (fewer[1].view(np.uint32) == runs[0][1][:1].view(np.uint32)).all()
    # the switch that keeps every call eager
    monkeypatch.setenv("YVEX_B200_MOE_GRAPH", "off")
    off = run_rows(B, be, ops, job, x, logits)
    assert off[0] == B.OK and off[4].graph_launches == 0 and (off[1].view(np.uint32) == runs[0][1].view(np.uint32)).all()
    assert be.close() == B.OK


def test_token_transaction_hash_router_and_bf16_router_rows(B, port):
    """The two other router forms of the transaction: a hash router (the token's table row names the experts, the
    weights still come from the scores) and router weights stored as BF16 rows (projected by the dequant matvec
    instead of the F32 double-accumulation kernel); the chosen experts' outputs against the CPU port."""
    spec, weights, router, x, _ = layer_inputs("small_router")
    H, E, k = spec.hidden, spec.experts, spec.topk
    table = np.array([[5, 2], [1, 7], [0, 3]], np.int32)
    router16 = synth.bf16_bits(router)                               # [E, H] uint16
    be = B.Backend()
    arena = B.ResidentArena(be, dict(weights, router=router, router16=router16, hash_table=table))
    job = B.moe_job(arena, spec, router=True, router_class=0, hash_rows=3)
    attach_workspace(B, be, job, 1)
    # hash router, token 1 -> experts 1 and 7
    job.token_id, job.token_id_present = 1, 1
    rc, res, a = run_token(B, be, job, spec, x[0])
    assert rc == B.OK, be.message()
    assert list(res.router.selected_experts[:k]) == [1, 7]
    logits = np.array(res.router.router_logits[:E], np.float64)
    scores = np.sqrt(np.logaddexp(0.0, logits))
    want_w = scores[[1, 7]] / scores[[1, 7]].sum() * spec.scaling if spec.normalize else scores[[1, 7]] * spec.scaling
    assert np.abs(np.array(res.router.selected_weights[:k]) - want_w).max() <= 1e-6
    xr = synth.bf16_round(x[0])
    routed = np.zeros(H, np.float32)
    for r, e in enumerate([1, 7]):
        rc_e, y = port.expert(H, spec.inter, spec.limit, spec.gate_qtype, spec.up_qtype, spec.down_qtype, weights["gate"][e],
                              weights["up"][e], weights["down"][e], xr, float(res.router.selected_weights[r]))
        assert rc_e == 0
        routed += y
    assert rel_l2(a["routed"], routed) <= 1e-3
    job.token_id = 3                                                 # past the table
    assert run_token(B, be, job, spec, x[0])[0] == B.BOUNDS
    job.token_id_present = 0
    assert run_token(B, be, job, spec, x[0])[0] == B.BOUNDS
    # learned router with BF16 rows: the same selection as the F32 rows rounded to bf16 give on the CPU
    job2 = B.moe_job(arena, spec, router=True)
    v = job2.weights[B.W_ROUTER]
    v.qtype, v.encoded, v.encoded_bytes, v.row_bytes = synth.BF16, arena.host_ptr("router16"), router16.nbytes, H * 2
    rc, res, a = run_token(B, be, job2, spec, x[1])
    assert rc == B.OK, be.message()
    lg = synth.bf16_round(router).astype(np.float64) @ synth.bf16_round(x[1]).astype(np.float64)
    assert np.abs(np.array(res.router.router_logits[:E]) - lg).max() <= 1e-4 * (1 + np.abs(lg).max())
    order = sorted(range(E), key=lambda e: (-np.float32(np.sqrt(np.logaddexp(0.0, np.float32(lg[e])))), e))[:k]
    assert list(res.router.selected_experts[:k]) == order
    assert be.close() == B.OK
