"""CPU-side checks of the drop-in boundary: the shared library loads, exports every symbol the
public headers declare, and refuses bad arguments / unsupported qtypes before touching a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from yvex_b200 import build
    build.build()
    from yvex_b200 import lib as L
    return L


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        text = open(os.path.join(inc, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(yvex_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_symbols() if not hasattr(lib.lib, n)]
    assert not missing, missing
    assert len(declared_symbols()) >= 12
    assert b"sm_100a" in lib.lib.yvex_b200_version()


def test_qtype_registry_is_fail_closed(lib):
    supported = [q for q in range(0, 64) if lib.lib.yvex_b200_qtype_supported(q)]
    assert supported == [0, 1, 8, 10, 12, 16, 30, 39]
    e, b = C.c_uint(), C.c_uint()
    assert lib.lib.yvex_b200_qtype_geometry(16, C.byref(e), C.byref(b)) == 1 and (e.value, b.value) == (256, 66)
    assert lib.lib.yvex_b200_qtype_geometry(12, C.byref(e), C.byref(b)) == 1 and (e.value, b.value) == (256, 144)
    assert lib.lib.yvex_b200_qtype_geometry(43, C.byref(e), C.byref(b)) == 0


def test_entry_points_refuse_before_launch(lib):
    # No device is needed: every refusal below happens before the first CUDA call. Pointers are
    # dummies that must never be dereferenced.
    dummy = C.c_void_p(0x1000)
    L = lib.lib
    # unsupported qtype ids (Q3_K = 11 and Q5_K = 13 have no codec, 43 is unknown)
    for q in (11, 13, 43):
        assert L.yvex_b200_gemv(q, dummy, 8, 256, 110, dummy, 1, None, dummy, 0, dummy, None) == -5
        assert L.yvex_b200_dequant_rows(q, dummy, 8, 256, 110, dummy, dummy, None) == -5
    # row width not block divisible / inconsistent row bytes -> bounds
    assert L.yvex_b200_gemv(16, dummy, 8, 200, 66, dummy, 1, None, dummy, 0, dummy, None) == -7
    assert L.yvex_b200_gemv(16, dummy, 8, 256, 64, dummy, 1, None, dummy, 0, dummy, None) == -7
    # missing pointers -> invalid argument
    assert L.yvex_b200_gemv(16, None, 8, 256, 66, dummy, 1, None, dummy, 0, dummy, None) == -10
    # attention: bad scale, position out of range
    assert L.yvex_b200_attention_gqa_decode(dummy, dummy, dummy, 1, 4, 1, 128, 64, 64, 1.0, dummy, dummy, 1 << 20,
                                            dummy, None) == -7
    assert L.yvex_b200_attention_gqa_decode(dummy, dummy, dummy, 1, 4, 1, 128, 64, 3, -1.0, dummy, dummy, 1 << 20,
                                            dummy, None) == -10
    g = lib.MoeGeometry()
    g.hidden, g.experts, g.topk, g.inter, g.shared_inter = 512, 8, 2, 256, 256
    g.scaling, g.limit, g.normalize, g.router_class = 1.5, 10.0, 1, 1
    g.gate_qtype, g.up_qtype, g.down_qtype = 16, 16, 11          # Q3_K down: admitted storage, no codec
    w = lib.MoeWeights()
    for name, _ in lib.MoeWeights._fields_:
        setattr(w, name, 0x1000)
    assert L.yvex_b200_moe_decode(C.byref(g), C.byref(w), dummy, None, None, 1, dummy, None, None, dummy, 1 << 30,
                                  dummy, None) == -5
    g.down_qtype = 10
    assert L.yvex_b200_moe_decode(C.byref(g), C.byref(w), dummy, None, None, 65, dummy, None, None, dummy, 1 << 30,
                                  dummy, None) == -5      # narrow entry refuses wide batches
    assert L.yvex_b200_moe_decode(C.byref(g), C.byref(w), dummy, None, None, 1, dummy, None, None, dummy, 16,
                                  dummy, None) == -2      # workspace too small
    assert lib.moe_workspace_bytes(g, 1) % 256 == 0 and lib.moe_workspace_bytes(g, 1) > 0


def test_host_boundary_refuses_other_backend_kinds_and_missing_devices(lib):
    import torch
    from yvex_b200 import backend as B
    for kind in (B.KIND_CPU, B.KIND_METAL):
        be = B.Backend(kind=kind)
        assert be.rc == B.UNSUPPORTED and not be.handle.value        # no CPU path, no cross-backend fallback
    assert B.moe_ops(B.Backend(kind=B.KIND_CPU)) is None
    assert lib.lib.yvex_status_name(-5) == b"unsupported"
    if not torch.cuda.is_available():
        be = B.Backend()
        assert be.rc == B.BACKEND and not be.handle.value            # fails loudly without a device
    bad = B.Backend(device=b"tpu:0")
    assert bad.rc == B.INVALID_ARG


def test_compute_without_device_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("device present")
    with pytest.raises(RuntimeError):
        lib.Status()


def layout_table(text):
    return dict(line.rsplit(" ", 1) for line in text.strip().splitlines())


def test_boundary_structs_are_laid_out_as_the_reference_declares_them(lib):
    """Every sizeof / offsetof of the structs that cross the host boundary equals the table
    tests/abi_probe.c printed when it was compiled against the reference's own headers
    (tests/golden/abi_layout.txt, written by tests/golden/make_abi_layout.py), so a caller built
    against those headers can hand its structs over as they are."""
    from yvex_b200 import backend as B
    ours = layout_table(B._lib.yvex_backend_abi_layout().decode())
    want = layout_table(open(os.path.join(ROOT, "tests", "golden", "abi_layout.txt")).read())
    assert ours == want
    assert len(ours) > 190
    # where the reference checkout is at hand, the committed table is still what its headers give
    ref = os.environ.get("YVEX_REF") or os.path.join(os.path.dirname(ROOT), "reference")
    if os.path.isdir(os.path.join(ref, "include", "yvex")):
        import importlib.util
        spec = importlib.util.spec_from_file_location("make_abi_layout", os.path.join(ROOT, "tests", "golden", "make_abi_layout.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        assert layout_table(mod.reference_table(ref)) == want


def test_ctypes_mirror_matches_the_compiled_layout(lib):
    from yvex_b200 import backend as B
    table = layout_table(B._lib.yvex_backend_abi_layout().decode())
    mirror = {"yvex_moe_weight_view": B.WeightView, "yvex_moe_layer_plan": B.LayerPlan,
              "yvex_execution_memory_facts": B.MemoryFacts, "yvex_expert_worklist_observation": B.WorklistObservation,
              "yvex_moe_device_completion_slot": B.CompletionSlot, "yvex_moe_device_completion": B.Completion,
              "yvex_moe_layer_job": B.LayerJob, "yvex_moe_row_batch": B.RowBatch, "yvex_moe_row_batch_output": B.RowBatchOutput,
              "yvex_moe_row_batch_result": B.RowBatchResult, "yvex_moe_input_summary": B.MoeInputSummary,
              "yvex_moe_input_layer_record": B.MoeInputRecord, "yvex_error": B.Error,
              "yvex_moe_router_result": B.RouterResult, "yvex_moe_layer_result": B.LayerResult,
              "yvex_quant_failure": B.QuantFailure}
    for name, cls in mirror.items():
        assert C.sizeof(cls) == int(table[f"sizeof {name}"]), name
        for field, _ in cls._fields_:
            assert getattr(cls, field).offset == int(table[f"offsetof {name}.{field}"]), (name, field)
    ops = {f: getattr(B.MoeOperations, f).offset for f, _ in B.MoeOperations._fields_}
    for f in ("derived_layout_plan", "derived_layout_build", "workspace_required", "execute_rows", "complete_rows"):
        assert ops[f] == int(table[f"offsetof yvex_backend_moe_operations.{f}"])


def test_expert_parallel_entry_refuses_bad_arguments_before_touching_nccl(lib):
    from yvex_b200 import backend as B
    err, need, ep = B.Error(), B.ull(), B.vp()
    plan = B.LayerPlan(schema_version=1, hidden_width=512, routed_experts=8, experts_per_token=2, expert_intermediate_width=256,
                       shared_intermediate_width=256)
    fn = B._lib.yvex_moe_ep_workspace_required
    assert fn(C.byref(plan), 64, 3, C.byref(need), C.byref(err)) == B.INVALID_ARG        # 3 ranks do not divide 8 experts
    assert fn(C.byref(plan), 0, 2, C.byref(need), C.byref(err)) == B.INVALID_ARG
    assert fn(C.byref(plan), 64, 2, C.byref(need), C.byref(err)) == B.OK and need.value % 256 == 0 and need.value > 64 * 2 * 2 * 512
    more = B.ull()
    assert fn(C.byref(plan), 64, 4, C.byref(more), C.byref(err)) == B.OK and more.value > need.value      # room for every rank's pairs
    ident = (C.c_ubyte * 128)()
    assert B._lib.yvex_moe_ep_open(C.byref(ep), None, ident, 2, 0, 1000, C.byref(err)) == B.INVALID_ARG and not ep.value
    assert B._lib.yvex_moe_ep_execute_rows(None, None, None, None, None, C.byref(err)) == B.INVALID_ARG
    assert B._lib.yvex_moe_ep_close(C.byref(ep), C.byref(err)) == B.OK
