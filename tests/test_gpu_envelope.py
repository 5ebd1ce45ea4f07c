"""GPU parity of the mHC envelope (yvex_b200_mhc_prepare / yvex_b200_mhc_post) against the frozen
outputs of the unmodified reference and against the CPU oracle, through the C ABI.

Tolerances: gates and the stream combination are doubles rounded to f32 on both sides and must
agree to 1e-6 relative; the collapsed/normalized rows and the re-expanded rows are bf16-rounded, so
an element may differ by one bf16 step (2^-8 relative) where a sum lands on a rounding boundary
after a different summation order: at most 0.5 % of the elements may differ at all, none by more
than one step, and the relative L2 error stays below 1e-3 (the layer-output bound of
tests/live/moe_deepseek.c:232-241)."""
import numpy as np
import pytest

from golden_cases import CASES, ENVELOPE_POLICY, envelope_inputs, layer_inputs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from yvex_b200 import lib
    return lib


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bf16_close(got, want):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    differ = got.view(np.uint32) != want.view(np.uint32)
    step = np.abs(want) * 2.0 ** -7 + 1e-30
    return differ.mean() <= 5e-3 and np.all(np.abs(got - want)[differ] <= step[differ]) and rel_l2(got, want) <= 1e-3


def run_prepare(L, name):
    H, S, T, seed = CASES["envelope"][name]
    fn, scale, base, norm, expanded = envelope_inputs(name)
    m = L.mhc_of(H, S, dev(fn), dev(scale), dev(base), dev(norm), **ENVELOPE_POLICY)
    st = L.Status()
    x = dev(expanded)
    normalized, post, comb = L.mhc_prepare(m, x, st)
    assert st.read() == 0
    return m, st, x, normalized, post, comb


@pytest.mark.parametrize("name", list(CASES["envelope"]))
def test_mhc_prepare_and_post_vs_frozen_reference(L, golden, name):
    H, S, T, seed = CASES["envelope"][name]
    m, st, x, normalized, post, comb = run_prepare(L, name)
    want_post = golden[f"envelope_{name}_post"].view(np.float32)
    want_comb = golden[f"envelope_{name}_comb"].view(np.float32)
    assert np.allclose(post.cpu().numpy(), want_post, rtol=1e-6, atol=1e-7)
    assert np.allclose(comb.cpu().numpy(), want_comb, rtol=1e-6, atol=1e-7)
    assert bf16_close(normalized.cpu().numpy(), golden[f"envelope_{name}_norm"].view(np.float32))
    # post on the reference's own gates, so only this kernel is under test
    core = np.random.default_rng(seed + 7).standard_normal((T, H)).astype(np.float32)
    if name == "small":
        return                                           # covered end to end below
    out = L.mhc_post(m, dev(core), x, dev(want_post), dev(want_comb), st)
    assert st.read() == 0
    want = golden[f"envelope_{name}_out"].view(np.float32)
    assert bf16_close(out.cpu().numpy(), want)


def test_envelope_around_the_layer_end_to_end(L, golden):
    """expanded rows -> prepare -> MoE layer (router projection on device) -> post -> expanded rows."""
    import torch
    H, S, T, seed = CASES["envelope"]["small"]
    m, st, x, normalized, post, comb = run_prepare(L, "small")
    spec, weights, router, _, _ = layer_inputs("small_router")
    geom = L.geometry_of(spec)
    wdev = {k: dev(v) for k, v in weights.items()}
    wdev["router"] = dev(router)
    w = L.weights_of(wdev)
    sel = torch.empty((T, spec.topk), dtype=torch.int32, device="cuda")
    core = L.moe_layer(geom, w, normalized, st, selected=sel)[0]
    out = L.mhc_post(m, core, x, post, comb, st)
    assert st.read() == 0
    assert np.array_equal(sel.cpu().numpy().astype(np.uint16), golden["envelope_small_sel"])
    want = golden["envelope_small_out"].view(np.float32)
    assert rel_l2(out.cpu().numpy(), want) <= 1e-3


def test_envelope_refusals(L):
    import torch
    fn, scale, base, norm, expanded = envelope_inputs("two_streams")
    st = L.Status()
    x = dev(expanded)
    ok = L.mhc_of(768, 2, dev(fn), dev(scale), dev(base), dev(norm), **ENVELOPE_POLICY)
    before = L.lib.yvex_b200_launch_count()
    with pytest.raises(L.YvexError) as e:
        L.mhc_prepare(L.mhc_of(768, 8, dev(fn), dev(scale), dev(base), dev(norm), **ENVELOPE_POLICY), x, st)
    assert e.value.code == -7                                            # more streams than the 64 mixing rows allow
    bad_policy = dict(ENVELOPE_POLICY, mhc_epsilon=0.0)
    with pytest.raises(L.YvexError) as e:
        L.mhc_prepare(L.mhc_of(768, 2, dev(fn), dev(scale), dev(base), dev(norm), **bad_policy), x, st)
    assert e.value.code == -10
    assert L.lib.yvex_b200_launch_count() == before                     # refused before any launch
    # a non-finite input raises the numerics status instead of publishing
    bad = expanded.copy()
    bad[0, 3] = np.nan
    L.mhc_prepare(ok, dev(bad), st)
    torch.cuda.synchronize()
    assert st.read() == 1
