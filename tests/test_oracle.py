"""Pins the CPU restatement (oracle/yvex_oracle.c) before anything trusts it:

1. against the golden blocks and known answers the reference's own unit tests hold
   (tests/unit/quant_numeric.c:502-609, tests/unit/runtime_moe.c:111-212,
   tests/unit/qtype_support.c:54-56, tests/unit/gguf_qtype_abi.c:35,251);
2. bit-for-bit against outputs of the unmodified reference frozen in tests/golden/;
3. where the compiled reference is present, bit-for-bit against it live.
"""
import math

import numpy as np
import pytest

from golden_cases import CASES, ENVELOPE_POLICY, attention_inputs, envelope_inputs, layer_inputs
from golden.make_golden import iq2_exhaustive_blocks
from yvex_b200 import synth

OK, FORMAT, UNSUPPORTED, BOUNDS, INVALID = 0, -4, -5, -7, -10


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


# ---- 1. the reference's own golden vectors -------------------------------------------------

def test_q8_0_golden_block(port):
    # tests/unit/quant_numeric.c:516-527: scale 1.0 (00 3c), codes 7f 81 01 ff.
    blk = np.zeros(34, np.uint8)
    blk[:6] = [0x00, 0x3C, 0x7F, 0x81, 0x01, 0xFF]
    rc, out = port.decode_block(synth.Q8_0, blk, 32)
    assert rc == OK
    assert out[:4].tolist() == [127.0, -127.0, 1.0, -1.0] and not out[4:].any()


def test_q2_k_golden_block(port):
    # tests/unit/quant_numeric.c:560-573: scales 0x01, codes 0xe4, d = 1.0.
    blk = np.zeros(84, np.uint8)
    blk[:16] = 0x01
    blk[16:80] = 0xE4
    blk[80:82] = [0x00, 0x3C]
    rc, out = port.decode_block(synth.Q2_K, blk, 256)
    assert rc == OK
    assert out.tolist() == [float((i % 128) // 32) for i in range(256)]


def test_mxfp4_golden_block(port):
    # tests/unit/quant_numeric.c:529-540: E8M0 127 -> scale 1 * 0.5, nibbles 1 (low) / 2 (high).
    blk = np.full(17, 0x21, np.uint8)
    blk[0] = 127
    rc, out = port.decode_block(39, blk, 32)
    assert rc == OK and (out[:16] == 0.5).all() and (out[16:] == 1.0).all()
    blk[:] = 0x77
    blk[0] = 254
    assert port.decode_block(39, blk, 32)[0] == FORMAT


def test_malformed_scales_refuse(port):
    # tests/unit/quant_numeric.c:575-594.
    blk = np.zeros(34, np.uint8)
    blk[1] = 0x7C
    assert port.decode_block(synth.Q8_0, blk, 32)[0] == FORMAT
    blk = np.zeros(84, np.uint8)
    blk[81] = 0x7C
    assert port.decode_block(synth.Q2_K, blk, 256)[0] == FORMAT
    blk = np.zeros(66, np.uint8)
    blk[1] = 0xBC  # d = -1.0
    assert port.decode_block(synth.IQ2_XXS, blk, 256)[0] == FORMAT
    assert port.decode_block(synth.IQ2_XXS, np.zeros(65, np.uint8), 256)[0] == FORMAT


def test_q4_k_is_storage_only_unless_extension(port):
    # tests/unit/qtype_support.c:54-56, tests/unit/gguf_qtype_abi.c:35: geometry 256/144, no codec.
    assert port.geometry(synth.Q4_K) == (256, 144)
    assert port.capability(synth.Q4_K) == 1
    assert port.decode_block(synth.Q4_K, np.zeros(144, np.uint8), 256)[0] == UNSUPPORTED
    assert port.capability(synth.Q4_K, allow_q4k=True) & 4
    assert port.capability(43) == -1
    assert port.decode_block(43, np.zeros(4, np.uint8), 1)[0] == UNSUPPORTED


def test_router_known_answers(port):
    # tests/unit/runtime_moe.c:111-171.
    spec = synth.MoELayerSpec(4, 4, 2, 2)
    router = np.array([[1, 0, 0, 0], [2, 0, 0, 0], [2, 0, 0, 0], [0, 0, 0, 0]], np.float32)
    bias = np.array([5, 0, 0, 0], np.float32)
    x = np.array([1, 0, 0, 0], np.float32)
    score = lambda v: math.sqrt(v + math.log1p(math.exp(-v)))
    L = port.layer(spec, {}, router=router, bias=bias)
    rc, sel, w, _, _ = port.route(L, x)
    assert rc == OK and sel.tolist() == [0, 1]
    a, b = score(1.0), score(2.0)
    assert abs(w[0] - a / (a + b) * 1.5) < 1e-6 and abs(w[1] - b / (a + b) * 1.5) < 1e-6
    bias[0] = 0
    rc, sel, _, _, _ = port.route(L, x)
    assert rc == OK and sel.tolist() == [1, 2]
    table = np.array([3, 1], np.int32)
    L = port.layer(spec, {}, router=router, hash_table=table, hash_rows=8, router_class=0)
    rc, sel, _, _, _ = port.route(L, x, token_id=4)
    assert rc == OK and sel.tolist() == [3, 1]
    table[1] = 3
    assert port.route(L, x, token_id=4)[0] == FORMAT
    assert port.route(L, x, token_id=8)[0] == BOUNDS


def test_expert_known_answer(port):
    # tests/unit/runtime_moe.c:178-212 (F32 weights, bf16 boundaries matched exactly).
    gate = np.array([[1, 2], [-1, 1]], np.float32)
    up = np.array([[2, 0], [1, 3]], np.float32)
    down = np.array([[1, 0.5], [-0.25, 2]], np.float32)
    x = np.array([1, 2], np.float32)
    mid = []
    for r in range(2):
        g = float(gate[r] @ x)
        u = float(up[r] @ x)
        mid.append(float(synth.bf16_round(np.array([g / (1 + math.exp(-g)) * u * 0.25], np.float32))[0]))
    want = synth.bf16_round((down.astype(np.float32) @ np.array(mid, np.float32)))
    rc, out = port.expert(2, 2, 10.0, 0, 0, 0, gate, up, down, x, 0.25)
    assert rc == OK and bits(out).tolist() == bits(want).tolist()


def test_worklist_is_expert_major_and_stable(port):
    # src/graph/worklist.c:369-441: ascending expert, ascending pair inside a bucket, empty
    # experts get no bucket.
    sel = np.array([[3, 1], [1, 0], [3, 5]], np.uint64)
    rc, order, src, be, bo, bc = port.worklist(sel, 8)
    assert rc == OK
    assert be.tolist() == [0, 1, 3, 5] and bc.tolist() == [1, 2, 2, 1]
    assert bo.tolist() == [0, 1, 3, 5, 6]
    assert order.tolist() == [3, 1, 2, 0, 4, 5] and src.tolist() == [1, 0, 1, 0, 2, 2]


def test_f16_bf16_exhaustive_against_numpy(port):
    # tests/unit/quant_numeric.c:188-259 walks all 65 536 encodings; numpy's float16 is IEEE.
    codes = np.arange(65536, dtype=np.uint16)
    want = codes.view(np.float16).astype(np.float32)
    got = np.array([port.f16_decode(int(c)) for c in codes[::7]], np.float32)
    w = want[::7]
    nan = np.isnan(w)
    assert (bits(got)[~nan] == bits(w)[~nan]).all() and np.isnan(got[nan]).all()
    vals = np.random.default_rng(5).standard_normal(4096).astype(np.float32)
    vals[:4] = [0.0, -0.0, 1.00390625, 3.3895314e38]
    enc = np.array([port.bf16_encode(float(v)) for v in vals], np.uint16)
    assert (enc == synth.bf16_bits(vals)).all()


# ---- 2. frozen outputs of the unmodified reference -----------------------------------------

@pytest.mark.parametrize("name", list(CASES["matvec"]))
def test_decode_and_matvec_match_frozen_reference(port, golden, name):
    qtype, rows, width, seed = CASES["matvec"][name]
    w = synth.random_blocks(qtype, rows, width, seed)
    x = np.random.default_rng(seed + 1).standard_normal(width).astype(np.float32)
    rc, dec = port.decode_rows(qtype, w, rows, width)
    assert rc == OK and (bits(dec) == golden[f"decode_{name}"]).all()
    rc, y = port.matvec(qtype, w, rows, width, x)
    assert rc == OK and (bits(y) == golden[f"matvec_{name}"]).all()


def test_iq2_xxs_every_grid_sign_and_subscale(port, golden):
    blocks = iq2_exhaustive_blocks()
    rc, dec = port.decode_rows(synth.IQ2_XXS, blocks, blocks.shape[0], 256)
    assert rc == OK and (bits(dec) == golden["decode_iq2_exhaustive"]).all()


@pytest.mark.parametrize("name", list(CASES["layer"]))
def test_layer_matches_frozen_reference(port, golden, name):
    spec, weights, router, x, logits = layer_inputs(name)
    L = port.layer(spec, weights, router=router)
    rc, y, sel, w = port.moe_tokens(L, x, logits=logits, threads=8)
    assert rc == OK
    assert (sel == golden[f"layer_{name}_sel"]).all()
    assert (bits(w) == golden[f"layer_{name}_w"]).all()
    assert (bits(y) == golden[f"layer_{name}_out"]).all()


@pytest.mark.parametrize("name", list(CASES["attention"]))
def test_attention_matches_frozen_reference(port, golden, name):
    q, k, v, pos, scale = attention_inputs(name)
    rc, out = port.attention_gqa_decode(synth.bf16_bits(q).reshape(q.shape),
                                        synth.bf16_bits(k).reshape(k.shape),
                                        synth.bf16_bits(v).reshape(v.shape), pos, scale, threads=4)
    assert rc == OK and (bits(out) == golden[f"attention_{name}"]).all()


# ---- 3. live comparison with the compiled reference ----------------------------------------

@pytest.mark.parametrize("name", list(CASES["envelope"]))
def test_mhc_envelope_matches_frozen_reference(port, golden, name):
    """prepare (gates, Sinkhorn, collapse, RMSNorm, bf16 rounding) and post bit-for-bit; the "small"
    case runs the small_router layer between the two."""
    H, S, T, seed = CASES["envelope"][name]
    fn, scale, base, norm, expanded = envelope_inputs(name)
    M = port.mhc(H, S, fn, scale, base, norm, **ENVELOPE_POLICY)
    got = [port.mhc_prepare(M, expanded[t]) for t in range(T)]
    assert all(g[0] == 0 for g in got)
    normalized = np.stack([g[1] for g in got])
    posts, combs = np.stack([g[2] for g in got]), np.stack([g[3] for g in got])
    assert np.array_equal(normalized.view(np.uint32), golden[f"envelope_{name}_norm"])
    assert np.array_equal(posts.view(np.uint32), golden[f"envelope_{name}_post"])
    assert np.array_equal(combs.view(np.uint32), golden[f"envelope_{name}_comb"])
    # the stream combination is (almost) doubly stochastic after the Sinkhorn rounds
    c = combs.reshape(T, S, S)
    assert np.allclose(c.sum(axis=1), 1.0, atol=1e-4)
    core = np.random.default_rng(seed + 7).standard_normal((T, H)).astype(np.float32)
    if name == "small":
        spec, weights, router, _, _ = layer_inputs("small_router")
        rc, core, sel, _ = port.moe_tokens(port.layer(spec, weights, router=router), normalized, threads=4)
        assert rc == 0 and np.array_equal(sel.astype(np.uint16), golden["envelope_small_sel"])
    outs = np.stack([port.mhc_post(M, core[t], expanded[t], posts[t], combs[t])[1] for t in range(T)])
    assert np.array_equal(outs.view(np.uint32), golden[f"envelope_{name}_out"])


def test_mhc_envelope_refuses_bad_geometry_and_numerics(port):
    fn, scale, base, norm, expanded = envelope_inputs("two_streams")
    H, S = 768, 2
    bad = expanded[0].copy()
    bad[5] = np.inf
    assert port.mhc_prepare(port.mhc(H, S, fn, scale, base, norm, **ENVELOPE_POLICY), bad)[0] == -4
    nan_base = base.copy()
    nan_base[1] = np.nan
    assert port.mhc_prepare(port.mhc(H, S, fn, scale, nan_base, norm, **ENVELOPE_POLICY), expanded[0])[0] == -4
    # (streams + 2) * streams must fit the reference's 64 mixing rows (src/graph/moe.c:455)
    assert port.mhc_prepare(port.mhc(64, 8, np.zeros((80, 8 * 64), np.float32), scale, np.zeros(80, np.float32),
                                     np.ones(64, np.float32), **ENVELOPE_POLICY), np.zeros(8 * 64, np.float32))[0] == -10


def test_geometry_and_capability_table_match_reference(port, ref):
    for q in range(0, 45):
        assert port.geometry(q) == ref.geometry(q), q
        rc = ref.capability(q)
        mine = port.capability(q)
        assert (mine < 0) == (rc < 0), q
        if rc >= 0:  # the reference also reports encoder availability (bit 1); not on this path
            assert (mine & ~2) == (rc & ~2), q


@pytest.mark.parametrize("qtype", [synth.IQ2_XXS, synth.Q2_K, synth.Q8_0])
def test_random_rows_match_reference_live(port, ref, qtype):
    w = synth.random_blocks(qtype, 48, 2048, 77 + qtype, lo=6e-8, hi=2.0)
    x = np.random.default_rng(3).standard_normal(2048).astype(np.float32)
    a, b = port.decode_rows(qtype, w, 48, 2048), ref.decode_rows(qtype, w, 48, 2048)
    assert a[0] == b[0] == OK and (bits(a[1]) == bits(b[1])).all()
    a, b = port.matvec(qtype, w, 48, 2048, x), ref.matvec(qtype, w, 48, 2048, x)
    assert a[0] == b[0] == OK and (bits(a[1]) == bits(b[1])).all()


def test_refusals_match_reference_live(port, ref):
    w = synth.random_blocks(synth.IQ2_XXS, 1, 256, 1)
    x = np.ones(256, np.float32)
    for lib in (port, ref):
        assert lib.matvec(synth.Q4_K, np.zeros((1, 144), np.uint8), 1, 256, x)[0] == UNSUPPORTED
        assert lib.matvec(synth.IQ2_XXS, w, 1, 200, x)[0] == BOUNDS
    x[7] = np.inf
    assert port.matvec(synth.IQ2_XXS, w, 1, 256, x)[0] == ref.matvec(synth.IQ2_XXS, w, 1, 256, x)[0] == FORMAT


def test_q4_k_extension_is_self_consistent(port):
    # No reference decoder exists for Q4_K (parity unpinned): check the restatement against an
    # independent numpy reading of the public block description.
    w = synth.random_blocks(synth.Q4_K, 3, 512, 9)
    rc, dec = port.decode_rows(synth.Q4_K, w, 3, 512, allow_q4k=True)
    assert rc == OK
    blk = w.reshape(-1, 144)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = blk[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    s = blk[:, 4:16].astype(np.uint32)
    want = np.zeros((blk.shape[0], 256), np.float32)
    for j in range(8):
        if j < 4:
            sc, m = s[:, j] & 63, s[:, j + 4] & 63
        else:
            sc = (s[:, j + 4] & 15) | ((s[:, j - 4] >> 6) << 4)
            m = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
        q = blk[:, 16 + 32 * (j // 2):48 + 32 * (j // 2)]
        code = (q >> 4) if j & 1 else (q & 15)
        scale = (d * sc.astype(np.float32)).astype(np.float32)
        mn = (dmin * m.astype(np.float32)).astype(np.float32)
        want[:, 32 * j:32 * j + 32] = scale[:, None] * code.astype(np.float32) - mn[:, None]
    assert (bits(dec.reshape(-1, 256)) == bits(want)).all()


def test_sink_attention_restatement_properties():
    """The sink only adds exp(sink - max) to the denominator: a very negative sink gives plain softmax attention
    over the rows, no rows give a zero output, and a dominant sink shrinks the output towards zero."""
    from oracle_lib import sink_attention
    rng = np.random.default_rng(5)
    q, rows = rng.standard_normal((3, 64)).astype(np.float32), rng.standard_normal((40, 64)).astype(np.float32)
    out = sink_attention(q, rows, np.full(3, -1e30, np.float32), 0.125, round_bf16=False)
    s = (rows.astype(np.float64) @ q.astype(np.float64).T) * 0.125
    p = np.exp(s - s.max(axis=0))
    want = (p / p.sum(axis=0)).T @ rows.astype(np.float64)
    assert np.abs(out - want).max() <= 1e-5
    assert not sink_attention(q, rows[:0], np.zeros(3, np.float32), 0.125).any()
    big = sink_attention(q, rows, np.full(3, 50.0, np.float32), 0.125, round_bf16=False)
    assert np.abs(big).max() < 1e-12 * 1e3 + np.abs(out).max() * 1e-15 + 1e-9
