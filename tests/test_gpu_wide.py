"""GPU parity tests of the wide (prefill) MoE path: expert-major permute, grouped dequant GEMM on
tcgen05/TMEM, SwiGLU, rank-ordered unpermute. Same oracle, same tolerances as the narrow path:
identical expert selection, relative L2 <= 1e-3 against the CPU path. The reference's own op table
stops at 62 rows (src/graph/worklist.c:316); per-token semantics are the CPU path's, so parity is
checked token by token."""
import numpy as np
import pytest

from golden_cases import CASES, layer_inputs
from yvex_b200 import synth

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


def run_layer(L, spec, weights, router, x, logits, wide=True):
    t = {k: dev(v.reshape(-1)) for k, v in weights.items()}
    if router is not None:
        t["router"] = dev(router)
    st = L.Status()
    out, sel, w = L.moe_layer(L.geometry_of(spec), L.weights_of(t), dev(x), st,
                              logits=None if logits is None else dev(logits), wide=wide)
    return out.cpu().numpy(), sel.cpu().numpy(), w.cpu().numpy(), st.read()


@pytest.mark.parametrize("name", list(CASES["layer"]))
def test_wide_layer_vs_frozen_reference(L, golden, name):
    spec, weights, router, x, logits = layer_inputs(name)           # IQ2_XXS gate/up, Q2_K down
    out, sel, w, status = run_layer(L, spec, weights, router, x, logits)
    assert status == 0
    assert (sel == golden[f"layer_{name}_sel"]).all()
    want = golden[f"layer_{name}_out"].view(np.float32)
    assert rel_l2(out, want) <= 1e-3, rel_l2(out, want)
    assert (synth.bf16_round(out).view(np.uint32) == out.view(np.uint32)).all()


@pytest.mark.parametrize("down", [synth.Q4_K, synth.Q2_K, synth.IQ2_XXS])
def test_wide_layer_ragged_groups_vs_oracle(L, port, down):
    """300 tokens over 8 experts: groups larger than one 128-column tile, ragged tails, and the
    shared expert's 3 token blocks. Q4_K is checked against this repository's restatement
    (reference-unpinned), the others against the reference-pinned port."""
    H, E, k, I, T = 512, 8, 2, 512, 300
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=down)
    rng = np.random.default_rng(41 + down)
    x = rng.standard_normal((T, H)).astype(np.float32)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[:, 5] -= 50.0                                   # expert 5 receives no token: empty group
    weights = synth.moe_weights(spec, 40 + down)
    Lp = port.layer(spec, weights, allow_q4k=True)
    rc, want, sel0, w0 = port.moe_tokens(Lp, x, logits=logits, threads=8)
    out, sel, w, status = run_layer(L, spec, weights, None, x, logits)
    assert rc == 0 and status == 0 and (sel == sel0).all() and not (sel == 5).any()
    assert rel_l2(out, want) <= 1e-3, rel_l2(out, want)
    per_token = np.linalg.norm(out - want, axis=1) / np.linalg.norm(want, axis=1)
    assert per_token.max() <= 4e-3, per_token.max()


@pytest.mark.parametrize("gate", [synth.Q2_K, synth.Q4_K])
def test_wide_layer_affine_gate_and_up_vs_oracle(L, port, gate):
    """Gate and up weights of a qtype with a min term: the fused gate/up GEMM then needs the sub-block
    sums of the ACTIVATION rows as its second operand. 300 tokens over 8 experts, ragged groups."""
    H, E, k, I, T = 512, 8, 2, 256, 300
    spec = synth.MoELayerSpec(H, E, k, I, gate_qtype=gate, down_qtype=synth.IQ2_XXS)
    rng = np.random.default_rng(70 + gate)
    x = rng.standard_normal((T, H)).astype(np.float32)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    weights = synth.moe_weights(spec, 71 + gate)
    Lp = port.layer(spec, weights, allow_q4k=True)
    rc, want, sel0, w0 = port.moe_tokens(Lp, x, logits=logits, threads=8)
    out, sel, w, status = run_layer(L, spec, weights, None, x, logits)
    assert rc == 0 and status == 0 and (sel == sel0).all()
    assert rel_l2(out, want) <= 1e-3, rel_l2(out, want)


def test_expert_parallel_building_blocks_match_single_device_layer_bit_for_bit(L):
    """The expert-parallel decomposition (route -> per-pair rows on the expert shard -> combine on
    the home rank), run here on one rank that owns every expert, and again with the experts split
    into two shards executed one after the other, must equal the fused wide layer exactly: pairs
    travel as whole bf16 rows and are summed in rank order."""
    import torch
    from yvex_b200.ep import DeviceOps, ExpertParallelLayer
    H, E, k, I, T = 512, 8, 2, 256, 200
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q4_K)
    rng = np.random.default_rng(5)
    x, logits = dev(rng.standard_normal((T, H)).astype(np.float32)), dev(rng.standard_normal((T, E)).astype(np.float32))
    t = {kk: dev(v.reshape(-1)) for kk, v in synth.moe_weights(spec, 9).items()}
    st = L.Status()
    g, w = L.geometry_of(spec), L.weights_of(t)
    want, sel0, _ = L.moe_layer(g, w, x, st, logits=logits, wide=True)
    layer = ExpertParallelLayer(E, k, DeviceOps(g, g, w, st))
    got, sel, _ = layer.forward(x, logits)
    assert st.read() == 0 and torch.equal(sel, sel0)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # two shards of 4 experts, pairs routed to each by hand
    xh = x.to(torch.bfloat16).to(torch.float16)
    sel, wts, _ = L.moe_route(g, w, st, logits=logits)
    y = torch.empty((T * k, H), dtype=torch.bfloat16, device="cuda")
    half = synth.MoELayerSpec(H, E // 2, k, I, down_qtype=synth.Q4_K)
    for shard in range(2):
        ts = dict(t)
        for name in ("gate", "up", "down"):
            per = t[name].numel() // E
            ts[name] = t[name][shard * 4 * per:(shard + 1) * 4 * per]
        mask = (sel.reshape(-1) // 4) == shard
        idx = mask.nonzero().reshape(-1)
        rows = xh.index_select(0, idx // k)
        y[idx] = L.moe_expert_rows(L.geometry_of(half), L.weights_of(ts), rows, (sel.reshape(-1)[idx] % 4).contiguous(),
                                   wts.reshape(-1)[idx].contiguous(), st)
    ysh = L.moe_expert_rows(g, w, xh, torch.full((T,), -1, dtype=torch.int32, device="cuda"),
                            torch.ones(T, device="cuda"), st)
    out2 = L.moe_combine(y, ysh, k, st)
    assert st.read() == 0 and torch.equal(out2.view(torch.int32), want.view(torch.int32))


def test_rows_stored_by_address_and_bad_trailers_are_dropped(L):
    """The down GEMM's epilogue stores every pair's row at home_bases[home rank] + home pair * hidden * 2 (here both
    "ranks" are buffers of this device): equal to the rows the list-order entry returns; a trailer that names a rank or
    a pair out of range sets status 2 and leaves its row unwritten."""
    import torch
    H, E, k, I, T = 512, 8, 2, 256, 150
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q2_K)
    rng = np.random.default_rng(77)
    x, logits = dev(rng.standard_normal((T, H)).astype(np.float32)), dev(rng.standard_normal((T, E)).astype(np.float32))
    t = {kk: dev(v.reshape(-1)) for kk, v in synth.moe_weights(spec, 78).items()}
    st = L.Status()
    g, w = L.geometry_of(spec), L.weights_of(t)
    xh = x.to(torch.bfloat16).to(torch.float16)
    sel, wts, _ = L.moe_route(g, w, st, logits=logits)
    payload, inverse, counts = L.ep_dispatch_payload(xh, sel, wts, E, 1, 1, st, rank=0)
    want = L.moe_expert_rows_payload(g, w, payload, st)                     # rows in payload order
    home = torch.zeros((2, T * k, H), dtype=torch.bfloat16, device="cuda")
    bases = torch.tensor([home[0].data_ptr(), home[1].data_ptr()], dtype=torch.int64, device="cuda")
    trailers = payload[:, 2 * H:].view(torch.int32)                        # {local expert, weight, home pair, home rank}
    trailers[::2, 3] = 1                                                    # every other pair lives on "rank" 1
    L.moe_expert_rows_scatter(g, w, payload, bases, T * k, st)
    torch.cuda.synchronize()
    assert st.read() == 0
    pair = trailers[:, 2].long()
    rank = trailers[:, 3].long()
    got = home[rank, pair]
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert int((home.view(torch.int16) != 0).any(dim=2).sum()) == T * k    # nothing stored anywhere else
    home.zero_()
    trailers[0, 3] = 2                                                      # no such rank
    trailers[1, 2] = T * k                                                  # no such pair
    L.moe_expert_rows_scatter(g, w, payload, bases, T * k, st)
    torch.cuda.synchronize()
    assert st.read() == 2
    assert int((home.view(torch.int16) != 0).any(dim=2).sum()) == T * k - 2


def tokens_covering_all_experts(sel, count):
    """Indices of `count` rows of `sel` [T, k] chosen greedily so that every expert is selected by at least one."""
    sel = np.asarray(sel)
    need = set(np.unique(sel).tolist())
    picked = []
    for t in range(sel.shape[0]):
        hit = need.intersection(sel[t].tolist())
        if hit:
            picked.append(t)
            need -= hit
        if not need:
            break
    rest = [t for t in range(sel.shape[0] - 1, -1, -1) if t not in set(picked)]
    picked += rest[:max(0, count - len(picked))]
    return np.array(sorted(picked[:max(count, len(picked))]), np.int64)


def test_wide_matches_narrow_path_at_prefill_size(L, port):
    """Config-3 geometry (2048 tokens, hidden 4096, 64 experts top-6, inter 1536, IQ2_XXS + Q4_K):
    a sample of rows must agree with the narrow path run on those rows alone (rows are
    independent), and 64 rows that between them route to every one of the 64 experts must agree
    with the CPU path (each expert's weight offsets and tile positions are then exercised)."""
    import os
    import torch
    from yvex_b200.workloads import MoEWorkload
    wl = MoEWorkload("c3", 3)
    x, logits = wl.tokens(2048)
    st = L.Status()
    g, w = L.geometry_of(wl.spec), L.weights_of(wl.tensors)
    out, sel, wt = L.moe_layer(g, w, x, st, logits=logits, wide=True)
    idx = torch.tensor([0, 1, 127, 128, 777, 1500, 2046, 2047], device="cuda")
    out_n, sel_n, _ = L.moe_layer(g, w, x[idx].contiguous(), st, logits=logits[idx].contiguous(), wide=False)
    assert st.read() == 0 and (sel[idx] == sel_n).all()
    assert rel_l2(out[idx].cpu().numpy(), out_n.cpu().numpy()) <= 5e-4
    hw, _ = wl.host_copy()
    Lp = port.layer(wl.spec, hw, allow_q4k=True)
    pick = tokens_covering_all_experts(sel.cpu().numpy(), 64)
    assert pick.size >= 64 and set(np.unique(sel.cpu().numpy()[pick]).tolist()) == set(range(64))
    tp = torch.from_numpy(pick).cuda()
    rc, want, sel0, _ = port.moe_tokens(Lp, x[tp].cpu().numpy(), logits=logits[tp].cpu().numpy(), threads=os.cpu_count() or 8)
    assert rc == 0 and (sel[tp].cpu().numpy() == sel0).all()
    got = out[tp].cpu().numpy()
    assert rel_l2(got, want) <= 1e-3
    per_token = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    assert per_token.max() <= 4e-3, per_token.max()


def test_wide_config3_pinned_twin_vs_oracle(L, port):
    """The same geometry with Q2_K down weights - the qtype the reference's own MoE path decodes - so
    that the prefill path has a reference-pinned check at full size, on 64 rows covering all experts."""
    import os
    import torch
    from yvex_b200.workloads import MoEWorkload
    wl = MoEWorkload("c3", 3, down_qtype=synth.Q2_K)
    x, logits = wl.tokens(2048)
    st = L.Status()
    out, sel, _ = L.moe_layer(L.geometry_of(wl.spec), L.weights_of(wl.tensors), x, st, logits=logits, wide=True)
    hw, _ = wl.host_copy()
    Lp = port.layer(wl.spec, hw)
    pick = tokens_covering_all_experts(sel.cpu().numpy(), 64)
    tp = torch.from_numpy(pick).cuda()
    rc, want, sel0, _ = port.moe_tokens(Lp, x[tp].cpu().numpy(), logits=logits[tp].cpu().numpy(), threads=os.cpu_count() or 8)
    assert rc == 0 and st.read() == 0 and (sel[tp].cpu().numpy() == sel0).all()
    assert rel_l2(out[tp].cpu().numpy(), want) <= 1e-3


def test_wide_config5_size_properties(L, port):
    """Config-5 geometry on one device (16 384 tokens, hidden 7168, 256 experts top-8 + shared, inter 2048,
    IQ2_XXS + Q4_K). Size-independent properties: rows are independent, so a permuted batch gives the
    permuted result bit for bit (other column blocks, other tiles, same per-row arithmetic) and a
    sample of rows agrees with the decode path run on those rows alone; 16 rows spread over the batch
    are checked against the CPU path within the layer tolerance."""
    import os
    import torch
    from yvex_b200.workloads import MoEWorkload
    wl = MoEWorkload("c5", 5)
    T = wl.cfg["tokens"]
    x, logits = wl.tokens(T)
    st = L.Status()
    g, w = L.geometry_of(wl.spec), L.weights_of(wl.tensors)
    ws = torch.empty(L.moe_workspace_bytes(g, T, True), dtype=torch.uint8, device="cuda")
    out, sel, wt = L.moe_layer(g, w, x, st, logits=logits, wide=True, workspace=ws)
    assert st.read() == 0 and torch.isfinite(out).all()
    perm = torch.randperm(T, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    out_p, sel_p, _ = L.moe_layer(g, w, x[perm].contiguous(), st, logits=logits[perm].contiguous(), wide=True, workspace=ws)
    assert st.read() == 0 and (sel_p == sel[perm]).all()
    assert torch.equal(out_p.view(torch.int32), out[perm].view(torch.int32))
    idx = torch.tensor([0, 255, 256, 4095, 9000, 16383], device="cuda")
    out_n, sel_n, _ = L.moe_layer(g, w, x[idx].contiguous(), st, logits=logits[idx].contiguous(), wide=False)
    assert st.read() == 0 and (sel[idx] == sel_n).all()
    assert rel_l2(out[idx].cpu().numpy(), out_n.cpu().numpy()) <= 5e-4
    hw, _ = wl.host_copy()
    Lp = port.layer(wl.spec, hw, allow_q4k=True)
    some = torch.arange(16, device="cuda") * 1023 + 7                       # 16 rows across the batch: 128 pairs + 16 shared
    rc, want, sel0, _ = port.moe_tokens(Lp, x[some].cpu().numpy(), logits=logits[some].cpu().numpy(), threads=min(16, os.cpu_count() or 8))
    assert rc == 0 and (sel[some].cpu().numpy() == sel0).all()
    got = out[some].cpu().numpy()
    assert rel_l2(got, want) <= 1e-3
    assert (np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)).max() <= 4e-3


@pytest.mark.parametrize("world,tokens,topk,experts", [(8, 300, 8, 256), (2, 64, 6, 64), (4, 1, 4, 16)])
def test_ep_dispatch_matches_the_tensor_formulation(L, world, tokens, topk, experts):
    """yvex_b200_ep_dispatch against the stable-argsort formulation the layer uses without it."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(tokens)
    per_rank, H = experts // world, 256
    sel = torch.stack([torch.randperm(experts, device="cuda", generator=g)[:topk] for _ in range(tokens)]).to(torch.int32)
    wts = torch.rand((tokens, topk), device="cuda", generator=g)
    xh = torch.randn((tokens, H), device="cuda", generator=g).to(torch.float16)
    st = L.Status()
    send_rows, meta, inverse, counts = L.ep_dispatch(xh, sel, wts, per_rank, world, st)
    assert st.read() == 0
    dest = (sel // per_rank).reshape(-1).to(torch.int64)
    order = torch.argsort(dest, stable=True)
    assert torch.equal(counts, torch.bincount(dest, minlength=world))
    assert torch.equal(send_rows, xh.index_select(0, torch.div(order, topk, rounding_mode="floor")))
    want_meta = torch.stack(((sel % per_rank).reshape(-1), wts.reshape(-1).view(torch.int32)), dim=1).index_select(0, order)
    assert torch.equal(meta, want_meta)
    want_inv = torch.empty_like(order)
    want_inv[order] = torch.arange(order.numel(), device="cuda")
    assert torch.equal(inverse.to(torch.int64), want_inv)
    # an expert id outside world * per_rank raises the argument status instead of indexing past the bins
    bad = sel.clone()
    bad[0, 0] = experts
    L.ep_dispatch(xh, bad, wts, per_rank, world, st)
    torch.cuda.synchronize()
    assert st.read() == 2
