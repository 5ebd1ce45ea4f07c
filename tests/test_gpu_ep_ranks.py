"""The expert-parallel layer on two real ranks (one process per GPU, NCCL): the sharded, pipelined
exchange must reproduce the single-device wide layer bit for bit on every rank's own tokens.
Skipped on boxes with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, segments, overlap, peer_return, peer_dispatch, ret):
    import torch
    import torch.distributed as dist
    from yvex_b200 import lib, synth
    from yvex_b200.ep import DeviceOps, ExpertParallelLayer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    H, E, k, I, T = 512, 8, 2, 256, 600
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q2_K)
    rng = np.random.default_rng(17)                                   # the same inputs and weights on every rank
    x_all = torch.from_numpy(rng.standard_normal((T * world, H)).astype(np.float32)).to(dev)
    lg_all = torch.from_numpy(rng.standard_normal((T * world, E)).astype(np.float32)).to(dev)
    lg_all[:, 5] -= 50.0                                              # one expert receives nothing
    full = {n: torch.from_numpy(np.ascontiguousarray(v.reshape(-1))).to(dev) for n, v in synth.moe_weights(spec, 18).items()}
    per = E // world
    shard = dict(full)
    for name in ("gate", "up", "down"):
        n = full[name].numel() // E
        shard[name] = full[name][rank * per * n:(rank + 1) * per * n]
    st = lib.Status(dev)
    g_full = lib.geometry_of(spec)
    g_local = lib.geometry_of(synth.MoELayerSpec(H, per, k, I, down_qtype=synth.Q2_K))
    layer = ExpertParallelLayer(E, k, DeviceOps(g_full, g_local, lib.weights_of(shard), st, overlap=overlap, peer_return=peer_return,
                                                    peer_dispatch=peer_dispatch),
                                segments=segments)
    x, lg = x_all[rank * T:(rank + 1) * T].contiguous(), lg_all[rank * T:(rank + 1) * T].contiguous()
    ok = True
    for _ in range(3):                                                # buffers are reused from the second step on
        out, sel, _ = layer.forward(x, lg)
        want, sel0, _ = lib.moe_layer(g_full, lib.weights_of(full), x, st, logits=lg, wide=True)
        torch.cuda.synchronize()
        ok = ok and torch.equal(sel, sel0) and torch.equal(out.view(torch.int32), want.view(torch.int32))
    ret[rank] = (bool(ok), st.read(), layer.ops.home is not None, layer.ops.inbox is not None)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("segments,overlap,peer_return,peer_dispatch", [
    (1, False, True, True), (2, False, True, True), (1, False, False, True), (1, False, True, False), (2, True, True, False),
    (2, True, False, False), (1, False, False, False), (4, True, False, False)])
def test_two_ranks_match_the_single_device_layer_bit_for_bit(segments, overlap, peer_return, peer_dispatch):
    """peer_return: the down GEMM's epilogue stores every pair's row straight into its home rank's memory
    (plain peer stores), else the rows come back by a second all-to-all-v."""
    import torch
    import torch.multiprocessing as mp
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), segments, overlap, peer_return, peer_dispatch, ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, 0, peer_return, peer_dispatch), 1: (True, 0, peer_return, peer_dispatch)}


# ---- the C11 orchestration over NCCL send/recv groups (yvex_moe_ep_*) -------------------------------------------

def _c_worker(rank, world, id_path, absent_step, ret):
    """One rank of the C11 expert-parallel entry: its own backend, its shard resident, host rows in and out."""
    import ctypes as C
    import time
    import torch
    from yvex_b200 import backend as B, lib, synth
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    H, E, k, I, T = 512, 8, 2, 256, 300 + 50 * rank                     # the ranks bring different row counts
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=synth.Q2_K)
    rng = np.random.default_rng(23)
    counts = [300 + 50 * r for r in range(world)]
    x_all = rng.standard_normal((sum(counts), H)).astype(np.float32)
    lg_all = rng.standard_normal((sum(counts), E)).astype(np.float32)
    lg_all[:, 3] -= 50.0                                                # one expert receives nothing
    first = sum(counts[:rank])
    x, lg = np.ascontiguousarray(x_all[first:first + T]), np.ascontiguousarray(lg_all[first:first + T])
    full = synth.moe_weights(spec, 24)
    per = E // world
    shard = dict(full)
    for name in ("gate", "up", "down"):
        rows = full[name].shape[0] // E
        shard[name] = np.ascontiguousarray(full[name][rank * per * rows:(rank + 1) * per * rows])
    be = B.Backend(device=f"cuda:{rank}".encode())
    assert be.rc == B.OK, be.message()
    arena = B.ResidentArena(be, shard)
    local_spec = synth.MoELayerSpec(H, per, k, I, down_qtype=synth.Q2_K)
    job = B.moe_job(arena, local_spec, router=False)                    # views of the shard ...
    job._plan.routed_experts = E                                        # ... under the plan of the whole layer
    ident = (C.c_ubyte * 128)()
    if rank == 0:
        assert B._lib.yvex_moe_ep_unique_id(ident, C.byref(be.err)) == B.OK, be.message()
        with open(id_path + ".tmp", "wb") as f:
            f.write(bytes(ident))
        os.replace(id_path + ".tmp", id_path)
    else:
        until = time.time() + 60
        while not os.path.exists(id_path) and time.time() < until:
            time.sleep(0.05)
        C.memmove(ident, open(id_path, "rb").read(), 128)
    ep = B.vp()
    assert B._lib.yvex_moe_ep_open(C.byref(ep), be.h, ident, world, rank, 3000 if absent_step else 60000, C.byref(be.err)) == B.OK, be.message()
    need = B.ull()
    assert B._lib.yvex_moe_ep_workspace_required(job.layer, max(counts), world, C.byref(need), C.byref(be.err)) == B.OK
    rc, ws, _ = be.tensor(need.value)
    assert rc == B.OK and B._lib.yvex_backend_workspace_attach(be.h, ws, C.byref(be.err)) == B.OK
    out = np.zeros((T, H), np.float32)
    sel = np.zeros((T, k), np.uint64)
    wts = np.zeros((T, k), np.float32)
    batch = B.row_batch(T, H, host_rows=x.ctypes.data_as(B.vp), router_logits=lg.ctypes.data_as(B.vp))
    o = B.row_output(out.ctypes.data_as(B.vp), out.size, sel.ctypes.data_as(B.vp), wts.ctypes.data_as(B.vp), sel.size)
    codes, same = [], True
    st = lib.Status(torch.device("cuda", rank))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.device("cuda", rank))
    want, sel0, _ = lib.moe_layer(lib.geometry_of(spec), lib.weights_of({n: dev(v.reshape(-1)) for n, v in full.items()}), dev(x), st,
                                  logits=dev(lg), wide=True)
    torch.cuda.synchronize()
    for step in range(3):
        if absent_step is not None and step == absent_step and rank == 1:
            time.sleep(8.0)                                             # stays alive, idle, until the peer's deadline has passed
            break                                                       # and leaves between steps, nothing of its own in flight
        res = B.RowBatchResult()
        rc = B._lib.yvex_moe_ep_execute_rows(ep, C.byref(job), C.byref(batch), C.byref(o), C.byref(res), C.byref(be.err))
        codes.append(rc)
        if rc == B.OK:
            same = same and (out.view(np.uint32) == want.cpu().numpy().view(np.uint32)).all() and (sel == sel0.cpu().numpy()).all()
            same = same and res.completed == 1 and res.row_expert_pairs == T * k
    B._lib.yvex_moe_ep_close(C.byref(ep), C.byref(be.err))
    ret[rank] = (codes, bool(same), st.read())
    be.close()


def _run_c_ranks(absent_step, tmp_path):
    import torch
    import torch.multiprocessing as mp
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    ret = mp.Manager().dict()
    mp.spawn(_c_worker, args=(2, str(tmp_path / "nccl_id"), absent_step, ret), nprocs=2, join=True)
    return dict(ret)


def test_c11_orchestration_over_nccl_matches_the_single_device_layer(tmp_path):
    """yvex_moe_ep_execute_rows on two ranks with different row counts: every rank's rows equal the single-device wide
    layer's bit for bit, three steps in a row."""
    from yvex_b200 import backend as B
    assert _run_c_ranks(None, tmp_path) == {0: ([B.OK] * 3, True, 0), 1: ([B.OK] * 3, True, 0)}


def test_c11_orchestration_times_out_when_a_peer_is_absent(tmp_path):
    """Rank 1 stops taking part after the first step (between steps, with nothing of its own in flight): rank 0's next
    call ends with YVEX_ERR_TIMEOUT once the deadline has passed, the call after it with YVEX_ERR_STATE."""
    from yvex_b200 import backend as B
    got = _run_c_ranks(1, tmp_path)
    assert got[1] == ([B.OK], True, 0)
    assert got[0] == ([B.OK, B.TIMEOUT, B.STATE], True, 0)
