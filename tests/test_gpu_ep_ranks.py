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
