"""Host-side logic of the expert-parallel layer (dispatch / combine permutations, split sizes,
expert sharding) on CPU: two gloo ranks with stand-in compute ops must reproduce the one-process
result bit for bit, including a rank that receives no pair at all."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from yvex_b200.ep import ExpertParallelLayer, TorchOps

E, K, H, T = 8, 3, 32, 10


class FakeOps(TorchOps):
    """Deterministic stand-ins: expert e multiplies a row by (e + 1) * weight, shared by 0.5."""

    def __init__(self, rank, per_rank):
        self.rank, self.per_rank = rank, per_rank

    def ingress(self, x):
        return x.to(torch.bfloat16).to(torch.float16)

    def route(self, x, logits):
        w, sel = torch.topk(logits, K, dim=1)
        return sel.to(torch.int32), torch.sigmoid(w).to(torch.float32)

    def expert_rows(self, rows_h, ids, wts):
        glob = torch.where(ids < 0, torch.full_like(ids, -1), ids + self.rank * self.per_rank)
        factor = torch.where(glob < 0, torch.full_like(wts, 0.5), (glob + 1).float() * wts)
        return (rows_h.float() * factor[:, None]).to(torch.bfloat16)

    def combine(self, y_routed, y_shared, topk, routed_rows=None):
        if routed_rows is not None:                      # rows named by index, as the device combine reads them
            y_routed = y_routed.index_select(0, routed_rows.to(torch.int64))
        acc = torch.zeros(y_shared.shape, dtype=torch.float32)
        yr = y_routed.float().reshape(-1, topk, y_shared.shape[1])
        for r in range(topk):
            acc = acc + yr[:, r]
        return (acc + y_shared.float()).to(torch.bfloat16).float()


def inputs(skew):
    g = torch.Generator().manual_seed(7)
    x = torch.randn((T, H), generator=g)
    logits = torch.randn((T, E), generator=g)
    if skew:
        logits[:, E // 2:] -= 100.0          # every pair goes to rank 0's experts
    return x, logits


def single(skew):
    x, logits = inputs(skew)
    out, sel, _ = ExpertParallelLayer(E, K, FakeOps(0, E)).forward(x, logits)
    return out, sel


def worker(rank, world, port, skew, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, logits = inputs(skew)
    lo, hi = rank * T // world, (rank + 1) * T // world
    layer = ExpertParallelLayer(E, K, FakeOps(rank, E // world))
    out, sel, _ = layer.forward(x[lo:hi].contiguous(), logits[lo:hi].contiguous())
    ret[rank] = (out, sel)
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("skew", [False, True])
def test_two_rank_layer_matches_single_process_bit_for_bit(skew):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(worker, args=(world, free_port(), skew, ret), nprocs=world, join=True)
    want, want_sel = single(skew)
    got = torch.cat([ret[r][0] for r in range(world)])
    got_sel = torch.cat([ret[r][1] for r in range(world)])
    assert torch.equal(got_sel, want_sel)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))



def worker_segments(rank, world, port, segments, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, logits = inputs(False)
    lo, hi = rank * T // world, (rank + 1) * T // world
    layer = ExpertParallelLayer(E, K, FakeOps(rank, E // world), segments=segments)
    ret[rank] = layer.forward(x[lo:hi].contiguous(), logits[lo:hi].contiguous())[0]
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("segments", [1, 2, 4])
def test_expert_segments_do_not_change_the_result(segments):
    """The exchange pipelined over 1, 2 or 4 ranges of each rank's experts gives the same bits."""
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(worker_segments, args=(world, free_port(), segments, ret), nprocs=world, join=True)
    want, _ = single(False)
    got = torch.cat([ret[r] for r in range(world)])
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


def worker_leaver(rank, world, port, mode, ret):
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    x, logits = inputs(False)
    lo, hi = rank * T // world, (rank + 1) * T // world
    layer = ExpertParallelLayer(E, K, FakeOps(rank, E // world))
    layer.forward(x[lo:hi].contiguous(), logits[lo:hi].contiguous())         # one good step first
    if rank == 1:
        # the failure is made on the host: this rank stalls past the deadline (or leaves) before the next exchange
        if mode == "stall":
            time.sleep(9)
        ret[rank] = "left"
        os._exit(0)
    from yvex_b200.ep import ERR_TIMEOUT, ExchangeError
    t0 = time.time()
    try:
        layer.forward(x[lo:hi].contiguous(), logits[lo:hi].contiguous())
        ret[rank] = "no error"
    except ExchangeError as exc:
        ret[rank] = ("timeout" if exc.code == ERR_TIMEOUT else f"code {exc.code}", time.time() - t0)
    os._exit(0)


@pytest.mark.parametrize("mode", ["stall", "leave"])
def test_a_rank_that_stalls_or_leaves_ends_the_exchange_with_a_timeout(mode):
    """The surviving rank gets an error from the host wrapper within the process group's deadline
    (never a hang): YVEX_ERR_TIMEOUT. The failing rank does its failing between steps, on the host."""
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(worker_leaver, args=(world, free_port(), mode, ret), nprocs=world, join=True)
    assert ret[1] == "left"
    kind, seconds = ret[0]
    assert kind == "timeout" and seconds < 30.0, ret[0]
