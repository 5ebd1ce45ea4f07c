"""Expert-parallel MoE layer across the GPUs of one box (one process per GPU).

Routed experts are sharded in contiguous blocks (expert e lives on rank e // (E / world)); the
router, the shared expert and the tokens' home ranks are replicated / sharded by token. One
layer is: route locally -> all-to-all-v dispatch of the bf16-exact token rows (as fp16) with
their (local expert id, route weight) -> grouped dequant GEMMs on the receiving rank -> all-to-all-v
of the per-pair bf16 rows back -> the home rank sums its k rows in rank order (f32) + its shared
row -> bf16. Because per-pair rows (not partial sums) travel, the result is bit-identical to the
single-device layer. The reference has no multi-device path at all (single process, one GPU);
per-pair semantics are those of its CPU path (src/graph/moe.c:587-622, src/runtime/moe.c:619-632).

Collectives go through torch.distributed (NCCL over NVLink on GPUs, gloo in the CPU tests); the
compute calls go through the C-ABI of libyvex_b200.so (`DeviceOps`). The host logic takes the ops
as a parameter so the world_size-2 gloo tests can drive it without a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DeviceOps:
    """The layer's compute steps on the current CUDA device, via the C-ABI."""

    def __init__(self, geom_full, geom_local, weights_local, status):
        from . import lib
        self.lib, self.geom_full, self.geom_local = lib, geom_full, geom_local
        self.weights, self.status = weights_local, status

    def ingress(self, x):
        return x.to(torch.bfloat16).to(torch.float16)          # RNE to bf16, then its fp16 image

    def route(self, x, logits):
        sel, wts, _ = self.lib.moe_route(self.geom_full, self.weights, self.status,
                                         rows_f32=None if logits is not None else x.to(torch.bfloat16).float(),
                                         logits=logits)
        return sel, wts

    def dispatch(self, xh, sel, wts, per_rank, world):
        """Send order, send rows, metadata, inverse index and split sizes in one library call."""
        return self.lib.ep_dispatch(xh, sel.contiguous(), wts.contiguous(), per_rank, world, self.status)

    def expert_rows(self, rows_h, ids, wts):
        return self.lib.moe_expert_rows(self.geom_local, self.weights, rows_h, ids, wts, self.status)

    def combine(self, y_routed, y_shared, topk, routed_rows=None):
        return self.lib.moe_combine(y_routed, y_shared, topk, self.status, routed_rows=routed_rows)


class ExpertParallelLayer:
    def __init__(self, experts, topk, ops, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.experts, self.topk, self.per_rank, self.ops = experts, topk, experts // self.world, ops

    def _all_to_all(self, send, send_counts, recv_counts, recv=None):
        if recv is None:
            recv = send.new_empty((sum(recv_counts),) + tuple(send.shape[1:]))
        if self.world == 1:
            recv.copy_(send)
        else:
            dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        return recv

    def forward(self, x, logits=None):
        """x [t, hidden] f32 (this rank's tokens), logits [t, experts] or None -> out [t, hidden] f32."""
        k, ops = self.topk, self.ops
        t = x.shape[0]
        xh = ops.ingress(x)
        sel, wts = ops.route(x, logits)                                   # [t, k] int32 / f32
        fused = getattr(ops, "dispatch", None)
        if fused is not None:                                             # one call instead of the tensor ops below
            send_rows, meta, inverse, send_counts_t = fused(xh, sel, wts, self.per_rank, self.world)
        else:
            dest = (sel // self.per_rank).reshape(-1).to(torch.int64)
            order = torch.argsort(dest, stable=True)                      # pairs grouped by destination rank
            send_counts_t = torch.bincount(dest, minlength=self.world)
        recv_counts_t = torch.empty_like(send_counts_t)
        if self.world == 1:
            recv_counts_t.copy_(send_counts_t)
        else:
            dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        # the send buffers do not depend on the counts: enqueue them before the host reads the counts,
        # so the device has work while the host waits
        if fused is None:
            send_rows = xh.index_select(0, torch.div(order, k, rounding_mode="floor"))
            meta = torch.stack(((sel % self.per_rank).reshape(-1).to(torch.int32),
                                wts.reshape(-1).contiguous().view(torch.int32)), dim=1).index_select(0, order).contiguous()
            inverse = torch.empty(order.numel(), dtype=torch.int32, device=order.device)
            inverse[order] = torch.arange(order.numel(), dtype=torch.int32, device=order.device)
        send_counts, recv_counts = send_counts_t.tolist(), recv_counts_t.tolist()
        # One pair list per rank: the received routed pairs, then this rank's own tokens for the (replicated)
        # shared expert as pairs of expert -1 with weight 1 - one set of grouped GEMM launches instead of two.
        # The routed rows are received straight into the head of the list's row buffer.
        n_recv = sum(recv_counts)
        rows_all = xh.new_empty((n_recv + t, xh.shape[1]))
        self._all_to_all(send_rows, send_counts, recv_counts, recv=rows_all[:n_recv])
        rows_all[n_recv:].copy_(xh)
        recv_meta = self._all_to_all(meta, send_counts, recv_counts)
        ids = torch.cat((recv_meta[:, 0], torch.full((t,), -1, dtype=torch.int32, device=x.device)))
        pair_w = torch.cat((recv_meta[:, 1].contiguous().view(torch.float32), torch.ones(t, dtype=torch.float32, device=x.device)))
        y_all = ops.expert_rows(rows_all, ids, pair_w)
        y_recv, y_shared = y_all[:n_recv], y_all[n_recv:]

        y_back = self._all_to_all(y_recv, recv_counts, send_counts)      # reverse direction, same splits
        # pair (token, rank) sits at row inverse[...] of y_back: the combine reads through that index
        return ops.combine(y_back, y_shared, k, routed_rows=inverse), sel, wts
