"""Expert-parallel MoE layer across the GPUs of one box (one process per GPU).

Routed experts are sharded in contiguous blocks (expert e lives on rank e // (E / world)); the
router, the shared expert and the tokens' home ranks are replicated / sharded by token. One
layer is: route locally -> every pair's bf16-exact token row (as fp16, with a 16-byte trailer naming
its local expert, route weight, home pair and home rank) reaches its expert's rank -> grouped dequant
GEMMs there -> the per-pair bf16 rows reach their home rank -> it sums its k rows in rank order
(f32) + its shared row -> bf16. Because per-pair rows (not partial sums) travel, the result is
bit-identical to the single-device layer. The reference has no multi-device path at all (single
process, one GPU); per-pair semantics are those of its CPU path (src/graph/moe.c:587-622,
src/runtime/moe.c:619-632).

How rows travel. On GPUs whose memory can be mapped into each other (symmetric memory), both
movements are fused into the kernels beside them and use plain peer stores over NVLink: the dispatch
kernel writes every record straight into the expert rank's receive buffer (offsets from an
all-gather of the counts), and the down GEMM's epilogue writes every result row straight into its
home rank's buffer; two one-element all-reduces serve as barriers and no row goes through a
collective (`DeviceOps(peer_dispatch=True, peer_return=True)`, the default). Either movement, or
both, can instead be an all-to-all-v (`False`, or no peer access). The receive buffers hold the worst
routing (every pair of every rank), so the push starts as soon as the counts are on the device, on a
stream of its own beside the shared expert's GEMMs.
The exchange-based step can be pipelined: with `segments` > 1 and `DeviceOps(overlap=True)` a rank's
local experts are cut into equal ranges whose rows travel on a communication stream while the GEMMs of
the previous range run (cutting by EXPERT keeps every expert's rows together, so tiles stay full).

Order of a step. The shared expert needs no exchange: its GEMMs are enqueued first and cover the one
host read of the counts. All per-step buffers are allocated once and reused.

Collectives go through torch.distributed (NCCL on GPUs, gloo in the CPU tests); the compute calls go
through the C-ABI of libyvex_b200.so (`DeviceOps`). The host logic takes the ops as a parameter so the
world_size-2 gloo tests can drive it without a GPU (`TorchOps` is the plain tensor formulation of
every step; `DeviceOps` replaces each with a library call).
"""
from __future__ import annotations

import contextlib
import os

import torch
import torch.distributed as dist

TRAILER_BYTES = 16
ERR_TIMEOUT, ERR_BACKEND = -11, -6                    # yvex_status values (include/yvex_b200_backend.h)


class ExchangeError(RuntimeError):
    """A collective of the layer failed on the host side: a peer left or stalled past the process group's
    timeout (code ERR_TIMEOUT), or the communication backend reported another error (ERR_BACKEND). Nothing
    was enqueued behind the failed exchange; the device is not waiting for anyone."""

    def __init__(self, code, what):
        super().__init__(f"expert-parallel exchange failed ({'timeout' if code == ERR_TIMEOUT else 'backend'}): {what}")
        self.code = code


class TorchOps:
    """Every step of the layer as plain tensor operations: the specification of `DeviceOps`, and
    what the CPU tests run (subclasses supply ingress / route / expert_rows / combine)."""

    streams = None                                    # no side stream: steps run in program order
    buf = {}                                          # step buffers (none: every step allocates what it returns)

    def prepare(self, tokens, hidden, topk, world, segments):
        pass

    def pack(self, rows_h, ids, wts, home_pairs):
        """rows_h [n, H] fp16 + trailer {int32 id, f32 weight, int32 home pair, 0} -> uint8 [n, 2H + 16]."""
        n = rows_h.shape[0]
        trailer = torch.zeros((n, 4), dtype=torch.int32, device=rows_h.device)
        trailer[:, 0] = ids
        trailer[:, 1] = wts.contiguous().view(torch.int32)
        trailer[:, 2] = home_pairs
        return torch.cat((rows_h.contiguous().view(torch.uint8).reshape(n, -1), trailer.view(torch.uint8).reshape(n, -1)), dim=1)

    def unpack(self, payload, hidden):
        n = payload.shape[0]
        rows = payload[:, :2 * hidden].contiguous().view(torch.float16).reshape(n, hidden)
        trailer = payload[:, 2 * hidden:].contiguous().view(torch.int32).reshape(n, 4)
        return rows, trailer[:, 0].contiguous(), trailer[:, 1].contiguous().view(torch.float32)

    def dispatch(self, xh, sel, wts, per_rank, world, segments):
        """-> (payload [T*k, 2H+16] uint8 in send order, inverse [T*k] int32, counts [segments*world] int64).
        Send order: by (segment of the local expert, destination rank), stable in the pair index."""
        k = sel.shape[1]
        flat = sel.reshape(-1).to(torch.int64)
        dest, local = flat // per_rank, flat % per_rank
        bins = (local * segments // per_rank) * world + dest
        order = torch.argsort(bins, stable=True)
        counts = torch.bincount(bins, minlength=world * segments)
        rows = xh.index_select(0, torch.div(order, k, rounding_mode="floor"))
        payload = self.pack(rows, local[order].to(torch.int32), wts.reshape(-1)[order], order.to(torch.int32))
        inverse = torch.empty(order.numel(), dtype=torch.int32, device=order.device)
        inverse[order] = torch.arange(order.numel(), dtype=torch.int32, device=order.device)
        return payload, inverse, counts

    def expert_rows_payload(self, payload, hidden, out=None):
        rows, ids, wts = self.unpack(payload, hidden)
        y = self.expert_rows(rows, ids, wts)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def shared_rows(self, xh):
        t = xh.shape[0]
        return self.expert_rows(xh, torch.full((t,), -1, dtype=torch.int32, device=xh.device),
                                torch.ones(t, dtype=torch.float32, device=xh.device))


class DeviceOps(TorchOps):
    """The layer's compute steps on the current CUDA device, via the C-ABI. Owns the step buffers."""

    def __init__(self, geom_full, geom_local, weights_local, status, overlap=False, peer_return=True, peer_dispatch=True):
        from . import lib
        self.lib, self.geom_full, self.geom_local = lib, geom_full, geom_local
        self.weights, self.status = weights_local, status
        self.overlap = overlap
        self.peer_return = peer_return          # results go home by peer stores from the down GEMM's epilogue
        self.home, self.home_flip = None, 0
        self.peer_dispatch = peer_dispatch      # rows reach their expert's rank by peer stores from the dispatch kernel
        self.inbox = None
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.cta_limit = 140                   # CTAs of the persistent GEMM while an exchange runs beside it
        self.streams = None
        self.buf = {}

    def prepare(self, tokens, hidden, topk, world, segments):
        """Allocates (once per shape) everything a step needs: send / receive records, returned rows,
        pair-list workspaces. Receive-side capacities start at twice the balanced load and grow on demand."""
        key = (tokens, hidden, topk, world, segments)
        if self.buf.get("key") == key:
            return
        dev = torch.device("cuda", torch.cuda.current_device())
        pairs, pitch = tokens * topk, 2 * hidden + TRAILER_BYTES
        b = {"key": key, "pitch": pitch}
        b["payload"] = torch.empty((pairs, pitch), dtype=torch.uint8, device=dev)
        b["inverse"] = torch.empty(pairs, dtype=torch.int32, device=dev)
        b["counts"] = torch.empty(world * segments, dtype=torch.int64, device=dev)
        b["counts_in"] = torch.empty(world * segments, dtype=torch.int64, device=dev)
        b["counts_host"] = torch.empty(2 * world * segments, dtype=torch.int64).pin_memory()
        b["plan_ws"] = torch.empty(int(self.lib.lib.yvex_b200_ep_dispatch_workspace_bytes(pairs, world * segments)),
                                   dtype=torch.uint8, device=dev)
        b["y_back"] = torch.empty((pairs, hidden), dtype=torch.bfloat16, device=dev)
        b["y_shared"] = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        b["shared_ids"] = torch.full((tokens,), -1, dtype=torch.int32, device=dev)
        b["shared_w"] = torch.ones(tokens, dtype=torch.float32, device=dev)
        b["out"] = torch.empty((tokens, hidden), dtype=torch.float32, device=dev)
        b["shared_ws"] = torch.empty(int(self.lib.lib.yvex_b200_moe_expert_rows_workspace_bytes(self.geom_local, tokens)),
                                     dtype=torch.uint8, device=dev)
        b["seg"] = [None] * segments
        self.buf = b
        self.home = self._home_buffers(pairs, hidden, dev) if self.peer_return and world > 1 else None
        self.inbox = self._inbox(pairs, pitch, world, segments, dev) if self.peer_dispatch and world > 1 else None
        if self.overlap and world > 1 and self.streams is None:
            self.streams = (torch.cuda.Stream(device=dev, priority=-1),)          # communication stream, high priority
            # the persistent GEMM leaves a few SMs to the exchange kernels that run beside it
            self.lib.lib.yvex_b200_moe_wide_set_cta_limit(self.cta_limit)

    def _home_buffers(self, pairs, hidden, dev):
        """Two buffers [pairs, hidden] bf16 that every peer can store into (symmetric memory; the rendezvous is a
        collective, every rank reaches it in its first step), used alternately so that a fast peer's next step
        never lands in rows this rank is still summing. None when peer access cannot be set up: the rows then
        come back by an exchange."""
        try:
            import torch.distributed._symmetric_memory as symm
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")       # plain peer stores only
            out = []
            for _ in range(2):
                t = symm.empty(pairs * hidden, dtype=torch.bfloat16, device=dev)
                hdl = symm.rendezvous(t, dist.group.WORLD)
                bases = torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64, device=dev)
                out.append((t.view(pairs, hidden), bases, hdl))
            self.home_flag = torch.zeros(1, dtype=torch.float32, device=dev)
            return out
        except Exception as exc:                                                 # no peer access on this box
            import warnings
            warnings.warn(f"peer return disabled: {type(exc).__name__}: {exc}")
            return None

    def _inbox(self, pairs, pitch, world, segments, dev):
        """Receive buffers every peer can store into, one per segment, each large enough for the worst routing
        (every pair of every rank: the push then needs no decision from the host and can start as soon as the
        counts are known on the device), with their pair-list workspaces, the per-bin addresses and the
        all-gathered counts. None when peer access cannot be set up."""
        try:
            import torch.distributed._symmetric_memory as symm
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            cap = world * pairs
            # with both peer paths, one range and gate/up weights without a min term the rows can be pushed straight
            # into expert-major order (one bin per (local expert, destination)): the receiver then sorts nothing
            per = int(self.geom_local.experts)
            ordered = segments == 1 and self.home is not None and int(self.geom_local.gate_qtype) not in (10, 12) and per * world <= 1024
            bins = world * (per if ordered else segments)
            bases = torch.empty(bins, dtype=torch.int64)
            recv = []
            for s in range(segments):
                t = symm.empty(cap * pitch, dtype=torch.uint8, device=dev)
                hdl = symm.rendezvous(t, dist.group.WORLD)
                for b in range(bins) if ordered else range(s * world, (s + 1) * world):
                    bases[b] = int(hdl.buffer_ptrs[b % world])
                recv.append((t.view(cap, pitch), hdl))
            return {"cap": cap, "recv": recv, "bases": bases.to(dev), "ordered": ordered, "bin_segments": per if ordered else segments,
                    "counts": torch.empty(bins, dtype=torch.int64, device=dev),
                    "plan_ws": torch.empty(int(self.lib.lib.yvex_b200_ep_dispatch_workspace_bytes(pairs, bins)), dtype=torch.uint8,
                                           device=dev),
                    "ws": [torch.empty(int(self.lib.lib.yvex_b200_moe_expert_rows_workspace_bytes(self.geom_local, cap)),
                                       dtype=torch.uint8, device=dev) for _ in range(segments)],
                    "y": [None] * segments,
                    "counts_all": torch.empty(world * bins, dtype=torch.int64, device=dev),
                    "counts_all_host": torch.empty(world * bins, dtype=torch.int64).pin_memory(),
                    "flag": torch.zeros(1, dtype=torch.float32, device=dev),
                    "stream": torch.cuda.Stream(device=dev, priority=-1)}
        except Exception as exc:
            import warnings
            warnings.warn(f"peer dispatch disabled: {type(exc).__name__}: {exc}")
            return None

    def plan(self, sel, per_rank, world, segments):
        box = self.inbox
        return self.lib.ep_dispatch_plan(sel.contiguous(), per_rank, world, box["bin_segments"], self.status, self.buf["inverse"],
                                         box["counts"], box["plan_ws"])

    def push(self, xh, sel, wts, per_rank, world, segments):
        box = self.inbox
        self.lib.ep_dispatch_push(xh, sel.contiguous(), wts.contiguous(), per_rank, world, self.rank, box["bin_segments"],
                                  box["counts_all"], box["bases"], box["cap"], self.status, box["plan_ws"], expert_major=box["ordered"])

    def segment_buffers(self, seg, rows):
        """Receive records, result rows and pair-list workspace of one segment, grown when a step needs more."""
        b = self.buf
        cur = b["seg"][seg]
        if cur is None or cur["cap"] < rows:
            cap = max(rows + rows // 4, 2 * b["key"][0] * b["key"][2] // b["key"][4], 1024)
            dev = b["payload"].device
            cur = {"cap": cap,
                   "recv": torch.empty((cap, b["pitch"]), dtype=torch.uint8, device=dev),
                   "y": torch.empty((cap, b["key"][1]), dtype=torch.bfloat16, device=dev),
                   "ws": torch.empty(int(self.lib.lib.yvex_b200_moe_expert_rows_workspace_bytes(self.geom_local, cap)),
                                     dtype=torch.uint8, device=dev)}
            b["seg"][seg] = cur
        return cur

    def ingress(self, x):
        return x.to(torch.bfloat16).to(torch.float16)          # RNE to bf16, then its fp16 image

    def route(self, x, logits):
        sel, wts, _ = self.lib.moe_route(self.geom_full, self.weights, self.status,
                                         rows_f32=None if logits is not None else x.to(torch.bfloat16).float(),
                                         logits=logits)
        return sel, wts

    def dispatch(self, xh, sel, wts, per_rank, world, segments):
        b = self.buf
        self.lib.ep_dispatch_payload(xh, sel.contiguous(), wts.contiguous(), per_rank, world, segments, self.status,
                                     b["payload"], b["inverse"], b["counts"], b["plan_ws"], rank=self.rank)
        return b["payload"], b["inverse"], b["counts"]

    def expert_rows(self, rows_h, ids, wts, workspace=None, out=None):
        return self.lib.moe_expert_rows(self.geom_local, self.weights, rows_h, ids, wts, self.status, workspace=workspace, out=out)

    def shared_rows(self, xh):
        b = self.buf
        return self.expert_rows(xh, b["shared_ids"], b["shared_w"], workspace=b["shared_ws"], out=b["y_shared"])

    def expert_rows_payload(self, payload, hidden, out=None, workspace=None, home=None, ordered=None):
        if ordered is not None:                # the records already stand in expert-major order: (counts_all, world)
            self.lib.moe_expert_rows_sorted(self.geom_local, self.weights, payload, ordered[0], ordered[1], self.rank, home[1],
                                            home[0].shape[0], self.status, workspace)
            return None
        if home is not None:                   # (rows [pairs, hidden], bases): store every row at its home rank
            self.lib.moe_expert_rows_scatter(self.geom_local, self.weights, payload, home[1], home[0].shape[0], self.status,
                                             workspace=workspace)
            return None
        return self.lib.moe_expert_rows_payload(self.geom_local, self.weights, payload, self.status, workspace=workspace, out=out)

    def combine(self, y_routed, y_shared, topk, routed_rows=None):
        return self.lib.moe_combine(y_routed, y_shared, topk, self.status, routed_rows=routed_rows, out=self.buf.get("out"))


class ExpertParallelLayer:
    def __init__(self, experts, topk, ops, group=None, segments=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.experts, self.topk, self.per_rank, self.ops = experts, topk, experts // self.world, ops
        if segments is None:
            segments = 1
        if self.per_rank % segments:
            raise ValueError("segments must divide the experts of a rank")
        self.segments = segments
        self.timings = None                    # when a dict: host-side cuda events of the last step's phases

    def _collective(self, recv, send, recv_counts=None, send_counts=None):
        """all_to_all_single with the failure of a peer turned into ExchangeError: the process group's
        timeout bounds the wait on the host, so a rank that left or stalled cannot hang this one."""
        try:
            dist.all_to_all_single(recv, send, recv_counts, send_counts, group=self.group)
        except Exception as exc:                                            # DistBackendError, RuntimeError("Timed out ...")
            text = str(exc)
            late = any(w in text.lower() for w in ("timed out", "timeout", "connection closed", "connection reset", "peer"))
            raise ExchangeError(ERR_TIMEOUT if late else ERR_BACKEND, text.splitlines()[0] if text else type(exc).__name__) from exc

    def _all_to_all(self, recv, send, recv_counts, send_counts):
        if self.world == 1:
            recv.copy_(send)
        else:
            self._collective(recv, send, recv_counts, send_counts)

    def forward(self, x, logits=None):
        """x [t, hidden] f32 (this rank's tokens), logits [t, experts] or None -> (out [t, hidden] f32, sel, wts)."""
        k, ops, W, S = self.topk, self.ops, self.world, self.segments
        t, hidden = x.shape
        ops.prepare(t, hidden, k, W, S)
        side = ops.streams[0] if ops.streams else None
        on_side = (lambda: torch.cuda.stream(side)) if side is not None else contextlib.nullcontext
        main = torch.cuda.current_stream() if side is not None else None

        def after(stream_from, stream_to):
            if side is not None:
                ev = torch.cuda.Event()
                ev.record(stream_from)
                stream_to.wait_event(ev)

        marks = []

        def mark(name):
            """Phase boundary on the compute stream (only while self.timings is a dict)."""
            if self.timings is not None and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        xh = ops.ingress(x)
        sel, wts = ops.route(x, logits)                                   # [t, k] int32 / f32
        if W > 1 and getattr(ops, "inbox", None):
            out = self._forward_pushed(x, xh, sel, wts, mark)
            if marks:
                self.timings["marks"] = marks
            return out, sel, wts
        payload, inverse, counts = ops.dispatch(xh, sel, wts, self.per_rank, W, S)
        mark("route_plan")
        # split sizes: one tiny exchange and the step's only host read
        after(main, side)
        host = ops.buf.get("counts_host")
        with on_side():
            counts_in = ops.buf.get("counts_in")
            if counts_in is None:
                counts_in = torch.empty_like(counts)
            if W == 1:
                counts_in.copy_(counts)
            else:
                self._exchange_counts(counts_in, counts)
            if host is not None:
                host[:W * S].copy_(counts, non_blocking=True)
                host[W * S:].copy_(counts_in, non_blocking=True)
                done = torch.cuda.Event()
                done.record()
        # the shared expert needs nothing from other ranks: its GEMMs cover the host read and the first dispatch
        y_shared = ops.shared_rows(xh)
        mark("shared_expert")
        if host is not None:
            done.synchronize()
            send_c, recv_c = host[:W * S].view(S, W).tolist(), host[W * S:].view(S, W).tolist()
        else:
            send_c, recv_c = counts.view(S, W).tolist(), counts_in.view(S, W).tolist()

        hidden_pitch = payload.shape[1]
        y_back = ops.buf.get("y_back")
        if y_back is None:
            y_back = torch.empty((t * k, hidden), dtype=torch.bfloat16, device=x.device)
        home = None
        if W > 1 and getattr(ops, "home", None):
            ops.home_flip ^= 1
            home = ops.home[ops.home_flip]
        send_off, seg_bufs = 0, []
        # dispatch of every segment, in order, on the communication stream
        with on_side():
            for s in range(S):
                n_send, n_recv = sum(send_c[s]), sum(recv_c[s])
                if hasattr(ops, "segment_buffers"):
                    sb = ops.segment_buffers(s, n_recv)
                    recv, y_seg, ws = sb["recv"][:n_recv], sb["y"][:n_recv], sb["ws"]
                else:
                    recv, y_seg, ws = payload.new_empty((n_recv, hidden_pitch)), None, None
                self._all_to_all(recv, payload[send_off:send_off + n_send], recv_c[s], send_c[s])
                ev = None
                if side is not None:
                    ev = torch.cuda.Event()
                    ev.record(side)
                seg_bufs.append((recv, y_seg, ws, ev, send_off, n_send, n_recv))
                send_off += n_send
        # GEMMs of segment s on the compute stream, its results leave while segment s + 1 computes
        back_events = []
        for s, (recv, y_seg, ws, ev, off, n_send, n_recv) in enumerate(seg_bufs):
            if ev is not None:
                main.wait_event(ev)
            if home is not None:
                if n_recv:
                    ops.expert_rows_payload(recv, hidden, workspace=ws, home=home)
                mark(f"segment{s}_wait_and_gemm")
                continue
            if n_recv:
                y_seg = ops.expert_rows_payload(recv, hidden, out=y_seg, workspace=ws) if ws is not None \
                    else ops.expert_rows_payload(recv, hidden)
            else:
                y_seg = y_back.new_empty((0, hidden))
            mark(f"segment{s}_wait_and_gemm")
            after(main, side)
            with on_side():
                self._all_to_all(y_back[off:off + n_send], y_seg, send_c[s], recv_c[s])      # reverse direction, same splits
                if side is not None:
                    e2 = torch.cuda.Event()
                    e2.record(side)
                    back_events.append(e2)
        for e2 in back_events:
            main.wait_event(e2)
        if home is not None:
            # every rank's GEMMs have stored their rows once this (tiny) collective has passed on every stream
            try:
                dist.all_reduce(ops.home_flag, group=self.group)
            except Exception as exc:
                raise ExchangeError(ERR_TIMEOUT, str(exc).splitlines()[0] if str(exc) else type(exc).__name__) from exc
            out = ops.combine(home[0], y_shared, k)                             # rows already sit in pair order
        else:
            # pair (token, rank) sits at row inverse[...] of y_back: the combine reads through that index
            out = ops.combine(y_back, y_shared, k, routed_rows=inverse)
        mark("return_wait_and_combine")
        if marks:
            self.timings["marks"] = marks
            self.timings["pairs_received"] = [b[6] for b in seg_bufs]
        return out, sel, wts

    def _forward_pushed(self, x, xh, sel, wts, mark):
        """The step without a bulk collective: the dispatch kernel stores every row straight into its expert's rank
        (symmetric receive buffers), the down GEMM's epilogue stores every result straight into its home rank. What
        remains of NCCL is one all-gather of the counts and two one-element all-reduces used as barriers.
        """
        k, ops, W, S = self.topk, self.ops, self.world, self.segments
        t, hidden = x.shape
        box, bins = ops.inbox, W * S
        inverse, counts = ops.plan(sel, self.per_rank, W, S)
        try:
            dist.all_gather_into_tensor(box["counts_all"], counts, group=self.group)
        except Exception as exc:
            raise ExchangeError(ERR_TIMEOUT, str(exc).splitlines()[0] if str(exc) else type(exc).__name__) from exc
        box["counts_all_host"].copy_(box["counts_all"], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        mark("route_plan")
        # the rows leave on a stream of their own, beside the shared expert's GEMMs, which also cover the host's
        # read of the counts (the receive buffers hold the worst case, so nothing has to be decided first)
        main, side = torch.cuda.current_stream(), box["stream"]
        side.wait_event(done)
        with torch.cuda.stream(side):
            ops.push(xh, sel, wts, self.per_rank, W, S)
            pushed = torch.cuda.Event()
            pushed.record()
        y_shared = ops.shared_rows(xh)
        mark("shared_expert")
        done.synchronize()
        table = box["counts_all_host"].view(W, box["bin_segments"], W)   # [source][segment or local expert][destination]
        if box["ordered"]:
            n_recv = [int(table[:, :, self.rank].sum())]
        else:
            n_recv = [int(table[:, s, self.rank].sum()) for s in range(S)]
        main.wait_event(pushed)
        self._barrier(box["flag"])                                        # every rank's rows have landed
        home = None
        if getattr(ops, "home", None):
            ops.home_flip ^= 1
            home = ops.home[ops.home_flip]
        y_back = ops.buf.get("y_back")
        for s in range(S):
            recv = box["recv"][s][0][:n_recv[s]]
            if box["ordered"]:
                if n_recv[s]:
                    ops.expert_rows_payload(recv, hidden, workspace=box["ws"][s], home=home, ordered=(box["counts_all"], W))
            elif home is not None:
                if n_recv[s]:
                    ops.expert_rows_payload(recv, hidden, workspace=box["ws"][s], home=home)
            else:
                if box["y"][s] is None:
                    box["y"][s] = torch.empty((box["cap"], hidden), dtype=torch.bfloat16, device=x.device)
                y_seg = box["y"][s][:n_recv[s]]
                if n_recv[s]:
                    ops.expert_rows_payload(recv, hidden, out=y_seg, workspace=box["ws"][s])
                off = int(table[self.rank, :s, :].sum())
                n_send = int(table[self.rank, s, :].sum())
                self._all_to_all(y_back[off:off + n_send], y_seg, table[self.rank, s, :].tolist(), table[:, s, self.rank].tolist())
            mark(f"segment{s}_wait_and_gemm")
        if home is not None:
            self._barrier(ops.home_flag)                                  # every rank's GEMMs have stored their rows
            out = ops.combine(home[0], y_shared, k)
        else:
            out = ops.combine(y_back, y_shared, k, routed_rows=inverse)
        mark("return_wait_and_combine")
        if self.timings is not None:
            self.timings["pairs_received"] = n_recv
        return out

    def _barrier(self, flag):
        try:
            dist.all_reduce(flag, group=self.group)
        except Exception as exc:
            raise ExchangeError(ERR_TIMEOUT, str(exc).splitlines()[0] if str(exc) else type(exc).__name__) from exc

    def _exchange_counts(self, counts_in, counts):
        """counts is [segments][world]; rank r must receive entry [s][me] of every rank r' as its [s][r']."""
        S, W = self.segments, self.world
        send = counts.view(S, W).t().contiguous().view(-1)                 # [world][segments]
        recv = torch.empty_like(send)
        self._collective(recv, send)
        counts_in.copy_(recv.view(W, S).t().contiguous().view(-1))
