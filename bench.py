#!/usr/bin/env python
"""Benchmark of the quantized MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload c1|c2|c3|c4|c5]

One "step" is one pass of the MoE FFN layer over one batch of synthetic tokens. Prints ONE JSON
line (rank 0). `value` is device-timed throughput with inputs resident in HBM; `e2e` is the same
metric through the host-buffer call (pinned host rows in, host rows out, copies inside the timed
region). L2 is flushed between timed steps (a 256 MiB buffer is rewritten outside the timed
region). `--impl reference` times the reference's own CPU implementation of the same layer on
the host cores (the compiled reference when oracle/_ref is present, else the plain-C port).

At N > 1 the expert-parallel layer runs with the library's defaults; for experiments the environment can
turn its peer-memory paths off (YVEX_EP_PEER_DISPATCH=0, YVEX_EP_PEER_RETURN=0: rows then travel by NCCL
all-to-all-v) and shape the exchange-based pipeline (YVEX_EP_SEGMENTS, YVEX_EP_OVERLAP=1, YVEX_EP_CTAS);
YVEX_BENCH_C11=1 adds `c11_nccl_exchange`: the same step through the C11 orchestration over NCCL send/recv groups.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum, one capture per workload).
TRAFFIC = {"c1": 4389376, "c2": 22777600, "c4": 2160352104,
           "c3_gate_up_gemm": 361532672, "c3_down_gemm": 367173120,
           "c5_gate_up_gemm": 10006566912, "c5_down_gemm": 5925237760}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and clock-event reasons while the timed region runs: NVML queries from a
    thread every 10 ms (read-only), or `nvidia-smi -lms 100` when the NVML module is missing."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index
        self.stop, self.thread, self.handle, self.nvml = threading.Event(), None, None, None

    def _nvml_handle(self):
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml, self.handle = pynvml, handle
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            return True
        except Exception:
            return False

    def _poll(self):
        n, h = self.nvml, self.handle
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while True:
            try:
                mask = int(reasons_fn(h))
                self.rows.append([str(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)), str(self.max_mhz), "",
                                  *["Active" if mask & self.REASONS[k] else "Not Active"
                                    for k in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")]])
            except Exception:
                pass
            if self.stop.wait(0.01):
                return

    def __enter__(self):
        if self._nvml_handle():
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        self.stop.set()
        if self.handle is not None and self.thread:
            self.thread.join(timeout=2)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def oracle_backend(prefer_reference):
    """The CPU checker used as a timed baseline: the compiled reference when asked for and
    present, else this repository's plain-C port of it."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle_lib import Port, Ref
    if prefer_reference and Ref.available():
        return Ref(), "reference"
    return Port(), "port"


def cpu_layer_tokens_per_s(workload, tokens_per_step, steps, threads, prefer_reference=False):
    """Times the CPU path on `tokens_per_step` tokens per step with `threads` host threads."""
    backend, kind = oracle_backend(prefer_reference)
    w, router = workload.host_copy()
    L = backend.layer(workload.spec, w, router=router, allow_q4k=True)
    x, logits = workload.tokens(tokens_per_step)
    x = x.cpu().numpy()
    logits = None if logits is None else logits.cpu().numpy()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        rc, _, _, _ = backend.moe_tokens(L, x, logits=logits, threads=threads)
        times.append(time.perf_counter() - t0)
        if rc != 0:
            raise RuntimeError(f"CPU path refused with status {rc}")
    return tokens_per_step * len(times) / sum(times), kind, sum(times) / len(times)


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation on the host cores, rank 0 only."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from yvex_b200 import synth
    from yvex_b200.workloads import MoEWorkload
    cores = os.cpu_count() or 1
    if args.workload in ("c1", "c4"):
        return run_reference_kernel(args, cores)
    # The reference has no Q4_K decoder (src/gguf/quant_registry.c:67): when the compiled
    # reference is present its arm runs the Q2_K-down twin of the layer, the qtype its own MoE
    # path ships with; otherwise the port runs the layer exactly as configured.
    _, kind = oracle_backend(True)
    down = synth.Q2_K if kind == "reference" else synth.Q4_K
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    wl = MoEWorkload(args.workload, 1, device=dev, down_qtype=down)
    per_step = max(cores, 1)
    tps, kind, sec = cpu_layer_tokens_per_s(wl, per_step, max(1, min(args.steps, 3)), cores, True)
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
            "steps": min(args.steps, 3), "warmup": 0, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64-accum (reference CPU path)", "data": "synthetic",
            "config": {"workload": wl.name + ("-q2k-down" if down == synth.Q2_K else ""), **wl.cfg,
                       "tokens_per_step": per_step},
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": f"{per_step} tokens per step, one thread per token"},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_reference_kernel(args, cores):
    """Reference arm of the single-kernel workloads: the reference's CPU matvec (config 1) or CPU
    attention (config 4) on the host cores, on a bounded sample of the workload."""
    oracle, kind = oracle_backend(True)
    from yvex_b200 import synth
    rng = np.random.default_rng(synth.BASE_SEED)
    steps = max(1, min(args.steps, 3))
    if args.workload == "c1":
        rows = width = 4096
        w = synth.random_blocks(synth.IQ2_XXS, rows, width, 1)
        x = rng.standard_normal(width).astype(np.float32)
        algo = w.size + 4 * width + 4 * rows
        t0 = time.perf_counter()
        for _ in range(steps):
            oracle.matvec(synth.IQ2_XXS, w, rows, width, x, threads=cores)
        sec = (time.perf_counter() - t0) / steps
        metric, cfg, sample = "dequant_gemv_hbm_gbs", {"workload": "c1", "rows": rows, "width": width, "qtype": "IQ2_XXS"}, \
            "one 4096x4096 IQ2_XXS matvec per step, rows split over all cores"
    else:
        if not hasattr(oracle, "attention_gqa_decode"):
            # the compiled reference exposes its attention one f32 head at a time; the port runs the
            # same arithmetic (src/backend/cpu.c:319-411) over a bf16 GQA cache with threads over heads
            oracle, kind = oracle_backend(False)
        S, Hq, Hkv, D, ctx = 1, 32, 8, 128, 32768
        bits = lambda a: synth.bf16_bits(a).reshape(a.shape)
        q = bits(rng.standard_normal((S, Hq, D)).astype(np.float32))
        k = bits(rng.standard_normal((S, Hkv, ctx, D)).astype(np.float32))
        v = bits(rng.standard_normal((S, Hkv, ctx, D)).astype(np.float32))
        algo = 2 * k.size * 2 + q.size * 2 + S * Hq * D * 4
        t0 = time.perf_counter()
        for _ in range(steps):
            oracle.attention_gqa_decode(q, k, v, ctx - 1, D ** -0.5, threads=cores)
        sec = (time.perf_counter() - t0) / steps
        metric, cfg, sample = "attention_decode_hbm_gbs", {"workload": "c4", "sessions": S, "q_heads": Hq, "kv_heads": Hkv,
                                                          "head_dim": D, "context": ctx}, \
            "one of the 16 sessions per step, heads split over all cores"
    value = algo / sec / 1e9
    line = {"impl": "reference", "metric": metric, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": 0, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64-accum (reference CPU path)", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_native(args):
    import torch
    import torch.distributed as dist
    from yvex_b200 import lib, synth
    from yvex_b200.workloads import MoEWorkload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    peaks = measured_peaks()

    wl = MoEWorkload(args.workload, 1, device=dev)
    geom = lib.geometry_of(wl.spec)
    weights = lib.weights_of(wl.tensors)
    tokens = wl.cfg["tokens"]
    wide = tokens > 64
    pool = 16 if not wide else 1
    xs = [wl.tokens(tokens) for _ in range(pool)]
    ws = torch.empty(lib.moe_workspace_bytes(geom, tokens, wide), dtype=torch.uint8, device=dev)
    out = torch.empty((tokens, wl.cfg["hidden"]), dtype=torch.float32, device=dev)
    sel = torch.empty((tokens, wl.spec.topk), dtype=torch.int32, device=dev)
    wts = torch.empty((tokens, wl.spec.topk), dtype=torch.float32, device=dev)
    status = lib.Status(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    host_in = [torch.empty((tokens, wl.cfg["hidden"]), dtype=torch.float32).pin_memory() for _ in range(pool)]
    host_lg = []
    for i, (x, lg) in enumerate(xs):
        host_in[i].copy_(x)
        host_lg.append(None if lg is None else lg.cpu().pin_memory())
    host_out = torch.empty((tokens, wl.cfg["hidden"]), dtype=torch.float32).pin_memory()
    dev_in = torch.empty_like(out)
    dev_lg = None if xs[0][1] is None else torch.empty_like(xs[0][1])

    def step(i):
        x, lg = xs[i % pool]
        lib.moe_layer(geom, weights, x, status, logits=lg, wide=wide, workspace=ws, out=out, selected=sel, wts=wts)

    def step_e2e(i):
        dev_in.copy_(host_in[i % pool], non_blocking=True)
        if dev_lg is not None:
            dev_lg.copy_(host_lg[i % pool], non_blocking=True)
        lib.moe_layer(geom, weights, dev_in, status, logits=dev_lg, wide=wide, workspace=ws, out=out,
                      selected=sel, wts=wts)
        host_out.copy_(out, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush.fill_(i & 0xFF)          # evict L2 between timed steps (outside the timed span)
            starts[i].record()
            fn(i)
            stops[i].record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in zip(starts, stops)]

    for i in range(args.warmup):
        step(i)
        step_e2e(i)
    barrier()
    launches0 = lib.lib.yvex_b200_launch_count()
    with ClockSampler(local) as clocks:
        ms = timed(step, args.steps)
        launches = lib.lib.yvex_b200_launch_count() - launches0
        barrier()
        ms_e2e = timed(step_e2e, args.steps)
        barrier()
        # per-phase timing for the roofline of the dominant kernel
        n_ph = 7                         # 0..5 in order; 6 = after SwiGLU (between 3 and 4, wide path only)
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(n_ph)] for _ in range(args.steps)]
        for row in evs:
            for e in row:
                e.record()
        torch.cuda.synchronize()
        import ctypes as C
        phase_ms = [[] for _ in range(n_ph - 1)]
        arr_t = C.c_void_p * n_ph
        for i in range(args.steps):
            arr = arr_t(*[e.cuda_event for e in evs[i]])
            flush.fill_(i & 0xFF)
            lib.lib.yvex_b200_phase_events(arr, n_ph)
            step(i)
            lib.lib.yvex_b200_phase_events(None, 0)
        torch.cuda.synchronize()
        order = [0, 1, 2, 3] if not wide else [0, 1, 2, 3, 6, 4, 5]
        used = len(order)
        for i in range(args.steps):
            for p in range(used - 1):
                phase_ms[p].append(evs[i][order[p]].elapsed_time(evs[i][order[p + 1]]))
    if status.read() != 0:
        raise RuntimeError(f"device status word = {status.read()} after the timed region")

    total = torch.tensor([sum(ms), sum(ms_e2e)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    t_dev, t_e2e = total.tolist()
    value = world * tokens * args.steps / (t_dev / 1e3)
    e2e = world * tokens * args.steps / (t_e2e / 1e3)
    phases = [sum(p) / len(p) for p in phase_ms[:used - 1]]
    names = (["route", "gate_up", "down_combine"] if not wide
             else ["route", "permute_gather", "gate_up_gemm", "swiglu", "down_gemm", "combine"])
    roofline = None
    if wide:
        # dense contraction: count only real (token, expert) pairs, the shared expert included
        pairs = tokens * (wl.spec.topk + 1)
        flops = {"gate_up_gemm": pairs * 4.0 * wl.cfg["hidden"] * wl.cfg["inter"],
                 "down_gemm": pairs * 2.0 * wl.cfg["hidden"] * wl.cfg["inter"]}
        top = max(flops, key=lambda k: phases[names.index(k)])
        ach = flops[top] / (phases[names.index(top)] * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": ach / peaks["bf16_tflops"], "traffic": TRAFFIC.get(f"{wl.name}_{top}"),
                    "algorithmic_bytes": None, "peak_source": peaks["source"],
                    "peak_sustained": peaks["bf16_tflops_sustained"],
                    "layer_achieved": pairs * 6.0 * wl.cfg["hidden"] * wl.cfg["inter"] / (t_dev / args.steps * 1e-3) / 1e12}
    if not wide:
        pb = wl.phase_bytes_decode()
        cand = {"gate_up": (pb["gate_up"], phases[1]), "down": (pb["down"], phases[2])}
        top = max(cand, key=lambda k: cand[k][1])
        ach = cand[top][0] / (cand[top][1] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"], "traffic": TRAFFIC.get(wl.name) if top == "gate_up" else None,
                    "algorithmic_bytes": cand[top][0], "peak_source": peaks["source"],
                    "layer_achieved": wl.bytes_per_token_decode() / (t_dev / args.steps * 1e-3) / 1e9}
    if rank == 0:
        cpu = None
        if world == 1:
            cores = os.cpu_count() or 1
            try:
                tps, kind, _ = cpu_layer_tokens_per_s(wl, cores, 1, cores)
                cpu = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                       "sample": f"{cores} tokens of the same layer, one thread per token (plain-C port; the "
                                 "reference has no Q4_K decoder)"}
            except Exception as exc:  # the baseline must never take the GPU number down with it
                cpu = {"value": None, "unit": UNIT, "cores": cores, "kind": "port", "sample": f"failed: {exc}"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": t_dev / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16-mma/f32-accum, bf16 rounding points",
                "data": "synthetic",
                "config": {"workload": wl.name, **wl.cfg, "gate_up_qtype": "IQ2_XXS", "down_qtype": "Q4_K",
                           "l2": "flushed between steps (256 MiB rewrite)", "parallelism": f"replicas x{world}"},
                "clocks": clocks.summary(),
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(tokens * wl.cfg["hidden"] * 4 + (0 if dev_lg is None else dev_lg.numel() * 4)),
                        "d2h_bytes_per_step": int(tokens * wl.cfg["hidden"] * 4)},
                "gpu_launches": int(launches),
                "phases_ms": dict(zip(names, phases)),
                "roofline": roofline, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def ep_parity_check(torch, dist, lib, layer_out, geom_full, weights_full, x, lg, status, world, count=8):
    """Outside the timed region: `count` of this rank's rows run once more on this rank alone, through the
    single-device wide layer (every rank holds the full weight packs) - the sharded result must equal it
    bit for bit, because whole bf16 pair rows travel and are summed in rank order - and through the
    decode path (other kernels, other accumulation order): identical selection, relative L2 <= 1e-3."""
    t_loc = x.shape[0]
    idx = torch.linspace(0, t_loc - 1, count, device=x.device).long()
    xs, ls = x[idx].contiguous(), lg[idx].contiguous()
    want, sel_w, _ = lib.moe_layer(geom_full, weights_full, xs, status, logits=ls, wide=True)
    near, sel_n, _ = lib.moe_layer(geom_full, weights_full, xs, status, logits=ls, wide=False)
    got = layer_out[idx]
    bad_rows = (got.view(torch.int32) != want.view(torch.int32)).any(dim=1).sum()
    rel = (got.double() - near.double()).norm() / near.double().norm().clamp_min(1e-30)
    sel_bad = (sel_w != sel_n).any(dim=1).sum()
    stats = torch.stack([bad_rows.double(), sel_bad.double(), rel.double()])
    worst = stats.clone()
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    mismatched, sel_mismatched, rel_max = int(stats[0].item()), int(stats[1].item()), float(worst[2].item())
    if mismatched or sel_mismatched or not rel_max <= 1e-3 or status.read() != 0:
        raise RuntimeError(f"parity check failed: {mismatched} rows differ bitwise from the single-device wide layer, "
                           f"{sel_mismatched} selections differ, rel L2 vs decode path {rel_max:.3e}")
    return {"tokens": count * world, "mismatched": mismatched, "selection_mismatched": sel_mismatched,
            "against": "single-device wide layer on the same rows (bitwise) and decode path (rel L2 <= 1e-3)",
            "rel_l2_vs_decode_path": rel_max}


def pinned_twin(torch, lib, args, flush, status, dev):
    """Config 5 with Q2_K down weights - the qtype the reference's own MoE path decodes - device-timed
    like the main line, and checked against the compiled reference (the port where it is absent) on 4 rows."""
    from yvex_b200 import synth
    from yvex_b200.workloads import MoEWorkload
    wl = MoEWorkload("c5", 1, device=dev, down_qtype=synth.Q2_K)
    T = wl.cfg["tokens"]
    geom, weights = lib.geometry_of(wl.spec), lib.weights_of(wl.tensors)
    x, lg = wl.tokens(T)
    ws = torch.empty(lib.moe_workspace_bytes(geom, T, True), dtype=torch.uint8, device=dev)
    out = torch.empty((T, wl.cfg["hidden"]), dtype=torch.float32, device=dev)

    def step(i):
        lib.moe_layer(geom, weights, x, status, logits=lg, wide=True, workspace=ws, out=out)
    for i in range(args.warmup):
        step(i)
    ms = _timed_events(torch, step, args.steps, before=lambda i: flush.fill_(i & 0xFF))
    oracle, kind = oracle_backend(True)
    idx = torch.tensor([0, 5461, 10922, 16383], device=dev)
    hw, _ = wl.host_copy()
    L = oracle.layer(wl.spec, hw)
    rc, want, sel0, _ = oracle.moe_tokens(L, x[idx].cpu().numpy(), logits=lg[idx].cpu().numpy(), threads=4)
    got = out[idx].cpu().numpy().astype(np.float64)
    rel = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
    if rc != 0 or not rel <= 1e-3 or status.read() != 0:
        raise RuntimeError(f"Q2_K-down twin differs from the CPU {kind}: rc {rc}, rel L2 {rel:.3e}")
    t = sum(ms) / len(ms)
    return {"workload": "c5-q2k-down", "value": T / (t * 1e-3), "unit": UNIT, "ms_per_step": t,
            "checked_against": kind, "checked_tokens": 4, "rel_l2": rel}


def run_native_ep(args):
    """Config 5: the expert-parallel layer. Total work is fixed (16384 tokens, 256 experts) and
    split over the ranks (strong scaling): tokens by home rank, experts in contiguous shards."""
    import ctypes as C

    import torch
    import torch.distributed as dist
    from yvex_b200 import lib
    from yvex_b200.ep import DeviceOps, ExpertParallelLayer
    from yvex_b200.workloads import MoEWorkload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    wl = MoEWorkload(args.workload, 1, device=dev)            # same seed on every rank: identical packs
    spec, cfg = wl.spec, wl.cfg
    T, E, H, I = cfg["tokens"], cfg["experts"], cfg["hidden"], cfg["inter"]
    e_loc, t_loc = E // world, T // world
    x_all, lg_all = wl.tokens(T)
    x = x_all[rank * t_loc:(rank + 1) * t_loc].contiguous()
    lg = lg_all[rank * t_loc:(rank + 1) * t_loc].contiguous()
    del x_all, lg_all
    shard = {}
    for name, rows in (("gate", I), ("up", I), ("down", H)):
        per = wl.tensors[name].numel() // E
        shard[name] = wl.tensors[name][rank * e_loc * per:(rank + 1) * e_loc * per]
    for name in ("shared_gate", "shared_up", "shared_down"):
        shard[name] = wl.tensors[name]
    geom_full = lib.geometry_of(spec)
    spec_local = type(spec)(H, e_loc, spec.topk, I, down_qtype=spec.down_qtype)
    geom_local = lib.geometry_of(spec_local)
    status = lib.Status(dev)
    # experiment knobs (defaults are what the library picks): segments of the exchange pipeline, whether the exchange runs
    # on its own stream beside the GEMMs, CTAs of the persistent GEMM
    ops = DeviceOps(geom_full, geom_local, lib.weights_of(shard), status, overlap=os.environ.get("YVEX_EP_OVERLAP", "0") != "0",
                    peer_return=os.environ.get("YVEX_EP_PEER_RETURN", "1") != "0",
                    peer_dispatch=os.environ.get("YVEX_EP_PEER_DISPATCH", "1") != "0")
    seg_env = os.environ.get("YVEX_EP_SEGMENTS")
    layer = ExpertParallelLayer(E, spec.topk, ops, segments=int(seg_env) if seg_env else None)
    if os.environ.get("YVEX_EP_CTAS"):
        ops.cta_limit = int(os.environ["YVEX_EP_CTAS"])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    host_x, host_lg = x.cpu().pin_memory(), lg.cpu().pin_memory()
    host_out = torch.empty((t_loc, H), dtype=torch.float32).pin_memory()
    dev_x, dev_lg = torch.empty_like(x), torch.empty_like(lg)

    def step(i):
        return layer.forward(x, lg)[0]

    if world == 1:
        # One GPU owns every expert: nothing to exchange, so the step is the single-device wide layer
        # (routed and shared experts in the same grouped GEMM launches).
        weights_full = lib.weights_of(wl.tensors)
        ws_wide = torch.empty(lib.moe_workspace_bytes(geom_full, T, True), dtype=torch.uint8, device=dev)
        out_dev = torch.empty((T, H), dtype=torch.float32, device=dev)

        def step(i):  # noqa: F811
            lib.moe_layer(geom_full, weights_full, x, status, logits=lg, wide=True, workspace=ws_wide, out=out_dev)
            return out_dev

    def step_e2e(i):
        dev_x.copy_(host_x, non_blocking=True)
        dev_lg.copy_(host_lg, non_blocking=True)
        host_out.copy_(layer.forward(dev_x, dev_lg)[0], non_blocking=True)

    e2e_api = "ExpertParallelLayer.forward (C-ABI device layer + NCCL), pinned host rows in/out"
    if world == 1:
        # One GPU: the end-to-end leg goes through the C11 host boundary itself - resident weights
        # named by host pointers, host rows in, host rows out, one synchronous execute_rows_wide.
        from yvex_b200 import backend as B
        be = B.Backend(device=f"cuda:{local}".encode())
        if be.rc != B.OK:
            raise RuntimeError("host boundary failed to open: " + be.message())
        arena = B.ResidentArena(be, {k: v.cpu().numpy() for k, v in wl.tensors.items()})
        job = B.moe_job(arena, spec, router=False, family=b"sm100-f16-tcgen05-expert")
        bops, need = B.moe_ops(be), B.ull()
        assert bops.workspace_required_wide(job.layer, T, C.byref(need), C.byref(be.err)) == B.OK
        rcw, bws, _ = be.tensor(need.value)
        assert rcw == B.OK and B._lib.yvex_backend_workspace_attach(be.h, bws, C.byref(be.err)) == B.OK
        batch = B.row_batch(T, H, host_rows=host_x.data_ptr(), router_logits=host_lg.data_ptr())
        bout = B.row_output(host_out.data_ptr(), T * H)
        bres = B.RowBatchResult()
        e2e_api = "yvex_backend_moe_operations.execute_rows_wide (C11 host boundary), pinned host rows in/out"

        def step_e2e(i):  # noqa: F811
            rc_b = bops.execute_rows_wide(be.h, C.byref(job), C.byref(batch), C.byref(bout), C.byref(bres), C.byref(be.err))
            if rc_b != B.OK:
                raise RuntimeError("execute_rows_wide: " + be.message())

        def two_sessions(steps):
            """The same steps issued the way a server with two execution sessions issues them: two backend objects
            (each with its own resident copy of the weights, workspace and stream) take alternate steps with deferred
            completion, so one session's host copies run beside the other's GEMMs. Every step still copies its rows
            in from pinned host memory and its result rows back out inside the timed region."""
            be2 = B.Backend(device=f"cuda:{local}".encode())
            if be2.rc != B.OK:
                raise RuntimeError("second session failed to open: " + be2.message())
            arena2 = B.ResidentArena(be2, {k: v.cpu().numpy() for k, v in wl.tensors.items()})
            job2 = B.moe_job(arena2, spec, router=False, family=b"sm100-f16-tcgen05-expert")
            rc2, ws2, _ = be2.tensor(need.value)
            assert rc2 == B.OK and B._lib.yvex_backend_workspace_attach(be2.h, ws2, C.byref(be2.err)) == B.OK
            out2 = torch.empty((T, H), dtype=torch.float32).pin_memory()
            sess = []
            for b_, j_, o_ in ((be, job, host_out), (be2, job2, out2)):
                slot = B.CompletionSlot()
                comp = B.Completion(1, C.pointer(slot))
                j_.device_completion = C.pointer(comp)
                sess.append(dict(be=b_, job=j_, out=B.row_output(o_.data_ptr(), T * H), res=B.RowBatchResult(), ops=B.moe_ops(b_),
                                 keep=(slot, comp), pending=False))

            def finish(s_):
                if s_["pending"] and s_["ops"].complete_rows(s_["be"].h, 0, C.byref(s_["res"]), C.byref(s_["be"].err)) != B.OK:
                    raise RuntimeError("complete_rows: " + s_["be"].message())
                s_["pending"] = False

            def run(n):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for i in range(n):
                    s_ = sess[i & 1]
                    finish(s_)
                    if s_["ops"].execute_rows_wide(s_["be"].h, C.byref(s_["job"]), C.byref(batch), C.byref(s_["out"]), C.byref(s_["res"]),
                                                   C.byref(s_["be"].err)) != B.OK:
                        raise RuntimeError("execute_rows_wide (deferred): " + s_["be"].message())
                    s_["pending"] = True
                for s_ in sess:
                    finish(s_)
                return time.perf_counter() - t0

            try:
                run(2)
                n = max(4, steps + (steps & 1))
                t = run(n)
                same = torch.equal(out2.view(torch.int32), host_out.view(torch.int32))
            finally:
                job.device_completion = None
                be2.close()
            if not same:
                raise RuntimeError("the two sessions' result rows differ")
            return {"value": T * n / t, "unit": UNIT, "steps": n, "ms_per_step": t / n * 1e3, "l2": "inputs larger than L2 (4.5 GB per step)",
                    "api": "two yvex_backend objects alternate steps: execute_rows_wide with deferred completion, complete_rows "
                           "before a session's next step; pinned host rows in and out every step"}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, wall=False):
        out = []
        for i in range(steps):
            flush.fill_(i & 0xFF)
            barrier()
            if wall:                       # the boundary call synchronises its own stream before it returns
                t0 = time.perf_counter()
                fn(i)
                out.append((time.perf_counter() - t0) * 1e3)
                continue
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(i)
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return out

    for i in range(args.warmup):
        step(i)
        step_e2e(i)
    barrier()
    launches0 = lib.lib.yvex_b200_launch_count()
    with ClockSampler(local) as clocks:
        ms = timed(step, args.steps)
        launches = lib.lib.yvex_b200_launch_count() - launches0
        ms_e2e = timed(step_e2e, args.steps, wall=world == 1)
        # GEMM phases of one pair list, timed with the library's phase events, and (N > 1) the spans of the
        # pipelined step on the compute stream
        n_ph, gemm_ms, pair_counts, spans = 7, [[], [], []], [], {}       # events 0..5 in order, 6 = after SwiGLU

        def phase_probe(run):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_ph)]
            for e in evs:
                e.record()
            arr = (C.c_void_p * n_ph)(*[e.cuda_event for e in evs])
            lib.lib.yvex_b200_phase_events(arr, n_ph)
            y = run()
            lib.lib.yvex_b200_phase_events(None, 0)
            torch.cuda.synchronize()
            gemm_ms[0].append(evs[2].elapsed_time(evs[3]))
            gemm_ms[1].append(evs[6].elapsed_time(evs[4]))
            gemm_ms[2].append(evs[3].elapsed_time(evs[6]))
            return y

        if world == 1:
            for i in range(min(args.steps, 5)):
                flush.fill_(i & 0xFF)
                phase_probe(lambda: step(i))
                pair_counts.append(T * (spec.topk + 1))
        else:
            real_payload = ops.expert_rows_payload

            def probed(payload, hidden, **kw):
                if payload.shape[0] and not probed.done:
                    probed.done = True
                    pair_counts.append(payload.shape[0])
                    return phase_probe(lambda: real_payload(payload, hidden, **kw))
                return real_payload(payload, hidden, **kw)

            ops.expert_rows_payload = probed
            for i in range(min(args.steps, 5)):
                probed.done = False
                flush.fill_(i & 0xFF)
                step(i)
            ops.expert_rows_payload = real_payload
            layer.timings = {}
            for i in range(min(args.steps, 5)):
                flush.fill_(i & 0xFF)
                barrier()
                step(i)
                torch.cuda.synchronize()
                marks = layer.timings["marks"]
                for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                    spans.setdefault(name, []).append(a.elapsed_time(b))
            layer.timings = None
        torch.cuda.synchronize()
    if status.read() != 0:
        raise RuntimeError(f"device status word = {status.read()} after the timed region")
    # result check at this world size, outside the timed region
    weights_all = lib.weights_of(wl.tensors)
    parity = ep_parity_check(torch, dist, lib, step(0), geom_full, weights_all, x, lg, status, world)
    if world == 1:
        # the end-to-end leg's host rows must be the device-timed leg's rows
        torch.cuda.synchronize()
        if not torch.equal(host_out.view(torch.int32), step(0).cpu().view(torch.int32)):
            raise RuntimeError("execute_rows_wide (host rows) differs from the device-resident layer")
    twin = gemv = sessions2 = c11 = None
    if world > 1 and os.environ.get("YVEX_BENCH_C11", "0") != "0":
        # opt-in (YVEX_BENCH_C11=1): the same step through the C11 orchestration (yvex_moe_ep_execute_rows: NCCL send/recv
        # groups, pinned host rows in and out), beside the Python layer's peer-memory path that the headline measures
        try:
            c11 = c11_exchange_record(torch, dist, args, wl, spec, shard, host_x, host_lg, local, rank, world, step(0))
        except Exception as exc:
            c11 = {"value": None, "failed": f"{type(exc).__name__}: {exc}"}
    if world == 1 and rank == 0:
        try:
            sessions2 = two_sessions(args.steps)
        except RuntimeError:
            raise
        except Exception as exc:                                # e.g. out of memory for the second resident copy
            sessions2 = {"value": None, "failed": str(exc)}
        try:
            twin = pinned_twin(torch, lib, args, flush, status, dev)
        except RuntimeError:
            raise
        except Exception as exc:                                # e.g. out of memory beside the main workload
            twin = {"workload": "c5-q2k-down", "value": None, "failed": str(exc)}
        # the second half of the metric: HBM GB/s of the dequant-fused matvec (config 1 and its variants)
        from yvex_b200 import synth
        torch.cuda.empty_cache()
        gen = torch.Generator(device=dev)
        gen.manual_seed(synth.BASE_SEED + 0)
        with ClockSampler(local) as gemv_clocks:
            gemv, _keep = gemv_records(torch, lib, synth, dev, peaks, max(3, min(args.steps, 10)), args.warmup, status, gen)
        del _keep
        gemv["clocks"] = gemv_clocks.summary()
    # per-step max over ranks, then summed: every step is bracketed by a barrier
    tm = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    t_dev, t_e2e = tm.sum(dim=1).tolist()
    value = T * args.steps / (t_dev / 1e3)
    e2e = T * args.steps / (t_e2e / 1e3)
    if rank == 0:
        gu = sum(gemm_ms[0]) / len(gemm_ms[0])
        dn = sum(gemm_ms[1]) / len(gemm_ms[1])
        sw = sum(gemm_ms[2]) / len(gemm_ms[2])
        pairs = sum(pair_counts) / len(pair_counts)
        top, t_top, fl = ("gate_up_gemm", gu, pairs * 4.0 * H * I) if gu >= dn else ("down_gemm", dn, pairs * 2.0 * H * I)
        ach = fl / (t_top * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]                             # burst: the timed region runs near the maximum SM clock
        roofline = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "traffic": TRAFFIC.get(f"c5_{top}") if world == 1 else None,
                    "peak_source": peaks["source"] + " (burst)", "peak_sustained": peaks["bf16_tflops_sustained"],
                    "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                    "other_gemm": {"kernel": "down_gemm" if top == "gate_up_gemm" else "gate_up_gemm",
                                   "achieved": (pairs * (2.0 if top == "gate_up_gemm" else 4.0) * H * I) /
                                               ((dn if top == "gate_up_gemm" else gu) * 1e-3) / 1e12},
                    "pairs_per_launch": pairs,
                    "layer_achieved": T * (spec.topk + 1) * 6.0 * H * I / world / (t_dev / args.steps * 1e-3) / 1e12}
        cpu = None
        if world == 1:
            cores = os.cpu_count() or 1
            try:
                tps, kind, _ = cpu_layer_tokens_per_s(wl, cores, 1, cores)
                cpu = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                       "sample": f"{cores} tokens of the same layer, one thread per token (plain-C port; the "
                                 "reference has no Q4_K decoder)"}
            except Exception as exc:
                cpu = {"value": None, "unit": UNIT, "cores": cores, "kind": "port", "sample": f"failed: {exc}"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": t_dev / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16-mma/f32-accum, bf16 rounding points",
                "data": "synthetic",
                "config": {"workload": wl.name, **cfg, "gate_up_qtype": "IQ2_XXS", "down_qtype": "Q4_K",
                           "l2": "flushed between steps (256 MiB rewrite)",
                           "parallelism": (f"ep{world}: {e_loc} experts and {t_loc} tokens per rank, NCCL all-to-all-v, "
                                           f"{layer.segments} expert segment(s), exchange {'beside' if ops.streams else 'between'} the GEMMs"
                                           if world > 1
                                           else "ep1: all experts on one device, fused wide layer, no exchange")},
                "clocks": clocks.summary(),
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(T * (H + E) * 4),
                        "d2h_bytes_per_step": int(T * H * 4), "api": e2e_api},
                **({"e2e_two_sessions": sessions2} if sessions2 else {}),
                **({"c11_nccl_exchange": c11} if c11 else {}),
                "gpu_launches": int(launches * world),
                "phases_ms": {"gate_up_gemm": gu, "swiglu": sw, "down_gemm": dn,
                              **({"pairs_in_timed_gemm": pairs, "step_spans_rank0": {k: sum(v) / len(v) for k, v in spans.items()}}
                                 if world > 1 else {})},
                "parity": parity, "twin": twin, "gemv": gemv,
                "roofline": roofline, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def c11_exchange_record(torch, dist, args, wl, spec, shard, host_x, host_lg, local, rank, world, want):
    """Every rank: its shard resident on a host-boundary backend, yvex_moe_ep_open over an identifier broadcast from rank
    0, then timed yvex_moe_ep_execute_rows calls (wall clock around a synchronous call, max over ranks)."""
    import ctypes as C
    from yvex_b200 import backend as B
    T, H, E = wl.cfg["tokens"], wl.cfg["hidden"], wl.cfg["experts"]
    t_loc, dev = T // world, torch.device("cuda", local)
    be = B.Backend(device=f"cuda:{local}".encode())
    if be.rc != B.OK:
        raise RuntimeError("host boundary failed to open: " + be.message())
    arena = B.ResidentArena(be, {k: v.cpu().numpy() for k, v in shard.items()})
    local_spec = type(spec)(H, E // world, spec.topk, wl.cfg["inter"], down_qtype=spec.down_qtype)
    job = B.moe_job(arena, local_spec, router=False, family=b"sm100-f16-tcgen05-expert")
    job._plan.routed_experts = E
    ident = (C.c_ubyte * 128)()
    if rank == 0 and B._lib.yvex_moe_ep_unique_id(ident, C.byref(be.err)) != B.OK:
        raise RuntimeError("yvex_moe_ep_unique_id: " + be.message())
    box = torch.tensor(list(bytes(ident)), dtype=torch.uint8, device=dev)
    dist.broadcast(box, 0)
    C.memmove(ident, bytes(box.cpu().tolist()), 128)
    ep, need = B.vp(), B.ull()
    if B._lib.yvex_moe_ep_open(C.byref(ep), be.h, ident, world, rank, 60000, C.byref(be.err)) != B.OK:
        raise RuntimeError("yvex_moe_ep_open: " + be.message())
    try:
        assert B._lib.yvex_moe_ep_workspace_required(job.layer, t_loc, world, C.byref(need), C.byref(be.err)) == B.OK
        rcw, ws, _ = be.tensor(need.value)
        assert rcw == B.OK and B._lib.yvex_backend_workspace_attach(be.h, ws, C.byref(be.err)) == B.OK, be.message()
        out = torch.empty((t_loc, H), dtype=torch.float32).pin_memory()
        batch = B.row_batch(t_loc, H, host_rows=host_x.data_ptr(), router_logits=host_lg.data_ptr())
        bout, res = B.row_output(out.data_ptr(), t_loc * H), B.RowBatchResult()
        times = []
        for i in range(2 + max(3, min(args.steps, 10))):
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            if B._lib.yvex_moe_ep_execute_rows(ep, C.byref(job), C.byref(batch), C.byref(bout), C.byref(res), C.byref(be.err)) != B.OK:
                raise RuntimeError("yvex_moe_ep_execute_rows: " + be.message())
            if i >= 2:
                times.append(time.perf_counter() - t0)
        same = torch.equal(out.view(torch.int32), want.cpu().view(torch.int32))
        tm = torch.tensor(times, dtype=torch.float64, device=dev)
        ok = torch.tensor([int(same)], device=dev)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        t = float(tm.mean())
        return {"value": T / t, "unit": UNIT, "ms_per_step": t * 1e3, "steps": len(times), "bitwise_equal_to_the_timed_layer": bool(ok.item()),
                "api": "yvex_moe_ep_execute_rows (C11, ncclSend/ncclRecv groups), pinned host rows in and out, no overlap of exchange and GEMMs"}
    finally:
        B._lib.yvex_moe_ep_close(C.byref(ep), C.byref(be.err))
        be.close()


def _timed_events(torch, fn, steps, before=None):
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if before:
            before(i)
        starts[i].record()
        fn(i)
        stops[i].record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in zip(starts, stops)]


def gemv_records(torch, lib, synth, dev, peaks, steps, warmup, status, gen):
    """HBM throughput of the dequant-fused matvec, every case streaming >= 1.1 GB of distinct weight
    bytes per step (inputs larger than L2): `batch` = 256 (128, 64) DIFFERENT 4096 x 4096 matrices with
    their own input rows in one persistent launch; `one_matrix` = the same bytes as a single tall
    matrix; `per_launch` = one launch per matrix, replayed from a CUDA graph; `output_head` = a BF16
    [129280 x 4096] matrix, the shape of the reference model's logits projection."""
    from yvex_b200.workloads import device_blocks
    rows = width = 4096
    out = {}

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ms = _timed_events(torch, lambda i: fn(), steps)
        return sum(ms) / len(ms) * 1e-3

    def rec(algo, t):
        gbs = algo / t / 1e9
        return {"GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_8TBs": gbs / 8000.0, "ms": t * 1e3}

    for name, q, count in (("IQ2_XXS", synth.IQ2_XXS, 256), ("Q4_K", synth.Q4_K, 128), ("Q8_0", synth.Q8_0, 64),
                           ("Q2_K", synth.Q2_K, 200), ("MXFP4", synth.MXFP4, 128)):
        rb = synth.row_bytes(q, width)
        enc = device_blocks(torch, q, rows * count, width, gen, dev)
        xs = torch.randn((count, width), device=dev, generator=gen)
        ys = torch.empty((count, rows), dtype=torch.float32, device=dev)
        algo = count * (rows * rb + 4 * width + 4 * rows)
        case = {"matrices": count, "bytes_per_step": algo}
        case["batch"] = rec(algo, timed(lambda: lib.gemv_batch(q, enc, count, rows, width, xs, status, out=ys, row_bytes=rb)))
        tall = torch.empty((1, rows * count), dtype=torch.float32, device=dev)
        case["one_matrix"] = rec(count * rows * rb + 4 * width + 4 * rows * count,
                                 timed(lambda: lib.gemv(q, enc, rows * count, width, xs[0], status, out=tall, row_bytes=rb)))
        mats = [enc[i * rows * rb:(i + 1) * rows * rb] for i in range(count)]

        def launch_all():
            for i in range(count):
                lib.gemv(q, mats[i], rows, width, xs[i], status, out=ys[i:i + 1], row_bytes=rb)
        launch_all()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch_all()
        case["per_launch"] = rec(algo, timed(graph.replay))
        if name == "IQ2_XXS":
            one = _timed_events(torch, lambda i: lib.gemv(q, mats[i % count], rows, width, xs[i % count], status, out=ys[0:1],
                                                          row_bytes=rb), 50)
            case["single_launch_us"] = sorted(one)[len(one) // 2] * 1e3
            keep = (enc, xs, ys, mats, rb)
        out[name] = case
        del graph
        if name != "IQ2_XXS":
            del enc, xs, ys, mats, tall
    vocab, hidden = 129280, 4096
    head = torch.randn((vocab, hidden), device=dev, generator=gen).to(torch.bfloat16).view(torch.uint8).reshape(-1)
    hx = torch.randn(hidden, device=dev, generator=gen)
    hy = torch.empty((1, vocab), dtype=torch.float32, device=dev)
    algo = vocab * hidden * 2 + 4 * hidden + 4 * vocab
    out["output_head_BF16"] = dict(rec(algo, timed(lambda: lib.gemv(synth.BF16, head, vocab, hidden, hx, status, out=hy,
                                                                    row_bytes=hidden * 2))),
                                   rows=vocab, width=hidden, bytes_per_step=algo)
    if status.read() != 0:
        raise RuntimeError(f"device status word = {status.read()} in the matvec records")
    return out, keep


def run_gemv_stream(args):
    """Config 1: the 4096 x 4096 IQ2_XXS dequant GEMV. One matrix (4.3 MB) fits in L2, so a step is
    256 DIFFERENT matrices (1.1 GB streamed once, no reuse) in one persistent batch launch; GB/s =
    algorithmic bytes of the 256 products / step time. Q4_K, Q8_0, the one-launch-per-matrix graph, a
    single tall matrix and the BF16 output-head shape are reported beside it."""
    import ctypes as C
    import torch
    from yvex_b200 import backend as B
    from yvex_b200 import lib, synth
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if int(os.environ.get("RANK", "0")) != 0:
        return                                         # replicas only: one rank measures
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    rows = width = 4096
    gen = torch.Generator(device=dev)
    gen.manual_seed(synth.BASE_SEED + 0)
    status = lib.Status(dev)
    with ClockSampler(local) as clocks:
        records, (enc, xs, ys, mats, rb) = gemv_records(torch, lib, synth, dev, peaks, args.steps, args.warmup, status, gen)
    count = records["IQ2_XXS"]["matrices"]
    gbs, t = records["IQ2_XXS"]["batch"]["GB/s"], records["IQ2_XXS"]["batch"]["ms"] * 1e-3
    # result check of the timed configuration: 4 of the 256 products against the CPU port
    port, kind = oracle_backend(False)
    got = lib.gemv_batch(synth.IQ2_XXS, enc, count, rows, width, xs, status, row_bytes=rb).cpu().numpy()
    for m in (0, 85, 170, 255):
        rc, want = port.matvec(synth.IQ2_XXS, mats[m].cpu().numpy().reshape(rows, rb), rows, width, xs[m].cpu().numpy(), threads=os.cpu_count() or 1)
        err = float(np.abs(got[m] - want).max() / max(np.abs(want).max(), 1e-30))
        if rc != 0 or not err <= 2e-5:
            raise RuntimeError(f"batched matvec {m} differs from the CPU port: {err:.3e}")
    # end to end through the host boundary: host x in, resident weights, host y out, one call per matrix
    be = B.Backend(device=f"cuda:{local}".encode())
    e2e_n = 64
    arena = B.ResidentArena(be, {"w": enc[:e2e_n * rows * rb].cpu().numpy()})
    hx = xs[:e2e_n].cpu().numpy()
    tin = be.from_array(hx[0:1], B.F32, [1, width])
    tout = be.tensor(rows * 4, B.F32, [1, rows])[1]
    facts = B.Facts()

    def e2e_step():
        for i in range(e2e_n):
            be.write(tin, hx[i:i + 1])
            rc = B._lib.yvex_backend_cuda_encoded_matvec(be.h, arena.host_ptr("w") + i * rows * rb, rows * rb, synth.IQ2_XXS,
                                                         rows, width, rb, 1, tin, None, 0, None, tout, 0, C.byref(facts),
                                                         C.byref(be.err))
            if rc != B.OK:
                raise RuntimeError(be.message())
            be.read(tout, np.float32, rows)
    e2e_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    t_e2e = (time.perf_counter() - t0) / args.steps
    e2e_algo = e2e_n * (rows * rb + 4 * width + 4 * rows)
    be.close()
    # CPU baseline: the port's matvec on one matrix, all cores over rows
    cores = os.cpu_count() or 1
    w0 = mats[0].cpu().numpy()
    x0 = xs[0].cpu().numpy()
    t0 = time.perf_counter()
    port.matvec(synth.IQ2_XXS, w0, rows, width, x0, threads=cores)
    t_cpu = time.perf_counter() - t0
    line = {"metric": "dequant_gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8-mma/s32-accum (exact integer products), f32 in/out", "data": "synthetic",
            "config": {"workload": "c1", "rows": rows, "width": width, "qtype": "IQ2_XXS", "matrices_per_step": count,
                       "l2": "inputs larger than L2: 256 distinct matrices (1.1 GB) per step, one batch launch",
                       "parallelism": f"replicas only (1 of {world} ranks measures)"},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_algo / t_e2e / 1e9, "unit": "GB/s", "h2d_bytes_per_step": e2e_n * width * 4,
                    "d2h_bytes_per_step": e2e_n * rows * 4,
                    "api": f"yvex_backend_cuda_encoded_matvec, {e2e_n} calls per step, host x in / host y out per call"},
            "gpu_launches": args.steps,
            "parity": {"checked_matrices": 4, "against": "CPU port, max abs error / max |y| <= 2e-5"},
            "gemv": records,
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel<StreamIq2>", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "algorithmic_bytes": count * (rows * rb + 4 * width + 4 * rows), "peak_source": peaks["source"],
                         "frac_of_nominal_8TBs": gbs / 8000.0},
            "cpu_baseline": {"value": (rows * rb + 4 * width + 4 * rows) / t_cpu / 1e9, "unit": "GB/s", "cores": cores,
                             "kind": kind, "sample": "one 4096x4096 IQ2_XXS matvec, rows split over all cores"}}
    print(json.dumps(line), flush=True)


def run_attention(args):
    """Config 4: GQA decode attention, 16 sessions x 32 q heads / 8 kv heads x d128 over a bf16 KV
    cache of 32768 positions (2.1 GB read per step, larger than L2)."""
    import ctypes as C
    import torch
    from yvex_b200 import backend as B
    from yvex_b200 import lib, synth
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    peaks = measured_peaks()
    S, Hq, Hkv, D, ctx = 16, 32, 8, 128, 32768
    gen = torch.Generator(device=dev)
    gen.manual_seed(synth.BASE_SEED + 3)
    q = torch.randn((S, Hq, D), device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn((S, Hkv, ctx, D), device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn((S, Hkv, ctx, D), device=dev, generator=gen).to(torch.bfloat16)
    out = torch.empty((S, Hq, D), dtype=torch.float32, device=dev)
    ws = torch.empty(int(lib.lib.yvex_b200_attention_workspace_bytes(S, Hq, Hkv, D, ctx)), dtype=torch.uint8, device=dev)
    status = lib.Status(dev)
    scale, pos = D ** -0.5, ctx - 1
    algo = 2 * k.numel() * 2 + q.numel() * 2 + out.numel() * 4

    def step(i):
        lib.attention_gqa_decode(q, k, v, pos, scale, status, workspace=ws, out=out)
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    l0 = lib.lib.yvex_b200_launch_count()
    with ClockSampler(local) as clocks:
        ms = _timed_events(torch, step, args.steps)
    launches = lib.lib.yvex_b200_launch_count() - l0
    if status.read() != 0:
        raise RuntimeError(f"device status word = {status.read()}")
    t = sum(ms) / len(ms) * 1e-3
    gbs = algo / t / 1e9
    # end to end through the host boundary: the KV cache is resident (as in serving), q comes from
    # the host and the output goes back to the host every step
    be = B.Backend(device=f"cuda:{local}".encode())
    bits = lambda a: a.view(torch.int16).cpu().numpy().view(np.uint16)
    tq, tk, tv = be.from_array(bits(q), B.BF16), be.from_array(bits(k), B.BF16), be.from_array(bits(v), B.BF16)
    tout = be.tensor(out.numel() * 4, B.F32, list(out.shape))[1]
    tws = be.tensor(max(ws.numel(), 256))[1]
    assert B._lib.yvex_backend_workspace_attach(be.h, tws, C.byref(be.err)) == B.OK
    hq = bits(q)

    def e2e_step():
        be.write(tq, hq)
        rc = B._lib.yvex_backend_attention_gqa_decode(be.h, tq, tk, tv, S, Hq, Hkv, D, ctx, pos, scale, tout, C.byref(be.err))
        if rc != B.OK:
            raise RuntimeError(be.message())
        return be.read(tout, np.float32, out.numel())[1]
    got = e2e_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    t_e2e = (time.perf_counter() - t0) / args.steps
    if not np.array_equal(got.view(np.uint32), out.cpu().numpy().reshape(-1).view(np.uint32)):
        raise RuntimeError("host-boundary result differs from the device-layer result")
    B._lib.yvex_backend_workspace_detach(be.h, C.byref(be.err))
    be.close()
    # CPU baseline: the port on one session (1/16 of the work), all cores over heads
    port, kind = oracle_backend(False)
    cores = os.cpu_count() or 1
    t0 = time.perf_counter()
    port.attention_gqa_decode(bits(q[:1]), bits(k[:1]), bits(v[:1]), pos, scale, threads=cores)
    t_cpu = time.perf_counter() - t0
    line = {"metric": "attention_decode_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 in, f32 accumulate and out", "data": "synthetic",
            "config": {"workload": "c4", "sessions": S, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": ctx,
                       "l2": "inputs larger than L2 (2.1 GB of K/V per step)",
                       "parallelism": f"replicas only (1 of {world} ranks measures)"},
            "clocks": clocks.summary(),
            "e2e": {"value": algo / t_e2e / 1e9, "unit": "GB/s", "h2d_bytes_per_step": q.numel() * 2,
                    "d2h_bytes_per_step": out.numel() * 4,
                    "api": "yvex_backend_attention_gqa_decode; KV cache resident, q from host, out to host"},
            "gpu_launches": int(launches),
            "sessions_per_s": S / t,
            "roofline": {"bound": "hbm", "kernel": "gqa_decode_kernel<128,4>", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": TRAFFIC["c4"], "algorithmic_bytes": algo,
                         "peak_source": peaks["source"]},
            "cpu_baseline": {"value": (algo / S) / t_cpu / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
                             "sample": "one of the 16 sessions (32 heads x 32768 keys), heads split over all cores"}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c1":
        run_gemv_stream(args)
    elif args.workload == "c4":
        run_attention(args)
    elif args.workload == "c5":
        run_native_ep(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
