"""The benchmark configurations as device-resident synthetic workloads (seeded; no dataset).

Weights are generated directly on the GPU (uniform random payload bytes, f16 block scales uniform
in [1e-4, 1e-3], exactly the distribution the configs state); `host_copy()` hands the CPU checkers
the very same bytes.
"""
from __future__ import annotations

import numpy as np

from . import synth

CONFIGS = {
    # name: hidden, experts, topk, inter, tokens, router mode
    "c2": dict(hidden=4096, experts=64, topk=6, inter=1536, tokens=1, router="weights"),
    "c3": dict(hidden=4096, experts=64, topk=6, inter=1536, tokens=2048, router="logits"),
    "c5": dict(hidden=7168, experts=256, topk=8, inter=2048, tokens=16384, router="logits"),
}


def device_blocks(torch, qtype, rows, width, gen, device):
    elems, nbytes, scale_at = synth.BLOCKS[qtype]
    nblk = rows * (width // elems)
    raw = torch.randint(0, 256, (nblk, nbytes), dtype=torch.uint8, device=device, generator=gen)
    for off in scale_at:
        d = (torch.rand(nblk, device=device, generator=gen) * 9e-4 + 1e-4).to(torch.float16)
        raw[:, off:off + 2] = d.view(torch.uint8).reshape(nblk, 2)
    if qtype == synth.MXFP4:                 # byte 0 is an E8M0 exponent: scales 2^-17 .. 2^-4, as synth.random_blocks
        raw[:, 0] = torch.randint(110, 124, (nblk,), dtype=torch.uint8, device=device, generator=gen)
    return raw.reshape(-1)


class MoEWorkload:
    def __init__(self, name, seed_index, device="cuda", down_qtype=synth.Q4_K, experts_range=None):
        import torch
        cfg = CONFIGS[name]
        self.name, self.cfg, self.device = name, cfg, device
        self.spec = synth.MoELayerSpec(cfg["hidden"], cfg["experts"], cfg["topk"], cfg["inter"],
                                       down_qtype=down_qtype)
        gen = torch.Generator(device=device)
        gen.manual_seed(synth.BASE_SEED + seed_index)
        s, H, I, E = self.spec, cfg["hidden"], cfg["inter"], cfg["experts"]
        t = {}
        t["gate"] = device_blocks(torch, s.gate_qtype, E * I, H, gen, device)
        t["up"] = device_blocks(torch, s.up_qtype, E * I, H, gen, device)
        t["down"] = device_blocks(torch, s.down_qtype, E * H, I, gen, device)
        t["shared_gate"] = device_blocks(torch, s.gate_qtype, I, H, gen, device)
        t["shared_up"] = device_blocks(torch, s.up_qtype, I, H, gen, device)
        t["shared_down"] = device_blocks(torch, s.down_qtype, H, I, gen, device)
        if cfg["router"] == "weights":
            t["router"] = torch.randn((E, H), device=device, generator=gen) * 0.02
        self.tensors = t
        self.gen = gen

    def tokens(self, count):
        import torch
        x = torch.randn((count, self.cfg["hidden"]), device=self.device, generator=self.gen)
        logits = None
        if self.cfg["router"] == "logits":
            logits = torch.randn((count, self.cfg["experts"]), device=self.device, generator=self.gen)
        return x, logits

    def host_copy(self):
        s, H, I, E = self.spec, self.cfg["hidden"], self.cfg["inter"], self.cfg["experts"]
        w = {k: v.cpu().numpy() for k, v in self.tensors.items() if k != "router"}
        router = self.tensors["router"].cpu().numpy() if "router" in self.tensors else None
        return w, router

    def bytes_per_token_decode(self):
        """Algorithmic bytes of one decode token: every active weight byte once, router once,
        input and output rows once."""
        s = self.spec
        per_expert = s.weight_bytes_per_expert()
        router = s.experts * s.hidden * 4 if self.cfg["router"] == "weights" else s.experts * 4
        return (s.topk + 1) * per_expert + router + 2 * s.hidden * 4

    def phase_bytes_decode(self):
        s = self.spec
        n = s.topk + 1
        gate_up = n * 2 * s.inter * synth.row_bytes(s.gate_qtype, s.hidden) + s.hidden * 4 + n * s.inter * 4
        down = n * s.hidden * synth.row_bytes(s.down_qtype, s.inter) + n * s.inter * 4 + s.hidden * 4
        return {"gate_up": gate_up, "down": down}
