"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

No dataset or checkpoint is involved anywhere: weights are random GGUF blocks (every bit pattern
of the payload bytes is a valid code), activations are N(0,1). Block layouts follow the
reference's geometry table (src/gguf/qtype.c:15-104) and its decoders' field offsets
(src/gguf/quant_block.c:715-767, :819-833).
"""
from __future__ import annotations

import numpy as np

F32, F16, Q8_0, Q2_K, Q4_K, IQ2_XXS, I32, BF16, MXFP4 = 0, 1, 8, 10, 12, 16, 26, 30, 39

# qtype -> (elements per block, bytes per block, byte offsets of the f16 scale fields)
BLOCKS = {
    Q8_0: (32, 34, (0,)),
    Q2_K: (256, 84, (80, 82)),
    Q4_K: (256, 144, (0, 2)),
    IQ2_XXS: (256, 66, (0,)),
    MXFP4: (32, 17, ()),                # byte 0 is an E8M0 exponent, not an f16 scale: see random_blocks
}
SCALAR_BYTES = {F32: 4, F16: 2, BF16: 2, I32: 4}
BASE_SEED = 0x5EED0000


def row_bytes(qtype: int, width: int) -> int:
    if qtype in SCALAR_BYTES:
        return width * SCALAR_BYTES[qtype]
    elems, nbytes, _ = BLOCKS[qtype]
    if width % elems:
        raise ValueError(f"row width {width} is not a multiple of the {elems}-element block")
    return width // elems * nbytes


def random_blocks(qtype: int, rows: int, width: int, seed: int, lo: float = 1e-4,
                  hi: float = 1e-3) -> np.ndarray:
    """uint8 [rows, row_bytes]: uniform random payload bytes, f16 scales uniform in [lo, hi]."""
    elems, nbytes, scale_at = BLOCKS[qtype]
    rng = np.random.default_rng(seed)
    nblk = rows * (width // elems)
    raw = rng.integers(0, 256, size=(nblk, nbytes), dtype=np.uint8)
    for off in scale_at:
        d = rng.uniform(lo, hi, size=nblk).astype(np.float16)
        raw[:, off:off + 2] = d.view(np.uint8).reshape(nblk, 2)
    if qtype == MXFP4:
        raw[:, 0] = rng.integers(110, 124, size=nblk, dtype=np.uint8)      # scales 2^-17 .. 2^-4 (0xff would be NaN)
    return raw.reshape(rows, -1)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 -> f32 (finite inputs), as src/gguf/quant_scalar.c:130-143."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lower = bits & 0xFFFF
    upper = bits >> 16
    upper = upper + ((lower > 0x8000) | ((lower == 0x8000) & ((upper & 1) == 1)))
    return (upper.astype(np.uint32) << 16).view(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


class MoELayerSpec:
    """Geometry + policy constants of one synthetic DeepSeek-style MoE FFN layer."""

    def __init__(self, hidden, experts, topk, inter, shared_inter=None, gate_qtype=IQ2_XXS,
                 down_qtype=Q4_K, scaling=1.5, limit=10.0, normalize=1):
        self.hidden, self.experts, self.topk, self.inter = hidden, experts, topk, inter
        self.shared_inter = inter if shared_inter is None else shared_inter
        self.gate_qtype = self.up_qtype = gate_qtype
        self.down_qtype = down_qtype
        self.scaling, self.limit, self.normalize = scaling, limit, normalize

    def weight_bytes_per_expert(self):
        return (2 * self.inter * row_bytes(self.gate_qtype, self.hidden)
                + self.hidden * row_bytes(self.down_qtype, self.inter))


def moe_weights(spec: MoELayerSpec, seed: int, experts=None) -> dict:
    """Host copies of the expert-major packs. `experts` limits the routed pack to a subset of
    expert ids (others are left zero-filled) so small parity cases need not build 64+ experts."""
    H, I, E = spec.hidden, spec.inter, spec.experts
    out = {}
    ids = range(E) if experts is None else sorted(set(experts))
    grb, drb = row_bytes(spec.gate_qtype, H), row_bytes(spec.down_qtype, I)
    gate = np.zeros((E, I, grb), np.uint8)
    up = np.zeros((E, I, grb), np.uint8)
    down = np.zeros((E, H, drb), np.uint8)
    for e in ids:
        gate[e] = random_blocks(spec.gate_qtype, I, H, seed * 1000003 + 3 * e)
        up[e] = random_blocks(spec.up_qtype, I, H, seed * 1000003 + 3 * e + 1)
        down[e] = random_blocks(spec.down_qtype, H, I, seed * 1000003 + 3 * e + 2)
    out["gate"], out["up"], out["down"] = gate, up, down
    Is = spec.shared_inter
    out["shared_gate"] = random_blocks(spec.gate_qtype, Is, H, seed * 1000003 + 900001)
    out["shared_up"] = random_blocks(spec.up_qtype, Is, H, seed * 1000003 + 900002)
    out["shared_down"] = random_blocks(spec.down_qtype, H, Is, seed * 1000003 + 900003)
    return out
