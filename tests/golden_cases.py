"""Seeded small cases shared by the golden generator, the CPU oracle tests and the GPU parity
tests. Inputs are always rebuilt from these seeds; tests/golden/reference_vectors.npz stores only
the reference's outputs for them."""
import numpy as np

from yvex_b200 import synth

CASES = {
    # name: (qtype, rows, width, seed). Odd block counts give rows that start on 2-, 4- and
    # 8-byte boundaries, which the 128-bit load paths must survive.
    "matvec": {
        "iq2_xxs": (synth.IQ2_XXS, 64, 1024, 11),
        "iq2_xxs_ragged": (synth.IQ2_XXS, 37, 1792, 12),
        "q8_0": (synth.Q8_0, 64, 1024, 13),
        "q8_0_ragged": (synth.Q8_0, 19, 96, 14),
        "q2_k": (synth.Q2_K, 64, 1024, 15),
        "q2_k_ragged": (synth.Q2_K, 21, 768, 16),
    },
    # name: (hidden, experts, topk, inter, tokens, router: "weights"|"logits", seed)
    "layer": {
        "small_router": (512, 8, 2, 256, 4, "weights", 21),
        "small_logits": (256, 16, 4, 256, 6, "logits", 22),
        "c2_shape": (4096, 64, 6, 1536, 1, "weights", 23),
    },
    # name: (hidden, streams, tokens, seed): the mHC envelope around the FFN; "layer_small" wraps the
    # "small_router" layer above (same hidden width) end to end
    "envelope": {
        "small": (512, 4, 3, 41),
        "wide_hidden": (4096, 4, 2, 42),
        "two_streams": (768, 2, 2, 43),
    },
    # name: (sessions, q_heads, kv_heads, head_dim, context, position, seed)
    "attention": {
        "small": (2, 8, 2, 128, 512, 511, 31),
        "masked": (1, 4, 4, 64, 300, 123, 32),
    },
}


def layer_inputs(name, down_qtype=synth.Q2_K):
    """(spec, weights, router or None, x [tokens, hidden], logits or None) for a layer case.
    Only the experts a token routes to are materialised for the C2-sized case."""
    H, E, k, I, T, mode, seed = CASES["layer"][name]
    spec = synth.MoELayerSpec(H, E, k, I, down_qtype=down_qtype)
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = logits = None
    if mode == "weights":
        router = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
        lg = (synth.bf16_round(x).astype(np.float64) @ router.astype(np.float64).T)
    else:
        logits = rng.standard_normal((T, E)).astype(np.float32)
        lg = logits.astype(np.float64)
    needed = None
    if E * spec.weight_bytes_per_expert() > (64 << 20):
        # sqrt(softplus) is monotonic, zero bias: top-k of the logits are the selected experts;
        # take a margin so float ties cannot miss one.
        needed = set(np.argsort(-lg, axis=1)[:, :k + 2].ravel().tolist())
    weights = synth.moe_weights(spec, seed, experts=needed)
    return spec, weights, router, x, logits


def attention_inputs(name):
    """(q [S,Hq,D] f32, k/v [S,Hkv,ctx,D] f32 - all exactly bf16-representable - position, scale)"""
    S, Hq, Hkv, D, ctx, pos, seed = CASES["attention"][name]
    rng = np.random.default_rng(seed)
    q = synth.bf16_round(rng.standard_normal((S, Hq, D)).astype(np.float32))
    k = synth.bf16_round(rng.standard_normal((S, Hkv, ctx, D)).astype(np.float32))
    v = synth.bf16_round(rng.standard_normal((S, Hkv, ctx, D)).astype(np.float32))
    return q, k, v, pos, float(D) ** -0.5


ENVELOPE_POLICY = dict(sinkhorn_iterations=20, rms_epsilon=1e-6, mhc_epsilon=1e-6, post_multiplier=2.0)


def envelope_inputs(name):
    """(mhc_fn [(S+2)S, S*H], scale [3], base [(S+2)S], norm [H], expanded [T, S*H]) - all f32."""
    H, S, T, seed = CASES["envelope"][name]
    rng = np.random.default_rng(seed)
    rows = (S + 2) * S
    fn = (rng.standard_normal((rows, S * H)) * 0.05).astype(np.float32)
    scale = np.array([0.7, 1.3, 0.9], np.float32)
    base = (rng.standard_normal(rows) * 0.3).astype(np.float32)
    norm = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    expanded = rng.standard_normal((T, S * H)).astype(np.float32)
    return fn, scale, base, norm, expanded


def moe_input_case():
    """(token_start, widths per layer, activations (all layers back to back, [tokens x width] each), token ids)."""
    rng = np.random.default_rng(51)
    widths, tokens = [4, 6], 3
    acts = rng.standard_normal(tokens * sum(widths)).astype(np.float32)
    return 7, widths, acts, np.array([5, 19, 1000003], np.uint32)


def moe_input_image(token_start, widths, activations, token_ids, layer_indices=None):
    """Serializes an external MoE input fixture (the reference's *.yvex-moe-input layout, src/runtime/moe_input.c:226-277)
    with its SHA-256 payload digests and input identity. The frozen reference-written image in tests/golden/ pins this
    writer (tests/test_moe_input.py re-derives that image's identities with the same arithmetic)."""
    import hashlib
    import struct
    acts = np.ascontiguousarray(activations, np.float32).tobytes()
    tids = np.ascontiguousarray(token_ids, np.uint32).tobytes()
    tokens, layers = len(token_ids), len(widths)
    ids = [bytes([c]) * 64 for c in b"1234"]
    records, offset = b"", 0
    for i, w in enumerate(widths):
        nbytes = 4 * w * tokens
        records += struct.pack("<6Q", i, layer_indices[i] if layer_indices else 3 * i + 1, w, w, offset, nbytes) + b"ab" * 32
        offset += nbytes
    head = struct.pack("<6Q", 1, token_start, tokens, layers, len(acts), len(tids))
    digests = [hashlib.sha256(acts).hexdigest().encode(), hashlib.sha256(tids).hexdigest().encode()]
    h = hashlib.sha256()
    text = lambda t: h.update(struct.pack("<Q", len(t)) + t)
    text(b"yvex.runtime.moe-input.v1")
    h.update(head)
    for t in ids + digests:
        text(t)
    for i in range(layers):
        r = records[112 * i:112 * (i + 1)]
        h.update(r[:48])
        text(r[48:])
    return b"YVEXMOEINPUT001\0" + head + b"".join(ids + digests) + h.hexdigest().encode() + records + acts + tids
