"""ctypes front-ends for the two CPU checkers (test infrastructure; never imported by the package).

`Port`  -> oracle/libyvex_oracle.so  this repository's plain-C restatement (always available:
           built from source by `make -C oracle port`).
`Ref`   -> oracle/_ref/libyvex_ref.so the unmodified reference sources + oracle/ref_harness.c
           (present only where it was built next to a reference checkout).
Both expose the same Python methods so a test can run the same case through either.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ORACLE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(ORACLE)
u64, u32, f32p = C.c_uint64, C.c_uint32, C.POINTER(C.c_float)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class _Layer(C.Structure):
    _fields_ = [("hidden", u64), ("experts", u64), ("topk", u64), ("inter", u64),
                ("shared_inter", u64), ("scaling", C.c_double), ("limit", C.c_double),
                ("normalize", C.c_int), ("router_class", C.c_int),
                ("gate_qtype", C.c_uint), ("up_qtype", C.c_uint), ("down_qtype", C.c_uint),
                ("router", C.c_void_p), ("bias", C.c_void_p), ("hash_table", C.c_void_p),
                ("hash_rows", u64), ("hash_stored_rows", u64),
                ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p),
                ("shared_down", C.c_void_p), ("allow_q4k", C.c_int)]


class _Mhc(C.Structure):
    _fields_ = [("hidden", u64), ("streams", u64), ("sinkhorn_iterations", u64), ("rms_epsilon", C.c_double),
                ("mhc_epsilon", C.c_double), ("post_multiplier", C.c_double), ("mhc_fn", C.c_void_p),
                ("scale", C.c_void_p), ("base", C.c_void_p), ("norm", C.c_void_p)]


class _Base:
    prefix = ""
    takes_allow = False

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self._keep = []

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def _allow(self, allow):
        return (int(allow),) if self.takes_allow else ()

    # -- layer description -------------------------------------------------------------------
    def layer(self, spec, weights, router=None, bias=None, hash_table=None, hash_rows=0,
              router_class=1, allow_q4k=False):
        L = _Layer()
        L.hidden, L.experts, L.topk, L.inter = spec.hidden, spec.experts, spec.topk, spec.inter
        L.shared_inter, L.scaling, L.limit = spec.shared_inter, spec.scaling, spec.limit
        L.normalize, L.router_class = spec.normalize, router_class
        L.gate_qtype, L.up_qtype, L.down_qtype = spec.gate_qtype, spec.up_qtype, spec.down_qtype
        keep = [router, bias, hash_table] + list(weights.values())
        L.router, L.bias, L.hash_table = _ptr(router), _ptr(bias), _ptr(hash_table)
        L.hash_rows = hash_rows
        L.hash_stored_rows = 0 if hash_table is None else hash_table.reshape(-1, spec.topk).shape[0]
        for k in ("gate", "up", "down", "shared_gate", "shared_up", "shared_down"):
            setattr(L, k, _ptr(weights.get(k)))
        L.allow_q4k = int(allow_q4k)
        L._keep = keep
        return L

    # -- mHC envelope of the MoE FFN ---------------------------------------------------------
    def mhc(self, hidden, streams, mhc_fn, scale, base, norm, sinkhorn_iterations=20, rms_epsilon=1e-6,
            mhc_epsilon=1e-6, post_multiplier=2.0):
        M = _Mhc(hidden, streams, sinkhorn_iterations, rms_epsilon, mhc_epsilon, post_multiplier)
        arrays = [np.ascontiguousarray(a, np.float32) for a in (mhc_fn, scale, base, norm)]
        M.mhc_fn, M.scale, M.base, M.norm = (_ptr(a) for a in arrays)
        M._keep = arrays
        return M

    def mhc_prepare(self, M, expanded):
        expanded = np.ascontiguousarray(expanded, np.float32)
        normalized = np.zeros(M.hidden, np.float32)
        post = np.zeros(M.streams, np.float32)
        combination = np.zeros(M.streams * M.streams, np.float32)
        rc = self._fn("mhc_prepare")(C.byref(M), _ptr(expanded), _ptr(normalized), _ptr(post), _ptr(combination))
        return rc, normalized, post, combination

    def mhc_post(self, M, core, expanded, post, combination):
        out = np.zeros(M.streams * M.hidden, np.float32)
        args = [np.ascontiguousarray(a, np.float32) for a in (core, expanded, post, combination)]
        rc = self._fn("mhc_post")(C.byref(M), *[_ptr(a) for a in args], _ptr(out))
        return rc, out

    # -- codecs ------------------------------------------------------------------------------
    def decode_rows(self, qtype, encoded, rows, width, allow_q4k=False):
        out = np.empty((rows, width), np.float32)
        rc = self._fn("decode_rows")(C.c_uint(qtype), _ptr(encoded), u64(rows), u64(width),
                                     _ptr(out), *self._allow(allow_q4k))
        return rc, out

    def decode_block(self, qtype, block, elements, allow_q4k=False):
        out = np.zeros(max(int(elements), 1), np.float32)
        rc = self._fn("decode_block")(C.c_uint(qtype), _ptr(block), C.c_size_t(block.size),
                                      _ptr(out), C.c_size_t(elements) if self.takes_allow
                                      else u64(elements), *self._allow(allow_q4k))
        return rc, out

    def matvec(self, qtype, encoded, rows, width, x, threads=1, allow_q4k=False):
        y = np.zeros(rows, np.float32)
        x = np.ascontiguousarray(x, np.float32)
        rc = self._fn("matvec")(C.c_uint(qtype), _ptr(encoded), u64(rows), u64(width), _ptr(x),
                                _ptr(y), C.c_int(threads), *self._allow(allow_q4k))
        return rc, y

    def route(self, L, x_or_logits, token_id=0, token_present=1):
        sel = np.zeros(L.topk, np.uint64)
        w = np.zeros(L.topk, np.float32)
        logits = np.zeros(L.experts, np.float32)
        scores = np.zeros(L.experts, np.float32)
        v = np.ascontiguousarray(x_or_logits, np.float32)
        rc = self._fn("route")(C.byref(L), _ptr(v), u32(token_id), C.c_int(token_present),
                               _ptr(sel), _ptr(w), _ptr(logits), _ptr(scores))
        return rc, sel, w, logits, scores

    def expert(self, H, I, limit, gq, uq, dq, gate, up, down, x, weight, allow_q4k=False):
        out = np.zeros(H, np.float32)
        x = np.ascontiguousarray(x, np.float32)
        rc = self._fn("expert")(u64(H), u64(I), C.c_double(limit), C.c_uint(gq), C.c_uint(uq),
                                C.c_uint(dq), _ptr(gate), _ptr(up), _ptr(down), _ptr(x),
                                C.c_float(weight), _ptr(out), *self._allow(allow_q4k))
        return rc, out

    def moe_tokens(self, L, x, logits=None, token_ids=None, threads=1):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, L.hidden)
        T = x.shape[0]
        out = np.zeros((T, L.hidden), np.float32)
        sel = np.zeros((T, L.topk), np.uint64)
        w = np.zeros((T, L.topk), np.float32)
        lg = None if logits is None else np.ascontiguousarray(logits, np.float32)
        ids = None if token_ids is None else np.ascontiguousarray(token_ids, np.uint32)
        rc = self._fn("moe_tokens")(C.byref(L), u64(T), _ptr(x), _ptr(lg), _ptr(ids), _ptr(out),
                                    _ptr(sel), _ptr(w), C.c_int(threads))
        return rc, out, sel, w

    def attention_head(self, q, k, v, position, scale, causal=1):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        out = np.zeros(q.shape[0], np.float32)
        rc = self._fn("attention_head")(_ptr(q), _ptr(k), _ptr(v), u64(k.shape[0]),
                                        u64(q.shape[0]), u64(position), C.c_float(scale),
                                        C.c_int(causal), _ptr(out))
        return rc, out


class Port(_Base):
    prefix = "oq_"
    takes_allow = True

    def __init__(self):
        path = os.path.join(ORACLE, "libyvex_oracle.so")
        src = os.path.join(ORACLE, "yvex_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            subprocess.check_call(["make", "-s", "-C", ORACLE, "port"])
        super().__init__(path)
        for n in ("f16_decode", "bf16_decode", "bf16_round"):
            getattr(self.lib, "oq_" + n).restype = C.c_float
        self.lib.oq_bf16_encode.restype = C.c_uint16
        self.lib.oq_bf16_encode.argtypes = [C.c_float]
        self.lib.oq_f16_decode.argtypes = [C.c_uint16]

    def geometry(self, qtype):
        e, b = C.c_uint(), C.c_uint()
        ok = self.lib.oq_geometry(C.c_uint(qtype), C.byref(e), C.byref(b))
        return (e.value, b.value) if ok else None

    def capability(self, qtype, allow_q4k=False):
        return self.lib.oq_capability(C.c_uint(qtype), C.c_int(int(allow_q4k)))

    def f16_decode(self, bits):
        return self.lib.oq_f16_decode(C.c_uint16(bits))

    def bf16_encode(self, v):
        return self.lib.oq_bf16_encode(C.c_float(v))

    def worklist(self, selected, experts):
        selected = np.ascontiguousarray(selected, np.uint64)
        rows, topk = selected.shape
        pairs = rows * topk
        order = np.zeros(pairs, np.uint32)
        src = np.zeros(pairs, np.uint32)
        be = np.zeros(experts, np.uint32)
        bo = np.zeros(experts + 1, np.uint32)
        bc = np.zeros(experts, np.uint32)
        n = u32()
        rc = self.lib.oq_worklist(_ptr(selected), u64(rows), u64(topk), u64(experts), _ptr(order),
                                  _ptr(src), _ptr(be), _ptr(bo), _ptr(bc), C.byref(n))
        return rc, order, src, be[:n.value], bo[:n.value + 1], bc[:n.value]

    def attention_gqa_decode(self, q, k, v, position, scale, threads=1):
        """q [S, Hq, D], k/v [S, Hkv, ctx, D] as uint16 bf16 bit patterns."""
        S, Hq, D = q.shape
        _, Hkv, ctx, _ = k.shape
        out = np.zeros((S, Hq, D), np.float32)
        rc = self.lib.oq_attention_gqa_decode(_ptr(q), _ptr(k), _ptr(v), u64(S), u64(Hq),
                                              u64(Hkv), u64(ctx), u64(D), u64(position),
                                              C.c_float(scale), _ptr(out), C.c_int(threads))
        return rc, out


class Ref(_Base):
    prefix = "ref_"
    takes_allow = False
    PATH = os.path.join(ORACLE, "_ref", "libyvex_ref.so")

    def __init__(self):
        super().__init__(self.PATH)
        self.lib.ref_f16_decode.restype = C.c_float
        self.lib.ref_f16_decode.argtypes = [C.c_uint16]
        self.lib.ref_bf16_encode.restype = C.c_uint16
        self.lib.ref_bf16_encode.argtypes = [C.c_float]

    @classmethod
    def available(cls):
        return os.path.exists(cls.PATH)

    def geometry(self, qtype):
        e, b = u64(), u64()
        rc = self.lib.ref_qtype_geometry(C.c_uint(qtype), C.byref(e), C.byref(b))
        return (e.value, b.value) if rc == 0 else None

    def capability(self, qtype, allow_q4k=False):
        return self.lib.ref_qtype_capability(C.c_uint(qtype))

    def f16_decode(self, bits):
        return self.lib.ref_f16_decode(C.c_uint16(bits))

    def bf16_encode(self, v):
        return self.lib.ref_bf16_encode(C.c_float(v))


def ref_moe_input_image(ref, token_start, widths, activations, token_ids):
    """A fixture file image sealed and written by the reference (Ref instance): bytes."""
    import tempfile
    tokens, layers = len(token_ids), len(widths)
    acts = np.ascontiguousarray(activations, np.float32)
    tids = np.ascontiguousarray(token_ids, np.uint32)
    w = (C.c_ulonglong * layers)(*widths)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "fixture.yvex-moe-input")
        ref.lib.ref_moe_input_write.argtypes = [C.c_char_p, C.c_ulonglong, C.c_ulonglong, C.c_ulonglong, C.c_void_p,
                                                C.c_void_p, C.c_void_p]
        rc = ref.lib.ref_moe_input_write(path.encode(), token_start, tokens, layers, w, acts.ctypes.data, tids.ctypes.data)
        if rc != 0:
            raise RuntimeError(f"reference refused the fixture: {rc}")
        return open(path, "rb").read()


def q8k_round_trip(x):
    """The values the reference's Q8_K activation path multiplies by, as its own test restates them
    (tests/unit/cuda/quant_qtype.c:161-186; device quantiser src/backend/cuda/kernels.cu:436-489): per 256
    values the FIRST element of largest magnitude gives inverse = -127 / value, every value becomes
    nearbyint(inverse * x) clamped to [-128, 127], divided by inverse. All arithmetic in float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    blocks = x.reshape(-1, 256)
    at = np.argmax(np.abs(blocks), axis=1)                      # first maximum
    peak = blocks[np.arange(blocks.shape[0]), at]
    out = np.zeros_like(blocks)
    live = np.abs(peak) > 0
    with np.errstate(divide="ignore", invalid="ignore"):
        inverse = np.where(live, np.float32(-127.0) / peak, np.float32(0)).astype(np.float32)
        q = np.clip(np.rint(inverse[:, None] * blocks), -128, 127).astype(np.int32).astype(np.float32)     # an int: no -0
        out[live] = (q[live] / inverse[live, None]).astype(np.float32)
    return out.reshape(x.shape)


def sink_attention(query, rows, sinks, scale, round_bf16=True):
    """The sink reducer of the reference's graph attention op for one token, restated (reduce_head,
    src/graph/core.c:428-465, with reduce_visit_row, :318-345; the rotary step that follows it there is left
    out): per head, pass 1 takes the maximum of the head's sink and every f64 score q . row * scale, pass 2
    seeds the denominator with exp(sink - max) and walks the rows in order, adding exp(score - max) to the
    denominator and (float)(p * row[lane]) to an f32 destination; the destination is divided by the
    denominator in double, narrowed to f32 and rounded to bf16 (the compute contract's rounding).
    Parity unpinned: the function is static inside the attention op and no fixture of the reference isolates it."""
    from yvex_b200 import synth
    query = np.ascontiguousarray(query, np.float32)
    rows = np.ascontiguousarray(rows, np.float32)
    out = np.zeros_like(query)
    for h in range(query.shape[0]):
        scores = (rows.astype(np.float64) @ query[h].astype(np.float64)) * float(scale)
        maximum = max(float(sinks[h]), float(scores.max())) if len(scores) else float(sinks[h])
        denominator = np.exp(float(sinks[h]) - maximum)
        dest = np.zeros(query.shape[1], np.float32)
        for i in range(rows.shape[0]):
            p = np.exp(scores[i] - maximum)
            denominator += p
            dest += (p * rows[i].astype(np.float64)).astype(np.float32)
        out[h] = (dest.astype(np.float64) / denominator).astype(np.float32)
    return synth.bf16_round(out) if round_bf16 else out
