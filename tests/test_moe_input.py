"""The reader of the reference's external MoE input fixtures (*.yvex-moe-input), on the CPU: a fixture
sealed and written by the reference itself (frozen in tests/golden/) must be admitted with the
reference's field values, and the malformed variants the reference's own format test builds
(tests/unit/runtime_moe.c:259-326) must be refused with its error codes."""
import ctypes as C
import hashlib
import os
import struct

import numpy as np
import pytest

from golden_cases import moe_input_case, moe_input_image


@pytest.fixture(scope="module")
def B():
    from yvex_b200 import build
    build.build()
    from yvex_b200 import backend
    return backend


def open_image(B, image):
    handle, err = B.vp(), B.Error()
    buf = (C.c_ubyte * len(image)).from_buffer_copy(image)
    rc = B._lib.yvex_moe_input_open_image(C.byref(handle), buf, len(image), C.byref(err))
    return rc, handle, err


def reseal(image):
    """Recomputes the two payload digests and the input identity of a (modified) image the way the format defines them."""
    b = bytearray(image)
    schema, start, tokens, layers, act_bytes, tok_bytes = struct.unpack_from("<6Q", b, 16)
    rec0, act0 = 512, 512 + 112 * layers
    tok0 = act0 + act_bytes
    b[64 + 64 * 4:64 + 64 * 5] = hashlib.sha256(bytes(b[act0:tok0])).hexdigest().encode()
    b[64 + 64 * 5:64 + 64 * 6] = hashlib.sha256(bytes(b[tok0:tok0 + tok_bytes])).hexdigest().encode()
    h = hashlib.sha256()
    text = lambda t: h.update(struct.pack("<Q", len(t)) + t)
    text(b"yvex.runtime.moe-input.v1")
    h.update(struct.pack("<6Q", schema, start, tokens, layers, act_bytes, tok_bytes))
    for i in range(6):
        text(bytes(b[64 + 64 * i:128 + 64 * i]))
    for i in range(layers):
        r = rec0 + 112 * i
        h.update(bytes(b[r:r + 48]))
        text(bytes(b[r + 48:r + 112]))
    b[64 + 64 * 6:64 + 64 * 7] = h.hexdigest().encode()
    return bytes(b)


def test_reference_written_fixture_is_admitted(B, golden):
    image = golden["moe_input_image"].tobytes()
    start, widths, acts, tids = moe_input_case()
    assert reseal(image) == image                          # the identity arithmetic restated above is the reference's
    rc, h, err = open_image(B, image)
    assert rc == B.OK, err.message
    s = B._lib.yvex_moe_input_summary_get(h).contents
    assert (s.schema_version, s.token_start, s.token_count, s.layer_count) == (1, start, len(tids), len(widths))
    assert s.activation_payload_bytes == acts.nbytes and s.token_id_payload_bytes == tids.nbytes
    assert s.logical_model_identity == b"1" * 64 and s.activation_payload_digest == hashlib.sha256(acts.tobytes()).hexdigest().encode()
    offset = 0
    for i, w in enumerate(widths):
        r = B._lib.yvex_moe_input_layer_record_at(h, i).contents
        assert (r.ordinal, r.layer_index, r.width, r.stride, r.payload_offset, r.payload_bytes) == (i, 3 * i + 1, w, w, offset, 4 * w * len(tids))
        view, stride = C.POINTER(C.c_float)(), B.ull()
        assert B._lib.yvex_moe_input_layer_view(h, i, C.byref(view), C.byref(stride), C.byref(err)) == B.OK and stride.value == w
        got = np.ctypeslib.as_array(view, shape=(len(tids) * w,))
        assert (got.view(np.uint32) == acts[offset // 4:offset // 4 + len(tids) * w].view(np.uint32)).all()
        offset += 4 * w * len(tids)
    assert [B._lib.yvex_moe_input_token_ids(h)[i] for i in range(len(tids))] == tids.tolist()
    view, stride = C.POINTER(C.c_float)(), B.ull()
    assert B._lib.yvex_moe_input_layer_view(h, 2, C.byref(view), C.byref(stride), C.byref(err)) == B.BOUNDS
    batch = B.RowBatch()
    assert B._lib.yvex_moe_input_row_batch(h, 1, C.byref(batch), C.byref(err)) == B.OK
    assert (batch.row_count, batch.row_width, batch.row_stride, batch.token_ids_present) == (len(tids), widths[1], widths[1], 1)
    B._lib.yvex_moe_input_close(C.byref(h))
    B._lib.yvex_moe_input_close(C.byref(h))                # closing twice is harmless, as in the reference
    assert not h.value


def test_test_writer_reproduces_the_reference_image(golden):
    start, widths, acts, tids = moe_input_case()
    ours = bytearray(moe_input_image(start, widths, acts, tids))
    ref = golden["moe_input_image"].tobytes()
    # the layer identity text is free-form hex: take the reference's, then every other byte must agree
    for i in range(len(widths)):
        ours[512 + 112 * i + 48:512 + 112 * (i + 1)] = ref[512 + 112 * i + 48:512 + 112 * (i + 1)]
    assert reseal(bytes(ours)) == ref


def test_malformed_fixtures_are_refused_with_the_reference_codes(B, golden, tmp_path):
    image = golden["moe_input_image"].tobytes()
    FORMAT, BOUNDS, IO = B.FORMAT, B.BOUNDS, -3
    bad = lambda img: open_image(B, img)[0]
    assert bad(image + b"\x00") == FORMAT                                   # trailing bytes
    assert bad(image[:-1]) == BOUNDS                                      # truncated
    assert bad(b"X" + image[1:]) == FORMAT                                # magic
    flipped = bytearray(image)
    flipped[512 + 112 * 2 + 5] ^= 0x40                                    # one activation bit: digest mismatch
    assert bad(bytes(flipped)) == FORMAT
    # the variants below are re-sealed, so only the structural rule can refuse them
    reordered = bytearray(image)
    struct.pack_into("<Q", reordered, 512 + 112, 0)                       # second record claims ordinal 0
    assert bad(reseal(bytes(reordered))) == FORMAT
    duplicate = bytearray(image)
    struct.pack_into("<Q", duplicate, 512 + 112 + 8, 1)                   # both records name layer 1
    assert bad(reseal(bytes(duplicate))) == FORMAT
    nan = bytearray(image)
    struct.pack_into("<f", nan, 512 + 112 * 2 + 12, float("nan"))
    assert bad(reseal(bytes(nan))) == FORMAT
    stride = bytearray(image)
    struct.pack_into("<Q", stride, 512 + 24, 5)                           # stride != width
    assert bad(reseal(bytes(stride))) == FORMAT
    assert bad(reseal(image)) == B.OK
    # files: a regular file within its bound is admitted, a symbolic link and an oversized file are not
    path = tmp_path / "input.yvex-moe-input"
    path.write_bytes(image)
    handle, err = B.vp(), B.Error()
    limits = B.MoeInputLimits(64 * 1024)
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(path).encode(), C.byref(limits), C.byref(err)) == B.OK, err.message
    B._lib.yvex_moe_input_close(C.byref(handle))
    link = tmp_path / "link.yvex-moe-input"
    os.symlink(path, link)
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(link).encode(), C.byref(limits), C.byref(err)) == IO
    small = B.MoeInputLimits(100)
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(path).encode(), C.byref(small), C.byref(err)) == BOUNDS
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(tmp_path / "absent").encode(), C.byref(limits), C.byref(err)) == IO
    assert B._lib.yvex_moe_input_open_file(C.byref(handle), str(path).encode(), None, C.byref(err)) == B.INVALID_ARG
