"""GQA decode attention through the entry point that uses the library's fixed device scratch array
instead of a caller workspace (yvex_b200_attention_gqa_decode_static). Collected last on purpose:
it must pass both alone and after every other GPU test has used the device.

The calls go straight through the C ABI; all buffers are created before the calls under test, and
the results are compared bit-for-bit with the ordinary entry point (same kernels, different
scratch) on two calls in a row, so stale contents of the array from the first call cannot leak
into the second."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from yvex_b200 import lib
    return lib


def _inputs(torch, sessions, q_heads, kv_heads, dim, context, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    q = torch.randn((sessions, q_heads, dim), device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn((sessions, kv_heads, context, dim), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((sessions, kv_heads, context, dim), device="cuda", generator=g).to(torch.bfloat16)
    return q, k, v


def _run_static(L, torch, q, k, v, position, scale, status, out):
    S, Hq, D = q.shape
    _, Hkv, ctx, _ = k.shape
    return L.lib.yvex_b200_attention_gqa_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), S, Hq, Hkv, D, ctx,
                                                       position, scale, out.data_ptr(), status.word.data_ptr(),
                                                       torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_workspace_entry_twice_in_a_row(L):
    import torch
    assert L.lib.yvex_b200_attention_static_scratch_bytes() == 8 << 20
    status = L.Status()
    # two different problems back to back: the second is smaller and uses a different split count,
    # so it would read leftovers of the first if any slot were consumed without being written
    cases = [(4, 32, 8, 128, 4096, 4095, 11), (2, 8, 8, 64, 1500, 777, 12)]
    prepared = []
    for (S, Hq, Hkv, D, ctx, pos, seed) in cases:
        q, k, v = _inputs(torch, S, Hq, Hkv, D, ctx, seed)
        want = L.attention_gqa_decode(q, k, v, pos, D ** -0.5, status)
        out = torch.full((S, Hq, D), float("nan"), dtype=torch.float32, device="cuda")
        prepared.append((q, k, v, pos, D ** -0.5, want, out))
    torch.cuda.synchronize()
    for (q, k, v, pos, scale, want, out) in prepared:
        assert _run_static(L, torch, q, k, v, pos, scale, status, out) == 0
    torch.cuda.synchronize()
    assert status.read() == 0
    for (_, _, _, _, _, want, out) in prepared:
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
    # and once more in the opposite order; the set-up call is behind us, so these calls must leave the
    # device's free memory and the tensor library's own pool exactly as they found them
    for (_, _, _, _, _, _, out) in prepared:
        out.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    pool_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for (q, k, v, pos, scale, want, out) in reversed(prepared):
        assert _run_static(L, torch, q, k, v, pos, scale, status, out) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == pool_before
    for (_, _, _, _, _, want, out) in prepared:
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))
    assert status.read() == 0


def test_static_scratch_refuses_oversized_and_bad_arguments(L):
    import torch
    status = L.Status()
    q, k, v = _inputs(torch, 1, 4, 1, 128, 64, 13)
    out = torch.zeros((1, 4, 128), dtype=torch.float32, device="cuda")
    dummy = C.c_void_p(0x1000)
    # partials of 4096 sessions x 64 heads x many splits exceed 8 MiB: refused before any launch,
    # so the dummy pointers are never dereferenced
    before = L.lib.yvex_b200_launch_count()
    rc = L.lib.yvex_b200_attention_gqa_decode_static(dummy, dummy, dummy, 4096, 64, 64, 128, 32768, 32767, 0.1,
                                                     dummy, dummy, None)
    assert rc == -7
    assert L.lib.yvex_b200_attention_gqa_decode_static(dummy, dummy, dummy, 1, 4, 1, 128, 64, 64, 0.1, dummy, dummy,
                                                       None) == -7           # position outside the context
    assert L.lib.yvex_b200_attention_gqa_decode_static(dummy, dummy, dummy, 1, 4, 0, 128, 64, 3, 0.1, dummy, dummy,
                                                       None) == -10
    assert L.lib.yvex_b200_launch_count() == before
    # a bad scale is caught by the shared argument checks
    assert _run_static(L, torch, q, k, v, 3, -1.0, status, out) == -10
