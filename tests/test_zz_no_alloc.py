"""The allocation-free flash-decoding entry point against the one that takes caller scratch.

Collected last on purpose (file name): the built-in scratch array is shared by
every call on the device and keeps its last contents, so the test must pass
both alone and after everything else has run in the same process.
"""

import ctypes as C
import math

import pytest
import torch

import oracle
from machete_b200 import _native as N
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
_FIRST_CALL_DONE = False


def _inputs(B, M, H, Hkv, D, Nkv, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, M, H, D, generator=g).to(BF).cuda()
    k = torch.randn(B, Nkv, Hkv, D, generator=g).to(BF).cuda()
    v = torch.randn(B, Nkv, Hkv, D, generator=g).to(BF).cuda()
    return q, k, v


def _with_scratch(q, k, v, S):
    B, M, H, D = q.shape
    Nkv, Hkv = k.shape[1], k.shape[2]
    o = torch.full_like(q, float("nan"))
    lse = torch.empty(B, H, M, device="cuda")
    op = torch.empty(B, H, S, M, D, device="cuda")
    lp = torch.empty(B, H, S, M, device="cuda")
    n = int(N.lib().mk_standalone_workspace_bytes())
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    rc = N.lib().mk_flash_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                 op.data_ptr(), lp.data_ptr(), B, M, H, Hkv, D, Nkv, S, 0,
                                 C.c_float(1.0 / math.sqrt(D)), ws.data_ptr(), n, None)
    N.check(rc, "mk_flash_decode")
    torch.cuda.synchronize()
    return o, lse


def _no_alloc(q, k, v, S, stream=None):
    B, M, H, D = q.shape
    Nkv, Hkv = k.shape[1], k.shape[2]
    o = torch.full_like(q, float("nan"))
    lse = torch.empty(B, H, M, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    rc = N.lib().mk_flash_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                         B, M, H, Hkv, D, Nkv, S, 0, C.c_float(1.0 / math.sqrt(D)),
                                         None if stream is None else C.c_void_p(stream.cuda_stream))
    N.check(rc, "mk_flash_decode_noalloc")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before       # nothing came from torch's allocator ...
    # ... nor from the driver: free device memory does not shrink.  (Not on the process's first call:
    # that one may make the runtime load the library's device image, which holds the scratch array.)
    global _FIRST_CALL_DONE
    if _FIRST_CALL_DONE:
        assert torch.cuda.mem_get_info()[0] >= free_before
    _FIRST_CALL_DONE = True
    st = (C.c_int32 * 16)()
    N.check(N.lib().mk_flash_decode_noalloc_status(st), "mk_flash_decode_noalloc_status")
    assert st[0] == 0, list(st)[:6]
    return o, lse


def test_two_calls_in_a_row_match_the_scratch_taking_entry_point():
    # two different shapes back to back: the second call finds the first one's leftovers in the scratch
    for (B, M, H, Hkv, D, Nkv, S, seed) in [(2, 1, 16, 4, 128, 777, 6, 9), (1, 1, 32, 8, 64, 2048, 9, 10)]:
        q, k, v = _inputs(B, M, H, Hkv, D, Nkv, seed)
        want_o, want_lse = _with_scratch(q, k, v, S)
        got_o, got_lse = _no_alloc(q, k, v, S)
        # same kernel, same split layout, same summation order: identical results
        assert torch.equal(got_o, want_o)
        assert torch.equal(got_lse, want_lse)
        assert torch.isfinite(got_o.float()).all()
        # and both agree with the oracle (the bar of every 16-bit result here: 2e-2 / cosine 0.999)
        assert_parity(got_o, oracle.attention_bshd(q.cpu().float(), k.cpu().float(), v.cpu().float()), "no-alloc flash decode")


def test_back_to_back_calls_on_a_side_stream_are_ordered_by_the_stream():
    """Two calls in a row on a stream that does not synchronise with the default stream, no host
    synchronisation in between: the second call's table uploads are queued behind the first
    call's kernel, so each call must still see its own program and produce its own result."""
    side = torch.cuda.Stream()
    cases = [(1, 1, 16, 4, 64, 1500, 8, 31), (2, 1, 8, 2, 128, 640, 5, 32)]
    ins = [_inputs(B, M, H, Hkv, D, Nkv, seed) for (B, M, H, Hkv, D, Nkv, S, seed) in cases]
    outs = [(torch.full_like(q, float("nan")), torch.empty(q.shape[0], q.shape[2], q.shape[1], device="cuda")) for q, _, _ in ins]
    torch.cuda.synchronize()
    for (B, M, H, Hkv, D, Nkv, S, _), (q, k, v), (o, lse) in zip(cases, ins, outs):
        rc = N.lib().mk_flash_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                             B, M, H, Hkv, D, Nkv, S, 0, C.c_float(1.0 / math.sqrt(D)),
                                             C.c_void_p(side.cuda_stream))
        N.check(rc, "mk_flash_decode_noalloc")
    side.synchronize()
    for (B, M, H, Hkv, D, Nkv, S, _), (q, k, v), (o, _lse) in zip(cases, ins, outs):
        want_o, _ = _with_scratch(q, k, v, S)
        assert torch.equal(o, want_o)


def test_oversized_request_is_refused_with_a_message():
    q, k, v = _inputs(1, 1, 8, 2, 64, 64, 0)
    o = torch.empty_like(q)
    lse = torch.empty(1, 8, 1, device="cuda")
    # 64 batches x 64 heads x 64 splits x 16 rows of head dim 128 is far beyond the 4 MiB of partials
    rc = N.lib().mk_flash_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                         64, 16, 64, 64, 128, 4096, 64, 0, C.c_float(0.1), None)
    assert rc != 0
    msg = N.last_error()
    assert "built-in" in msg and "mk_flash_decode" in msg
