"""The allocation-free flash-decoding entry point against the one that takes caller scratch.

Collected last on purpose (file name): the built-in scratch array is shared by
every call on the device and keeps its last contents, so the test must pass
both alone and after everything else has run in the same process.
"""

import ctypes as C
import math

import pytest
import torch

from machete_b200 import _native as N

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


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


def _no_alloc(q, k, v, S):
    B, M, H, D = q.shape
    Nkv, Hkv = k.shape[1], k.shape[2]
    o = torch.full_like(q, float("nan"))
    lse = torch.empty(B, H, M, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = N.lib().mk_flash_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                         B, M, H, Hkv, D, Nkv, S, 0, C.c_float(1.0 / math.sqrt(D)), None)
    N.check(rc, "mk_flash_decode_noalloc")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before       # nothing came from torch's allocator either
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
