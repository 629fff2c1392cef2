"""The tcgen05 prefill attention against an fp32 PyTorch attention of the same bf16 inputs.

Tolerance: the kernel rounds P to bf16 before P V (as every flash-attention forward does) and O once
more on the store; against an fp64 reference that is a few bf16 ulps of the output magnitude:
max-abs <= 2e-2 (the suite's bar; outputs are O(1)) and cosine >= 0.999."""

import math

import pytest
import torch

from machete_b200.kernels.attention import FlashAttentionSm100Op, flash_attention_schedule, flash_prefill
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _reference(q, k, v, causal):
    """q (B,H,M,D), k/v (B,Hkv,N,D) -> o (B,H,M,D), lse (B,H,M); the queries are the last M tokens."""
    B, H, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    g = H // Hkv
    kk = k.double().repeat_interleave(g, dim=1)
    vv = v.double().repeat_interleave(g, dim=1)
    s = q.double() @ kk.transpose(-1, -2) / math.sqrt(D)
    if causal:
        rows = torch.arange(M, device=q.device)[:, None] + (N - M)
        s = s.masked_fill(torch.arange(N, device=q.device)[None, :] > rows, float("-inf"))
    return torch.softmax(s, dim=-1) @ vv, torch.logsumexp(s, dim=-1)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,H,Hkv,M,N,causal", [(1, 4, 4, 128, 128, False), (1, 8, 2, 256, 256, True),
                                                 (2, 4, 1, 200, 333, True), (1, 2, 2, 1, 70, False),
                                                 (1, 4, 2, 129, 1000, False), (1, 32, 8, 512, 512, True)])
def test_prefill_matches_fp32_attention(D, B, H, Hkv, M, N, causal):
    g = torch.Generator(device="cuda").manual_seed(D + M + N)
    q = torch.randn(B, H, M, D, generator=g, device="cuda").to(BF)
    k = torch.randn(B, Hkv, N, D, generator=g, device="cuda").to(BF)
    v = torch.randn(B, Hkv, N, D, generator=g, device="cuda").to(BF)
    o = torch.full_like(q, 7.0)
    lse = torch.zeros(B, H, M, device="cuda")
    flash_prefill(q, k, v, o, causal=causal, lse=lse, check_status=True)
    want_o, want_lse = _reference(q, k, v, causal)
    assert_parity(o, want_o, f"prefill D={D} M={M} N={N} causal={causal}")
    assert float((lse.double() - want_lse).abs().max()) < 2e-3


def test_prefill_on_the_decode_layout_and_cache_views():
    """q / o (B, M, H, D) and K / V as views of a longer (B, T, Hkv, D) cache: what a prompt does."""
    B, T, H, Hkv, D, M = 2, 640, 8, 2, 64, 300
    g = torch.Generator(device="cuda").manual_seed(3)
    kc = torch.randn(B, T, Hkv, D, generator=g, device="cuda").to(BF)
    vc = torch.randn(B, T, Hkv, D, generator=g, device="cuda").to(BF)
    q = torch.randn(B, M, H, D, generator=g, device="cuda").to(BF)
    o = torch.zeros_like(q)
    flash_prefill(q, kc[:, :M], vc[:, :M], o, causal=True, layout="bmhd", check_status=True)
    want, _ = _reference(q.transpose(1, 2), kc[:, :M].transpose(1, 2), vc[:, :M].transpose(1, 2), True)
    assert_parity(o.transpose(1, 2), want, "prefill on cache views")


def test_op_mirror_and_dispatcher():
    q = torch.randn(1, 4, 256, 64, device="cuda").to(BF)
    k = torch.randn(1, 2, 256, 64, device="cuda").to(BF)
    v = torch.randn(1, 2, 256, 64, device="cuda").to(BF)
    o = torch.zeros_like(q)
    ops, cfg = flash_attention_schedule(q, k, v, o, causal=True, kv_group_size=2)
    assert cfg is None and ops[0].op_cls is FlashAttentionSm100Op and ops[0].tile_counts == (1, 4, 2, 1)
    FlashAttentionSm100Op.launch(ops[0], check_status=True)
    want, _ = _reference(q, k, v, True)
    assert_parity(o, want, "op mirror")
    with pytest.raises(NotImplementedError):
        FlashAttentionSm100Op.lower(ops[0], None)
    with pytest.raises(ValueError):
        flash_prefill(q, k, v, o[:, :, :, :32])
    with pytest.raises(ValueError):
        flash_prefill(q, k[:, :, :100], v[:, :, :100], o, causal=True)      # causal needs M <= N
