"""The CPU oracle against fixtures produced by the reference's own functions."""

from pathlib import Path

import pytest
import torch

import oracle

GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def cases():
    return torch.load(GOLD / "golden_ops.pt", weights_only=False)


def _run(c):
    op = c["op"]
    if op == "rmsnorm":
        return oracle.rmsnorm(c["x"], c["weight"], c["eps"], c["residual"], c["gemma"])
    if op == "fused_add_rmsnorm":
        return oracle.fused_add_rmsnorm(c["x"], c["residual_in"], c["weight"], c["eps"])
    if op == "rmsnorm_gated":
        return oracle.rmsnorm_gated(c["x"], c["gate"], c["weight"], c["eps"])
    if op == "rope":
        return oracle.rope(c["q"], c["cos"], c["sin"])
    if op == "qknorm_rope":
        return oracle.qknorm_rope(c["q"], c["norm_weight"], c["cos"], c["sin"], c["eps"])
    if op == "glu":
        return oracle.glu(c["x"], c["activation"])
    if op == "attention":
        return oracle.attention(c["q"], c["k"], c["v"], causal=c["causal"], kv_group_size=c["kv_group_size"])
    raise AssertionError(op)


def test_every_case_is_bit_identical(cases):
    assert len(cases) > 20
    for c in cases:
        got = _run(c)
        if c["op"] == "fused_add_rmsnorm":
            assert torch.equal(got[0], c["y"]) and torch.equal(got[1], c["residual_out"]), c["op"]
        else:
            assert got.dtype == c["y"].dtype and torch.equal(got, c["y"]), c["op"]


def test_bshd_wrapper_matches_flat_attention(cases):
    c = next(x for x in cases if x["op"] == "attention" and x["kv_group_size"] == 4 and not x["causal"])
    q, k, v = c["q"], c["k"], c["v"]          # (BH, M, D), (BHkv, N, D)
    H, Hkv = 8, 2
    q4 = q.view(1, H, q.shape[1], -1).permute(0, 2, 1, 3).contiguous()
    k4 = k.view(1, Hkv, k.shape[1], -1).permute(0, 2, 1, 3).contiguous()
    v4 = v.view(1, Hkv, v.shape[1], -1).permute(0, 2, 1, 3).contiguous()
    o = oracle.attention_bshd(q4, k4, v4)
    assert torch.equal(o.permute(0, 2, 1, 3).reshape(c["y"].shape), c["y"])


def test_split_partials_combine_to_full_attention():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(2, 1, 8, 64, generator=g).bfloat16()
    k = torch.randn(2, 300, 2, 64, generator=g).bfloat16()
    v = torch.randn(2, 300, 2, 64, generator=g).bfloat16()
    full = oracle.attention_bshd(q.float(), k.float(), v.float())
    bounds = [(0, 96), (96, 192), (192, 288), (288, 300), (300, 300)]   # ragged + an empty split
    op, lp = oracle.split_kv_partials(q, k, v, bounds)
    o, lse = oracle.combine_partials(op, lp)
    err, cos = oracle.parity_metrics(o, full)
    assert err < 1e-5 and cos > 0.999999
    assert torch.isinf(lp[:, :, 4]).all() and torch.isfinite(lse).all()


def test_nvfp4_quantiser_bit_exact():
    qcases = torch.load(GOLD / "golden_nvfp4.pt", weights_only=False)
    for c in qcases:
        packed, scales = oracle.quantize_nvfp4(c["weight"], c["group_size"])
        assert torch.equal(packed, c["packed"])
        assert torch.equal(scales, c["scales"])
        assert torch.equal(oracle.dequantize_nvfp4(packed, scales, c["group_size"]), c["dequant"])


def test_nvfp4_e4m3_layout_round_trip():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(16, 512, generator=g) * 0.02
    packed, scales, gs = oracle.quantize_nvfp4_e4m3(w)
    assert packed.shape == (16, 256) and scales.shape == (16, 32) and scales.dtype == torch.float8_e4m3fn
    deq = oracle.dequantize_nvfp4(packed, scales, 16, gs)
    # e2m1 has a 1-bit mantissa: worst relative step is 1/3 of the group amax spacing
    assert float((deq - w).abs().max()) <= float(w.abs().max()) * 0.26
    # idempotence: quantising the dequantised matrix reproduces the codes
    p2, s2, g2 = oracle.quantize_nvfp4_e4m3(deq)
    assert torch.equal(oracle.dequantize_nvfp4(p2, s2, 16, g2), deq)
