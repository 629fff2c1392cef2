"""Split-KV flash decoding + combine on the GPU against the oracle attention."""

import math

import pytest
import torch

import oracle
from machete_b200 import _native as N
from machete_b200.kernels.attention import flash_decoding_schedule
from machete_b200.megakernel import Megakernel
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def qkv(B, M, H, Hkv, D, Nkv, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, M, H, D, generator=g).to(BF), torch.randn(B, Nkv, Hkv, D, generator=g).to(BF),
            torch.randn(B, Nkv, Hkv, D, generator=g).to(BF))


@pytest.mark.parametrize("B,M,H,Hkv,D,Nkv,splits,causal", [
    (1, 1, 8, 2, 64, 333, 3, False),        # ragged N, GQA 4:1
    (2, 1, 32, 8, 128, 1024, 5, False),     # config-2 head layout, small N
    (1, 1, 32, 8, 64, 4096, 0, False),      # llama-1B decode, default splits
    (1, 16, 8, 2, 128, 96, 2, True),        # the reference's padded M=16 contract, causal
    (2, 16, 4, 4, 64, 200, 4, False),       # MHA, M=16
    (1, 1, 4, 1, 64, 40, 2, False),         # more splits than 16-token blocks can fill: empty split
])
def test_flash_decoding_schedule(B, M, H, Hkv, D, Nkv, splits, causal):
    q, k, v = qkv(B, M, H, Hkv, D, Nkv)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full_like(qd, float("nan"))
    ops, _ = flash_decoding_schedule(qd, kd, vd, o, num_splits=splits, causal=causal, kv_group_size=H // Hkv)
    mk = Megakernel(ops)
    mk.run()
    want = oracle.attention_bshd(q.float(), k.float(), v.float(), causal=causal)
    assert_parity(o, want, f"flash decode B{B} M{M} H{H}/{Hkv} D{D} N{Nkv}")
    # partials follow the split contract: normalised o_partial and lse = max*scale + ln(sum)
    sp = mk.native_ops[0]
    S, ts = sp.i[N.AT_SPLITS], sp.i[N.AT_TS]
    bounds = [(min(Nkv, s * ts), min(Nkv, s * ts + ts)) for s in range(S)]
    op_w, lse_w = oracle.split_kv_partials(q, k, v, bounds, causal=causal)
    op_g = ops[0].tensor_refs["o_partial"].cpu()
    lse_g = ops[0].tensor_refs["lse_partial"].cpu()
    finite = torch.isfinite(lse_w)
    assert torch.equal(torch.isfinite(lse_g), finite)
    assert float((lse_g[finite] - lse_w[finite]).abs().max()) < 2e-2
    assert_parity(op_g, op_w, "o_partial")
    lse = ops[1].tensor_refs["lse"].cpu()
    _, lse_full = oracle.combine_partials(op_w, lse_w)
    assert float((lse - lse_full).abs().max()) < 2e-2
    assert (mk.read_counters() == 0).all()


def test_strided_cache_views():
    """k/v as windows of a larger cache with a batch stride, as the layer schedule passes them."""
    B, H, Hkv, D, T, Nkv = 2, 8, 2, 64, 512, 300
    g = torch.Generator().manual_seed(7)
    kc = torch.randn(B, T, Hkv, D, generator=g).to(BF).cuda()
    vc = torch.randn(B, T, Hkv, D, generator=g).to(BF).cuda()
    q = torch.randn(B, 1, H, D, generator=g).to(BF).cuda()
    o = torch.empty_like(q)
    ops, _ = flash_decoding_schedule(q, kc[:, :Nkv], vc[:, :Nkv], o, num_splits=4, kv_group_size=4)
    Megakernel(ops).run()
    want = oracle.attention_bshd(q.cpu().float(), kc[:, :Nkv].cpu().float(), vc[:, :Nkv].cpu().float())
    assert_parity(o, want, "strided cache window")


def test_standalone_flash_decode_abi():
    B, M, H, Hkv, D, Nkv, S = 2, 1, 16, 4, 128, 777, 6
    q, k, v = qkv(B, M, H, Hkv, D, Nkv, seed=9)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full_like(qd, float("nan"))
    lse = torch.empty(B, H, M, device="cuda")
    op = torch.empty(B, H, S, M, D, device="cuda")
    lp = torch.empty(B, H, S, M, device="cuda")
    n = int(N.lib().mk_standalone_workspace_bytes())
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    import ctypes as C
    rc = N.lib().mk_flash_decode(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                 op.data_ptr(), lp.data_ptr(), B, M, H, Hkv, D, Nkv, S, 0,
                                 C.c_float(1.0 / math.sqrt(D)), ws.data_ptr(), n, None)
    N.check(rc, "mk_flash_decode")
    torch.cuda.synchronize()
    assert_parity(o, oracle.attention_bshd(q.float(), k.float(), v.float()), "mk_flash_decode")


def test_linearity_in_v_at_full_size():
    """Size-independent property at the benchmark's head layout: attention is linear in V."""
    B, M, H, Hkv, D, Nkv = 2, 1, 32, 8, 128, 8192
    q, k, v1 = qkv(B, M, H, Hkv, D, Nkv, seed=11)
    v2 = torch.randn_like(v1.float()).to(BF)
    outs = []
    for vv in (v1, v2, (v1.float() + v2.float()).to(BF)):
        o = torch.empty(B, M, H, D, dtype=BF, device="cuda")
        ops, _ = flash_decoding_schedule(q.cuda(), k.cuda(), vv.cuda(), o, kv_group_size=4)
        Megakernel(ops).run()
        outs.append(o.float().cpu())
    assert_parity(outs[2], outs[0] + outs[1], "linearity in V", atol=3e-2)


@pytest.mark.parametrize("B,H,Hkv,D,Nkv,splits", [
    (1, 16, 4, 128, 700, 4),     # Qwen3 head layout
    (3, 8, 2, 64, 130, 0),       # head dim 64, several sequences, default splits
    (1, 4, 4, 128, 33, 1),       # one split, one query head per KV head: the unit is not shared
])
def test_fused_qk_norm(B, H, Hkv, D, Nkv, splits):
    """The attention op given UNROTATED q and an unrotated last k row applies the per-head RMSNorm and
    the rotation itself: same output as normalising first (the oracle's qknorm_rope), and the finished
    k row is what ends up in the cache."""
    g = torch.Generator().manual_seed(5)
    q, k, v = qkv(B, 1, H, Hkv, D, Nkv, seed=9)
    qw = (1 + torch.randn(D, generator=g) * 0.1).to(BF)
    kw = (1 + torch.randn(D, generator=g) * 0.1).to(BF)
    ang = torch.rand(D // 2, generator=g) * 6.28
    cos, sin = torch.cos(ang).to(BF), torch.sin(ang).to(BF)
    new = Nkv - 1
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full_like(qd, float("nan"))
    ops, _ = flash_decoding_schedule(qd, kd, vd, o, num_splits=splits, kv_group_size=H // Hkv,
                                     qk_norm=dict(q_weight=qw.cuda(), k_weight=kw.cuda(), cos=cos.cuda(), sin=sin.cuda(),
                                                  eps=1e-6, new_token=new))
    mk = Megakernel(ops)
    mk.run()
    qn = oracle.qknorm_rope(q, qw, cos[None], sin[None], 1e-6)
    kn = k.clone()
    kn[:, new:new + 1] = oracle.qknorm_rope(k[:, new:new + 1], kw, cos[None], sin[None], 1e-6)
    want = oracle.attention_bshd(qn.float(), kn.float(), v.float(), causal=False)
    assert_parity(o, want, f"fused q/k norm B{B} H{H}/{Hkv} D{D} N{Nkv}")
    # the cache: the new row finished (bf16 rounding of the rotation: one ulp), every other row untouched
    got_k = kd.cpu()
    assert torch.equal(got_k[:, :new], k[:, :new])
    assert float((got_k[:, new].float() - kn[:, new].float()).abs().max()) <= 2e-2
    first = o.clone()
    kd.copy_(k)                 # a decode step rewrites the raw row before every launch
    mk.run()
    assert torch.equal(first, o)
    assert (mk.read_counters() == 0).all()
