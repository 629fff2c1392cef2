"""Parity at the benchmark configurations' own sizes.

The other GPU test files cover every op and fusion at sizes the oracle finishes
in a blink; here the same kernels run at the shapes the measured configurations
use: the small-M GEMM sweep (bf16 and block-scaled NVFP4), flash decoding at
batch 8 x 32 768 tokens, one full 16-layer 128 256-vocabulary decode step, and
the 8B-shape NVFP4 layer width at batch 1 and 8.  The CPU oracle is chunked
where a whole fp32 copy would not be reasonable.
"""

import math

import pytest
import torch

import oracle
from machete_b200 import _native as N
from machete_b200.kernels.attention import flash_decoding_schedule
from machete_b200.kernels.decode_matvec import MatvecNvfp4Sm120Op
from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
from machete_b200.kernels.gemm import GemmOp
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.megakernel import Megakernel, OverlapTileScheduler
from machete_b200.quantization import dequantize_nvfp4_weight, quantize_nvfp4_weight
from tests.util import assert_greedy_token, assert_parity, llama_weights, to_cpu

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def seeded(M, O, K, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, K, generator=g).to(BF), (torch.randn(O, K, generator=g) * 0.02).to(BF)


# ---- small-M GEMM sweep: M in {1, 4, 16} x K = 4096 x N in {4096, 14336}, and 16 x 1024 x 1024 -------------
SWEEP = [(M, N_, 4096) for M in (1, 4, 16) for N_ in (4096, 14336)] + [(16, 1024, 1024)]


@pytest.mark.parametrize("M,Nout,K", SWEEP)
def test_small_m_gemm_sweep_bf16(M, Nout, K):
    x, w = seeded(M, Nout, K, seed=11)
    c = torch.full((1, M, Nout), float("nan"), dtype=BF, device="cuda")
    mk = Megakernel(GemmOp.schedule(a=x.view(1, M, K).cuda(), b=w.cuda(), c=c))
    mk.run()
    assert_parity(c.view(M, Nout), oracle.matvec(x, w), f"GemmOp bf16 {M}x{K}x{Nout}")
    assert (mk.read_counters() == 0).all()


@pytest.mark.parametrize("M,Nout,K", SWEEP)
def test_small_m_gemm_sweep_nvfp4_block_scaled(M, Nout, K):
    """e2m1 values, an e4m3 scale per 16-element K block, one fp32 global scale."""
    x, w = seeded(M, Nout, K, seed=12)
    q = quantize_nvfp4_weight(w, group_size=16)
    y = torch.full((1, M, Nout), float("nan"), dtype=BF, device="cuda")
    mk = Megakernel(MatvecNvfp4Sm120Op.schedule(a=x.view(1, M, K).cuda(), weight_packed=q.packed.cuda(),
                                                weight_scales=q.scales.cuda(), y=y, group_size=16,
                                                global_scale=q.global_scale))
    mk.run()
    assert_parity(y.view(M, Nout), x.float() @ dequantize_nvfp4_weight(q).t(), f"NVFP4 {M}x{K}x{Nout}")


# ---- device-side unpacking, exactly ------------------------------------------------------------------------
@pytest.mark.parametrize("group", [32, 16])
def test_device_unpack_is_exact(group):
    """One-hot activation rows and an fp32 output read the dequantised weights back one column at a
    time: no sum, no rounding of the result.  What the kernel multiplies by is the e2m1 value times
    its block scale formed in fp16 (exact for an e4m3 scale; rounded to fp16 for an fp16 scale),
    times the fp32 global scale; it must equal that bit for bit, and the host dequantiser (which
    folds scale and global scale first) to one fp32 ulp."""
    O, K = 48, 512
    g = torch.Generator().manual_seed(13)
    w = torch.randn(O, K, generator=g) * 0.02
    q = quantize_nvfp4_weight(w, group_size=group)
    codes = torch.stack([q.packed & 0xF, q.packed >> 4], dim=-1).reshape(O, K).long()
    vals = torch.where(codes >= 8, -E2M1[codes - 8], E2M1[codes.clamp(max=7)])
    block = q.scales.float().repeat_interleave(group, dim=1)
    exact = (vals * block).half().float() * torch.tensor(q.global_scale, dtype=torch.float32)
    got = torch.empty(K, O)
    pk, sc = q.packed.cuda(), q.scales.cuda()
    for k0 in range(0, K, 32):
        eye = torch.zeros(1, 32, K, dtype=BF)
        eye[0, torch.arange(32), k0 + torch.arange(32)] = 1.0
        y = torch.full((1, 32, O), float("nan"), dtype=torch.float32, device="cuda")
        Megakernel(MatvecNvfp4Sm120Op.schedule(a=eye.cuda(), weight_packed=pk, weight_scales=sc, y=y, group_size=group,
                                               global_scale=q.global_scale)).run()
        got[k0:k0 + 32] = y[0].cpu()
    assert torch.equal(got.t().contiguous(), exact), "device dequantisation differs from e2m1 x scale x global scale"
    host = dequantize_nvfp4_weight(q)
    ulp = torch.finfo(torch.float32).eps * host.abs().clamp(min=torch.finfo(torch.float32).tiny)
    tol = ulp if group == 16 else host.abs() * 2.0 ** -11       # an fp16 block scale rounds the product to fp16
    assert bool(((got.t() - host).abs() <= tol).all())


# ---- flash decoding at its benchmark size ---------------------------------------------------------------
def test_flash_decoding_batch8_32k_tokens():
    """Batch 8, 32 query / 8 KV heads, head dim 128, 32 768 tokens, 32 splits."""
    B, H, Hkv, D, Nkv, S = 8, 32, 8, 128, 32768, 32
    g = torch.Generator().manual_seed(14)
    q = torch.randn(B, 1, H, D, generator=g).to(BF)
    k = torch.randn(B, Nkv, Hkv, D, generator=g).to(BF)
    v = torch.randn(B, Nkv, Hkv, D, generator=g).to(BF)
    o = torch.full((B, 1, H, D), float("nan"), dtype=BF, device="cuda")
    ops, _ = flash_decoding_schedule(q.cuda(), k.cuda(), v.cuda(), o, num_splits=S, kv_group_size=H // Hkv)
    mk = Megakernel(ops)
    mk.run()
    assert mk.native_ops[0].i[N.AT_SPLITS] == S
    for b in range(B):      # the oracle one sequence at a time: 0.27 GB of fp32 K/V each
        want = oracle.attention_bshd(q[b:b + 1].float(), k[b:b + 1].float(), v[b:b + 1].float())
        assert_parity(o[b:b + 1], want, f"flash decode 32k, sequence {b}")
    assert (mk.read_counters() == 0).all() and mk.status()[0] == 0


# ---- the 16-layer step at full width and vocabulary --------------------------------------------------------
def test_llama1b_full_size_step():
    """16 layers, hidden 2048, 32/8 heads of 64, intermediate 8192, vocabulary 128 256, KV length 4096."""
    L, T, hidden, nq, nkv, hd, inter, vocab = 16, 4096, 2048, 32, 8, 64, 8192, 128256
    cache_pos, B = T - 1, 1
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=15, device="cuda")
    g = torch.Generator().manual_seed(16)
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    x0 = torch.randn(B, 1, hidden, generator=g).to(BF)
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    xb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    rb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    tv = torch.zeros(B, 1, device="cuda")
    ti = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    ops, _keep = schedule_decode_model_sm100(
        batch=B, cache_pos=cache_pos, weights=w, k_cache=[t.cuda() for t in kcs], v_cache=[t.cuda() for t in vcs],
        x_buffers=xb, residual_buffers=rb, q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device="cuda"), final_norm=fn.cuda(), lm_head=lm.cuda(),
        top_values=tv, top_indices=ti, num_layers=L, x_in=x0.cuda(), residual_in=r0.cuda())
    mk = Megakernel(ops, scheduler=OverlapTileScheduler())
    mk.run()
    logits, _v, want_i, want_x, want_res = oracle.decode_model(
        weights=to_cpu(w), x=x0, residual=r0, k_caches=kcs, v_caches=vcs, cache_pos=cache_pos, final_norm=fn,
        lm_head=lm, num_layers=L, return_hidden=True)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, "full-size step")
    # The hidden state after 16 layers: cosine >= 0.999 as everywhere; the max-abs bar grows with the
    # depth, two bf16 ulps per layer (the layer's output and the residual stream it is added to),
    # because kernel and oracle round to bf16 at different points of every layer and each later
    # layer works on the already different input.
    assert_parity(xb[(L - 1) % 2], want_x, "last layer output", roundings=2 * L)
    assert_parity(rb[(L - 1) % 2], want_res, "residual stream after 16 layers", roundings=2 * L)
    assert (mk.read_counters() == 0).all() and mk.status()[0] == 0


# ---- the 8B-shape NVFP4 layer width ------------------------------------------------------------------------
MATS = ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")


@pytest.mark.parametrize("B", [1, 8, 32])
def test_qwen3_8b_width_two_layers_nvfp4(B):
    """Hidden 4096, 32/8 heads of 128, q/k RMSNorm, intermediate 12 288 (the down projection's K),
    block-scaled NVFP4; two layers and a small vocabulary keep the oracle at seconds.  Batch 32 does not
    fit the activation staging as one op (32 rows x 4096): it runs as four interleaved chunks of 8."""
    L, T, hidden, nq, nkv, hd, inter, vocab = 2, 512, 4096, 32, 8, 128, 12288, 8192
    cache_pos = 300
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=17, theta=1000000.0)
    g = torch.Generator().manual_seed(18)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    packed, deq = {"cos": w["cos"].cuda(), "sin": w["sin"].cuda(), "final_norm": fn.cuda()}, dict(w)
    for name, mat in [(f"layer.{l}.{m}", w[f"layer.{l}.{m}"]) for l in range(L) for m in MATS] + [("lm_head", lm)]:
        q = quantize_nvfp4_weight(mat, group_size=16)
        packed[f"{name}.packed"], packed[f"{name}.scales"] = q.packed.cuda(), q.scales.cuda()
        packed[f"{name}.global_scale"] = float(q.global_scale)
        deq[name] = dequantize_nvfp4_weight(q)
    for l in range(L):
        packed[f"layer.{l}.attn_norm"] = w[f"layer.{l}.attn_norm"].cuda()
        packed[f"layer.{l}.mlp_norm"] = w[f"layer.{l}.mlp_norm"].cuda()
        for nm in ("q_norm", "k_norm"):
            deq[f"layer.{l}.{nm}"] = (1 + torch.randn(hd, generator=g) * 0.1).to(BF)
            packed[f"layer.{l}.{nm}"] = deq[f"layer.{l}.{nm}"].cuda()
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    x0 = torch.randn(B, 1, hidden, generator=g).to(BF)
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    xb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    rb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    tv = torch.zeros(B, 1, device="cuda")
    ti = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    ops, _keep = schedule_decode_model_nvfp4_sm100(
        batch=B, cache_pos=cache_pos, weights=packed, k_cache=[t.cuda() for t in kcs], v_cache=[t.cuda() for t in vcs],
        x_buffers=xb, residual_buffers=rb, q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device="cuda"), top_values=tv, top_indices=ti, num_layers=L,
        x_in=x0.cuda(), residual_in=r0.cuda(), num_q_heads=nq, num_kv_heads=nkv, head_dim=hd, eps=1e-6)
    mk = Megakernel(ops, scheduler=OverlapTileScheduler())
    mk.run()
    logits, _v, want_i, want_x, want_res = oracle.decode_model(
        weights=deq, x=x0, residual=r0, k_caches=kcs, v_caches=vcs, cache_pos=cache_pos, final_norm=fn,
        lm_head=deq["lm_head"], num_layers=L, eps=1e-6, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd,
        return_hidden=True)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, f"8B width, batch {B}")
    # two bf16 ulps per layer, as for the 16-layer step above (values reach 8-16 here: an ulp is 0.0625)
    assert_parity(xb[(L - 1) % 2], want_x, "last layer output", roundings=2 * L)
    assert_parity(rb[(L - 1) % 2], want_res, "last residual stream", roundings=2 * L)
    assert (mk.read_counters() == 0).all() and mk.status()[0] == 0
