"""Whole decode step with NVFP4 weights on the GPU against the oracle on the dequantised weights.

Qwen3-8B head geometry (head dim 128, 4:1 GQA) at a reduced width so that the
oracle finishes in seconds; both scale layouts: the reference's (fp16 scale per
32 values) and the block-scaled one (e4m3 per 16 values + global scale).
"""

import pytest
import torch

import oracle
from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
from machete_b200.megakernel import Megakernel, OverlapTileScheduler
from machete_b200.quantization import dequantize_nvfp4_weight, quantize_nvfp4_weight
from tests.util import assert_greedy_token, assert_parity, llama_weights

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
MATS = ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")


@pytest.mark.parametrize("group,qk_norm,B", [(32, False, 1), (16, False, 1), (16, True, 1), (16, True, 3),
                                             (16, "unfused", 1), (16, "unfused", 2)])
def test_nvfp4_model_greedy_token(group, qk_norm, B):
    """qk_norm: False = Llama-style layers; True = q/k RMSNorm folded into the attention op;
    "unfused" = q/k RMSNorm as a separate QKNormRopeOp pass."""
    L, T, hidden, nq, nkv, hd, inter, vocab = 2, 256, 2048, 16, 4, 128, 4096, 4096 + 32
    cache_pos = 130
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=4, theta=1000000.0)
    g = torch.Generator().manual_seed(6)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    packed, deq = {"cos": w["cos"].cuda(), "sin": w["sin"].cuda(), "final_norm": fn.cuda()}, dict(w)
    for name, mat in [(f"layer.{l}.{m}", w[f"layer.{l}.{m}"]) for l in range(L) for m in MATS] + [("lm_head", lm)]:
        q = quantize_nvfp4_weight(mat, group_size=group)
        packed[f"{name}.packed"], packed[f"{name}.scales"] = q.packed.cuda(), q.scales.cuda()
        packed[f"{name}.global_scale"] = float(q.global_scale)
        deq[name] = dequantize_nvfp4_weight(q)           # what the kernel multiplies by, exactly
    for l in range(L):
        packed[f"layer.{l}.attn_norm"] = w[f"layer.{l}.attn_norm"].cuda()
        packed[f"layer.{l}.mlp_norm"] = w[f"layer.{l}.mlp_norm"].cuda()
        if qk_norm:    # Qwen3-style per-head RMSNorm of q and k before the rotation
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
        batch=B, cache_pos=cache_pos, weights=packed, k_cache=[k.cuda() for k in kcs], v_cache=[v.cuda() for v in vcs],
        x_buffers=xb, residual_buffers=rb, q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device="cuda"), top_values=tv, top_indices=ti, num_layers=L,
        x_in=x0.cuda(), residual_in=r0.cuda(), num_q_heads=nq, num_kv_heads=nkv, head_dim=hd, eps=1e-6,
        fuse_qk_norm=qk_norm != "unfused")
    mk = Megakernel(ops, scheduler=OverlapTileScheduler())
    mk.run()
    logits, _v, want_i, want_x, want_res = oracle.decode_model(
        weights=deq, x=x0, residual=r0, k_caches=[k.clone() for k in kcs], v_caches=[v.clone() for v in vcs],
        cache_pos=cache_pos, final_norm=fn, lm_head=deq["lm_head"], num_layers=L, eps=1e-6, num_q_heads=nq,
        num_kv_heads=nkv, head_dim=hd, return_hidden=True)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, f"nvfp4 group {group}")
    # the hidden state itself, not only its arg-max: the last layer's outputs sit in buffers (L - 1) % 2
    assert_parity(xb[(L - 1) % 2], want_x, "last layer output", roundings=2 * L)
    assert_parity(rb[(L - 1) % 2], want_res, "last residual stream", roundings=2 * L)
    first = ti.clone()
    mk.run()
    assert torch.equal(first, ti)
    assert (mk.read_counters() == 0).all()
