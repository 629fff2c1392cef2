"""From a checkpoint on disk to a decoded token: Hugging Face safetensors -> weight dict -> schedule ->
megakernel, bf16 and (quantised offline, stored, reloaded) NVFP4, against the oracle on the same weights."""

import json

import pytest
import torch

import oracle
from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.megakernel import Megakernel, OverlapTileScheduler
from machete_b200.quantization import NVFP4Tensor, dequantize_nvfp4_weight
from machete_b200.weights import (MATRICES, load_decoder_weights, load_hf_decoder, quantize_decoder_nvfp4,
                                  save_decoder_weights)
from tests.util import assert_greedy_token, assert_parity

pytestmark = pytest.mark.gpu
safetensors = pytest.importorskip("safetensors")
BF = torch.bfloat16
L, HIDDEN, NQ, NKV, HD, INTER, VOCAB, T = 2, 512, 8, 2, 64, 1024, 1024, 256


def _write_checkpoint(path, qk_norm):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(41)
    w = lambda *s: (torch.randn(*s, generator=g) * 0.03).to(BF)                 # noqa: E731
    nw = lambda n: (1 + torch.randn(n, generator=g) * 0.05).to(BF)             # noqa: E731
    tensors = {"model.embed_tokens.weight": (torch.randn(VOCAB, HIDDEN, generator=g) * 0.05).to(BF),
               "model.norm.weight": nw(HIDDEN)}
    for i in range(L):
        p = f"model.layers.{i}."
        tensors.update({
            p + "input_layernorm.weight": nw(HIDDEN), p + "post_attention_layernorm.weight": nw(HIDDEN),
            p + "self_attn.q_proj.weight": w(NQ * HD, HIDDEN), p + "self_attn.k_proj.weight": w(NKV * HD, HIDDEN),
            p + "self_attn.v_proj.weight": w(NKV * HD, HIDDEN), p + "self_attn.o_proj.weight": w(HIDDEN, NQ * HD),
            p + "mlp.gate_proj.weight": w(INTER, HIDDEN), p + "mlp.up_proj.weight": w(INTER, HIDDEN),
            p + "mlp.down_proj.weight": w(HIDDEN, INTER)})
        if qk_norm:
            tensors.update({p + "self_attn.q_norm.weight": nw(HD), p + "self_attn.k_norm.weight": nw(HD)})
    save_file(tensors, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps({"num_attention_heads": NQ, "num_key_value_heads": NKV,
                                                  "hidden_size": HIDDEN, "head_dim": HD, "rope_theta": 500000.0}))


def _state(B, seed):
    g = torch.Generator().manual_seed(seed)
    kcs = [torch.randn(B, T, NKV, HD, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, NKV, HD, generator=g).to(BF) for _ in range(L)]
    return kcs, vcs


def _buffers(B):
    z = lambda *s: torch.zeros(*s, dtype=BF, device="cuda")                     # noqa: E731
    return dict(x_buffers=[z(B, 1, HIDDEN) for _ in range(2)], residual_buffers=[z(B, 1, HIDDEN) for _ in range(2)],
                q_buf=z(B, 1, NQ * HD), attn_out_buf=z(B, 1, NQ * HD), mlp_h_buf=z(B, 1, INTER))


def test_bf16_checkpoint_decodes_like_the_oracle(tmp_path):
    _write_checkpoint(tmp_path, qk_norm=False)
    w = load_hf_decoder(str(tmp_path), max_len=T)                               # CPU dict: the oracle's weights
    wd = {k: v.cuda() for k, v in w.items()}
    B, pos = 2, 200
    kcs, vcs = _state(B, 42)
    tok = torch.tensor([7, 900])
    x0 = w["embedding"][tok].view(B, 1, HIDDEN).clone()
    r0 = torch.zeros(B, 1, HIDDEN, dtype=BF)
    tv, ti = torch.zeros(B, 1, device="cuda"), torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    bufs = _buffers(B)
    ops, _ = schedule_decode_model_sm100(
        batch=B, cache_pos=pos, weights=wd, k_cache=[t.cuda() for t in kcs], v_cache=[t.cuda() for t in vcs],
        final_norm=wd["final_norm"], lm_head=wd["lm_head"], top_values=tv, top_indices=ti, num_layers=L,
        x_in=x0.cuda(), residual_in=r0.cuda(), hidden_size=HIDDEN, intermediate_size=INTER, num_q_heads=NQ,
        num_kv_heads=NKV, head_dim=HD, **bufs)
    Megakernel(ops, scheduler=OverlapTileScheduler()).run()
    logits, _v, want_i, want_x, _r = oracle.decode_model(
        weights=w, x=x0, residual=r0, k_caches=kcs, v_caches=vcs, cache_pos=pos, final_norm=w["final_norm"],
        lm_head=w["lm_head"], num_layers=L, num_q_heads=NQ, num_kv_heads=NKV, head_dim=HD, return_hidden=True)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, "bf16 checkpoint")
    assert_parity(bufs["x_buffers"][(L - 1) % 2], want_x, "last layer output", roundings=2 * L)


def test_offline_nvfp4_file_decodes_like_the_oracle_on_the_dequantised_weights(tmp_path):
    _write_checkpoint(tmp_path, qk_norm=True)
    w = load_hf_decoder(str(tmp_path), max_len=T)
    path = tmp_path / "nvfp4.safetensors"
    save_decoder_weights(quantize_decoder_nvfp4(w, group_size=16), str(path))
    q = load_decoder_weights(str(path), device="cuda")                          # what a server would load
    assert f"layer.0.W_q.packed" in q and "layer.0.W_q" not in q and q["layer.1.q_norm"].shape == (HD,)
    deq = {k: v for k, v in w.items()}
    for name in [f"layer.{i}.{m}" for i in range(L) for m in MATRICES] + ["lm_head"]:
        t = NVFP4Tensor(q[f"{name}.packed"].cpu(), q[f"{name}.scales"].cpu(), 16, global_scale=q[f"{name}.global_scale"])
        deq[name] = dequantize_nvfp4_weight(t)
    B, pos = 1, 130
    kcs, vcs = _state(B, 43)
    x0 = w["embedding"][torch.tensor([11])].view(B, 1, HIDDEN).clone()
    r0 = torch.zeros(B, 1, HIDDEN, dtype=BF)
    tv, ti = torch.zeros(B, 1, device="cuda"), torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    bufs = _buffers(B)
    ops, _ = schedule_decode_model_nvfp4_sm100(
        batch=B, cache_pos=pos, weights=q, k_cache=[t.cuda() for t in kcs], v_cache=[t.cuda() for t in vcs],
        top_values=tv, top_indices=ti, num_layers=L, x_in=x0.cuda(), residual_in=r0.cuda(), num_q_heads=NQ,
        num_kv_heads=NKV, head_dim=HD, eps=1e-6, **bufs)
    Megakernel(ops, scheduler=OverlapTileScheduler()).run()
    logits, _v, want_i, want_x, _r = oracle.decode_model(
        weights=deq, x=x0, residual=r0, k_caches=kcs, v_caches=vcs, cache_pos=pos, final_norm=w["final_norm"],
        lm_head=deq["lm_head"], num_layers=L, eps=1e-6, num_q_heads=NQ, num_kv_heads=NKV, head_dim=HD,
        return_hidden=True)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, "nvfp4 checkpoint")
    assert_parity(bufs["x_buffers"][(L - 1) % 2], want_x, "last layer output", roundings=2 * L)
