"""Checkpoint loading: Hugging Face safetensors -> the schedules' weight dict, QKV interleaving,
offline NVFP4 quantisation and its on-disk round trip (CPU only)."""

import json

import pytest
import torch

from machete_b200.quantization import NVFP4Tensor, dequantize_nvfp4_weight, quantize_nvfp4_weight
from machete_b200.weights import (MATRICES, interleave_qkv_weight, load_decoder_weights, load_hf_decoder,
                                  quantize_decoder_nvfp4, rope_tables, save_decoder_weights)
from tests.util import rope_tables as util_tables

safetensors = pytest.importorskip("safetensors")


def _hf_checkpoint(tmp_path, layers=2, hidden=64, heads=4, kv_heads=2, hd=16, inter=128, vocab=96, qk_norm=False, shards=1):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(1)
    t = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)    # noqa: E731
    tensors = {"model.embed_tokens.weight": t(vocab, hidden), "model.norm.weight": t(hidden)}
    for i in range(layers):
        p = f"model.layers.{i}."
        tensors.update({
            p + "input_layernorm.weight": t(hidden), p + "post_attention_layernorm.weight": t(hidden),
            p + "self_attn.q_proj.weight": t(heads * hd, hidden), p + "self_attn.k_proj.weight": t(kv_heads * hd, hidden),
            p + "self_attn.v_proj.weight": t(kv_heads * hd, hidden), p + "self_attn.o_proj.weight": t(hidden, heads * hd),
            p + "mlp.gate_proj.weight": t(inter, hidden), p + "mlp.up_proj.weight": t(inter, hidden),
            p + "mlp.down_proj.weight": t(hidden, inter), p + "self_attn.rotary_emb.inv_freq": torch.zeros(hd // 2),
        })
        if qk_norm:
            tensors.update({p + "self_attn.q_norm.weight": t(hd), p + "self_attn.k_norm.weight": t(hd)})
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "hidden_size": hidden, "head_dim": hd,
           "rope_theta": 500000.0}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    names = sorted(tensors)
    if shards == 1:
        save_file(tensors, str(tmp_path / "model.safetensors"))
    else:
        weight_map = {}
        for s in range(shards):
            part = {n: tensors[n] for n in names[s::shards]}
            fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            save_file(part, str(tmp_path / fname))
            weight_map.update({n: fname for n in part})
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    return tensors, cfg


@pytest.mark.parametrize("shards,qk_norm", [(1, False), (3, True)])
def test_hf_checkpoint_maps_onto_the_weight_dict(tmp_path, shards, qk_norm):
    tensors, cfg = _hf_checkpoint(tmp_path, shards=shards, qk_norm=qk_norm)
    w = load_hf_decoder(str(tmp_path), max_len=40)
    for i in range(2):
        p = f"model.layers.{i}."
        assert torch.equal(w[f"layer.{i}.W_q"], tensors[p + "self_attn.q_proj.weight"])
        assert torch.equal(w[f"layer.{i}.W_down"], tensors[p + "mlp.down_proj.weight"])
        assert torch.equal(w[f"layer.{i}.attn_norm"], tensors[p + "input_layernorm.weight"])
        assert torch.equal(w[f"layer.{i}.mlp_norm"], tensors[p + "post_attention_layernorm.weight"])
        assert (f"layer.{i}.q_norm" in w) == qk_norm
    assert torch.equal(w["final_norm"], tensors["model.norm.weight"])
    assert w["lm_head"] is w["embedding"]                       # tied: no lm_head.weight in the file
    cos, sin = util_tables(40, 8, 500000.0)
    assert torch.equal(w["cos"], cos) and torch.equal(w["sin"], sin)
    assert "layer.2.W_q" not in w and not any("inv_freq" in k for k in w)
    # a partial load keeps the first layers only
    assert "layer.1.W_q" not in load_hf_decoder(str(tmp_path), max_len=8, num_layers=1)


def test_llama3_rope_scaling_rescales_only_the_low_frequencies():
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    plain_c, _ = rope_tables(64, 64, 500000.0, dtype=torch.float32)
    scaled_c, _ = rope_tables(64, 64, 500000.0, dtype=torch.float32, scaling=scaling)
    assert torch.equal(plain_c[:, :8], scaled_c[:, :8])         # the fastest frequencies are untouched
    assert not torch.equal(plain_c[:, -4:], scaled_c[:, -4:])   # the slowest ones are divided by the factor
    inv_last = 1.0 / (500000.0 ** (31 / 32))
    want = torch.cos(torch.arange(64, dtype=torch.float64) * inv_last / 32.0).float()
    assert float((scaled_c[:, -1] - want).abs().max()) < 1e-6


def test_qkv_interleave_is_per_kv_head_q_group_then_k_then_v():
    nkv, hd, group, hidden = 2, 4, 3, 5
    wq = torch.arange(nkv * group * hd * hidden, dtype=torch.float32).view(-1, hidden)
    wk = 1000 + torch.arange(nkv * hd * hidden, dtype=torch.float32).view(-1, hidden)
    wv = 2000 + torch.arange(nkv * hd * hidden, dtype=torch.float32).view(-1, hidden)
    w = interleave_qkv_weight(wq, wk, wv, num_kv_heads=nkv, head_dim=hd, kv_group_size=group)
    rows = (group + 2) * hd
    assert w.shape == (nkv * rows, hidden)
    for h in range(nkv):
        blk = w[h * rows:(h + 1) * rows]
        assert torch.equal(blk[:group * hd], wq[h * group * hd:(h + 1) * group * hd])
        assert torch.equal(blk[group * hd:group * hd + hd], wk[h * hd:(h + 1) * hd])
        assert torch.equal(blk[group * hd + hd:], wv[h * hd:(h + 1) * hd])
    with pytest.raises(ValueError):
        interleave_qkv_weight(wq[:-1], wk, wv, num_kv_heads=nkv, head_dim=hd, kv_group_size=group)


def test_offline_nvfp4_round_trip_through_a_file(tmp_path):
    _hf_checkpoint(tmp_path)
    w = load_hf_decoder(str(tmp_path), max_len=16)
    q = quantize_decoder_nvfp4(w, group_size=16)
    for i in range(2):
        for m in MATRICES:
            key = f"layer.{i}.{m}"
            assert key not in q and q[f"{key}.packed"].dtype == torch.uint8
            direct = quantize_nvfp4_weight(w[key], group_size=16)
            assert torch.equal(q[f"{key}.packed"], direct.packed) and q[f"{key}.global_scale"] == direct.global_scale
        assert torch.equal(q[f"layer.{i}.attn_norm"], w[f"layer.{i}.attn_norm"])
    path = tmp_path / "q.safetensors"
    save_decoder_weights(q, str(path))
    back = load_decoder_weights(str(path))
    assert set(back) == set(q)
    for k, v in q.items():
        if isinstance(v, torch.Tensor):
            assert back[k].dtype == v.dtype and torch.equal(back[k].view(torch.uint8), v.view(torch.uint8)), k
        else:
            assert back[k] == pytest.approx(v, rel=1e-7), k
    t = NVFP4Tensor(back["layer.0.W_o.packed"], back["layer.0.W_o.scales"], 16, global_scale=back["layer.0.W_o.global_scale"])
    ref = quantize_nvfp4_weight(w["layer.0.W_o"], group_size=16)
    assert float((dequantize_nvfp4_weight(t) - dequantize_nvfp4_weight(ref)).abs().max()) < 1e-6
