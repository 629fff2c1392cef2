"""Loading real checkpoints into the weight-dict layout the decode schedules take.

The reference's model schedules read a flat dict: ``cos`` / ``sin`` tables and,
per layer, ``layer.{i}.attn_norm``, ``mlp_norm``, ``W_q``, ``W_k``, ``W_v``,
``W_o``, ``W_gate``, ``W_up``, ``W_down`` (benchmarks/kernels/
benchmark_llama1b_sm120_decode.py:47-63 builds it from random tensors; the
NVFP4 layer reads ``layer.{i}.<name>_nvfp4``, src/machete/kernels/
decode_matvec/sm120.py:2676-2686).  The reference has no loader for real
weights; this module is the caller-side format work next to the hot path:

* Hugging Face ``*.safetensors`` checkpoints (single file or sharded with
  ``model.safetensors.index.json``) of Llama-3.x / Qwen3-style decoders are
  mapped onto that dict, with the RoPE tables computed from ``config.json``;
* the three projection matrices can be packed per KV head as
  ``[q heads of the group | k | v]``, the layout of the reference's fused
  QKV op (src/machete/kernels/llama1b/sm120.py:4330-4345);
* weights are quantised offline to block-scaled NVFP4 and stored / reloaded as
  safetensors (``<name>.packed`` uint8, ``<name>.scales`` e4m3,
  ``<name>.global_scale`` fp32), the keys ``schedule_decode_model_nvfp4_sm100``
  reads.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, Iterable, Optional

import torch

from .quantization import quantize_nvfp4_weight

_HF_LAYER = {
    "input_layernorm.weight": "attn_norm",
    "post_attention_layernorm.weight": "mlp_norm",
    "self_attn.q_proj.weight": "W_q",
    "self_attn.k_proj.weight": "W_k",
    "self_attn.v_proj.weight": "W_v",
    "self_attn.o_proj.weight": "W_o",
    "self_attn.q_norm.weight": "q_norm",     # Qwen3: per-head RMSNorm of q and k
    "self_attn.k_norm.weight": "k_norm",
    "mlp.gate_proj.weight": "W_gate",
    "mlp.up_proj.weight": "W_up",
    "mlp.down_proj.weight": "W_down",
}
MATRICES = ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")


def rope_tables(max_len: int, head_dim: int, theta: float, dtype=torch.bfloat16, device="cpu",
                scaling: Optional[dict] = None):
    """``(max_len, head_dim / 2)`` cos / sin tables for the split-half rotation (rope/ref.py:18-43).

    ``scaling``: a Hugging Face ``rope_scaling`` dict; ``rope_type == "llama3"`` (Llama-3.1 / 3.2)
    rescales the low frequencies, anything else (or None) leaves the plain theta schedule.
    """
    d2 = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, d2, dtype=torch.float64) / d2))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        old_len = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = ((old_len / wavelen) - low) / (high - low)
        scaled = torch.where(wavelen > old_len / low, inv / factor, inv)
        mid = (wavelen <= old_len / low) & (wavelen >= old_len / high)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    ang = torch.arange(max_len, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype).to(device), torch.sin(ang).to(dtype).to(device)


def _open_shards(path: str):
    """Yield (tensor name, loader) over a checkpoint file or directory."""
    from safetensors import safe_open

    if os.path.isdir(path):
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as fh:
                files = sorted(set(json.load(fh)["weight_map"].values()))
        else:
            files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        files = [os.path.join(path, f) for f in files]
    else:
        files = [path]
    if not files:
        raise FileNotFoundError(f"no .safetensors file under {path}")
    for f in files:
        with safe_open(f, framework="pt", device="cpu") as sf:
            for name in sf.keys():
                yield name, sf.get_tensor(name)


def load_hf_decoder(path: str, *, max_len: int, device="cpu", dtype=torch.bfloat16, num_layers: Optional[int] = None,
                    config: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """Read a Hugging Face Llama / Qwen3-style decoder checkpoint into the schedules' weight dict.

    Returns ``cos``, ``sin`` (``max_len`` rows), ``layer.{i}.*``, ``final_norm``, ``embedding`` and
    ``lm_head`` (the embedding itself when the checkpoint ties them).  ``config`` defaults to the
    ``config.json`` next to the weights and supplies ``rope_theta``, ``rope_scaling`` and the head
    geometry.  ``num_layers`` keeps only the first layers (for tests and partial loads).
    """
    if config is None:
        cfg_path = os.path.join(path if os.path.isdir(path) else os.path.dirname(path), "config.json")
        with open(cfg_path) as fh:
            config = json.load(fh)
    out: Dict[str, torch.Tensor] = {}
    seen_layers = set()
    for name, tensor in _open_shards(path):
        t = tensor.to(dtype)
        if name in ("model.embed_tokens.weight", "embed_tokens.weight"):
            out["embedding"] = t.to(device)
        elif name in ("model.norm.weight", "norm.weight"):
            out["final_norm"] = t.to(device)
        elif name == "lm_head.weight":
            out["lm_head"] = t.to(device)
        elif ".layers." in name:
            rest = name.split(".layers.", 1)[1]
            idx, field = rest.split(".", 1)
            if num_layers is not None and int(idx) >= num_layers:
                continue
            key = _HF_LAYER.get(field)
            if key is None:
                continue                  # rotary inv_freq buffers, biases this path does not use
            out[f"layer.{int(idx)}.{key}"] = t.to(device).contiguous()
            seen_layers.add(int(idx))
    if "embedding" not in out or "final_norm" not in out:
        raise ValueError("checkpoint lacks model.embed_tokens.weight / model.norm.weight")
    out.setdefault("lm_head", out["embedding"])           # tied embeddings (Llama-3.2-1B)
    n = max(seen_layers) + 1 if seen_layers else 0
    for i in range(n):
        missing = [k for k in ("attn_norm", "mlp_norm", *MATRICES) if f"layer.{i}.{k}" not in out]
        if missing:
            raise ValueError(f"layer {i} lacks {missing}")
    heads = int(config["num_attention_heads"])
    head_dim = int(config.get("head_dim") or config["hidden_size"] // heads)
    out["cos"], out["sin"] = rope_tables(max_len, head_dim, float(config.get("rope_theta", 10000.0)), dtype, device,
                                         config.get("rope_scaling"))
    return out


def interleave_qkv_weight(w_q, w_k, w_v, *, num_kv_heads: int, head_dim: int, kv_group_size: int):
    """Rows reordered per KV head as ``[its q heads | its k head | its v head]`` (one matrix, one stream)."""
    q_rows = kv_group_size * head_dim
    if w_q.shape[0] != num_kv_heads * q_rows or w_k.shape[0] != num_kv_heads * head_dim or w_v.shape != w_k.shape:
        raise ValueError("projection shapes do not match the head geometry")
    parts = []
    for h in range(num_kv_heads):
        parts += [w_q[h * q_rows:(h + 1) * q_rows], w_k[h * head_dim:(h + 1) * head_dim],
                  w_v[h * head_dim:(h + 1) * head_dim]]
    return torch.cat(parts, dim=0)


def quantize_decoder_nvfp4(weights: Dict[str, torch.Tensor], group_size: int = 16,
                           names: Iterable[str] = MATRICES, lm_head: bool = True) -> Dict[str, torch.Tensor]:
    """Offline quantisation: every projection matrix (and the LM head) becomes ``<name>.packed`` /
    ``<name>.scales`` / ``<name>.global_scale``; norms, tables and the embedding stay as they are."""
    wanted = set(names)
    out: Dict[str, torch.Tensor] = {}
    for key, t in weights.items():
        is_matrix = key.startswith("layer.") and key.rsplit(".", 1)[1] in wanted
        if is_matrix or (lm_head and key == "lm_head"):
            q = quantize_nvfp4_weight(t, group_size=group_size)
            out[f"{key}.packed"], out[f"{key}.scales"] = q.packed, q.scales
            out[f"{key}.global_scale"] = float(q.global_scale)
        else:
            out[key] = t
    return out


def save_decoder_weights(weights: Dict[str, object], path: str) -> None:
    """Store a weight dict (plain or NVFP4-quantised) as one safetensors file; fp32 scalars such as
    ``*.global_scale`` are stored as one-element tensors."""
    from safetensors.torch import save_file

    flat, seen = {}, {}
    for k, v in weights.items():
        t = v if isinstance(v, torch.Tensor) else torch.tensor([float(v)], dtype=torch.float32)
        t = t.detach().cpu().contiguous()
        ptr = t.untyped_storage().data_ptr()
        if ptr in seen and seen[ptr] != k:      # tied tensors: the file format wants distinct storage
            t = t.clone()
        seen[ptr] = k
        flat[k] = t
    save_file(flat, path)


def load_decoder_weights(path: str, device="cpu") -> Dict[str, object]:
    """Inverse of :func:`save_decoder_weights` (``*.global_scale`` comes back as a Python float)."""
    from safetensors import safe_open

    out: Dict[str, object] = {}
    with safe_open(path, framework="pt", device="cpu") as sf:
        for name in sf.keys():
            t = sf.get_tensor(name)
            out[name] = float(t.item()) if name.endswith(".global_scale") else t.to(device)
    return out


__all__ = ["rope_tables", "load_hf_decoder", "interleave_qkv_weight", "quantize_decoder_nvfp4", "save_decoder_weights",
           "load_decoder_weights", "MATRICES"]
