"""fp32 CPU restatement of the reference's PyTorch reference functions for the decode path.

TEST INFRASTRUCTURE.  Every function states the reference definition it
follows (paths inside the reference project).  Parity status: PINNED — each
function is checked against the reference's own function on seeded inputs by
``tests/golden/make_golden.py`` (which imports the reference where it is
mounted and stores inputs + reference outputs as fixtures under
``tests/golden/``); ``tests/test_oracle_golden.py`` replays the fixtures
against this file.

All functions take torch tensors on the CPU and compute in float32.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

__all__ = [
    "rmsnorm", "fused_add_rmsnorm", "rmsnorm_gated", "rope", "qknorm_rope", "glu", "attention", "attention_bshd",
    "split_kv_partials", "combine_partials", "E2M1_LUT", "quantize_nvfp4", "dequantize_nvfp4",
    "quantize_nvfp4_e4m3", "matvec", "rms_q_matvec_rope", "rms_kv_matvec_cache", "matvec_residual",
    "rms_gate_up_silu", "final_rms_lm_head", "decode_layer", "decode_model", "top1", "parity_metrics",
]


# ---- norms -----------------------------------------------------------------------------------
def rmsnorm(x, weight, eps=1e-6, residual=False, gemma=False):
    """src/machete/kernels/rms_norm/ref.py:17-39 ``rmsnorm_pytorch``."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    w = weight.float()
    if gemma:
        w = 1.0 + w
    y = xf * torch.rsqrt(var + eps) * w
    if residual:
        y = y + xf
    return y.to(x.dtype)


def fused_add_rmsnorm(x, residual_in, weight, eps=1e-6, gemma=False):
    """src/machete/kernels/rms_norm/ref.py:80-88: the sum is rounded to x.dtype before the norm."""
    residual_out = (x.float() + residual_in.float()).to(x.dtype)
    return rmsnorm(residual_out, weight, eps=eps, gemma=gemma), residual_out


def rmsnorm_gated(x, gate, weight, eps=1e-6, gemma=False):
    """src/machete/kernels/rms_norm/ref.py:104-114: y = rmsnorm(x) * silu(gate)."""
    normed = rmsnorm(x, weight, eps=eps, gemma=gemma)
    g = gate.float()
    return (normed.float() * (g * torch.sigmoid(g))).to(x.dtype)


# ---- rotary ----------------------------------------------------------------------------------
def rope(q, cos, sin):
    """src/machete/kernels/rope/ref.py:18-43: split-half rotation, partial rotary tail unchanged.

    q: (B, S, H, D); cos/sin: (>=S, D2).
    """
    b, s, h, d = q.shape
    d2 = cos.shape[1]
    q0, q1 = q[..., :d2], q[..., d2:2 * d2]
    c = cos[:s].view(1, s, 1, d2)
    sn = sin[:s].view(1, s, 1, d2)
    out = q.clone()
    out[..., :d2] = q0 * c - q1 * sn
    out[..., d2:2 * d2] = q1 * c + q0 * sn
    return out


def qknorm_rope(q, norm_weight, cos, sin, eps=1e-6):
    """src/machete/kernels/qknorm_rope/ref.py:10-39: per-head RMSNorm rounded to q.dtype, then RoPE."""
    b, s, h, d = q.shape
    d2 = cos.shape[1]
    qf = q.float()
    rms = (qf.pow(2).mean(dim=-1, keepdim=True) + eps).rsqrt()
    qn = (qf * rms * norm_weight.float()).to(q.dtype)
    q0, q1 = qn[..., :d2], qn[..., d2:2 * d2]
    c = cos[:s].view(1, s, 1, d2)
    sn = sin[:s].view(1, s, 1, d2)
    out = qn.clone()
    out[..., :d2] = q0 * c - q1 * sn
    out[..., d2:2 * d2] = q1 * c + q0 * sn
    return out


# ---- GLU -------------------------------------------------------------------------------------
def glu(x, activation="silu"):
    """src/machete/kernels/glu/ref.py:8-33: y = act(x[..., :D]) * x[..., D:]."""
    d = x.shape[-1] // 2
    gate, up = x[..., :d].float(), x[..., d:].float()
    if activation == "silu":
        gate = gate * torch.sigmoid(gate)
    elif activation == "relu":
        gate = torch.relu(gate)
    elif activation != "identity":
        raise ValueError(f"Unknown activation: {activation}")
    return (gate * up).to(x.dtype)


# ---- attention -------------------------------------------------------------------------------
def attention(q, k, v, causal=False, scale=None, kv_group_size=1):
    """src/machete/kernels/attention/ref.py:12-45 ``flash_attention_pytorch``.

    q: (BH_q, M, D); k, v: (BH_kv, N, D); causal mask is lower-left aligned:
    row i attends to columns 0..i + N - M.
    """
    if kv_group_size > 1:
        k = k.repeat_interleave(kv_group_size, dim=0)
        v = v.repeat_interleave(kv_group_size, dim=0)
    scale = scale or (q.shape[-1] ** -0.5)
    scores = torch.bmm(q.float(), k.float().transpose(-2, -1)) * scale
    if causal:
        m, n = q.shape[1], k.shape[1]
        row = torch.arange(m).unsqueeze(1)
        col = torch.arange(n).unsqueeze(0)
        scores.masked_fill_((col > row + (n - m)).unsqueeze(0), float("-inf"))
    return torch.bmm(torch.softmax(scores, dim=-1), v.float()).to(q.dtype)


def attention_bshd(q, k, v, causal=False):
    """The same attention on the layouts of the decode path: q (B, M, H, D), k/v (B, N, H_kv, D) -> (B, M, H, D).

    Head h of q uses KV head h // (H / H_kv) (reference flash_decoding.py:1324).
    """
    B, M, H, D = q.shape
    N, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    qf = q.permute(0, 2, 1, 3).reshape(B * H, M, D)
    kf = k.permute(0, 2, 1, 3).reshape(B * Hkv, N, D)
    vf = v.permute(0, 2, 1, 3).reshape(B * Hkv, N, D)
    o = attention(qf, kf, vf, causal=causal, kv_group_size=g)
    return o.reshape(B, H, M, D).permute(0, 2, 1, 3).contiguous()


def split_kv_partials(q, k, v, bounds, causal=False):
    """Normalised per-split outputs and log-sum-exps, the split op's contract
    (reference flash_decoding.py:1139-1172): ``o_partial (B, H, S, M, D)``,
    ``lse_partial (B, H, S, M)`` with ``lse = max * scale + ln(sum)``.
    ``bounds`` lists the ``(begin, end)`` token range of every split.
    """
    B, M, H, D = q.shape
    N, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    scale = D ** -0.5
    S = len(bounds)
    o = torch.zeros(B, H, S, M, D)
    lse = torch.full((B, H, S, M), float("-inf"))
    qf, kf, vf = q.float(), k.float(), v.float()
    for s, (t0, t1) in enumerate(bounds):
        if t1 <= t0:
            continue
        for h in range(H):
            kh = kf[:, t0:t1, h // g]                       # (B, n, D)
            sc = torch.einsum("bmd,bnd->bmn", qf[:, :, h], kh) * scale
            if causal:
                row = torch.arange(M).view(1, M, 1)
                col = torch.arange(t0, t1).view(1, 1, -1)
                sc = sc.masked_fill(col > row + (N - M), float("-inf"))
            l = torch.logsumexp(sc, dim=-1)                  # (B, M)
            p = torch.exp(sc - torch.where(torch.isinf(l), torch.zeros_like(l), l).unsqueeze(-1))
            p = torch.where(torch.isinf(l).unsqueeze(-1), torch.zeros_like(p), p)
            o[:, h, s] = torch.einsum("bmn,bnd->bmd", p, vf[:, t0:t1, h // g])
            lse[:, h, s] = l
    return o, lse


def combine_partials(o_partial, lse_partial):
    """Reference flash_decoding.py:1858-1950: o = sum_s e^{lse_s - max} o_s / sum_s e^{lse_s - max}.

    Returns ``o (B, M, H, D)`` fp32 and ``lse (B, H, M)``.
    """
    mx = lse_partial.max(dim=2, keepdim=True).values
    safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    w = torch.exp(lse_partial - safe)                        # (B, H, S, M)
    den = w.sum(dim=2)                                       # (B, H, M)
    o = (w.unsqueeze(-1) * o_partial).sum(dim=2) / den.clamp_min(1e-38).unsqueeze(-1)
    o = torch.where((den > 0).unsqueeze(-1), o, torch.zeros_like(o))
    lse = torch.where(den > 0, safe.squeeze(2) + torch.log(den.clamp_min(1e-38)), torch.full_like(den, float("-inf")))
    return o.permute(0, 2, 1, 3).contiguous(), lse


# ---- NVFP4 -----------------------------------------------------------------------------------
E2M1_LUT = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])
_THRESH = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def _codes(normalized, rows, cols):
    mag = torch.bucketize(normalized.abs().contiguous(), _THRESH).to(torch.uint8)
    codes = (mag | ((normalized < 0).to(torch.uint8) << 3)).reshape(rows, cols)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()


def quantize_nvfp4(weight, group_size=32):
    """src/machete/quantization/nvfp4.py:78-105: (packed uint8 (R, C/2), fp16 scales (R, C/G)).

    scale = amax/6 per group (1.0 when the group is all zero); the codes use
    the unrounded fp32 scale; a value exactly on a threshold takes the lower
    code (``bucketize`` with right=False); low nibble = even column.
    """
    rows, cols = weight.shape
    w = weight.float().reshape(rows, cols // group_size, group_size)
    amax = w.abs().amax(dim=-1)
    scales = torch.where(amax > 0, amax / 6.0, torch.ones_like(amax))
    return _codes(w / scales.unsqueeze(-1), rows, cols), scales.to(torch.float16).contiguous()


def dequantize_nvfp4(packed, scales, group_size=32, global_scale=1.0):
    """src/machete/quantization/nvfp4.py:109-122."""
    rows, cols = packed.shape[0], packed.shape[1] * 2
    codes = torch.empty(rows, cols, dtype=torch.long)
    codes[:, 0::2] = (packed & 0x0F).long()
    codes[:, 1::2] = (packed >> 4).long()
    vals = E2M1_LUT[codes].reshape(rows, cols // group_size, group_size)
    return (vals * (scales.float() * global_scale).unsqueeze(-1)).reshape(rows, cols)


def quantize_nvfp4_e4m3(weight):
    """Block-scaled NVFP4 of the benchmark configs: e4m3 scale per 16 values + fp32 global scale.

    Not a reference function (the reference only has the fp16/32 layout): the
    published NVFP4 recipe, global = amax/(448*6), block = e4m3(amax_b/6/global),
    codes against the decoded block*global.  Returns (packed, scales_e4m3, global).
    """
    rows, cols = weight.shape
    w = weight.float().reshape(rows, cols // 16, 16)
    amax = w.abs().amax(dim=-1)
    t = float(amax.max())
    g = t / (448.0 * 6.0) if t > 0 else 1.0
    block = (amax / 6.0 / g).clamp(max=448.0).to(torch.float8_e4m3fn)
    dec = block.float() * g
    safe = torch.where(dec > 0, dec, torch.ones_like(dec))
    return _codes(w / safe.unsqueeze(-1), rows, cols), block.contiguous(), g


# ---- projections and fused decode ops ------------------------------------------------------------
def matvec(a, w):
    """fp32 truth of every projection: ``a.float() @ w.float().T`` (reference tests/kernels/test_gemm.py:85-98)."""
    return a.float() @ w.float().t()


def _rms_h(x, residual_in, norm_weight, eps):
    """h = rms(x + residual_in) * w in fp32, plus the bf16-rounded residual stream."""
    if residual_in is None:
        r = x
    else:
        r = (x.float() + residual_in.float()).to(x.dtype)
    rf = r.float()
    h = rf * torch.rsqrt(rf.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    return h, r


def rms_q_matvec_rope(x, residual_in, norm_weight, weight, cos, sin, eps=1e-5, head_dim=None):
    """src/machete/kernels/decode_matvec/sm100.py:224-253: residual_out = x + residual_in;
    q = rope(rms(residual_out) * w @ W^T).  Returns (q fp32 (B, S, O), residual_out)."""
    h, r = _rms_h(x, residual_in, norm_weight, eps)
    q = h @ weight.float().t()
    B, S, O = q.shape
    hd = head_dim or 2 * cos.shape[1]
    if cos is not None:
        q = rope(q.view(B, S, O // hd, hd), cos.float(), sin.float()).reshape(B, S, O)
    return q, r


def rms_kv_matvec_cache(x, residual_in, norm_weight, weight, cos, sin, cache, cache_pos, eps=1e-5, apply_rope=True):
    """src/machete/kernels/decode_matvec/sm100.py:256-324: project, rotate (K only), write rows
    [cache_pos, cache_pos + S) of ``cache (B, T, H, HD)`` in place (rounded to the cache dtype)."""
    h, _ = _rms_h(x, residual_in, norm_weight, eps)
    kv = h @ weight.float().t()
    B, S, O = kv.shape
    hd = cache.shape[-1]
    kv = kv.view(B, S, O // hd, hd)
    if apply_rope:
        kv = rope(kv, cos.float(), sin.float())
    cache[:, cache_pos:cache_pos + S] = kv.to(cache.dtype)
    return kv


def matvec_residual(a, weight, residual_in):
    """src/machete/kernels/decode_matvec/sm100.py:327-383: a @ W^T + residual_in (fp32)."""
    return matvec(a, weight) + residual_in.float()


def rms_gate_up_silu(x, norm_weight, gate_weight, up_weight, eps=1e-5):
    """src/machete/kernels/decode_matvec/sm100.py:485-571: silu(h Wg^T) * (h Wu^T), h = rms(x) * w."""
    h, _ = _rms_h(x, None, norm_weight, eps)
    g = h @ gate_weight.float().t()
    u = h @ up_weight.float().t()
    return g * torch.sigmoid(g) * u


def final_rms_lm_head(x, norm_weight, weight, eps=1e-5, residual_in=None):
    """src/machete/kernels/decode_matvec/sm100.py:574-654 (logits, fp32)."""
    h, _ = _rms_h(x, residual_in, norm_weight, eps)
    return h @ weight.float().t()


def top1(logits):
    """Greedy token: (max value, argmax index) over the last dim; ties take the lowest index."""
    v, i = logits.max(dim=-1)
    return v, i.to(torch.int32)


def decode_layer(*, weights, layer_idx, x_in, residual_in, k_cache, v_cache, cache_pos, eps=1e-5,
                 num_q_heads=32, num_kv_heads=8, head_dim=64, round_intermediates=True):
    """One decoder layer exactly as ``schedule_decode_layer_sm100`` composes it
    (src/machete/kernels/decode_matvec/sm100.py:666-823).

    Inputs are the layer's (MLP delta ``x_in``, residual stream ``residual_in``),
    both (B, S, hidden) bf16; the caches are updated in place.  Every tensor
    the schedule stores in bf16 between ops (residual, q, attention output,
    MLP hidden) is rounded here as well when ``round_intermediates`` is set, so
    the result is what the op chain produces with exact fp32 arithmetic
    inside each op.  Returns (x_out, residual_out) in bf16.
    """
    dt = x_in.dtype
    rnd = (lambda t: t.to(dt)) if round_intermediates else (lambda t: t)
    p = f"layer.{layer_idx}"
    B, S, _ = x_in.shape
    cos = weights["cos"][cache_pos:cache_pos + S]
    sin = weights["sin"][cache_pos:cache_pos + S]
    if f"{p}.q_norm" in weights:
        # Qwen3-style: unrotated projections stored in the tensor dtype, then per-head RMSNorm + RoPE
        # (composition of src/machete/kernels/qwen_3_5/sm120.py:2986-2994 on qknorm_rope/ref.py:10-39)
        q, res = rms_q_matvec_rope(x_in, residual_in, weights[f"{p}.attn_norm"], weights[f"{p}.W_q"], None, None, eps,
                                   head_dim)
        q = qknorm_rope(q.to(dt).view(B, S, num_q_heads, head_dim), weights[f"{p}.q_norm"], cos, sin, eps)
        q = q.reshape(B, S, num_q_heads * head_dim).float()
        rms_kv_matvec_cache(x_in, residual_in, weights[f"{p}.attn_norm"], weights[f"{p}.W_k"], cos, sin, k_cache,
                            cache_pos, eps, False)
        k_cache[:, cache_pos:cache_pos + S] = qknorm_rope(k_cache[:, cache_pos:cache_pos + S].clone(),
                                                          weights[f"{p}.k_norm"], cos, sin, eps)
    else:
        q, res = rms_q_matvec_rope(x_in, residual_in, weights[f"{p}.attn_norm"], weights[f"{p}.W_q"], cos, sin, eps,
                                   head_dim)
        rms_kv_matvec_cache(x_in, residual_in, weights[f"{p}.attn_norm"], weights[f"{p}.W_k"], cos, sin, k_cache,
                            cache_pos, eps, True)
    rms_kv_matvec_cache(x_in, residual_in, weights[f"{p}.attn_norm"], weights[f"{p}.W_v"], cos, sin, v_cache,
                        cache_pos, eps, False)
    q4 = rnd(q).view(B, S, num_q_heads, head_dim)
    n = cache_pos + S
    attn = attention_bshd(q4, k_cache[:, :n], v_cache[:, :n], causal=False)
    attn = rnd(attn.float()).reshape(B, S, num_q_heads * head_dim)
    res2 = rnd(matvec_residual(attn, weights[f"{p}.W_o"], res))
    hmid = rnd(rms_gate_up_silu(res2, weights[f"{p}.mlp_norm"], weights[f"{p}.W_gate"], weights[f"{p}.W_up"], eps))
    x_out = rnd(matvec(hmid, weights[f"{p}.W_down"]))
    return x_out.to(dt), res2.to(dt)


def decode_model(*, weights, x, residual, k_caches, v_caches, cache_pos, final_norm, lm_head, num_layers, eps=1e-5,
                 num_q_heads=32, num_kv_heads=8, head_dim=64, return_hidden=False):
    """Whole decode step: layers, final add + norm, LM head, greedy token
    (composition of src/machete/kernels/llama1b/sm120.py:4679-4762 on the sm100 layer).
    Returns (logits fp32 (B, S, V), top values, top indices); with ``return_hidden`` also the last
    layer's (x_out, residual_out), the two tensors whose sum the final norm reads."""
    for l in range(num_layers):
        x, residual = decode_layer(weights=weights, layer_idx=l, x_in=x, residual_in=residual, k_cache=k_caches[l],
                                   v_cache=v_caches[l], cache_pos=cache_pos, eps=eps, num_q_heads=num_q_heads,
                                   num_kv_heads=num_kv_heads, head_dim=head_dim)
    logits = final_rms_lm_head(x, final_norm, lm_head, eps, residual_in=residual)
    v, i = top1(logits)
    if return_hidden:
        return logits, v, i, x, residual
    return logits, v, i


def parity_metrics(got, want) -> Tuple[float, float]:
    """(max abs error, cosine similarity) of two tensors, computed in fp64."""
    g, w = got.double().flatten(), want.double().flatten()
    err = float((g - w).abs().max()) if g.numel() else 0.0
    den = float(g.norm() * w.norm())
    cos = float((g @ w) / den) if den > 0 else 1.0
    return err, cos
