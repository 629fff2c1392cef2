"""Shared helpers of the test-suite: seeded inputs and the parity bar."""

from __future__ import annotations

import math

import torch

import oracle

BF16_MAX_ABS = 2e-2      # max-abs error bound for bf16 math against the fp32 oracle
BF16_COSINE = 0.999      # cosine-similarity bound


def bf16_ulp(value: float) -> float:
    """Spacing of bf16 numbers (8 significant bits) at magnitude ``value``."""
    return 2.0 ** (math.floor(math.log2(abs(value))) - 7) if value else 0.0


def parity_bar(want, roundings: int = 1) -> float:
    """THE parity bar of this suite for 16-bit results against the fp32 oracle: max-abs error at most
    2e-2, or ``roundings`` bf16 ulps of the largest expected value where that is more (a tensor stored
    in bf16 cannot be closer than half an ulp, and a residual stream of magnitude 3 has ulps of
    1.6e-2; ``roundings`` counts the bf16 stores on the path that the fp32 oracle does not make)."""
    top = float(want.detach().abs().max()) if want.numel() else 0.0
    return max(BF16_MAX_ABS, roundings * bf16_ulp(top))


def assert_parity(got, want, what="", atol=None, cos=BF16_COSINE, roundings=1):
    """max-abs error <= parity_bar(want, roundings) (or an explicit ``atol``) and cosine >= 0.999."""
    got, want = got.detach().cpu().float(), want.detach().cpu().float()
    bar = parity_bar(want, roundings) if atol is None else atol
    err, c = oracle.parity_metrics(got, want)
    assert err <= bar and c >= cos, f"{what}: max-abs {err:.4g} (<= {bar:.4g}), cosine {c:.6f} (>= {cos})"


def assert_greedy_token(got_index, got_value, logits, want_index, what=""):
    """The arg-max index must equal the oracle's, bit for bit, unless the oracle's own top two logits
    are closer than the parity bar (then either is a correct greedy token); the value the kernel
    reports must be the oracle's logit at the index it chose, within the bar.  The bar counts two
    roundings: the hidden state the head reads was stored in 16 bits twice (layer output, residual)."""
    bar = parity_bar(logits, roundings=2)
    top2 = logits.float().topk(2, dim=-1).values
    for b in range(logits.shape[0]):
        gi = int(got_index[b].reshape(-1)[0])
        if float(top2[b].reshape(-1, 2)[0, 0] - top2[b].reshape(-1, 2)[0, 1]) > bar:
            assert gi == int(want_index[b].reshape(-1)[0]), f"{what}: greedy token differs for row {b}"
        assert abs(float(got_value[b].reshape(-1)[0]) - float(logits[b].reshape(-1, logits.shape[-1])[0, gi])) <= bar, \
            f"{what}: reported maximum differs from the oracle's logit for row {b}"


def rope_tables(length, d2, theta=500000.0, dtype=torch.bfloat16, device="cpu"):
    inv = 1.0 / (theta ** (torch.arange(0, d2, dtype=torch.float32) / d2))
    ang = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype).to(device), torch.sin(ang).to(dtype).to(device)


def llama_weights(num_layers, hidden, inter, q_dim, kv_dim, d2, max_len, seed=0, device="cpu", theta=500000.0):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16

    def w(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(bf).to(device)

    def nw(n):
        return (1.0 + torch.randn(n, generator=g) * 0.02).to(bf).to(device)

    cos, sin = rope_tables(max_len, d2, theta, bf, device)
    weights = {"cos": cos, "sin": sin}
    for l in range(num_layers):
        p = f"layer.{l}"
        weights[f"{p}.attn_norm"], weights[f"{p}.mlp_norm"] = nw(hidden), nw(hidden)
        weights[f"{p}.W_q"], weights[f"{p}.W_k"], weights[f"{p}.W_v"] = w(q_dim, hidden), w(kv_dim, hidden), w(kv_dim, hidden)
        weights[f"{p}.W_o"] = w(hidden, q_dim)
        weights[f"{p}.W_gate"], weights[f"{p}.W_up"] = w(inter, hidden), w(inter, hidden)
        weights[f"{p}.W_down"] = w(hidden, inter)
    return weights


def to_cpu(weights):
    return {k: v.detach().cpu() for k, v in weights.items()}
