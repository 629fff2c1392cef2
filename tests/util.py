"""Shared helpers of the test-suite: seeded inputs and the parity bar."""

from __future__ import annotations

import math

import torch

import oracle

BF16_MAX_ABS = 2e-2      # max-abs error bound for bf16 math against the fp32 oracle
BF16_COSINE = 0.999      # cosine-similarity bound


def assert_parity(got, want, what="", atol=BF16_MAX_ABS, cos=BF16_COSINE):
    err, c = oracle.parity_metrics(got.detach().cpu().float(), want.detach().cpu().float())
    assert err <= atol and c >= cos, f"{what}: max-abs {err:.4g} (<= {atol}), cosine {c:.6f} (>= {cos})"


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
