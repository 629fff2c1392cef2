"""Generate the golden fixtures in this directory from the reference's own functions.

Run where a checkout of the reference is available, with ``REFERENCE_ROOT`` pointing at it::

    REFERENCE_ROOT=<checkout of b-albar/machete> python tests/golden/make_golden.py

It loads the reference's PyTorch reference modules *by file path* (they need
only ``torch``), runs them on seeded inputs and stores inputs and outputs in
``golden_ops.pt`` and ``golden_nvfp4.pt``.  The tests never need the reference:
they replay these files against ``oracle/`` and against the CUDA kernels.
"""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import torch

REF = Path(os.environ.get("REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))) / "src" / "machete"
HERE = Path(__file__).resolve().parent


def load(rel: str, name: str):
    spec = importlib.util.spec_from_file_location(name, REF / rel)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod   # dataclasses resolve annotations through sys.modules
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    rms = load("kernels/rms_norm/ref.py", "ref_rms")
    rope = load("kernels/rope/ref.py", "ref_rope")
    qkn = load("kernels/qknorm_rope/ref.py", "ref_qkn")
    glu = load("kernels/glu/ref.py", "ref_glu")
    att = load("kernels/attention/ref.py", "ref_att")
    nv = load("quantization/nvfp4.py", "ref_nvfp4")

    g = torch.Generator().manual_seed(42)
    bf = torch.bfloat16

    def rn(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(dtype)

    cases = []
    # RMSNorm family
    for dtype in (bf, torch.float16, torch.float32):
        x, w = rn(2, 3, 256, dtype=dtype), (1 + rn(256, dtype=torch.float32, scale=0.02)).to(dtype)
        for residual in (False, True):
            for gemma in (False, True):
                cases.append(dict(op="rmsnorm", x=x, weight=w, eps=1e-6, residual=residual, gemma=gemma,
                                  y=rms.rmsnorm_pytorch(x, w, eps=1e-6, residual=residual, gemma=gemma)))
    x, r, w = rn(1, 4, 2048), rn(1, 4, 2048), (1 + rn(2048, dtype=torch.float32, scale=0.02)).to(bf)
    y, ro = rms.fused_add_rmsnorm_pytorch(x, r, w, eps=1e-5)
    cases.append(dict(op="fused_add_rmsnorm", x=x, residual_in=r, weight=w, eps=1e-5, y=y, residual_out=ro))
    gate = rn(1, 4, 2048)
    cases.append(dict(op="rmsnorm_gated", x=x, gate=gate, weight=w, eps=1e-6,
                      y=rms.rmsnorm_gated_pytorch(x, gate, w, eps=1e-6)))
    # RoPE: full and partial rotary
    for hd, d2 in ((64, 32), (128, 64), (128, 32)):
        q = rn(2, 5, 4, hd)
        ang = torch.rand(16, d2, generator=g) * 6.28
        cos, sin = torch.cos(ang).to(bf), torch.sin(ang).to(bf)
        cases.append(dict(op="rope", q=q, cos=cos, sin=sin, y=rope.rope_pytorch(q, cos, sin)))
        nw = (1 + rn(hd, dtype=torch.float32, scale=0.1)).to(bf)
        cases.append(dict(op="qknorm_rope", q=q, norm_weight=nw, cos=cos, sin=sin, eps=1e-6,
                          y=qkn.qknorm_rope_pytorch(q, nw, cos, sin, eps=1e-6)))
    # GLU
    x = rn(2, 3, 512)
    for act in ("silu", "relu", "identity"):
        cases.append(dict(op="glu", x=x, activation=act, y=glu.glu_pytorch(x, act)))
    # attention: MHA, GQA, causal, decode-shaped
    for (bhq, group, m, n, d, causal) in ((4, 1, 1, 100, 64, False), (8, 4, 1, 333, 64, False),
                                          (8, 4, 16, 96, 128, True), (4, 2, 16, 64, 128, False)):
        q, k, v = rn(bhq, m, d), rn(bhq // group, n, d), rn(bhq // group, n, d)
        cases.append(dict(op="attention", q=q, k=k, v=v, causal=causal, kv_group_size=group,
                          y=att.flash_attention_pytorch(q, k, v, causal=causal, kv_group_size=group)))
    torch.save(cases, HERE / "golden_ops.pt")

    # NVFP4: random weights, exact threshold ties, zero groups, negative zero
    qcases = []
    w = rn(8, 256, dtype=torch.float32, scale=0.02)
    w[1, :32] = 0.0                                      # an all-zero group -> scale 1.0
    tie = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]) / 6.0 * 0.12   # land on the thresholds
    w[2, :8] = tie
    w[2, 8:16] = -tie
    w[2, 16] = 0.12                                      # the group's amax
    for dtype in (torch.float32, bf, torch.float16):
        wq = w.to(dtype)
        q = nv.quantize_nvfp4_weight(wq, group_size=32)
        qcases.append(dict(weight=wq, group_size=32, packed=q.packed, scales=q.scales,
                           dequant=nv.dequantize_nvfp4_weight(q)))
    torch.save(qcases, HERE / "golden_nvfp4.pt")
    print("wrote", HERE / "golden_ops.pt", HERE / "golden_nvfp4.pt")


if __name__ == "__main__":
    main()
