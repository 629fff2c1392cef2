"""Dump the op-level dependency pairs of fixed op lists as JSON, with whichever package is importable.

Run twice by tests/test_dep_edges_differential.py: once in a subprocess whose PYTHONPATH points at
the reference's ``src`` (package ``machete``: its InstructionStreamBuilder resolves the pairs,
src/machete/megakernel/scheduling.py:962-1120), once in-process against ``machete_b200``
(``resolve_dep_pairs``).  CPU tensors only; the reference's schedule helpers ask the CUDA runtime
for the SM count and shared memory, so those two queries are stubbed.

usage: python dep_edges_driver.py {reference|ours} OUT.json
"""

import json
import sys

import torch


class _Props:
    multi_processor_count = 148
    shared_memory_per_block_optin = 232448
    major, minor = 10, 0
    name = "stub"
    total_memory = 180 << 30


def _layer_ops(pkg, seq_len, cache_pos, splits):
    sm100 = __import__(f"{pkg}.kernels.decode_matvec.sm100", fromlist=["x"])
    bf = torch.bfloat16
    H, I, NQ, NKV, HD, B, T = 2048, 8192, 32, 8, 64, 1, 2048
    w = {"cos": torch.zeros(T, HD // 2, dtype=bf), "sin": torch.zeros(T, HD // 2, dtype=bf)}
    for name, shape in (("attn_norm", (H,)), ("mlp_norm", (H,)), ("W_q", (NQ * HD, H)), ("W_k", (NKV * HD, H)),
                        ("W_v", (NKV * HD, H)), ("W_o", (H, NQ * HD)), ("W_gate", (I, H)), ("W_up", (I, H)),
                        ("W_down", (H, I))):
        w[f"layer.0.{name}"] = torch.zeros(shape, dtype=bf)
    z = lambda *s: torch.zeros(*s, dtype=bf)                                   # noqa: E731
    sched = sm100.schedule_decode_layer_sm100(
        layer_idx=0, batch=B, seq_len=seq_len, cache_pos=cache_pos, weights=w, k_cache=z(B, T, NKV, HD),
        v_cache=z(B, T, NKV, HD), x_in=z(B, seq_len, H), residual_in=z(B, seq_len, H), x_out=z(B, seq_len, H),
        residual_out=z(B, seq_len, H), q_buf=z(B, seq_len, NQ * HD), attn_out_buf=z(B, seq_len, NQ * HD),
        mlp_h_buf=z(B, seq_len, I), page_size=32768, fa_num_splits=splits)
    return list(sched.ops), sched


def _chain_ops(pkg):
    """RMSNorm -> Gemm -> GLU -> Gemm, each stage reading the previous one's output tensor."""
    imp = lambda m: __import__(f"{pkg}.kernels.{m}", fromlist=["x"])           # noqa: E731
    RMSNormOp, GemmOp, GLUOp = imp("rms_norm").RMSNormOp, imp("gemm").GemmOp, imp("glu").GLUOp
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16)                       # noqa: E731
    B, S, D, I = 1, 64, 256, 512
    x, w, y = z(B, S, D), z(D), z(B, S, D)
    w1, h, g, w2, out = z(2 * I, D), z(B, S, 2 * I), z(B, S, I), z(D, I), z(B, S, D)
    ops = []
    ops += RMSNormOp.schedule(x=x, weight=w, y=y)
    ops += GemmOp.schedule(a=y, b=w1, c=h)
    ops += GLUOp.schedule(x=h, y=g)
    ops += GemmOp.schedule(a=g, b=w2, c=out)
    # a second block reusing the scratch tensors: write-after-read and write-after-write pairs
    ops += RMSNormOp.schedule(x=out, weight=w, y=y)
    ops += GemmOp.schedule(a=y, b=w1, c=h)
    return ops, (x, w, y, w1, h, g, w2, out)


def _pairs_reference(ops):
    from machete.megakernel.scheduling import InstructionStreamBuilder

    b = InstructionStreamBuilder()
    for op in ops:
        b.add_op(op)
    pairs = b._resolve_named_dep_pairs(b._build_buffer_producers(), b._build_tensor_ptr_deps())
    return sorted({(p.producer_idx, p.consumer_idx) for p in pairs})


def _pairs_ours(ops):
    from machete_b200.megakernel.scheduling import resolve_dep_pairs

    return sorted({(p, c) for p, c, _, _ in resolve_dep_pairs(ops)})


def main(which, out_path):
    pkg = "machete" if which == "reference" else "machete_b200"
    if which == "reference":
        torch.cuda.get_device_properties = lambda *a, **k: _Props()
        torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    pairs_of = _pairs_reference if which == "reference" else _pairs_ours
    result = {}
    cases = {
        "layer_decode_1008": lambda: _layer_ops(pkg, 1, 1008, 4),
        "layer_decode_4095": lambda: _layer_ops(pkg, 1, 2047, 8),
        "layer_s16_1008": lambda: _layer_ops(pkg, 16, 1008, 4),
        "norm_gemm_glu_gemm": lambda: _chain_ops(pkg),
    }
    for name, make in cases.items():
        try:
            ops, keep = make()
        except Exception as exc:  # a case one side cannot schedule is reported, not hidden
            result[name] = {"error": f"{type(exc).__name__}: {exc}"}
            continue
        result[name] = {"ops": [op.op_cls.__name__ for op in ops], "pairs": pairs_of(ops)}
    with open(out_path, "w") as fh:
        json.dump(result, fh)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
