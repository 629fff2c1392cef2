"""``GemmOp``: ``C[B,S,N] = A[B,S,K] @ W[N,K]^T`` with fp32 accumulation.

API mirror of the reference (src/machete/kernels/gemm/gemm.py:290-1160):
``schedule(tile_sizes=None, page_size, activation=None, has_a_scale=0,
a=, b=, c=)``, ``tile_sizes`` keys ``S, N, K`` (``K`` is popped into
``static_dims["tile_K"]``), ``activation in {None, 'relu', 'silu'}``.

Up to 32 rows (``B*S``) run as one pass of the weight-streaming tensor-core
matvec unit; more rows are processed in chunks of 32, each chunk re-streaming
the weights; from 64 rows up ``GemmSm100Op`` / ``gemm_sm100`` (a tcgen05 tile, its own
launch) is the faster path.  ``has_a_scale`` (a training-backward feature) is
rejected.
"""

from __future__ import annotations

from ... import _native as N
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._matvec import dense_weight, lower_matvec

_ACT = {None: N.TR_NONE, "relu": N.TR_RELU, "silu": N.TR_SILU}
ACT_MAP = {"relu": 1, "silu": 2}


class GemmOp(Op):
    uses_dense_weights = True
    reads = {
        "a": (None, ("B", "S", "K")),
        "a_scale": (None, ("B", "S", "K")),
        "b": (None, ("N", "K")),
    }
    writes = {"c": (None, ("B", "S", "N"))}
    tile = ("B", "S", "N")
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, activation=None, has_a_scale=0, **tensors):
        if activation not in _ACT:
            raise ValueError(f"Unknown activation: {activation}")
        if has_a_scale:
            raise ValueError("GemmOp: a_scale (activation-backward scaling) is not supported by the decode build")
        tensors = dict(tensors)
        tensors.setdefault("a_scale", tensors["a"])
        ts = dict(tile_sizes or {})
        ts.setdefault("B", 1)
        ts.setdefault("S", 16)
        ts.setdefault("N", 16)
        tile_k = ts.pop("K", 512)
        op = cls._schedule_single(tile_sizes=ts, **tensors)
        op.static_dims["tile_K"] = tile_k
        op.static_dims["page_size"] = page_size
        op.static_dims["has_a_scale"] = has_a_scale
        if activation is not None:
            op.static_dims["activation"] = ACT_MAP[activation]
        op.params["activation"] = activation
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=max(op.static_dims.get("page_size", DEFAULT_PAGE_SIZE) for op in ops))

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        a, b, c = t["a"], t["b"], t["c"]
        B, S, K = (int(v) for v in a.shape)
        n_out = int(b.shape[0])
        tr = _ACT[sop.params.get("activation")]
        w = dense_weight(b)
        M = B * S
        if M <= 32:
            return [lower_matvec(cls.__name__, ctx, w0=w, x=a, out=c, out_strides=(c.stride(0), c.stride(1), n_out),
                                 tr=tr, kind="gemm")]
        # more rows: chunks of 32 rows of the flattened (B*S, K) activations
        if not (a.is_contiguous() and c.is_contiguous()):
            raise ValueError("GemmOp: more than 32 rows need contiguous a and c")
        a2, c2 = a.view(1, M, K), c.view(1, M, n_out)
        out = []
        for r0 in range(0, M, 32):
            r1 = min(M, r0 + 32)
            ac, cc = a2[:, r0:r1], c2[:, r0:r1]
            nop = lower_matvec(f"{cls.__name__}[{r0}:{r1}]", ctx, w0=w, x=ac, out=cc,
                               out_strides=(cc.stride(0), cc.stride(1), n_out), tr=tr, kind="gemm")
            nop.keep += [a2, c2]
            out.append(nop)
        return out


from .gemm_sm100 import GemmSm100Op, PackedWeight, gemm_pack_weight, gemm_sm100, gemm_workspace  # noqa: E402

__all__ = ["GemmOp", "ACT_MAP", "GemmSm100Op", "gemm_sm100", "gemm_workspace", "gemm_pack_weight",
           "PackedWeight"]
