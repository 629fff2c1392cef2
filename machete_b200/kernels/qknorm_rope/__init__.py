"""Per-head RMSNorm + RoPE in place on ``q (M, H, D)``.

Reference: src/machete/kernels/qknorm_rope/qknorm_rope.py:47-165; numerics of
``qknorm_rope_pytorch`` (qknorm_rope/ref.py:10-39): the normalised value is
rounded to the tensor dtype before the rotation, row ``m`` uses ``cos[m]``.
"""

from __future__ import annotations

from ... import _native as N
from ...megakernel.lowering import Region, elem_type, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._elementwise import ew_op


class QKNormRopeOp(Op):
    reads = {
        "q": (None, ("M", "H", "D")),
        "norm_weight": (None, ("D",)),
        "cos": (None, ("S", "D2")),
        "sin": (None, ("S", "D2")),
    }
    writes = {"q": (None, ("M", "H", "D"))}
    tile = ("M", "H")
    dynamic_dims = ("M",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-6, cache_rows=None, **tensors):
        """``cache_rows=(lo, hi)``: ``q`` is the view of token rows [lo, hi) of a KV cache that a later
        attention op reads; only the splits that cover those rows then wait for this op."""
        q, cos, sin = tensors["q"], tensors["cos"], tensors["sin"]
        if q.ndim != 3:
            raise ValueError(f"QKNormRopeOp: q must be (M, H, D), got {tuple(q.shape)}")
        if cos.shape != sin.shape or 2 * cos.shape[1] > q.shape[-1] or cos.shape[0] < q.shape[0]:
            raise ValueError("QKNormRopeOp: cos/sin must be (S >= M, D2) with 2*D2 <= D")
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("M", 1)
        tile_sizes.setdefault("H", 1)
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        if cache_rows is not None:
            op.params["cache_rows"] = (int(cache_rows[0]), int(cache_rows[1]))
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=ops[0].static_dims.get("page_size", DEFAULT_PAGE_SIZE))

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        q, w, cos, sin = t["q"], t["norm_weight"], t["cos"], t["sin"]
        M, H, D = (int(v) for v in q.shape)
        if q.stride(-1) != 1 or cos.stride(-1) != 1 or sin.stride(-1) != 1 or cos.stride(0) != sin.stride(0):
            raise ValueError("QKNormRopeOp: q, cos and sin need unit innermost strides and a shared table stride")
        if any(x.dtype != q.dtype for x in (w, cos, sin)) or not w.is_contiguous():
            raise ValueError("QKNormRopeOp: norm_weight, cos and sin must have q's dtype")
        op = ew_op(cls.__name__, N.OP_QKNORM_ROPE, M * H, "qknorm_rope")
        op.i = {N.EW_ROWS: M, N.EW_H: H, N.EW_D: D, N.EW_D2: int(cos.shape[1]), N.EW_T: elem_type(q, "QKNormRopeOp")}
        op.f = {N.EW_F_EPS: float(sop.static_dims.get("eps", 1e-6))}
        op.p = {N.EW_P_X: q.data_ptr(), N.EW_P_W: w.data_ptr(), N.EW_P_COS: cos.data_ptr(),
                N.EW_P_SIN: sin.data_ptr()}
        op.s = {N.EW_S_X: q.stride(0), N.EW_S_X_H: q.stride(1), N.EW_S_COS: cos.stride(0)}
        op.reads = [Region(meta_of(q, "q")), Region(meta_of(w, "norm_weight")), Region(meta_of(cos, "cos")),
                    Region(meta_of(sin, "sin"))]
        op.writes = [Region(meta_of(q, "q"))]
        op.keep = [q, w, cos, sin]
        rows = sop.params.get("cache_rows")
        if rows is not None:
            op.writes[-1].axis, op.writes[-1].lo, op.writes[-1].hi = 1, rows[0], rows[1]
            op.kind = "cache_append"
        return [op]


__all__ = ["QKNormRopeOp"]
