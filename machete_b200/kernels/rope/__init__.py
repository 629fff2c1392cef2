"""RoPE in place on ``q (B, S, NH, HD)`` (reference: src/machete/kernels/rope/rope.py:41-157).

Split-half rotation ``o[:d2] = q0*c - q1*s; o[d2:2*d2] = q1*c + q0*s`` with the
tail ``[2*d2, HD)`` untouched (partial rotary), as the reference's oracle
``rope_pytorch`` (rope/ref.py:18-43).
"""

from __future__ import annotations

from ... import _native as N
from ...megakernel.lowering import Region, elem_type, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._elementwise import ew_op


class RopeOp(Op):
    reads = {
        "q": (None, ("B", "S", "NH", "HD")),
        "cos": (None, ("SL", "D2")),
        "sin": (None, ("SL", "D2")),
    }
    writes = {"q": (None, ("B", "S", "NH", "HD"))}
    tile = ("B", "S", "NH")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, **tensors):
        q, cos, sin = tensors["q"], tensors["cos"], tensors["sin"]
        if q.ndim != 4:
            raise ValueError(f"RopeOp: q must be (B, S, NH, HD), got {tuple(q.shape)}")
        if cos.shape != sin.shape or 2 * cos.shape[1] > q.shape[-1]:
            raise ValueError("RopeOp: cos/sin must be (SL, D2) with 2*D2 <= HD")
        if cos.shape[0] < q.shape[1]:
            raise ValueError("RopeOp: cos/sin tables are shorter than the sequence")
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 1)
        tile_sizes.setdefault("NH", int(q.shape[2]))
        if q.shape[2] % tile_sizes["NH"]:
            raise ValueError(f"RopeOp: tile_size_NH={tile_sizes['NH']} must divide NH={q.shape[2]}")
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=ops[0].static_dims.get("page_size", DEFAULT_PAGE_SIZE))

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        q, cos, sin = t["q"], t["cos"], t["sin"]
        B, S, NH, HD = (int(v) for v in q.shape)
        if q.stride(-1) != 1 or cos.stride(-1) != 1 or sin.stride(-1) != 1 or cos.stride(0) != sin.stride(0):
            raise ValueError("RopeOp: q, cos and sin need unit innermost strides and a shared table stride")
        if cos.dtype != q.dtype or sin.dtype != q.dtype:
            raise ValueError("RopeOp: cos/sin must have q's dtype")
        if B != 1 and q.stride(0) != q.stride(1) * S:
            raise ValueError("RopeOp: (B, S) must collapse into rows")
        op = ew_op(cls.__name__, N.OP_ROPE, B * S, "rope")
        op.i = {N.EW_ROWS: B * S, N.EW_S: S, N.EW_H: NH, N.EW_D: HD, N.EW_D2: int(cos.shape[1]),
                N.EW_T: elem_type(q, "RopeOp")}
        op.p = {N.EW_P_X: q.data_ptr(), N.EW_P_COS: cos.data_ptr(), N.EW_P_SIN: sin.data_ptr()}
        op.s = {N.EW_S_X: q.stride(1), N.EW_S_X_H: q.stride(2), N.EW_S_COS: cos.stride(0)}
        op.reads = [Region(meta_of(q, "q")), Region(meta_of(cos, "cos")), Region(meta_of(sin, "sin"))]
        op.writes = [Region(meta_of(q, "q"))]
        op.keep = [q, cos, sin]
        return [op]


__all__ = ["RopeOp"]
