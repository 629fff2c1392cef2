"""GLU: ``y = act(x[..., :D]) * x[..., D:]`` (reference: src/machete/kernels/glu/glu.py:316-719)."""

from __future__ import annotations

from ... import _native as N
from ...megakernel.lowering import Region, elem_type, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._elementwise import ew_op, rows_view

_ACT = {"silu": N.TR_SILU, "relu": N.TR_RELU, "identity": N.TR_NONE}


class GLUOp(Op):
    """Gated linear unit on a packed ``[gate | up]`` last dimension."""

    reads = {"x": (None, ("B", "S", "N"))}
    writes = {"y": (None, ("B", "S", "D"))}
    tile = ("B", "S", "D")
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, tile_sizes=None, activation="silu", page_size=DEFAULT_PAGE_SIZE, **tensors):
        if activation not in _ACT:
            raise ValueError(f"Unknown activation: {activation}")
        x, y = tensors["x"], tensors["y"]
        if x.shape[-1] != 2 * y.shape[-1]:
            raise ValueError(f"GLUOp: x last dim {x.shape[-1]} must be twice y last dim {y.shape[-1]}")
        tile_sizes = dict(tile_sizes or {})
        tile_sizes = {"B": 1, "S": min(int(tile_sizes.get("S", 16)), int(x.shape[1])),
                      "D": int(tile_sizes.get("D", y.shape[-1]))}
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["activation"] = activation
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=ops[0].static_dims.get("page_size", DEFAULT_PAGE_SIZE))

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        x, y = t["x"], t["y"]
        if x.dtype != y.dtype:
            raise ValueError("GLUOp: x and y must share a dtype")
        rows, xs = rows_view(x, "x")
        _, ys = rows_view(y, "y")
        op = ew_op(cls.__name__, N.OP_GLU, rows, "glu")
        op.i = {N.EW_ROWS: rows, N.EW_D: int(y.shape[-1]), N.EW_T: elem_type(x, "GLUOp"),
                N.EW_ACT: _ACT[sop.static_dims.get("activation", "silu")]}
        op.p = {N.EW_P_X: x.data_ptr(), N.EW_P_Y: y.data_ptr()}
        op.s = {N.EW_S_X: xs, N.EW_S_Y: ys}
        op.reads = [Region(meta_of(x, "x"))]
        op.writes = [Region(meta_of(y, "y"))]
        op.keep = [x, y]
        return [op]


DirectGLUOp = GLUOp

__all__ = ["GLUOp", "DirectGLUOp"]
