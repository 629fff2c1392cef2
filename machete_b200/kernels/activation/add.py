"""Elementwise add: ``y = x + add`` (reference: src/machete/kernels/activation/add.py:11-31)."""

from __future__ import annotations

from ... import _native as N
from ...megakernel.lowering import Region, elem_type, meta_of
from ...megakernel.ops import Op
from .._elementwise import ew_op, rows_view


def lower_add(name, x, add, y):
    if x.shape != add.shape or x.shape != y.shape or x.dtype != add.dtype or x.dtype != y.dtype:
        raise ValueError(f"{name}: x, add and y must share shape and dtype")
    rows, xs = rows_view(x, "x")
    _, as_ = rows_view(add, "add")
    _, ys = rows_view(y, "y")
    op = ew_op(name, N.OP_ADD, rows, "add")
    op.i = {N.EW_ROWS: rows, N.EW_D: int(x.shape[-1]), N.EW_T: elem_type(x, name)}
    op.p = {N.EW_P_X: x.data_ptr(), N.EW_P_W: add.data_ptr(), N.EW_P_Y: y.data_ptr()}
    op.s = {N.EW_S_X: xs, N.EW_S_W: as_, N.EW_S_Y: ys}
    op.reads = [Region(meta_of(x, "x")), Region(meta_of(add, "add"))]
    op.writes = [Region(meta_of(y, "y"))]
    op.keep = [x, add, y]
    return op


class AddOp(Op):
    """y = x + add on (B, S, D) tensors."""

    reads = {"x": (None, ("B", "S", "D")), "add": (None, ("B", "S", "D"))}
    writes = {"y": (None, ("B", "S", "D"))}
    tile = ("B", "S")
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, tile_sizes=None, **tensors):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 1)
        return [cls._schedule_single(tile_sizes=tile_sizes, **tensors)]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        return [lower_add(cls.__name__, t["x"], t["add"], t["y"])]
