"""RMSNorm forward and its variants.

API mirror of the reference's ``RMSNormOp`` (src/machete/kernels/rms_norm/
rms_norm.py:162-322): ``schedule(tile_sizes, residual, gemma, per_row_weight,
page_size, **tensors)`` with ``x, y (B, S, D)``, ``weight (D,)`` or
``(B, S, D)``, optional ``residual_in``/``residual_out`` (fused add: the sum is
rounded to the tensor dtype before normalising, rms_norm.py:448-456) and
``gate`` (gated: ``y = rms(x) * silu(gate)``).  Numerics follow the oracle
``rmsnorm_pytorch`` / ``fused_add_rmsnorm_pytorch`` (rms_norm/ref.py:17-116).

``eps``: the reference op hard-codes 1e-6 (rms_norm.py:51, 477) and silently
drops an ``eps=`` keyword; this op honours the keyword and defaults to 1e-6.
"""

from __future__ import annotations

import torch

from ... import _native as N
from ...megakernel.lowering import Region, elem_type, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._elementwise import ew_op, rows_view

RMSNORM_EPS = 1e-6


class RMSNormOp(Op):
    reads = {
        "x": (None, ("B", "S", "D")),
        "weight": (None, ("B", "S", "D")),
        "residual_in": (None, ("B", "S", "D")),
        "gate": (None, ("B", "S", "D")),
    }
    writes = {
        "y": (None, ("B", "S", "D")),
        "residual_out": (None, ("B", "S", "D")),
    }
    tile = ("B", "S", "D")
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, tile_sizes=None, residual=False, gemma=False, per_row_weight=False,
                 page_size=DEFAULT_PAGE_SIZE, eps=RMSNORM_EPS, **tensors):
        tensors = {k: v for k, v in tensors.items() if isinstance(v, torch.Tensor)}
        x, y = tensors["x"], tensors["y"]
        w = tensors["weight"]
        shared_weight = w.ndim == 1
        if shared_weight:
            if w.shape[0] != x.shape[-1]:
                raise ValueError(f"RMSNormOp: weight has {w.shape[0]} elements, x has D={x.shape[-1]}")
            tensors["weight"] = w.reshape(1, 1, -1).expand(x.shape[0], x.shape[1], -1)
        has_residual = "residual_in" in tensors
        has_gate = "gate" in tensors
        tensors.setdefault("residual_in", x)
        tensors.setdefault("residual_out", y)
        tensors.setdefault("gate", x)
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes["S"] = max(1, min(int(tile_sizes.get("S", 8)), int(x.shape[1])))
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        sd = op.static_dims
        if residual:
            sd["residual"] = 1
        if gemma:
            sd["gemma"] = 1
        if has_residual:
            sd["has_residual"] = 1
        if has_gate:
            sd["has_gate"] = 1
        if per_row_weight or not shared_weight:
            sd["per_row_weight"] = 1
        sd["page_size"] = page_size
        sd["eps"] = float(eps)
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=ops[0].static_dims.get("page_size", DEFAULT_PAGE_SIZE))

    @classmethod
    def lower(cls, sop, ctx):
        t, sd = sop.tensor_refs, sop.static_dims
        x, y, w = t["x"], t["y"], t["weight"]
        if y.dtype != x.dtype or w.dtype != x.dtype:
            raise ValueError("RMSNormOp: x, y and weight must share a dtype")
        rows, xs = rows_view(x, "x")
        _, ys = rows_view(y, "y")
        flags = 0
        if sd.get("residual"):
            flags |= N.EWF_RESIDUAL
        if sd.get("gemma"):
            flags |= N.EWF_GEMMA
        op = ew_op(cls.__name__, N.OP_RMSNORM, rows, "rmsnorm")
        op.p = {N.EW_P_X: x.data_ptr(), N.EW_P_Y: y.data_ptr(), N.EW_P_W: w.data_ptr()}
        op.s = {N.EW_S_X: xs, N.EW_S_Y: ys}
        op.reads = [Region(meta_of(x, "x")), Region(meta_of(w, "weight"))]
        op.writes = [Region(meta_of(y, "y"))]
        op.keep = [x, y, w]
        if sd.get("per_row_weight"):
            flags |= N.EWF_ROW_WEIGHT
            op.s[N.EW_S_W] = rows_view(w, "weight")[1]
        if sd.get("has_residual"):
            ri, ro = t["residual_in"], t["residual_out"]
            if ri.dtype != x.dtype or ro.dtype != x.dtype or ri.shape != x.shape or ro.shape != x.shape:
                raise ValueError("RMSNormOp: residual tensors must match x")
            flags |= N.EWF_FUSED_ADD
            op.p[N.EW_P_RES_IN], op.p[N.EW_P_RES_OUT] = ri.data_ptr(), ro.data_ptr()
            op.s[N.EW_S_RI], op.s[N.EW_S_RO] = rows_view(ri, "residual_in")[1], rows_view(ro, "residual_out")[1]
            op.reads.append(Region(meta_of(ri, "residual_in")))
            op.writes.append(Region(meta_of(ro, "residual_out")))
            op.keep += [ri, ro]
        if sd.get("has_gate"):
            g = t["gate"]
            if g.dtype != x.dtype or g.shape != x.shape:
                raise ValueError("RMSNormOp: gate must match x")
            flags |= N.EWF_GATED
            op.p[N.EW_P_GATE] = g.data_ptr()
            op.s[N.EW_S_G] = rows_view(g, "gate")[1]
            op.reads.append(Region(meta_of(g, "gate")))
            op.keep.append(g)
        op.i = {N.EW_ROWS: rows, N.EW_D: int(x.shape[-1]), N.EW_FLAGS: flags, N.EW_T: elem_type(x, "RMSNormOp")}
        op.f = {N.EW_F_EPS: float(sd.get("eps", RMSNORM_EPS))}
        return [op]


__all__ = ["RMSNormOp", "RMSNORM_EPS"]
