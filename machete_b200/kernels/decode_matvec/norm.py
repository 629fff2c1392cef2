"""``RmsAddNormSm120Op``: fused residual add + RMSNorm as an op of its own.

API mirror of the reference's decode helper (src/machete/kernels/decode_matvec/sm120.py:1458-1518:
``x, residual_in (B, S, K)``, ``norm_weight (K,)`` -> ``residual_out = x + residual_in``,
``y = rms(x + residual_in) * norm_weight``; ``schedule(tile_sizes=None, page_size, eps=1e-5)``).
The decode layers of this build fuse that work into the staging of the projection that follows, so
the op is only needed by schedules that want the normalised row in memory.  It runs on the native
RMSNorm handler with the fused add (``kernels/rms_norm``); like ``RMSNormOp`` it normalises the sum
AFTER rounding it to the tensor dtype (the reference's op normalises the unrounded fp32 sum: the two
differ by at most half a unit in the last place of a 16-bit value).
"""

from __future__ import annotations

from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from ..rms_norm import RMSNormOp


class RmsAddNormSm120Op(Op):
    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
    }
    writes = {
        "residual_out": (None, ("B", "S", "K")),
        "y": (None, ("B", "S", "K")),
    }
    tile = ("B", "S")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, **tensors):
        ts = dict(tile_sizes or {})
        ts.setdefault("B", 1)
        ts.setdefault("S", 16)
        op = cls._schedule_single(tile_sizes=ts, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        (inner,) = RMSNormOp.schedule(x=t["x"], weight=t["norm_weight"], y=t["y"], residual_in=t["residual_in"],
                                      residual_out=t["residual_out"], eps=float(sop.static_dims.get("eps", 1e-5)))
        lowered = RMSNormOp.lower(inner, ctx)
        for nop in lowered:
            nop.name = cls.__name__
            nop.keep.append(inner)
        return lowered


RmsAddNormSm100Op = RmsAddNormSm120Op

__all__ = ["RmsAddNormSm120Op", "RmsAddNormSm100Op"]
