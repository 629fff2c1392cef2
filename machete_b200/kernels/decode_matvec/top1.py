"""Greedy-token LM head: fused final add + RMSNorm + vocabulary matvec + arg-max.

The reference's B200 path writes full bf16 logits (``FinalRmsLmHeadSm100Op``,
src/machete/kernels/decode_matvec/sm100.py:574) and only its sm120 path has a
top-1 head, as a partial/reduce pair (``Llama1BFinalAddRmsTop1PartialLmHead
KStreamSm120Op`` / ``Llama1BReduceTop1PartialsSm120Op``,
src/machete/kernels/llama1b/sm120.py:3151, 3464).  Here every vocabulary unit
folds its 16 rows into one 64-bit key per activation row with ``atomicMax``
(order-preserving float bits in the high word, ``~index`` in the low word, so
ties resolve to the lowest index exactly like ``argmax``), and a one-unit
finalise op unpacks the keys and clears them for the next launch.
"""

from __future__ import annotations

import torch

from ... import _native as N
from ...megakernel.lowering import NativeOp, Region, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Float32, Int32, Int64, Op
from .._matvec import Weight, dense_weight, lower_matvec, nvfp4_weight


class FinalAddRmsTop1LmHeadSm100Op(Op):
    uses_dense_weights = True
    """keys[b, s] = max over vocab of (logit, index); logits = rms(x + residual_in) * w @ W^T."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight": (None, ("V", "K")),
    }
    writes = {"top_keys": (Int64, ("B", "S"))}
    tile = ("B", "S", "V")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, index_offset=0, **tensors):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 16)
        tile_sizes.setdefault("V", 16)
        keys = tensors["top_keys"]
        if keys.dtype != torch.int64 or not keys.is_contiguous():
            raise ValueError("top_keys must be a contiguous int64 (B, S) tensor, zero-initialised")
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        op.static_dims["index_offset"] = int(index_offset)   # first vocabulary row of this rank's shard
        return [op]

    @classmethod
    def _weight(cls, sop) -> Weight:
        return dense_weight(sop.tensor_refs["weight"])

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        has_res = "residual_in" in t and t["residual_in"] is not None
        nop = lower_matvec(cls.__name__, ctx, w0=cls._weight(sop), x=t["x"], out=t["top_keys"],
                           out_strides=(0, 0, 0), pro=N.PRO_ADD_RMS if has_res else N.PRO_RMS,
                           norm_weight=t["norm_weight"], residual_in=t.get("residual_in"), epi=N.EPI_TOP1,
                           eps=float(sop.static_dims.get("eps", 1e-5)), kind="lm_head_top1",
                           index_offset=int(sop.static_dims.get("index_offset", 0)))
        nop.zero_on_reset = [t["top_keys"]]      # the finalise op clears them; an aborted launch may not get there
        return [nop]


class FinalAddRmsTop1LmHeadNvfp4Sm100Op(FinalAddRmsTop1LmHeadSm100Op):
    """NVFP4-weight variant (``weight_packed``, ``weight_scales``)."""

    uses_nvfp4 = True
    uses_dense_weights = False
    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight_packed": (None, ("V", "K2")),
        "weight_scales": (None, ("V", "G")),
    }
    writes = {"top_keys": (Int64, ("B", "S"))}
    tile = ("B", "S", "V")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, group_size=32, global_scale=1.0,
                 index_offset=0, **tensors):
        ops = super().schedule(tile_sizes=tile_sizes, page_size=page_size, eps=eps, index_offset=index_offset,
                               **tensors)
        ops[0].static_dims["group_size"] = group_size
        ops[0].params["global_scale"] = float(global_scale)
        return ops

    @classmethod
    def _weight(cls, sop) -> Weight:
        t = sop.tensor_refs
        return nvfp4_weight(t["weight_packed"], t["weight_scales"], int(sop.static_dims["group_size"]),
                            sop.params.get("global_scale", 1.0))


class ReduceTop1Sm100Op(Op):
    """Unpack ``top_keys`` into ``top_values (B, S) f32`` / ``top_indices (B, S) i32`` and clear the keys."""

    reads = {"top_keys": (Int64, ("B", "S"))}
    writes = {"top_values": (Float32, ("B", "S")), "top_indices": (Int32, ("B", "S"))}
    tile = ("B",)
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, feedback=None, **tensors):
        """``feedback`` (not in the reference): ``dict(embedding=(V, hidden) table, x_in=(B, S, hidden)
        input rows of the next step, position=one-element int32 CUDA tensor or None)`` makes the op
        copy each greedy token's embedding row into ``x_in`` and advance the position by S, so the
        next launch decodes the next token with no host work in between."""
        for name, dt in (("top_values", torch.float32), ("top_indices", torch.int32)):
            if tensors[name].dtype != dt or not tensors[name].is_contiguous():
                raise ValueError(f"{name} must be a contiguous {dt} (B, S) tensor")
        op = cls._schedule_single(tile_sizes={}, **tensors)
        op.static_dims["page_size"] = page_size
        if feedback is not None:
            emb, x_in = feedback["embedding"], feedback["x_in"]
            if emb.ndim != 2 or emb.stride(1) != 1 or x_in.ndim != 3 or x_in.stride(2) != 1 or emb.dtype != x_in.dtype \
                    or emb.shape[1] != x_in.shape[2] or x_in.shape[0] * x_in.shape[1] != tensors["top_indices"].numel():
                raise ValueError("feedback: embedding must be (V, hidden) and x_in (B, S, hidden) of one 16-bit dtype")
            if not x_in.is_contiguous():
                raise ValueError("feedback: x_in must be contiguous")
            op.params["feedback"] = dict(feedback)
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        keys, vals, idxs = t["top_keys"], t["top_values"], t["top_indices"]
        op = NativeOp(name=cls.__name__, opcode=N.OP_TOP1_FINAL, n_units=1, kind="top1_final")
        op.i = {N.EW_ROWS: keys.numel()}
        op.p = {N.EW_P_X: keys.data_ptr(), N.EW_P_Y: vals.data_ptr(), N.EW_P_W: idxs.data_ptr()}
        op.reads = [Region(meta_of(keys, "top_keys"))]
        op.writes = [Region(meta_of(keys, "top_keys")), Region(meta_of(vals, "top_values")),
                     Region(meta_of(idxs, "top_indices"))]
        op.keep = [keys, vals, idxs]
        fb = sop.params.get("feedback")
        if fb is not None:
            emb, x_in, pos = fb["embedding"], fb["x_in"], fb.get("position")
            op.i.update({N.EW_FLAGS: N.EWF_FEEDBACK, N.EW_D: int(emb.shape[1]), N.EW_S: int(x_in.shape[1])})
            op.p.update({N.EW_P_RES_IN: emb.data_ptr(), N.EW_P_RES_OUT: x_in.data_ptr(),
                         N.EW_P_GATE: pos.data_ptr() if pos is not None else 0})
            op.s = {N.EW_S_RI: emb.stride(0), N.EW_S_RO: int(emb.shape[1])}
            op.reads.append(Region(meta_of(emb, "embedding")))
            op.writes.append(Region(meta_of(x_in, "x_in")))
            op.keep += [emb, x_in] + ([pos] if pos is not None else [])
        return [op]


def schedule_final_top1_sm100(*, x, residual_in, final_norm, lm_head, top_values, top_indices, seq_len,
                              page_size=DEFAULT_PAGE_SIZE, eps=1e-5, lm_head_scales=None, group_size=32,
                              global_scale=1.0, tp_peers=None, feedback=None):
    """Final add + RMSNorm + LM head + greedy token, without materialising logits.

    With ``tp_peers`` the LM head is this rank's vocabulary shard (rows
    ``rank * V_local ...``): the ranks exchange their best keys inside the
    kernel and every rank ends up with the global greedy token.
    """
    keys = torch.zeros(top_values.shape, dtype=torch.int64, device=top_values.device)
    tiles = {"S": seq_len, "V": 16}
    idx0 = 0 if tp_peers is None else tp_peers.rank * int(lm_head.shape[0])
    if lm_head_scales is None:
        ops = FinalAddRmsTop1LmHeadSm100Op.schedule(x=x, residual_in=residual_in, norm_weight=final_norm,
                                                    weight=lm_head, top_keys=keys, tile_sizes=tiles,
                                                    page_size=page_size, eps=eps, index_offset=idx0)
    else:
        ops = FinalAddRmsTop1LmHeadNvfp4Sm100Op.schedule(
            x=x, residual_in=residual_in, norm_weight=final_norm, weight_packed=lm_head,
            weight_scales=lm_head_scales, top_keys=keys, tile_sizes=tiles, page_size=page_size, eps=eps,
            group_size=group_size, global_scale=global_scale, index_offset=idx0)
    final_keys = keys
    if tp_peers is not None:
        from ..allreduce import AllReduceTop1KeysSm100Op

        final_keys = torch.zeros_like(keys)
        ops += AllReduceTop1KeysSm100Op.schedule(peers=tp_peers, top_keys=keys, top_keys_out=final_keys)
    ops += ReduceTop1Sm100Op.schedule(top_keys=final_keys, top_values=top_values, top_indices=top_indices,
                                      page_size=page_size, feedback=feedback)
    return ops


__all__ = ["FinalAddRmsTop1LmHeadSm100Op", "FinalAddRmsTop1LmHeadNvfp4Sm100Op", "ReduceTop1Sm100Op",
           "schedule_final_top1_sm100"]
