"""Instruction-shaped decode ops for B200 and the per-layer schedule that chains them.

Same class names, tensor declarations, ``schedule()`` keywords and
``static_dims`` keys as the reference's B200 decode ops
(src/machete/kernels/decode_matvec/sm100.py: ``_RmsProjectionSm100Base`` :78,
``RmsQMatvecRopeSm100Op`` :224, ``RmsKMatvecRopeCacheSm100Op`` :256,
``RmsVMatvecCacheSm100Op`` :293, ``MatvecResidualSm100Op`` :327,
``MatvecSm100Op`` :386, ``ResidualAddSm100Op`` :441, ``RmsGateUpSiluSm100Op``
:485, ``FinalRmsLmHeadSm100Op`` :574, ``schedule_decode_layer_sm100`` :666,
``schedule_final_sm100`` :826).  The device work is different: every op here
lowers to the TMA-streamed tensor-core matvec unit instead of a
one-warp-per-row scalar loop, the RMSNorm is computed once per CTA instead of
once per 16-output tile, and the RoPE partner comes out of the same
accumulator fragment instead of a second dot product.
"""

from __future__ import annotations

import torch

from dataclasses import dataclass

from ... import _native as N
from ...megakernel.lowering import NativeOp, Region, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op
from .._matvec import dense_weight, flat_out_strides, lower_matvec

SM100_DECODE_HIDDEN_DEFAULT = 2048
SM100_DECODE_HEAD_DIM_DEFAULT = 64
SM100_DECODE_ROTARY_D2_DEFAULT = 32
SM100_DECODE_Q_DIM_DEFAULT = 2048
SM100_DECODE_KV_DIM_DEFAULT = 512
SM100_DECODE_INTERMEDIATE_DEFAULT = 8192
SM100_DECODE_VOCAB_DEFAULT = 128256
SM100_DECODE_MATVEC_BLOCK = 16
SM100_DECODE_REDUCTION_DIM_PER_WARP = 512
SM100_DECODE_NUM_Q_HEADS_DEFAULT = SM100_DECODE_Q_DIM_DEFAULT // SM100_DECODE_HEAD_DIM_DEFAULT
SM100_DECODE_NUM_KV_HEADS_DEFAULT = SM100_DECODE_KV_DIM_DEFAULT // SM100_DECODE_HEAD_DIM_DEFAULT
SM100_DECODE_KV_GROUP_SIZE_DEFAULT = SM100_DECODE_NUM_Q_HEADS_DEFAULT // SM100_DECODE_NUM_KV_HEADS_DEFAULT


class _DecodeMatvecSm100Base(Op):
    uses_dense_weights = True   # bf16/fp16 weight pages (sizes the ring page)
    """Shared schedule/config helpers of the decode matvec ops."""

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        page_size = max(op.static_dims.get("page_size", DEFAULT_PAGE_SIZE) for op in ops)
        return MegakernelConfig(page_size=page_size)

    @staticmethod
    def _default_tiles(tile_sizes, out_dim):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 16)
        tile_sizes.setdefault(out_dim, 16)
        return tile_sizes


class _RmsProjectionSm100Base(_DecodeMatvecSm100Base):
    """RMS(x + residual_in) followed by one projection matrix."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight": (None, ("O", "K")),
        "cos": (None, ("S", "D2")),
        "sin": (None, ("S", "D2")),
    }
    writes = {"residual_out": (None, ("B", "S", "K"))}
    tile = ("B", "S", "O")
    dynamic_dims = ("B",)

    apply_rope = 0
    write_q = 0
    write_cache = 0

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, cache_pos=0, dynamic_pos=False,
                 **tensors):
        """``dynamic_pos`` (not in the reference, which re-schedules per position): the op follows the
        program's device-resident cache position p (``MegakernelConfig.position``) — ``cos`` / ``sin``
        are then the FULL tables (row p is read), ``dst_cache`` the full cache (row p is written) and
        ``cache_pos`` must be 0."""
        tile_sizes = cls._default_tiles(tile_sizes, "O")
        if tile_sizes["O"] != 16:
            raise ValueError(f"{cls.__name__}: tile size O must be 16")
        if dynamic_pos and cache_pos:
            raise ValueError(f"{cls.__name__}: with dynamic_pos the position comes from the device, cache_pos must be 0")
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        op.static_dims["cache_pos"] = cache_pos
        op.static_dims["dynamic_pos"] = int(bool(dynamic_pos))
        op.static_dims["head_dim"] = tensors["cos"].shape[1] * 2
        op.static_dims["reduction_tile_K"] = min(SM100_DECODE_REDUCTION_DIM_PER_WARP, tensors["x"].shape[-1])
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        hd = int(sop.static_dims["head_dim"])
        kw = dict(
            w0=dense_weight(t["weight"]), x=t["x"], pro=N.PRO_ADD_RMS, norm_weight=t["norm_weight"],
            residual_in=t["residual_in"], eps=float(sop.static_dims.get("eps", 1e-5)), head_dim=hd,
        )
        if cls.apply_rope:
            kw.update(mode=N.MV_ROPE, tr=N.TR_ROPE, cos=t["cos"], sin=t["sin"])
        if cls.write_q:
            out = t["q"]
            kw.update(out=out, out_strides=(out.stride(0), out.stride(1), hd), residual_out=t["residual_out"])
        else:
            out = t["dst_cache"]
            if out.shape[-1] != hd or out.stride(-1) != 1:
                raise ValueError(f"{cls.__name__}: dst_cache must be (B, T, H, {hd}) with contiguous head rows")
            pos = int(sop.static_dims.get("cache_pos", 0))
            if pos + t["x"].shape[1] > out.shape[1]:
                raise ValueError(f"{cls.__name__}: cache_pos {pos} + S exceeds the cache length {out.shape[1]}")
            kw.update(out=out, out_strides=(out.stride(0), out.stride(1), out.stride(2)), pos=pos)
        nop = lower_matvec(cls.__name__, ctx, kind="rms_proj", **kw)
        dyn = bool(sop.static_dims.get("dynamic_pos", 0))
        if dyn:
            # q lands in a one-token buffer: only its RoPE row follows the position
            nop.i[N.MV_DYNPOS] = N.MV_DYN_TABLES | (N.MV_DYN_OUT if cls.write_cache else 0)
            if cls.write_cache:
                nop.pos_limit = int(t["dst_cache"].shape[1])
        if cls.write_cache:
            # only rows [cache_pos, cache_pos + S) of the cache are written (any row, with a dynamic position)
            pos = int(sop.static_dims.get("cache_pos", 0))
            hi = int(t["dst_cache"].shape[1]) if dyn else pos + int(t["x"].shape[1])
            nop.writes[-1].axis, nop.writes[-1].lo, nop.writes[-1].hi = 1, pos, hi
            nop.kind = "cache_append"
        return [nop]


class RmsQMatvecRopeSm100Op(_RmsProjectionSm100Base):
    """residual_out = x + residual_in; q = rope(rms(residual_out) * w @ Wq^T)."""

    writes = {
        "residual_out": (None, ("B", "S", "K")),
        "q": (None, ("B", "S", "O")),
    }
    apply_rope = 1
    write_q = 1


class RmsKMatvecRopeCacheSm100Op(_RmsProjectionSm100Base):
    """k = rope(rms(x + residual_in) * w @ Wk^T), appended to the cache at ``cache_pos``."""

    writes = {"dst_cache": (None, ("B", "T", "H", "HD"))}
    apply_rope = 1
    write_cache = 1


class RmsVMatvecCacheSm100Op(_RmsProjectionSm100Base):
    """v = rms(x + residual_in) * w @ Wv^T, appended to the cache at ``cache_pos``."""

    writes = {"dst_cache": (None, ("B", "T", "H", "HD"))}
    write_cache = 1


class MatvecResidualSm100Op(_DecodeMatvecSm100Base):
    """residual_out = a @ W^T + residual_in (in place allowed)."""

    reads = {
        "a": (None, ("B", "S", "K")),
        "weight": (None, ("O", "K")),
        "residual_in": (None, ("B", "S", "O")),
    }
    writes = {"residual_out": (None, ("B", "S", "O"))}
    tile = ("B", "S", "O")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, **tensors):
        op = cls._schedule_single(tile_sizes=cls._default_tiles(tile_sizes, "O"), **tensors)
        op.static_dims["page_size"] = page_size
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["residual_out"]
        return [lower_matvec(cls.__name__, ctx, w0=dense_weight(t["weight"]), x=t["a"], out=out,
                             out_strides=flat_out_strides(out), epi=N.EPI_RESIDUAL,
                             epi_residual=t["residual_in"], kind="matvec_residual")]


class MatvecSm100Op(_DecodeMatvecSm100Base):
    """y = a @ W^T."""

    reads = {
        "a": (None, ("B", "S", "K")),
        "weight": (None, ("O", "K")),
    }
    writes = {"y": (None, ("B", "S", "O"))}
    tile = ("B", "S", "O")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, **tensors):
        op = cls._schedule_single(tile_sizes=cls._default_tiles(tile_sizes, "O"), **tensors)
        op.static_dims["page_size"] = page_size
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["y"]
        return [lower_matvec(cls.__name__, ctx, w0=dense_weight(t["weight"]), x=t["a"], out=out,
                             out_strides=flat_out_strides(out), kind="matvec")]


class ResidualAddSm100Op(_DecodeMatvecSm100Base):
    """residual_out = x + residual_in."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
    }
    writes = {"residual_out": (None, ("B", "S", "K"))}
    tile = ("B", "S", "K")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, **tensors):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 16)
        tile_sizes.setdefault("K", SM100_DECODE_REDUCTION_DIM_PER_WARP)
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        from ..activation.add import lower_add

        t = sop.tensor_refs
        return [lower_add(cls.__name__, t["x"], t["residual_in"], t["residual_out"])]


class RmsGateUpSiluSm100Op(_DecodeMatvecSm100Base):
    """y = silu(h @ Wg^T) * (h @ Wu^T), h = rms(x) * w."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "gate_weight": (None, ("D", "K")),
        "up_weight": (None, ("D", "K")),
    }
    writes = {"y": (None, ("B", "S", "D"))}
    tile = ("B", "S", "D")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, **tensors):
        op = cls._schedule_single(tile_sizes=cls._default_tiles(tile_sizes, "D"), **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        op.static_dims["reduction_tile_K"] = min(SM100_DECODE_REDUCTION_DIM_PER_WARP, tensors["x"].shape[-1])
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["y"]
        return [lower_matvec(cls.__name__, ctx, w0=dense_weight(t["gate_weight"]),
                             w1=dense_weight(t["up_weight"]), x=t["x"], out=out,
                             out_strides=flat_out_strides(out), mode=N.MV_PAIR, tr=N.TR_SILU_MUL,
                             pro=N.PRO_RMS, norm_weight=t["norm_weight"],
                             eps=float(sop.static_dims.get("eps", 1e-5)), kind="gate_up")]


class FinalRmsLmHeadSm100Op(_DecodeMatvecSm100Base):
    """logits = rms(x) * w @ W_lm^T."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight": (None, ("V", "K")),
    }
    writes = {"logits": (None, ("B", "S", "V"))}
    tile = ("B", "S", "V")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, **tensors):
        tile_sizes = cls._default_tiles(tile_sizes, "V")
        if tile_sizes["V"] != 16:
            raise ValueError("FinalRmsLmHeadSm100Op: tile size V must be 16")
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        op.static_dims["page_size"] = page_size
        op.static_dims["eps"] = eps
        op.static_dims["reduction_tile_K"] = min(SM100_DECODE_REDUCTION_DIM_PER_WARP, tensors["x"].shape[-1])
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["logits"]
        return [lower_matvec(cls.__name__, ctx, w0=dense_weight(t["weight"]), x=t["x"], out=out,
                             out_strides=flat_out_strides(out), pro=N.PRO_RMS, norm_weight=t["norm_weight"],
                             eps=float(sop.static_dims.get("eps", 1e-5)), kind="lm_head")]


@dataclass
class DecodeLayerSchedule:
    """Scheduled ops and view keep-alives for one decoder layer."""

    ops: list
    attention_config: object
    keep_alive: list


def schedule_decode_layer_sm100(
    *,
    layer_idx,
    batch,
    seq_len,
    cache_pos,
    weights,
    k_cache,
    v_cache,
    x_in,
    residual_in,
    x_out,
    residual_out,
    q_buf,
    attn_out_buf,
    mlp_h_buf,
    page_size=DEFAULT_PAGE_SIZE,
    eps=1e-5,
    fa_num_splits=0,
    hidden_size=SM100_DECODE_HIDDEN_DEFAULT,
    intermediate_size=SM100_DECODE_INTERMEDIATE_DEFAULT,
    num_q_heads=SM100_DECODE_NUM_Q_HEADS_DEFAULT,
    num_kv_heads=SM100_DECODE_NUM_KV_HEADS_DEFAULT,
    head_dim=SM100_DECODE_HEAD_DIM_DEFAULT,
    kv_group_size=SM100_DECODE_KV_GROUP_SIZE_DEFAULT,
    matvec_block=SM100_DECODE_MATVEC_BLOCK,
    tp_peers=None,
    dynamic_position=False,
):
    """One decoder layer: RMS+Q/RoPE, RMS+K/RoPE/cache, RMS+V/cache, split-KV
    attention + combine, O-proj + residual, RMS+gate/up+SiLU and the down
    projection as ``intermediate/hidden`` K-blocks accumulated into ``x_out``.

    Unlike the reference, attention always goes through flash decoding (its
    short-KV branch uses a prefill attention kernel this build does not have).

    ``tp_peers`` (a ``PeerBuffers``) switches to Megatron-style tensor
    parallelism: ``weights`` then hold THIS RANK's shards (W_q/W_k/W_v/W_gate/
    W_up split by output rows, W_o/W_down split by K), ``num_q_heads`` /
    ``num_kv_heads`` / ``intermediate_size`` are the local counts, and the two
    K-split projections write fp32 partials that an in-kernel all-reduce adds
    across ranks (plus the residual for the O-projection).
    """
    from ..attention.flash_decoding import flash_decoding_schedule

    pfx = f"layer.{layer_idx}"
    if dynamic_position:
        # ``dynamic_position`` (not in the reference): the step follows the program's device-resident
        # cache position (MegakernelConfig.position) instead of ``cache_pos``: the ops get the full
        # RoPE tables and the full caches, and read / write the row of the current position.
        if seq_len != 1:
            raise ValueError("a device-resident position decodes one token per sequence and step")
        cache_pos = 0
        if weights["cos"].shape[0] < k_cache.shape[1]:
            raise ValueError(f"RoPE tables hold {weights['cos'].shape[0]} positions, the cache {k_cache.shape[1]}")
        cos, sin = weights["cos"][:seq_len], weights["sin"][:seq_len]   # row 0: the kernel adds the position
        k_window, v_window = k_cache, v_cache
    else:
        cos = weights["cos"][cache_pos: cache_pos + seq_len]
        sin = weights["sin"][cache_pos: cache_pos + seq_len]
        k_window = k_cache[:, : cache_pos + seq_len]
        v_window = v_cache[:, : cache_pos + seq_len]
    q_4d = q_buf.view(batch, seq_len, num_q_heads, head_dim)
    o_4d = attn_out_buf.view(batch, seq_len, num_q_heads, head_dim)
    tiles = {"S": seq_len, "O": matvec_block}
    common = dict(x=x_in, residual_in=residual_in, norm_weight=weights[f"{pfx}.attn_norm"], cos=cos, sin=sin,
                  tile_sizes=tiles, page_size=page_size, eps=eps, dynamic_pos=dynamic_position)

    ops = []
    ops += RmsQMatvecRopeSm100Op.schedule(weight=weights[f"{pfx}.W_q"], residual_out=residual_out, q=q_buf,
                                          **common)
    ops += RmsKMatvecRopeCacheSm100Op.schedule(weight=weights[f"{pfx}.W_k"], dst_cache=k_window,
                                               cache_pos=cache_pos, **common)
    ops += RmsVMatvecCacheSm100Op.schedule(weight=weights[f"{pfx}.W_v"], dst_cache=v_window,
                                           cache_pos=cache_pos, **common)
    fa_ops, fa_config = flash_decoding_schedule(
        q=q_4d, k=k_window, v=v_window, o=o_4d, kv_group_size=kv_group_size, page_size=page_size,
        num_splits=fa_num_splits, dynamic_len=dynamic_position,
    )
    ops += fa_ops
    tp_keep = []
    if tp_peers is not None:
        from ..allreduce import AllReduceSm100Op

        o_part = torch.empty(residual_out.shape, dtype=torch.float32, device=residual_out.device)
        x_part = torch.empty(x_out.shape, dtype=torch.float32, device=x_out.device)
        tp_keep = [o_part, x_part]
        ops += MatvecSm100Op.schedule(a=attn_out_buf, weight=weights[f"{pfx}.W_o"], y=o_part, tile_sizes=tiles,
                                      page_size=page_size)
        ops += AllReduceSm100Op.schedule(peers=tp_peers, x=o_part, residual_in=residual_out, y=residual_out)
    else:
        ops += MatvecResidualSm100Op.schedule(a=attn_out_buf, weight=weights[f"{pfx}.W_o"],
                                              residual_in=residual_out, residual_out=residual_out,
                                              tile_sizes=tiles, page_size=page_size)
    ops += RmsGateUpSiluSm100Op.schedule(x=residual_out, norm_weight=weights[f"{pfx}.mlp_norm"],
                                         gate_weight=weights[f"{pfx}.W_gate"], up_weight=weights[f"{pfx}.W_up"],
                                         y=mlp_h_buf, tile_sizes={"S": seq_len, "D": matvec_block},
                                         page_size=page_size, eps=eps)
    down_keep = []
    if tp_peers is not None:
        # one matvec over this rank's K range, then the exchange
        ops += MatvecSm100Op.schedule(a=mlp_h_buf, weight=weights[f"{pfx}.W_down"], y=x_part, tile_sizes=tiles,
                                      page_size=page_size)
        ops += AllReduceSm100Op.schedule(peers=tp_peers, x=x_part, y=x_out)
        return DecodeLayerSchedule(ops=ops, attention_config=fa_config,
                                   keep_alive=[cos, sin, q_4d, k_window, v_window, o_4d, *tp_keep])
    for blk in range(intermediate_size // hidden_size):
        start, stop = blk * hidden_size, (blk + 1) * hidden_size
        a_block = mlp_h_buf[:, :, start:stop]
        w_block = weights[f"{pfx}.W_down"][:, start:stop]
        down_keep += [a_block, w_block]
        if blk == 0:
            ops += MatvecSm100Op.schedule(a=a_block, weight=w_block, y=x_out, tile_sizes=tiles, page_size=page_size)
        else:
            ops += MatvecResidualSm100Op.schedule(a=a_block, weight=w_block, residual_in=x_out, residual_out=x_out,
                                                  tile_sizes=tiles, page_size=page_size)
    return DecodeLayerSchedule(ops=ops, attention_config=fa_config,
                               keep_alive=[cos, sin, q_4d, k_window, v_window, o_4d, *down_keep])


def schedule_final_sm100(*, x, residual_in, residual_out, final_norm, lm_head=None, logits=None, seq_len,
                         page_size=DEFAULT_PAGE_SIZE, eps=1e-5):
    """Final residual add and, optionally, the fused final RMS + LM-head matvec."""
    ops = ResidualAddSm100Op.schedule(x=x, residual_in=residual_in, residual_out=residual_out,
                                      tile_sizes={"S": seq_len, "K": SM100_DECODE_REDUCTION_DIM_PER_WARP},
                                      page_size=page_size)
    if lm_head is not None:
        if logits is None:
            raise ValueError("logits must be provided when lm_head is scheduled")
        ops += FinalRmsLmHeadSm100Op.schedule(x=residual_out, norm_weight=final_norm, weight=lm_head, logits=logits,
                                              tile_sizes={"S": seq_len, "V": SM100_DECODE_MATVEC_BLOCK},
                                              page_size=page_size, eps=eps)
    return ops


__all__ = [
    "MatvecSm100Op", "FinalRmsLmHeadSm100Op", "MatvecResidualSm100Op", "ResidualAddSm100Op",
    "RmsGateUpSiluSm100Op", "RmsKMatvecRopeCacheSm100Op", "RmsQMatvecRopeSm100Op", "RmsVMatvecCacheSm100Op",
    "DecodeLayerSchedule", "schedule_decode_layer_sm100", "schedule_final_sm100",
]
