"""Decode matvec ops with packed NVFP4 weights.

Same class names and ``schedule()`` keywords as the reference's NVFP4 decode
ops (src/machete/kernels/decode_matvec/sm120.py: ``_RmsProjectionNvfp4Sm120Base``
:596, ``RmsMatvecNvfp4Sm120Op`` :859, ``MatvecNvfp4Sm120Op`` :1105,
``MatvecResidualNvfp4Sm120Op`` :1379, ``RmsGateUpSiluNvfp4Sm120Op`` :1612,
``FinalRmsLmHeadNvfp4Sm120Op`` :1845); the reference targets RTX-class
Blackwell with byte loads and a scalar dot, here the packed rows and their
scales are streamed by TMA and dequantised in registers for the f16
tensor-core path.  Tensors: ``weight_packed (O, K/2) uint8`` (two E2M1 codes
per byte, low nibble first) and ``weight_scales (O, K/group)``.

Two layouts are accepted: ``group_size=32`` with fp16 scales (the reference's)
and ``group_size=16`` with e4m3 scales plus a per-tensor fp32
``global_scale`` keyword (NVIDIA's block-scaled NVFP4).
"""

from __future__ import annotations

from ... import _native as N
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op, Uint8
from .._matvec import flat_out_strides, lower_matvec, nvfp4_weight

SM120_DECODE_REDUCTION_DIM_PER_WARP = 512


def _check_nvfp4(packed, scales, k, group_size, what="weight"):
    if packed.shape[1] * 2 != k:
        raise ValueError(f"{what}_packed K2 must equal K / 2")
    if scales.shape[1] != k // group_size:
        raise ValueError(f"{what}_scales G must equal K / group_size")


def _finalize(op, *, page_size, group_size, k_dim, global_scale):
    op.static_dims["page_size"] = page_size
    op.static_dims["group_size"] = group_size
    op.static_dims["reduction_tile_K"] = min(SM120_DECODE_REDUCTION_DIM_PER_WARP, k_dim)
    op.params["global_scale"] = float(global_scale)
    return [op]


class _Nvfp4Base(Op):
    uses_nvfp4 = True

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=max(op.static_dims.get("page_size", DEFAULT_PAGE_SIZE) for op in ops))

    @staticmethod
    def _tiles(tile_sizes, out_dim):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.setdefault("B", 1)
        tile_sizes.setdefault("S", 16)
        tile_sizes.setdefault(out_dim, 16)
        return tile_sizes

    @staticmethod
    def _weight(sop, packed="weight_packed", scales="weight_scales", scale_key="global_scale"):
        t = sop.tensor_refs
        return nvfp4_weight(t[packed], t[scales], int(sop.static_dims["group_size"]),
                            sop.params.get(scale_key, sop.params.get("global_scale", 1.0)))


class _RmsProjectionNvfp4Sm120Base(_Nvfp4Base):
    """RMS(x + residual_in) followed by one packed NVFP4 projection."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight_packed": (Uint8, ("O", "K2")),
        "weight_scales": (None, ("O", "G")),
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
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, cache_pos=0, group_size=32,
                 head_dim=None, global_scale=1.0, dynamic_pos=False, **tensors):
        """``dynamic_pos`` (not in the reference): the cache row (and the RoPE table row) follow the
        program's device-resident position; ``cos`` / ``sin`` are then the whole tables and
        ``dst_cache`` the whole cache."""
        k = tensors["x"].shape[-1]
        _check_nvfp4(tensors["weight_packed"], tensors["weight_scales"], k, group_size)
        op = cls._schedule_single(tile_sizes=cls._tiles(tile_sizes, "O"), **tensors)
        op.static_dims["eps"] = eps
        op.static_dims["cache_pos"] = cache_pos
        op.static_dims["dynamic_pos"] = int(bool(dynamic_pos))
        op.static_dims["head_dim"] = int(head_dim or tensors["cos"].shape[1] * 2)
        return _finalize(op, page_size=page_size, group_size=group_size, k_dim=k, global_scale=global_scale)

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        hd = int(sop.static_dims["head_dim"])
        kw = dict(w0=cls._weight(sop), x=t["x"], pro=N.PRO_ADD_RMS, norm_weight=t["norm_weight"],
                  residual_in=t["residual_in"], eps=float(sop.static_dims.get("eps", 1e-5)), head_dim=hd)
        if cls.apply_rope:
            kw.update(mode=N.MV_ROPE, tr=N.TR_ROPE, cos=t["cos"], sin=t["sin"])
        if cls.write_q:
            out = t["q"]
            kw.update(out=out, out_strides=(out.stride(0), out.stride(1), hd), residual_out=t.get("residual_out"))
        else:
            out = t["dst_cache"]
            pos = int(sop.static_dims.get("cache_pos", 0))
            if out.shape[-1] != hd or out.stride(-1) != 1 or pos + t["x"].shape[1] > out.shape[1]:
                raise ValueError(f"{cls.__name__}: dst_cache must be (B, T > cache_pos, H, {hd})")
            kw.update(out=out, out_strides=(out.stride(0), out.stride(1), out.stride(2)), pos=pos)
        nop = lower_matvec(cls.__name__, ctx, kind="rms_proj", **kw)
        dyn = bool(sop.static_dims.get("dynamic_pos", 0))
        if dyn:
            nop.i[N.MV_DYNPOS] = (N.MV_DYN_TABLES if cls.apply_rope else 0) | (N.MV_DYN_OUT if cls.write_cache else 0)
            if cls.write_cache:
                nop.pos_limit = int(t["dst_cache"].shape[1])
        if cls.write_cache:
            pos = int(sop.static_dims.get("cache_pos", 0))
            hi = int(t["dst_cache"].shape[1]) if dyn else pos + int(t["x"].shape[1])
            nop.writes[-1].axis, nop.writes[-1].lo, nop.writes[-1].hi = 1, pos, hi
            nop.kind = "cache_append"
        return [nop]


class RmsQMatvecRopeNvfp4Sm120Op(_RmsProjectionNvfp4Sm120Base):
    writes = {"residual_out": (None, ("B", "S", "K")), "q": (None, ("B", "S", "O"))}
    apply_rope = 1
    write_q = 1


class RmsKMatvecRopeCacheNvfp4Sm120Op(_RmsProjectionNvfp4Sm120Base):
    writes = {"dst_cache": (None, ("B", "T", "H", "HD"))}
    apply_rope = 1
    write_cache = 1


class RmsVMatvecCacheNvfp4Sm120Op(_RmsProjectionNvfp4Sm120Base):
    writes = {"dst_cache": (None, ("B", "T", "H", "HD"))}
    write_cache = 1


class RmsMatvecNvfp4Sm120Op(_Nvfp4Base):
    """y = rms(x + residual_in) * w @ W^T (no RoPE); writes residual_out when given."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "residual_in": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight_packed": (Uint8, ("O", "K2")),
        "weight_scales": (None, ("O", "G")),
    }
    writes = {"residual_out": (None, ("B", "S", "K")), "y": (None, ("B", "S", "O"))}
    tile = ("B", "S", "O")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, group_size=32, global_scale=1.0,
                 write_residual=True, **tensors):
        k = tensors["x"].shape[-1]
        _check_nvfp4(tensors["weight_packed"], tensors["weight_scales"], k, group_size)
        op = cls._schedule_single(tile_sizes=cls._tiles(tile_sizes, "O"), **tensors)
        op.static_dims["eps"] = eps
        op.params["write_residual"] = bool(write_residual)
        return _finalize(op, page_size=page_size, group_size=group_size, k_dim=k, global_scale=global_scale)

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["y"]
        return [lower_matvec(cls.__name__, ctx, w0=cls._weight(sop), x=t["x"], out=out,
                             out_strides=flat_out_strides(out), pro=N.PRO_ADD_RMS, norm_weight=t["norm_weight"],
                             residual_in=t["residual_in"],
                             residual_out=t["residual_out"] if sop.params.get("write_residual", True) else None,
                             eps=float(sop.static_dims.get("eps", 1e-5)), kind="rms_proj")]


class _MatvecNvfp4Sm120Base(_Nvfp4Base):
    reads = {
        "a": (None, ("B", "S", "K")),
        "weight_packed": (Uint8, ("O", "K2")),
        "weight_scales": (None, ("O", "G")),
    }
    tile = ("B", "S", "O")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, group_size=32, global_scale=1.0, **tensors):
        k = tensors["a"].shape[-1]
        _check_nvfp4(tensors["weight_packed"], tensors["weight_scales"], k, group_size)
        op = cls._schedule_single(tile_sizes=cls._tiles(tile_sizes, "O"), **tensors)
        return _finalize(op, page_size=page_size, group_size=group_size, k_dim=k, global_scale=global_scale)


class MatvecNvfp4Sm120Op(_MatvecNvfp4Sm120Base):
    """y = a @ dequant(W)^T."""

    writes = {"y": (None, ("B", "S", "O"))}

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["y"]
        return [lower_matvec(cls.__name__, ctx, w0=cls._weight(sop), x=t["a"], out=out,
                             out_strides=flat_out_strides(out), kind="matvec")]


class MatvecResidualNvfp4Sm120Op(_MatvecNvfp4Sm120Base):
    """residual_out = a @ dequant(W)^T + residual_in."""

    reads = dict(_MatvecNvfp4Sm120Base.reads, residual_in=(None, ("B", "S", "O")))
    writes = {"residual_out": (None, ("B", "S", "O"))}

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["residual_out"]
        return [lower_matvec(cls.__name__, ctx, w0=cls._weight(sop), x=t["a"], out=out,
                             out_strides=flat_out_strides(out), epi=N.EPI_RESIDUAL,
                             epi_residual=t["residual_in"], kind="matvec_residual")]


class RmsGateUpSiluNvfp4Sm120Op(_Nvfp4Base):
    """y = silu(h @ Wg^T) * (h @ Wu^T), h = rms(x) * w, packed NVFP4 gate/up weights."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "gate_packed": (Uint8, ("D", "K2")),
        "gate_scales": (None, ("D", "G")),
        "up_packed": (Uint8, ("D", "K2")),
        "up_scales": (None, ("D", "G")),
    }
    writes = {"y": (None, ("B", "S", "D"))}
    tile = ("B", "S", "D")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, group_size=32, prefetch_nvfp4=True,
                 global_scale=1.0, up_global_scale=None, **tensors):
        """``global_scale`` / ``up_global_scale``: the fp32 tensor scales of the gate and the up matrix
        (block-scaled layout; ``up_global_scale=None`` = the same as the gate's)."""
        k = tensors["x"].shape[-1]
        _check_nvfp4(tensors["gate_packed"], tensors["gate_scales"], k, group_size, "gate")
        _check_nvfp4(tensors["up_packed"], tensors["up_scales"], k, group_size, "up")
        op = cls._schedule_single(tile_sizes=cls._tiles(tile_sizes, "D"), **tensors)
        op.static_dims["eps"] = eps
        op.static_dims["prefetch_nvfp4"] = bool(prefetch_nvfp4)
        op.params["up_global_scale"] = float(global_scale if up_global_scale is None else up_global_scale)
        return _finalize(op, page_size=page_size, group_size=group_size, k_dim=k, global_scale=global_scale)

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["y"]
        return [lower_matvec(cls.__name__, ctx, w0=cls._weight(sop, "gate_packed", "gate_scales"),
                             w1=cls._weight(sop, "up_packed", "up_scales", "up_global_scale"), x=t["x"], out=out,
                             out_strides=flat_out_strides(out), mode=N.MV_PAIR, tr=N.TR_SILU_MUL, pro=N.PRO_RMS,
                             norm_weight=t["norm_weight"], eps=float(sop.static_dims.get("eps", 1e-5)),
                             kind="gate_up")]


class FinalRmsLmHeadNvfp4Sm120Op(_Nvfp4Base):
    """logits = rms(x) * w @ dequant(W_lm)^T."""

    reads = {
        "x": (None, ("B", "S", "K")),
        "norm_weight": (None, ("K",)),
        "weight_packed": (Uint8, ("V", "K2")),
        "weight_scales": (None, ("V", "G")),
    }
    writes = {"logits": (None, ("B", "S", "V"))}
    tile = ("B", "S", "V")
    dynamic_dims = ("B",)

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, eps=1e-5, group_size=32, global_scale=1.0,
                 **tensors):
        k = tensors["x"].shape[-1]
        _check_nvfp4(tensors["weight_packed"], tensors["weight_scales"], k, group_size)
        op = cls._schedule_single(tile_sizes=cls._tiles(tile_sizes, "V"), **tensors)
        op.static_dims["eps"] = eps
        return _finalize(op, page_size=page_size, group_size=group_size, k_dim=k, global_scale=global_scale)

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        out = t["logits"]
        return [lower_matvec(cls.__name__, ctx, w0=cls._weight(sop), x=t["x"], out=out,
                             out_strides=flat_out_strides(out), pro=N.PRO_RMS, norm_weight=t["norm_weight"],
                             eps=float(sop.static_dims.get("eps", 1e-5)), kind="lm_head")]


__all__ = [
    "RmsQMatvecRopeNvfp4Sm120Op", "RmsKMatvecRopeCacheNvfp4Sm120Op", "RmsVMatvecCacheNvfp4Sm120Op",
    "RmsMatvecNvfp4Sm120Op", "MatvecNvfp4Sm120Op", "MatvecResidualNvfp4Sm120Op", "RmsGateUpSiluNvfp4Sm120Op",
    "FinalRmsLmHeadNvfp4Sm120Op",
]
