"""Shared lowering of every weight-streaming matvec op onto ``MK_OP_MATVEC``.

One native handler (``csrc/op_matvec.cuh``) serves GemmOp at decode sizes and
the whole decode-matvec family; the op classes differ only in which prologue
(RMSNorm, fused residual add), row mapping (plain / RoPE partners / gate-up
pairs), transform and epilogue they select here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import _native as N
from ..megakernel.lowering import (LowerCtx, NativeOp, Region, bf16_page_need, elem_type, fp4_page_need,
                                    meta_of)


@dataclass
class Weight:
    """A weight matrix in one of the native formats."""

    fmt: int
    data: torch.Tensor                  # (O, K) bf16/fp16, or packed (O, K/2) uint8
    scales: Optional[torch.Tensor] = None   # (O, K/group)
    global_scale: float = 1.0

    @property
    def rows(self) -> int:
        return int(self.data.shape[0])

    @property
    def cols(self) -> int:
        return int(self.data.shape[1]) * (2 if self.fmt >= N.W_NVFP4_F16S32 else 1)


def dense_weight(w: torch.Tensor) -> Weight:
    if w.ndim != 2:
        raise ValueError(f"weight must be rank-2 (O, K), got shape {tuple(w.shape)}")
    if w.stride(1) != 1:
        raise ValueError("weight rows must be K-contiguous")
    if w.dtype == torch.bfloat16:
        return Weight(N.W_BF16, w)
    if w.dtype == torch.float16:
        return Weight(N.W_FP16, w)
    raise ValueError(f"weight dtype {w.dtype} unsupported (bf16 or fp16)")


def nvfp4_weight(packed: torch.Tensor, scales: torch.Tensor, group_size: int, global_scale: float = 1.0) -> Weight:
    if packed.dtype != torch.uint8 or packed.ndim != 2 or packed.stride(1) != 1:
        raise ValueError("packed NVFP4 weight must be a rank-2 uint8 tensor with contiguous rows")
    if scales.ndim != 2 or scales.stride(1) != 1 or scales.shape[0] != packed.shape[0]:
        raise ValueError("NVFP4 scales must be rank-2 (O, K/group) with contiguous rows")
    K = packed.shape[1] * 2
    if group_size == 32 and scales.dtype == torch.float16:
        fmt = N.W_NVFP4_F16S32
    elif group_size == 16 and scales.element_size() == 1:
        fmt = N.W_NVFP4_E4M3S16
    else:
        raise ValueError(
            f"unsupported NVFP4 layout: group_size={group_size}, scale dtype {scales.dtype} "
            f"(fp16 scales per 32 values, or e4m3 scales per 16 values)"
        )
    if scales.shape[1] != K // group_size:
        raise ValueError("weight_scales G must equal K / group_size")
    return Weight(fmt, packed, scales, float(global_scale))


def lower_matvec(
    name: str,
    ctx: LowerCtx,
    *,
    w0: Weight,
    w1: Optional[Weight] = None,
    x: torch.Tensor,                       # (B, S, K)
    out: torch.Tensor,
    out_strides,                           # (stride_B, stride_S, stride_H) in elements
    head_dim: Optional[int] = None,        # output head size for (head, dim) addressing; None = flat
    pos: int = 0,
    mode: int = N.MV_PLAIN,
    pro: int = N.PRO_NONE,
    epi: int = N.EPI_STORE,
    tr: int = N.TR_NONE,
    norm_weight: Optional[torch.Tensor] = None,
    residual_in: Optional[torch.Tensor] = None,
    residual_out: Optional[torch.Tensor] = None,
    epi_residual: Optional[torch.Tensor] = None,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    eps: float = 1e-5,
    out_rows: Optional[int] = None,
    kind: str = "matvec",
    index_offset: int = 0,
) -> NativeOp:
    if x.ndim != 3 or x.stride(-1) != 1:
        raise ValueError(f"{name}: activations must be (B, S, K) with unit innermost stride")
    B, S, K = (int(v) for v in x.shape)
    M = B * S
    if M > 32:
        raise ValueError(f"{name}: {M} activation rows; the decode matvec path handles at most 32")
    if w0.cols != K:
        raise ValueError(f"{name}: weight K={w0.cols} does not match activation K={K}")
    fp4 = w0.fmt >= N.W_NVFP4_F16S32
    if w1 is not None and (w1.fmt != w0.fmt or w1.rows != w0.rows or w1.cols != K):
        raise ValueError(f"{name}: paired weights must share format and shape")
    kc = min(ctx.kc_fp4 if fp4 else ctx.kc_bf16, K)
    if fp4:
        if K % 256 or (K > 2048 and K % 2048):
            raise ValueError(f"{name}: NVFP4 matvec needs K % 256 == 0 and, above 2048, K % 2048 == 0; got {K}")
        kc = min(K, 2048)     # one 128-byte scale tile row covers 2048 K-values
    else:
        if K % 64:
            raise ValueError(f"{name}: matvec needs K % 64 == 0, got {K}")
        kc = max(64, kc // 64 * 64)
        # An op with a unit or two per CTA finishes when its slowest page does: shorter K-slices put
        # more consumer warps on each unit (a page is the grain at which warps share a unit).
        n_rows_units = -(-(w0.rows if out_rows is None else out_rows) // (8 if mode == N.MV_PAIR else 16))
        if ctx.small_op_kc and n_rows_units <= 2 * ctx.num_sms and -(-K // kc) < 4:
            kc = max(ctx.small_op_kc, 64 * (-(-K // 4) // 64))
    xt = elem_type(x, f"{name}: x")
    if w0.fmt == N.W_BF16 and xt != N.T_BF16:
        raise ValueError(f"{name}: bf16 weights need bf16 activations")
    if w0.fmt == N.W_FP16 and xt != N.T_FP16:
        raise ValueError(f"{name}: fp16 weights need fp16 activations")
    O = w0.rows if out_rows is None else out_rows
    hd = int(head_dim) if head_dim else O
    if mode == N.MV_PLAIN:
        n_units = -(-O // 16)
        rows_per_unit = 16
    elif mode == N.MV_PAIR:
        n_units = -(-O // 8)
        rows_per_unit = 16
    else:
        d2 = int(cos.shape[1])
        if hd != 2 * d2 or d2 % 8 or O % hd:
            raise ValueError(f"{name}: RoPE epilogue needs head_dim == 2*D2, D2 % 8 == 0 and O % head_dim == 0")
        n_units = (O // hd) * (d2 // 8)
        rows_per_unit = 16

    # Consumer warps per unit: an op with few units per CTA spreads each unit's
    # K-slices over several warps, an op with many keeps one warp per unit.
    n_pages = -(-K // kc)
    units_per_cta = -(-n_units // max(1, ctx.num_sms))
    split = 1 if units_per_cta >= 2 * N.NUM_CONSUMER_WARPS else min(N.NUM_CONSUMER_WARPS, n_pages)

    wrow = int(w0.data.stride(0)) * w0.data.element_size()
    bytes_per_row = K // 2 + (K // 16) if fp4 else K * 2
    op = NativeOp(name=name, opcode=N.OP_MATVEC, n_units=n_units, kind=kind)
    op.i = {
        N.MV_O: O, N.MV_K: K, N.MV_M: M, N.MV_S: S, N.MV_MODE: mode, N.MV_PRO: pro, N.MV_EPI: epi,
        N.MV_TR: tr, N.MV_HD: hd, N.MV_D2: int(cos.shape[1]) if cos is not None else 0, N.MV_POS: int(pos),
        N.MV_WFMT: w0.fmt, N.MV_KC: kc, N.MV_OUT_T: elem_type(out, f"{name}: out") if epi != N.EPI_TOP1 else 0,
        N.MV_X_T: xt, N.MV_ROWS_PER_UNIT: rows_per_unit, N.MV_SPLIT: split, N.MV_IDX0: int(index_offset),
    }
    op.f = {N.MV_F_EPS: eps, N.MV_F_GSCALE: w0.global_scale, N.MV_F_GSCALE1: (w1 or w0).global_scale}
    op.p = {N.MV_P_W0: w0.data.data_ptr(), N.MV_P_W1: (w1 or w0).data.data_ptr(), N.MV_P_X: x.data_ptr(),
            N.MV_P_OUT: out.data_ptr()}
    op.s = {N.MV_S_WROW: wrow, N.MV_S_X_B: x.stride(0), N.MV_S_X_S: x.stride(1),
            N.MV_S_O_B: out_strides[0], N.MV_S_O_S: out_strides[1], N.MV_S_O_H: out_strides[2]}
    op.reads = [Region(meta_of(w0.data, "weight"), loader=True), Region(meta_of(x, "x"), act=True)]
    op.keep = [w0.data, x, out]
    if w1 is not None:
        if int(w1.data.stride(0)) * w1.data.element_size() != wrow:
            raise ValueError(f"{name}: paired weights must share the row stride")
        op.reads.append(Region(meta_of(w1.data, "weight1"), loader=True))
        op.keep.append(w1.data)
    if fp4:
        op.p[N.MV_P_SC0] = w0.scales.data_ptr()
        op.p[N.MV_P_SC1] = (w1 or w0).scales.data_ptr()
        op.s[N.MV_S_SCROW] = int(w0.scales.stride(0)) * w0.scales.element_size()
        op.reads.append(Region(meta_of(w0.scales, "scales"), loader=True))
        op.keep.append(w0.scales)
        if w1 is not None:
            op.reads.append(Region(meta_of(w1.scales, "scales1"), loader=True))
            op.keep.append(w1.scales)
    if pro != N.PRO_NONE:
        if norm_weight is None:
            raise ValueError(f"{name}: RMSNorm prologue needs norm_weight")
        if norm_weight.dtype != x.dtype or norm_weight.numel() != K:
            raise ValueError(f"{name}: norm_weight must be ({K},) of the activation dtype")
        op.p[N.MV_P_NORM_W] = norm_weight.data_ptr()
        op.reads.append(Region(meta_of(norm_weight, "norm_weight")))
        op.keep.append(norm_weight)
    if pro == N.PRO_ADD_RMS:
        if residual_in is None:
            raise ValueError(f"{name}: fused-add prologue needs residual_in")
        if residual_in.shape != x.shape or residual_in.dtype != x.dtype or residual_in.stride(-1) != 1:
            raise ValueError(f"{name}: residual_in must match x")
        op.p[N.MV_P_RES_IN] = residual_in.data_ptr()
        op.s[N.MV_S_RI_B], op.s[N.MV_S_RI_S] = residual_in.stride(0), residual_in.stride(1)
        op.reads.append(Region(meta_of(residual_in, "residual_in"), act=True))
        op.keep.append(residual_in)
        if residual_out is not None:
            if residual_out.shape != x.shape or residual_out.dtype != x.dtype or residual_out.stride(-1) != 1:
                raise ValueError(f"{name}: residual_out must match x")
            ro = meta_of(residual_out, "residual_out")
            for other in (meta_of(x), meta_of(residual_in)):
                from ..megakernel.ops import tensor_meta_overlaps
                if tensor_meta_overlaps(ro, other):
                    raise ValueError(
                        f"{name}: residual_out may not alias x or residual_in (every CTA re-reads them "
                        f"while one CTA writes the sum)"
                    )
            op.p[N.MV_P_RES_OUT] = residual_out.data_ptr()
            op.s[N.MV_S_RO_B], op.s[N.MV_S_RO_S] = residual_out.stride(0), residual_out.stride(1)
            op.writes.append(Region(ro))
            op.writes_res_out = True
            op.keep.append(residual_out)
    if epi == N.EPI_RESIDUAL:
        if epi_residual is None or epi_residual.ndim != 3 or epi_residual.stride(-1) != 1:
            raise ValueError(f"{name}: residual epilogue needs a (B, S, O) residual")
        if epi_residual.dtype != x.dtype:
            raise ValueError(f"{name}: residual dtype must match the activations")
        op.p[N.MV_P_EPI_RES] = epi_residual.data_ptr()
        op.s[N.MV_S_ER_B], op.s[N.MV_S_ER_S] = epi_residual.stride(0), epi_residual.stride(1)
        op.reads.append(Region(meta_of(epi_residual, "epi_residual")))
        op.keep.append(epi_residual)
    if tr == N.TR_ROPE:
        if cos is None or sin is None or cos.shape != sin.shape or cos.dtype != x.dtype or cos.shape[0] < S:
            raise ValueError(f"{name}: cos/sin must be (>=S, D2) tables of the activation dtype")
        if cos.stride(1) != 1 or sin.stride(1) != 1 or cos.stride(0) != sin.stride(0):
            raise ValueError(f"{name}: cos/sin must share a row stride and be contiguous along D2")
        op.p[N.MV_P_COS], op.p[N.MV_P_SIN] = cos.data_ptr(), sin.data_ptr()
        op.s[N.MV_S_COS] = cos.stride(0)
        op.reads += [Region(meta_of(cos, "cos")), Region(meta_of(sin, "sin"))]
        op.keep += [cos, sin]
    op.writes.append(Region(meta_of(out, "out")))
    op.pages = -(-K // kc)
    op.unit_bytes = rows_per_unit * bytes_per_row
    op.page_need = fp4_page_need(kc) if fp4 else bf16_page_need(kc)
    op.act_bytes = M * (K * 2 + 64)
    op.act_sig = (
        x.data_ptr(), tuple(x.stride()), tuple(x.shape),
        residual_in.data_ptr() if (pro == N.PRO_ADD_RMS) else 0,
        tuple(residual_in.stride()) if (pro == N.PRO_ADD_RMS) else (),
        norm_weight.data_ptr() if pro != N.PRO_NONE else 0, pro, float(eps), xt,
        N.T_BF16 if w0.fmt == N.W_BF16 else N.T_FP16,
    )
    return op


def flat_out_strides(out: torch.Tensor):
    """Strides for a flat (B, S, O) output."""
    if out.ndim != 3 or out.stride(-1) != 1:
        raise ValueError(f"expected a (B, S, O) output with unit innermost stride, got {tuple(out.shape)}")
    return (int(out.stride(0)), int(out.stride(1)), int(out.shape[-1]))
