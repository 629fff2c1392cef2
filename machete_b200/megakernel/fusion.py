"""Program lowering with peephole fusion.

``lower_program`` turns the scheduled ops into native op records.  With
``ctx.fuse`` it also rewrites one pattern the reference's layer schedule
produces: the down projection issued as ``intermediate / hidden`` K-blocks —
``MatvecSm100Op`` on ``W[:, 0:h]`` followed by ``MatvecResidualSm100Op`` on
``W[:, h:2h] ...`` accumulating in place (src/machete/kernels/decode_matvec/
sm100.py:794-817).  The blocks are slices of one weight and one activation
buffer, so they collapse into a single full-K matvec: one dependency stage
instead of four, fp32 accumulation across the whole K instead of a bf16
round trip per block.
"""

from __future__ import annotations

from typing import List

import torch

from .. import _native as N
from .lowering import LowerCtx, NativeOp
from .ops import ScheduledOp, last_dim_slice_region


# Bytes of staged activations (rows x (K * 2 + 64)) that still leave six 18 KB / three 32 KB weight
# pages in shared memory: a matvec op stages its whole input, so batch x K is bounded by this.
STAGING_BUDGET = 100 * 1024


def _kblock_chain(ops: List[ScheduledOp], start: int):
    """Length of a fusable down-projection K-block chain starting at ``start`` (0 if none)."""
    first = ops[start]
    if first.op_cls.__name__ not in ("MatvecSm100Op", "MatvecSm120Op"):
        return 0, None
    a0, w0, y = first.tensor_refs["a"], first.tensor_refs["weight"], first.tensor_refs["y"]
    if a0.storage_offset() != 0 and a0.stride(-1) != 1:
        return 0, None
    k = int(a0.shape[-1])
    n = 1
    while start + n < len(ops):
        nxt = ops[start + n]
        if nxt.op_cls.__name__ not in ("MatvecResidualSm100Op", "MatvecResidualSm120Op"):
            break
        t = nxt.tensor_refs
        a, w = t["a"], t["weight"]
        same_out = t["residual_in"].data_ptr() == y.data_ptr() and t["residual_out"].data_ptr() == y.data_ptr()
        if not same_out or a.shape != a0.shape or w.shape != w0.shape:
            break
        if a.stride() != a0.stride() or w.stride() != w0.stride():
            break
        esz = a.element_size()
        if a.data_ptr() != a0.data_ptr() + n * k * esz or w.data_ptr() != w0.data_ptr() + n * k * esz:
            break
        if a.untyped_storage().data_ptr() != a0.untyped_storage().data_ptr():
            break
        if w.untyped_storage().data_ptr() != w0.untyped_storage().data_ptr():
            break
        n += 1
    if n < 2:
        return 0, None
    # the fused op stages all n*k activations of every row at once: keep the K-blocks when that does not fit
    if int(a0.shape[0]) * int(a0.shape[1]) * (n * k * a0.element_size() + 64) > STAGING_BUDGET:
        return 0, None
    # the slices must tile one contiguous row range of the parents
    if a0.stride(-2) < n * k or w0.stride(0) < n * k:
        return 0, None
    a_full = torch.as_strided(a0, (a0.shape[0], a0.shape[1], n * k), a0.stride())
    w_full = torch.as_strided(w0, (w0.shape[0], n * k), w0.stride())
    return n, (a_full, w_full, y)


def lower_program(ops: List[ScheduledOp], ctx: LowerCtx) -> List[NativeOp]:
    from ..kernels._matvec import dense_weight, flat_out_strides, lower_matvec

    out: List[NativeOp] = []
    i = 0
    while i < len(ops):
        sop = ops[i]
        if ctx.fuse:
            n, fused = _kblock_chain(ops, i)
            if n:
                a_full, w_full, y = fused
                nop = lower_matvec("FusedDownProj", ctx, w0=dense_weight(w_full), x=a_full, out=y,
                                   out_strides=flat_out_strides(y), kind="matvec")
                nop.keep += [a_full, w_full]
                out.append(nop)
                i += n
                continue
        if ctx.fuse and i + 1 < len(ops):
            fused_attn = _fuse_attention(sop, ops[i + 1], ctx)
            if fused_attn is not None:
                out.append(fused_attn)
                i += 2
                continue
        lowered = sop.op_cls.lower(sop, ctx)
        out.extend(lowered)
        i += 1
    return out


def _fuse_attention(split_sop: ScheduledOp, combine_sop: ScheduledOp, ctx: LowerCtx):
    """Split-KV attention followed by the combine of the same partials -> one op.

    The unit that completes a (batch, kv head, query tile) group combines the
    group's splits itself, so the combine needs no dependency stage of its own
    (and no CTA-wide event): one op boundary less per layer.
    """
    if split_sop.op_cls.__name__ != "FlashDecodingSplitBSHDOp" or \
            combine_sop.op_cls.__name__ != "FlashDecodingCombineBSHDOp":
        return None
    ts, tc = split_sop.tensor_refs, combine_sop.tensor_refs
    if ts["o_partial"].data_ptr() != tc["o_partial"].data_ptr() or \
            ts["lse_partial"].data_ptr() != tc["lse_partial"].data_ptr():
        return None
    o = tc["o"]
    if int(split_sop.static_dims["num_splits"]) > 128 or o.data_ptr() % 16 or any(st % 8 for st in o.stride()[:-1]):
        return None
    split = split_sop.op_cls.lower(split_sop, ctx)[0]
    comb = combine_sop.op_cls.lower(combine_sop, ctx)[0]
    groups = split.i[N.AT_B] * split.i[N.AT_HKV] * split.i[N.AT_MT]
    arrive = torch.zeros(groups, dtype=torch.int32, device=ts["q"].device)
    split.name = "FlashDecodingFused"
    split.i[N.AT_FUSE_COMBINE] = 1
    split.i[N.AT_O_T] = comb.i[N.AT_O_T]
    split.p[N.AT_P_O], split.p[N.AT_P_LSE] = comb.p[N.AT_P_O], comb.p[N.AT_P_LSE]
    split.p[N.AT_P_ARRIVE] = arrive.data_ptr()
    for k in (N.AT_S_O_B, N.AT_S_O_M, N.AT_S_O_H):
        split.s[k] = comb.s[k]
    split.writes = list(split.writes) + list(comb.writes)
    split.keep = list(split.keep) + list(comb.keep) + [arrive]
    split.zero_on_reset = [arrive]
    # consumers wait for the whole op (every unit signals; a group's last unit signals after its combine)
    split.n_groups, split.unit_group = 1, None
    return split
