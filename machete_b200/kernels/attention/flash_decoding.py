"""Split-KV flash decoding ops and ``flash_decoding_schedule``.

API mirror of the reference (src/machete/kernels/attention/flash_decoding.py:
``FlashDecodingSplitBSHDOp`` :1175, ``FlashDecodingCombineBSHDOp`` :1858,
``flash_decoding_schedule`` :1958): q/o are ``(B, M, H, D)``, k/v are
``(B, N, H_kv, D)`` (KV-cache views with arbitrary B/N/H strides), the split
op writes normalised fp32 ``o_partial (B, H, SPLIT, M, D)`` and
``lse_partial (B, H, SPLIT, M)``, the combine op writes ``o`` and
``lse (B, H, M)``.

Differences that matter for speed, not for results: a work unit serves one KV
head and all of its query heads (the reference tiles per query head and
re-reads each KV head ``group`` times), ``M == 1`` is native (the reference
needs ``M % 16 == 0``; padded inputs are accepted too), and the default split
count fills the SMs with KV-head units.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ... import _native as N
from ...megakernel.lowering import NativeOp, Region, attn_page_tokens, elem_type, meta_of
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Float32, Op

_DEFAULT_SMS = 148


def _num_sms(device) -> int:
    if torch.cuda.is_available() and torch.device(device).type == "cuda":
        return N.device_info(torch.device(device).index or 0)["num_sms"]
    return _DEFAULT_SMS


def default_num_splits(B: int, H_kv: int, m_tiles: int, N_kv: int, num_sms: int, min_tokens: int = 64) -> int:
    """Splits per (batch, KV head, query tile) so that units ~ a multiple of the SM count."""
    base = max(1, B * H_kv * m_tiles)
    max_splits = max(1, min(64, N_kv // min_tokens))
    # fill whole waves of SMs: the split count with the best wave efficiency wins,
    # a larger count must gain at least 3% to displace a smaller one (fewer partials)
    best, best_eff = 1, 0.0
    for s in range(1, max_splits + 1):
        units = base * s
        eff = units / (math.ceil(units / num_sms) * num_sms)
        if eff > best_eff + 0.03:
            best, best_eff = s, eff
    return best


class FlashDecodingSplitBSHDOp(Op):
    """Split-KV decode attention on native BSHD tensors."""

    reads = {
        "q": (None, ("B", "M", "H", "D")),
        "k": (None, ("B", "N", "H_kv", "D")),
        "v": (None, ("B", "N", "H_kv", "D")),
    }
    writes = {
        "o_partial": (Float32, ("B", "H", "SPLIT", "M", "D")),
        "lse_partial": (Float32, ("B", "H", "SPLIT", "M")),
    }
    tile = ("B", "H", "SPLIT")
    dynamic_dims = ("B", "M", "N", "SPLIT")
    tma_loads = {"q"}

    @classmethod
    def schedule(cls, tile_sizes=None, causal=False, page_size=DEFAULT_PAGE_SIZE, kv_group_size=1,
                 num_splits=0, qk_norm=None, dynamic_len=False, **tensors):
        """``qk_norm`` (not in the reference's signature): ``dict(q_weight, k_weight, cos, sin, eps,
        new_token)`` makes the op take UNROTATED q and an unrotated k row ``new_token`` (with
        ``dynamic_len``: the row of the device-resident position; ``cos`` / ``sin`` are then the whole
        ``(T, head_dim / 2)`` tables) and apply the
        per-head RMSNorm + split-half rotation itself (the reference schedules a separate
        ``QKNormRopeOp`` pass for that, src/machete/kernels/qwen_3_5/sm120.py:2986-2994); the finished
        k row is written back to the cache.  ``cos`` / ``sin`` are the ``(head_dim / 2,)`` table rows
        of that token."""
        q, k, v = tensors["q"], tensors["k"], tensors["v"]
        if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
            raise ValueError("flash decoding expects BSHD q and KV-cache k/v (rank 4)")
        B, M, H, D = (int(x) for x in q.shape)
        N_kv, H_kv = int(k.shape[1]), int(k.shape[2])
        if k.shape[0] != B or k.shape[3] != D or v.shape != k.shape:
            raise ValueError("q, k, v shapes are inconsistent")
        if q.element_size() != 2:
            raise ValueError("flash decoding needs fp16/bf16 tensors")
        if H % H_kv:
            raise ValueError(f"H={H} must be a multiple of H_kv={H_kv}")
        if kv_group_size not in (1, H // H_kv) and H != H_kv:
            raise ValueError(f"kv_group_size={kv_group_size} does not match H/H_kv={H // H_kv}")
        group = H // H_kv
        m_tiles = -(-(M * group) // 16)
        if num_splits <= 0:
            num_splits = default_num_splits(B, H_kv, m_tiles, N_kv, _num_sms(q.device))
        num_splits = max(1, min(int(num_splits), max(1, N_kv // 16)))
        o_partial = torch.empty(B, H, num_splits, M, D, dtype=torch.float32, device=q.device)
        lse_partial = torch.empty(B, H, num_splits, M, dtype=torch.float32, device=q.device)
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.update({"B": 1, "H": 1, "SPLIT": 1})
        tensors = dict(tensors, o_partial=o_partial, lse_partial=lse_partial)
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        sd = op.static_dims
        sd["page_size"] = page_size
        sd["num_splits"] = num_splits
        sd.update({"M": M, "N": N_kv, "H": H, "SPLIT": num_splits})
        sd["k_b_stride"], sd["k_n_stride"], sd["k_h_stride"] = k.stride(0), k.stride(1), k.stride(2)
        sd["v_b_stride"], sd["v_n_stride"], sd["v_h_stride"] = v.stride(0), v.stride(1), v.stride(2)
        if dynamic_len:
            # not in the reference: k / v are the FULL caches and the op attends to tokens [0, p + 1),
            # p being the program's device-resident cache position (MegakernelConfig.position)
            if causal or M != 1:
                raise ValueError("dynamic_len needs one token per sequence and no causal mask")
            sd["dynamic_len"] = 1
        if causal:
            sd["causal"] = 1
        if kv_group_size > 1:
            sd["kv_group_size"] = kv_group_size
        if qk_norm is not None:
            if M != 1 or group > 16:
                raise ValueError("fused q/k norm needs one token per sequence and at most 16 query heads per KV head")
            for name in ("q_weight", "k_weight"):
                w = qk_norm[name]
                if w.dtype != torch.bfloat16 or w.numel() != D or not w.is_contiguous() or w.data_ptr() % 16:
                    raise ValueError(f"qk_norm[{name!r}] must be a contiguous, 16-byte aligned bf16 ({D},) tensor")
            for name in ("cos", "sin"):
                r = qk_norm[name]
                if dynamic_len:
                    # the token follows the device-resident position: the whole (T, head_dim / 2) table
                    if r.dtype != torch.bfloat16 or r.ndim != 2 or r.shape[1] != D // 2 or r.stride(1) != 1 \
                            or r.stride(0) % 8 or r.data_ptr() % 16 or r.shape[0] < N_kv:
                        raise ValueError(f"qk_norm[{name!r}] must be the bf16 (>= {N_kv}, {D // 2}) table, 16-byte "
                                         "aligned rows, when the window follows the cache position")
                elif r.dtype != torch.bfloat16 or r.numel() != D // 2 or r.stride(-1) != 1 or r.data_ptr() % 16:
                    raise ValueError(f"qk_norm[{name!r}] must be the bf16 ({D // 2},) table row of the new token, "
                                     "16-byte aligned (full split-half rotation)")
            if not dynamic_len and not 0 <= int(qk_norm["new_token"]) < N_kv:
                raise ValueError("qk_norm['new_token'] must be a row of the cache window")
            if dynamic_len and qk_norm["cos"].stride(0) != qk_norm["sin"].stride(0):
                raise ValueError("qk_norm cos / sin tables must share their row stride")
            op.params["qk_norm"] = dict(qk_norm)
        return [op], o_partial, lse_partial

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=max(op.static_dims.get("page_size", DEFAULT_PAGE_SIZE) for op in ops))

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        q, k, v = t["q"], t["k"], t["v"]
        B, M, H, D = (int(x) for x in q.shape)
        N_kv, H_kv = int(k.shape[1]), int(k.shape[2])
        if D not in (64, 128):
            raise ValueError(f"flash decoding supports head_dim 64 and 128, got {D}")
        if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
            raise ValueError("flash decoding kernels are bf16")
        for name, x in (("q", q), ("k", k), ("v", v)):
            if x.stride(-1) != 1:
                raise ValueError(f"{name} needs a unit innermost stride")
        group = H // H_kv
        S = int(sop.static_dims["num_splits"])
        mt = -(-(M * group) // 16)
        per_split = -(-N_kv // S)
        ts = max(16, -(-per_split // 16) * 16)   # tokens per split, a multiple of 16
        tn = attn_page_tokens(D, ctx.page_bytes)
        if tn <= 0:
            raise ValueError("ring page too small for flash decoding")
        n_units = B * H_kv * mt * S
        op = NativeOp(name=cls.__name__, opcode=N.OP_ATTN_SPLIT, n_units=n_units, kind="attn_split")
        op.i = {N.AT_B: B, N.AT_M: M, N.AT_H: H, N.AT_HKV: H_kv, N.AT_D: D, N.AT_N: N_kv, N.AT_SPLITS: S,
                N.AT_CAUSAL: int(bool(sop.static_dims.get("causal", 0))), N.AT_MT: mt, N.AT_TS: ts,
                N.AT_O_T: N.T_BF16}
        op.f = {N.AT_F_SCALE: 1.0 / math.sqrt(D)}
        op.p = {N.AT_P_Q: q.data_ptr(), N.AT_P_K: k.data_ptr(), N.AT_P_V: v.data_ptr(),
                N.AT_P_OPART: t["o_partial"].data_ptr(), N.AT_P_LSEPART: t["lse_partial"].data_ptr()}
        op.s = {N.AT_S_Q_B: q.stride(0), N.AT_S_Q_M: q.stride(1), N.AT_S_Q_H: q.stride(2),
                N.AT_S_K_B: k.stride(0), N.AT_S_K_N: k.stride(1), N.AT_S_K_H: k.stride(2),
                N.AT_S_V_B: v.stride(0), N.AT_S_V_N: v.stride(1), N.AT_S_V_H: v.stride(2)}
        op.reads = [Region(meta_of(q, "q")), Region(meta_of(k, "k"), loader=True), Region(meta_of(v, "v"), loader=True)]
        op.writes = [Region(meta_of(t["o_partial"], "o_partial")), Region(meta_of(t["lse_partial"], "lse_partial"))]
        op.keep = [q, k, v, t["o_partial"], t["lse_partial"]]
        if sop.static_dims.get("dynamic_len"):
            op.i[N.AT_DYNPOS] = 1
            op.pos_limit = int(k.shape[1])
        qkn = sop.params.get("qk_norm")
        if qkn is not None:
            # with a device-resident position the slot carries the tables' row stride instead of the token
            op.i[N.AT_QKNORM] = 1
            op.i[N.AT_NEW_TOK] = int(qkn["cos"].stride(0)) if sop.static_dims.get("dynamic_len") else int(qkn["new_token"])
            op.f[N.AT_F_EPS] = float(qkn.get("eps", 1e-6))
            op.p.update({N.AT_P_QNW: qkn["q_weight"].data_ptr(), N.AT_P_KNW: qkn["k_weight"].data_ptr(),
                         N.AT_P_COS: qkn["cos"].data_ptr(), N.AT_P_SIN: qkn["sin"].data_ptr()})
            op.keep += [qkn["q_weight"], qkn["k_weight"], qkn["cos"], qkn["sin"]]
        sp = np.arange(n_units) % S
        tb = np.minimum(N_kv, sp * ts)
        te = np.minimum(N_kv, tb + ts)
        op.pages = (-(-(te - tb) // tn)).astype(np.int32)
        op.unit_bytes = ((te - tb) * D * 2 * 2).astype(np.int64)
        op.page_need = 4 * D * (64 if D == 64 else 32)
        # one completion counter per (batch, kv head): the combine of a head waits only for it
        op.n_groups = B * H_kv
        op.unit_group = (np.arange(n_units) // (mt * S)).astype(np.int64)
        op._split_tb, op._split_te = tb, te

        def loader_dep_units(producer, unit, tb=tb, te=te):
            # a cache-append producer writes token rows [lo, hi): only splits that cover them wait
            # (with a device-resident position hi is the cache length: every unit carries the wait
            # and the loader decides per launch which one holds the new row)
            for w in producer.writes:
                if w.axis == 1 and producer.kind == "cache_append":
                    return bool(tb[unit] < w.hi and te[unit] > w.lo)
            return True

        op.loader_dep_units = loader_dep_units
        return [op]


class FlashDecodingCombineBSHDOp(Op):
    """Log-sum-exp combine of the split partials into ``o`` (B, M, H, D)."""

    reads = {
        "o_partial": (Float32, ("B", "H", "SPLIT", "M", "D")),
        "lse_partial": (Float32, ("B", "H", "SPLIT", "M")),
    }
    writes = {
        "o": (None, ("B", "M", "H", "D")),
        "lse": (Float32, ("B", "H", "M")),
    }
    tile = ("B", "H")
    dynamic_dims = ("B", "M", "SPLIT")

    @classmethod
    def schedule(cls, tile_sizes=None, **tensors):
        tile_sizes = dict(tile_sizes or {})
        tile_sizes.update({"B": 1, "H": 1})
        op = cls._schedule_single(tile_sizes=tile_sizes, **tensors)
        o = tensors.get("o")
        if o is not None:
            op.static_dims["o_b_stride"] = o.stride(0)
            op.static_dims["o_m_stride"] = o.stride(1)
            op.static_dims["o_h_stride"] = o.stride(2)
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        opart, lpart, o, lse = t["o_partial"], t["lse_partial"], t["o"], t["lse"]
        B, H, S, M, D = (int(x) for x in opart.shape)
        if not opart.is_contiguous() or not lpart.is_contiguous() or not lse.is_contiguous():
            raise ValueError("partials and lse must be contiguous")
        if o.stride(-1) != 1:
            raise ValueError("o needs a unit innermost stride")
        op = NativeOp(name=cls.__name__, opcode=N.OP_ATTN_COMBINE, n_units=B * H, kind="attn_combine")
        op.i = {N.AT_B: B, N.AT_M: M, N.AT_H: H, N.AT_HKV: H, N.AT_D: D, N.AT_N: 0, N.AT_SPLITS: S,
                N.AT_O_T: elem_type(o, "o")}
        op.p = {N.AT_P_OPART: opart.data_ptr(), N.AT_P_LSEPART: lpart.data_ptr(), N.AT_P_O: o.data_ptr(),
                N.AT_P_LSE: lse.data_ptr()}
        op.s = {N.AT_S_O_B: o.stride(0), N.AT_S_O_M: o.stride(1), N.AT_S_O_H: o.stride(2)}
        op.reads = [Region(meta_of(opart, "o_partial")), Region(meta_of(lpart, "lse_partial"))]
        op.writes = [Region(meta_of(o, "o")), Region(meta_of(lse, "lse"))]
        op.keep = [opart, lpart, o, lse]
        op.unit_bytes = 0

        def fine_dep(consumer, producer, B=B, H=H, ptr=opart.data_ptr()):
            if producer.kind != "attn_split" or producer.p.get(N.AT_P_OPART) != ptr:
                return None
            h_kv = producer.i[N.AT_HKV]
            group = H // h_kv
            return [[(u // H) * h_kv + (u % H) // group] for u in range(B * H)]

        op.fine_dep = fine_dep
        return [op]


def flash_decoding_schedule(q, k, v, o, num_splits=0, page_size=DEFAULT_PAGE_SIZE, causal=False,
                            kv_group_size=1, qk_norm=None, dynamic_len=False):
    """Schedule split-KV flash decoding followed by its combine.

    Returns ``(ops, config)`` like the reference.  ``qk_norm``: see ``FlashDecodingSplitBSHDOp.schedule``.
    """
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4 or o.ndim != 4:
        raise ValueError("flash_decoding_schedule expects rank-4 BSHD tensors")
    B, M, H, D = q.shape
    lse = torch.empty(B, H, M, dtype=torch.float32, device=q.device)
    split_ops, o_partial, lse_partial = FlashDecodingSplitBSHDOp.schedule(
        q=q, k=k, v=v, num_splits=num_splits, page_size=page_size, causal=causal, kv_group_size=kv_group_size,
        qk_norm=qk_norm, dynamic_len=dynamic_len,
    )
    combine_ops = FlashDecodingCombineBSHDOp.schedule(o_partial=o_partial, lse_partial=lse_partial, o=o, lse=lse)
    ops = split_ops + combine_ops
    return ops, FlashDecodingSplitBSHDOp.kernel_config(ops)


# generic aliases the reference also exports
FlashDecodingSplitOp = FlashDecodingSplitBSHDOp
FlashDecodingCombineOp = FlashDecodingCombineBSHDOp

__all__ = [
    "FlashDecodingSplitOp", "FlashDecodingSplitBSHDOp", "FlashDecodingCombineOp", "FlashDecodingCombineBSHDOp",
    "flash_decoding_schedule", "default_num_splits",
]
