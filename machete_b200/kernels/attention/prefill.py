"""Prefill attention on the tcgen05 tensor cores (``mk_flash_prefill_bf16``).

API mirror of the reference's SM100 attention op (src/machete/kernels/attention/sm_100.py:88-…:
``q (B, H, M, D)``, ``k, v (B, H_kv, N, D)``, ``o (B, H, M, D)``, optional ``lse (B, H, M)``;
``schedule(causal=, kv_group_size=, ...)``) and of ``flash_attention_schedule``
(attention/__init__.py:48-130).  There the op is a handler inside the interpreter; here it is a
launch of its own (``csrc/attn_prefill_sm100.cu``) next to the decode megakernel, which keeps its
split-KV decode attention for a handful of query rows.  ``flash_prefill`` also takes the decode
path's own layouts — ``q / o (B, M, H, D)`` and cache views ``k / v (B, N, H_kv, D)`` — so that a
prompt's attention can run straight on the KV cache (``layout="bmhd"``).
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional

import torch

from ... import _native as N
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op

_status_blocks: Dict[int, torch.Tensor] = {}


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = f"{what}: {N.lib().mk_flash_prefill_last_error().decode('utf-8', 'replace')} (code {rc})"
    raise ValueError(msg) if rc in (-2, -3) else RuntimeError(msg)


def _strides(t: torch.Tensor, layout: str):
    """(batch, head, row) element strides of a 4-D tensor in ``bhmd`` or ``bmhd`` order."""
    if layout == "bhmd":
        return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    return (C.c_int64 * 3)(t.stride(0), t.stride(2), t.stride(1))


def flash_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, *, causal: bool = False,
                  scale: Optional[float] = None, lse: Optional[torch.Tensor] = None, layout: str = "bhmd",
                  timeout_ms: int = 1000, check_status: bool = False) -> torch.Tensor:
    """``o = softmax(scale * q k^T) v`` on the current stream; bf16, head dim 64 or 128.

    ``layout="bhmd"``: ``q, o (B, H, M, D)``, ``k, v (B, H_kv, N, D)`` (the reference's op);
    ``layout="bmhd"``: ``q, o (B, M, H, D)``, ``k, v (B, N, H_kv, D)`` (the decode path's buffers and
    KV cache views).  ``causal``: the queries are the last M of the N tokens.  ``lse``: optional
    ``(B, H, M)`` fp32 output.  ``check_status`` synchronises and raises if a device-side wait ran out.
    """
    if layout not in ("bhmd", "bmhd"):
        raise ValueError(f"layout must be 'bhmd' or 'bmhd', got {layout!r}")
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        if not t.is_cuda:
            raise RuntimeError("flash_prefill runs on a CUDA device only; there is no CPU path")
        if t.dtype != torch.bfloat16 or t.dim() != 4 or t.stride(-1) != 1:
            raise ValueError(f"flash_prefill: {name} must be a 4-D bfloat16 tensor with a contiguous head dimension")
    hd, md = (1, 2) if layout == "bhmd" else (2, 1)
    B, H, M, D = int(q.shape[0]), int(q.shape[hd]), int(q.shape[md]), int(q.shape[3])
    Hkv, Nk = int(k.shape[hd]), int(k.shape[md])
    if k.shape != v.shape or k.shape[0] != B or k.shape[3] != D or o.shape != q.shape:
        raise ValueError(f"flash_prefill: shapes q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)} o{tuple(o.shape)} do not match")
    if lse is not None and (lse.dtype != torch.float32 or tuple(lse.shape) != (B, H, M) or not lse.is_contiguous()):
        raise ValueError("flash_prefill: lse must be a contiguous float32 (B, H, M) tensor")
    dev = q.device.index if q.device.index is not None else torch.cuda.current_device()
    ws = _status_blocks.get(dev)
    if ws is None:
        ws = torch.zeros(512, dtype=torch.uint8, device=q.device)
        _status_blocks[dev] = ws
    base = (ws.data_ptr() + 255) // 256 * 256
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        _check(N.lib().mk_flash_prefill_bf16(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr() if lse is not None else None,
            B, H, Hkv, M, Nk, D, _strides(q, layout), _strides(k, layout), _strides(v, layout), _strides(o, layout),
            float(scale if scale is not None else 1.0 / math.sqrt(D)), int(bool(causal)), C.c_void_p(base), 256,
            int(timeout_ms), C.c_void_p(stream)), "mk_flash_prefill_bf16")
        if check_status:
            st = (C.c_int32 * 4)()
            _check(N.lib().mk_flash_prefill_status(C.c_void_p(base), st), "mk_flash_prefill_status")
            if st[0] != 0:
                ws.zero_()
                raise RuntimeError(f"flash_prefill aborted: wait {st[0]} ran out (cta={st[1]}, warp={st[2]}, tile={st[3]})")
    return o


class FlashAttentionSm100Op(Op):
    """The reference's op declaration; execution is a launch of its own (see the module docstring)."""

    reads = {"q": (None, ("B", "H", "M", "D")), "k": (None, ("B", "H_kv", "N", "D")), "v": (None, ("B", "H_kv", "N", "D"))}
    writes = {"o": (None, ("B", "H", "M", "D"))}
    tile = ("B", "H", "M", "D")
    tma_loads = {"q"}

    @classmethod
    def schedule(cls, causal=False, page_size=DEFAULT_PAGE_SIZE, kv_group_size=1, write_lse=None, lse=None,
                 num_mma_warps=None, tile_sizes=None, **tensors):
        q, k = tensors["q"], tensors["k"]
        if q.shape[1] != k.shape[1] * kv_group_size:
            raise ValueError(f"FlashAttentionSm100Op: {q.shape[1]} query heads are not {kv_group_size} x {k.shape[1]} KV heads")
        ts = dict(tile_sizes or {})
        ts.setdefault("B", 1)
        ts.setdefault("H", 1)
        ts.setdefault("M", 128)
        ts.setdefault("D", int(q.shape[-1]))
        op = cls._schedule_single(tile_sizes=ts, **tensors)
        op.static_dims.update(causal=int(bool(causal)), kv_group_size=int(kv_group_size), page_size=page_size)
        op.params.update(causal=bool(causal), lse=lse)
        return [op]

    @classmethod
    def launch(cls, sop, **kw) -> torch.Tensor:
        t = sop.tensor_refs
        return flash_prefill(t["q"], t["k"], t["v"], t["o"], causal=sop.params["causal"], lse=sop.params.get("lse"), **kw)

    @classmethod
    def lower(cls, sop, ctx):
        raise NotImplementedError("FlashAttentionSm100Op runs as its own launch (FlashAttentionSm100Op.launch / "
                                  "flash_prefill), not as an op of the decode megakernel; the decode step uses "
                                  "flash_decoding_schedule")


__all__ = ["flash_prefill", "FlashAttentionSm100Op"]
