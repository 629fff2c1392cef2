"""Batch chunks: decode batches whose staged activations exceed shared memory.

Every matvec op of the decode path stages ALL of its activation rows in shared memory
(rows x K), which bounds rows x K per op; the reference tiles the sequence/batch dimension of
its matvec ops instead (``tile_sizes={"S": ...}``, src/machete/kernels/decode_matvec/sm100.py:111).
The equivalent here is done on the schedule: the batch is cut into chunks, the model is scheduled
once per chunk on row views of every batch-indexed tensor, and the chunk programs are interleaved
op by op.  Chunks touch disjoint rows, so the inferred dependencies keep each chunk's chain and
nothing else; a chunk's pass over a weight matrix follows the previous chunk's pass at once, so
all but the first read the matrix from L2 (126 MB on B200), not from HBM — except for matrices
larger than L2 (the LM head), which are streamed once per chunk.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

# Bytes of staged activations that still leave a useful page ring (see megakernel/fusion.py).
STAGING_BUDGET = 100 * 1024

_ROW_TENSORS = ("q_buf", "attn_out_buf", "mlp_h_buf", "logits", "top_values", "top_indices", "x_in", "residual_in")
_ROW_LISTS = ("k_cache", "v_cache", "x_buffers", "residual_buffers")


def rows_that_fit(k: int, budget: int = STAGING_BUDGET) -> int:
    """Activation rows of width ``k`` (16-bit) one op can stage."""
    return max(1, budget // (k * 2 + 64))


def pick_batch_chunk(batch: int, seq_len: int, widest_k: int, budget: int = STAGING_BUDGET) -> int:
    """Largest divisor of ``batch`` whose rows (x ``seq_len``) of width ``widest_k`` fit the budget."""
    fit = rows_that_fit(widest_k, budget) // max(1, seq_len)
    for c in range(min(batch, max(1, fit)), 0, -1):
        if batch % c == 0:
            return c
    return 1


def schedule_in_batch_chunks(schedule: Callable[..., Tuple[list, list]], chunk: int, **kw) -> Tuple[list, list]:
    """Call ``schedule(batch=chunk, ...)`` per chunk on row views and interleave the ops op by op."""
    batch = int(kw["batch"])
    if chunk < 1 or batch % chunk:
        raise ValueError(f"batch_chunk {chunk} must divide the batch {batch}")
    if kw.get("tp_peers") is not None or kw.get("position") is not None:
        raise ValueError("batch chunks are not combined with tensor parallelism or a device-resident position")
    per_chunk: List[list] = []
    keep: list = []
    for b0 in range(0, batch, chunk):
        sub: Dict[str, object] = dict(kw)
        sub["batch"] = chunk
        for name in _ROW_TENSORS:
            t = kw.get(name)
            if isinstance(t, torch.Tensor):
                if t.shape[0] != batch:
                    raise ValueError(f"{name}: first dimension {t.shape[0]} is not the batch {batch}")
                sub[name] = t[b0:b0 + chunk]
        for name in _ROW_LISTS:
            ts = kw.get(name)
            if ts is not None:
                sub[name] = [t[b0:b0 + chunk] for t in ts]
        ops, k = schedule(**sub)
        per_chunk.append(ops)
        keep += list(k) + [v for v in sub.values() if isinstance(v, torch.Tensor)]
        keep += [t for name in _ROW_LISTS for t in (sub.get(name) or [])]
    n = len(per_chunk[0])
    if any(len(ops) != n for ops in per_chunk):
        raise RuntimeError("batch chunks scheduled different op lists")
    # ops that the lowering fuses when adjacent stay adjacent: they interleave as one group
    bounds = [i for i in range(n) if not _continues_group(per_chunk[0], i)] + [n]
    merged = [op for lo, hi in zip(bounds[:-1], bounds[1:]) for ops in per_chunk for op in ops[lo:hi]]
    return merged, keep


def _continues_group(ops: list, i: int) -> bool:
    """Does op ``i`` belong with op ``i - 1`` (attention split + combine, a K-block accumulation chain)?"""
    if i == 0:
        return False
    prev, cur = ops[i - 1], ops[i]
    pn, cn = prev.op_cls.__name__, cur.op_cls.__name__
    if pn.startswith("FlashDecodingSplit") and cn.startswith("FlashDecodingCombine"):
        return True
    if cn.startswith("MatvecResidual") and pn.startswith("Matvec"):
        out_prev = prev.tensor_ptrs.get("y", prev.tensor_ptrs.get("residual_out"))
        return out_prev is not None and out_prev == cur.tensor_ptrs.get("residual_out") == cur.tensor_ptrs.get("residual_in")
    return False


__all__ = ["STAGING_BUDGET", "rows_that_fit", "pick_batch_chunk", "schedule_in_batch_chunks"]
