"""Attention: split-KV flash decoding with its combine (ops of the decode megakernel) and the
tcgen05 prefill kernel (a launch of its own)."""

from .flash_decoding import (FlashDecodingCombineBSHDOp, FlashDecodingCombineOp, FlashDecodingSplitBSHDOp,
                             FlashDecodingSplitOp, default_num_splits, flash_decoding_schedule)
from .prefill import FlashAttentionSm100Op, flash_prefill

FlashAttentionOp = FlashAttentionSm100Op


def flash_attention_schedule(q, k, v, o, causal=False, page_size=None, kv_group_size=1, lse=None, write_lse=None,
                             num_mma_warps=None):
    """Dispatcher of the reference (kernels/attention/__init__.py:48-130): ``(ops, config)``.

    Short-query problems (``M <= 64``, tensors ``(B, M, H, D)`` / ``(B, N, H_kv, D)``) go to flash
    decoding, whose ops run inside the decode megakernel.  Longer ones (the reference's
    ``(B, H, M, D)`` / ``(B, H_kv, N, D)`` layout) return the prefill op's record; run it with
    ``FlashAttentionSm100Op.launch(ops[0])`` (it is not a megakernel op, ``config`` is None).
    """
    from ...megakernel.ops import DEFAULT_PAGE_SIZE

    if q.shape[1] <= 64 and q.shape[1] % 16 == 0 and k.shape[2] * kv_group_size == q.shape[2]:
        return flash_decoding_schedule(q, k, v, o, causal=causal, page_size=page_size or DEFAULT_PAGE_SIZE,
                                       kv_group_size=kv_group_size)
    return FlashAttentionSm100Op.schedule(q=q, k=k, v=v, o=o, causal=causal, kv_group_size=kv_group_size, lse=lse,
                                          page_size=page_size or DEFAULT_PAGE_SIZE), None


__all__ = ["FlashDecodingSplitOp", "FlashDecodingSplitBSHDOp", "FlashDecodingCombineOp",
           "FlashDecodingCombineBSHDOp", "flash_decoding_schedule", "flash_attention_schedule",
           "default_num_splits", "FlashAttentionSm100Op", "FlashAttentionOp", "flash_prefill"]
