"""Decode attention: split-KV flash decoding and its combine."""

from .flash_decoding import (FlashDecodingCombineBSHDOp, FlashDecodingCombineOp, FlashDecodingSplitBSHDOp,
                             FlashDecodingSplitOp, default_num_splits, flash_decoding_schedule)


def flash_attention_schedule(q, k, v, o, causal=False, page_size=None, kv_group_size=1, lse=None, write_lse=None,
                             num_mma_warps=None):
    """Dispatcher kept for API parity (reference kernels/attention/__init__.py:48-130).

    The reference sends short-query problems to flash decoding and everything
    else to its prefill kernels; only the decode path exists in this build.
    """
    from ...megakernel.ops import DEFAULT_PAGE_SIZE

    if q.shape[1] > 64:
        raise ValueError("flash_attention_schedule: only the decode path (M <= 64) is available in this build")
    return flash_decoding_schedule(q, k, v, o, causal=causal, page_size=page_size or DEFAULT_PAGE_SIZE,
                                   kv_group_size=kv_group_size)


__all__ = ["FlashDecodingSplitOp", "FlashDecodingSplitBSHDOp", "FlashDecodingCombineOp",
           "FlashDecodingCombineBSHDOp", "flash_decoding_schedule", "flash_attention_schedule",
           "default_num_splits"]
