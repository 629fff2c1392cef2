"""Llama-3.2-1B-shape decode: aliases, constants and the whole-model schedule.

The aliases and constants follow the reference's package
(src/machete/kernels/llama1b/sm100.py:3-29).  ``schedule_decode_model_sm100``
is this build's counterpart of ``schedule_decode_model_sm120``
(src/machete/kernels/llama1b/sm120.py:4679-4762) for B200: ``num_layers``
decoder layers with ping-pong activation buffers, then the final norm and
either bf16 logits or the fused greedy-token head.
"""

from __future__ import annotations

from ...megakernel.ops import DEFAULT_PAGE_SIZE
from .._batching import pick_batch_chunk, schedule_in_batch_chunks
from ..decode_matvec.sm100 import DecodeLayerSchedule as Llama1BLayerSchedule
from ..decode_matvec.sm100 import FinalRmsLmHeadSm100Op as Llama1BFinalRmsLmHeadSm100Op
from ..decode_matvec.sm100 import MatvecResidualSm100Op as Llama1BMatvecResidualSm100Op
from ..decode_matvec.sm100 import MatvecSm100Op as Llama1BDownMatvecSm100Op
from ..decode_matvec.sm100 import ResidualAddSm100Op as Llama1BResidualAddSm100Op
from ..decode_matvec.sm100 import RmsGateUpSiluSm100Op as Llama1BRmsGateUpSiluSm100Op
from ..decode_matvec.sm100 import RmsKMatvecRopeCacheSm100Op as Llama1BRmsKCacheSm100Op
from ..decode_matvec.sm100 import RmsQMatvecRopeSm100Op as Llama1BRmsQSm100Op
from ..decode_matvec.sm100 import RmsVMatvecCacheSm100Op as Llama1BRmsVCacheSm100Op
from ..decode_matvec.sm100 import schedule_decode_layer_sm100, schedule_final_sm100
from ..decode_matvec.top1 import schedule_final_top1_sm100

LLAMA1B_HIDDEN = 2048
LLAMA1B_HEAD_DIM = 64
LLAMA1B_ROTARY_D2 = 32
LLAMA1B_Q_DIM = 2048
LLAMA1B_KV_DIM = 512
LLAMA1B_INTERMEDIATE = 8192
LLAMA1B_VOCAB = 128256
LLAMA1B_MATVEC_BLOCK = 16
LLAMA1B_REDUCTION_DIM_PER_WARP = 512
LLAMA1B_CONSUMER_WARPS = 4
LLAMA1B_NUM_LAYERS = 16


def schedule_decode_model_sm100(
    *,
    batch,
    cache_pos,
    weights,
    k_cache,
    v_cache,
    x_buffers,
    residual_buffers,
    q_buf,
    attn_out_buf,
    mlp_h_buf,
    final_norm=None,
    lm_head=None,
    logits=None,
    top_values=None,
    top_indices=None,
    num_layers=LLAMA1B_NUM_LAYERS,
    seq_len=1,
    page_size=DEFAULT_PAGE_SIZE,
    eps=1e-5,
    fa_num_splits=0,
    hidden_size=LLAMA1B_HIDDEN,
    intermediate_size=LLAMA1B_INTERMEDIATE,
    num_q_heads=LLAMA1B_Q_DIM // LLAMA1B_HEAD_DIM,
    num_kv_heads=LLAMA1B_KV_DIM // LLAMA1B_HEAD_DIM,
    head_dim=LLAMA1B_HEAD_DIM,
    x_in=None,
    residual_in=None,
    tp_peers=None,
    position=None,
    embedding=None,
    batch_chunk=None,
):
    """Schedule a full decode step: ``(ops, keep_alive)``.

    ``k_cache`` / ``v_cache`` are per-layer lists of ``(B, T, H_kv, head_dim)``
    tensors; ``x_buffers`` / ``residual_buffers`` hold two ``(B, S, hidden)``
    ping-pong buffers each: layer ``i`` reads pair ``i % 2`` and writes the
    other.  The layer input is the pair (MLP delta ``x``, residual stream).
    With ``x_in`` / ``residual_in`` the first layer reads those tensors instead
    of pair 0, so the step never overwrites its own inputs and can be
    re-launched unchanged.

    ``tp_peers``: tensor parallelism over the ranks of a ``PeerBuffers``;
    ``weights``, the KV caches, ``q_buf`` / ``attn_out_buf`` / ``mlp_h_buf``, the
    head counts, ``intermediate_size`` and ``lm_head`` are then this rank's
    shards (see ``schedule_decode_layer_sm100``); full logits are not
    supported under tensor parallelism, only the greedy-token head.
    """
    # ``batch_chunk`` (None = as many rows as one op can stage, 0 = never chunk): a batch whose
    # activations do not fit shared memory runs as interleaved chunks (kernels/_batching.py)
    if batch_chunk is None:
        batch_chunk = 0
        if tp_peers is None and position is None:
            c = pick_batch_chunk(batch, seq_len, max(hidden_size, num_q_heads * head_dim))
            batch_chunk = c if c < batch else 0
    if batch_chunk and batch_chunk < batch:
        kw = dict(locals())
        kw.pop("batch_chunk")
        kw.pop("c", None)
        return schedule_in_batch_chunks(lambda **sub: schedule_decode_model_sm100(batch_chunk=0, **sub), batch_chunk, **kw)
    dynamic = position is not None
    if dynamic:
        # Generation loop (not in the reference, which re-schedules for every position,
        # src/machete/kernels/decode_matvec/sm100.py:116, 704-709): ``position`` is a one-element
        # int32 CUDA tensor holding the cache position of the token being decoded; the program
        # reads it at the start of every launch (pass it as ``MegakernelConfig(position=...)`` too),
        # writes the greedy token's embedding row (``embedding``, default: the tied ``lm_head``)
        # into ``x_in`` and advances the position, so every further launch decodes the next token.
        if x_in is None or top_indices is None or logits is not None or seq_len != 1:
            raise ValueError("position= needs x_in, the top-1 head and one token per step")
        # one element: every sequence of the batch sits at the same position; ``batch`` elements: each
        # sequence has its own (sequences of different lengths decode side by side)
        if position.numel() not in (1, batch):
            raise ValueError(f"position must hold 1 or {batch} (= batch) elements, got {position.numel()}")
        if tp_peers is not None and embedding is None:
            raise ValueError("position= under tensor parallelism needs the full embedding table (embedding=)")
    if tp_peers is not None and logits is not None:
        raise ValueError("tensor parallelism supports the top-1 head only (logits would need an all-gather)")
    if len(x_buffers) < 2 or len(residual_buffers) < 2:
        raise ValueError("x_buffers and residual_buffers must each contain two ping-pong buffers")
    if (x_in is None) != (residual_in is None):
        raise ValueError("x_in and residual_in must be given together")
    ops, keep = [], []
    cur = 0
    cur_x, cur_r = x_buffers[0], residual_buffers[0]
    if x_in is not None:
        cur, cur_x, cur_r = 1, x_in, residual_in      # layer 0 writes pair 0
    for layer_idx in range(num_layers):
        nxt = 1 - cur
        layer = schedule_decode_layer_sm100(
            layer_idx=layer_idx, batch=batch, seq_len=seq_len, cache_pos=cache_pos, weights=weights,
            k_cache=k_cache[layer_idx], v_cache=v_cache[layer_idx], x_in=cur_x,
            residual_in=cur_r, x_out=x_buffers[nxt], residual_out=residual_buffers[nxt],
            q_buf=q_buf, attn_out_buf=attn_out_buf, mlp_h_buf=mlp_h_buf, page_size=page_size, eps=eps,
            fa_num_splits=fa_num_splits, hidden_size=hidden_size, intermediate_size=intermediate_size,
            num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
            kv_group_size=num_q_heads // num_kv_heads, tp_peers=tp_peers, dynamic_position=dynamic,
        )
        ops += layer.ops
        keep += layer.keep_alive
        cur = nxt
        cur_x, cur_r = x_buffers[cur], residual_buffers[cur]
    if final_norm is not None and lm_head is not None:
        if logits is not None and (top_values is not None or top_indices is not None):
            raise ValueError("Provide either logits or top_values/top_indices, not both")
        if logits is not None:
            ops += schedule_final_sm100(x=x_buffers[cur], residual_in=residual_buffers[cur],
                                        residual_out=residual_buffers[1 - cur], final_norm=final_norm,
                                        lm_head=lm_head, logits=logits, seq_len=seq_len, page_size=page_size,
                                        eps=eps)
        elif top_values is not None and top_indices is not None:
            ops += schedule_final_top1_sm100(x=x_buffers[cur], residual_in=residual_buffers[cur],
                                             final_norm=final_norm, lm_head=lm_head, top_values=top_values,
                                             top_indices=top_indices, seq_len=seq_len, page_size=page_size,
                                             eps=eps, tp_peers=tp_peers,
                                             feedback=dict(embedding=lm_head if embedding is None else embedding,
                                                           x_in=x_in, position=position) if dynamic else None)
        else:
            raise ValueError("logits or both top_values/top_indices must be provided when lm_head is scheduled")
    return ops, keep


__all__ = [n for n in dir() if n.startswith(("LLAMA1B_", "Llama1B", "schedule_"))]
