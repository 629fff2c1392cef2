"""Decode-layer and whole-model schedules with NVFP4 weights on B200.

Same composition as ``schedule_decode_layer_sm100`` (the reference's bf16
B200 layer, src/machete/kernels/decode_matvec/sm100.py:666-823) built from the
NVFP4 op family the reference only has for sm_120
(src/machete/kernels/decode_matvec/sm120.py:596-2464): RMS + packed Q/K/V
projections with RoPE and the KV-cache append, split-KV attention, packed
O-projection with the residual, RMS + packed gate/up with SiLU, packed down
projection, and the greedy-token head over a packed LM head.

``weights`` holds, per matrix ``layer.{i}.W_x``, the keys ``...W_x.packed``
(uint8 ``(rows, K/2)``) and ``...W_x.scales`` (fp16 ``(rows, K/32)`` — the
reference's layout — or float8_e4m3fn ``(rows, K/16)`` with one fp32
``global_scale`` per matrix under ``...W_x.global_scale``).

Qwen3-style layers: when ``weights`` holds ``layer.{i}.q_norm`` / ``.k_norm``
(``(head_dim,)``), the Q and K projections are stored unrotated and a per-head
RMSNorm + RoPE pass (``QKNormRopeOp``, the composition of the reference's
src/machete/kernels/qwen_3_5/sm120.py:2986-2994) runs on ``q`` and on the new
cache row before attention.

``tp_peers`` (a ``PeerBuffers``) shards the layer Megatron-style exactly as the
bf16 layer does: ``weights`` hold this rank's shards (row-split Q/K/V/gate/up,
K-split O/down), head counts are the local ones, and the two K-split
projections write fp32 partials that the in-kernel all-reduce sums.
"""

from __future__ import annotations

import torch

from ...megakernel.ops import DEFAULT_PAGE_SIZE
from .._batching import pick_batch_chunk, schedule_in_batch_chunks
from ..qknorm_rope import QKNormRopeOp
from .nvfp4 import (MatvecNvfp4Sm120Op, MatvecResidualNvfp4Sm120Op, RmsGateUpSiluNvfp4Sm120Op,
                    RmsKMatvecRopeCacheNvfp4Sm120Op, RmsMatvecNvfp4Sm120Op, RmsQMatvecRopeNvfp4Sm120Op,
                    RmsVMatvecCacheNvfp4Sm120Op)
from .sm100 import DecodeLayerSchedule
from .top1 import schedule_final_top1_sm100


from ...megakernel.fusion import STAGING_BUDGET as _STAGING_BUDGET


def _w(weights, key):
    packed, scales = weights[f"{key}.packed"], weights[f"{key}.scales"]
    group = 16 if scales.element_size() == 1 else 32
    return dict(packed=packed, scales=scales, group_size=group, global_scale=float(weights.get(f"{key}.global_scale", 1.0)))


def schedule_decode_layer_nvfp4_sm100(*, layer_idx, batch, seq_len, cache_pos, weights, k_cache, v_cache, x_in,
                                      residual_in, x_out, residual_out, q_buf, attn_out_buf, mlp_h_buf,
                                      page_size=DEFAULT_PAGE_SIZE, eps=1e-6, fa_num_splits=0, num_q_heads=32,
                                      num_kv_heads=8, head_dim=128, tp_peers=None, fuse_qk_norm=True,
                                      dynamic_position=False):
    """One decoder layer with packed weights: ``DecodeLayerSchedule`` like the bf16 layer.

    ``fuse_qk_norm``: with q/k norm weights present, let the attention op apply the norm and the
    rotation itself (one dependency stage less per layer) instead of scheduling ``QKNormRopeOp``.
    ``dynamic_position`` (not in the reference): the step follows the program's device-resident cache
    position instead of ``cache_pos`` (see ``schedule_decode_layer_sm100``); a q/k-norm layer then needs
    the fused form."""
    from ..attention.flash_decoding import flash_decoding_schedule

    pfx = f"layer.{layer_idx}"
    if dynamic_position:
        if seq_len != 1:
            raise ValueError("a device-resident position decodes one token per sequence and step")
        if weights["cos"].shape[0] < k_cache.shape[1]:
            raise ValueError(f"RoPE tables hold {weights['cos'].shape[0]} positions, the cache {k_cache.shape[1]}")
        cache_pos = 0
        cos, sin = weights["cos"][:seq_len], weights["sin"][:seq_len]   # row 0: the kernel adds the position
        k_window, v_window = k_cache, v_cache
    else:
        cos = weights["cos"][cache_pos: cache_pos + seq_len]
        sin = weights["sin"][cache_pos: cache_pos + seq_len]
        k_window = k_cache[:, : cache_pos + seq_len]
        v_window = v_cache[:, : cache_pos + seq_len]
    q_4d = q_buf.view(batch, seq_len, num_q_heads, head_dim)
    o_4d = attn_out_buf.view(batch, seq_len, num_q_heads, head_dim)

    def proj(cls, key, **extra):
        w = _w(weights, f"{pfx}.{key}")
        return cls.schedule(x=x_in, residual_in=residual_in, norm_weight=weights[f"{pfx}.attn_norm"], cos=cos, sin=sin,
                            weight_packed=w["packed"], weight_scales=w["scales"], group_size=w["group_size"],
                            global_scale=w["global_scale"], tile_sizes={"S": seq_len, "O": 16}, page_size=page_size,
                            eps=eps, head_dim=head_dim, dynamic_pos=dynamic_position, **extra)

    ops, extra_keep, qk_norm = [], [], None
    if f"{pfx}.q_norm" in weights:
        if seq_len != 1 and batch != 1:
            raise ValueError("the QK-norm layer takes one token per sequence or one sequence")
        wq = _w(weights, f"{pfx}.W_q")
        ops += RmsMatvecNvfp4Sm120Op.schedule(x=x_in, residual_in=residual_in, norm_weight=weights[f"{pfx}.attn_norm"],
                                              weight_packed=wq["packed"], weight_scales=wq["scales"], y=q_buf,
                                              residual_out=residual_out, group_size=wq["group_size"],
                                              global_scale=wq["global_scale"], tile_sizes={"S": seq_len, "O": 16},
                                              page_size=page_size, eps=eps)
        ops += proj(RmsVMatvecCacheNvfp4Sm120Op, "W_k", dst_cache=k_window, cache_pos=cache_pos)   # unrotated
        ops += proj(RmsVMatvecCacheNvfp4Sm120Op, "W_v", dst_cache=v_window, cache_pos=cache_pos)
        if fuse_qk_norm and seq_len == 1 and num_q_heads // num_kv_heads <= 16 and cos.shape[1] * 2 == head_dim:
            # the attention op normalises and rotates q and the new k row itself: no extra stage
            qk_norm = dict(q_weight=weights[f"{pfx}.q_norm"], k_weight=weights[f"{pfx}.k_norm"], eps=eps,
                           new_token=cache_pos,
                           cos=weights["cos"] if dynamic_position else cos[0],
                           sin=weights["sin"] if dynamic_position else sin[0])
        elif dynamic_position:
            raise ValueError("a device-resident position needs the fused q/k norm (one token per sequence, "
                             "at most 16 query heads per KV head, full split-half rotation)")
        else:
            # row m = (b, s) of the (M, H, D) views takes the table row of token s
            cos_m, sin_m = cos.repeat(batch, 1), sin.repeat(batch, 1)
            q_rows = q_buf.view(batch * seq_len, num_q_heads, head_dim)
            k_rows = k_cache[:, cache_pos] if seq_len == 1 else k_cache[0, cache_pos: cache_pos + seq_len]
            ops += QKNormRopeOp.schedule(q=q_rows, norm_weight=weights[f"{pfx}.q_norm"], cos=cos_m, sin=sin_m, eps=eps,
                                         page_size=page_size)
            ops += QKNormRopeOp.schedule(q=k_rows, norm_weight=weights[f"{pfx}.k_norm"], cos=cos_m, sin=sin_m, eps=eps,
                                         page_size=page_size, cache_rows=(cache_pos, cache_pos + seq_len))
            extra_keep += [cos_m, sin_m, q_rows, k_rows]
    else:
        ops += proj(RmsQMatvecRopeNvfp4Sm120Op, "W_q", residual_out=residual_out, q=q_buf)
        ops += proj(RmsKMatvecRopeCacheNvfp4Sm120Op, "W_k", dst_cache=k_window, cache_pos=cache_pos)
        ops += proj(RmsVMatvecCacheNvfp4Sm120Op, "W_v", dst_cache=v_window, cache_pos=cache_pos)
    fa_ops, fa_config = flash_decoding_schedule(q=q_4d, k=k_window, v=v_window, o=o_4d,
                                                kv_group_size=num_q_heads // num_kv_heads, page_size=page_size,
                                                num_splits=fa_num_splits, qk_norm=qk_norm,
                                                dynamic_len=dynamic_position)
    ops += fa_ops
    wo = _w(weights, f"{pfx}.W_o")
    if tp_peers is not None:
        from ..allreduce import AllReduceSm100Op

        o_part = torch.empty(residual_out.shape, dtype=torch.float32, device=residual_out.device)
        x_part = torch.empty(x_out.shape, dtype=torch.float32, device=x_out.device)
        extra_keep += [o_part, x_part]
        ops += MatvecNvfp4Sm120Op.schedule(a=attn_out_buf, weight_packed=wo["packed"], weight_scales=wo["scales"],
                                           y=o_part, group_size=wo["group_size"], global_scale=wo["global_scale"],
                                           tile_sizes={"S": seq_len, "O": 16}, page_size=page_size)
        ops += AllReduceSm100Op.schedule(peers=tp_peers, x=o_part, residual_in=residual_out, y=residual_out)
    else:
        ops += MatvecResidualNvfp4Sm120Op.schedule(a=attn_out_buf, weight_packed=wo["packed"],
                                                   weight_scales=wo["scales"], residual_in=residual_out,
                                                   residual_out=residual_out, group_size=wo["group_size"],
                                                   global_scale=wo["global_scale"],
                                                   tile_sizes={"S": seq_len, "O": 16}, page_size=page_size)
    wg, wu = _w(weights, f"{pfx}.W_gate"), _w(weights, f"{pfx}.W_up")
    ops += RmsGateUpSiluNvfp4Sm120Op.schedule(x=residual_out, norm_weight=weights[f"{pfx}.mlp_norm"],
                                              gate_packed=wg["packed"], gate_scales=wg["scales"],
                                              up_packed=wu["packed"], up_scales=wu["scales"], y=mlp_h_buf,
                                              group_size=wg["group_size"], global_scale=wg["global_scale"],
                                              up_global_scale=wu["global_scale"],
                                              tile_sizes={"S": seq_len, "D": 16}, page_size=page_size, eps=eps)
    wd = _w(weights, f"{pfx}.W_down")
    # The activations of a matvec op are staged whole in shared memory.  When batch x intermediate
    # does not leave room for the weight pages, the down projection runs as K-blocks accumulated
    # into x_out, like the reference's bf16 layer (src/machete/kernels/decode_matvec/sm100.py:794-817).
    k_down, n_blk = int(mlp_h_buf.shape[-1]), 1
    while batch * seq_len * ((k_down // n_blk) * 2 + 64) > _STAGING_BUDGET or (n_blk > 1 and k_down % (n_blk * 2048)):
        n_blk += 1
        if n_blk > max(1, k_down // 2048):
            raise ValueError(f"batch {batch} x K {k_down}: the staged activations do not fit shared memory")
    g = wd["group_size"]

    def down_block(lo, hi, **out):
        a_blk = mlp_h_buf if (lo, hi) == (0, k_down) else mlp_h_buf[:, :, lo:hi]
        wp = wd["packed"] if (lo, hi) == (0, k_down) else wd["packed"][:, lo // 2: hi // 2]
        ws = wd["scales"] if (lo, hi) == (0, k_down) else wd["scales"][:, lo // g: hi // g]
        extra_keep.extend([a_blk, wp, ws])
        cls = MatvecResidualNvfp4Sm120Op if "residual_in" in out else MatvecNvfp4Sm120Op
        return cls.schedule(a=a_blk, weight_packed=wp, weight_scales=ws, group_size=g, global_scale=wd["global_scale"],
                            tile_sizes={"S": seq_len, "O": 16}, page_size=page_size, **out)

    if tp_peers is not None:
        # this rank's K range; a packed K above 2048 must be a multiple of 2048 (one scale tile row per
        # page), so e.g. 12 288 / 4 = 3072 runs as 2048 + 1024, each block with its own exchange:
        # x_out = sum(block 0), then x_out = sum(block 1) + x_out
        if n_blk > 1:
            raise ValueError("tensor-parallel NVFP4 layer: batch x local intermediate size does not fit shared memory")
        edges = [0, k_down] if (k_down <= 2048 or k_down % 2048 == 0) else \
            list(range(0, k_down, 2048)) + [k_down]
        for i, (lo, hi) in enumerate(zip(edges[:-1], edges[1:])):
            part = x_part if i == 0 else torch.empty_like(x_part)
            extra_keep.append(part)
            ops += down_block(lo, hi, y=part)
            ops += AllReduceSm100Op.schedule(peers=tp_peers, x=part, y=x_out,
                                             **({"residual_in": x_out} if i else {}))
    else:
        kb = k_down // n_blk
        for blk in range(n_blk):
            if blk == 0:
                ops += down_block(0, kb, y=x_out)
            else:
                ops += down_block(blk * kb, (blk + 1) * kb, residual_in=x_out, residual_out=x_out)
    return DecodeLayerSchedule(ops=ops, attention_config=fa_config,
                               keep_alive=[cos, sin, q_4d, k_window, v_window, o_4d, *extra_keep])


def schedule_decode_model_nvfp4_sm100(*, batch, cache_pos, weights, k_cache, v_cache, x_buffers, residual_buffers,
                                      q_buf, attn_out_buf, mlp_h_buf, top_values, top_indices, num_layers, x_in,
                                      residual_in, seq_len=1, page_size=DEFAULT_PAGE_SIZE, eps=1e-6, fa_num_splits=0,
                                      num_q_heads=32, num_kv_heads=8, head_dim=128, tp_peers=None, fuse_qk_norm=True,
                                      batch_chunk=None, position=None, embedding=None):
    """A full greedy decode step with packed weights: ``(ops, keep_alive)``.

    Layer ``i`` reads the pair (``x``, residual) it is given and writes the
    ping-pong pair ``x_buffers[j]`` / ``residual_buffers[j]``; the first layer
    reads ``x_in`` / ``residual_in`` so that the step can be re-launched.  The
    LM head is ``weights['lm_head.packed']`` / ``['lm_head.scales']``.  Under ``tp_peers`` the
    LM head is this rank's vocabulary shard and the ranks exchange their top-1 keys.

    ``position`` (not in the reference; see ``schedule_decode_model_sm100``): a 1- or ``batch``-element
    int32 CUDA tensor with the cache position of the token being decoded.  The program reads it at the
    start of every launch (pass it as ``MegakernelConfig(position=...)`` too), copies the greedy token's
    row of ``embedding`` (a ``(vocab, hidden)`` table of ``x_in``'s dtype: the packed LM head cannot
    serve as one) into ``x_in`` and advances the position: one handle decodes consecutive tokens.
    """
    # ``batch_chunk`` (None = as many rows as one op can stage, 0 = never chunk): a batch whose
    # activations do not fit shared memory runs as interleaved chunks (kernels/_batching.py)
    if batch_chunk is None:
        batch_chunk = 0
        if tp_peers is None and position is None:
            c = pick_batch_chunk(batch, seq_len, max(int(x_in.shape[-1]), num_q_heads * head_dim))
            batch_chunk = c if c < batch else 0
    if batch_chunk and batch_chunk < batch:
        kw = dict(locals())
        kw.pop("batch_chunk")
        kw.pop("c", None)
        return schedule_in_batch_chunks(lambda **sub: schedule_decode_model_nvfp4_sm100(batch_chunk=0, **sub),
                                        batch_chunk, **kw)
    dynamic = position is not None
    if dynamic:
        if seq_len != 1 or embedding is None:
            raise ValueError("position= needs one token per step and the embedding table (embedding=)")
        if position.numel() not in (1, batch):
            raise ValueError(f"position must hold 1 or {batch} (= batch) elements, got {position.numel()}")
    ops, keep = [], []
    cur, cur_x, cur_r = 1, x_in, residual_in
    for layer_idx in range(num_layers):
        nxt = 1 - cur
        layer = schedule_decode_layer_nvfp4_sm100(
            layer_idx=layer_idx, batch=batch, seq_len=seq_len, cache_pos=cache_pos, weights=weights,
            k_cache=k_cache[layer_idx], v_cache=v_cache[layer_idx], x_in=cur_x, residual_in=cur_r,
            x_out=x_buffers[nxt], residual_out=residual_buffers[nxt], q_buf=q_buf, attn_out_buf=attn_out_buf,
            mlp_h_buf=mlp_h_buf, page_size=page_size, eps=eps, fa_num_splits=fa_num_splits, num_q_heads=num_q_heads,
            num_kv_heads=num_kv_heads, head_dim=head_dim, tp_peers=tp_peers, fuse_qk_norm=fuse_qk_norm,
            dynamic_position=dynamic)
        ops += layer.ops
        keep += layer.keep_alive
        cur = nxt
        cur_x, cur_r = x_buffers[cur], residual_buffers[cur]
    lm = _w(weights, "lm_head")
    ops += schedule_final_top1_sm100(x=cur_x, residual_in=cur_r, final_norm=weights["final_norm"], lm_head=lm["packed"],
                                     lm_head_scales=lm["scales"], group_size=lm["group_size"],
                                     global_scale=lm["global_scale"], top_values=top_values, top_indices=top_indices,
                                     seq_len=seq_len, page_size=page_size, eps=eps, tp_peers=tp_peers,
                                     feedback=dict(embedding=embedding, x_in=x_in, position=position) if dynamic else None)
    return ops, keep


__all__ = ["schedule_decode_layer_nvfp4_sm100", "schedule_decode_model_nvfp4_sm100"]
