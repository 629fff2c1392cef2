"""Host scheduler: dependency inference, fusion, placement, table invariants, deadlock freedom."""

import numpy as np
import pytest
import torch

from machete_b200.kernels.attention import flash_decoding_schedule
from machete_b200.kernels.decode_matvec import (MatvecResidualSm100Op, MatvecSm100Op, schedule_decode_layer_sm100,
                                                schedule_final_sm100)
from machete_b200.kernels.gemm import GemmOp
from machete_b200.kernels.glu import GLUOp
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.kernels.rms_norm import RMSNormOp
from machete_b200.megakernel import (BackwardScheduler, Megakernel, MegakernelConfig, OverlapTileScheduler,
                                     simulate)
from tests.util import llama_weights

BF = torch.bfloat16


def small_model(num_layers=2, B=1, T=256, hidden=256, inter=512, nq=4, nkv=2, hd=64, vocab=512):
    w = llama_weights(num_layers, hidden, inter, nq * hd, nkv * hd, hd // 2, T)
    kc = [torch.zeros(B, T, nkv, hd, dtype=BF) for _ in range(num_layers)]
    vc = [torch.zeros(B, T, nkv, hd, dtype=BF) for _ in range(num_layers)]
    xb = [torch.zeros(B, 1, hidden, dtype=BF) for _ in range(2)]
    rb = [torch.zeros(B, 1, hidden, dtype=BF) for _ in range(2)]
    bufs = dict(q_buf=torch.zeros(B, 1, nq * hd, dtype=BF), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF),
                mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF))
    return w, kc, vc, xb, rb, bufs, dict(hidden_size=hidden, intermediate_size=inter, num_q_heads=nq,
                                         num_kv_heads=nkv, head_dim=hd)


def test_chain_dependencies_and_counters():
    x = torch.zeros(1, 4, 256, dtype=BF)
    y = torch.zeros_like(x)
    h = torch.zeros(1, 4, 1024, dtype=BF)
    g = torch.zeros(1, 4, 512, dtype=BF)
    out = torch.zeros(1, 4, 256, dtype=BF)
    ops = RMSNormOp.schedule(x=x, weight=torch.ones(256, dtype=BF), y=y)
    ops += GemmOp.schedule(a=y, b=torch.zeros(1024, 256, dtype=BF), c=h)
    ops += GLUOp.schedule(x=h, y=g)
    ops += GemmOp.schedule(a=g, b=torch.zeros(256, 512, dtype=BF), c=out)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=8))
    deps = mk.program.deps
    assert [d.coarse for d in deps] == [[], [0], [1], [2]]
    assert mk.num_barriers == 4
    final = simulate(mk.program)
    assert (final == mk.program.counter_expected[:len(final)]).all()
    assert mk.total_tiles == sum(op.n_units for op in mk.native_ops)


def test_war_and_in_place_edges():
    a = torch.zeros(1, 1, 256, dtype=BF)
    b = torch.zeros(1, 1, 256, dtype=BF)
    w = torch.zeros(256, 256, dtype=BF)
    ops = MatvecSm100Op.schedule(a=a, weight=w, y=b)                       # 0: writes b
    ops += MatvecSm100Op.schedule(a=b, weight=w, y=torch.zeros_like(a))    # 1: reads b
    ops += MatvecSm100Op.schedule(a=a, weight=w, y=b)                      # 2: overwrites b -> WAR on 1
    ops += MatvecResidualSm100Op.schedule(a=a, weight=w, residual_in=b, residual_out=b)   # 3: in place on b
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=4, fuse=False))
    deps = [d.coarse for d in mk.program.deps]
    assert deps[1] == [0]
    assert deps[2] == [1]          # WAW on op 0 is implied by op 1
    assert deps[3] == [2]
    simulate(mk.program)


def test_layer_schedule_dependencies_and_fusion():
    w, kc, vc, xb, rb, bufs, dims = small_model(num_layers=1)
    layer = schedule_decode_layer_sm100(layer_idx=0, batch=1, seq_len=1, cache_pos=200, weights=w, k_cache=kc[0],
                                        v_cache=vc[0], x_in=xb[0], residual_in=rb[0], x_out=xb[1],
                                        residual_out=rb[1], kv_group_size=2, **bufs, **dims)
    names = [op.op_cls.__name__ for op in layer.ops]
    assert names[:3] == ["RmsQMatvecRopeSm100Op", "RmsKMatvecRopeCacheSm100Op", "RmsVMatvecCacheSm100Op"]
    assert names[3:5] == ["FlashDecodingSplitBSHDOp", "FlashDecodingCombineBSHDOp"]
    assert names[5:] == ["MatvecResidualSm100Op", "RmsGateUpSiluSm100Op", "MatvecSm100Op", "MatvecResidualSm100Op"]
    fused = Megakernel(layer.ops, config=MegakernelConfig(num_sms=16))
    plain = Megakernel(layer.ops, config=MegakernelConfig(num_sms=16, fuse=False))
    # fusion folds the combine into the split op and the four down-proj K-blocks into one matvec
    assert [o.name for o in fused.native_ops][3] == "FlashDecodingFused"
    assert [o.name for o in fused.native_ops][-1] == "FusedDownProj" and len(fused.native_ops) == 7
    assert len(plain.native_ops) == 9
    d = fused.program.deps
    assert d[0].coarse == [] and d[1].coarse == [] and d[2].coarse == []
    assert d[3].coarse == [0, 1, 2] and d[3].loader == [1, 2]           # split waits for q, k, v; loader for k, v
    assert d[4].coarse == [3] and d[5].coarse == [4] and d[6].coarse == [5]
    dp = plain.program.deps
    assert dp[4].coarse == [] and list(dp[4].fine) == [3]               # unfused: the combine waits per KV head
    # q/k/v share one staged activation; o-proj, gate/up and down each stage their own
    keys = [int(k) for k in fused.program.ops["act_key"]]
    assert keys[0] == keys[1] == keys[2] != 0
    assert len({keys[0], keys[4], keys[5], keys[6]}) == 4
    # only the split units that cover the appended token row carry loader waits
    ins = fused.program.instrs
    split = ins[ins["op"] == 3]
    n_splits = fused.native_ops[3].i[6]
    with_lw = split[split["n_lwaits"] > 0]["unit"]
    assert len(with_lw) == 2 and all(u % n_splits == n_splits - 1 for u in with_lw)
    for prog in (fused.program, plain.program):
        final = simulate(prog)
        assert (final == prog.counter_expected[:len(final)]).all()


def test_act_keys_change_across_layers_and_residual_out_written_once():
    w, kc, vc, xb, rb, bufs, dims = small_model(num_layers=3)
    tv, ti = torch.zeros(1, 1), torch.zeros(1, 1, dtype=torch.int32)
    ops, _ = schedule_decode_model_sm100(batch=1, cache_pos=100, weights=w, k_cache=kc, v_cache=vc, x_buffers=xb,
                                         residual_buffers=rb, final_norm=torch.ones(256, dtype=BF),
                                         lm_head=torch.zeros(512, 256, dtype=BF), top_values=tv, top_indices=ti,
                                         num_layers=3, **bufs, **dims)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=32), scheduler=OverlapTileScheduler())
    keys = [int(k) for k in mk.program.ops["act_key"]]
    q_ops = [i for i, o in enumerate(mk.native_ops) if o.name == "RmsQMatvecRopeSm100Op"]
    assert len({keys[i] for i in q_ops}) == 3          # layers 0 and 2 reuse buffers but not keys
    ev = mk.program.events
    for i in q_ops:
        mine = ev[ev["op"] == i]
        flagged = mine[(mine["flags"] & 1) == 1]              # residual_out is written by one CTA
        assert len(flagged) == 1
        # one counter per op: every CTA signals its units in bulk, and the bulk sizes add up
        assert ((mine["flags"] & 2) == 2).all()
        assert int(mine["bulk_units"].sum()) == mk.native_ops[i].n_units
    final = simulate(mk.program)
    assert (final == mk.program.counter_expected[:len(final)]).all()
    # every CTA list is a subsequence of program order
    p = mk.program
    for c in range(p.num_ctas):
        rows = p.instrs[p.cta_instr_begin[c]:p.cta_instr_begin[c + 1]]
        assert (np.diff(rows["op"]) >= 0).all()


def test_placements_cover_every_unit_once():
    w, kc, vc, xb, rb, bufs, dims = small_model(num_layers=1)
    layer = schedule_decode_layer_sm100(layer_idx=0, batch=1, seq_len=1, cache_pos=10, weights=w, k_cache=kc[0],
                                        v_cache=vc[0], x_in=xb[0], residual_in=rb[0], x_out=xb[1],
                                        residual_out=rb[1], kv_group_size=2, **bufs, **dims)
    for sched in (BackwardScheduler(), OverlapTileScheduler()):
        mk = Megakernel(layer.ops, config=MegakernelConfig(num_sms=7), scheduler=sched)
        ins = mk.program.instrs
        for j, op in enumerate(mk.native_ops):
            units = np.sort(ins[ins["op"] == j]["unit"])
            assert (units == np.arange(op.n_units)).all()
        spread = mk.program.bytes_per_cta
        if isinstance(sched, OverlapTileScheduler):
            assert spread.max() - spread.min() <= max(o.bytes_of(0) for o in mk.native_ops)


def test_simulator_detects_a_lost_signal():
    x = torch.zeros(1, 1, 256, dtype=BF)
    ops = MatvecSm100Op.schedule(a=x, weight=torch.zeros(256, 256, dtype=BF), y=torch.zeros_like(x))
    ops += MatvecSm100Op.schedule(a=ops[0].tensor_refs["y"], weight=torch.zeros(256, 256, dtype=BF), y=torch.zeros_like(x))
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=4))
    mk.program.waits["expected"][:] += 1          # nobody will ever signal that often
    with pytest.raises(RuntimeError, match="deadlock"):
        simulate(mk.program)


def test_flash_decoding_schedule_shapes_and_splits():
    q = torch.zeros(2, 1, 8, 64, dtype=BF)
    k = torch.zeros(2, 1000, 2, 64, dtype=BF)
    o = torch.zeros_like(q)
    ops, cfg = flash_decoding_schedule(q, k, k.clone(), o, num_splits=5, kv_group_size=4)
    split, comb = ops
    assert split.tensor_refs["o_partial"].shape == (2, 8, 5, 1, 64)
    assert split.tensor_refs["lse_partial"].shape == (2, 8, 5, 1)
    assert split.static_dims["num_splits"] == 5 and comb.tensor_refs["lse"].shape == (2, 8, 1)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=8, fuse=False))
    sp = mk.native_ops[0]
    assert sp.n_units == 2 * 2 * 1 * 5 and sp.n_groups == 4            # one counter per (batch, kv head)
    fused = Megakernel(ops, config=MegakernelConfig(num_sms=8)).native_ops
    assert len(fused) == 1 and fused[0].n_groups == 1 and fused[0].i[11] == 1   # combine folded into the split op
    ts = sp.i[9]
    assert ts % 16 == 0 and ts * 5 >= 1000
    assert int(np.sum(sp.unit_bytes)) == 2 * 2 * 1000 * 64 * 2 * 2     # K and V read exactly once
    with pytest.raises(ValueError):
        flash_decoding_schedule(q, k[..., :32], k[..., :32], o)


def test_final_schedule_and_too_many_rows():
    x = torch.zeros(1, 1, 256, dtype=BF)
    ops = schedule_final_sm100(x=x, residual_in=x.clone(), residual_out=x.clone(), final_norm=torch.ones(256, dtype=BF),
                               lm_head=torch.zeros(1000, 256, dtype=BF), logits=torch.zeros(1, 1, 1000, dtype=BF),
                               seq_len=1)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=4))
    assert [o.n_units for o in mk.native_ops] == [1, 63]
    big = torch.zeros(1, 64, 256, dtype=BF)
    with pytest.raises(ValueError, match="at most 32"):
        Megakernel(MatvecSm100Op.schedule(a=big, weight=torch.zeros(256, 256, dtype=BF), y=torch.zeros_like(big)),
                   config=MegakernelConfig(num_sms=4))


@pytest.mark.parametrize("fuse", [False, True])
def test_qk_norm_nvfp4_layer_schedules_without_deadlock(fuse):
    """The Qwen3-style layer (unrotated Q/K projections, per-head RMSNorm + RoPE on q and on the new
    cache row, then attention) lowers and simulates to completion on a small grid: as a separate
    pass that keeps the cache-row refinement for K, or folded into the attention op."""
    from machete_b200 import _native as N
    from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
    from machete_b200.megakernel import Megakernel, MegakernelConfig, OverlapTileScheduler, simulate
    from machete_b200.quantization import quantize_nvfp4_weight
    from tests.util import llama_weights

    BF = torch.bfloat16
    L, T, hidden, nq, nkv, hd, inter, vocab, B = 2, 96, 512, 4, 2, 128, 1024, 256, 2
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=2)
    packed = {"cos": w["cos"], "sin": w["sin"], "final_norm": torch.ones(hidden, dtype=BF)}
    names = [f"layer.{l}.{m}" for l in range(L) for m in ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")]
    w["lm_head"] = (torch.randn(vocab, hidden) * 0.02).to(BF)
    for name in names + ["lm_head"]:
        q = quantize_nvfp4_weight(w[name], group_size=16)
        packed[f"{name}.packed"], packed[f"{name}.scales"], packed[f"{name}.global_scale"] = (
            q.packed, q.scales, float(q.global_scale))
    for l in range(L):
        for nm in ("attn_norm", "mlp_norm"):
            packed[f"layer.{l}.{nm}"] = w[f"layer.{l}.{nm}"]
        packed[f"layer.{l}.q_norm"] = torch.ones(hd, dtype=BF)
        packed[f"layer.{l}.k_norm"] = torch.ones(hd, dtype=BF)
    z = lambda *s: torch.zeros(*s, dtype=BF)   # noqa: E731
    ops, _keep = schedule_decode_model_nvfp4_sm100(
        batch=B, cache_pos=40, weights=packed, k_cache=[z(B, T, nkv, hd) for _ in range(L)],
        v_cache=[z(B, T, nkv, hd) for _ in range(L)], x_buffers=[z(B, 1, hidden), z(B, 1, hidden)],
        residual_buffers=[z(B, 1, hidden), z(B, 1, hidden)], q_buf=z(B, 1, nq * hd), attn_out_buf=z(B, 1, nq * hd),
        mlp_h_buf=z(B, 1, inter), top_values=torch.zeros(B, 1), top_indices=torch.zeros(B, 1, dtype=torch.int32),
        num_layers=L, x_in=z(B, 1, hidden), residual_in=z(B, 1, hidden), num_q_heads=nq, num_kv_heads=nkv, head_dim=hd,
        fuse_qk_norm=fuse)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=8), scheduler=OverlapTileScheduler())
    qk = [o for o in mk.native_ops if o.name == "QKNormRopeOp"]
    attn = [o for o in mk.native_ops if o.name == "FlashDecodingFused"]
    if fuse:
        assert not qk and len(attn) == L
        assert all(o.i[N.AT_QKNORM] == 1 and o.i[N.AT_NEW_TOK] == 40 and o.p[N.AT_P_QNW] and o.p[N.AT_P_COS] for o in attn)
    else:
        assert len(qk) == 2 * L and not any(o.i.get(N.AT_QKNORM) for o in attn)
        assert [o.kind for o in qk] == ["qknorm_rope", "cache_append"] * L
        assert all(o.writes[-1].axis == 1 and (o.writes[-1].lo, o.writes[-1].hi) == (40, 41) for o in qk[1::2])
    final = simulate(mk.program)
    assert (final == mk.program.counter_expected[:len(final)]).all()


def test_batch_chunks_interleave_groups_and_keep_chunks_independent():
    """A batch too large to stage: the model is scheduled per chunk on row views and interleaved;
    the chunks' dependency chains do not touch each other."""
    import torch

    from machete_b200.kernels._batching import pick_batch_chunk, rows_that_fit, schedule_in_batch_chunks
    from machete_b200.kernels.llama1b import schedule_decode_model_sm100
    from machete_b200.megakernel.scheduling import resolve_dep_pairs
    from tests.util import llama_weights

    assert rows_that_fit(4096) == 12 and pick_batch_chunk(32, 1, 4096) == 8 and pick_batch_chunk(8, 1, 4096) == 8
    assert pick_batch_chunk(7, 1, 16384) == 1 and pick_batch_chunk(30, 1, 4096) == 10
    BF = torch.bfloat16
    B, L, T, hidden, nq, nkv, hd, inter, vocab = 32, 2, 64, 4096, 32, 8, 128, 8192, 256
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=1)
    z = lambda *s: torch.zeros(*s, dtype=BF)          # noqa: E731
    kw = dict(batch=B, cache_pos=40, weights=w, k_cache=[z(B, T, nkv, hd) for _ in range(L)],
              v_cache=[z(B, T, nkv, hd) for _ in range(L)], x_buffers=[z(B, 1, hidden) for _ in range(2)],
              residual_buffers=[z(B, 1, hidden) for _ in range(2)], q_buf=z(B, 1, nq * hd), attn_out_buf=z(B, 1, nq * hd),
              mlp_h_buf=z(B, 1, inter), final_norm=z(hidden), lm_head=z(vocab, hidden), top_values=torch.zeros(B, 1),
              top_indices=torch.zeros(B, 1, dtype=torch.int32), num_layers=L, x_in=z(B, 1, hidden),
              residual_in=z(B, 1, hidden), hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv,
              head_dim=hd)
    ops, _ = schedule_decode_model_sm100(**kw)                  # chunking picked by itself: 4 chunks of 8
    one, _ = schedule_decode_model_sm100(**{**kw, "batch": 8, **{k: (v[:8] if isinstance(v, torch.Tensor) and v.shape[0] == B
                                                                       else [t[:8] for t in v] if isinstance(v, list) else v)
                                                                   for k, v in kw.items() if k != "batch"}})
    assert len(ops) == 4 * len(one)
    names = [o.op_cls.__name__ for o in ops]
    assert names[:4] == ["RmsQMatvecRopeSm100Op"] * 4
    # split + combine stay adjacent (they fuse), and so does the down projection's K-block chain
    i = names.index("FlashDecodingSplitBSHDOp")
    assert names[i:i + 4] == ["FlashDecodingSplitBSHDOp", "FlashDecodingCombineBSHDOp"] * 2
    j = names.index("MatvecSm100Op")
    assert names[j:j + 4] == ["MatvecSm100Op", "MatvecResidualSm100Op", "MatvecSm100Op", "MatvecResidualSm100Op"]
    # the same x row range in every op of a chunk, and no dependency pair across chunks
    rows = [int(o.tensor_refs[o.op_cls.INPUTS[0]].shape[0]) for o in ops]
    assert set(rows) == {8}
    chunk_of = {}
    base = kw["q_buf"].data_ptr()
    for idx, o in enumerate(ops):
        t = o.tensor_refs
        probe = t.get("q", t.get("a", None))
        if probe is not None and probe.untyped_storage().data_ptr() == kw["q_buf"].untyped_storage().data_ptr():
            chunk_of[idx] = (probe.data_ptr() - base) // (8 * nq * hd * 2)
    pairs = resolve_dep_pairs(ops)
    assert pairs and all(chunk_of[p] == chunk_of[c] for p, c, _, _ in pairs if p in chunk_of and c in chunk_of)
    mk = Megakernel(ops)
    final = simulate(mk.program)                  # no deadlock: every counter reaches its expected count
    assert (final == mk.program.counter_expected[:len(final)]).all()
    with pytest.raises(ValueError):
        schedule_in_batch_chunks(schedule_decode_model_sm100, 5, **kw)
    with pytest.raises(ValueError):
        schedule_decode_model_sm100(**{**kw, "batch_chunk": 8, "position": torch.zeros(1, dtype=torch.int32)})


def test_nvfp4_model_with_device_resident_position_lowers_and_simulates():
    """`position=` on the packed-weight model: the cache-append ops and the attention op follow the
    position (the fused q/k norm gets the whole rotation tables and their row stride), the final op
    feeds the token back, the program still simulates to completion; the unfused q/k-norm pass and a
    missing embedding table are refused."""
    from machete_b200 import _native as N
    from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
    from machete_b200.quantization import quantize_nvfp4_weight

    L, T, hidden, nq, nkv, hd, inter, vocab, B = 2, 96, 512, 4, 2, 128, 1024, 256, 2
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=3)
    packed = {"cos": w["cos"], "sin": w["sin"], "final_norm": torch.ones(hidden, dtype=BF)}
    w["lm_head"] = (torch.randn(vocab, hidden) * 0.02).to(BF)
    for name in [f"layer.{l}.{m}" for l in range(L) for m in ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")] \
            + ["lm_head"]:
        q = quantize_nvfp4_weight(w[name], group_size=16)
        packed[f"{name}.packed"], packed[f"{name}.scales"], packed[f"{name}.global_scale"] = (
            q.packed, q.scales, float(q.global_scale))
    for l in range(L):
        for nm in ("attn_norm", "mlp_norm"):
            packed[f"layer.{l}.{nm}"] = w[f"layer.{l}.{nm}"]
        packed[f"layer.{l}.q_norm"] = torch.ones(hd, dtype=BF)
        packed[f"layer.{l}.k_norm"] = torch.ones(hd, dtype=BF)
    z = lambda *s: torch.zeros(*s, dtype=BF)   # noqa: E731
    position = torch.zeros(B, dtype=torch.int32)
    emb = z(vocab, hidden)

    def schedule(**kw):
        return schedule_decode_model_nvfp4_sm100(
            batch=B, cache_pos=0, weights=packed, k_cache=[z(B, T, nkv, hd) for _ in range(L)],
            v_cache=[z(B, T, nkv, hd) for _ in range(L)], x_buffers=[z(B, 1, hidden), z(B, 1, hidden)],
            residual_buffers=[z(B, 1, hidden), z(B, 1, hidden)], q_buf=z(B, 1, nq * hd), attn_out_buf=z(B, 1, nq * hd),
            mlp_h_buf=z(B, 1, inter), top_values=torch.zeros(B, 1), top_indices=torch.zeros(B, 1, dtype=torch.int32),
            num_layers=L, x_in=z(B, 1, hidden), residual_in=z(B, 1, hidden), num_q_heads=nq, num_kv_heads=nkv,
            head_dim=hd, **kw)

    ops, _keep = schedule(position=position, embedding=emb)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=8, position=position), scheduler=OverlapTileScheduler())
    attn = [o for o in mk.native_ops if o.name == "FlashDecodingFused"]
    assert len(attn) == L
    for o in attn:
        assert o.i[N.AT_DYNPOS] == 1 and o.i[N.AT_QKNORM] == 1 and o.pos_limit == T
        assert o.i[N.AT_NEW_TOK] == w["cos"].stride(0)                     # the tables' row stride, not a token
        assert o.p[N.AT_P_COS] == w["cos"].data_ptr() and o.p[N.AT_P_SIN] == w["sin"].data_ptr()
    appends = [o for o in mk.native_ops if o.kind == "cache_append"]
    assert len(appends) == 2 * L
    for o in appends:
        assert o.i[N.MV_DYNPOS] == N.MV_DYN_OUT and o.pos_limit == T         # K and V stay unrotated here
        assert (o.writes[-1].lo, o.writes[-1].hi) == (0, T)                  # any row may be the one written
    final = simulate(mk.program)
    assert (final == mk.program.counter_expected[:len(final)]).all()
    with pytest.raises(ValueError, match="embedding"):
        schedule(position=position)
    with pytest.raises(ValueError, match="fused q/k norm"):
        schedule(position=position, embedding=emb, fuse_qk_norm=False)
    with pytest.raises(ValueError, match="position must hold"):
        schedule(position=torch.zeros(B + 1, dtype=torch.int32), embedding=emb)
