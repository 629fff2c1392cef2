"""Decoding consecutive tokens from ONE handle with a device-resident cache position.

The program is scheduled once.  Every launch reads the position from a device
scalar, appends this token's K/V rows at it, attends to the window that ends
there, picks the greedy token, copies its embedding row into the input buffer
and advances the position — no host work between launches.  The oracle runs
the same loop on the CPU: the tokens must agree step by step.
"""

import pytest
import torch

import oracle
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.megakernel import Megakernel, MegakernelConfig, OverlapTileScheduler
from tests.util import llama_weights, parity_bar, to_cpu

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("B,start", [(1, 60), (2, 125)])
def test_eight_consecutive_tokens_match_the_oracle(B, start):
    """`start` is chosen so that the window crosses a 64-token page (and a split boundary) on the way."""
    L, T, hidden, nq, nkv, hd, inter, vocab = 2, 256, 512, 8, 2, 64, 1024, 1024
    steps = 8
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=31, device="cuda")
    g = torch.Generator().manual_seed(32)
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    emb = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF)       # tied embedding / LM head
    x0 = emb[torch.arange(B) + 3].view(B, 1, hidden).clone()
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    dev = "cuda"
    x_in, kd, vd = x0.to(dev), [t.to(dev) for t in kcs], [t.to(dev) for t in vcs]
    position = torch.tensor([start], dtype=torch.int32, device=dev)
    tv = torch.zeros(B, 1, device=dev)
    ti = torch.zeros(B, 1, dtype=torch.int32, device=dev)
    dims = dict(hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    ops, _keep = schedule_decode_model_sm100(
        batch=B, cache_pos=0, weights=w, k_cache=kd, v_cache=vd,
        x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), final_norm=fn.to(dev), lm_head=emb.to(dev),
        top_values=tv, top_indices=ti, num_layers=L, x_in=x_in, residual_in=r0.to(dev), position=position, **dims)
    mk = Megakernel(ops, config=MegakernelConfig(position=position), scheduler=OverlapTileScheduler())
    wc = to_cpu(w)
    x = x0.clone()
    for step in range(steps):
        pos = start + step
        mk.run()
        assert int(position.item()) == pos + 1                     # the kernel advanced the position itself
        logits, _v, want_i = oracle.decode_model(weights=wc, x=x, residual=r0, k_caches=kcs, v_caches=vcs, cache_pos=pos,
                                                 final_norm=fn, lm_head=emb, num_layers=L, num_q_heads=nq,
                                                 num_kv_heads=nkv, head_dim=hd)
        got = ti.cpu()
        bar = parity_bar(logits, roundings=2 * L)      # the depth-aware bar of the whole-model tests
        top2 = logits.topk(2, dim=-1).values
        for b in range(B):
            # a near-tie would let the two loops drift apart for good: the seeds of this test have none
            assert float(top2[b, 0, 0] - top2[b, 0, 1]) > bar, "test input has a near-tie: pick another seed"
            assert int(got[b, 0]) == int(want_i[b, 0]), f"step {step}, row {b}: token differs"
            assert abs(float(tv[b, 0]) - float(logits[b, 0, int(got[b, 0])])) <= bar
        # the K/V rows of this position were appended (the oracle did the same to its caches)
        for l in range(L):
            assert float((kd[l][:, pos].cpu().float() - kcs[l][:, pos].float()).abs().max()) <= 2 * bar
        # the fed-back input row is the embedding of the greedy token, bit for bit
        x = emb[got[:, 0].long()].view(B, 1, hidden).clone()
        assert torch.equal(x_in.cpu(), x)
        assert mk.status()[0] == 0 and (mk.read_counters() == 0).all()


def test_graph_replay_decodes_consecutive_tokens():
    """One captured launch, replayed: each replay is the next token (what an e2e serving loop does)."""
    B, L, T, hidden, nq, nkv, hd, inter, vocab, start = 1, 1, 192, 512, 8, 2, 64, 1024, 512, 100
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=33, device="cuda")
    g = torch.Generator().manual_seed(34)
    dev = "cuda"
    kd = [torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)]
    vd = [torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)]
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF).to(dev)
    emb = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF).to(dev)
    x_in = emb[5].view(1, 1, hidden).clone()
    position = torch.tensor([start], dtype=torch.int32, device=dev)
    tv, ti = torch.zeros(B, 1, device=dev), torch.zeros(B, 1, dtype=torch.int32, device=dev)

    def build(pos_tensor, x, k, v):
        ops, _ = schedule_decode_model_sm100(
            batch=B, cache_pos=0, weights=w, k_cache=k, v_cache=v,
            x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
            residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
            q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
            mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), final_norm=fn, lm_head=emb, top_values=tv,
            top_indices=ti, num_layers=L, x_in=x, residual_in=torch.zeros(B, 1, hidden, dtype=BF, device=dev),
            position=pos_tensor, hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
        return Megakernel(ops, config=MegakernelConfig(position=pos_tensor), scheduler=OverlapTileScheduler())

    # reference run: plain launches on copies of the state
    k2, v2, x2, p2 = [kd[0].clone()], [vd[0].clone()], x_in.clone(), position.clone()
    plain = build(p2, x2, k2, v2)
    want = []
    for _ in range(6):
        plain.run()
        want.append(int(ti.item()))
    mk = build(position, x_in, kd, vd)
    mk.compile()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    host_tok = torch.zeros(B, 1, dtype=torch.int32).pin_memory()
    with torch.cuda.graph(graph, stream=side):
        mk.run(sync=False, validate=False)
        host_tok.copy_(ti, non_blocking=True)
    # the capture itself does not run the kernel: the position is still `start`
    got = []
    for _ in range(6):
        graph.replay()
        torch.cuda.synchronize()
        got.append(int(host_tok.item()))
    assert got == want
    assert int(position.item()) == start + 6


def test_position_past_the_cache_runs_nothing_and_reports_it():
    """A position outside the cache would append past its end: the launch does no work, the status
    names the position, and the handle decodes again once the position is back inside."""
    B, L, T, hidden, nq, nkv, hd, inter, vocab = 1, 1, 128, 512, 8, 2, 64, 1024, 512
    dev = "cuda"
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=35, device=dev)
    g = torch.Generator().manual_seed(36)
    kd = [torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)]
    vd = [torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)]
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF).to(dev)
    emb = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF).to(dev)
    x_in = emb[5].view(1, 1, hidden).clone()
    position = torch.tensor([T], dtype=torch.int32, device=dev)              # one past the last row
    tv, ti = torch.zeros(B, 1, device=dev), torch.full((B, 1), -1, dtype=torch.int32, device=dev)
    q_buf = torch.zeros(B, 1, nq * hd, dtype=BF, device=dev)
    ops, _ = schedule_decode_model_sm100(
        batch=B, cache_pos=0, weights=w, k_cache=kd, v_cache=vd,
        x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        q_buf=q_buf, attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), final_norm=fn, lm_head=emb, top_values=tv,
        top_indices=ti, num_layers=L, x_in=x_in, residual_in=torch.zeros(B, 1, hidden, dtype=BF, device=dev),
        position=position, hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    mk = Megakernel(ops, config=MegakernelConfig(position=position), scheduler=OverlapTileScheduler())
    k_before, x_before = kd[0].clone(), x_in.clone()
    with pytest.raises(RuntimeError, match="position is outside"):
        mk.run()
    assert torch.equal(kd[0], k_before) and torch.equal(x_in, x_before) and int(ti.item()) == -1
    assert int(position.item()) == T and float(q_buf.abs().max()) == 0.0
    for bad in (-1, T + 5):
        position.fill_(bad)
        with pytest.raises(RuntimeError, match="position is outside"):
            mk.run()
    position.fill_(T - 1)                                                   # the last row: a normal step
    mk.run()
    assert mk.status()[0] == 0 and int(position.item()) == T and 0 <= int(ti.item()) < vocab
    assert not torch.equal(kd[0][:, T - 1], k_before[:, T - 1]) and torch.equal(kd[0][:, :T - 1], k_before[:, :T - 1])


def test_sequences_of_different_lengths_decode_side_by_side():
    """One position per batch row: each sequence appends, rotates and attends at its own position,
    and every launch moves all of them on.  The oracle decodes each sequence on its own."""
    B, L, T, hidden, nq, nkv, hd, inter, vocab = 3, 2, 256, 512, 8, 2, 64, 1024, 1024
    starts, steps = [60, 125, 10], 6
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=37, device="cuda")
    g = torch.Generator().manual_seed(38)
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    emb = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF)
    x0 = emb[torch.tensor([3, 400, 77])].view(B, 1, hidden).clone()
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    dev = "cuda"
    x_in, kd, vd = x0.to(dev), [t.to(dev) for t in kcs], [t.to(dev) for t in vcs]
    position = torch.tensor(starts, dtype=torch.int32, device=dev)
    tv, ti = torch.zeros(B, 1, device=dev), torch.zeros(B, 1, dtype=torch.int32, device=dev)
    ops, _keep = schedule_decode_model_sm100(
        batch=B, cache_pos=0, weights=w, k_cache=kd, v_cache=vd,
        x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), final_norm=fn.to(dev), lm_head=emb.to(dev),
        top_values=tv, top_indices=ti, num_layers=L, x_in=x_in, residual_in=r0.to(dev), position=position,
        hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    mk = Megakernel(ops, config=MegakernelConfig(position=position), scheduler=OverlapTileScheduler())
    wc = to_cpu(w)
    x = x0.clone()
    for step in range(steps):
        mk.run()
        assert position.cpu().tolist() == [s0 + step + 1 for s0 in starts]
        got = ti.cpu()
        for b in range(B):
            pos = starts[b] + step
            kb, vb = [t[b:b + 1] for t in kcs], [t[b:b + 1] for t in vcs]      # views: the oracle appends in place
            logits, _v, want_i = oracle.decode_model(weights=wc, x=x[b:b + 1], residual=r0[b:b + 1], k_caches=kb, v_caches=vb,
                                                     cache_pos=pos, final_norm=fn, lm_head=emb, num_layers=L,
                                                     num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
            bar = parity_bar(logits, roundings=2 * L)
            top2 = logits.topk(2, dim=-1).values
            assert float(top2[0, 0, 0] - top2[0, 0, 1]) > bar, "test input has a near-tie: pick another seed"
            assert int(got[b, 0]) == int(want_i[0, 0]), f"step {step}, sequence {b}: token differs"
            for l in range(L):
                assert float((kd[l][b, pos].cpu().float() - kcs[l][b, pos].float()).abs().max()) <= 2 * bar
        x = emb[got[:, 0].long()].view(B, 1, hidden).clone()
        assert torch.equal(x_in.cpu(), x)
    # one sequence past its cache: nothing runs, the status names that row's position
    position[1] = T
    with pytest.raises(RuntimeError, match="position is outside"):
        mk.run()
    with pytest.raises(ValueError):
        schedule_decode_model_sm100(
            batch=B, cache_pos=0, weights=w, k_cache=kd, v_cache=vd,
            x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
            residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
            q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
            mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), final_norm=fn.to(dev), lm_head=emb.to(dev),
            top_values=tv, top_indices=ti, num_layers=L, x_in=x_in, residual_in=r0.to(dev),
            position=torch.zeros(2, dtype=torch.int32, device=dev),
            hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)


@pytest.mark.parametrize("qk_norm,B,seed", [(True, 1, 46), (True, 2, 52), (False, 1, 48)])
def test_nvfp4_model_decodes_consecutive_tokens_from_one_handle(qk_norm, B, seed):
    """The packed-weight model with a device-resident position (Qwen3 head geometry: head dim 128, q/k
    RMSNorm + rotation inside the attention op, whose table row follows the position too): six tokens
    from one handle against the oracle on the dequantised weights, step by step.  (The seeds are picked
    so that no step has a near-tie between its two best logits.)"""
    from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
    from machete_b200.quantization import dequantize_nvfp4_weight, quantize_nvfp4_weight

    L, T, hidden, nq, nkv, hd, inter, vocab, start, steps = 2, 128, 1024, 8, 2, 128, 2048, 256, 29, 6
    mats = ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=41, theta=1000000.0)
    g = torch.Generator().manual_seed(seed)
    emb = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    dev = "cuda"
    packed, deq = {"cos": w["cos"].to(dev), "sin": w["sin"].to(dev), "final_norm": fn.to(dev)}, dict(w)
    for name, mat in [(f"layer.{l}.{m}", w[f"layer.{l}.{m}"]) for l in range(L) for m in mats] + [("lm_head", lm)]:
        q = quantize_nvfp4_weight(mat, group_size=16)
        packed[f"{name}.packed"], packed[f"{name}.scales"] = q.packed.to(dev), q.scales.to(dev)
        packed[f"{name}.global_scale"] = float(q.global_scale)
        deq[name] = dequantize_nvfp4_weight(q)
    for l in range(L):
        packed[f"layer.{l}.attn_norm"] = w[f"layer.{l}.attn_norm"].to(dev)
        packed[f"layer.{l}.mlp_norm"] = w[f"layer.{l}.mlp_norm"].to(dev)
        if qk_norm:
            for nm in ("q_norm", "k_norm"):
                deq[f"layer.{l}.{nm}"] = (1 + torch.randn(hd, generator=g) * 0.1).to(BF)
                packed[f"layer.{l}.{nm}"] = deq[f"layer.{l}.{nm}"].to(dev)
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF) for _ in range(L)]
    kd, vd = [t.to(dev) for t in kcs], [t.to(dev) for t in vcs]
    x0 = emb[torch.arange(B) + 7].view(B, 1, hidden).clone()
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    x_in = x0.to(dev)
    # one position per sequence when there are two: they start two tokens apart
    pos0 = [start + 2 * b for b in range(B)]
    position = torch.tensor(pos0, dtype=torch.int32, device=dev)
    tv, ti = torch.zeros(B, 1, device=dev), torch.zeros(B, 1, dtype=torch.int32, device=dev)
    ops, _keep = schedule_decode_model_nvfp4_sm100(
        batch=B, cache_pos=0, weights=packed, k_cache=kd, v_cache=vd,
        x_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        residual_buffers=[torch.zeros(B, 1, hidden, dtype=BF, device=dev) for _ in range(2)],
        q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev), attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device=dev),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device=dev), top_values=tv, top_indices=ti, num_layers=L,
        x_in=x_in, residual_in=r0.to(dev), num_q_heads=nq, num_kv_heads=nkv, head_dim=hd, eps=1e-6,
        position=position, embedding=emb.to(dev))
    mk = Megakernel(ops, config=MegakernelConfig(position=position), scheduler=OverlapTileScheduler())
    x = x0.clone()
    for step in range(steps):
        mk.run()
        assert position.cpu().tolist() == [p + step + 1 for p in pos0]
        got = ti.cpu()
        for b in range(B):      # the oracle takes one position: row by row
            pos = pos0[b] + step
            logits, _v, want_i = oracle.decode_model(
                weights=deq, x=x[b:b + 1], residual=r0[b:b + 1], k_caches=[k[b:b + 1] for k in kcs],
                v_caches=[v[b:b + 1] for v in vcs], cache_pos=pos, final_norm=fn, lm_head=deq["lm_head"], num_layers=L,
                eps=1e-6, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
            bar = parity_bar(logits, roundings=2 * L)
            top2 = logits.topk(2, dim=-1).values
            assert float(top2[0, 0, 0] - top2[0, 0, 1]) > bar, "test input has a near-tie: pick another seed"
            assert int(got[b, 0]) == int(want_i[0, 0]), f"step {step}, row {b}: token differs"
            assert abs(float(tv[b, 0]) - float(logits[0, 0, int(got[b, 0])])) <= bar
            for l in range(L):   # this position's K/V rows were appended (the oracle appended to its views)
                assert float((kd[l][b, pos].cpu().float() - kcs[l][b, pos].float()).abs().max()) <= 2 * bar
        x = emb[got[:, 0].long()].view(B, 1, hidden).clone()
        assert torch.equal(x_in.cpu(), x)
        assert mk.status()[0] == 0 and (mk.read_counters() == 0).all()
