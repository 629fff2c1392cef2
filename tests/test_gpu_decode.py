"""Decode layer and whole-model steps through the megakernel against the oracle."""

import pytest
import torch

import oracle
from machete_b200.kernels.decode_matvec import schedule_decode_layer_sm100, schedule_final_sm100
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.megakernel import Megakernel, MegakernelConfig, OverlapTileScheduler
from tests.util import assert_greedy_token, assert_parity, llama_weights, to_cpu

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def layer_inputs(B, S, T, hidden, nq, nkv, hd, inter, cache_pos, seed=0):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    kc = torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)
    vc = torch.randn(B, T, nkv, hd, generator=g).to(BF).to(dev)
    x_in = torch.randn(B, S, hidden, generator=g).to(BF).to(dev)
    res_in = torch.randn(B, S, hidden, generator=g).to(BF).to(dev)
    bufs = dict(q_buf=torch.zeros(B, S, nq * hd, dtype=BF, device=dev),
                attn_out_buf=torch.zeros(B, S, nq * hd, dtype=BF, device=dev),
                mlp_h_buf=torch.zeros(B, S, inter, dtype=BF, device=dev))
    return kc, vc, x_in, res_in, bufs


@pytest.mark.parametrize("fuse,sched", [(True, None), (False, None), (True, "overlap")])
def test_config0_llama1b_layer(fuse, sched):
    """BASELINE config 0: one Llama-3.2-1B-shape layer, batch 1, KV length 1024, eps 1e-5, theta 500000."""
    B, S, T, hidden, nq, nkv, hd, inter = 1, 1, 1024, 2048, 32, 8, 64, 8192
    cache_pos = T - 1
    w = llama_weights(1, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=0, device="cuda")
    kc, vc, x_in, res_in, bufs = layer_inputs(B, S, T, hidden, nq, nkv, hd, inter, cache_pos)
    x_out = torch.full((B, S, hidden), float("nan"), dtype=BF, device="cuda")
    res_out = torch.full((B, S, hidden), float("nan"), dtype=BF, device="cuda")
    kc_ref, vc_ref = kc.cpu().clone(), vc.cpu().clone()
    layer = schedule_decode_layer_sm100(layer_idx=0, batch=B, seq_len=S, cache_pos=cache_pos, weights=w, k_cache=kc,
                                        v_cache=vc, x_in=x_in, residual_in=res_in, x_out=x_out, residual_out=res_out,
                                        eps=1e-5, **bufs)
    mk = Megakernel(layer.ops, config=MegakernelConfig(fuse=fuse),
                    scheduler=OverlapTileScheduler() if sched else None)
    mk.run()
    want_x, want_res = oracle.decode_layer(weights=to_cpu(w), layer_idx=0, x_in=x_in.cpu(), residual_in=res_in.cpu(),
                                           k_cache=kc_ref, v_cache=vc_ref, cache_pos=cache_pos, eps=1e-5)
    assert_parity(kc[:, cache_pos], kc_ref[:, cache_pos], "appended K row")
    assert_parity(vc[:, cache_pos], vc_ref[:, cache_pos], "appended V row")
    assert torch.equal(kc[:, :cache_pos].cpu(), kc_ref[:, :cache_pos])      # older rows untouched
    assert_parity(res_out, want_res, "residual stream", roundings=2)         # the stream is stored twice in bf16
    assert_parity(x_out, want_x, "layer output")
    assert (mk.read_counters() == 0).all() and mk.status()[0] == 0
    # a second launch of the same handle gives the same bits (counters self-reset, no host work)
    first = x_out.clone()
    mk.run()
    assert torch.equal(first, x_out)


def test_llama1b_layer_at_batch_16_keeps_the_down_projection_in_k_blocks():
    """Config 3's largest batch at the real layer shape: 16 rows x 8192 intermediate values do not fit the
    activation staging, so the four K-blocks of the down projection stay separate ops (the oracle adds them
    in fp32; the chain rounds to bf16 in between, as the reference's does)."""
    B, S, T, hidden, nq, nkv, hd, inter = 16, 1, 256, 2048, 32, 8, 64, 8192
    cache_pos = 200
    w = llama_weights(1, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=3, device="cuda")
    kc, vc, x_in, res_in, bufs = layer_inputs(B, S, T, hidden, nq, nkv, hd, inter, cache_pos, seed=3)
    x_out = torch.full((B, S, hidden), float("nan"), dtype=BF, device="cuda")
    res_out = torch.full((B, S, hidden), float("nan"), dtype=BF, device="cuda")
    kc_ref, vc_ref = kc.cpu().clone(), vc.cpu().clone()
    layer = schedule_decode_layer_sm100(layer_idx=0, batch=B, seq_len=S, cache_pos=cache_pos, weights=w, k_cache=kc,
                                        v_cache=vc, x_in=x_in, residual_in=res_in, x_out=x_out, residual_out=res_out,
                                        eps=1e-5, **bufs)
    mk = Megakernel(layer.ops, scheduler=OverlapTileScheduler())
    mk.run()
    names = [o.name for o in mk.native_ops]
    assert "FusedDownProj" not in names and names.count("MatvecResidualSm100Op") == 1 + 3   # O-proj + 3 K-blocks
    want_x, want_res = oracle.decode_layer(weights=to_cpu(w), layer_idx=0, x_in=x_in.cpu(), residual_in=res_in.cpu(),
                                           k_cache=kc_ref, v_cache=vc_ref, cache_pos=cache_pos, eps=1e-5)
    assert_parity(res_out, want_res, "residual stream", roundings=2)
    assert_parity(x_out, want_x, "layer output at batch 16", roundings=4)   # three more bf16 stores than the oracle
    assert (mk.read_counters() == 0).all() and mk.status()[0] == 0


def test_padded_sixteen_row_step_and_batch():
    """The reference's 16-row contract (M % 16 == 0, non-causal over the window) and batch 2."""
    B, S, T, hidden, nq, nkv, hd, inter = 2, 16, 128, 512, 8, 2, 64, 1024
    cache_pos = 64
    w = llama_weights(1, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=1, device="cuda")
    kc, vc, x_in, res_in, bufs = layer_inputs(B, S, T, hidden, nq, nkv, hd, inter, cache_pos, seed=1)
    x_out = torch.empty(B, S, hidden, dtype=BF, device="cuda")
    res_out = torch.empty(B, S, hidden, dtype=BF, device="cuda")
    kc_ref, vc_ref = kc.cpu().clone(), vc.cpu().clone()
    layer = schedule_decode_layer_sm100(layer_idx=0, batch=B, seq_len=S, cache_pos=cache_pos, weights=w, k_cache=kc,
                                        v_cache=vc, x_in=x_in, residual_in=res_in, x_out=x_out, residual_out=res_out,
                                        hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv,
                                        head_dim=hd, kv_group_size=nq // nkv, **bufs)
    Megakernel(layer.ops).run()
    want_x, want_res = oracle.decode_layer(weights=to_cpu(w), layer_idx=0, x_in=x_in.cpu(), residual_in=res_in.cpu(),
                                           k_cache=kc_ref, v_cache=vc_ref, cache_pos=cache_pos, num_q_heads=nq,
                                           num_kv_heads=nkv, head_dim=hd)
    assert_parity(kc[:, cache_pos:cache_pos + S], kc_ref[:, cache_pos:cache_pos + S], "appended K rows")
    assert_parity(x_out, want_x, "layer output (B=2, S=16)")
    assert_parity(res_out, want_res, "residual", roundings=2)


@pytest.mark.parametrize("B,chunk", [(1, None), (4, None), (16, None), (32, 8), (12, 4)])
def test_multi_layer_model_greedy_token(B, chunk):
    """Four layers + final norm + LM head + arg-max; the token index must match exactly.  ``chunk``: the
    batch runs as interleaved chunks of that many rows (what a batch too large to stage does by itself)."""
    L, T, hidden, nq, nkv, hd, inter, vocab = 4, 512, 1024, 16, 4, 64, 2048, 8192 + 48
    cache_pos = 300
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=2, device="cuda")
    g = torch.Generator().manual_seed(5)
    kcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF).cuda() for _ in range(L)]
    vcs = [torch.randn(B, T, nkv, hd, generator=g).to(BF).cuda() for _ in range(L)]
    x0 = torch.randn(B, 1, hidden, generator=g).to(BF)
    r0 = torch.zeros(B, 1, hidden, dtype=BF)
    xb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    rb = [torch.zeros(B, 1, hidden, dtype=BF, device="cuda") for _ in range(2)]
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    tv = torch.zeros(B, 1, device="cuda")
    ti = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    dims = dict(hidden_size=hidden, intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    ops, keep = schedule_decode_model_sm100(
        batch=B, cache_pos=cache_pos, weights=w, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
        q_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        attn_out_buf=torch.zeros(B, 1, nq * hd, dtype=BF, device="cuda"),
        mlp_h_buf=torch.zeros(B, 1, inter, dtype=BF, device="cuda"), final_norm=fn.cuda(), lm_head=lm.cuda(),
        top_values=tv, top_indices=ti, num_layers=L, x_in=x0.cuda(), residual_in=r0.cuda(), batch_chunk=chunk, **dims)
    kc_ref, vc_ref = [t.cpu().clone() for t in kcs], [t.cpu().clone() for t in vcs]
    mk = Megakernel(ops, scheduler=OverlapTileScheduler())
    if chunk:
        assert len(ops) == (B // chunk) * (L * 9 + 2)           # every op once per chunk (2 down-projection K-blocks)
        assert [o.name for o in mk.native_ops].count("FlashDecodingFused") == (B // chunk) * L
    mk.run()
    logits, want_v, want_i = oracle.decode_model(weights=to_cpu(w), x=x0, residual=r0, k_caches=kc_ref, v_caches=vc_ref,
                                                 cache_pos=cache_pos, final_norm=fn, lm_head=lm, num_layers=L,
                                                 num_q_heads=nq, num_kv_heads=nkv, head_dim=hd)
    assert_greedy_token(ti.cpu(), tv.cpu(), logits, want_i, f"batch {B}")
    assert (mk.read_counters() == 0).all()
    # second launch: the keys were cleared by the finalise op, so the answer is stable
    first = ti.clone()
    mk.run()
    assert torch.equal(first, ti)


def test_logits_path_matches_top1():
    B, hidden, vocab = 2, 512, 1000
    g = torch.Generator().manual_seed(8)
    x = torch.randn(B, 1, hidden, generator=g).to(BF)
    r = torch.randn(B, 1, hidden, generator=g).to(BF)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    logits = torch.empty(B, 1, vocab, dtype=BF, device="cuda")
    ro = torch.empty(B, 1, hidden, dtype=BF, device="cuda")
    ops = schedule_final_sm100(x=x.cuda(), residual_in=r.cuda(), residual_out=ro, final_norm=fn.cuda(), lm_head=lm.cuda(),
                               logits=logits, seq_len=1)
    Megakernel(ops).run()
    want = oracle.final_rms_lm_head(x, fn, lm, 1e-5, residual_in=r)
    assert_parity(logits, want, "logits")
    assert torch.equal(ro.cpu(), (x.float() + r.float()).to(BF))


def test_run_is_capturable_in_a_cuda_graph():
    """`Megakernel.run(sync=False)` issues one kernel launch and nothing else, so a step with its
    host-to-device and device-to-host copies can be replayed as one CUDA graph (what `bench.py`'s
    end-to-end leg does): new input in the pinned buffer, replay, read the logits."""
    B, hidden, vocab = 1, 512, 1000
    g = torch.Generator().manual_seed(12)
    fn = (1 + torch.randn(hidden, generator=g) * 0.02).to(BF)
    lm = (torch.randn(vocab, hidden, generator=g) * 0.02).to(BF)
    x_dev = torch.zeros(B, 1, hidden, dtype=BF, device="cuda")
    r_dev = torch.zeros(B, 1, hidden, dtype=BF, device="cuda")
    logits = torch.empty(B, 1, vocab, dtype=BF, device="cuda")
    ro = torch.empty(B, 1, hidden, dtype=BF, device="cuda")
    host_x = torch.zeros(B, 1, hidden, dtype=BF).pin_memory()
    host_logits = torch.zeros(B, 1, vocab, dtype=BF).pin_memory()
    ops = schedule_final_sm100(x=x_dev, residual_in=r_dev, residual_out=ro, final_norm=fn.cuda(), lm_head=lm.cuda(),
                               logits=logits, seq_len=1)
    mk = Megakernel(ops)
    mk.run()                                   # compiles outside the capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        x_dev.copy_(host_x, non_blocking=True)
        mk.run(sync=False, validate=False)
        host_logits.copy_(logits, non_blocking=True)
    for seed in (1, 2):
        x = torch.randn(B, 1, hidden, generator=torch.Generator().manual_seed(seed)).to(BF)
        host_x.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        mk.wait()
        want = oracle.final_rms_lm_head(x, fn, lm, 1e-5, residual_in=torch.zeros_like(x))
        assert_parity(host_logits, want, f"logits of replay {seed}")
