"""Tensor-parallel host logic on CPU: two gloo ranks build the sharded decode program.

Covers what needs no GPU: the ranks agree on every inbox / flag offset and
epoch base without exchanging them, each rank's program is deadlock-free
(`simulate`), the all-reduce ops carry the right rank / world fields, and the
sharding itself is sound (K-split partials add up to the unsplit product, the
vocabulary-split arg-max equals the global one).
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from machete_b200 import _native as N
from machete_b200.kernels.llama1b import schedule_decode_model_sm100
from machete_b200.megakernel import Megakernel, MegakernelConfig, OverlapTileScheduler, simulate
from machete_b200.megakernel.peer import PeerBuffers
from tests.util import llama_weights

BF = torch.bfloat16
DIMS = dict(hidden=256, inter=1024, nq=8, nkv=8, hd=64, vocab=1024, layers=2, T=128)


def shard_weights(w, rank, world, d):
    """Megatron split of a `llama_weights` dict: rows for Q/K/V/gate/up/LM head, K for O/down."""
    out = {}
    for k, v in w.items():
        name = k.split(".")[-1]
        if name in ("W_q", "W_k", "W_v", "W_gate", "W_up"):
            out[k] = v.chunk(world, dim=0)[rank].contiguous()
        elif name in ("W_o", "W_down"):
            out[k] = v.chunk(world, dim=1)[rank].contiguous()
        else:
            out[k] = v
    return out


def build_rank_program(rank, world):
    d = DIMS
    torch.manual_seed(0)
    w = llama_weights(d["layers"], d["hidden"], d["inter"], d["nq"] * d["hd"], d["nkv"] * d["hd"], d["hd"] // 2, d["T"])
    lm = (torch.randn(d["vocab"], d["hidden"]) * 0.02).to(BF)
    ws = shard_weights(w, rank, world, d)
    nq, nkv, inter = d["nq"] // world, d["nkv"] // world, d["inter"] // world
    kc = [torch.zeros(1, d["T"], nkv, d["hd"], dtype=BF) for _ in range(d["layers"])]
    vc = [torch.zeros(1, d["T"], nkv, d["hd"], dtype=BF) for _ in range(d["layers"])]
    xb = [torch.zeros(1, 1, d["hidden"], dtype=BF) for _ in range(2)]
    rb = [torch.zeros(1, 1, d["hidden"], dtype=BF) for _ in range(2)]
    peers = PeerBuffers(PeerBuffers.bytes_for_model(1, d["hidden"], d["layers"]), rank=rank, world_size=world)
    tv, ti = torch.zeros(1, 1), torch.zeros(1, 1, dtype=torch.int32)
    ops, _ = schedule_decode_model_sm100(
        batch=1, cache_pos=40, weights=ws, k_cache=kc, v_cache=vc, x_buffers=xb, residual_buffers=rb,
        q_buf=torch.zeros(1, 1, nq * d["hd"], dtype=BF), attn_out_buf=torch.zeros(1, 1, nq * d["hd"], dtype=BF),
        mlp_h_buf=torch.zeros(1, 1, inter, dtype=BF), final_norm=torch.ones(d["hidden"], dtype=BF),
        lm_head=lm.chunk(world, dim=0)[rank].contiguous(), top_values=tv, top_indices=ti, num_layers=d["layers"],
        hidden_size=d["hidden"], intermediate_size=inter, num_q_heads=nq, num_kv_heads=nkv, head_dim=d["hd"],
        tp_peers=peers)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=16), scheduler=OverlapTileScheduler())
    return mk, peers


def build_rank_program_nvfp4(rank, world):
    """The same with packed NVFP4 weights and Qwen3-style q/k norm (head dim 128): every matrix is
    quantised whole and the packed bytes / scale columns are split, as a loader of a real checkpoint would."""
    from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
    from machete_b200.quantization import quantize_nvfp4_weight

    d = dict(DIMS, hd=128, nq=8, nkv=8, hidden=1024, inter=12288, vocab=2048)   # 12288 / 4 ranks = 3072 = 2048 + 1024
    torch.manual_seed(0)
    w = llama_weights(d["layers"], d["hidden"], d["inter"], d["nq"] * d["hd"], d["nkv"] * d["hd"], d["hd"] // 2, d["T"])
    w["lm_head"] = (torch.randn(d["vocab"], d["hidden"]) * 0.02).to(BF)
    packed = {"cos": w["cos"], "sin": w["sin"], "final_norm": torch.ones(d["hidden"], dtype=BF)}
    for name in [f"layer.{l}.{m}" for l in range(d["layers"]) for m in
                 ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")] + ["lm_head"]:
        qz = quantize_nvfp4_weight(w[name], group_size=16)
        mat = name.split(".")[-1]
        dim = 1 if mat in ("W_o", "W_down") else 0
        packed[f"{name}.packed"] = qz.packed.chunk(world, dim=dim)[rank].contiguous()
        packed[f"{name}.scales"] = qz.scales.chunk(world, dim=dim)[rank].contiguous()
        packed[f"{name}.global_scale"] = float(qz.global_scale)
    for l in range(d["layers"]):
        for nm in ("attn_norm", "mlp_norm"):
            packed[f"layer.{l}.{nm}"] = w[f"layer.{l}.{nm}"]
        packed[f"layer.{l}.q_norm"] = packed[f"layer.{l}.k_norm"] = torch.ones(d["hd"], dtype=BF)
    nq, nkv, inter = d["nq"] // world, d["nkv"] // world, d["inter"] // world
    z = lambda *s: torch.zeros(*s, dtype=BF)   # noqa: E731
    peers = PeerBuffers(PeerBuffers.bytes_for_model(1, d["hidden"], d["layers"], 3), rank=rank, world_size=world)
    ops, _ = schedule_decode_model_nvfp4_sm100(
        batch=1, cache_pos=40, weights=packed, k_cache=[z(1, d["T"], nkv, d["hd"]) for _ in range(d["layers"])],
        v_cache=[z(1, d["T"], nkv, d["hd"]) for _ in range(d["layers"])],
        x_buffers=[z(1, 1, d["hidden"]) for _ in range(2)], residual_buffers=[z(1, 1, d["hidden"]) for _ in range(2)],
        q_buf=z(1, 1, nq * d["hd"]), attn_out_buf=z(1, 1, nq * d["hd"]), mlp_h_buf=z(1, 1, inter),
        top_values=torch.zeros(1, 1), top_indices=torch.zeros(1, 1, dtype=torch.int32), num_layers=d["layers"],
        x_in=z(1, 1, d["hidden"]), residual_in=z(1, 1, d["hidden"]), num_q_heads=nq, num_kv_heads=nkv,
        head_dim=d["hd"], tp_peers=peers)
    mk = Megakernel(ops, config=MegakernelConfig(num_sms=16), scheduler=OverlapTileScheduler())
    return mk, peers


def _worker(rank, world, port, q, nvfp4=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mk, peers = (build_rank_program_nvfp4 if nvfp4 else build_rank_program)(rank, world)
        final = simulate(mk.program)
        ok_counters = bool((final == mk.program.counter_expected[:len(final)]).all())
        ar = [(o.name, int(o.i[N.AR_RANK]), int(o.i[N.AR_P]), int(o.i[N.AR_N]), int(o.i[N.AR_MODE]),
               int(o.s[N.AR_S_INBOX]), int(o.s[N.AR_S_FLAGS]), int(o.i[N.AR_EPOCH_BASE]), int(o.n_units))
              for o in mk.native_ops if o.opcode == N.OP_ALLREDUCE]
        gathered = [None] * world
        dist.all_gather_object(gathered, ar)
        q.put((rank, ok_counters, gathered, len(mk.native_ops)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,nvfp4", [(2, False), (8, False), (4, True)])
def test_ranks_agree_on_the_exchange_layout(world, nvfp4):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, nvfp4)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_counters, gathered, n_ops in results:
        assert ok_counters                                   # every counter reaches its expected value: no lost signal
        a = gathered[0]
        # O-proj + down per layer and the key exchange; the NVFP4 case splits its local down-projection
        # K range of 3072 into 2048 + 1024, each with its own exchange
        per_layer = 3 if nvfp4 else 2
        assert all(len(g) == per_layer * DIMS["layers"] + 1 for g in gathered)
        for r, g in enumerate(gathered):
            for ra, rg in zip(a, g):
                assert ra[0] == rg[0] and ra[2:] == rg[2:]    # same op, world, size, mode, offsets, epoch base, units
                assert rg[1] == r and rg[2] == world          # and each carries its own rank
        offs = [r[5] for r in a] + [r[6] for r in a]
        assert len(set(offs)) == len(offs)                   # regions are distinct
        assert a[-1][4] == N.AR_MAX_KEY and all(r[4] == N.AR_SUM for r in a[:-1])


def test_sharded_math_adds_up():
    """K-split partials summed in rank order equal the unsplit matvec; split arg-max equals the global one."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 1024, generator=g).to(BF)
    w = (torch.randn(256, 1024, generator=g) * 0.02).to(BF)
    full = oracle.matvec(x, w)
    for world in (2, 4, 8):
        parts = [oracle.matvec(xs.contiguous(), ws.contiguous())
                 for xs, ws in zip(x.chunk(world, dim=1), w.chunk(world, dim=1))]
        acc = torch.zeros_like(parts[0])
        for p in parts:                                      # the kernel adds inbox slots in rank order
            acc = acc + p
        assert float((acc - full).abs().max()) < 1e-3
        logits = oracle.matvec(x, w).flatten()
        shard = logits.numel() // world
        best = max(((float(logits[r * shard:(r + 1) * shard].max()),
                     -(r * shard + int(logits[r * shard:(r + 1) * shard].argmax()))) for r in range(world)))
        assert -best[1] == int(logits.argmax())


def test_peer_buffers_reject_bad_worlds():
    with pytest.raises(ValueError):
        PeerBuffers(1024, rank=0, world_size=1)
    with pytest.raises(ValueError):
        PeerBuffers(1024, rank=0, world_size=16)
    pb = PeerBuffers(1024, rank=1, world_size=2)
    assert pb.alloc(100) == 0 and pb.alloc(100) == 256
    with pytest.raises(ValueError):
        pb.alloc(4096)
    assert pb.next_epoch_base() != pb.next_epoch_base()
