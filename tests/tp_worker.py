"""One rank of the 2/4/8-GPU tensor-parallel parity check (launched by tests/test_gpu_tp.py under torchrun).

Every rank builds the same seeded model, keeps its Megatron shard, runs the
sharded decode step with the in-kernel all-reduce, and rank 0 compares the
result with the unsharded step on its own GPU and with the CPU oracle.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import oracle  # noqa: E402
from machete_b200.kernels.llama1b import schedule_decode_model_sm100  # noqa: E402
from machete_b200.megakernel import Megakernel, MegakernelConfig, OverlapTileScheduler  # noqa: E402
from machete_b200.megakernel.peer import PeerBuffers  # noqa: E402
from tests.test_tp_host import shard_weights  # noqa: E402
from tests.util import llama_weights  # noqa: E402

BF = torch.bfloat16
D = dict(hidden=2048, inter=8192, nq=32, nkv=8, hd=64, vocab=32256, layers=2, T=512, pos=300)
# TP_MODE=nvfp4: Qwen3-style geometry (head dim 128, per-head q/k RMSNorm) with packed weights
D4 = dict(hidden=2048, inter=4096, nq=16, nkv=4, hd=128, vocab=4160, layers=2, T=256, pos=130)
D4["inter"] = int(os.environ.get("TP_INTER", D4["inter"]))   # 6144: two ranks get a K range of 3072 = 2048 + 1024 (two blocks, two exchanges)
MATS = ("W_q", "W_k", "W_v", "W_o", "W_gate", "W_up", "W_down")


def quantise_model(weights, lm, d):
    """Quantise every matrix whole (one global scale per matrix); returns (packed dict, dequantised dict)."""
    from machete_b200.quantization import dequantize_nvfp4_weight, quantize_nvfp4_weight

    g = torch.Generator().manual_seed(11)
    packed, deq = {"cos": weights["cos"], "sin": weights["sin"]}, dict(weights)
    names = [f"layer.{l}.{m}" for l in range(d["layers"]) for m in MATS]
    for name, mat in [(n, weights[n]) for n in names] + [("lm_head", lm)]:
        q = quantize_nvfp4_weight(mat, group_size=16)
        packed[f"{name}.packed"], packed[f"{name}.scales"] = q.packed, q.scales
        packed[f"{name}.global_scale"] = float(q.global_scale)
        deq[name] = dequantize_nvfp4_weight(q)
    for l in range(d["layers"]):
        for nm in ("attn_norm", "mlp_norm"):
            packed[f"layer.{l}.{nm}"] = weights[f"layer.{l}.{nm}"]
        for nm in ("q_norm", "k_norm"):
            deq[f"layer.{l}.{nm}"] = packed[f"layer.{l}.{nm}"] = (1 + torch.randn(d["hd"], generator=g) * 0.1).to(BF)
    return packed, deq


def shard_packed(packed, rank, world):
    """Megatron split of the packed tensors: rows for Q/K/V/gate/up/LM head, K (bytes and scale columns) for O/down."""
    out = {}
    for k, v in packed.items():
        parts = k.split(".")
        mat = parts[-2] if parts[-1] in ("packed", "scales") else None
        if mat in ("W_q", "W_k", "W_v", "W_gate", "W_up", "lm_head"):
            out[k] = v.chunk(world, dim=0)[rank].contiguous()
        elif mat in ("W_o", "W_down"):
            out[k] = v.chunk(world, dim=1)[rank].contiguous()
        else:
            out[k] = v
    return out


def build_nvfp4(packed, dev, world, rank, peers):
    from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100

    d = D4
    nq, nkv, inter = d["nq"] // world, d["nkv"] // world, d["inter"] // world
    g = torch.Generator().manual_seed(7)
    kfull = [torch.randn(1, d["T"], d["nkv"], d["hd"], generator=g).to(BF) for _ in range(d["layers"])]
    vfull = [torch.randn(1, d["T"], d["nkv"], d["hd"], generator=g).to(BF) for _ in range(d["layers"])]
    x_in = torch.randn(1, 1, d["hidden"], generator=g).to(BF)
    kc = [k.chunk(world, dim=2)[rank].contiguous().to(dev) for k in kfull]
    vc = [v.chunk(world, dim=2)[rank].contiguous().to(dev) for v in vfull]
    w = {k: (v.to(dev) if torch.is_tensor(v) else v)
         for k, v in (shard_packed(packed, rank, world) if world > 1 else packed).items()}
    w["final_norm"] = torch.ones(d["hidden"], dtype=BF, device=dev)
    z = lambda *s: torch.zeros(*s, dtype=BF, device=dev)   # noqa: E731
    tv = torch.zeros(1, 1, device=dev)
    ti = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    ops, keep = schedule_decode_model_nvfp4_sm100(
        batch=1, cache_pos=d["pos"], weights=w, k_cache=kc, v_cache=vc, x_buffers=[z(1, 1, d["hidden"]) for _ in range(2)],
        residual_buffers=[z(1, 1, d["hidden"]) for _ in range(2)], q_buf=z(1, 1, nq * d["hd"]),
        attn_out_buf=z(1, 1, nq * d["hd"]), mlp_h_buf=z(1, 1, inter), top_values=tv, top_indices=ti,
        num_layers=d["layers"], x_in=x_in.to(dev), residual_in=z(1, 1, d["hidden"]), num_q_heads=nq,
        num_kv_heads=nkv, head_dim=d["hd"], eps=1e-6, tp_peers=peers)
    mk = Megakernel(ops, config=MegakernelConfig(timeout_ms=int(os.environ.get("TP_TIMEOUT_MS", "2000"))), device=dev, scheduler=OverlapTileScheduler())
    return mk, tv, ti, None, None, (kfull, vfull, x_in), (keep, w)


def build(weights, lm, dev, world, rank, peers):
    d = D
    nq, nkv, inter = d["nq"] // world, d["nkv"] // world, d["inter"] // world
    g = torch.Generator().manual_seed(7)
    kfull = [torch.randn(1, d["T"], d["nkv"], d["hd"], generator=g).to(BF) for _ in range(d["layers"])]
    vfull = [torch.randn(1, d["T"], d["nkv"], d["hd"], generator=g).to(BF) for _ in range(d["layers"])]
    x_in = torch.randn(1, 1, d["hidden"], generator=g).to(BF)
    kc = [k.chunk(world, dim=2)[rank].contiguous().to(dev) for k in kfull]
    vc = [v.chunk(world, dim=2)[rank].contiguous().to(dev) for v in vfull]
    w = {k: v.to(dev) for k, v in (shard_weights(weights, rank, world, d) if world > 1 else weights).items()}
    xb = [torch.zeros(1, 1, d["hidden"], dtype=BF, device=dev) for _ in range(2)]
    rb = [torch.zeros(1, 1, d["hidden"], dtype=BF, device=dev) for _ in range(2)]
    tv = torch.zeros(1, 1, device=dev)
    ti = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    ops, keep = schedule_decode_model_sm100(
        batch=1, cache_pos=d["pos"], weights=w, k_cache=kc, v_cache=vc, x_buffers=xb, residual_buffers=rb,
        q_buf=torch.zeros(1, 1, nq * d["hd"], dtype=BF, device=dev),
        attn_out_buf=torch.zeros(1, 1, nq * d["hd"], dtype=BF, device=dev),
        mlp_h_buf=torch.zeros(1, 1, inter, dtype=BF, device=dev),
        final_norm=torch.ones(d["hidden"], dtype=BF, device=dev),
        lm_head=(lm.chunk(world, dim=0)[rank] if world > 1 else lm).contiguous().to(dev),
        top_values=tv, top_indices=ti, num_layers=d["layers"], hidden_size=d["hidden"], intermediate_size=inter,
        num_q_heads=nq, num_kv_heads=nkv, head_dim=d["hd"], x_in=x_in.to(dev),
        residual_in=torch.zeros(1, 1, d["hidden"], dtype=BF, device=dev), tp_peers=peers)
    mk = Megakernel(ops, config=MegakernelConfig(timeout_ms=int(os.environ.get("TP_TIMEOUT_MS", "2000"))), device=dev, scheduler=OverlapTileScheduler())
    return mk, tv, ti, xb, rb, (kfull, vfull, x_in), keep


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    nvfp4 = os.environ.get("TP_MODE", "bf16") == "nvfp4"
    d = D4 if nvfp4 else D
    weights = llama_weights(d["layers"], d["hidden"], d["inter"], d["nq"] * d["hd"], d["nkv"] * d["hd"], d["hd"] // 2,
                            d["T"], seed=1, **({"theta": 1000000.0} if nvfp4 else {}))
    lm = (torch.randn(d["vocab"], d["hidden"], generator=torch.Generator().manual_seed(2)) * 0.02).to(BF)
    peers = PeerBuffers(PeerBuffers.bytes_for_model(1, d["hidden"], d["layers"]) * 2, device=dev)
    oracle_kw = {}
    if nvfp4:
        packed, deq = quantise_model(weights, lm, d)
        mk, tv, ti, xb, rb, _, _keep = build_nvfp4(packed, dev, world, rank, peers)
        weights, lm = deq, deq["lm_head"]        # what the kernel multiplies by, exactly
        oracle_kw = dict(eps=1e-6, num_q_heads=d["nq"], num_kv_heads=d["nkv"], head_dim=d["hd"])
    else:
        mk, tv, ti, xb, rb, _, _keep = build(weights, lm, dev, world, rank, peers)
    mk.compile()
    tokens = []
    for _ in range(3):                       # several launches: epochs advance, inboxes alternate
        dist.barrier()
        mk.run()
        tokens.append((int(ti.item()), float(tv.item())))
    recovered = True
    if os.environ.get("TP_FAULT") == "1":
        # A rank that never joins one step (the failure is made on the host: the last rank simply
        # does not launch).  The others' bounded wait for its words gives up with a status, nobody
        # hangs; then, between steps and with no kernel in flight, the group agrees on a launch
        # count again and the next step must give the same token as before.
        failed = True
        if rank != world - 1:
            try:
                mk.run()
                failed = False
            except RuntimeError as exc:
                # the first wait to run out names the abort: the wait for the peer's words, or another
                # CTA's wait for the exchange op to complete
                failed = "megakernel aborted" in str(exc)
        dist.barrier()
        counts = [None] * world
        dist.all_gather_object(counts, mk.launch_count())
        agreed = mk.resync_launch_count()
        dist.barrier()
        mk.run()
        again = (int(ti.item()), float(tv.item()))
        recovered = failed and len(set(counts)) == 2 and agreed == max(counts) and again == tokens[0]
        print(f"rank {rank}: launch counts {counts} -> {agreed}, token after recovery {again}", flush=True)
    gathered = [None] * world
    dist.all_gather_object(gathered, tokens)
    ok = all(g == gathered[0] for g in gathered) and len(set(tokens)) == 1 and recovered
    msg = f"rank {rank}: tokens {tokens}"
    if rank == 0:
        if nvfp4:
            one, tv1, ti1, _, _, (kfull, vfull, x_in), _k2 = build_nvfp4(packed, dev, 1, 0, None)
        else:
            one, tv1, ti1, _, _, (kfull, vfull, x_in), _k2 = build(weights, lm, dev, 1, 0, None)
        one.run()
        want_idx, want_val = int(ti1.item()), float(tv1.item())
        _logits, o_val, o_idx = oracle.decode_model(weights=weights, x=x_in, residual=torch.zeros_like(x_in),
                                                    k_caches=[k.clone() for k in kfull],
                                                    v_caches=[v.clone() for v in vfull], cache_pos=d["pos"],
                                                    final_norm=torch.ones(d["hidden"], dtype=BF), lm_head=lm,
                                                    num_layers=d["layers"], **oracle_kw)
        # One bar for every comparison (tests/util.py): 2e-2 or two bf16 ulps of the largest logit.  The
        # sharded step, the unsharded step and the oracle must agree on the greedy token unless the
        # oracle's own top two logits are closer than that bar (the three sum K in different orders).
        from tests.util import parity_bar

        bar = parity_bar(_logits, roundings=2)
        top2 = _logits.flatten().topk(2).values
        clear_winner = float(top2[0] - top2[1]) > bar
        ok = ok and abs(tokens[0][1] - want_val) <= bar
        if clear_winner:
            ok = ok and tokens[0][0] == want_idx and int(o_idx.flatten()[0]) == tokens[0][0]
        ok = ok and abs(tokens[0][1] - float(_logits.flatten()[tokens[0][0]])) <= bar
        msg += f" | single-GPU ({want_idx}, {want_val:.4f}) | oracle ({int(o_idx.flatten()[0])}, {float(o_val.flatten()[0]):.4f})"
    print(msg, flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
