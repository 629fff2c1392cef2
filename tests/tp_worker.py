"""One rank of the 2-GPU tensor-parallel parity check (launched by tests/test_gpu_tp.py under torchrun).

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
D = dict(hidden=2048, inter=8192, nq=32, nkv=8, hd=64, vocab=32064, layers=2, T=512, pos=300)


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
    mk = Megakernel(ops, config=MegakernelConfig(timeout_ms=2000), device=dev, scheduler=OverlapTileScheduler())
    return mk, tv, ti, xb, rb, (kfull, vfull, x_in), keep


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    d = D
    weights = llama_weights(d["layers"], d["hidden"], d["inter"], d["nq"] * d["hd"], d["nkv"] * d["hd"], d["hd"] // 2,
                            d["T"], seed=1)
    lm = (torch.randn(d["vocab"], d["hidden"], generator=torch.Generator().manual_seed(2)) * 0.02).to(BF)
    peers = PeerBuffers(PeerBuffers.bytes_for_model(1, d["hidden"], d["layers"]) * 2, device=dev)
    mk, tv, ti, xb, rb, _, _keep = build(weights, lm, dev, world, rank, peers)
    mk.compile()
    tokens = []
    for _ in range(3):                       # several launches: epochs advance, inboxes alternate
        dist.barrier()
        mk.run()
        tokens.append((int(ti.item()), float(tv.item())))
    gathered = [None] * world
    dist.all_gather_object(gathered, tokens)
    ok = all(g == gathered[0] for g in gathered) and len(set(tokens)) == 1
    msg = f"rank {rank}: tokens {tokens}"
    if rank == 0:
        one, tv1, ti1, _, _, (kfull, vfull, x_in), _k2 = build(weights, lm, dev, 1, 0, None)
        one.run()
        want_idx, want_val = int(ti1.item()), float(tv1.item())
        _logits, o_val, o_idx = oracle.decode_model(weights=weights, x=x_in, residual=torch.zeros_like(x_in),
                                                    k_caches=[k.clone() for k in kfull],
                                                    v_caches=[v.clone() for v in vfull], cache_pos=d["pos"],
                                                    final_norm=torch.ones(d["hidden"], dtype=BF), lm_head=lm,
                                                    num_layers=d["layers"])
        ok = ok and tokens[0][0] == want_idx and abs(tokens[0][1] - want_val) < 2e-2
        ok = ok and int(o_idx.flatten()[0]) == tokens[0][0]
        msg += f" | single-GPU ({want_idx}, {want_val:.4f}) | oracle ({int(o_idx.flatten()[0])}, {float(o_val.flatten()[0]):.4f})"
    print(msg, flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
