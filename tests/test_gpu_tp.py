"""Tensor-parallel decode on 2, 4 and 8 GPUs: the sharded step with the in-kernel all-reduce must
produce the token of the unsharded step and of the CPU oracle.

Each rank is its own process on its own GPU (kernels that wait on one another
must never share a GPU), launched with torchrun; a case is skipped on a box
with fewer GPUs than ranks.  All device-side waits are bounded, so a failure is
an error code, not a hang.
"""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shard_programs_compile_at_llama1b_shapes(world):
    """One GPU is enough to validate the sharded programs: every rank's shapes (K = 256 O-proj shards,
    one KV head per rank, 16032-row vocabulary shards ...) must pass the library's checks and get their
    tensor maps.  The program is compiled, not launched (its peers do not exist here)."""
    from machete_b200.kernels.llama1b import schedule_decode_model_sm100
    from machete_b200.megakernel import Megakernel, OverlapTileScheduler
    from machete_b200.megakernel.peer import PeerBuffers
    from tests.util import llama_weights

    BF, dev = torch.bfloat16, "cuda"
    hidden, nq, nkv, hd, inter, vocab, L, T = 2048, 32 // world, 8 // world, 64, 8192 // world, 128256 // world, 2, 512
    w = llama_weights(L, hidden, inter, nq * hd, nkv * hd, hd // 2, T, seed=3, device=dev)
    for l in range(L):   # `llama_weights` builds square-ish layers: O-proj and down are the K-split ones
        assert w[f"layer.{l}.W_o"].shape == (hidden, nq * hd) and w[f"layer.{l}.W_down"].shape == (hidden, inter)
    peers = PeerBuffers(PeerBuffers.bytes_for_model(1, hidden, L), rank=world - 1, world_size=world)   # table only
    tv, ti = torch.zeros(1, 1, device=dev), torch.zeros(1, 1, dtype=torch.int32, device=dev)
    z = lambda *s: torch.zeros(*s, dtype=BF, device=dev)   # noqa: E731
    ops, _keep = schedule_decode_model_sm100(
        batch=1, cache_pos=300, weights=w, k_cache=[z(1, T, nkv, hd) for _ in range(L)],
        v_cache=[z(1, T, nkv, hd) for _ in range(L)], x_buffers=[z(1, 1, hidden), z(1, 1, hidden)],
        residual_buffers=[z(1, 1, hidden), z(1, 1, hidden)], q_buf=z(1, 1, nq * hd), attn_out_buf=z(1, 1, nq * hd),
        mlp_h_buf=z(1, 1, inter), final_norm=torch.ones(hidden, dtype=BF, device=dev), lm_head=z(vocab, hidden),
        top_values=tv, top_indices=ti, num_layers=L, hidden_size=hidden, intermediate_size=inter, num_q_heads=nq,
        num_kv_heads=nkv, head_dim=hd, x_in=z(1, 1, hidden), residual_in=z(1, 1, hidden), tp_peers=peers)
    mk = Megakernel(ops, scheduler=OverlapTileScheduler())
    mk.compile()                       # mk_create: validation + tensor maps; raises on any rejected shape
    assert mk.total_tiles > 0


@pytest.mark.parametrize("mode,world", [("bf16", 2), ("nvfp4", 2), ("nvfp4_split", 2), ("bf16_fault", 2), ("bf16", 4),
                                        ("nvfp4", 4), ("bf16", 8)])
def test_sharded_decode_matches_single_gpu_and_oracle(mode, world):
    """bf16: the Llama-1B-shape layers; nvfp4: Qwen3-style layers (head dim 128, q/k RMSNorm, 4 KV heads)
    with packed weights; nvfp4_split: an intermediate size whose per-rank K range (3072) has to run as
    2048 + 1024 with an exchange each; bf16_fault: after the normal steps the last rank skips one
    step, the others' wait for it times out with a status, the group re-agrees on the launch count
    (``Megakernel.resync_launch_count``) and the step after that matches again.  One process per GPU;
    skipped on a box with fewer GPUs than ranks."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_MODE=mode.split("_")[0])
    if mode == "nvfp4_split":
        env["TP_INTER"] = "6144"
    if mode == "bf16_fault":
        env.update(TP_FAULT="1", TP_TIMEOUT_MS="300")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "single-GPU" in r.stdout, tail
