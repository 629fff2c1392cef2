#!/usr/bin/env python
"""Benchmark of the decode-step megakernel.

Headline workload (``config.workload``): the full 16-layer Llama-3.2-1B-shape
decode step as one persistent kernel — hidden 2048, 32 query / 8 KV heads,
head_dim 64, GLU intermediate 8192, tied 128256-vocab LM head with the greedy
token computed in the kernel, random-init bf16 weights ~N(0, 0.02), decode
batch 1, KV length 4096.  A "step" is one launch = one token per sequence.

One JSON line is printed by rank 0:

* ``value``   tokens/s with the inputs resident in HBM: CUDA events around
              blocks of exactly ``--steps`` back-to-back launches, max over
              ranks; blocks are repeated until half a second has been timed and
              the MEDIAN block is reported (``blocks`` says how many ran), so
              the clock sampler always has rows inside the timed region;
* ``e2e``     the same metric through the public API with host buffers: per
              step the token embedding is copied from pinned host memory, the
              step runs, and the greedy token is read back.  For the bf16
              single-GPU-per-sequence workload the steps decode CONSECUTIVE
              positions from one handle (the cache position lives on the device
              and the kernel advances it), ending at the workload's KV length;
* ``roofline`` algorithmic bytes per step (weights + LM head + KV, read once)
              divided by the measured kernel time, against the measured HBM
              copy bandwidth of this pool's B200s;
* ``cpu_baseline`` / ``parity`` the CPU oracle (a port of the reference's
              PyTorch reference functions) on the host cores, on the SAME
              weights, KV cache and input as the GPU step: its time, and
              whether both produced the same greedy token;
* ``cfg4``    the tensor-parallel configuration at this N: 36-layer
              Qwen3-8B-shape step with block-scaled NVFP4 weights, batch 1 and
              8 (µs/step, tokens/s, per-GPU algorithmic bytes, fraction);
* ``cfg0`` / ``cfg1`` / ``cfg2`` (N = 1): one layer at KV 1024, the small-M
              GEMM sweep in bf16 and NVFP4, flash decoding at batch 8 x 32 768;
* ``gemm_sm100`` / ``prefill_attention`` (N = 1): the tcgen05 GEMM tile at
              64 / 128 / 256 rows and the tcgen05 prefill attention, with the
              library kernels (cuBLAS, torch SDPA) timed beside them.

``--impl reference`` times the CPU port alone (the reference ships no
compiled code; its own path for this step is PyTorch on the host).

Multi-GPU (``--gpus N`` under torchrun).  The headline model fits one GPU and
its decode streams are independent, so N ranks decode N sequences with a full
replica each and no data-path collective (``scaling: weak``).  The model the
task shards is the 8B-shape one: ``cfg4`` runs it Megatron tensor-parallel
over the N ranks with the all-reduce inside the kernel (``--model qwen3-8b``
makes it the headline, ``--parallel tp`` shards the Llama shape too).
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA1B = dict(name="llama-3.2-1b-shape", hidden=2048, inter=8192, nq=32, nkv=8, hd=64, vocab=128256, layers=16,
               theta=500000.0, kv_len=4096, eps=1e-5, qk_norm=False)
# Qwen3-8B shape: per-head q/k RMSNorm, NVFP4 weights, KV length 8192 (run with --model qwen3-8b)
QWEN3_8B = dict(name="qwen3-8b-shape", hidden=4096, inter=12288, nq=32, nkv=8, hd=128, vocab=151936, layers=36,
                theta=1000000.0, kv_len=8192, eps=1e-6, qk_norm=True)
MODELS = {"llama1b": LLAMA1B, "qwen3-8b": QWEN3_8B}
FALLBACK_HBM_GBS = 6650.0
# dram read + write bytes per algorithmic byte, from one ncu capture of a 4-layer + LM-head case
# of the same kernel (profiles/mk_persistent_kernel_llama1b_decode.md); DRAM traffic is
# proportional to the layers streamed, so the ratio carries over to the full workload.
NCU_TRAFFIC_RATIO = 1.006
NOMINAL_HBM_GBS = 8000.0
MIN_TIMED_SECONDS = 0.5
L2_BYTES = 126 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="llama1b", choices=sorted(MODELS),
                    help="llama1b: the headline workload (bf16); qwen3-8b: 36 layers with q/k RMSNorm, NVFP4 weights")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--kv-len", type=int, default=0, help="0 = the model's default (4096 / 8192)")
    ap.add_argument("--layers", type=int, default=0, help="0 = the model's layer count")
    ap.add_argument("--vocab", type=int, default=0, help="0 = the model's vocabulary")
    ap.add_argument("--kc", type=int, default=0, help="K columns per weight page (0 = default)")
    ap.add_argument("--scheduler", default="overlap", choices=["overlap", "roundrobin"])
    ap.add_argument("--weights", default="", choices=["", "bf16", "nvfp4"],
                    help="nvfp4: packed e2m1 weights, e4m3 scale per 16 values + fp32 global scale (the default and "
                         "only choice for qwen3-8b); the headline workload is llama1b in bf16")
    ap.add_argument("--parallel", default="", choices=["", "tp", "replicas"],
                    help="N > 1: tensor-parallel decode of ONE stream (in-kernel all-reduce) or N independent "
                         "replicas; default: replicas for llama1b (it fits one GPU), tp for qwen3-8b")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--stage-trace", action="store_true",
                    help="trace one launch of the workload on the device and print the per-op table (analysis only)")
    ap.add_argument("--only", default="", choices=["", "cfg0", "cfg1", "cfg2", "gemm_sm100", "prefill_attention"],
                    help="run one single-GPU sub-record alone and print it (for profiling that kernel)")
    ap.add_argument("--no-sub", action="store_true", help="skip the cfg0 / cfg1 / cfg2 / cfg4 sub-records")
    ap.add_argument("--sub-steps", type=int, default=30, help="launches per timed block of a sub-record")
    args = ap.parse_args()
    fill_defaults(args)
    if MODELS[args.model]["qk_norm"] and args.weights != "nvfp4":
        ap.error("the q/k-norm layer is scheduled with NVFP4 weights only")
    return args


def fill_defaults(args):
    model = MODELS[args.model]
    args.kv_len = args.kv_len or model["kv_len"]
    args.layers = args.layers or model["layers"]
    args.vocab = args.vocab or model["vocab"]
    args.weights = args.weights or ("nvfp4" if model["qk_norm"] else "bf16")
    args.parallel = args.parallel or ("tp" if model["qk_norm"] else "replicas")
    return args


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(cfg, batch, kv_len, layers, vocab, bytes_per_weight=2.0):
    """Weights + LM head + KV read once per step (the byte accounting of the roofline).

    ``bytes_per_weight``: 2 for bf16, 0.5625 for NVFP4 (4-bit code + one scale byte per 16 values).
    """
    h, i, q, kv = cfg["hidden"], cfg["inter"], cfg["nq"] * cfg["hd"], cfg["nkv"] * cfg["hd"]
    per_layer = (q * h + 2 * kv * h + h * q + 2 * i * h + h * i) * bytes_per_weight
    kv_bytes = kv_len * kv * 2 * 2
    return int(layers * per_layer + vocab * h * bytes_per_weight + batch * layers * kv_bytes)


def make_weights(cfg, layers, vocab, kv_len, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    h, i, q, kv, d2 = cfg["hidden"], cfg["inter"], cfg["nq"] * cfg["hd"], cfg["nkv"] * cfg["hd"], cfg["hd"] // 2

    def w(*shape):
        return (torch.randn(*shape, generator=g, device=device) * 0.02).to(bf)

    def nw(n):
        return (1.0 + torch.randn(n, generator=g, device=device) * 0.02).to(bf)

    inv = 1.0 / (cfg["theta"] ** (torch.arange(0, d2, dtype=torch.float32, device=device) / d2))
    ang = torch.arange(kv_len, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    weights = {"cos": torch.cos(ang).to(bf), "sin": torch.sin(ang).to(bf)}
    for l in range(layers):
        p = f"layer.{l}"
        weights[f"{p}.attn_norm"], weights[f"{p}.mlp_norm"] = nw(h), nw(h)
        weights[f"{p}.W_q"], weights[f"{p}.W_k"], weights[f"{p}.W_v"] = w(q, h), w(kv, h), w(kv, h)
        weights[f"{p}.W_o"] = w(h, q)
        weights[f"{p}.W_gate"], weights[f"{p}.W_up"] = w(i, h), w(i, h)
        weights[f"{p}.W_down"] = w(h, i)
        if cfg.get("qk_norm"):
            weights[f"{p}.q_norm"], weights[f"{p}.k_norm"] = nw(cfg["hd"]), nw(cfg["hd"])
    weights["final_norm"] = nw(h)
    if vocab:
        weights["lm_head"] = w(vocab, h)          # stands for the tied embedding matrix
    return weights


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def wait_first(self, timeout_s=5.0):
        """Block until nvidia-smi has produced its first row (it takes a while to start)."""
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < timeout_s:
            time.sleep(0.01)

    def mark(self):
        """Index of the next row: brackets the rows that fall inside the timed region."""
        return len(self.rows)

    def stop(self, first=0, last=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[first:last]:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except Exception:  # noqa: BLE001
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- the CPU leg --------------------------------------------------------------------------------------------
def cpu_step(args, cfg, weights_cpu, kcs, vcs, x, r, budget_s=25.0):
    """The CPU oracle on the given weights, caches and input; bounded: whole steps if they fit the
    budget, else one layer + LM head extrapolated.  Returns (seconds per step, what was sampled,
    (logits, token) of a whole step or None)."""
    import oracle

    torch.set_num_threads(os.cpu_count() or 1)
    L = args.kv_len
    kw = dict(num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"], head_dim=cfg["hd"])

    def layer(l, xx, rr, kc, vc):
        return oracle.decode_layer(weights=weights_cpu, layer_idx=l, x_in=xx, residual_in=rr, k_cache=kc, v_cache=vc,
                                   cache_pos=L - 1, eps=cfg["eps"], **kw)

    def head(xx, rr):
        return oracle.final_rms_lm_head(xx, weights_cpu["final_norm"], weights_cpu["lm_head"], cfg["eps"], rr)

    def whole():
        xx, rr = x, r
        for l in range(args.layers):
            xx, rr = layer(l, xx, rr, kcs[l].clone(), vcs[l].clone())
        return head(xx, rr)

    layer(0, x, r, kcs[0].clone(), vcs[0].clone())  # warm-up
    t0 = time.perf_counter()
    layer(0, x, r, kcs[0].clone(), vcs[0].clone())
    t_layer = time.perf_counter() - t0
    t0 = time.perf_counter()
    head(x, r)
    t_head = time.perf_counter() - t0
    est = t_layer * args.layers + t_head
    if est <= budget_s:
        reps = max(1, min(5, int(budget_s // max(est, 1e-3))))
        times, logits = [], None
        for _ in range(reps):
            t0 = time.perf_counter()
            logits = whole()
            times.append(time.perf_counter() - t0)
        v, i = oracle.top1(logits)
        return statistics.median(times), f"{reps} full steps ({args.layers} layers + LM head), median", (logits, i)
    return est, f"1 layer + LM head timed once, extrapolated to {args.layers} layers", None


def run_reference(args, rank, world):
    """The reference's own path for this step is PyTorch on the host: time the CPU port."""
    if rank != 0:
        return
    cfg = MODELS[args.model]
    weights = make_weights(cfg, args.layers, args.vocab, args.kv_len, "cpu", seed=0)
    g = torch.Generator().manual_seed(100)
    bf = torch.bfloat16
    B, L = args.batch, args.kv_len
    kcs = [torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g).to(bf) for _ in range(args.layers)]
    vcs = [torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g).to(bf) for _ in range(args.layers)]
    x = torch.randn(B, 1, cfg["hidden"], generator=g).to(bf)
    r = torch.zeros(B, 1, cfg["hidden"], dtype=bf)
    # each "step" is one bounded CPU pass; W + K passes are capped to keep the run within minutes
    budget = 240.0 / max(1, args.steps + args.warmup)
    secs, sample, _ = cpu_step(args, cfg, weights, kcs, vcs, x, r, budget_s=max(5.0, budget))
    tok_s = args.batch / secs
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world, tp=False, note=None):
    if world == 1:
        par = "single gpu"
    elif tp:
        par = f"tp{world}: Megatron tensor parallel, all-reduce after O-proj and down-proj inside the kernel"
    else:
        par = f"{world} independent replicas (one sequence set per GPU, no collective)" + (f"; {note}" if note else "")
    return {
        "workload": f"{MODELS[args.model]['name']} {args.layers}-layer decode step, batch {args.batch}, "
                    f"kv {args.kv_len}, vocab {args.vocab}, {args.weights}, greedy token",
        "global_batch": args.batch * (1 if tp else world), "kv_len": args.kv_len, "parallelism": par,
        "l2": "inputs (GBs of weights and KV per step, divided by the ranks under tp) larger than L2; no flush needed",
    }


# ---- building and timing one decode workload ----------------------------------------------------------------
class Workload:
    pass


def build_workload(args, dev, rank, world, use_dist, gen=False):
    """Weights, caches and the scheduled program of one decode workload on this rank."""
    from machete_b200.kernels.llama1b import schedule_decode_model_sm100
    from machete_b200.megakernel import BackwardScheduler, Megakernel, MegakernelConfig, OverlapTileScheduler

    if use_dist:
        import torch.distributed as dist
    w = Workload()
    cfg = dict(MODELS[args.model])
    B, L, bf = args.batch, args.kv_len, torch.bfloat16
    # tensor parallel: one decode stream sharded Megatron-style over the ranks, unless the peer mapping
    # cannot be set up on this box (then N independent replicas, and the line says so)
    peers, tp_note, vocab = None, None, args.vocab
    if use_dist and args.parallel == "tp":
        ok = 1
        try:
            if cfg["nq"] % world or cfg["nkv"] % world or cfg["inter"] % world or args.vocab % (16 * world):
                raise ValueError(f"heads / intermediate / vocabulary do not divide by {world}")
            from machete_b200.megakernel.peer import PeerBuffers

            # one exchange after the O projection, one per K-block of the down projection (a packed
            # local K above 2048 that is not a multiple of 2048 runs as 2048-blocks)
            k_loc = cfg["inter"] // world
            blocks = -(-k_loc // 2048) if (args.weights == "nvfp4" and k_loc > 2048 and k_loc % 2048) else 1
            peers = PeerBuffers(PeerBuffers.bytes_for_model(B, cfg["hidden"], args.layers, 1 + blocks), device=dev)
        except Exception as exc:  # noqa: BLE001
            ok, tp_note = 0, f"tp unavailable: {type(exc).__name__}: {exc}"[:200]
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peers, tp_note = None, tp_note or "tp unavailable on another rank"
        else:
            cfg.update(nq=cfg["nq"] // world, nkv=cfg["nkv"] // world, inter=cfg["inter"] // world)
            vocab = args.vocab // world
    tp = peers is not None
    weights = make_weights(cfg, args.layers, vocab, L, dev, seed=rank)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    kcs = [torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g, device=dev).to(bf) for _ in range(args.layers)]
    vcs = [torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g, device=dev).to(bf) for _ in range(args.layers)]
    x_in = torch.randn(B, 1, cfg["hidden"], generator=g, device=dev).to(bf)     # the token embedding
    r_in = torch.zeros(B, 1, cfg["hidden"], dtype=bf, device=dev)
    xb = [torch.zeros(B, 1, cfg["hidden"], dtype=bf, device=dev) for _ in range(2)]
    rb = [torch.zeros(B, 1, cfg["hidden"], dtype=bf, device=dev) for _ in range(2)]
    tv = torch.zeros(B, 1, device=dev)
    ti = torch.zeros(B, 1, dtype=torch.int32, device=dev)
    nvfp4 = args.weights == "nvfp4"
    bufs = dict(q_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
                attn_out_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
                mlp_h_buf=torch.zeros(B, 1, cfg["inter"], dtype=bf, device=dev))
    if nvfp4:
        from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
        from machete_b200.quantization import quantize_nvfp4_weight

        packed = {k: v for k, v in weights.items() if not (".W_" in k or k == "lm_head")}
        for k in [k for k in weights if ".W_" in k or k == "lm_head"]:
            q4 = quantize_nvfp4_weight(weights.pop(k), group_size=16)
            packed[f"{k}.packed"], packed[f"{k}.scales"], packed[f"{k}.global_scale"] = q4.packed, q4.scales, float(q4.global_scale)
        weights = packed
        torch.cuda.empty_cache()
        ops, keep = schedule_decode_model_nvfp4_sm100(
            batch=B, cache_pos=L - 1, weights=weights, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
            top_values=tv, top_indices=ti, num_layers=args.layers, x_in=x_in, residual_in=r_in,
            num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"], head_dim=cfg["hd"], eps=cfg["eps"], tp_peers=peers, **bufs)
    else:
        ops, keep = schedule_decode_model_sm100(
            batch=B, cache_pos=L - 1, weights=weights, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
            final_norm=weights["final_norm"], lm_head=weights["lm_head"], top_values=tv, top_indices=ti,
            num_layers=args.layers, x_in=x_in, residual_in=r_in, hidden_size=cfg["hidden"],
            intermediate_size=cfg["inter"], num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"], head_dim=cfg["hd"],
            eps=cfg["eps"], tp_peers=peers, **bufs)
    sched = OverlapTileScheduler() if args.scheduler == "overlap" else BackwardScheduler()
    mk = Megakernel(ops, config=MegakernelConfig(native_kc=args.kc or None), device=dev, scheduler=sched)
    mk.compile()
    w.mk_gen = w.position = None
    if gen and not tp and not nvfp4:
        # the same step scheduled once for ANY position: the end-to-end leg decodes consecutive tokens with it
        w.position = torch.zeros(1, dtype=torch.int32, device=dev)
        ops_g, keep_g = schedule_decode_model_sm100(
            batch=B, cache_pos=0, weights=weights, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
            final_norm=weights["final_norm"], lm_head=weights["lm_head"], top_values=tv, top_indices=ti,
            num_layers=args.layers, x_in=x_in, residual_in=r_in, hidden_size=cfg["hidden"],
            intermediate_size=cfg["inter"], num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"], head_dim=cfg["hd"],
            eps=cfg["eps"], position=w.position, **bufs)
        w.mk_gen = Megakernel(ops_g, config=MegakernelConfig(native_kc=args.kc or None, position=w.position),
                              device=dev, scheduler=OverlapTileScheduler() if args.scheduler == "overlap" else BackwardScheduler())
        w.mk_gen.compile()
        w.keep_gen = keep_g
    w.mk, w.cfg, w.tp, w.tp_note, w.vocab, w.nvfp4 = mk, cfg, tp, tp_note, vocab, nvfp4
    w.weights, w.kcs, w.vcs, w.x_in, w.r_in, w.ti, w.tv, w.keep = weights, kcs, vcs, x_in, r_in, ti, tv, (keep, xb, rb, bufs, peers)
    w.alg_bytes = algorithmic_bytes(cfg, B, L, args.layers, vocab, 0.5625 if nvfp4 else 2.0)   # per GPU
    return w


def time_launches(launch, steps, warmup, dev, use_dist, sampler=None, min_seconds=MIN_TIMED_SECONDS, max_blocks=200):
    """Blocks of exactly ``steps`` launches between CUDA events on the launching stream, repeated
    until ``min_seconds`` have been timed; returns (median ms per step over the blocks — each block
    the max over ranks —, number of blocks, clock-sample row range)."""
    if use_dist:
        import torch.distributed as dist

    def barrier():
        torch.cuda.synchronize(dev)
        if use_dist:
            dist.barrier()
            torch.cuda.synchronize(dev)

    stream = torch.cuda.current_stream(dev)
    for _ in range(max(3, warmup)):
        launch()
    barrier()
    first_row = sampler.mark() if sampler else 0
    per_step, total = [], 0.0
    while True:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record(stream)
        for _ in range(steps):
            launch()
        stop.record(stream)
        barrier()
        t = torch.tensor([start.elapsed_time(stop)], device=dev)
        if use_dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        per_step.append(ms / steps)
        total += ms * 1e-3
        if total >= min_seconds or len(per_step) >= max_blocks:
            break
    last_row = sampler.mark() if sampler else 0
    return statistics.median(per_step), len(per_step), (first_row, max(last_row, first_row + 1))


def time_workload(w, steps, warmup, dev, use_dist, sampler=None):
    ms, blocks, rows = time_launches(lambda: w.mk.run(sync=False, validate=False), steps, warmup, dev, use_dist, sampler)
    w.mk.wait()
    return ms, blocks, rows


# ---- sub-records ----------------------------------------------------------------------------------------------
def sub_args(args, **over):
    a = argparse.Namespace(**vars(args))
    a.kv_len = a.layers = a.vocab = 0
    a.weights = a.parallel = ""
    for k, v in over.items():
        setattr(a, k, v)
    return fill_defaults(a)


def record_cfg4(args, dev, rank, world, use_dist, peak):
    """The tensor-parallel configuration at this N: Qwen3-8B shape, block-scaled NVFP4, batch 1, 8 and (one GPU) 32."""
    out = {"workload": "qwen3-8b-shape 36-layer decode step, kv 8192, vocab 151936, nvfp4 (e4m3 scale per 16 "
                       "values + fp32 global scale), greedy token", "n_gpus": world,
           "parallelism": "single gpu" if world == 1 else f"tp{world} (in-kernel all-reduce)", "batches": {}}
    # batch 32 does not fit the activation staging as one op: on one GPU it runs as interleaved chunks of 8
    # rows (kernels/_batching.py); the chunked schedule is not combined with tensor parallelism
    for batch in ((1, 8, 32) if world == 1 else (1, 8)):
        a = sub_args(args, model="qwen3-8b", batch=batch, parallel="tp")
        try:
            w = build_workload(a, dev, rank, world, use_dist)
            ms, blocks, _ = time_workload(w, args.sub_steps, 5, dev, use_dist)
            tp = w.tp or world == 1
            achieved = w.alg_bytes / (ms * 1e-3) / 1e9
            out["batches"][str(batch)] = {
                "us_per_step": ms * 1e3, "tokens_per_s": batch * (1 if tp else world) / (ms * 1e-3),
                "algorithmic_bytes_per_gpu": w.alg_bytes, "achieved_gbs_per_gpu": achieved, "frac": achieved / peak,
                "steps": args.sub_steps, "blocks": blocks, "tensor_parallel": bool(w.tp), "note": w.tp_note}
            del w
        except Exception as exc:  # noqa: BLE001
            out["batches"][str(batch)] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        gc.collect()
        torch.cuda.empty_cache()
    return out


def time_graph(fn, iters, dev, replays=5):
    """``fn(i)`` for i in range(iters) captured into ONE CUDA graph (a single-op launch runs for a few
    microseconds, less than the host side of the call takes), replayed ``replays`` times between CUDA
    events: microseconds per launch."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize(dev)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(iters):
            fn(i)
    torch.cuda.synchronize(dev)
    graph.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / (replays * iters) * 1e3


def rotating(make, nbytes, floor=3):
    """Enough independent copies of a small workload that consecutive launches miss in L2."""
    return [make(i) for i in range(max(floor, -(-2 * L2_BYTES // max(1, nbytes)) + 1))]


def record_cfg1(args, dev, peak):
    """Small-M GEMM sweep, bf16 and block-scaled NVFP4: weights are smaller than L2, so launches
    rotate over copies of the weight matrix (together more than twice L2)."""
    from machete_b200.kernels.decode_matvec import MatvecNvfp4Sm120Op
    from machete_b200.kernels.gemm import GemmOp
    from machete_b200.megakernel import Megakernel
    from machete_b200.quantization import quantize_nvfp4_weight

    bf = torch.bfloat16
    shapes = [(M, N_, 4096) for M in (1, 4, 16) for N_ in (4096, 14336)] + [(16, 1024, 1024)]
    out = {"l2": "launches rotate over weight copies totalling more than twice L2; one CUDA graph of all launches",
           "bf16": {}, "nvfp4": {}}
    for fmt in ("bf16", "nvfp4"):
        for (M, Nout, K) in shapes:
            g = torch.Generator(device=dev).manual_seed(7)
            x = torch.randn(1, M, K, generator=g, device=dev).to(bf)
            y = torch.zeros(1, M, Nout, dtype=bf, device=dev)
            wbytes = Nout * K * (2 if fmt == "bf16" else 0.5625)

            def make(i, fmt=fmt, Nout=Nout, K=K, x=x, y=y, g=g):
                wt = (torch.randn(Nout, K, generator=g, device=dev) * 0.02).to(bf)
                if fmt == "bf16":
                    return Megakernel(GemmOp.schedule(a=x, b=wt, c=y)).compile()
                q = quantize_nvfp4_weight(wt, group_size=16)
                return Megakernel(MatvecNvfp4Sm120Op.schedule(a=x, weight_packed=q.packed, weight_scales=q.scales, y=y,
                                                              group_size=16, global_scale=q.global_scale)).compile()

            mks = rotating(make, int(wbytes))
            # every replay walks all copies (more than twice L2) at least once
            iters = len(mks) * -(-40 // len(mks))
            us = time_graph(lambda i: mks[i % len(mks)].run(sync=False, validate=False), iters, dev)
            for m_ in mks:
                m_.wait()
            ms = us * 1e-3
            alg = wbytes + M * K * 2 + M * Nout * 2
            out[fmt][f"{M}x{K}x{Nout}"] = {"us": ms * 1e3, "algorithmic_bytes": int(alg),
                                           "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac": alg / (ms * 1e-3) / 1e9 / peak}
            del mks
            gc.collect()
            torch.cuda.empty_cache()
    return out


def record_gemm_sm100(args, dev, peak):
    """The tcgen05 GEMM tile at 64 / 128 / 256 activation rows.  Launches are captured in one CUDA graph
    (the host side of a call, two tensor-map encodes, costs more than these kernels run) and rotate
    over weight copies totalling more than twice L2; cuBLAS through torch.matmul is timed the same way."""
    from machete_b200.kernels.gemm import gemm_pack_weight, gemm_sm100

    bf = torch.bfloat16
    tflops_peak = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            tflops_peak = float(json.load(fh)["bf16_tflops"])
    except Exception:  # noqa: BLE001
        tflops_peak = 1590.0
    out = {"l2": "launches rotate over weight copies totalling more than twice L2; one CUDA graph of all launches",
           "tensor_peak_tflops": tflops_peak, "shapes": {}}
    iters = 40

    def timed(fn):
        return time_graph(fn, iters, dev)

    for (Nout, K) in ((4096, 4096), (14336, 4096), (4096, 14336)):
        g = torch.Generator(device=dev).manual_seed(9)
        ws = rotating(lambda i: (torch.randn(Nout, K, generator=g, device=dev) * 0.02).to(bf), Nout * K * 2)
        for M in (64, 128, 256):
            a = torch.randn(1, M, K, generator=g, device=dev).to(bf)
            c = torch.zeros(1, M, Nout, dtype=bf, device=dev)
            us = timed(lambda i: gemm_sm100(a, ws[i % len(ws)], c))
            us_lib = timed(lambda i: torch.matmul(a[0], ws[i % len(ws)].t(), out=c[0]))
            alg = (Nout * K + M * K + M * Nout) * 2
            flops = 2.0 * M * Nout * K
            out["shapes"][f"{M}x{K}x{Nout}"] = {
                "us": us, "tflops": flops / us / 1e6, "frac_tensor": flops / us / 1e6 / tflops_peak,
                "achieved_gbs": alg / us / 1e3, "frac_hbm": alg / us / 1e3 / peak, "cublas_us": us_lib}
        del ws
        gc.collect()
        torch.cuda.empty_cache()
    return out


def record_prefill_attention(args, dev, peak):
    """The tcgen05 prefill attention at the two model shapes (32 query / 8 KV heads, causal), with the library
    kernel behind torch's scaled_dot_product_attention timed beside it.  K and V (16-34 MB) stay in L2 by
    design: every query tile of a head re-reads them, so the bound is the tensor pipe, not HBM."""
    from machete_b200.kernels.attention import flash_prefill

    bf = torch.bfloat16
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            tflops_peak = float(json.load(fh)["bf16_tflops"])
    except Exception:  # noqa: BLE001
        tflops_peak = 1590.0
    out = {"tensor_peak_tflops": tflops_peak, "shapes": {}}

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / iters * 1e3

    for (H, Hkv, M, D) in ((32, 8, 4096, 64), (32, 8, 4096, 128), (32, 8, 1024, 128)):
        g = torch.Generator(device=dev).manual_seed(10)
        q = torch.randn(1, H, M, D, generator=g, device=dev).to(bf)
        k = torch.randn(1, Hkv, M, D, generator=g, device=dev).to(bf)
        v = torch.randn(1, Hkv, M, D, generator=g, device=dev).to(bf)
        o = torch.zeros_like(q)
        us = timed(lambda: flash_prefill(q, k, v, o, causal=True))
        us_lib = timed(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True))
        flops = 4.0 * H * M * M * D * 0.5
        out["shapes"][f"H{H}/{Hkv} M{M} D{D} causal"] = {"us": us, "tflops": flops / us / 1e6,
                                                        "frac_tensor": flops / us / 1e6 / tflops_peak, "sdpa_us": us_lib}
    return out


def record_cfg2(args, dev, peak):
    """Flash decoding alone: batch 8, 32 query / 8 KV heads, head dim 128, 32 768 tokens, 32 splits + combine."""
    from machete_b200.kernels.attention import flash_decoding_schedule
    from machete_b200.megakernel import Megakernel

    B, H, Hkv, D, Nkv, S = 8, 32, 8, 128, 32768, 32
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(8)
    q = torch.randn(B, 1, H, D, generator=g, device=dev).to(bf)
    k = torch.randn(B, Nkv, Hkv, D, generator=g, device=dev).to(bf)
    v = torch.randn(B, Nkv, Hkv, D, generator=g, device=dev).to(bf)
    o = torch.zeros_like(q)
    ops, _ = flash_decoding_schedule(q, k, v, o, num_splits=S, kv_group_size=H // Hkv)
    mk = Megakernel(ops).compile()
    ms, blocks, _ = time_launches(lambda: mk.run(sync=False, validate=False), args.sub_steps, 5, dev, False, min_seconds=0.1)
    alg = 2 * B * Nkv * Hkv * D * 2
    return {"workload": f"flash decoding B{B} H{H}/{Hkv} D{D} N{Nkv}, {S} splits + log-sum-exp combine (one fused op)",
            "us": ms * 1e3, "algorithmic_bytes": alg, "achieved_gbs": alg / (ms * 1e-3) / 1e9,
            "frac": alg / (ms * 1e-3) / 1e9 / peak, "l2": "1 GiB of K/V per launch, larger than L2"}


def record_cfg0(args, dev, peak):
    """One Llama-1B-shape layer, batch 1, KV 1024 (the case the reference can run on the CPU): the GPU
    time over rotating weight copies, and the CPU oracle's time for the same layer."""
    import oracle
    from machete_b200.kernels.decode_matvec import schedule_decode_layer_sm100
    from machete_b200.megakernel import Megakernel, OverlapTileScheduler

    cfg, bf, T = LLAMA1B, torch.bfloat16, 1024
    keepers = []

    def make(i):
        wts = make_weights(cfg, 1, 0, T, dev, seed=50 + i)
        g = torch.Generator(device=dev).manual_seed(60 + i)
        kc = torch.randn(1, T, cfg["nkv"], cfg["hd"], generator=g, device=dev).to(bf)
        vc = torch.randn(1, T, cfg["nkv"], cfg["hd"], generator=g, device=dev).to(bf)
        x = torch.randn(1, 1, cfg["hidden"], generator=g, device=dev).to(bf)
        r = torch.randn(1, 1, cfg["hidden"], generator=g, device=dev).to(bf)
        xo, ro = torch.zeros_like(x), torch.zeros_like(x)
        layer = schedule_decode_layer_sm100(
            layer_idx=0, batch=1, seq_len=1, cache_pos=T - 1, weights=wts, k_cache=kc, v_cache=vc, x_in=x, residual_in=r,
            x_out=xo, residual_out=ro, q_buf=torch.zeros(1, 1, 2048, dtype=bf, device=dev),
            attn_out_buf=torch.zeros(1, 1, 2048, dtype=bf, device=dev),
            mlp_h_buf=torch.zeros(1, 1, cfg["inter"], dtype=bf, device=dev), eps=cfg["eps"])
        keepers.append((wts, kc, vc, x, r, xo, ro, layer))
        return Megakernel(layer.ops, scheduler=OverlapTileScheduler()).compile()

    alg = algorithmic_bytes(cfg, 1, T, 1, 0)
    mks = rotating(make, alg)
    it = [0]

    def launch():
        mks[it[0] % len(mks)].run(sync=False, validate=False)
        it[0] += 1

    ms, blocks, _ = time_launches(launch, args.sub_steps, 5, dev, False, min_seconds=0.05)
    wts, kc, vc, x, r = [t if isinstance(t, dict) else t.cpu() for t in keepers[0][:5]]
    wcpu = {k_: v_.cpu() for k_, v_ in wts.items()}
    torch.set_num_threads(os.cpu_count() or 1)
    times = []
    for _ in range(4):
        t0 = time.perf_counter()
        oracle.decode_layer(weights=wcpu, layer_idx=0, x_in=x, residual_in=r, k_cache=kc.clone(), v_cache=vc.clone(),
                            cache_pos=T - 1, eps=cfg["eps"])
        times.append(time.perf_counter() - t0)
    return {"workload": "one llama-3.2-1b-shape layer, batch 1, kv 1024, bf16", "us": ms * 1e3, "algorithmic_bytes": alg,
            "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac": alg / (ms * 1e-3) / 1e9 / peak,
            "cpu_oracle_ms": statistics.median(times[1:]) * 1e3, "cpu_cores": os.cpu_count(),
            "l2": "launches rotate over layer copies totalling more than twice L2"}


def main():
    args = parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the native path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    if args.only:
        fn = {"cfg0": record_cfg0, "cfg1": record_cfg1, "cfg2": record_cfg2, "gemm_sm100": record_gemm_sm100,
              "prefill_attention": record_prefill_attention}[args.only]
        if rank == 0:
            print(json.dumps({"only": args.only, args.only: fn(args, dev, measured_peak()[0])}), flush=True)
        if use_dist:
            dist.barrier()
            dist.destroy_process_group()
        return
    w = build_workload(args, dev, rank, world, use_dist, gen=not args.no_e2e)
    mk, cfg, tp, B, bf = w.mk, w.cfg, w.tp, args.batch, torch.bfloat16

    if args.stage_trace:
        # per-op timeline of ONE traced launch (tracing costs a few stores per page: the untraced time is
        # printed beside it); rank 0 only
        for _ in range(5):
            mk.run()
        ms_plain, _, _ = time_launches(lambda: mk.run(sync=False, validate=False), 50, 5, dev, False, min_seconds=0.05)
        mk.enable_trace(4096)
        mk.run()
        rows = mk.stage_table()
        if rank == 0:
            print(json.dumps({"stage_trace": {"untraced_us_per_step": ms_plain * 1e3, "layers": args.layers,
                                              "vocab": args.vocab, "ops": rows}}), flush=True)
        if use_dist:
            dist.barrier()
            dist.destroy_process_group()
        return
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_first()
    ms_step, blocks, rows = time_workload(w, args.steps, args.warmup, dev, use_dist, sampler if rank == 0 else None)
    clocks = sampler.stop(*rows) if rank == 0 else None

    def barrier():
        torch.cuda.synchronize(dev)
        if use_dist:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        x_in, ti = w.x_in, w.ti
        host_x = x_in.cpu().pin_memory()           # the same embedding: the token must not change
        host_tok = torch.zeros(B, 1, dtype=torch.int32).pin_memory()
        n_e2e = max(10, min(args.steps, 100))
        # consecutive positions from one handle where the workload has the position on the device: the
        # 3 + 3 warm-up steps and the timed ones end exactly at the workload's KV length
        run_mk, first_pos = mk, None
        if w.mk_gen is not None and n_e2e + 6 < args.kv_len:
            run_mk, first_pos = w.mk_gen, args.kv_len - (n_e2e + 6)
            w.position.fill_(first_pos)
        mk_static, mk = mk, run_mk
        for _ in range(3):
            x_in.copy_(host_x, non_blocking=True)
            mk.run(sync=False, validate=False)
            host_tok.copy_(ti, non_blocking=True)
            torch.cuda.synchronize(dev)
        # the copy in, the step and the copy out as ONE CUDA graph launch per step (single process per
        # GPU without a peer exchange; under tensor parallelism the plain calls are used)
        graph = None
        if not tp:
            try:
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=side):
                    x_in.copy_(host_x, non_blocking=True)
                    mk.run(sync=False, validate=False)
                    host_tok.copy_(ti, non_blocking=True)
                torch.cuda.synchronize(dev)
                for _ in range(3):
                    g_.replay()
                    torch.cuda.synchronize(dev)
                mk.wait()                      # raises if a captured launch misbehaved
                graph = g_
            except Exception:  # noqa: BLE001
                graph = None
                torch.cuda.synchronize(dev)

        def one_step():
            if graph is not None:
                graph.replay()
            else:
                x_in.copy_(host_x, non_blocking=True)
                mk.run(sync=False, validate=False)
                host_tok.copy_(ti, non_blocking=True)
            torch.cuda.synchronize(dev)      # the token is needed on the host before the next step

        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            one_step()
        e2e_s = (time.perf_counter() - t0) / n_e2e
        te = torch.tensor([e2e_s], device=dev)
        if use_dist:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te.item())
        e2e = {"value": B * (1 if tp else world) / e2e_s, "unit": "tokens/s", "us_per_step": e2e_s * 1e6,
               "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_tok.numel() * 4, "steps": n_e2e,
               "launch": "one CUDA graph per step: copy in, Megakernel.run(), copy out" if graph is not None
               else "x_in.copy_(pinned), Megakernel.run(), token.copy_ to pinned"}
        mk.wait()
        if first_pos is not None:
            last = int(w.position.item())       # kv_len, or 3 short of it when the graph warm-up did not run
            e2e["positions"] = {"first_timed": last - n_e2e, "end": last, "kv_len": args.kv_len,
                                "how": "one handle, device-resident cache position advanced by the kernel"}
        else:
            e2e["positions"] = {"fixed": args.kv_len - 1, "how": "the static program of the timed region"}
        mk = mk_static
        x_in.copy_(host_x)                       # the fed-back row goes; the parity leg below uses the original input
        torch.cuda.synchronize(dev)

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = w.alg_bytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "decode_tokens_per_s", "value": B * (1 if tp else world) / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "blocks": blocks,
            "ms_per_step": ms_step, "us_per_step": ms_step * 1e3, "higher_is_better": True,
            "scaling": "strong" if tp else "weak", "vs_baseline": None,
            "dtype": "bf16" if not w.nvfp4 else "nvfp4 weights, f16 tensor-core math, fp32 accumulate",
            "data": "synthetic", "config": workload_config(args, world, tp, w.tp_note),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBps": achieved / NOMINAL_HBM_GBS,
                         "algorithmic_bytes_per_step": w.alg_bytes, "kernel": "mk_persistent_kernel",
                         "traffic": int(w.alg_bytes * NCU_TRAFFIC_RATIO),
                         "traffic_from": "ncu dram bytes of a 4-layer capture x layers (profiles/), not this run"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps * blocks,
            "kernel_config": {"ctas": mk.grid[0], "threads": mk.block[0], "smem": mk.smem_size, "pages": mk.num_pages,
                              "page_bytes": mk.page_bytes, "instructions": mk.total_tiles,
                              "counters": mk.num_barriers, "scheduler": args.scheduler},
        }
        if not args.no_cpu_baseline and world == 1 and not w.nvfp4:
            # the CPU oracle on the very same weights, caches and embedding
            mk.run()
            got_tok, got_val = int(w.ti[0, 0]), float(w.tv[0, 0])
            wcpu = {k: v.cpu() for k, v in w.weights.items()}
            secs, sample, full = cpu_step(args, cfg, wcpu, [t.cpu() for t in w.kcs], [t.cpu() for t in w.vcs],
                                          w.x_in.cpu(), w.r_in.cpu())
            line["cpu_baseline"] = {"value": B / secs, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": sample, "ms_per_step": secs * 1e3}
            if full is not None:
                logits, tok = full
                line["parity"] = {"token_equal": bool(int(tok[0, 0]) == got_tok), "gpu_token": got_tok,
                                  "cpu_token": int(tok[0, 0]),
                                  "logit_abs_err": abs(got_val - float(logits[0, 0, got_tok]))}
            del wcpu
    # sub-records: the other configurations (every rank takes part in cfg4, which is tensor parallel)
    if not args.no_sub:
        peak = measured_peak()[0]
        del w, mk
        gc.collect()
        torch.cuda.empty_cache()
        if args.model == "llama1b":
            cfg4 = record_cfg4(args, dev, rank, world, use_dist, peak)
            if rank == 0:
                line["cfg4"] = cfg4
        if world == 1 and rank == 0 and args.model == "llama1b":
            for name, fn in (("cfg0", record_cfg0), ("cfg1", record_cfg1), ("cfg2", record_cfg2),
                             ("gemm_sm100", record_gemm_sm100), ("prefill_attention", record_prefill_attention)):
                try:
                    line[name] = fn(args, dev, peak)
                except Exception as exc:  # noqa: BLE001
                    line[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                gc.collect()
                torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
