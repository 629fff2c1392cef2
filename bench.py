#!/usr/bin/env python
"""Benchmark of the decode-step megakernel.

Workload at N = 1 (``config.workload``): the full 16-layer Llama-3.2-1B-shape
decode step as one persistent kernel — hidden 2048, 32 query / 8 KV heads,
head_dim 64, GLU intermediate 8192, tied 128256-vocab LM head with the greedy
token computed in the kernel, random-init bf16 weights ~N(0, 0.02), decode
batch 1, KV length 4096.  A "step" is one launch = one token per sequence.

One JSON line is printed by rank 0:

* ``value``   tokens/s with the inputs resident in HBM (CUDA events around K
              back-to-back launches, max over ranks);
* ``e2e``     the same metric through the public API with host buffers: per
              step the token embedding is copied from pinned host memory, the
              step runs, and the greedy token is read back;
* ``roofline`` algorithmic bytes per step (weights + LM head + KV, read once)
              divided by the measured kernel time, against the measured HBM
              copy bandwidth of this pool's B200s;
* ``cpu_baseline`` the CPU oracle (a port of the reference's PyTorch reference
              functions) timed on the host cores, as a reported baseline.

``--impl reference`` times that CPU port alone (the reference ships no
compiled code; its own path is PyTorch on the host).

Multi-GPU (``--gpus N`` under torchrun): every rank decodes its own sequence
with a full replica of the model (no data-path collective), so the aggregate
is N independent steps per step time ("weak" scaling).
"""

from __future__ import annotations

import argparse
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
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
    ap.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                    help="N > 1: tensor-parallel decode of ONE stream (in-kernel all-reduce) or N independent replicas")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    model = MODELS[args.model]
    args.kv_len = args.kv_len or model["kv_len"]
    args.layers = args.layers or model["layers"]
    args.vocab = args.vocab or model["vocab"]
    args.weights = args.weights or ("nvfp4" if model["qk_norm"] else "bf16")
    if model["qk_norm"] and args.weights != "nvfp4":
        ap.error("the q/k-norm layer is scheduled with NVFP4 weights only")
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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


def cpu_step_seconds(args, cfg, weights_cpu, budget_s=25.0):
    """Time the CPU oracle on the same workload; bounded: whole step if it fits, else a layer sample."""
    import oracle

    torch.set_num_threads(os.cpu_count() or 1)
    B, L = args.batch, args.kv_len
    g = torch.Generator().manual_seed(1)
    bf = torch.bfloat16
    kc = (torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g)).to(bf)
    vc = (torch.randn(B, L, cfg["nkv"], cfg["hd"], generator=g)).to(bf)
    x = torch.randn(B, 1, cfg["hidden"], generator=g).to(bf)
    r = torch.zeros(B, 1, cfg["hidden"], dtype=bf)

    def layer(l):
        return oracle.decode_layer(weights=weights_cpu, layer_idx=l, x_in=x, residual_in=r, k_cache=kc, v_cache=vc,
                                   cache_pos=L - 1, num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"], head_dim=cfg["hd"])

    def head():
        return oracle.top1(oracle.final_rms_lm_head(x, weights_cpu["final_norm"], weights_cpu["lm_head"], 1e-5, r))

    layer(0)  # warm-up
    t0 = time.perf_counter()
    layer(0)
    t_layer = time.perf_counter() - t0
    t0 = time.perf_counter()
    head()
    t_head = time.perf_counter() - t0
    n_layers = args.layers
    est = t_layer * n_layers + t_head
    if est <= budget_s:
        reps = max(1, min(5, int(budget_s // max(est, 1e-3))))
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            for l in range(n_layers):
                layer(l)
            head()
            times.append(time.perf_counter() - t0)
        return statistics.median(times), f"{reps} full steps ({n_layers} layers + LM head), median"
    return est, f"1 layer + LM head timed once, extrapolated to {n_layers} layers"


def run_reference(args, rank, world):
    """The reference's own path for this step is PyTorch on the host: time the CPU port."""
    if rank != 0:
        return
    cfg = MODELS[args.model]
    weights = make_weights(cfg, args.layers, args.vocab, args.kv_len, "cpu", seed=0)
    # each "step" is one bounded CPU pass; W + K passes are capped to keep the run within minutes
    budget = 240.0 / max(1, args.steps + args.warmup)
    secs, sample = cpu_step_seconds(args, cfg, weights, budget_s=max(5.0, budget))
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
        par = f"{world} independent replicas (one sequence set per GPU)" + (f"; {note}" if note else "")
    return {
        "workload": f"{MODELS[args.model]['name']} {args.layers}-layer decode step, batch {args.batch}, "
                    f"kv {args.kv_len}, vocab {args.vocab}, {args.weights}, greedy token",
        "global_batch": args.batch * (1 if tp else world), "kv_len": args.kv_len, "parallelism": par,
        "l2": "inputs (GBs of weights and KV per step, divided by the ranks under tp) larger than L2; no flush needed",
    }


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

    from machete_b200.kernels.llama1b import schedule_decode_model_sm100
    from machete_b200.megakernel import BackwardScheduler, Megakernel, MegakernelConfig, OverlapTileScheduler

    cfg = dict(MODELS[args.model])
    B, L, bf = args.batch, args.kv_len, torch.bfloat16
    # N > 1: one decode stream sharded Megatron-style over the ranks, unless the peer mapping
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
    if nvfp4:
        from machete_b200.kernels.decode_matvec.nvfp4_model import schedule_decode_model_nvfp4_sm100
        from machete_b200.quantization import quantize_nvfp4_weight

        packed = {k: v for k, v in weights.items() if not (".W_" in k or k == "lm_head")}
        for k in [k for k in weights if ".W_" in k or k == "lm_head"]:
            q4 = quantize_nvfp4_weight(weights.pop(k), group_size=16)
            packed[f"{k}.packed"], packed[f"{k}.scales"], packed[f"{k}.global_scale"] = q4.packed, q4.scales, float(q4.global_scale)
        weights = packed
        torch.cuda.empty_cache()
    ops, keep = (schedule_decode_model_nvfp4_sm100(
        batch=B, cache_pos=L - 1, weights=weights, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
        q_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
        attn_out_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
        mlp_h_buf=torch.zeros(B, 1, cfg["inter"], dtype=bf, device=dev), top_values=tv, top_indices=ti,
        num_layers=args.layers, x_in=x_in, residual_in=r_in, num_q_heads=cfg["nq"], num_kv_heads=cfg["nkv"],
        head_dim=cfg["hd"], eps=cfg["eps"], tp_peers=peers) if nvfp4 else None) or schedule_decode_model_sm100(
        batch=B, cache_pos=L - 1, weights=weights, k_cache=kcs, v_cache=vcs, x_buffers=xb, residual_buffers=rb,
        q_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
        attn_out_buf=torch.zeros(B, 1, cfg["nq"] * cfg["hd"], dtype=bf, device=dev),
        mlp_h_buf=torch.zeros(B, 1, cfg["inter"], dtype=bf, device=dev), final_norm=weights["final_norm"],
        lm_head=weights["lm_head"], top_values=tv, top_indices=ti, num_layers=args.layers, x_in=x_in,
        residual_in=r_in, hidden_size=cfg["hidden"], intermediate_size=cfg["inter"], num_q_heads=cfg["nq"],
        num_kv_heads=cfg["nkv"], head_dim=cfg["hd"], eps=cfg["eps"], tp_peers=peers)
    sched = OverlapTileScheduler() if args.scheduler == "overlap" else BackwardScheduler()
    mk = Megakernel(ops, config=MegakernelConfig(native_kc=args.kc or None), device=dev, scheduler=sched)
    mk.compile()

    def barrier():
        torch.cuda.synchronize(dev)
        if use_dist:
            dist.barrier()
            torch.cuda.synchronize(dev)

    stream = torch.cuda.current_stream(dev)
    for _ in range(max(3, args.warmup)):
        mk.run(sync=False, validate=False)
    mk.wait()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_first()
    barrier()
    first_row = sampler.mark()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(args.steps):
        mk.run(sync=False, validate=False)
    stop.record(stream)
    barrier()
    mk.wait()
    last_row = sampler.mark()
    ms_total = start.elapsed_time(stop)
    clocks = sampler.stop(first_row, max(last_row, first_row + 1)) if rank == 0 else None
    t = torch.tensor([ms_total], device=dev)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps

    # end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        host_x = torch.randn(B, 1, cfg["hidden"]).to(bf).pin_memory()
        host_tok = torch.zeros(B, 1, dtype=torch.int32).pin_memory()
        n_e2e = max(10, min(args.steps, 100))
        for _ in range(3):
            x_in.copy_(host_x, non_blocking=True)
            mk.run(sync=False, validate=False)
            host_tok.copy_(ti, non_blocking=True)
            torch.cuda.synchronize(dev)
        # the copy in, the step and the copy out as ONE CUDA graph launch per step (single GPU; under
        # tensor parallelism the plain calls are used): three driver calls become one
        graph = None
        if not use_dist:
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

    if rank == 0:
        peak, peak_kind = measured_peak()
        alg = algorithmic_bytes(cfg, B, L, args.layers, vocab, 0.5625 if nvfp4 else 2.0)   # per GPU (this rank's shard under tp)
        achieved = alg / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "decode_tokens_per_s", "value": B * (1 if tp else world) / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "us_per_step": ms_step * 1e3, "higher_is_better": True, "scaling": "strong" if tp else "weak",
            "vs_baseline": None, "dtype": "bf16" if not nvfp4 else "nvfp4 weights, f16 tensor-core math, fp32 accumulate",
            "data": "synthetic", "config": workload_config(args, world, tp, tp_note),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBps": achieved / NOMINAL_HBM_GBS,
                         "algorithmic_bytes_per_step": alg, "kernel": "mk_persistent_kernel",
                         "traffic": int(alg * NCU_TRAFFIC_RATIO)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps,
            "kernel_config": {"ctas": mk.grid[0], "threads": mk.block[0], "smem": mk.smem_size, "pages": mk.num_pages,
                              "page_bytes": mk.page_bytes, "instructions": mk.total_tiles,
                              "counters": mk.num_barriers, "scheduler": args.scheduler},
        }
        if not args.no_cpu_baseline and world == 1 and not nvfp4:
            wcpu = {k: v.cpu() for k, v in weights.items()}
            secs, sample = cpu_step_seconds(args, cfg, wcpu)
            line["cpu_baseline"] = {"value": B / secs, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": sample, "ms_per_step": secs * 1e3}
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
