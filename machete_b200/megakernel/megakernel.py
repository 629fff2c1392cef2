"""``Megakernel``: turns scheduled ops into a native program and launches it.

Host runtime behind the reference's public entry point
(src/machete/megakernel/megakernel.py: ``MegakernelConfig`` :174-221,
``Megakernel.__init__`` :490, ``compile`` :1594, ``run`` :2183,
``bench_spec`` :2206, ``create_megakernel`` :2293).  The constructor lowers
every ``ScheduledOp`` through its op class, infers dependencies and builds the
tables; ``compile()`` uploads them through the C ABI (``mk_create``);
``run()`` is one kernel launch (``mk_run``) with no per-launch host work: the
kernel resets its own counters, so launches can be queued back to back or
captured in a CUDA graph.
"""

from __future__ import annotations

import ctypes as C
import warnings
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import _native as N
from .lowering import LowerCtx, NativeOp
from .paged_memory import NativeSmemPlan
from .ops import ScheduledOp
from .scheduling import BackwardScheduler, BuiltProgram, InstructionStreamBuilder, TileScheduler

MAX_PAGES = 32
NUM_DMA_WARPS = 1
NUM_CONSUMER_WARPS = N.NUM_CONSUMER_WARPS
CTRL_BYTES = 4096 + NUM_CONSUMER_WARPS * 2048   # control block + split-K partial slots (csrc/shell.cuh)

# Used when no CUDA device is present (table building and CPU tests): B200.
_DEFAULT_SMS = 148
_DEFAULT_SMEM_OPTIN = 232448


@dataclass
class MegakernelConfig:
    """Launch configuration.

    Field-compatible with the reference dataclass; fields that steer its JIT
    or warp-role split (``threads_per_block``, ``dma_reg_count``,
    ``mma_reg_count``, ``opt_level``, ``loader_idle_sleep_ns``,
    ``relaxed_global_barriers``, ``global_barrier_sleep_ns``) are accepted and
    ignored: the precompiled kernel always runs 1 loader + 7 consumer warps.
    ``page_size`` is likewise accepted for parity with ``schedule(page_size=)``;
    the native ring page is sized from the ops (``native_kc``).
    """

    threads_per_block: int = 256
    num_sms: Optional[int] = None
    page_size: int = 49152
    num_pages: Optional[int] = None
    tracing: bool = False
    dma_reg_count: int = 40
    mma_reg_count: int = 232
    loader_idle_sleep_ns: int = 100
    relaxed_global_barriers: bool = True
    global_barrier_sleep_ns: int = 8
    opt_level: int = 2
    peer_buffers: Optional[Dict[str, List[Any]]] = None
    peer_barriers: Optional[Any] = None
    device_idx: int = 0
    num_devices: int = 1
    # native extensions
    native_kc: Optional[int] = None      # K columns per bf16 weight page (default 1024: 32 KB pages)
    native_kc_fp4: Optional[int] = None  # K columns per NVFP4 weight page (default 2048)
    timeout_ms: int = 1000               # bound of every device-side wait
    fuse: bool = True                    # allow peephole fusion of op chains
    # Device-resident cache position: a one-element int32 CUDA tensor that ops scheduled with a
    # dynamic position read at the start of every launch and that the token-feedback form of the
    # top-1 head advances at the end (consecutive launches decode consecutive tokens).
    position: Optional[Any] = None
    # first position the caches do not hold (None: the smallest cache length of the position-following ops);
    # a launch that finds the position outside [0, position_limit) runs nothing and reports status 7
    position_limit: Optional[int] = None


_IGNORED_CONFIG = {
    "threads_per_block": 256, "dma_reg_count": 40, "mma_reg_count": 232, "loader_idle_sleep_ns": 100,
    "relaxed_global_barriers": True, "global_barrier_sleep_ns": 8, "opt_level": 2, "page_size": 49152,
}
_warned_config = False


def _warn_ignored_config(cfg: "MegakernelConfig") -> None:
    """One warning per process when a caller tunes a knob the precompiled kernel does not have."""
    global _warned_config
    changed = sorted(k for k, default in _IGNORED_CONFIG.items() if getattr(cfg, k) != default and k != "page_size")
    if changed and not _warned_config:
        _warned_config = True
        warnings.warn(
            f"MegakernelConfig fields {changed} steer the reference's JIT and warp-role split; the precompiled "
            "sm_100a kernel (1 loader + 7 consumer warps) accepts and ignores them", stacklevel=3)


def _device_index(device) -> int:
    if isinstance(device, int):
        return device
    dev = torch.device(device)
    if dev.type != "cuda":
        raise ValueError(f"Megakernel runs on CUDA devices only, got {device!r}")
    return dev.index if dev.index is not None else (torch.cuda.current_device() if torch.cuda.is_available() else 0)


class Megakernel:
    """A decode-step program for the persistent sm_100a kernel.

    Args:
        ops: list of ``ScheduledOp`` in program order.
        config: ``MegakernelConfig`` (optional).
        device: CUDA device of the tensors.
        scheduler: unit-placement policy (``BackwardScheduler`` by default).
    """

    def __init__(self, ops: Sequence[ScheduledOp], config: Optional[MegakernelConfig] = None,
                 device="cuda", scheduler: Optional[TileScheduler] = None):
        ops = list(ops)
        if not ops:
            raise ValueError("Megakernel needs at least one scheduled op")
        self.ops = ops
        self.config = config or MegakernelConfig()
        self.scheduler = scheduler or BackwardScheduler()
        self._device = device
        self._handle = C.c_void_p()
        self._workspace = None
        self._arrays = None

        cfg = self.config
        _warn_ignored_config(cfg)
        if cfg.num_sms is not None and cfg.num_sms < 1:
            raise ValueError("num_sms must be positive")
        sms, smem = _DEFAULT_SMS, _DEFAULT_SMEM_OPTIN
        if torch.cuda.is_available():
            info = N.device_info(_device_index(device))
            sms, smem = info["num_sms"], info["smem_optin"]
        self._smem_optin = smem
        self.num_sms = cfg.num_sms if cfg.num_sms is not None else sms

        kc = cfg.native_kc or 1024
        kc4 = cfg.native_kc_fp4 or 2048
        ctx = LowerCtx(num_sms=self.num_sms, page_bytes=0, smem_optin=smem, kc_bf16=kc, kc_fp4=kc4, fuse=cfg.fuse)
        # page size: the largest need of any op, rounded to 1 KB
        self._page_bytes = self._plan_page_bytes(ops, ctx)
        ctx.page_bytes = self._page_bytes

        from .fusion import lower_program

        self.native_ops: List[NativeOp] = lower_program(ops, ctx)
        builder = InstructionStreamBuilder(self.num_sms)
        for nop in self.native_ops:
            builder.add_op(nop)
        self.program: BuiltProgram = builder.build(self.scheduler)

        self._act_bytes = -(-self.program.act_bytes // 1024) * 1024
        plan = NativeSmemPlan(CTRL_BYTES, self._act_bytes, self._page_bytes, smem_optin=smem, max_pages=MAX_PAGES)
        n_pages = plan.num_pages
        if cfg.num_pages is not None:
            n_pages = min(n_pages, int(cfg.num_pages))
        if n_pages < 2:
            raise ValueError(
                f"shared memory too small: {self._act_bytes} B of staged activations leave room for "
                f"{n_pages} pages of {self._page_bytes} B (need >= 2); reduce batch x K"
            )
        self._n_pages = int(n_pages)

    # -- planning ---------------------------------------------------------------------------
    @staticmethod
    def _plan_page_bytes(ops, ctx: LowerCtx) -> int:
        need = 16384  # attention pages: 4 * D * block tokens
        from .lowering import bf16_page_need, fp4_page_need

        uses_fp4 = any(getattr(op.op_cls, "uses_nvfp4", False) for op in ops)
        uses_dense = any(getattr(op.op_cls, "uses_dense_weights", False) for op in ops)
        if uses_dense or not uses_fp4:
            need = max(need, bf16_page_need(ctx.kc_bf16))
        if uses_fp4:
            need = max(need, fp4_page_need(ctx.kc_fp4))
        return -(-need // 1024) * 1024

    # -- properties mirrored from the reference -------------------------------------------------
    @property
    def total_tiles(self) -> int:
        return int(self.program.cta_instr_begin[-1])

    @property
    def num_barriers(self) -> int:
        return int(self.program.n_counters)

    @property
    def smem_size(self) -> int:
        return CTRL_BYTES + self._act_bytes + self._n_pages * self._page_bytes

    @property
    def grid(self):
        return (self.program.num_ctas, 1, 1)

    @property
    def block(self):
        return ((NUM_CONSUMER_WARPS + NUM_DMA_WARPS) * 32, 1, 1)

    @property
    def num_pages(self) -> int:
        return self._n_pages

    @property
    def page_bytes(self) -> int:
        return self._page_bytes

    @property
    def algorithmic_bytes(self) -> int:
        """HBM bytes the program streams once per launch (weights, scales, KV)."""
        return self.program.total_bytes

    # -- compile / run ------------------------------------------------------------------------
    def compile(self) -> "Megakernel":
        """Upload the program tables to the device (idempotent)."""
        if self._handle:
            return self
        lib = N.lib()
        dev = _device_index(self._device)
        p = self.program
        arrays = {
            "ops": np.ascontiguousarray(p.ops), "instrs": np.ascontiguousarray(p.instrs),
            "ib": np.ascontiguousarray(p.cta_instr_begin), "events": np.ascontiguousarray(p.events),
            "eb": np.ascontiguousarray(p.cta_event_begin), "waits": np.ascontiguousarray(p.waits),
        }
        prog = N.Program()
        prog.n_ops = len(p.ops)
        prog.n_instrs = int(p.cta_instr_begin[-1])
        prog.n_events = int(p.cta_event_begin[-1])
        prog.n_waits = len(p.waits)
        prog.n_counters = p.n_counters
        prog.n_ctas = p.num_ctas
        prog.page_bytes = self._page_bytes
        prog.n_pages = self._n_pages
        prog.act_bytes = self._act_bytes
        prog.timeout_ms = int(self.config.timeout_ms)
        prog.device = dev
        prog.ops = arrays["ops"].ctypes.data
        prog.instrs = arrays["instrs"].ctypes.data
        prog.cta_instr_begin = arrays["ib"].ctypes.data
        prog.events = arrays["events"].ctypes.data
        prog.cta_event_begin = arrays["eb"].ctypes.data
        prog.waits = arrays["waits"].ctypes.data
        pos = self.config.position
        if pos is not None:
            if pos.dtype != torch.int32 or not 1 <= pos.numel() <= 32 or not pos.is_cuda or not pos.is_contiguous():
                raise ValueError("MegakernelConfig.position must be a contiguous int32 CUDA tensor with one element, "
                                 "or one per batch row (at most 32)")
            prog.position = pos.data_ptr()
            prog.position_count = int(pos.numel())
            limits = [op.pos_limit for op in self.native_ops if op.pos_limit is not None]
            if self.config.position_limit is not None:
                limits.append(int(self.config.position_limit))
            if not limits:
                raise ValueError("MegakernelConfig.position is set but no op follows it (schedule with a dynamic position)")
            prog.position_limit = min(limits)
        nbytes = int(lib.mk_workspace_bytes(C.byref(prog)))
        self._workspace = torch.empty(nbytes + 256, dtype=torch.uint8, device=torch.device("cuda", dev))
        base = self._workspace.data_ptr()
        aligned = (base + 255) // 256 * 256
        prog.workspace = aligned
        prog.workspace_bytes = nbytes
        handle = C.c_void_p()
        N.check(lib.mk_create(C.byref(prog), C.byref(handle)), "mk_create")
        self._handle = handle
        self._arrays = arrays
        self._dev = dev
        return self

    def run(self, stream=None, sync: bool = True, validate: bool = True) -> None:
        """Launch one pass of the program.

        ``stream``: a ``torch.cuda.Stream`` / raw handle, default = torch's
        current stream.  ``sync=True`` waits for completion and raises
        ``RuntimeError`` if a device-side wait expired.  ``validate=True``
        checks that the scheduled tensors were not reallocated.
        """
        if validate:
            self._validate_tensors()
        self.compile()
        if stream is None:
            handle = torch.cuda.current_stream(self._dev).cuda_stream
        elif hasattr(stream, "cuda_stream"):
            handle = stream.cuda_stream
        else:
            handle = int(stream)
        N.check(N.lib().mk_run(self._handle, C.c_void_p(handle)), "mk_run")
        if sync:
            self.wait()

    def prepare_run(self, stream=None, validate: bool = True, reset_barriers: bool = True) -> dict:
        """Everything of ``run()`` that is not the launch: validate, compile, resolve the stream.

        Mirror of the reference's ``prepare_run`` (megakernel/megakernel.py:2122-2161).  Returns the
        launch state for :meth:`launch_prepared`.  ``reset_barriers`` is accepted for signature
        parity: the kernel clears its own dependency counters at the end of every launch.
        """
        if validate:
            self._validate_tensors()
        self.compile()
        if stream is None:
            handle = torch.cuda.current_stream(self._dev).cuda_stream
        elif hasattr(stream, "cuda_stream"):
            handle = stream.cuda_stream
        else:
            handle = int(stream)
        return {"stream": handle, "handle": self._handle}

    def launch_prepared(self, state: dict, stream=None, trace_buffer_ptr=None, sync: bool = False) -> None:
        """Launch with a state from :meth:`prepare_run` (reference: megakernel/megakernel.py:2163-2181).

        ``stream`` overrides the prepared stream; ``trace_buffer_ptr`` is accepted for signature
        parity (tracing is attached with :meth:`enable_trace`).
        """
        handle = state["stream"] if stream is None else getattr(stream, "cuda_stream", stream)
        N.check(N.lib().mk_run(state["handle"], C.c_void_p(int(handle))), "mk_run")
        if sync:
            self.wait()

    def launch_count(self) -> int:
        """Launches this handle has completed (aborted ones included); see ``mk_launch_count``."""
        self.compile()
        out = C.c_int32()
        N.check(N.lib().mk_launch_count(self._handle, C.byref(out)), "mk_launch_count")
        return int(out.value)

    def set_launch_count(self, count: int) -> None:
        self.compile()
        N.check(N.lib().mk_set_launch_count(self._handle, int(count), None), "mk_set_launch_count")

    def resync_launch_count(self, group=None) -> int:
        """Tensor-parallel recovery: set every rank's launch count to the group maximum.

        The in-kernel all-reduce tags its messages with the launch number, so after one rank missed
        or aborted a launch (a peer timeout surfaces as ``RuntimeError`` from :meth:`wait`) the ranks
        agree on a count here, between steps and with no kernel in flight, before launching again.
        """
        import torch.distributed as dist

        t = torch.tensor([self.launch_count()], dtype=torch.int64, device=torch.device("cuda", self._dev))
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        self.set_launch_count(int(t.item()))
        return int(t.item())

    def wait(self) -> None:
        """Drain the device and surface device-side errors."""
        torch.cuda.synchronize(self._dev)
        st = self.status()
        if st[0] != 0:
            N.lib().mk_reset(self._handle, None)
            # scratch the kernel keeps at zero between launches (top-1 keys, attention arrival counters)
            # may hold values of the aborted launch
            for nop in self.native_ops:
                for t in nop.zero_on_reset:
                    t.zero_()
            torch.cuda.synchronize(self._dev)
            raise RuntimeError(
                f"megakernel aborted: {N.STATUS_NAMES.get(int(st[0]), st[0])} "
                f"(cta={st[1]}, instr={st[2]}, aux={st[3]}, aux2={st[4]}, warp={st[5]})"
            )

    def status(self) -> np.ndarray:
        out = (C.c_int32 * 16)()
        N.check(N.lib().mk_status(self._handle, out), "mk_status")
        return np.frombuffer(out, dtype=np.int32).copy()

    def read_counters(self) -> np.ndarray:
        n = self.program.n_counters
        out = (C.c_int32 * max(1, n))()
        N.check(N.lib().mk_read_counters(self._handle, out, n), "mk_read_counters")
        return np.frombuffer(out, dtype=np.int32)[:n].copy()

    def update_op(self, index: int, native_op: NativeOp, stream=None) -> None:
        """Replace op record ``index`` on the device (e.g. a new cache position)."""
        self.compile()
        rec = np.zeros(1, dtype=N.OP_DTYPE)
        rec[0] = native_op.record(int(self.program.ops[index]["act_key"]))
        handle = None if stream is None else C.c_void_p(getattr(stream, "cuda_stream", stream))
        N.check(N.lib().mk_update_op(self._handle, index, rec.ctypes.data, handle), "mk_update_op")
        self.native_ops[index] = native_op

    # -- tracing --------------------------------------------------------------------------------
    TRACE_DTYPE = np.dtype([("t", "<u8"), ("code", "<u4"), ("arg", "<u4")])
    TRACE_CODES = {1: "load_begin", 2: "load_issued", 3: "page_ready", 4: "page_done", 5: "unit_begin",
                   6: "unit_end", 7: "event_begin", 8: "event_deps", 9: "event_end", 10: "lwait_done"}

    def enable_trace(self, records_per_warp: int = 4096) -> None:
        """Record globaltimer-stamped events of every warp on the next launches.

        The counterpart of ``MegakernelConfig.tracing`` in the reference
        (megakernel/tracing.py:51-153); costs a few global stores per page, so
        timings taken with tracing on are for analysis only.
        """
        self.compile()
        warps = self.program.num_ctas * (NUM_CONSUMER_WARPS + NUM_DMA_WARPS)
        nbytes = warps * (records_per_warp * 16 + 4)
        self._trace_buf = torch.zeros(nbytes + 16, dtype=torch.uint8, device=torch.device("cuda", self._dev))
        self._trace_cap = records_per_warp
        N.check(N.lib().mk_set_trace(self._handle, C.c_void_p(self._trace_buf.data_ptr()), nbytes,
                                     records_per_warp), "mk_set_trace")

    def disable_trace(self) -> None:
        if self._handle:
            N.check(N.lib().mk_set_trace(self._handle, None, 0, 0), "mk_set_trace")

    def read_trace(self):
        """Return ``{(cta, warp): structured array of (t, code, arg)}`` of the last launch.

        ``t`` is in nanoseconds on a time base common to all CTAs.  The device
        stamps records with its cycle counter and brackets every warp's ring
        with (cycle counter, nanosecond timer) pairs (codes 30 / 31); the
        cycles are mapped linearly between the two pairs here.
        """
        torch.cuda.synchronize(self._dev)
        raw = self._trace_buf.cpu().numpy()
        warps_per_cta = NUM_CONSUMER_WARPS + NUM_DMA_WARPS
        warps = self.program.num_ctas * warps_per_cta
        cap = self._trace_cap
        recs = raw[:warps * cap * 16].view(self.TRACE_DTYPE).reshape(warps, cap)
        counts = raw[warps * cap * 16: warps * cap * 16 + warps * 4].view(np.int32)
        out = {}
        for wi in range(warps):
            n = min(int(counts[wi]), cap)
            arr = recs[wi, :n].copy()
            clk = np.flatnonzero(arr["code"] == 30)
            if len(clk) >= 2 and clk[-1] + 1 < n:
                c0, g0 = int(arr["t"][clk[0]]), int(arr["t"][clk[0] + 1])
                c1, g1 = int(arr["t"][clk[-1]]), int(arr["t"][clk[-1] + 1])
                scale = (g1 - g0) / max(1, c1 - c0)
                keep = arr["code"] < 30
                arr = arr[keep]
                # integer arithmetic around g0: the timer's magnitude (~2**60 ns) exceeds float64's exact range
                delta = np.rint((arr["t"].astype(np.int64) - c0) * scale).astype(np.int64)
                arr["t"] = (np.int64(g0) + delta).astype(np.uint64)
            out[(wi // warps_per_cta, wi % warps_per_cta)] = arr
        return out

    def export_chrome_trace(self, path: str, ctas=(0,)) -> None:
        """Write the begin/end pairs of the chosen CTAs as a Chrome / Perfetto trace."""
        import json

        tr = self.read_trace()
        t0 = min((int(a["t"][0]) for a in tr.values() if len(a)), default=0)
        pairs = {1: (2, "load"), 3: (4, "page"), 5: (6, "unit"), 7: (9, "event")}
        events = []
        for (cta, warp), arr in tr.items():
            if cta not in ctas:
                continue
            open_at = {}
            for r in arr:
                code, arg, t = int(r["code"]), int(r["arg"]), (int(r["t"]) - t0) / 1e3
                if code in pairs:
                    open_at[(pairs[code][0], arg)] = (t, pairs[code][1])
                elif (code, arg) in open_at:
                    tb, name = open_at.pop((code, arg))
                    events.append({"name": f"{name} {arg}", "ph": "X", "ts": tb, "dur": t - tb, "pid": cta,
                                   "tid": warp})
        with open(path, "w") as fh:
            json.dump({"traceEvents": events}, fh)

    def stage_table(self) -> list:
        """Where the last traced launch spent its time, op by op (microseconds from the first record).

        One dict per native op: ``begin`` = first unit started on any CTA, ``end`` = last unit
        signalled, ``gap`` = begin minus the latest end of any earlier op (negative when ops overlap),
        ``poll`` / ``stage`` = median over CTAs of the op-entry event's wait for the producers and of
        the activation staging, ``page`` = median time a consumer warp held one page, ``units``.
        """
        tr = self.read_trace()
        instr_op = self.program.instrs["op"]
        n = len(self.native_ops)
        t0 = min((int(a["t"][0]) for a in tr.values() if len(a)), default=0)
        begin, end = np.full(n, np.iinfo(np.int64).max), np.zeros(n, dtype=np.int64)
        poll = [[] for _ in range(n)]
        stage = [[] for _ in range(n)]
        page = [[] for _ in range(n)]
        for (cta, warp), arr in tr.items():
            if warp == 0:
                continue
            ev_begin, ev_deps, ready, cur = {}, {}, 0, None
            for r in arr:
                code, arg, t = int(r["code"]), int(r["arg"]), int(r["t"]) - t0
                if code == 7:
                    ev_begin[arg] = t
                elif code == 8:
                    ev_deps[arg] = t
                    if arg in ev_begin:
                        poll[arg].append(t - ev_begin[arg])
                elif code == 9 and arg in ev_deps:
                    stage[arg].append(t - ev_deps[arg])
                elif code == 5:
                    cur = int(instr_op[arg])
                    begin[cur] = min(begin[cur], t)
                elif code == 3:
                    ready = t
                elif code == 4 and cur is not None:
                    page[cur].append(t - ready)
                elif code == 6:
                    o = int(instr_op[arg])
                    end[o] = max(end[o], t)
        med = lambda v: float(np.median(v)) / 1e3 if v else None          # noqa: E731
        rows, latest = [], 0
        for o, nop in enumerate(self.native_ops):
            b = int(begin[o]) if begin[o] != np.iinfo(np.int64).max else 0
            rows.append({"op": o, "name": nop.name, "units": int(nop.n_units), "begin": b / 1e3, "end": int(end[o]) / 1e3,
                         "span": (int(end[o]) - b) / 1e3, "gap": (b - latest) / 1e3, "poll": med(poll[o]),
                         "stage": med(stage[o]), "page": med(page[o])})
            latest = max(latest, int(end[o]))
        return rows

    def bench_spec(self, setup_fn=None, keep_alive=None) -> dict:
        """A launch closure plus byte accounting for benchmark harnesses."""
        self.compile()

        def launch():
            self.run(sync=False, validate=False)

        return {"launch": launch, "setup": setup_fn, "bytes": self.algorithmic_bytes, "keep_alive": keep_alive}

    def _validate_tensors(self) -> None:
        for op in self.ops:
            for name, ptr in op.tensor_ptrs.items():
                ref = op.tensor_refs.get(name)
                if ref is not None and ref.data_ptr() != ptr:
                    raise RuntimeError(
                        f"{op.op_cls.__name__}: tensor '{name}' was reallocated after schedule(); "
                        f"tensors are captured by pointer"
                    )

    def __del__(self):
        try:
            if self._handle:
                N.lib().mk_destroy(self._handle)
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def create_megakernel(ops, num_sms=None, **cfg) -> Megakernel:
    """Convenience constructor (reference megakernel.py:2293)."""
    known = {f for f in MegakernelConfig.__dataclass_fields__}
    unknown = set(cfg) - known
    if unknown:
        warnings.warn(f"create_megakernel: ignoring unknown config fields {sorted(unknown)}", stacklevel=2)
    config = MegakernelConfig(num_sms=num_sms, **{k: v for k, v in cfg.items() if k in known})
    return Megakernel(ops, config=config)


__all__ = ["Megakernel", "MegakernelConfig", "create_megakernel", "NUM_DMA_WARPS"]
