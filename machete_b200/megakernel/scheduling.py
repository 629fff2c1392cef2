"""Host scheduler: dependency inference, unit placement and program tables.

Counterpart of the reference's ``InstructionStreamBuilder`` and tile
schedulers (src/machete/megakernel/scheduling.py:445-2424).  The contract is
the same — ops are listed in program order, dependencies are inferred from
which tensors alias (RAW, WAR and WAW, then transitively reduced,
scheduling.py:915-1120), work is dealt statically to one persistent CTA per SM,
and completion is tracked by monotonic counters compared with ``>=``
(megakernel/interpreter.py:33-77) — but the tables are this build's own:

* an instruction is one *unit* of one CTA (64 bytes, ``mk_instr_t``; matvec and
  attention units are shared by several consumer warps of that CTA), stored
  per CTA contiguously rather than interleaved;
* every op has an *entry event* on each CTA that holds units of it: all
  consumer warps of the CTA meet there, wait for the op's producers and stage
  its activations, so units themselves carry waits only for finer-grained
  edges (attention combine -> the splits of its own KV head);
* loader-side waits exist only where the loader reads memory produced in the
  same launch (the KV rows appended by this step); weights never wait.

Deadlock freedom: each CTA executes a subsequence of the global program order
and every wait refers to an earlier op of that order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import _native as N
from .lowering import NativeOp, Region
from .instruction_format import BarrierFormula, TileInstruction  # noqa: F401  (the reference exports them here)
from .ops import tensor_meta_overlaps

INSTRUCTION_WORDS = 8
"""int32 words per instruction row (``mk_instr_t``)."""


# ---- placement policies ---------------------------------------------------------------------
class TileScheduler:
    """Decides which CTA runs each unit.  Units are presented in program order."""

    def bind_num_blocks(self, n: int) -> "TileScheduler":
        self.num_blocks = n
        return self

    def place(self, ops: Sequence[NativeOp], num_ctas: int) -> List[np.ndarray]:
        raise NotImplementedError


class BackwardScheduler(TileScheduler):
    """Round-robin over CTAs, continuing across op boundaries.

    Takes the place of the reference's default scheduler (scheduling.py:445);
    the static strided assignment is the same idea as its
    ``block_id + k * num_blocks`` instruction fetch (replay_loops.py:107-155).
    """

    def place(self, ops, num_ctas):
        out, rr = [], 0
        for op in ops:
            out.append(((np.arange(op.n_units, dtype=np.int64) + rr) % num_ctas).astype(np.int32))
            rr = (rr + op.n_units) % num_ctas
        return out


class OverlapTileScheduler(TileScheduler):
    """Level placement: every op is spread evenly, lightest CTAs first.

    Ops of a decode step run one after another (each needs the whole output of
    its producer), so what bounds the step is, per op, the CTA with the most
    units of that op.  Each op therefore gives every CTA at most
    ``ceil(n_units / num_ctas)`` units, dealing them round-robin over the CTAs
    ordered by the bytes they have streamed so far; the leftovers of one op
    thus fill the CTAs that the previous ops left lighter.

    Accepts the reference's constructor keywords (scheduling.py:486-506) so
    existing call sites keep working; they tune a readiness simulation this
    scheduler does not need.
    """

    _warned = False

    def __init__(self, fetch_stride=None, adaptive_fetch_stride=False, prefer_data_movement=True,
                 prefer_ready_consumers=False, use_controller_waits_for_readiness=False):
        tuned = (fetch_stride is not None or adaptive_fetch_stride or not prefer_data_movement
                 or prefer_ready_consumers or use_controller_waits_for_readiness)
        if tuned and not OverlapTileScheduler._warned:
            import warnings

            OverlapTileScheduler._warned = True
            warnings.warn("OverlapTileScheduler keywords tune the reference's readiness simulation; the level "
                          "placement used here accepts and ignores them", stacklevel=2)
        self.fetch_stride = fetch_stride
        self.adaptive_fetch_stride = adaptive_fetch_stride
        self.prefer_data_movement = prefer_data_movement
        self.prefer_ready_consumers = prefer_ready_consumers
        self.use_controller_waits_for_readiness = use_controller_waits_for_readiness

    def place(self, ops, num_ctas):
        load = np.zeros(num_ctas, dtype=np.int64)
        out = []
        for op in ops:
            order = np.argsort(load, kind="stable").astype(np.int32)
            a = order[np.arange(op.n_units) % num_ctas].astype(np.int32)
            for u in range(op.n_units):
                # a unit with no streamed bytes still costs a little time
                load[a[u]] += max(op.bytes_of(u), 2048)
            out.append(a)
        return out


# ---- dependency inference -------------------------------------------------------------------
@dataclass
class OpDeps:
    coarse: List[int] = field(default_factory=list)        # producers waited at the op-entry event
    act_version: Tuple[int, ...] = ()                      # latest writers of the staged inputs
    fine: Dict[int, List[List[int]]] = field(default_factory=dict)  # producer -> per-unit group lists
    loader: List[int] = field(default_factory=list)        # producers the loader must wait for


def infer_dependencies(ops: Sequence[NativeOp]) -> List[OpDeps]:
    """Op-level dependency edges from tensor aliasing, transitively reduced."""
    n = len(ops)
    reads_by_storage: Dict[int, List[Tuple[int, Region]]] = {}
    writes_by_storage: Dict[int, List[Tuple[int, Region]]] = {}
    closure = [0] * n  # bitset of ops that must be complete once op j is complete
    result: List[OpDeps] = []
    for j, op in enumerate(ops):
        found: Dict[int, bool] = {}  # producer -> needed by a loader-side read?
        act_version: List[int] = []
        for r in op.reads:
            latest = -1
            for i, w in writes_by_storage.get(r.meta.storage_ptr, ()):
                if i != j and r.overlaps(w):
                    found[i] = found.get(i, False) or r.loader
                    latest = max(latest, i)
            if r.act:
                act_version.append(latest)
        for w in op.writes:
            for i, w2 in writes_by_storage.get(w.meta.storage_ptr, ()):
                if i != j and w.overlaps(w2):
                    found.setdefault(i, False)
            for i, r2 in reads_by_storage.get(w.meta.storage_ptr, ()):
                if i != j and w.overlaps(r2):
                    found.setdefault(i, False)
        # transitive reduction: drop i when another kept producer already implies it
        cand = sorted(found, reverse=True)
        kept: List[int] = []
        implied = 0
        for i in cand:
            if (implied >> i) & 1:
                continue
            kept.append(i)
            implied |= closure[i] | (1 << i)
        kept.sort()
        deps = OpDeps(act_version=tuple(act_version))
        for i in kept:
            fine = op.fine_dep(op, ops[i]) if op.fine_dep is not None else None
            if fine is not None:
                deps.fine[i] = fine
            else:
                deps.coarse.append(i)
        # loader waits are never reduced away by consumer-side implication:
        # the loader runs ahead of the consumers and must see the producer itself
        deps.loader = sorted(i for i, ld in found.items() if ld)
        closure[j] = implied
        result.append(deps)
        for r in op.reads:
            reads_by_storage.setdefault(r.meta.storage_ptr, []).append((j, r))
        for w in op.writes:
            writes_by_storage.setdefault(w.meta.storage_ptr, []).append((j, w))
    return result, closure


# ---- op-pair resolution on scheduled ops ----------------------------------------------------
def resolve_dep_pairs(ops) -> List[Tuple[int, int, str, str]]:
    """Ordered ``(producer, consumer, producer buffer, consumer buffer)`` pairs of a scheduled-op list.

    The op-level contract of the reference builder (src/machete/megakernel/scheduling.py:915-1120),
    stated on ``ScheduledOp`` records before any lowering or fusion:

    * read-after-write: each declared input depends on the nearest earlier op that writes a buffer
      of the same name at the same address, else on the latest earlier op with an output that
      overlaps it in memory; every earlier accumulating (reduce-store) writer that overlaps the
      input is a producer as well;
    * ordering of storage reuse: an op that writes a tensor follows every earlier op that reads or
      writes overlapping memory (two accumulating writers of the same memory commute);
    * the second kind is dropped where another path already orders the two ops; read-after-write
      pairs are always kept, because consumers take their tile mapping from them.

    ``infer_dependencies`` below works on lowered ops and reduces every kind of edge; the two agree
    on the ordering they impose (their transitive closures are equal on unfused programs).
    """
    def outs(op):
        return [(n, op.tensor_metas.get(n)) for n in op.op_cls.OUTPUTS]

    def ins(op):
        return [(n, op.tensor_metas.get(n)) for n in op.op_cls.INPUTS]

    def accumulates(op, name):
        return name in getattr(op.op_cls, "_TMA_REDUCE_STORES", ())

    def touching(metas, m):
        return next((n for n, x in metas if x is not None and tensor_meta_overlaps(x, m)), None)

    pairs: Dict[Tuple[int, int, str, str], bool] = {}       # insertion-ordered; value: read-after-write?
    for j, op in enumerate(ops):
        for name, meta in ins(op):
            ptr = op.tensor_ptrs.get(name)
            prod = None
            for i in range(j - 1, -1, -1):                  # same name, same address: nearest wins
                if name in ops[i].op_cls.OUTPUTS:
                    p = ops[i].tensor_ptrs.get(name)
                    if p is None or ptr is None or p == ptr:
                        prod = i
                        break
            if prod is None and meta is not None:           # another name for the same memory: latest wins
                prod = next((i for i in range(j - 1, -1, -1) if touching(outs(ops[i]), meta)), None)
            if prod is not None:
                src = name
                same_name = name in ops[prod].op_cls.OUTPUTS and (
                    ops[prod].tensor_ptrs.get(name) is None or ptr is None or ops[prod].tensor_ptrs.get(name) == ptr)
                if not same_name and meta is not None:
                    src = touching(outs(ops[prod]), meta) or name
                pairs.setdefault((prod, j, src, name), True)
            if meta is not None:
                for i in range(j - 1, -1, -1):
                    for n, m in outs(ops[i]):
                        if m is not None and accumulates(ops[i], n) and tensor_meta_overlaps(m, meta):
                            pairs[(i, j, n, name)] = True
    raw = {(p, c) for (p, c, _, _), is_raw in pairs.items() if is_raw}
    for j, op in enumerate(ops):
        for name, meta in outs(op):
            if meta is None:
                continue
            for i in range(j - 1, -1, -1):
                hit = touching(ins(ops[i]), meta) or touching(outs(ops[i]), meta)
                if hit is None:
                    continue
                both_accumulate = any(
                    accumulates(op, a) and accumulates(ops[i], b) and ma is not None and mb is not None
                    and tensor_meta_overlaps(ma, mb) for a, ma in outs(op) for b, mb in outs(ops[i]))
                if not both_accumulate:
                    pairs.setdefault((i, j, hit, name), False)
    succ: Dict[int, set] = {}
    for p, c, _, _ in pairs:
        succ.setdefault(p, set()).add(c)

    def other_path(src, dst):
        todo, seen = [n for n in succ.get(src, ()) if n != dst], set()
        while todo:
            n = todo.pop()
            if n == dst:
                return True
            if n not in seen:
                seen.add(n)
                todo.extend(succ.get(n, ()))
        return False

    return [k for k in pairs if (k[0], k[1]) in raw or not other_path(k[0], k[1])]


def closure_of(pairs, n_ops: int) -> List[int]:
    """Bitset per op of every op that must be complete before it (transitive closure of ``pairs``)."""
    before = [0] * n_ops
    by_consumer: Dict[int, List[int]] = {}
    for p, c in pairs:
        by_consumer.setdefault(c, []).append(p)
    for j in range(n_ops):                                  # producers always precede consumers in program order
        for i in by_consumer.get(j, ()):
            before[j] |= before[i] | (1 << i)
    return before


# ---- program tables -------------------------------------------------------------------------
@dataclass
class BuiltProgram:
    ops: np.ndarray
    instrs: np.ndarray
    cta_instr_begin: np.ndarray
    events: np.ndarray
    cta_event_begin: np.ndarray
    waits: np.ndarray
    n_counters: int
    num_ctas: int
    act_bytes: int
    page_need: int
    counter_base: List[int]
    counter_expected: np.ndarray     # final value of every counter after one launch
    deps: List[OpDeps]
    placement: List[np.ndarray]
    bytes_per_cta: np.ndarray
    total_bytes: int
    native_ops: List[NativeOp]


class InstructionStreamBuilder:
    """Collects lowered ops and emits the program tables for ``mk_create``."""

    def __init__(self, num_ctas: int):
        if num_ctas < 1:
            raise ValueError("num_ctas must be positive")
        self.num_ctas = num_ctas
        self.ops: List[NativeOp] = []

    def add_op(self, op: NativeOp) -> int:
        if op.n_units < 0:
            raise ValueError(f"{op.name}: negative unit count")
        self.ops.append(op)
        return len(self.ops) - 1

    def build(self, scheduler: Optional[TileScheduler] = None) -> BuiltProgram:
        ops = self.ops
        if not ops:
            raise ValueError("cannot build an empty program")
        scheduler = scheduler or BackwardScheduler()
        total_units = sum(op.n_units for op in ops)
        num_ctas = max(1, min(self.num_ctas, total_units))
        deps, closure = infer_dependencies(ops)

        # activation-staging keys: equal signature + equal producers of the inputs
        act_keys, sig_ids = [], {}
        for j, op in enumerate(ops):
            if op.act_sig is None:
                act_keys.append(0)
                continue
            # the staged data is a function of the inputs' contents, i.e. of their
            # latest writers: the same buffers re-written by a later layer get a new key
            key = (op.act_sig, deps[j].act_version)
            act_keys.append(sig_ids.setdefault(key, len(sig_ids) + 1))

        counter_base, n_counters = [], 0
        for op in ops:
            counter_base.append(n_counters)
            n_counters += op.n_groups
        counter_expected = np.zeros(max(1, n_counters), dtype=np.int64)
        for j, op in enumerate(ops):
            counter_expected[counter_base[j]:counter_base[j] + op.n_groups] = op.group_sizes()

        placement = scheduler.place(ops, num_ctas)

        waits: List[Tuple[int, int]] = []
        wait_cache: Dict[tuple, int] = {}

        def wait_list(pairs: Sequence[Tuple[int, int]]) -> Tuple[int, int]:
            pairs = tuple(pairs)
            if not pairs:
                return 0, 0
            off = wait_cache.get(pairs)
            if off is None:
                off = len(waits)
                waits.extend(pairs)
                wait_cache[pairs] = off
            return len(pairs), off

        def all_groups(i: int) -> List[Tuple[int, int]]:
            sizes = ops[i].group_sizes()
            return [(counter_base[i] + g, int(sizes[g])) for g in range(ops[i].n_groups) if sizes[g] > 0]

        cta_instrs: List[List[tuple]] = [[] for _ in range(num_ctas)]
        cta_events: List[List[tuple]] = [[] for _ in range(num_ctas)]
        cta_known = [0] * num_ctas       # ops known complete on this CTA (bitset)
        cta_staged = [0] * num_ctas      # activation key staged in the CTA's shared memory (0 = none)
        bytes_per_cta = np.zeros(num_ctas, dtype=np.int64)

        for j, op in enumerate(ops):
            d = deps[j]
            where = placement[j]
            seen_cta = set()
            res_out_cta = int(where[0]) if (op.writes_res_out and op.n_units > 0) else -1
            loader_pairs_all = [p for i in d.loader for p in all_groups(i)]
            # one counter for the whole op: each CTA signals its units in bulk
            per_cta = np.bincount(np.asarray(where[:op.n_units], dtype=np.int64), minlength=num_ctas)
            bulk = op.n_groups == 1
            for u in range(op.n_units):
                cta = int(where[u])
                if cta not in seen_cta:
                    seen_cta.add(cta)
                    need = [i for i in d.coarse if not (cta_known[cta] >> i) & 1]
                    pairs = [p for i in need for p in all_groups(i)]
                    nw, off = wait_list(pairs)
                    flags = N.EVF_WRITE_RES_OUT if cta == res_out_cta else 0
                    # An op that waits for nothing new and finds its activations already
                    # staged (same key as the op before it, e.g. K and V after Q) needs no
                    # event: its units start on whichever consumer warps are free, next to
                    # the previous op's, read their record from the op table and signal
                    # one by one.
                    staged_already = (op.opcode == N.OP_MATVEC and act_keys[j] != 0
                                      and act_keys[j] == cta_staged[cta])
                    if not (staged_already and nw == 0 and flags == 0):
                        if bulk:
                            flags |= N.EVF_BULK_SIGNAL
                        cta_events[cta].append(
                            (len(cta_instrs[cta]), j, nw, off, flags, int(per_cta[cta]) if bulk else 0))
                        if op.opcode == N.OP_MATVEC:
                            cta_staged[cta] = act_keys[j]
                    for i in d.coarse:
                        cta_known[cta] |= closure[i] | (1 << i)
                # fine-grained consumer waits
                fpairs: List[Tuple[int, int]] = []
                for i, per_unit in d.fine.items():
                    sizes = ops[i].group_sizes()
                    for g in per_unit[u]:
                        fpairs.append((counter_base[i] + g, int(sizes[g])))
                nw, woff = wait_list(fpairs)
                # loader waits
                lpairs: Sequence[Tuple[int, int]] = ()
                if d.loader and op.pages_of(u) > 0:
                    if op.loader_dep_units is None:
                        lpairs = loader_pairs_all
                    else:
                        lpairs = [p for i in d.loader if op.loader_dep_units(ops[i], u) for p in all_groups(i)]
                nl, loff = wait_list(lpairs)
                cta_instrs[cta].append(
                    (j, u, counter_base[j] + op.group_of(u), nw, woff, nl, loff, op.pages_of(u))
                )
                bytes_per_cta[cta] += op.bytes_of(u)

        instrs = np.zeros(total_units, dtype=N.INSTR_DTYPE)
        ibegin = np.zeros(num_ctas + 1, dtype=np.int32)
        n_events = sum(len(e) for e in cta_events)
        events = np.zeros(max(1, n_events), dtype=N.EVENT_DTYPE)
        ebegin = np.zeros(num_ctas + 1, dtype=np.int32)
        io = eo = 0
        for c in range(num_ctas):
            rows = cta_instrs[c]
            if rows:
                arr = np.array(rows, dtype=np.int32)
                blk = instrs[io:io + len(rows)]
                for k, name in enumerate(("op", "unit", "signal", "n_waits", "wait_off", "n_lwaits",
                                          "lwait_off", "n_pages")):
                    blk[name] = arr[:, k]
            io += len(rows)
            ibegin[c + 1] = io
            for (pos, opi, nw, off, flags, bulk_units) in cta_events[c]:
                ev = events[eo]
                ev["pos"], ev["op"], ev["n_waits"], ev["wait_off"], ev["flags"] = pos, opi, nw, off, flags
                ev["bulk_units"] = bulk_units
                eo += 1
            ebegin[c + 1] = eo
        events = events[:max(1, n_events)]

        op_table = np.zeros(len(ops), dtype=N.OP_DTYPE)
        for j, op in enumerate(ops):
            op_table[j] = op.record(act_keys[j])
        wait_table = np.zeros(max(1, len(waits)), dtype=N.WAIT_DTYPE)
        if waits:
            w = np.array(waits, dtype=np.int32)
            wait_table["counter"][:len(waits)] = w[:, 0]
            wait_table["expected"][:len(waits)] = w[:, 1]

        return BuiltProgram(
            ops=op_table, instrs=instrs, cta_instr_begin=ibegin, events=events, cta_event_begin=ebegin,
            waits=wait_table, n_counters=n_counters, num_ctas=num_ctas,
            act_bytes=max((op.act_bytes for op in ops), default=0),
            page_need=max((op.page_need for op in ops), default=0),
            counter_base=counter_base, counter_expected=counter_expected, deps=deps, placement=placement,
            bytes_per_cta=bytes_per_cta, total_bytes=int(bytes_per_cta.sum()), native_ops=list(ops),
        )


def simulate(prog: BuiltProgram, n_events_hint: int = 0) -> np.ndarray:
    """Replay a built program on the host and return the final counter values.

    Executes every CTA's instruction list in order, honouring event, unit and
    loader waits, and raises ``RuntimeError`` if no CTA can make progress (a
    dependency cycle or a wait on a counter nobody signals).  Used by the CPU
    tests as the deadlock and lost-signal check the device cannot offer.
    """
    num_ctas = prog.num_ctas
    counters = np.zeros(max(1, prog.n_counters), dtype=np.int64)
    pc = prog.cta_instr_begin[:-1].astype(np.int64).copy()
    ev = prog.cta_event_begin[:-1].astype(np.int64).copy()
    end = prog.cta_instr_begin[1:]
    ev_end = prog.cta_event_begin[1:]
    n_real_events = int(prog.cta_event_begin[-1])

    def satisfied(n, off):
        for k in range(off, off + n):
            if counters[prog.waits["counter"][k]] < prog.waits["expected"][k]:
                return False
        return True

    remaining = int(prog.cta_instr_begin[-1])
    while remaining > 0:
        progressed = False
        for c in range(num_ctas):
            while pc[c] < end[c]:
                local = pc[c] - prog.cta_instr_begin[c]
                blocked = False
                while ev[c] < ev_end[c] and ev[c] < n_real_events and prog.events["pos"][ev[c]] <= local:
                    e = prog.events[ev[c]]
                    if not satisfied(int(e["n_waits"]), int(e["wait_off"])):
                        blocked = True
                        break
                    ev[c] += 1
                if blocked:
                    break
                ins = prog.instrs[pc[c]]
                if not satisfied(int(ins["n_waits"]), int(ins["wait_off"])):
                    break
                if not satisfied(int(ins["n_lwaits"]), int(ins["lwait_off"])):
                    break
                if ins["signal"] >= 0:
                    counters[ins["signal"]] += 1
                pc[c] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            stuck = [int(c) for c in range(num_ctas) if pc[c] < end[c]]
            raise RuntimeError(f"program deadlocks: CTAs {stuck[:8]} cannot make progress")
    return counters[:max(1, prog.n_counters)]


__all__ = [
    "INSTRUCTION_WORDS", "TileScheduler", "BackwardScheduler", "OverlapTileScheduler", "OpDeps",
    "infer_dependencies", "BuiltProgram", "InstructionStreamBuilder", "simulate",
]
