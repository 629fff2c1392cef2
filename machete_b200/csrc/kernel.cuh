// The persistent decode kernel (device side).
//
// One CTA per SM.  Warp 0 is the loader: it walks the CTA's instruction list
// and streams every unit's pages (weight K-slices and K/V token blocks, both by
// tiled TMA) into a shared-memory ring, running as far ahead of the consumers
// as the ring allows — weights carry no data dependency, so the HBM stream
// continues across op boundaries while consumers wait on dependency counters.
// Warps 1..7 are consumers.  A unit owns one consumer slot per participant
// (matvec and attention units are shared page by page, every other unit has
// one); a consumer that becomes free draws the next slot from a ticket
// counter, waits for its pages, computes, and the participant that completes
// the unit signals its counter.  Op-entry events make all consumers of the
// CTA meet, wait for the op's producers and stage its activations (RMSNorm and
// residual add fused).
//
// The kernel is a template over what a program needs (activation-tile class,
// weight family, and a feature mask): the instruction cache of an SM holds
// 128 KB behind a 32 KB first level, every op boundary of a decode step runs
// code that was last used one layer earlier, and a kernel that carries the
// code of ops the program never uses pays for it in instruction misses on
// exactly that path.
//
// Counterpart of the reference's ring loop (megakernel/replay_loops.py:27-824).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "op_allreduce.cuh"
#include "op_attn.cuh"
#include "op_elementwise.cuh"
#include "op_matvec.cuh"

namespace mk {

// The consumers' view of an instruction record: one record per lane, 32 at a
// time; a field is fetched from the owning lane with a shuffle when needed.
constexpr int kInsMatvec = (int)0x80000000;   // bit 31 of `flags`: the unit is shared page by page
__device__ __forceinline__ InsRegs load_instr(const mk_instr_t* p) {
  const int4* q = reinterpret_cast<const int4*>(p);
  const int4 a = q[0], b = q[1], c2 = q[2], d = q[3];
  InsRegs r;
  r.op = a.x; r.unit = a.y; r.signal = a.z; r.n_waits = a.w;
  r.wait_off = b.x; r.n_pages = b.w;
  r.flags = (c2.x | c2.y) != 0 ? (c2.w | kInsMatvec) : 0;
  r.row_a = d.x; r.row_b = d.y; r.off_a = d.z; r.off_b = d.w;
  return r;
}
__device__ __forceinline__ InsRegs empty_instr() {
  InsRegs r;
  r.op = r.unit = r.signal = r.n_waits = r.wait_off = r.n_pages = r.flags = 0;
  r.row_a = r.row_b = r.off_a = r.off_b = 0;
  return r;
}

// The loader's view: everything needed to issue the unit's tiled-TMA pages
// (tensor-map address, first rows, tiles per page).
struct LoaderInstr {
  int op, unit, n_lwaits, lwait_off, n_pages;
  uint64_t maps;
  int row_a, row_b, tiles, flags;
};
__device__ __forceinline__ LoaderInstr load_loader_instr(const mk_instr_t* p) {
  const int4* q = reinterpret_cast<const int4*>(p);
  const int4 a = q[0], b = q[1], c2 = q[2], d = q[3];
  LoaderInstr r;
  r.op = a.x; r.unit = a.y; r.n_lwaits = b.y; r.lwait_off = b.z; r.n_pages = b.w;
  r.maps = (uint64_t)(uint32_t)c2.x | ((uint64_t)(uint32_t)c2.y << 32);
  r.tiles = c2.z; r.flags = c2.w; r.row_a = d.x; r.row_b = d.y;
  return r;
}
__device__ __forceinline__ LoaderInstr bcast_loader_instr(const LoaderInstr& m, int src) {
  LoaderInstr r;
  r.op = __shfl_sync(0xffffffffu, m.op, src);
  r.unit = __shfl_sync(0xffffffffu, m.unit, src);
  r.n_lwaits = __shfl_sync(0xffffffffu, m.n_lwaits, src);
  r.lwait_off = __shfl_sync(0xffffffffu, m.lwait_off, src);
  r.n_pages = __shfl_sync(0xffffffffu, m.n_pages, src);
  r.maps = __shfl_sync(0xffffffffu, m.maps, src);
  r.row_a = __shfl_sync(0xffffffffu, m.row_a, src);
  r.row_b = __shfl_sync(0xffffffffu, m.row_b, src);
  r.tiles = __shfl_sync(0xffffffffu, m.tiles, src);
  r.flags = __shfl_sync(0xffffffffu, m.flags, src);
  return r;
}

static __device__ void loader_loop(Ctx& c, int ibeg, int iend) {
  const ProgramView& pv = *c.pv;
  const int NP = pv.n_pages;
  const uint64_t policy = l2_evict_first_policy();
  uint32_t seq = 0;
  RingPos rp;
  rp.slot = 0;
  rp.k = 0;
  for (int base = ibeg; base < iend && !c.dead; base += 32) {
    const int n = min(32, iend - base);
    LoaderInstr mine;
    memset(&mine, 0, sizeof(mine));
    if (c.lane < n) mine = load_loader_instr(pv.instrs + base + c.lane);
    for (int i = 0; i < n && !c.dead; ++i) {
      const LoaderInstr ins = bcast_loader_instr(mine, i);
      c.instr_idx = base + i;
      if (ins.n_pages == 0) continue;
      int n_pages = ins.n_pages;
      bool need_wait = ins.n_lwaits > 0;
      if (ins.flags & MK_LDF_DYN) {
        // the window follows the device-resident position: tokens [0, pos + 1); only the unit
        // that holds the row appended in this launch waits for it
        const int pos = c.ctrl->pos[(ins.row_b >> 16) & 31];      // the unit's batch row
        n_pages = at_dyn_pages(ins.row_a, ins.n_pages, ins.tiles, pos + 1);
        need_wait = need_wait && pos >= ins.row_a && pos < ins.row_a + ins.n_pages * ins.tiles;
        if (n_pages == 0) continue;
      }
      if (need_wait) {
        if (!wait_counters(c, ins.n_lwaits, ins.lwait_off)) break;
        trace(c, TRC_LWAIT_DONE, base + i);
      }
      if (ins.maps == 0) continue;   // only units with tensor maps stream pages
      // Pages are issued by lane 0 alone in a tight loop from the fields of the
      // instruction record (no op-table read on this path; a one-thread wait
      // needs no vote).  Fill k of a slot needs fill k-1 handed back:
      // empty-barrier phase k-1.  A split-KV attention page is one K box and one
      // V box (two each for head dim 128), a matvec page two weight boxes
      // (plus two scale boxes for NVFP4).
      const bool attn = (ins.flags & MK_LDF_ATTN) != 0;
      if (attn && need_wait) fence_proxy_async_all();   // the awaited K/V rows were written by plain stores
      int issued = 0;
      if (c.lane == 0) {
        const uint8_t* maps = reinterpret_cast<const uint8_t*>(ins.maps);
        const bool pair = (ins.flags & MK_LDF_PAIR) != 0;
        MvLoad ml;
        ml.fp4 = (ins.flags & MK_LDF_FP4) != 0;
        ml.tm_a = maps;
        ml.tm_b = maps + (pair ? 128 : 0);
        ml.ts_a = maps + 256;
        ml.ts_b = maps + (pair ? 384 : 256);
        ml.rowA0 = ins.row_a;
        ml.rowB0 = ins.row_b;
        ml.tiles_per_page = ins.tiles;
        ml.half = (uint32_t)ins.tiles * 1024u;
        RingPos q = rp;
#pragma unroll 1
        for (; issued < n_pages; ++issued, ring_next(q, NP)) {
          if (!wait_mbar_one(c, empty_bar(c, q.slot), (q.k & 1u) ^ 1u, MK_ST_TIMEOUT_PAGE_EMPTY, (int)(seq + issued)))
            break;
          trace(c, TRC_LOAD_BEGIN, seq + issued);
          const uint32_t page = c.pages_u32 + q.slot * (uint32_t)pv.page_bytes;
          if (attn)
            at_load_issue(maps, maps + 128, (ins.flags & MK_LDF_D128) != 0, ins.tiles, ins.row_a + issued * ins.tiles,
                          ins.row_b & 0xffff, ins.row_b >> 16, page, full_bar(c, q.slot), policy);
          else
            mv_load_issue(ml, issued, page, full_bar(c, q.slot), policy);
          trace(c, TRC_LOAD_ISSUED, seq + issued);
        }
      }
      issued = __shfl_sync(0xffffffffu, issued, 0);
      if (issued < n_pages) c.dead = true;   // lane 0 gave up (abort flag is already raised)
      ring_advance(rp, issued, NP);
      seq += (uint32_t)issued;
    }
  }
  // Every copy this warp issued must have landed before the CTA may exit.
  // On the normal path the consumers already observed all of them; after an
  // abandoned wait they may not have, so drain with a bounded wait.
  if (c.dead) {
    const uint32_t first = seq > (uint32_t)NP ? seq - NP : 0u;
    for (uint32_t s = first; s < seq; ++s) {
      const uint32_t bar = full_bar(c, s % NP);
      const uint32_t par = (s / NP) & 1u;
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(bar, par)) {
        if (globaltimer_ns() - t0 > pv.timeout_ns) break;
      }
    }
  }
}

// Returns whether this warp completed the unit (and therefore signals it).
template <int NTC, int WFC, int FEAT>
__device__ __forceinline__ bool run_unit(Ctx& c, const mk_op_t* op, const UnitArgs& u) {
  const int opcode = op->opcode;
  if constexpr (NTC >= 0) {   // NTC < 0: a kernel for programs without a matvec op
    if (opcode == MK_OP_MATVEC) return mv_dispatch<NTC, WFC, FEAT>(c, op, u);
  }
  if constexpr ((FEAT & (MK_F_AT64 | MK_F_AT128)) != 0) {
    if (opcode == MK_OP_ATTN_SPLIT) return at_dispatch<FEAT>(c, op, u);
  }
  if constexpr ((FEAT & MK_F_COMBINE) != 0) {
    if (opcode == MK_OP_ATTN_COMBINE) {
      at_combine_unit(c, op, u.unit);
      return true;
    }
  }
  if constexpr ((FEAT & MK_F_EW) != 0) {
    switch (opcode) {
      case MK_OP_RMSNORM: ew_rmsnorm(c, op, u.unit); return true;
      case MK_OP_ROPE: ew_rope(c, op, u.unit); return true;
      case MK_OP_QKNORM_ROPE: ew_qknorm_rope(c, op, u.unit); return true;
      case MK_OP_GLU: ew_glu(c, op, u.unit); return true;
      case MK_OP_ADD: ew_add(c, op, u.unit); return true;
      default: break;
    }
  }
  if constexpr ((FEAT & MK_F_TOP1) != 0) {
    if (opcode == MK_OP_TOP1_FINAL) {
      ew_top1_final(c, op, u.unit);
      return true;
    }
  }
  if constexpr ((FEAT & MK_F_AR) != 0) {
    if (opcode == MK_OP_ALLREDUCE) {
      ew_allreduce(c, op, u.unit);
      return true;
    }
  }
  if (opcode == MK_OP_NOP) return true;
  // an op this kernel variant was not built for (mk_create never selects such a variant)
  if (c.lane == 0) report(c, MK_ST_BAD_OP, opcode, u.op);
  c.dead = true;
  return true;
}

template <int NTC, int WFC, int FEAT>
__device__ void consumer_loop(Ctx& c, int ibeg, int iend, int ebeg, int eend) {
  const ProgramView& pv = *c.pv;
  const int w = c.warp - 1;
  constexpr int T = kConsumerWarps * 32;
  const int NP = pv.n_pages;
  uint32_t mv_ord = 0;  // shared units before the cursor (selects the split-K slot set)
  int staged_key = 0;
  int cached_op = -1;                  // op whose record sits in shared memory
  const mk_op_t* cached_rec = nullptr;
  uint32_t* bulk_done = nullptr;
  int bulk_units = 0;                  // > 0: units of cached_op are signalled in bulk

  // Consumer slots are handed out through a ticket counter: a unit owns as
  // many consecutive tickets as it has participants (one for a unit that is
  // not shared), and a consumer that becomes free draws the next ticket, so a
  // warp that is held up (by an epilogue, by a page that is late) never has
  // a fixed share of later work waiting behind it.  Tickets rise, so each
  // consumer walks the instruction list forward only; passing an op-entry
  // event on the way means taking part in it.
  int i = ibeg;          // instruction under the cursor
  int base = ibeg;       // `mine` holds the records of [base, base + 32)
  uint32_t first_slot = 0;  // ticket of the first slot of instruction i
  RingPos rp_i;             // ring position of the first page of instruction i
  rp_i.slot = 0;
  rp_i.k = 0;
  InsRegs mine = empty_instr();
  if (base + c.lane < iend) mine = load_instr(pv.instrs + base + c.lane);

  // An event record is held one word per lane (mk_event_t is 16 words); its
  // position alone is kept in a register of its own.
  int ev = ebeg;
  auto load_ev = [&](int e) -> int {
    return e < eend ? reinterpret_cast<const int32_t*>(pv.events + e)[c.lane & 15] : 0;
  };
  int cur_w = load_ev(ev);
  int cur_pos = ev < eend ? __shfl_sync(0xffffffffu, cur_w, 0) : 0x7fffffff;
  // the record of the first event's op goes into slot 0 before this warp can reach that event's barrier
  if (w == 1 && ev < eend) {
    const int op0 = __shfl_sync(0xffffffffu, cur_w, 1);
    if (c.lane < (int)(sizeof(mk_op_t) / 16))
      reinterpret_cast<uint4*>(&c.ctrl->op_cache[0])[c.lane] = reinterpret_cast<const uint4*>(pv.ops + op0)[c.lane];
  }

  auto do_event = [&]() {
    // Every consumer warp runs this, dead or not: the barriers must balance.
    const int k = ev - ebeg;
    const int e_op = __shfl_sync(0xffffffffu, cur_w, 1);
    const int e_nw = __shfl_sync(0xffffffffu, cur_w, 2);
    const int e_woff = __shfl_sync(0xffffffffu, cur_w, 3);
    const int e_flags = __shfl_sync(0xffffffffu, cur_w, 4);
    const int e_bulk = __shfl_sync(0xffffffffu, cur_w, 5);
    trace(c, TRC_EVENT_BEGIN, e_op);
    // request the next event record now: its latency hides behind the barrier
    const int nxt_w = load_ev(ev + 1);
    // refill the instruction window here, off the critical path, when it is half used
    if (i - base >= 16) {
      base = i;
      mine = empty_instr();
      if (base + c.lane < iend) mine = load_instr(pv.instrs + base + c.lane);
    }
    // The first warp to arrive polls the producers' counters while the others
    // finish their units of the previous op.
    int first = 0;
    if (c.lane == 0) first = atomicAdd(&c.ctrl->ev_arrive, 1u) == (uint32_t)k * kConsumerWarps;
    first = __shfl_sync(0xffffffffu, first, 0);
    if (first) wait_event(c, cur_w, e_nw, e_woff);
    // All units before the event are complete after this barrier, and so are the op's producers.
    named_bar_sync(kConsumerBarrier, T);
    trace(c, TRC_EVENT_DEPS, e_op);
    const mk_op_t* op = &c.ctrl->op_cache[k & 1];
    // warp 1 requests the record of the next event's op: it lands while the activations are staged
    const bool have_next = ev + 1 < eend;
    uint4 nrec = make_uint4(0, 0, 0, 0);
    if (w == 1 && have_next) {
      const int nop = __shfl_sync(0xffffffffu, nxt_w, 1);
      if (c.lane < (int)(sizeof(mk_op_t) / 16)) nrec = reinterpret_cast<const uint4*>(pv.ops + nop)[c.lane];
    }
    bulk_units = (e_flags & MK_EVF_BULK_SIGNAL) ? e_bulk : 0;
    bulk_done = &c.ctrl->bulk_done[k & 1];
    cached_op = e_op;
    cached_rec = op;
    if constexpr (NTC >= 0) {
      if (op->opcode == MK_OP_MATVEC) {
        const bool need = (op->act_key == 0) || (op->act_key != staged_key);
        // rows x chunks requested per thread and trip to L2 (see mv_stage)
        constexpr int kStageRows = NTC == 1 ? (WFC == 0 ? 1 : 2) : 4, kStageChunks = NTC == 1 ? 4 : 2;
        mv_stage<kStageRows, kStageChunks, WFC>(c, op, need, (e_flags & MK_EVF_WRITE_RES_OUT) != 0);
        staged_key = op->act_key;
      }
    }
    if (w == 1 && have_next) {
      // units of the op two events back (the slot's last user) are complete since the barrier above
      if (c.lane < (int)(sizeof(mk_op_t) / 16)) reinterpret_cast<uint4*>(&c.ctrl->op_cache[(k + 1) & 1])[c.lane] = nrec;
      if (c.lane == 0) c.ctrl->bulk_done[(k + 1) & 1] = 0;
    }
    named_bar_sync(kConsumerBarrier, T);
    trace(c, TRC_EVENT_END, e_op);
    ++ev;
    cur_w = nxt_w;
    cur_pos = ev < eend ? __shfl_sync(0xffffffffu, cur_w, 0) : 0x7fffffff;
  };

  for (;;) {
    uint32_t ticket = 0;
    if (c.lane == 0) ticket = atomicAdd(&c.ctrl->ticket, 1u);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    bool found = false;
    int n_pages = 0, lflags = 0;
    for (;;) {
      // events due before instruction i; the ones behind the last instruction are
      // taken when the cursor reaches the end of the list (every event position is
      // at most the length of the list), so this is the only place events run
      while (cur_pos <= i - ibeg) do_event();
      if (i >= iend) break;
      if (i - base >= 32) {
        base = i;
        mine = empty_instr();
        if (base + c.lane < iend) mine = load_instr(pv.instrs + base + c.lane);
      }
      n_pages = __shfl_sync(0xffffffffu, mine.n_pages, i - base);
      lflags = __shfl_sync(0xffffffffu, mine.flags, i - base);
      const bool shared = (lflags & kInsMatvec) != 0;
      int split = (lflags >> MK_LDF_SPLIT_SHIFT) & MK_LDF_SPLIT_MASK;
      if (lflags & MK_LDF_DYN) {
        // an attention unit whose window follows the device-resident position: the pages in use, and
        // with them the participants, are a function of the position (the same on every warp)
        const int t_begin = __shfl_sync(0xffffffffu, mine.row_a, i - base);
        const int brow = (__shfl_sync(0xffffffffu, mine.row_b, i - base) >> 16) & 31;
        n_pages = at_dyn_pages(t_begin, n_pages, at_page_tokens((lflags & MK_LDF_D128) ? 128 : 64, pv.page_bytes),
                               c.ctrl->pos[brow] + 1);
        split = max(1, min(split, n_pages));
        lflags = (lflags & ~(MK_LDF_SPLIT_MASK << MK_LDF_SPLIT_SHIFT)) | (split << MK_LDF_SPLIT_SHIFT);
      }
      const uint32_t slots = shared ? (uint32_t)split : 1u;
      if (ticket < first_slot + slots) {
        found = true;
        break;
      }
      first_slot += slots;
      ring_advance(rp_i, n_pages, NP);
      if (shared && split > 1) ++mv_ord;
      ++i;
    }
    if (!found) break;
    if (!c.dead) {
      const int idx = i - base;
      UnitArgs u;
      u.mine = &mine;
      u.idx = idx;
      u.op = __shfl_sync(0xffffffffu, mine.op, idx);
      u.unit = __shfl_sync(0xffffffffu, mine.unit, idx);
      u.n_pages = n_pages;
      u.flags = lflags;
      u.part = (int)(ticket - first_slot);
      u.ord = mv_ord;
      u.rp0 = rp_i;
      u.rp = rp_i;
      ring_advance(u.rp, u.part, NP);
      const int n_waits = __shfl_sync(0xffffffffu, mine.n_waits, idx);
      c.instr_idx = i;
      if (n_waits == 0 || wait_counters(c, n_waits, __shfl_sync(0xffffffffu, mine.wait_off, idx))) {
        trace(c, TRC_UNIT_BEGIN, i);
        const mk_op_t* op = u.op == cached_op ? cached_rec : pv.ops + u.op;
        const bool finished = run_unit<NTC, WFC, FEAT>(c, op, u);
        if (!c.dead && finished) {
          const int signal = __shfl_sync(0xffffffffu, mine.signal, idx);
          if (bulk_units > 0 && u.op == cached_op)
            signal_unit_bulk(c, bulk_done, signal, bulk_units);
          else
            signal_unit(c, signal);
        }
        trace(c, TRC_UNIT_END, i);
      }
    }
  }
}

// NTC / WFC specialise the matvec path (see mv_dispatch), FEAT names the other ops the
// variant carries (MK_F_*); <0, -1, MK_F_ALL> handles any program.
template <int NTC, int WFC, int FEAT>
__global__ void __launch_bounds__(kThreads, 1) mk_persistent_kernel(const __grid_constant__ ProgramView pv) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Ctx c;
  c.pv = &pv;
  c.ctrl = reinterpret_cast<Ctrl*>(smem);
  c.act = smem + kCtrlBytes;
  c.pages = smem + kCtrlBytes + pv.act_bytes;
  c.act_u32 = smem_u32(c.act);
  c.pages_u32 = smem_u32(c.pages);
  c.warp = threadIdx.x >> 5;
  c.lane = threadIdx.x & 31;
  c.instr_idx = -1;
  c.dead = false;
  trace_init<(FEAT & MK_F_TRACE) != 0>(c);

  if (threadIdx.x == 0) {
    for (int i = 0; i < pv.n_pages; ++i) {
      mbar_init(smem_u32(&c.ctrl->full[i]), 32);
      mbar_init(smem_u32(&c.ctrl->empty[i]), 1);
    }
    for (int i = 0; i < kMaxPages; ++i) c.ctrl->released[i] = 0;
    for (int i = 0; i < 4; ++i) c.ctrl->mv_arrive[i] = c.ctrl->mv_done[i] = 0;
    c.ctrl->abort_flag = 0;
    c.ctrl->is_last = 0;
    c.ctrl->ticket = 0;
    c.ctrl->ev_arrive = 0;
    c.ctrl->pos_bad = 0;
    c.ctrl->bulk_done[0] = c.ctrl->bulk_done[1] = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // one position per batch row (or one for all): a warp reads them side by side
    int v = 0;
    if (pv.dyn_pos != nullptr) {
      v = reinterpret_cast<const volatile int32_t*>(pv.dyn_pos)[min((int)threadIdx.x, pv.pos_count - 1)];
      if ((int)threadIdx.x < pv.pos_count && (uint32_t)v >= (uint32_t)pv.pos_limit) c.ctrl->pos_bad = 1 + (int)threadIdx.x;
    }
    c.ctrl->pos[threadIdx.x] = v;
  }
  __syncthreads();

  const int ibeg = pv.cta_instr_begin[blockIdx.x], iend = pv.cta_instr_begin[blockIdx.x + 1];
  const int ebeg = pv.cta_event_begin[blockIdx.x], eend = pv.cta_event_begin[blockIdx.x + 1];
  // A position outside the caches the program was scheduled for would write past them: every CTA
  // reads the same values, so all of them skip the program together and the launch ends at once.
  const int bad_pos = c.ctrl->pos_bad;          // 1 + the batch row of an offending position
  if (bad_pos) {
    if (threadIdx.x == 0) report(c, MK_ST_BAD_POSITION, c.ctrl->pos[bad_pos - 1], pv.pos_limit);
  } else if (c.warp == 0) {
    loader_loop(c, ibeg, iend);
  } else {
    consumer_loop<NTC, WFC, FEAT>(c, ibeg, iend, ebeg, eend);
  }
  trace_flush(c);
  __syncthreads();

  // The last CTA to finish clears the dependency counters, so the next launch
  // (or graph replay) starts from zero without a host-side memset.
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(&pv.state->done_ctas, 1);
    c.ctrl->is_last = (prev == (int)gridDim.x - 1) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  if (c.ctrl->is_last) {
    const bool ok = *reinterpret_cast<volatile int32_t*>(&pv.state->abort_flag) == 0;
    if (ok)
      for (int i = threadIdx.x; i < pv.n_counters; i += blockDim.x) pv.counters[i] = 0;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      pv.state->done_ctas = 0;
      pv.state->launches += 1;
    }
  }
}

}  // namespace mk

// One compiled kernel: <activation-tile class, weight family, features>.
typedef void (*mk_kernel_fn)(const mk::ProgramView);
struct mk_variant {
  int ntc, wfc, feat;
  mk_kernel_fn fn;
};
