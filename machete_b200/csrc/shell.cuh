// Persistent-kernel shell: shared-memory map, page ring, bounded waits and the
// device-visible program view.  This is the build's counterpart of the
// reference's ring loop and smem layout (megakernel/replay_loops.py:27-824,
// megakernel/paged_memory.py:270-434), with a different division of labour:
// one loader warp streams pages for *all* upcoming work units of the CTA, and
// each consumer warp owns whole units, so no intra-unit cross-warp sync exists.
#pragma once
#include "../../include/machete_b200.h"
#include "prims.cuh"

namespace mk {

// 1 loader + 7 consumers = 8 warps, two per SM sub-partition: each thread may
// then use up to 255 registers (9 warps would put 3 on one sub-partition and
// cap the whole kernel at 168, which spilled).
constexpr int kConsumerWarps = 7;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxPages = 32;
constexpr int kCtrlStructBytes = 4096;  // mbarriers + flags + reduction scratch
// Split-K partial accumulators of the matvec units: one slot per consumer warp
// (32 lanes x 4 floats per activation n-tile), kPartialBytes in all.
constexpr int kPartialBytes = kConsumerWarps * 2048;
constexpr int kCtrlBytes = kCtrlStructBytes + kPartialBytes;
constexpr uint32_t kConsumerBarrier = 1;

// What a kernel variant is built to run (template parameter FEAT).  A program
// needs the union of its ops' features; mk_create picks the smallest variant
// that covers it.
enum {
  MK_F_AT64 = 1,     // split-KV attention, head dim 64
  MK_F_AT128 = 2,    // split-KV attention, head dim 128
  MK_F_QKNORM = 4,   // attention with the fused per-head q/k RMSNorm + rotation
  MK_F_EW = 8,       // the row-wise ops: RMSNorm, RoPE, QK-norm + RoPE, GLU, add
  MK_F_COMBINE = 16, // the stand-alone log-sum-exp combine op
  MK_F_AR = 32,      // the in-kernel all-reduce (tensor parallel)
  MK_F_TOP1 = 64,    // top-1 epilogue and its finalise op
  MK_F_TRACE = 128,  // event trace
  MK_F_ALL = 255
};

// Device status codes (status[0]).
enum {
  MK_ST_OK = 0,
  MK_ST_TIMEOUT_COUNTER = 1,  // dependency counter never reached `expected`
  MK_ST_TIMEOUT_PAGE_FULL = 2,
  MK_ST_TIMEOUT_PAGE_EMPTY = 3,
  MK_ST_BAD_OP = 4,
  MK_ST_TIMEOUT_PAGE_TURN = 5,  // earlier fills of a ring slot were never handed back
  MK_ST_TIMEOUT_PEER = 6,       // a peer rank's all-reduce flag never arrived
  MK_ST_BAD_POSITION = 7        // the device-resident cache position is outside [0, position_limit): nothing ran
};

// Device memory block owned by a handle (lives in the caller's workspace).
struct DeviceState {
  int32_t status[16];   // [0] code, [1] cta, [2] instr, [3] aux, [4] aux2
  int32_t abort_flag;   // set by the first CTA that times out
  int32_t done_ctas;    // CTAs that finished this launch
  int32_t launches;     // completed launches
  int32_t pad[13];
};

struct ProgramView {
  const mk_op_t* ops;
  const mk_instr_t* instrs;
  const int32_t* cta_instr_begin;
  const mk_event_t* events;
  const int32_t* cta_event_begin;
  const mk_wait_t* waits;
  int32_t* counters;
  DeviceState* state;
  int32_t n_counters;
  int32_t n_pages;
  int32_t page_bytes;
  int32_t act_bytes;
  uint64_t timeout_ns;
  // optional event trace: per (CTA, warp) a ring of trace_cap records, then
  // one record count per (CTA, warp) after all rings; null = tracing off
  struct TraceRec* trace;
  int32_t trace_cap;
  int32_t mv_sets;  // split-K slot sets in use: 4 (every matvec has M <= 8), 2 (M <= 16) or 1
  const int32_t* dyn_pos;  // device-resident cache position, or null
  int32_t pos_limit;       // positions >= this end the launch with MK_ST_BAD_POSITION before any op runs
  int32_t pos_count;       // entries behind dyn_pos: 1 (one position for every batch row) or one per row (<= 32)
};

// One trace event: a globaltimer stamp, an event code and an argument.
struct TraceRec {
  uint64_t t;
  uint32_t code;
  uint32_t arg;
};
enum {
  TRC_LOAD_BEGIN = 1,   // loader: ring slot free, about to issue (arg = ring seq)
  TRC_LOAD_ISSUED = 2,  // loader: copies issued (arg = ring seq)
  TRC_PAGE_READY = 3,   // consumer: page data visible (arg = ring seq)
  TRC_PAGE_DONE = 4,    // consumer: page handed back (arg = ring seq)
  TRC_UNIT_BEGIN = 5,   // consumer: unit starts (arg = instruction index)
  TRC_UNIT_END = 6,     // consumer: unit signalled (arg = instruction index)
  TRC_EVENT_BEGIN = 7,  // consumers meet at an op-entry event (arg = op)
  TRC_EVENT_DEPS = 8,   // event: producers complete (arg = op)
  TRC_EVENT_END = 9,    // event: activations staged (arg = op)
  TRC_LWAIT_DONE = 10,  // loader: loader-side wait satisfied (arg = instruction index)
  TRC_PAGE_CYCLES = 11, // consumer: SM cycles spent computing on the page just handed back (arg = cycles)
  TRC_MV_ARRIVED = 12,  // consumer: split-K partial handed in (arg = slot-set ordinal)
  TRC_MV_REDUCED = 13,  // consumer: partials of the unit summed, epilogue starts (arg = ordinal)
  TRC_MV_EPILOGUE = 14, // consumer: epilogue stores issued (arg = ordinal)
  TRC_AT_COUNTED = 15,  // attention: this split counted in (arg = 1 when it completes its group)
  TRC_AT_FETCHED = 16,  // attention combine: first batch of partials accumulated (arg = row pass)
  TRC_SYNC_CLOCK = 30,  // time base: t = the SM's cycle counter ...
  TRC_SYNC_NS = 31      // ... and t = the nanosecond timer at the same moment
};

// Shared-memory control block (first kCtrlBytes of dynamic smem).
struct Ctrl {
  uint64_t full[kMaxPages];
  uint64_t empty[kMaxPages];
  int32_t abort_flag;
  int32_t is_last;
  // Split-K slot sets: arrivals of the current user, and how many users of
  // the set have finished their epilogue.
  uint32_t mv_arrive[4];
  uint32_t mv_done[4];
  // units of an op finished on this CTA (bulk signalling); one word per op-record slot
  uint32_t bulk_done[2];
  uint32_t ticket;     // next consumer slot of the CTA (see consumer_loop)
  uint32_t ev_arrive;  // consumer warps that have reached an op-entry event (kConsumerWarps per event)
  int32_t pos_bad;     // a device-resident cache position was outside [0, pos_limit) when the launch started
  int32_t pad[1];
  // the device-resident cache position of every batch row as read when the launch started (all rows
  // share one value when the program has a single position; 0 without one)
  int32_t pos[32];
  // released[slot] = number of fills of the slot that consumers have handed back
  uint32_t released[kMaxPages];
  // per activation row and consumer warp: sum of squares of the staged row (RMSNorm)
  float red[kConsumerWarps * 32];
  float rstd[32];   // per activation row: the RMSNorm scale (two-pass staging only)
  // Records of the op the CTA is working on and of the op of its next op-entry
  // event (event k uses slot k & 1; the other slot is refilled one event ahead,
  // so an event never waits for its op record).
  __align__(16) mk_op_t op_cache[2];
};
static_assert(sizeof(Ctrl) <= kCtrlStructBytes, "control block too large");

// Per-thread execution context.
struct Ctx {
  const ProgramView* pv;
  Ctrl* ctrl;
  uint8_t* act;       // staged activations
  uint8_t* pages;     // page ring base
  uint32_t pages_u32; // shared-space address of the ring
  uint32_t act_u32;
  int warp;           // 0 = loader, 1.. = consumers
  int lane;
  int instr_idx;      // global index of the instruction being executed
  bool dead;          // a wait expired somewhere: skip work, keep barriers
  int trace_n;        // records this warp has written
  int trace_cap;
  TraceRec* trace_base;  // this warp's trace ring (lane 0 only), null = off
};

// The consumers' registers for one instruction record (one record per lane of
// a 32-record window; fields are fetched from the owning lane by shuffle).
struct InsRegs {
  int op, unit, signal, n_waits, wait_off, n_pages;
  int flags;                       // ld_flags, bit 31 = unit shared page by page
  int row_a, row_b, off_a, off_b;  // see mk_instr_t
};

// Position of a ring entry: slot index and how many times the slot was filled
// before (seq = k * n_pages + slot).  Kept incrementally, never divided.
struct RingPos {
  uint32_t slot, k;
};

// What the shell hands to a unit handler.
struct UnitArgs {
  const InsRegs* mine;  // the warp's instruction window
  int idx;              // lane of the window that holds this unit's record
  int op, unit, n_pages, flags;
  int part;             // this consumer's participant index within the unit
  uint32_t ord;         // shared units before this one on the CTA (selects the split-K slot set)
  RingPos rp0;          // ring position of the unit's first page
  RingPos rp;           // ring position of this participant's first page
};
__device__ __forceinline__ int ins_field(const int& field_of_mine, int idx) {
  return __shfl_sync(0xffffffffu, field_of_mine, idx);
}

// What a non-inlined unit handler hands back to the shell.
struct UnitResult {
  bool dead;
  bool signal;  // this warp finished the unit: it signals the unit's counter
  int trace_n;
};

// The per-warp ring base is resolved once at kernel start (null = tracing
// off), so a disabled trace point costs one predicated branch.  Records are
// stamped with the SM's cycle counter, which costs a few cycles to read (the
// nanosecond timer costs a fraction of a microsecond, enough to distort what
// is being measured); every ring opens and closes with a pair of records that
// hold the cycle counter and the nanosecond timer at the same moment, from
// which the host maps cycles to a time base common to all CTAs.
__device__ __forceinline__ uint64_t sm_clock() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_sync_pair(Ctx& c) {
  if (c.trace_n + 2 <= c.trace_cap) {
    TraceRec* r = c.trace_base + c.trace_n;
    r[0].t = sm_clock();
    r[0].code = TRC_SYNC_CLOCK;
    r[0].arg = 0;
    r[1].t = globaltimer_ns();
    r[1].code = TRC_SYNC_NS;
    r[1].arg = 0;
  }
  c.trace_n += 2;
}
template <bool TRACED>
__device__ __forceinline__ void trace_init(Ctx& c) {
  c.trace_n = 0;
  c.trace_cap = 0;
  c.trace_base = nullptr;   // stays null in a kernel built without tracing: every trace point folds away
  TraceRec* base = TRACED ? c.pv->trace : nullptr;
  if (TRACED && base != nullptr && c.lane == 0) {
    c.trace_cap = c.pv->trace_cap - 2;   // room for the closing pair
    c.trace_base = base + ((size_t)blockIdx.x * (kConsumerWarps + 1) + c.warp) * c.pv->trace_cap;
    trace_sync_pair(c);
  }
}
__device__ __forceinline__ void trace(Ctx& c, uint32_t code, uint32_t arg) {
  if (c.trace_base == nullptr) return;
  if (c.trace_n < c.trace_cap) {
    TraceRec* r = c.trace_base + c.trace_n;
    r->t = sm_clock();
    r->code = code;
    r->arg = arg;
  }
  ++c.trace_n;
}
__device__ __forceinline__ void trace_flush(Ctx& c) {
  if (c.trace_base == nullptr) return;
  if (c.trace_n > c.trace_cap) c.trace_n = c.trace_cap;   // overflowed: the closing pair goes into the reserve
  c.trace_cap += 2;
  trace_sync_pair(c);
  int32_t* counts = reinterpret_cast<int32_t*>(c.pv->trace + (size_t)gridDim.x * (kConsumerWarps + 1) * c.pv->trace_cap);
  counts[blockIdx.x * (kConsumerWarps + 1) + c.warp] = c.trace_n;
}

// Error reporting and the give-up decision live out of line: they run only
// after a wait has already spun for a while, and every bounded wait would
// otherwise carry a copy of them (the kernel's code size is what its op
// boundaries pay for in instruction-cache misses).
static __device__ __noinline__ void report_slow(const ProgramView* pv, Ctrl* ctrl, int instr_idx, int warp, int code,
                                                int aux, int aux2) {
  DeviceState* st = pv->state;
  if (atomicCAS(&st->status[0], 0, code) == 0) {
    st->status[1] = blockIdx.x;
    st->status[2] = instr_idx;
    st->status[3] = aux;
    st->status[4] = aux2;
    st->status[5] = warp;
  }
  atomicExch(&st->abort_flag, 1);
  atomicExch(&ctrl->abort_flag, 1);
  __threadfence();
}
__device__ __forceinline__ void report(Ctx& c, int code, int aux, int aux2) {
  report_slow(c.pv, c.ctrl, c.instr_idx, c.warp, code, aux, aux2);
}

// One thread's view: 1 = stop waiting (abort seen, or the time budget since *t0 is
// spent, which is reported); *t0 == 0 starts the clock.
static __device__ __noinline__ int expired_slow(const ProgramView* pv, Ctrl* ctrl, uint64_t* t0, int instr_idx, int warp,
                                                int code, int aux, int aux2) {
  if (*reinterpret_cast<volatile int32_t*>(&ctrl->abort_flag)) return 1;
  if (*reinterpret_cast<volatile int32_t*>(&pv->state->abort_flag)) {
    atomicExch(&ctrl->abort_flag, 1);
    return 1;
  }
  const uint64_t now = globaltimer_ns();
  if (*t0 == 0) {
    *t0 = now;
    return 0;
  }
  if (now - *t0 > pv->timeout_ns) {
    report_slow(pv, ctrl, instr_idx, warp, code, aux, aux2);
    return 1;
  }
  return 0;
}

__device__ __forceinline__ bool aborted(Ctx& c) {
  if (*reinterpret_cast<volatile int32_t*>(&c.ctrl->abort_flag)) return true;
  if (*reinterpret_cast<volatile int32_t*>(&c.pv->state->abort_flag)) {
    atomicExch(&c.ctrl->abort_flag, 1);
    return true;
  }
  return false;
}

// Slow path shared by the warp-wide bounded waits: lane 0 decides whether to
// give up and the decision is broadcast.
__device__ __forceinline__ bool give_up_check(Ctx& c, uint64_t& t0, int code, int aux, int aux2) {
  int give_up = 0;
  if (c.lane == 0) give_up = expired_slow(c.pv, c.ctrl, &t0, c.instr_idx, c.warp, code, aux, aux2);
  return __shfl_sync(0xffffffffu, give_up, 0) != 0;
}

// Wait until the mbarrier phase with `parity` has completed.  All lanes of
// the warp call this together and all observe the phase themselves.  The
// fast path is one try_wait plus one vote; the outcome is warp-uniform.
// Returns false (and marks the context dead) when the wait is abandoned.
__device__ __forceinline__ bool wait_mbar(Ctx& c, uint32_t bar, uint32_t parity, int code, int aux) {
  if (c.dead) return false;
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    }
    if (give_up_check(c, t0, code, aux, (int)parity)) {
      c.dead = true;
      return false;
    }
  }
}

// The same wait for a single thread (the loader's lane 0).  On give-up the
// abort flag is raised; the caller's warp learns of it at its next __syncwarp.
__device__ __forceinline__ bool wait_mbar_one(Ctx& c, uint32_t bar, uint32_t parity, int code, int aux) {
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (expired_slow(c.pv, c.ctrl, &t0, c.instr_idx, c.warp, code, aux, (int)parity)) return false;
  }
}

// Wait for every (counter >= expected) pair of a wait list.  Lane 0 polls;
// the warp reconverges afterwards.  Out of line: the op-entry events carry
// their waits inline (wait_event), so this runs only for unit-level waits,
// the loader's waits for rows appended in the same launch, and long lists.
static __device__ __noinline__ int wait_counters_slow(const ProgramView* pv, Ctrl* ctrl, int instr_idx, int warp, int n,
                                                      int off) {
  const mk_wait_t* w = pv->waits + off;
  for (int i = 0; i < n; ++i) {
    const int32_t* ctr = pv->counters + w[i].counter;
    const int32_t expected = w[i].expected;
    uint64_t t0 = 0;
    for (int spin = 0; ld_acquire_gpu(ctr) < expected; ++spin) {
      nanosleep(32);
      if ((spin & 15) == 15 && expired_slow(pv, ctrl, &t0, instr_idx, warp, MK_ST_TIMEOUT_COUNTER, w[i].counter, expected))
        return 0;
    }
  }
  return 1;
}
__device__ __forceinline__ bool wait_counters(Ctx& c, int n, int off) {
  if (c.dead) return false;
  int ok = 1;
  if (c.lane == 0 && n > 0) ok = wait_counters_slow(c.pv, c.ctrl, c.instr_idx, c.warp, n, off);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) c.dead = true;
  return ok != 0;
}

__device__ __forceinline__ uint32_t full_bar(Ctx& c, int slot) { return smem_u32(&c.ctrl->full[slot]); }
__device__ __forceinline__ uint32_t empty_bar(Ctx& c, int slot) { return smem_u32(&c.ctrl->empty[slot]); }

// Consumer warps run independently of one another, so a warp may ask for fill
// k of a slot while the slot is still two or more fills behind; an mbarrier
// only tells odd from even phases.  Waiting first until the k previous fills
// have been handed back pins the full-barrier to phase k (pending) or k + 1
// (complete), where the parity test is unambiguous.
__device__ __forceinline__ bool wait_released(Ctx& c, uint32_t slot, uint32_t k, int aux) {
  if (c.dead) return false;
  volatile uint32_t* r = &c.ctrl->released[slot];
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (__all_sync(0xffffffffu, *r >= k)) return true;
      nanosleep(40);
    }
    if (give_up_check(c, t0, MK_ST_TIMEOUT_PAGE_TURN, aux, (int)k)) {
      c.dead = true;
      return false;
    }
  }
}

__device__ __forceinline__ RingPos ring_at(uint32_t seq, int np) {
  RingPos r;
  r.k = seq / (uint32_t)np;
  r.slot = seq - r.k * (uint32_t)np;
  return r;
}
// Step `stride` entries ahead.
__device__ __forceinline__ void ring_advance(RingPos& r, int stride, int np) {
  r.slot += (uint32_t)stride;
  while (r.slot >= (uint32_t)np) {
    r.slot -= (uint32_t)np;
    ++r.k;
  }
}
__device__ __forceinline__ void ring_next(RingPos& r, int np) {
  if (++r.slot == (uint32_t)np) {
    r.slot = 0;
    ++r.k;
  }
}

// Pages in use of a split-KV attention unit whose window follows the cache
// position: `limit` pages of `tn` tokens were scheduled for tokens
// [t_begin, ...); the window ends at token `n_tokens`.
__device__ __forceinline__ int at_dyn_pages(int t_begin, int limit, int tn, int n_tokens) {
  const int left = n_tokens - t_begin;
  if (left <= 0) return 0;
  const int need = (left + tn - 1) >> (__ffs(tn) - 1);   // tn is 32 or 64 (at_page_tokens)
  return need < limit ? need : limit;
}

// Consumer side: wait until the ring entry holds data; returns its address.
__device__ __forceinline__ bool page_acquire(Ctx& c, const RingPos& r, uint32_t& page_addr) {
  page_addr = c.pages_u32 + r.slot * (uint32_t)c.pv->page_bytes;
  if (r.k > 0 && !wait_released(c, r.slot, r.k, (int)r.slot)) return false;
  return wait_mbar(c, full_bar(c, r.slot), r.k & 1u, MK_ST_TIMEOUT_PAGE_FULL, (int)r.slot);
}
// Consumer side: hand the ring entry back to the loader.
__device__ __forceinline__ void page_release(Ctx& c, const RingPos& r) {
  __syncwarp();
  if (c.lane == 0) {
    mbar_arrive(empty_bar(c, r.slot));
    *reinterpret_cast<volatile uint32_t*>(&c.ctrl->released[r.slot]) = r.k + 1u;
  }
}

// Signal completion of a work unit: all lanes' global writes are ordered
// before the counter increment.
__device__ __forceinline__ void signal_unit(Ctx& c, int counter) {
  __syncwarp();
  if (c.lane == 0 && counter >= 0) {
    // release at gpu scope is cumulative: it also publishes the other lanes'
    // writes that the __syncwarp above ordered before this point
    red_release_gpu_add(c.pv->counters + counter, 1);
  }
}


// Bounded wait until a shared-memory word reaches `want`.
__device__ __forceinline__ bool wait_smem_ge(Ctx& c, volatile uint32_t* word, uint32_t want, int aux) {
  if (c.dead) return false;
  uint64_t t0 = 0;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (__all_sync(0xffffffffu, *word >= want)) return true;
      nanosleep(20);
    }
    if (give_up_check(c, t0, MK_ST_TIMEOUT_PAGE_TURN, aux, (int)want)) {
      c.dead = true;
      return false;
    }
  }
}

// Bulk variant: the unit's finisher counts it in shared memory; whoever counts
// the CTA's last unit of the op publishes all of them with one device-scope
// release (the earlier finishers' writes reach it through the cta-scope
// fences around the shared-memory counter).
__device__ __forceinline__ void signal_unit_bulk(Ctx& c, uint32_t* done, int counter, int units) {
  __syncwarp();
  if (c.lane == 0 && counter >= 0) {
    __threadfence_block();
    const uint32_t old = atomicAdd(done, 1u);
    if (old == (uint32_t)(units - 1)) {
      __threadfence_block();
      red_release_gpu_add(c.pv->counters + counter, units);   // the release is the device-scope fence
    }
  }
}

// The wait that opens a dependency stage.  `ev_word` is the event record held
// one 32-bit word per lane (mk_event_t is 16 words): lanes 0-3 poll the four
// inline (counter, expected) pairs side by side; longer lists continue in the
// wait table.
__device__ __forceinline__ bool wait_event(Ctx& c, int ev_word, int n, int off) {
  if (c.dead) return false;
  if (n <= 0) return true;
  const int my_c = __shfl_sync(0xffffffffu, ev_word, 6 + (c.lane & 3));
  const int my_e = __shfl_sync(0xffffffffu, ev_word, 10 + (c.lane & 3));
  const bool mine = c.lane < (n < 4 ? n : 4);
  const int32_t* ctr = c.pv->counters + (mine ? my_c : 0);
  uint64_t t0 = 0;
  for (int spin = 0;; ++spin) {
    // Every poll is an acquire load: the one that sees the counter complete closes
    // the wait with no further trip to L2 (polling relaxed and acquiring once at the
    // end costs that extra trip on every op boundary).
    const bool ok = !mine || ld_acquire_gpu(ctr) >= my_e;
    if (__all_sync(0xffffffffu, ok)) break;
    if ((spin & 15) == 15 && give_up_check(c, t0, MK_ST_TIMEOUT_COUNTER, my_c, my_e)) {
      c.dead = true;
      return false;
    }
  }
  if (n > 4) return wait_counters(c, n - 4, off + 4);
  return true;
}

}  // namespace mk
