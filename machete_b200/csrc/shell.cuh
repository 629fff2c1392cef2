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

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxPages = 32;
constexpr int kCtrlBytes = 4096;  // mbarriers + flags + reduction scratch
constexpr uint32_t kConsumerBarrier = 1;

// Device status codes (status[0]).
enum {
  MK_ST_OK = 0,
  MK_ST_TIMEOUT_COUNTER = 1,  // dependency counter never reached `expected`
  MK_ST_TIMEOUT_PAGE_FULL = 2,
  MK_ST_TIMEOUT_PAGE_EMPTY = 3,
  MK_ST_BAD_OP = 4,
  MK_ST_TIMEOUT_PAGE_TURN = 5  // earlier fills of a ring slot were never handed back
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
};

// Shared-memory control block (first kCtrlBytes of dynamic smem).
struct Ctrl {
  uint64_t full[kMaxPages];
  uint64_t empty[kMaxPages];
  int32_t abort_flag;
  int32_t is_last;
  int32_t pad[14];
  // released[slot] = number of fills of the slot that consumers have handed back
  uint32_t released[kMaxPages];
  float red[kConsumerWarps * 32];  // block-reduction scratch (per row, per warp)
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

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
};

__device__ __forceinline__ void report(Ctx& c, int code, int aux, int aux2) {
  DeviceState* st = c.pv->state;
  if (atomicCAS(&st->status[0], 0, code) == 0) {
    st->status[1] = blockIdx.x;
    st->status[2] = c.instr_idx;
    st->status[3] = aux;
    st->status[4] = aux2;
    st->status[5] = c.warp;
  }
  atomicExch(&st->abort_flag, 1);
  atomicExch(&c.ctrl->abort_flag, 1);
  __threadfence();
}

__device__ __forceinline__ bool aborted(Ctx& c) {
  if (*reinterpret_cast<volatile int32_t*>(&c.ctrl->abort_flag)) return true;
  if (*reinterpret_cast<volatile int32_t*>(&c.pv->state->abort_flag)) {
    atomicExch(&c.ctrl->abort_flag, 1);
    return true;
  }
  return false;
}

// Wait until the mbarrier phase with `parity` has completed.  All lanes of
// the warp call this together.  Returns false (and marks the context dead)
// when the wait is abandoned.
__device__ __forceinline__ bool wait_mbar(Ctx& c, uint32_t bar, uint32_t parity, int code, int aux) {
  if (c.dead) return false;
  // The outcome must be warp-uniform (callers shuffle and __syncwarp right
  // after), so success needs every lane to have observed the phase and the
  // give-up decision is taken by lane 0 alone and broadcast.
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    }
    int give_up = 0;
    if (c.lane == 0) {
      if (aborted(c)) {
        give_up = 1;
      } else if (globaltimer_ns() - t0 > c.pv->timeout_ns) {
        report(c, code, aux, (int)parity);
        give_up = 1;
      }
    }
    give_up = __shfl_sync(0xffffffffu, give_up, 0);
    if (give_up) {
      c.dead = true;
      return false;
    }
  }
}

// Wait for every (counter >= expected) pair of a wait list.  Lane 0 polls;
// the warp reconverges afterwards.
__device__ __forceinline__ bool wait_counters(Ctx& c, int n, int off) {
  if (c.dead) return false;
  int ok = 1;
  if (c.lane == 0 && n > 0) {
    const mk_wait_t* w = c.pv->waits + off;
    for (int i = 0; i < n && ok; ++i) {
      const int32_t* ctr = c.pv->counters + w[i].counter;
      const int32_t expected = w[i].expected;
      if (ld_acquire_gpu(ctr) >= expected) continue;
      const uint64_t t0 = globaltimer_ns();
      for (;;) {
        bool hit = false;
#pragma unroll 1
        for (int k = 0; k < 16; ++k) {
          if (ld_acquire_gpu(ctr) >= expected) {
            hit = true;
            break;
          }
          nanosleep(32);
        }
        if (hit) break;
        if (aborted(c)) {
          ok = 0;
          break;
        }
        if (globaltimer_ns() - t0 > c.pv->timeout_ns) {
          report(c, MK_ST_TIMEOUT_COUNTER, w[i].counter, expected);
          ok = 0;
          break;
        }
      }
    }
  }
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
  if (__all_sync(0xffffffffu, *r >= k)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (__all_sync(0xffffffffu, *r >= k)) return true;
      nanosleep(20);
    }
    int give_up = 0;
    if (c.lane == 0) {
      if (aborted(c)) {
        give_up = 1;
      } else if (globaltimer_ns() - t0 > c.pv->timeout_ns) {
        report(c, MK_ST_TIMEOUT_PAGE_TURN, aux, (int)k);
        give_up = 1;
      }
    }
    give_up = __shfl_sync(0xffffffffu, give_up, 0);
    if (give_up) {
      c.dead = true;
      return false;
    }
  }
}

// Consumer side: wait until ring entry `seq` holds data; returns its address.
__device__ __forceinline__ bool page_acquire(Ctx& c, uint32_t seq, uint32_t& page_addr) {
  const int np = c.pv->n_pages;
  const uint32_t slot = seq % np;
  const uint32_t k = seq / np;
  page_addr = c.pages_u32 + slot * (uint32_t)c.pv->page_bytes;
  if (k > 0 && !wait_released(c, slot, k, (int)seq)) return false;
  return wait_mbar(c, full_bar(c, slot), k & 1u, MK_ST_TIMEOUT_PAGE_FULL, (int)seq);
}
// Consumer side: hand ring entry `seq` back to the loader.
__device__ __forceinline__ void page_release(Ctx& c, uint32_t seq) {
  __syncwarp();
  if (c.lane == 0) {
    const int np = c.pv->n_pages;
    const uint32_t slot = seq % np;
    mbar_arrive(empty_bar(c, slot));
    __threadfence_block();
    *reinterpret_cast<volatile uint32_t*>(&c.ctrl->released[slot]) = seq / np + 1u;
  }
}

// Signal completion of a work unit: all lanes' global writes are ordered
// before the counter increment.
__device__ __forceinline__ void signal_unit(Ctx& c, int counter) {
  __syncwarp();
  if (c.lane == 0 && counter >= 0) {
    __threadfence();
    red_release_gpu_add(c.pv->counters + counter, 1);
  }
}

}  // namespace mk
