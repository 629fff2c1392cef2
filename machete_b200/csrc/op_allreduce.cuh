// One-shot all-reduce over peer-mapped inboxes, inside the decode kernel.
//
// Tensor parallelism splits the O-projection and the down projection by K, so
// every rank holds a partial [rows, hidden] sum that must be added across
// ranks before the next op (2 exchanges per layer), and the vocabulary-split LM
// head leaves one (max, argmax) key per rank and row.  The payload is a few
// KB, so the exchange is latency-bound: each rank *pushes* its partial straight
// into every peer's inbox with plain peer stores over NVLink, raises a flag
// there, waits (bounded) for the peers' flags in its own memory and adds the
// inbox slots in rank order, which makes the result bit-identical on all ranks.
// No collective library call, no extra launch, no multicast.
//
// Stands in for the reference's GemmRowParallelOp peer reduce-store and peer
// barriers (kernels/gemm/gemm.py:1253-1363), which run P ranks in one process.
//
// Layout of the symmetric buffer (same offsets on every rank):
//   inbox: two buffers of [P][n] 8-byte words, slot r written by rank r.  For
//          sums a word is {fp32 value, epoch}: the data carries its own flag.
//          For keys a word is the 64-bit key, guarded by
//   flags: [P][units] u32, flag (r, u) = epoch of the last launch whose unit u
//          of rank r has been delivered (keys only)
// A launch uses epoch = epoch_base + launches + 1 and waits for flags >= epoch,
// so flags never need a reset.  A peer can run at most one launch ahead of
// this rank at the same op (it needs this rank's next contribution to go
// further), so the inbox is double-buffered by the parity of the epoch.
#pragma once
#include "shell.cuh"

namespace mk {

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Inbox data was written by a peer GPU: read it past the L1 cache.
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_sys_u2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u2(uint2* p, uint2 v) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Wait until the peers' flags of `unit` in this rank's memory reach `epoch`:
// lane r polls rank r's flag.  Bounded like every other wait of the kernel.
__device__ __forceinline__ bool ar_wait_flags(Ctx& c, const uint32_t* flags, int P, int rank, int units, int unit,
                                              uint32_t epoch) {
  if (c.dead) return false;
  const bool mine = c.lane < P && c.lane != rank;
  const uint32_t* f = flags + (size_t)c.lane * units + unit;
  uint64_t t0 = 0;
  for (int spin = 0;; ++spin) {
    const bool ok = !mine || (int32_t)(ld_acquire_sys_u32(f) - epoch) >= 0;
    if (__all_sync(0xffffffffu, ok)) return true;
    if ((spin & 15) == 15 && give_up_check(c, t0, MK_ST_TIMEOUT_PEER, unit, (int)epoch)) {
      c.dead = true;
      return false;
    }
  }
}

// unit = 256 consecutive elements (8 per lane) of the flattened [rows, D] sum,
// or (MK_AR_MAX_KEY) all rows' 64-bit top-1 keys in unit 0.
__device__ __forceinline__ void ew_allreduce(Ctx& c, const mk_op_t* op, int unit) {
  const int n = op->i[MK_AR_N], P = op->i[MK_AR_P], rank = op->i[MK_AR_RANK];
  const int units = op->n_units;
  const uint32_t epoch = (uint32_t)op->i[MK_AR_EPOCH_BASE] + (uint32_t)c.pv->state->launches + 1u;
  const int64_t elem = 8;   // a 64-bit key, or an fp32 with its epoch
  const int64_t half = ((int64_t)P * n * elem + 15) / 16 * 16;   // one of the two inbox buffers
  const int64_t inbox_off = op->s[MK_AR_S_INBOX] + (int64_t)(epoch & 1u) * half, flags_off = op->s[MK_AR_S_FLAGS];
  uint8_t* self = reinterpret_cast<uint8_t*>(op->p[MK_AR_P_PEER0 + rank]);
  const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(self + flags_off);

  if (op->i[MK_AR_MODE] == MK_AR_MAX_KEY) {
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(op->p[MK_AR_P_X]);
    unsigned long long mine = 0ull;
    if (c.lane < n) mine = atomicExch(keys + c.lane, 0ull);   // rows <= 32; leaves the local keys cleared
    for (int r = 0; r < P; ++r) {
      if (r == rank || c.lane >= n) continue;
      unsigned long long* dst =
          reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(op->p[MK_AR_P_PEER0 + r]) + inbox_off);
      dst[(size_t)rank * n + c.lane] = mine;
    }
    __threadfence_system();
    __syncwarp();
    if (c.lane < P && c.lane != rank)
      st_release_sys_u32(reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(op->p[MK_AR_P_PEER0 + c.lane]) +
                                                     flags_off) + (size_t)rank * units + unit, epoch);
    if (!ar_wait_flags(c, my_flags, P, rank, units, unit, epoch)) return;
    if (c.lane < n) {
      unsigned long long best = mine;
      const unsigned long long* in = reinterpret_cast<const unsigned long long*>(self + inbox_off);
      for (int r = 0; r < P; ++r) {
        if (r == rank) continue;
        const unsigned long long k = ld_sys_u64(in + (size_t)r * n + c.lane);
        best = k > best ? k : best;
      }
      reinterpret_cast<unsigned long long*>(op->p[MK_AR_P_Y])[c.lane] = best;
    }
    return;
  }

  const int idx = unit * 256 + c.lane * 8;
  const bool valid = idx < n;   // n is a multiple of 8
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  if (valid) {
    if (op->i[MK_AR_X_T] == MK_T_FP32) {
      const float4* x = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op->p[MK_AR_P_X]) + idx);
      const float4 a = x[0], b = x[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
      const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(op->p[MK_AR_P_X]) + idx);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = op->i[MK_AR_X_T] == MK_T_BF16 ? bf16lo(w[i]) : f16lo(w[i]);
        v[2 * i + 1] = op->i[MK_AR_X_T] == MK_T_BF16 ? bf16hi(w[i]) : f16hi(w[i]);
      }
    }
    // Push this rank's partial into slot `rank` of every peer's inbox.  Each
    // fp32 travels as one 8-byte word {value, epoch}: an 8-byte store arrives
    // whole, so the receiver polls the data itself and no fence or separate
    // flag (one more NVLink crossing) is needed.
    for (int r = 0; r < P; ++r) {
      if (r == rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(op->p[MK_AR_P_PEER0 + r]) + inbox_off) +
                   (size_t)rank * n + idx;
#pragma unroll
      for (int i = 0; i < 8; ++i) st_sys_u2(dst + i, make_uint2(__float_as_uint(v[i]), epoch));
    }
  }
  // add in rank order: every rank computes the same sum bit for bit
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const uint2* in = reinterpret_cast<const uint2*>(self + inbox_off);
  for (int r = 0; r < P; ++r) {
    if (r == rank) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
      continue;
    }
    // wait (bounded) until all 8 words of this lane carry the epoch
    uint2 w[8];
    uint64_t t0 = 0;
    for (int spin = 0;; ++spin) {
      bool ok = true;
      if (valid && !c.dead) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          w[i] = ld_sys_u2(in + (size_t)r * n + idx + i);
          ok = ok && w[i].y == epoch;
        }
      }
      if (__all_sync(0xffffffffu, ok)) break;
      if ((spin & 15) == 15 && give_up_check(c, t0, MK_ST_TIMEOUT_PEER, unit, r)) {
        c.dead = true;
        return;
      }
    }
    if (valid) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += __uint_as_float(w[i].x);
    }
  }
  if (!valid || c.dead) return;
  const int yt = op->i[MK_AR_Y_T];
  if (op->p[MK_AR_P_RES] != 0) {
    const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(op->p[MK_AR_P_RES]) + idx);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += op->i[MK_AR_R_T] == MK_T_BF16 ? bf16lo(w[i]) : f16lo(w[i]);
      acc[2 * i + 1] += op->i[MK_AR_R_T] == MK_T_BF16 ? bf16hi(w[i]) : f16hi(w[i]);
    }
  }
  if (yt == MK_T_FP32) {
    float4* y = reinterpret_cast<float4*>(reinterpret_cast<float*>(op->p[MK_AR_P_Y]) + idx);
    y[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    y[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = yt == MK_T_BF16 ? pack_bf16(acc[2 * i], acc[2 * i + 1]) : pack_f16(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(op->p[MK_AR_P_Y]) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace mk
