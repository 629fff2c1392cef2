// Weight-streaming matvec / small-M GEMM unit:  out[m, o] = epi(W[o, :] · pro(x[m, :])).
//
// One unit = 16 "virtual rows" of the weight matrix over the full K, streamed
// through the page ring in K-slices of Kc columns (one page = two tiled TMA
// copies of 8 rows x Kc columns).  The unit's pages are dealt to one or more
// consumer warps; each feeds its slices to mma.sync m16n8k16 with the weights
// as the A operand (M = 16 virtual rows) and the staged activations as the B
// operand (N = 8 batch rows per n-tile), so batch 1..32 share one code path
// and accumulate in fp32; partial sums of several warps meet in shared memory.
//
// Virtual rows 0-7 and 8-15 land in the same thread's accumulators
// (rows g and g+8 of the fragment), which is what lets RoPE partners
// (row d, row d + D2) and GLU partners (gate row, up row) be combined in
// registers with no exchange.
//
// Replaces the decode matvec family (kernels/decode_matvec/sm100.py:224-654,
// sm120.py:596-2464 for NVFP4) and GemmOp's decode branch
// (kernels/gemm/gemm.py:382-430).
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "shell.cuh"

namespace mk {

__device__ __forceinline__ int clamp8(int v) { return v < 0 ? 0 : (v > 8 ? 8 : v); }

__device__ __forceinline__ bool mv_is_fp4(int wfmt) { return wfmt >= MK_W_NVFP4_F16S32; }

// ---- loader ------------------------------------------------------------------
// Page layout (bf16 / fp16 weights), Kt = Kc / 64 K-tiles per page:
//   [half A: Kt tiles of 8 rows x 128 B][half B: Kt tiles of 8 rows x 128 B]
// Half A holds virtual rows 0-7, half B virtual rows 8-15.  Every tile is one
// 128-byte-swizzled box row group of a 3-D tensor map over the weight matrix
// (dims: 64 K-values, rows, K-tiles), so a whole half is ONE tiled TMA copy.
// NVFP4: the same with 256 packed values per 128-byte tile row (Kt4 = Kc / 256
// tiles), followed by two 1 KB scale tiles (8 rows x 128 B, one per half).
// Rows past the end of the matrix and K-tiles past K are zero-filled by TMA.
__device__ __forceinline__ uint32_t mv_half_bytes(int wfmt, int Kc) {
  return mv_is_fp4(wfmt) ? (uint32_t)(Kc / 256) * 1024u : (uint32_t)(Kc / 64) * 1024u;
}

// What the loader needs to issue the pages of one unit (from the instruction record).
struct MvLoad {
  const void* tm_a;
  const void* tm_b;
  const void* ts_a;
  const void* ts_b;
  int rowA0, rowB0;
  int tiles_per_page;   // K-tiles (weights) per page
  uint32_t half;
  bool fp4;
};

// Issue the copies of K-slice `p` into the page at `page` (shared address):
// two tiled TMA copies (four with NVFP4 scales) and one arrival for the whole
// loader warp.  Called by loader lane 0 only.
__device__ __forceinline__ void mv_load_issue(const MvLoad& l, int p, uint32_t page, uint32_t bar, uint64_t policy) {
  const int kt0 = p * l.tiles_per_page;
  if (!l.fp4) {
    mbar_expect_tx(bar, 2u * l.half);
    tma_load_3d(page, l.tm_a, 0, l.rowA0, kt0, bar, policy);
    tma_load_3d(page + l.half, l.tm_b, 0, l.rowB0, kt0, bar, policy);
  } else {
    // a scale tile row holds the 128 scale bytes of 2048 K-values = one page
    mbar_expect_tx(bar, 2u * l.half + 2048u);
    tma_load_3d(page, l.tm_a, 0, l.rowA0, kt0, bar, policy);
    tma_load_3d(page + l.half, l.tm_b, 0, l.rowB0, kt0, bar, policy);
    tma_load_3d(page + 2u * l.half, l.ts_a, 0, l.rowA0, p, bar, policy);
    tma_load_3d(page + 2u * l.half + 1024u, l.ts_b, 0, l.rowB0, p, bar, policy);
  }
  mbar_arrive_n(bar, 32);
}

// ---- activation staging -----------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& v, int ty, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (ty == MK_T_BF16) {
      f[2 * i] = bf16lo(w[i]);
      f[2 * i + 1] = bf16hi(w[i]);
    } else {
      f[2 * i] = f16lo(w[i]);
      f[2 * i + 1] = f16hi(w[i]);
    }
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8], int ty) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = (ty == MK_T_BF16) ? pack_bf16(f[2 * i], f[2 * i + 1]) : pack_f16(f[2 * i], f[2 * i + 1]);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
// Round every element to the storage type `ty` (what a store + reload does).
__device__ __forceinline__ void round8(float (&f)[8], int ty) {
  uint4 v = pack8(f, ty);
  unpack8(v, ty, f);
}

__device__ __forceinline__ int mv_act_type(const mk_op_t* op) {
  return op->i[MK_MV_WFMT] == MK_W_BF16 ? MK_T_BF16 : MK_T_FP16;
}

// With bf16 weights the RMSNorm scale is taken out of the staged row: the
// row is staged as bf16(x * w) in ONE pass while its sum of squares is
// collected, and the epilogue multiplies the accumulators by
// rsqrt(mean(x^2) + eps) — W·(x∘w)·r = r·(W·(x∘w)), r being one scalar per
// row.  The first mma then waits for one trip to the activations, not for a
// CTA-wide reduction and a second pass over the row.  (f16 staging, used with
// NVFP4 weights, keeps the two-pass form: an unnormalised row may leave the
// f16 range.)
__device__ __forceinline__ bool mv_rstd_in_epilogue(const mk_op_t* op) {
  return op->i[MK_MV_PRO] != MK_PRO_NONE && op->i[MK_MV_X_T] == MK_T_BF16 && op->i[MK_MV_WFMT] == MK_W_BF16;
}

// Stage pro(x) for all M rows into the shared activation buffer.  Called by
// all consumer threads (tid in [0, kConsumerWarps*32)); the caller places a
// consumer barrier before and after.  `stage` = fill the buffer,
// `write_res` = also materialise residual_out = x + residual_in in global.
//
// The code is kept small on purpose (loops are not unrolled beyond what the
// memory latency asks for): it runs once per op on every CTA, always from a
// cold instruction cache.
//   * no prologue, same type: the rows are copied global -> shared with
//     16-byte asynchronous copies, all in flight at once;
//   * RMSNorm prologue: R rows x H chunks per thread are requested together
//     (one trip to L2), then reduced; R x H = 1 x 4 for the bf16 kernel of up to 8
//     rows, 2 x 4 for its NVFP4 counterpart (K = 4096 in one trip), 4 x 2 otherwise.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <int R, int H, int WFC>
__device__ __forceinline__ void mv_stage(Ctx& c, const mk_op_t* op, bool stage, bool write_res) {
  const int tid = (c.warp - 1) * 32 + c.lane;
  constexpr int T = kConsumerWarps * 32;
  const int K = op->i[MK_MV_K], M = op->i[MK_MV_M], S = op->i[MK_MV_S];
  const int pro = op->i[MK_MV_PRO];
  // a kernel built for one weight family knows its activation types
  const int xt = WFC == 0 ? (int)MK_T_BF16 : op->i[MK_MV_X_T];
  const int at = WFC == 0 ? (int)MK_T_BF16 : (WFC == 2 ? (int)MK_T_FP16 : mv_act_type(op));
  // a bf16 kernel always takes the RMSNorm scale in the epilogue: the second pass is not even compiled
  const bool fused = WFC == 0 ? pro != MK_PRO_NONE : (WFC != 2 && mv_rstd_in_epilogue(op));
  const uint32_t xs = (uint32_t)K * 2u + 64u;
  const int chunks = K >> 3;
  const uint16_t* x = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_X]);
  const uint16_t* ri = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_RES_IN]);
  uint16_t* ro = reinterpret_cast<uint16_t*>(op->p[MK_MV_P_RES_OUT]);
  const uint16_t* nw = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_NORM_W]);
  const bool add = (pro == MK_PRO_ADD_RMS) && ri != nullptr;
  write_res = write_res && add && ro != nullptr;
  if (!stage && !write_res) return;
  const bool dyn_tab = (op->i[MK_MV_DYNPOS] & MK_MV_DYN_TABLES) != 0;
  if (stage && op->i[MK_MV_TR] == MK_TR_ROPE && tid < 2 * (dyn_tab ? M : S)) {
    // the epilogue's cos / sin rows: pull them into L1 while the activations are on their way
    // (with device-resident positions: the row of every batch row's own position)
    const uint8_t* tab = reinterpret_cast<const uint8_t*>(op->p[(tid & 1) ? MK_MV_P_SIN : MK_MV_P_COS]);
    const int row = dyn_tab ? c.ctrl->pos[(tid >> 1) & 31] : (tid >> 1);
    asm volatile("prefetch.global.L1 [%0];" ::"l"(tab + (size_t)row * (size_t)op->s[MK_MV_S_COS] * 2u));
  }
  auto row_off = [&](int m, int sb, int ss) -> int64_t {
    int b = m, s2 = 0;
    if (S != 1) {
      b = m / S;
      s2 = m - b * S;
    }
    return b * op->s[sb] + s2 * op->s[ss];
  };

  if (pro == MK_PRO_NONE && xt == at) {
    // plain copy
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + row_off(m, MK_MV_S_X_B, MK_MV_S_X_S);
      const uint32_t dst = c.act_u32 + (uint32_t)m * xs;
#pragma unroll 1
      for (int ch = tid; ch < chunks; ch += T) cp_async16(dst + (uint32_t)ch * 16u, xr + ch * 8);
    }
    cp_async_wait_all();
    return;
  }

  const uint4 z = make_uint4(0, 0, 0, 0);
  if (WFC != 0 && pro == MK_PRO_NONE) {
    // no prologue, the mma's type differs from the input's: a converting copy, eight chunks per
    // thread in flight (K = 12288 in one trip per row)
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + row_off(m, MK_MV_S_X_B, MK_MV_S_X_S);
      const uint32_t dst = c.act_u32 + (uint32_t)m * xs;
#pragma unroll 1
      for (int ch0 = tid; ch0 < chunks; ch0 += 8 * T) {
        uint4 v[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) v[h] = (ch0 + h * T < chunks) ? *reinterpret_cast<const uint4*>(xr + (ch0 + h * T) * 8) : z;
#pragma unroll
        for (int h = 0; h < 8; ++h) {
          if (ch0 + h * T >= chunks) break;
          float f[8];
          unpack8(v[h], xt, f);
          sts128(dst + (uint32_t)(ch0 + h * T) * 16u, pack8(f, at));
        }
      }
    }
    return;
  }
#pragma unroll 1
  for (int m0 = 0; m0 < M; m0 += R) {
    const uint16_t *xr[R], *rr[R];
    uint16_t* wr[R];
    float sum[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int m = min(m0 + j, M - 1);
      xr[j] = x + row_off(m, MK_MV_S_X_B, MK_MV_S_X_S);
      rr[j] = add ? ri + row_off(m, MK_MV_S_RI_B, MK_MV_S_RI_S) : x;
      wr[j] = write_res ? ro + row_off(m, MK_MV_S_RO_B, MK_MV_S_RO_S) : nullptr;
      sum[j] = 0.f;
    }
#pragma unroll 1
    for (int ch0 = tid; ch0 < chunks; ch0 += H * T) {
      uint4 v[R][H], r[R][H], wv[H];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const int ch = ch0 + h * T;
        const bool ok = ch < chunks;
        wv[h] = (ok && fused) ? *reinterpret_cast<const uint4*>(nw + ch * 8) : z;
        // two-pass form: the second pass reads this thread's norm weights; have them in L1 by then
        if (WFC != 0 && ok && !fused && pro != MK_PRO_NONE) asm volatile("prefetch.global.L1 [%0];" ::"l"(nw + ch * 8));
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const bool rok = ok && (R == 1 || m0 + j < M);   // rows past M are not fetched a second time
          v[j][h] = rok ? *reinterpret_cast<const uint4*>(xr[j] + ch * 8) : z;
          r[j][h] = (rok && add) ? *reinterpret_cast<const uint4*>(rr[j] + ch * 8) : z;
        }
      }
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const int ch = ch0 + h * T;
        if (ch >= chunks) break;
        float w[8];
        unpack8(wv[h], xt, w);
#pragma unroll
        for (int j = 0; j < R; ++j) {
          if (m0 + j >= M) break;
          float f[8];
          unpack8(v[j][h], xt, f);
          uint4 o = v[j][h];
          if (add) {
            float q[8];
            unpack8(r[j][h], xt, q);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] += q[i];
            round8(f, xt);
            o = pack8(f, xt);
            if (wr[j]) *reinterpret_cast<uint4*>(wr[j] + ch * 8) = o;
          }
          if (stage) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[j] += f[i] * f[i];
            if (fused) {
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] *= w[i];
              o = pack8(f, xt);
            }
            // not fused: keep the (rounded) input in its own type for now; pass 2 rescales
            sts128(c.act_u32 + (uint32_t)(m0 + j) * xs + (uint32_t)ch * 16u, o);
          }
        }
      }
    }
    if (stage && pro != MK_PRO_NONE) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const float t = warp_sum(sum[j]);
        if (c.lane == 0 && m0 + j < M) c.ctrl->red[(m0 + j) * kConsumerWarps + (c.warp - 1)] = t;
      }
    }
  }
  if (!stage || fused) return;
  if constexpr (WFC == 0) return;
  // second pass: normalise and convert to the mma's activation type
  named_bar_sync(kConsumerBarrier, T);
  if (tid < M) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) tot += c.ctrl->red[tid * kConsumerWarps + w];
    c.ctrl->rstd[tid] = rsqrtf(tot / (float)K + op->f[MK_MV_F_EPS]);
  }
  named_bar_sync(kConsumerBarrier, T);
#pragma unroll 1
  for (int ch = tid; ch < chunks; ch += T) {
    float w[8];
    unpack8(*reinterpret_cast<const uint4*>(nw + ch * 8), xt, w);
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint32_t a = c.act_u32 + (uint32_t)m * xs + (uint32_t)ch * 16u;
      float f[8];
      unpack8(lds128(a), xt, f);
      const float rstd = c.ctrl->rstd[m];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      sts128(a, pack8(f, at));
    }
  }
}

// ---- epilogue ----------------------------------------------------------------------
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ unsigned long long top1_key(float v, int idx) {
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

// Output addressing without divisions: the instruction record carries, for
// virtual rows 0-7 (a) and 8-15 (b), the first weight row and the element
// offset of that row's result inside one activation row's output (head *
// head stride + dim); what remains per activation row m is its (batch, s)
// offset, which at decode (S = 1) is m * batch stride.
struct MvOut {
  int rowA0, rowB0, offA, offB, chunk;
};

__device__ __forceinline__ void mv_put(const mk_op_t* op, int ot, int64_t off, float v) {
  if (ot == MK_T_FP32) {
    reinterpret_cast<float*>(op->p[MK_MV_P_OUT])[off] = v;
  } else if (ot == MK_T_BF16) {
    reinterpret_cast<uint16_t*>(op->p[MK_MV_P_OUT])[off] = (uint16_t)f2bf(v);
  } else {
    reinterpret_cast<uint16_t*>(op->p[MK_MV_P_OUT])[off] = (uint16_t)(pack_f16(v, 0.f) & 0xffffu);
  }
}

// One pass per (activation n-tile, column of the thread's pair): the loop is
// kept rolled (the accumulator pair is picked with selects) so that the
// epilogue, which runs once per unit from a cold instruction cache, stays a
// few hundred instructions whatever the batch.
template <int NT, int WFC, int FEAT>
__device__ __forceinline__ void mv_epilogue(Ctx& c, const mk_op_t* op, const MvOut& r, float (&acc)[NT][4]) {
  const int g = c.lane >> 2, t = c.lane & 3;
  const int O = op->i[MK_MV_O], K = op->i[MK_MV_K], M = op->i[MK_MV_M], S = op->i[MK_MV_S];
  const int mode = op->i[MK_MV_MODE], tr = op->i[MK_MV_TR], epi = op->i[MK_MV_EPI];
  const int xt = WFC == 0 ? (int)MK_T_BF16 : op->i[MK_MV_X_T];
  const int ot = op->i[MK_MV_OUT_T];
  // block-scaled NVFP4: one fp32 scale per matrix (rows a and b come from two matrices in pair mode)
  const bool gscaled = WFC != 0 && op->i[MK_MV_WFMT] == MK_W_NVFP4_E4M3S16;
  const float gs = gscaled ? op->f[MK_MV_F_GSCALE] : 1.f;
  const float gsb = (gscaled && mode == MK_MV_PAIR) ? op->f[MK_MV_F_GSCALE1] : gs;
  const bool fused = WFC == 0 ? op->i[MK_MV_PRO] != MK_PRO_NONE : (WFC != 2 && mv_rstd_in_epilogue(op));
  const float eps = op->f[MK_MV_F_EPS];
  const int nA = mode == MK_MV_ROPE ? 8 : clamp8(O - r.rowA0);
  const int nB = mode == MK_MV_ROPE ? 8 : clamp8(O - r.rowB0);
  const bool va = g < nA, vb = g < nB;
  const bool two = tr != MK_TR_SILU_MUL;
  // device-resident cache position: which of the table row and the output row follow it
  const bool dyn_t = (op->i[MK_MV_DYNPOS] & MK_MV_DYN_TABLES) != 0, dyn_o = (op->i[MK_MV_DYNPOS] & MK_MV_DYN_OUT) != 0;
#pragma unroll 1
  for (int q = 0; q < 2 * NT; ++q) {
    const int m0 = (q >> 1) * 8 + (q & 1);   // the smallest activation row any lane has in this pass
    if (m0 >= M) continue;
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (q == 2 * nt + e) {
          a = acc[nt][e];
          b = acc[nt][2 + e];
        }
    const int m = m0 + 2 * t;
    const bool vm = m < M;
    float scale = 1.f;
    if (fused) {
      // the row's RMSNorm scale, from the per-warp sums of squares the staging left behind
      const float* rs = c.ctrl->red + (vm ? m : 0) * kConsumerWarps;
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) tot += rs[w];
      scale = rsqrtf(tot / (float)K + eps);
    }
    a *= scale * gs;
    b *= scale * gsb;
    int bb = m, ss = 0;
    if (S != 1) {
      bb = m / S;
      ss = m - bb * S;
    }
    // the batch row's own cache position (a dynamic position means one token per sequence: bb = m)
    const int prow = (dyn_t || dyn_o) ? c.ctrl->pos[(vm ? bb : 0) & 31] : 0;
    const int tpos = dyn_t ? prow : 0, dpos = dyn_o ? prow : 0;
    if (tr == MK_TR_ROPE) {
      if (vm) {
        const int d = r.chunk * 8 + g;
        const uint16_t* cs = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_COS]) + (ss + tpos) * op->s[MK_MV_S_COS] + d;
        const uint16_t* sn = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_SIN]) + (ss + tpos) * op->s[MK_MV_S_COS] + d;
        const bool bf = xt == MK_T_BF16;
        const float cv = bf ? bf16lo(*cs) : f16lo(*cs);
        const float sv = bf ? bf16lo(*sn) : f16lo(*sn);
        const float a2 = a * cv - b * sv, b2 = b * cv + a * sv;
        a = a2;
        b = b2;
      }
    } else if (tr == MK_TR_SILU_MUL) {
      a = silu_f(a) * b;
    } else if (tr == MK_TR_RELU) {
      a = fmaxf(a, 0.f);
      b = fmaxf(b, 0.f);
    } else if (tr == MK_TR_SILU) {
      a = silu_f(a);
      b = silu_f(b);
    }
    if ((FEAT & MK_F_TOP1) != 0 && epi == MK_EPI_TOP1) {
      unsigned long long key = 0ull;
      const int idx0 = op->i[MK_MV_IDX0];
      if (va) key = top1_key(a, idx0 + r.rowA0 + g);
      if (vb) {
        const unsigned long long kb = top1_key(b, idx0 + r.rowB0 + g);
        key = kb > key ? kb : key;
      }
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
      }
      if (g == 0 && vm) atomicMax(reinterpret_cast<unsigned long long*>(op->p[MK_MV_P_OUT]) + m, key);
    } else if (vm) {
      if (epi == MK_EPI_RESIDUAL) {
        const uint16_t* er = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_EPI_RES]) + bb * op->s[MK_MV_S_ER_B] +
                             ss * op->s[MK_MV_S_ER_S];
        const uint16_t ra = va ? er[r.rowA0 + g] : (uint16_t)0, rb = (vb && two) ? er[r.rowB0 + g] : (uint16_t)0;
        a += (xt == MK_T_BF16) ? bf16lo(ra) : f16lo(ra);
        b += (xt == MK_T_BF16) ? bf16lo(rb) : f16lo(rb);
      }
      const int64_t mo = bb * op->s[MK_MV_S_O_B] + (int64_t)(ss + op->i[MK_MV_POS] + dpos) * op->s[MK_MV_S_O_S];
      if (va) mv_put(op, ot, mo + r.offA + g, a);
      if (vb && two) mv_put(op, ot, mo + r.offB + g, b);
    }
  }
}

// ---- consumer ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Eight e2m1 codes (one 32-bit word, nibble i = value i) -> four f16x2
// registers (v0,v1) (v2,v3) (v4,v5) (v6,v7), each times the f16x2 scale.  The
// word is split into its bytes inside the PTX block, so the conversion reads
// each byte in place: extracting the bytes with shifts and masks first costs
// more integer-pipe slots than the four conversions themselves (the integer
// pipe, 64 lanes per clock per SM, is what bounds this loop).
__device__ __forceinline__ void e2m1x8_scaled(uint32_t w, uint32_t scale, uint32_t (&r)[4]) {
  uint32_t c0, c1, c2, c3;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}"
      : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
      : "r"(w));
  r[0] = hmul2(c0, scale);
  r[1] = hmul2(c1, scale);
  r[2] = hmul2(c2, scale);
  r[3] = hmul2(c3, scale);
}

// Swizzled address of 16-byte chunk `c` of row `r` (0-7) inside a 1 KB tile.
__device__ __forceinline__ uint32_t tile_chunk(uint32_t tile, int r, int c) {
  return tile + (uint32_t)r * 128u + (uint32_t)((c ^ r) << 4);
}

// NT = n-tiles of 8 activation rows; NA = independent accumulator sets (the
// mma chain on one accumulator is latency-bound, so K-steps rotate over NA).
//
// All consumers that own a page of the unit call this.  Each accumulates its
// K-slices; with more than one participant the partial sums meet in a
// shared-memory slot set, and the last one to arrive adds them up in warp
// order (so the result does not depend on timing), runs the epilogue and
// returns true: it is the one that signals the unit.
//
// WFC fixes the weight-format family at compile time so that a kernel built
// for one family carries only that code: 0 = bf16, 2 = NVFP4 (either scale
// layout), -1 = decided per op at run time.
template <int NT, int NA, int WFC, int FEAT>
__device__ __forceinline__ bool mv_unit(Ctx& c, const mk_op_t* op, const UnitArgs& u) {
  const int part = u.part;
  const uint32_t ord = u.ord;
  const int parts = (u.flags >> MK_LDF_SPLIT_SHIFT) & MK_LDF_SPLIT_MASK;
  const int p0 = part;   // participant j takes pages j, j + parts, j + 2 parts, ...
  const int g = c.lane >> 2, t = c.lane & 3;
  const int K = op->i[MK_MV_K], Kc = op->i[MK_MV_KC], M = op->i[MK_MV_M];
  const int wfmt = WFC == 0 ? (int)MK_W_BF16 : op->i[MK_MV_WFMT];
  const bool dense = WFC == 0 ? true : (WFC == 2 ? false : (wfmt == MK_W_BF16 || wfmt == MK_W_FP16));
  const uint32_t xs = (uint32_t)K * 2u + 64u;
  const uint32_t half = mv_half_bytes(wfmt, Kc);
  const int NPG = c.pv->n_pages;
  if (part == 0 && op->i[MK_MV_EPI] == MK_EPI_RESIDUAL && op->i[MK_MV_S] == 1) {
    // whoever finishes the unit adds this residual: pull its lines into L1 now
    const int ra = ins_field(u.mine->row_a, u.idx), rb = ins_field(u.mine->row_b, u.idx);
    if (c.lane < 2 * M) {
      const uint16_t* er = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_EPI_RES]) +
                           (c.lane >> 1) * op->s[MK_MV_S_ER_B] + ((c.lane & 1) ? rb : ra);
      asm volatile("prefetch.global.L1 [%0];" ::"l"(er));
    }
  }
  float acc[NA][NT][4];
#pragma unroll
  for (int a = 0; a < NA; ++a)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[a][nt][e] = 0.f;

  uint32_t xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + g;
    xok[nt] = m < M;
    xrow[nt] = c.act_u32 + (uint32_t)(xok[nt] ? m : 0) * xs;
  }

  const int np = u.n_pages;
  RingPos rp = u.rp;
  for (int p = p0; p < np; p += parts, ring_advance(rp, parts, NPG)) {
    uint32_t page;
    if (!page_acquire(c, rp, page)) return false;
    trace(c, TRC_PAGE_READY, rp.k * (uint32_t)NPG + rp.slot);
    const long long cyc0 = clock64();
    const int k0 = p * Kc;
    const int kc = min(Kc, K - k0);
    if (dense) {
      // One K-tile = 64 K-values = 8 chunks of 16 B per row; this thread takes
      // chunks 2t and 2t+1 of rows g (half A) and g (half B): with the 128-byte
      // swizzle the 8 lanes of a shared-memory phase then hit 8 distinct chunks.
      // The mma wrappers are asm volatile, which the compiler does not move
      // loads across, so the software pipeline is written out by hand: tiles
      // are handled two at a time and (for one activation n-tile) the
      // fragments of the next pair are requested before the mma's of the
      // current pair are issued.
      const int tiles = kc >> 6;
      const uint32_t off0 = (uint32_t)g * 128u + (uint32_t)(((2 * t) ^ g) << 4);      // chunk 2t of row g
      const uint32_t off1 = (uint32_t)g * 128u + (uint32_t)(((2 * t + 1) ^ g) << 4);  // chunk 2t+1
      const uint32_t xo0 = (uint32_t)(k0 + 2 * t * 8) * 2u;                           // x offset of chunk 2t
      struct Frag {
        uint4 wa[2][2], wb[2][2], x[NT][2][2];   // [tile of the pair][chunk j]
      };
      auto load_pair = [&](Frag& f, int kt) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t ta = page + (uint32_t)(kt + u) * 1024u, tb = ta + half;
          f.wa[u][0] = lds128(ta + off0);
          f.wa[u][1] = lds128(ta + off1);
          f.wb[u][0] = lds128(tb + off0);
          f.wb[u][1] = lds128(tb + off1);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            // always load (rows past M read row 0 and are zeroed): no branch in the hot loop
            const uint4 x0 = lds128(xrow[nt] + xo0 + (uint32_t)(kt + u) * 128u);
            const uint4 x1 = lds128(xrow[nt] + xo0 + (uint32_t)(kt + u) * 128u + 16u);
            const uint32_t keep = xok[nt] ? 0xffffffffu : 0u;
            f.x[nt][u][0] = make_uint4(x0.x & keep, x0.y & keep, x0.z & keep, x0.w & keep);
            f.x[nt][u][1] = make_uint4(x1.x & keep, x1.y & keep, x1.z & keep, x1.w & keep);
          }
        }
      };
      // The two mma's on one 16-byte chunk feed the same accumulator; issuing
      // the first halves of all chunks before the second halves keeps dependent
      // mma's several issue slots apart.
      auto mma_pair = [&](const Frag& f, int valid, auto is_bf16) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (u < valid) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                constexpr int kSets = NA;
                const int a = (u * 2 + j) % kSets;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  const uint32_t a0 = half ? f.wa[u][j].z : f.wa[u][j].x, a1 = half ? f.wb[u][j].z : f.wb[u][j].x;
                  const uint32_t a2 = half ? f.wa[u][j].w : f.wa[u][j].y, a3 = half ? f.wb[u][j].w : f.wb[u][j].y;
                  const uint32_t b0 = half ? f.x[nt][u][j].z : f.x[nt][u][j].x;
                  const uint32_t b1 = half ? f.x[nt][u][j].w : f.x[nt][u][j].y;
                  if constexpr (decltype(is_bf16)::value)
                    mma_bf16(acc[a][nt], a0, a1, a2, a3, b0, b1);
                  else
                    mma_f16(acc[a][nt], a0, a1, a2, a3, b0, b1);
                }
              }
            }
          }
        }
      };
      // A page always holds whole tiles up to its capacity (TMA zero-fills past
      // K), so reading the second tile of the last pair is safe even when odd.
      auto run_page = [&](auto is_bf16) {
        if constexpr (NT == 1) {
          Frag f0, f1;
          load_pair(f0, 0);
#pragma unroll 1
          for (int kt = 0; kt < tiles; kt += 4) {
            if (kt + 2 < tiles) load_pair(f1, kt + 2);
            mma_pair(f0, min(2, tiles - kt), is_bf16);
            if (kt + 2 < tiles) {
              if (kt + 4 < tiles) load_pair(f0, kt + 4);
              mma_pair(f1, min(2, tiles - kt - 2), is_bf16);
            }
          }
        } else {
          Frag f;
#pragma unroll 1
          for (int kt = 0; kt < tiles; kt += 2) {
            load_pair(f, kt);
            mma_pair(f, min(2, tiles - kt), is_bf16);
          }
        }
      };
      if (WFC == 0 || wfmt == MK_W_BF16)
        run_page(std::true_type{});
      else
        run_page(std::false_type{});
    } else {
      // NVFP4: one tile row = 256 packed values; chunk ch = 32 consecutive K
      // values of a row with their block scales.  Values are scaled in f16
      // (exact for e2m1 x e4m3) and fed to the f16 tensor-core path.
      const int tiles = kc >> 8;
      const uint32_t sa = page + 2u * half, sb = sa + 1024u;
#pragma unroll 1
      for (int kt = 0; kt < tiles; ++kt) {
        const uint32_t ta = page + (uint32_t)kt * 1024u, tb = ta + half;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int ch = 2 * t + j;
          const uint4 plo = lds128(tile_chunk(ta, g, ch));
          const uint4 phi = lds128(tile_chunk(tb, g, ch));
          // scale bytes of this chunk: row g, byte kt*16 + ch*2 of the 128-byte scale row
          const uint32_t soff = (uint32_t)g * 128u + (uint32_t)((kt ^ g) << 4) + (uint32_t)ch * 2u;
          const uint32_t slo_raw = lds16(sa + soff);
          const uint32_t shi_raw = lds16(sb + soff);
          uint32_t slo[2], shi[2];  // f16x2 broadcast scale for values [0,16) and [16,32)
          if (wfmt == MK_W_NVFP4_F16S32) {
            slo[0] = slo[1] = slo_raw | (slo_raw << 16);
            shi[0] = shi[1] = shi_raw | (shi_raw << 16);
          } else {
            __half2_raw a2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)slo_raw, __NV_E4M3);
            __half2_raw b2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)shi_raw, __NV_E4M3);
            slo[0] = (uint32_t)a2.x | ((uint32_t)a2.x << 16);
            slo[1] = (uint32_t)a2.y | ((uint32_t)a2.y << 16);
            shi[0] = (uint32_t)b2.x | ((uint32_t)b2.x << 16);
            shi[1] = (uint32_t)b2.y | ((uint32_t)b2.y << 16);
          }
          const uint32_t pl[4] = {plo.x, plo.y, plo.z, plo.w};
          const uint32_t ph[4] = {phi.x, phi.y, phi.z, phi.w};
          const uint32_t xoff = (uint32_t)(k0 + kt * 256 + ch * 32) * 2u;
#pragma unroll
          for (int q = 0; q < 4; ++q) {  // 8 values (4 bytes) of each row -> two mma k-slots
            uint32_t al[4], ah[4];
            e2m1x8_scaled(pl[q], slo[q >> 1], al);
            e2m1x8_scaled(ph[q], shi[q >> 1], ah);
            const int a = q % NA;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint4 xb = make_uint4(0, 0, 0, 0);
              if (xok[nt]) xb = lds128(xrow[nt] + xoff + (uint32_t)q * 16u);
              mma_f16(acc[a][nt], al[0], ah[0], al[1], ah[1], xb.x, xb.y);
              mma_f16(acc[a][nt], al[2], ah[2], al[3], ah[3], xb.z, xb.w);
            }
          }
        }
      }
    }
    const long long cyc1 = clock64();
    page_release(c, rp);
    trace(c, TRC_PAGE_DONE, rp.k * (uint32_t)NPG + rp.slot);
    trace(c, TRC_PAGE_CYCLES, (uint32_t)(cyc1 - cyc0));
  }
#pragma unroll
  for (int a = 1; a < NA; ++a)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[0][nt][e] += acc[a][nt][e];

  // Split-K reduction across the participating consumers.
  // mv_sets (1, 2 or 4) slot sets share kPartialBytes; the host picks the
  // count so that the widest matvec op of the program fits a slot.
  if (parts > 1) {
    const int sets_log2 = __ffs(c.pv->mv_sets) - 1;
    const int kSlotFloats = (kPartialBytes / 4 / kConsumerWarps) >> sets_log2;
    const uint32_t set = ord & (uint32_t)(c.pv->mv_sets - 1), gen = ord >> sets_log2;
    float* slots = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.ctrl) + kCtrlStructBytes) +
                   (size_t)set * kConsumerWarps * kSlotFloats;
    // the set's previous users (units ord - kSets, ...) must have been reduced
    if (!wait_smem_ge(c, &c.ctrl->mv_done[set], gen, (int)ord)) return false;
    float* mine = slots + (size_t)part * kSlotFloats;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) mine[(nt * 4 + e) * 32 + c.lane] = acc[0][nt][e];
    __syncwarp();
    int last = 0;
    if (c.lane == 0) {
      __threadfence_block();
      last = atomicAdd(&c.ctrl->mv_arrive[set], 1u) == (uint32_t)(parts - 1);
      __threadfence_block();
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    trace(c, TRC_MV_ARRIVED, ord);
    if (!last) return false;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[0][nt][e] = 0.f;
    // in participant order: the sum does not depend on who arrived when
#pragma unroll 1
    for (int j = 0; j < parts; ++j) {
      const float* src = slots + (size_t)j * kSlotFloats;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][nt][e] += src[(nt * 4 + e) * 32 + c.lane];
    }
    __syncwarp();
    if (c.lane == 0) {
      c.ctrl->mv_arrive[set] = 0;
      __threadfence_block();
      *reinterpret_cast<volatile uint32_t*>(&c.ctrl->mv_done[set]) = gen + 1u;
    }
  }
  trace(c, TRC_MV_REDUCED, ord);
  MvOut r;
  r.rowA0 = ins_field(u.mine->row_a, u.idx);
  r.rowB0 = ins_field(u.mine->row_b, u.idx);
  r.offA = ins_field(u.mine->off_a, u.idx);
  r.offB = ins_field(u.mine->off_b, u.idx);
  r.chunk = (u.flags >> MK_LDF_CHUNK_SHIFT) & MK_LDF_CHUNK_MASK;
  mv_epilogue<NT, WFC, FEAT>(c, op, r, acc[0]);
  trace(c, TRC_MV_EPILOGUE, ord);
  return true;
}

// NTC / WFC: the activation-tile count (1, 2, 4) and weight family the kernel
// was built for, or 0 / -1 to decide per op.
template <int NTC, int WFC, int FEAT>
__device__ __forceinline__ bool mv_dispatch(Ctx& c, const mk_op_t* op, const UnitArgs& u) {
  if constexpr (NTC == 1) {
    return mv_unit<1, 4, WFC, FEAT>(c, op, u);
  } else if constexpr (NTC == 2) {
    return mv_unit<2, 2, WFC, FEAT>(c, op, u);
  } else if constexpr (NTC == 4) {
    return mv_unit<4, 1, WFC, FEAT>(c, op, u);
  } else {
    const int M = op->i[MK_MV_M];
    if (M <= 8) return mv_unit<1, 4, WFC, FEAT>(c, op, u);
    if (M <= 16) return mv_unit<2, 2, WFC, FEAT>(c, op, u);
    return mv_unit<4, 1, WFC, FEAT>(c, op, u);
  }
}

}  // namespace mk
