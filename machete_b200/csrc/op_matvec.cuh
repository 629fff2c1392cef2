// Weight-streaming matvec / small-M GEMM unit:  out[m, o] = epi(W[o, :] · pro(x[m, :])).
//
// One unit = 16 "virtual rows" of the weight matrix over the full K, streamed
// through the page ring in K-slices of Kc columns (16 row segments per page,
// one untiled TMA copy each).  The consumer warp feeds the slices to
// mma.sync m16n8k16 with the weights as the A operand (M = 16 virtual rows)
// and the staged activations as the B operand (N = 8 batch rows per n-tile),
// so batch 1..32 share one code path and accumulate in fp32.
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
#include "shell.cuh"

namespace mk {

struct MvRows {
  const uint8_t* wa;
  const uint8_t* wb;
  const uint8_t* sa;  // scales
  const uint8_t* sb;
  int rowA0, rowB0, nA, nB;
};

__device__ __forceinline__ int clamp8(int v) { return v < 0 ? 0 : (v > 8 ? 8 : v); }

__device__ __forceinline__ MvRows mv_rows(const mk_op_t* op, int unit) {
  MvRows r;
  const int O = op->i[MK_MV_O];
  const int mode = op->i[MK_MV_MODE];
  r.wa = reinterpret_cast<const uint8_t*>(op->p[MK_MV_P_W0]);
  r.sa = reinterpret_cast<const uint8_t*>(op->p[MK_MV_P_SC0]);
  if (mode == MK_MV_PLAIN) {
    r.wb = r.wa;
    r.sb = r.sa;
    r.rowA0 = unit * 16;
    r.rowB0 = unit * 16 + 8;
    r.nA = clamp8(O - r.rowA0);
    r.nB = clamp8(O - r.rowB0);
  } else if (mode == MK_MV_PAIR) {
    r.wb = reinterpret_cast<const uint8_t*>(op->p[MK_MV_P_W1]);
    r.sb = reinterpret_cast<const uint8_t*>(op->p[MK_MV_P_SC1]);
    r.rowA0 = r.rowB0 = unit * 8;
    r.nA = r.nB = clamp8(O - r.rowA0);
  } else {  // MK_MV_ROPE
    const int hd = op->i[MK_MV_HD], d2 = op->i[MK_MV_D2];
    const int upb = d2 >> 3;
    const int h = unit / upb, j = (unit - h * upb) * 8;
    r.wb = r.wa;
    r.sb = r.sa;
    r.rowA0 = h * hd + j;
    r.rowB0 = r.rowA0 + d2;
    r.nA = r.nB = 8;
  }
  return r;
}

__device__ __forceinline__ bool mv_is_fp4(int wfmt) { return wfmt >= MK_W_NVFP4_F16S32; }

// ---- loader ------------------------------------------------------------------
// Issue the copies of K-slice `p` of `unit` into the page at `page` (shared
// address).  All 32 loader lanes call this; every lane arrives on `bar` once.
__device__ __forceinline__ void mv_load_page(const mk_op_t* op, int unit, int p, uint32_t page, uint32_t bar,
                                             int lane) {
  const MvRows r = mv_rows(op, unit);
  const int K = op->i[MK_MV_K], Kc = op->i[MK_MV_KC];
  const int wfmt = op->i[MK_MV_WFMT];
  const int k0 = p * Kc;
  const int kc = min(Kc, K - k0);
  const int64_t wrow = op->s[MK_MV_S_WROW];
  const int nrows = r.nA + r.nB;
  if (!mv_is_fp4(wfmt)) {
    const uint32_t seg = (uint32_t)kc * 2u;
    const uint32_t rs = (uint32_t)Kc * 2u + 64u;
    if (lane == 0) mbar_arrive_expect_tx(bar, seg * (uint32_t)nrows);
    __syncwarp();
    if (lane < 16) {
      const int g = lane & 7;
      const bool hi = lane >= 8;
      const bool valid = g < (hi ? r.nB : r.nA);
      if (valid) {
        const uint8_t* src = (hi ? r.wb : r.wa) + (int64_t)((hi ? r.rowB0 : r.rowA0) + g) * wrow + (int64_t)k0 * 2;
        bulk_g2s(page + (uint32_t)lane * rs, src, seg, bar);
      }
    }
  } else {
    const uint32_t pseg = (uint32_t)kc / 2u, sseg = (uint32_t)kc / 16u;
    const uint32_t ps = (uint32_t)Kc / 2u + 64u, ss = (uint32_t)Kc / 16u + 16u;
    const int64_t srow = op->s[MK_MV_S_SCROW];
    if (lane == 0) mbar_arrive_expect_tx(bar, (pseg + sseg) * (uint32_t)nrows);
    __syncwarp();
    const int v = lane & 15;
    const int g = v & 7;
    const bool hi = v >= 8;
    const bool valid = g < (hi ? r.nB : r.nA);
    if (valid) {
      const int row = (hi ? r.rowB0 : r.rowA0) + g;
      if (lane < 16) {
        const uint8_t* src = (hi ? r.wb : r.wa) + (int64_t)row * wrow + k0 / 2;
        bulk_g2s(page + (uint32_t)v * ps, src, pseg, bar);
      } else {
        const uint8_t* src = (hi ? r.sb : r.sa) + (int64_t)row * srow + k0 / 16;
        bulk_g2s(page + 16u * ps + (uint32_t)v * ss, src, sseg, bar);
      }
    }
  }
  if (lane != 0) mbar_arrive(bar);
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

// Stage pro(x) for all M rows into the shared activation buffer.  Called by
// all consumer threads (tid in [0, kConsumerWarps*32)); the caller places a
// consumer barrier before and after.  `stage` = fill the buffer,
// `write_res` = also materialise residual_out = x + residual_in in global.
__device__ __forceinline__ void mv_stage(Ctx& c, const mk_op_t* op, bool stage, bool write_res) {
  const int tid = (c.warp - 1) * 32 + c.lane;
  constexpr int T = kConsumerWarps * 32;
  const int K = op->i[MK_MV_K], M = op->i[MK_MV_M], S = op->i[MK_MV_S];
  const int pro = op->i[MK_MV_PRO];
  const int xt = op->i[MK_MV_X_T];
  const int at = mv_act_type(op);
  const uint32_t xs = (uint32_t)K * 2u + 64u;
  const int chunks = K >> 3;
  const uint16_t* x = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_X]);
  const uint16_t* ri = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_RES_IN]);
  uint16_t* ro = reinterpret_cast<uint16_t*>(op->p[MK_MV_P_RES_OUT]);
  const uint16_t* nw = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_NORM_W]);
  const bool add = (pro == MK_PRO_ADD_RMS) && ri != nullptr;
  write_res = write_res && add && ro != nullptr;
  if (!stage && !write_res) return;

  for (int m = 0; m < M; ++m) {
    const int b = m / S, s = m - b * S;
    const uint16_t* xr = x + b * op->s[MK_MV_S_X_B] + s * op->s[MK_MV_S_X_S];
    const uint16_t* rr = add ? ri + b * op->s[MK_MV_S_RI_B] + s * op->s[MK_MV_S_RI_S] : nullptr;
    uint16_t* wr = write_res ? ro + b * op->s[MK_MV_S_RO_B] + s * op->s[MK_MV_S_RO_S] : nullptr;
    float sum = 0.f;
    for (int ch = tid; ch < chunks; ch += T) {
      uint4 v = *reinterpret_cast<const uint4*>(xr + ch * 8);
      float f[8];
      unpack8(v, xt, f);
      if (add) {
        uint4 rv = *reinterpret_cast<const uint4*>(rr + ch * 8);
        float r[8];
        unpack8(rv, xt, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += r[i];
        round8(f, xt);
        v = pack8(f, xt);
        if (wr) *reinterpret_cast<uint4*>(wr + ch * 8) = v;
      }
      if (stage) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += f[i] * f[i];
        // keep the (rounded) input in its own type for now; pass 2 rescales
        sts128(c.act_u32 + (uint32_t)m * xs + (uint32_t)ch * 16u, v);
      }
    }
    if (stage && pro != MK_PRO_NONE) {
      sum = warp_sum(sum);
      if (c.lane == 0) c.ctrl->red[m * kConsumerWarps + (c.warp - 1)] = sum;
    }
  }
  if (!stage) return;
  if (pro == MK_PRO_NONE && xt == at) return;
  named_bar_sync(kConsumerBarrier, T);
  const float eps = op->f[MK_MV_F_EPS];
  for (int m = 0; m < M; ++m) {
    float rstd = 1.f;
    if (pro != MK_PRO_NONE) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) tot += c.ctrl->red[m * kConsumerWarps + w];
      rstd = rsqrtf(tot / (float)K + eps);
    }
    for (int ch = tid; ch < chunks; ch += T) {
      const uint32_t a = c.act_u32 + (uint32_t)m * xs + (uint32_t)ch * 16u;
      uint4 v = lds128(a);
      float f[8];
      unpack8(v, xt, f);
      if (pro != MK_PRO_NONE) {
        uint4 wv = *reinterpret_cast<const uint4*>(nw + ch * 8);
        float w[8];
        unpack8(wv, xt, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      }
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

__device__ __forceinline__ void mv_store(const mk_op_t* op, int m, int o, float v) {
  const int S = op->i[MK_MV_S], hd = op->i[MK_MV_HD];
  const int b = m / S, s = m - b * S;
  const int head = o / hd, dim = o - head * hd;
  const int64_t off = b * op->s[MK_MV_S_O_B] + (int64_t)(s + op->i[MK_MV_POS]) * op->s[MK_MV_S_O_S] +
                      head * op->s[MK_MV_S_O_H] + dim;
  if (op->i[MK_MV_EPI] == MK_EPI_RESIDUAL) {
    const uint16_t* er = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_EPI_RES]);
    const uint16_t rv = er[b * op->s[MK_MV_S_ER_B] + s * op->s[MK_MV_S_ER_S] + o];
    v += (op->i[MK_MV_X_T] == MK_T_BF16) ? bf16lo(rv) : f16lo(rv);
  }
  const int ot = op->i[MK_MV_OUT_T];
  if (ot == MK_T_FP32) {
    reinterpret_cast<float*>(op->p[MK_MV_P_OUT])[off] = v;
  } else if (ot == MK_T_BF16) {
    reinterpret_cast<uint16_t*>(op->p[MK_MV_P_OUT])[off] = (uint16_t)f2bf(v);
  } else {
    reinterpret_cast<uint16_t*>(op->p[MK_MV_P_OUT])[off] = (uint16_t)(pack_f16(v, 0.f) & 0xffffu);
  }
}

template <int NT>
__device__ __forceinline__ void mv_epilogue(Ctx& c, const mk_op_t* op, const MvRows& r, int unit,
                                            float (&acc)[NT][4]) {
  const int g = c.lane >> 2, t = c.lane & 3;
  const int M = op->i[MK_MV_M];
  const int tr = op->i[MK_MV_TR], epi = op->i[MK_MV_EPI];
  const float gs = (op->i[MK_MV_WFMT] == MK_W_NVFP4_E4M3S16) ? op->f[MK_MV_F_GSCALE] : 1.f;
  const bool va = g < r.nA, vb = g < r.nB;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = nt * 8 + 2 * t + e;
      const bool vm = m < M;
      float a = acc[nt][e] * gs, b = acc[nt][2 + e] * gs;
      if (tr == MK_TR_ROPE) {
        if (vm) {
          const int S = op->i[MK_MV_S], hd = op->i[MK_MV_HD];
          const int s = m % S;
          const int d = (r.rowA0 % hd) + g;
          const uint16_t* cs = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_COS]) + s * op->s[MK_MV_S_COS] + d;
          const uint16_t* sn = reinterpret_cast<const uint16_t*>(op->p[MK_MV_P_SIN]) + s * op->s[MK_MV_S_COS] + d;
          const bool bf = op->i[MK_MV_X_T] == MK_T_BF16;
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
      if (epi == MK_EPI_TOP1) {
        unsigned long long key = 0ull;
        if (va) key = top1_key(a, r.rowA0 + g);
        if (vb) {
          const unsigned long long kb = top1_key(b, r.rowB0 + g);
          key = kb > key ? kb : key;
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
          key = other > key ? other : key;
        }
        if (g == 0 && vm) atomicMax(reinterpret_cast<unsigned long long*>(op->p[MK_MV_P_OUT]) + m, key);
      } else if (vm) {
        if (tr == MK_TR_SILU_MUL) {
          if (va) mv_store(op, m, r.rowA0 + g, a);
        } else {
          if (va) mv_store(op, m, r.rowA0 + g, a);
          if (vb) mv_store(op, m, r.rowB0 + g, b);
        }
      }
    }
  }
}

// ---- consumer ---------------------------------------------------------------------
// fp4 (e2m1) pair in one byte -> f16x2 (low nibble -> low half).
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
  __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
  return (uint32_t)h.x | ((uint32_t)h.y << 16);
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int NT>
__device__ __forceinline__ void mv_unit(Ctx& c, const mk_op_t* op, const mk_instr_t& ins, uint32_t seq) {
  const int unit = ins.unit;
  const int g = c.lane >> 2, t = c.lane & 3;
  const int K = op->i[MK_MV_K], Kc = op->i[MK_MV_KC], M = op->i[MK_MV_M];
  const int wfmt = op->i[MK_MV_WFMT];
  const uint32_t xs = (uint32_t)K * 2u + 64u;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

  uint32_t xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + g;
    xok[nt] = m < M;
    xrow[nt] = c.act_u32 + (uint32_t)(xok[nt] ? m : 0) * xs;
  }

  const int np = ins.n_pages;  // pages of this unit
  for (int p = 0; p < np; ++p) {
    uint32_t page;
    if (!page_acquire(c, seq + p, page)) return;
    const int k0 = p * Kc;
    const int kc = min(Kc, K - k0);
    if (wfmt == MK_W_BF16 || wfmt == MK_W_FP16) {
      const uint32_t rs = (uint32_t)Kc * 2u + 64u;
      const uint32_t arow_lo = page + (uint32_t)g * rs + (uint32_t)t * 16u;
      const uint32_t arow_hi = arow_lo + 8u * rs;
      const uint32_t xoff = (uint32_t)(k0 + t * 8) * 2u;
      const int steps = kc >> 5;
#pragma unroll 4
      for (int ks = 0; ks < steps; ++ks) {
        const uint4 alo = lds128(arow_lo + (uint32_t)ks * 64u);
        const uint4 ahi = lds128(arow_hi + (uint32_t)ks * 64u);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          uint4 xb = make_uint4(0, 0, 0, 0);
          if (xok[nt]) xb = lds128(xrow[nt] + xoff + (uint32_t)ks * 64u);
          if (wfmt == MK_W_BF16) {
            mma_bf16(acc[nt], alo.x, ahi.x, alo.y, ahi.y, xb.x, xb.y);
            mma_bf16(acc[nt], alo.z, ahi.z, alo.w, ahi.w, xb.z, xb.w);
          } else {
            mma_f16(acc[nt], alo.x, ahi.x, alo.y, ahi.y, xb.x, xb.y);
            mma_f16(acc[nt], alo.z, ahi.z, alo.w, ahi.w, xb.z, xb.w);
          }
        }
      }
    } else {
      // NVFP4: per step each thread owns 32 consecutive K values of rows g and
      // g+8 (16 packed bytes each) and their block scales; values are scaled
      // in f16 (exact for e2m1 x e4m3) and fed to the f16 tensor-core path.
      const uint32_t ps = (uint32_t)Kc / 2u + 64u, ss = (uint32_t)Kc / 16u + 16u;
      const uint32_t prow_lo = page + (uint32_t)g * ps + (uint32_t)t * 16u;
      const uint32_t prow_hi = prow_lo + 8u * ps;
      const uint32_t srow_lo = page + 16u * ps + (uint32_t)g * ss + (uint32_t)t * 2u;
      const uint32_t srow_hi = srow_lo + 8u * ss;
      const uint32_t xoff = (uint32_t)(k0 + t * 32) * 2u;
      const int steps = kc >> 7;
#pragma unroll 1
      for (int ks = 0; ks < steps; ++ks) {
        const uint4 plo = lds128(prow_lo + (uint32_t)ks * 64u);
        const uint4 phi = lds128(prow_hi + (uint32_t)ks * 64u);
        const uint32_t slo_raw = lds16(srow_lo + (uint32_t)ks * 8u);
        const uint32_t shi_raw = lds16(srow_hi + (uint32_t)ks * 8u);
        uint32_t slo[2], shi[2];  // f16x2 broadcast scale for values [0,16) and [16,32)
        if (wfmt == MK_W_NVFP4_F16S32) {
          slo[0] = slo[1] = slo_raw | (slo_raw << 16);
          shi[0] = shi[1] = shi_raw | (shi_raw << 16);
        } else {
          __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)slo_raw, __NV_E4M3);
          __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)shi_raw, __NV_E4M3);
          slo[0] = (uint32_t)a.x | ((uint32_t)a.x << 16);
          slo[1] = (uint32_t)a.y | ((uint32_t)a.y << 16);
          shi[0] = (uint32_t)b.x | ((uint32_t)b.x << 16);
          shi[1] = (uint32_t)b.y | ((uint32_t)b.y << 16);
        }
        const uint32_t pl[4] = {plo.x, plo.y, plo.z, plo.w};
        const uint32_t ph[4] = {phi.x, phi.y, phi.z, phi.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // 8 values (4 bytes) of each row -> two mma k-slots
          uint32_t al[4], ah[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            al[j] = hmul2(e2m1x2_to_f16x2((pl[q] >> (8 * j)) & 0xffu), slo[q >> 1]);
            ah[j] = hmul2(e2m1x2_to_f16x2((ph[q] >> (8 * j)) & 0xffu), shi[q >> 1]);
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint4 xb = make_uint4(0, 0, 0, 0);
            if (xok[nt]) xb = lds128(xrow[nt] + xoff + (uint32_t)ks * 256u + (uint32_t)q * 16u);
            mma_f16(acc[nt], al[0], ah[0], al[1], ah[1], xb.x, xb.y);
            mma_f16(acc[nt], al[2], ah[2], al[3], ah[3], xb.z, xb.w);
          }
        }
      }
    }
    page_release(c, seq + p);
  }
  const MvRows r = mv_rows(op, unit);
  mv_epilogue<NT>(c, op, r, unit, acc);
}

__device__ __forceinline__ void mv_dispatch(Ctx& c, const mk_op_t* op, const mk_instr_t& ins, uint32_t seq) {
  const int M = op->i[MK_MV_M];
  if (M <= 8)
    mv_unit<1>(c, op, ins, seq);
  else if (M <= 16)
    mv_unit<2>(c, op, ins, seq);
  else
    mv_unit<4>(c, op, ins, seq);
}

}  // namespace mk
