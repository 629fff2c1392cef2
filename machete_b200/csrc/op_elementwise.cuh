// Row-wise ops that need no staged pages: RMSNorm variants, RoPE, per-head
// QK-norm + RoPE, GLU, add, and the top-1 finalise.  One warp per unit, plain
// vectorised global loads: each is a few KB per row and latency-bound.
//
// Numerics follow the reference's PyTorch oracles: rms_norm/ref.py:17-116,
// rope/ref.py:18-43 (split-half rotation, partial rotary tail untouched),
// qknorm_rope/ref.py:10-39 (normalised value rounded to the tensor dtype
// before the rotation), glu/ref.py:8-33.
#pragma once
#include "shell.cuh"

namespace mk {

__device__ __forceinline__ float ld_elem(const void* p, int64_t i, int ty) {
  if (ty == MK_T_FP32) return reinterpret_cast<const float*>(p)[i];
  const uint16_t v = reinterpret_cast<const uint16_t*>(p)[i];
  return ty == MK_T_BF16 ? bf16lo(v) : f16lo(v);
}
__device__ __forceinline__ void st_elem(void* p, int64_t i, int ty, float f) {
  if (ty == MK_T_FP32)
    reinterpret_cast<float*>(p)[i] = f;
  else if (ty == MK_T_BF16)
    reinterpret_cast<uint16_t*>(p)[i] = (uint16_t)f2bf(f);
  else
    reinterpret_cast<uint16_t*>(p)[i] = (uint16_t)(pack_f16(f, 0.f) & 0xffffu);
}
__device__ __forceinline__ float round_to(float f, int ty) {
  if (ty == MK_T_FP32) return f;
  if (ty == MK_T_BF16) return bf16lo(f2bf(f));
  return f16lo(pack_f16(f, 0.f));
}
__device__ __forceinline__ float silu_e(float x) { return x / (1.f + __expf(-x)); }

// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w  (+ variants).
__device__ __forceinline__ void ew_rmsnorm(Ctx& c, const mk_op_t* op, int unit) {
  const int D = op->i[MK_EW_D], ty = op->i[MK_EW_T], fl = op->i[MK_EW_FLAGS];
  const int rows = op->i[MK_EW_ROWS];
  const float eps = op->f[MK_EW_F_EPS];
  const int row = unit;
  if (row >= rows) return;
  const char* x = reinterpret_cast<const char*>(op->p[MK_EW_P_X]);
  const int esz = ty == MK_T_FP32 ? 4 : 2;
  const void* xr = x + row * op->s[MK_EW_S_X] * esz;
  void* yr = reinterpret_cast<char*>(op->p[MK_EW_P_Y]) + row * op->s[MK_EW_S_Y] * esz;
  const void* wr = reinterpret_cast<const char*>(op->p[MK_EW_P_W]) +
                   ((fl & MK_EWF_ROW_WEIGHT) ? row * op->s[MK_EW_S_W] * esz : 0);
  const void* rir = (fl & MK_EWF_FUSED_ADD)
                        ? reinterpret_cast<const char*>(op->p[MK_EW_P_RES_IN]) + row * op->s[MK_EW_S_RI] * esz
                        : nullptr;
  void* ror = (fl & MK_EWF_FUSED_ADD)
                  ? reinterpret_cast<char*>(op->p[MK_EW_P_RES_OUT]) + row * op->s[MK_EW_S_RO] * esz
                  : nullptr;
  const void* gr = (fl & MK_EWF_GATED)
                       ? reinterpret_cast<const char*>(op->p[MK_EW_P_GATE]) + row * op->s[MK_EW_S_G] * esz
                       : nullptr;
  float sum = 0.f;
  for (int d = c.lane; d < D; d += 32) {
    float v = ld_elem(xr, d, ty);
    if (rir) {
      v = round_to(v + ld_elem(rir, d, ty), ty);
      st_elem(ror, d, ty, v);
    }
    sum += v * v;
  }
  sum = warp_sum(sum);
  const float rstd = rsqrtf(sum / (float)D + eps);
  __syncwarp();
  for (int d = c.lane; d < D; d += 32) {
    // the summed residual was written by this same lane in the first pass;
    // reading it back keeps in-place residual_in/residual_out aliasing correct
    float v = rir ? ld_elem(ror, d, ty) : ld_elem(xr, d, ty);
    float w = ld_elem(wr, d, ty);
    if (fl & MK_EWF_GEMMA) w += 1.f;
    float y = v * rstd * w;
    if (fl & MK_EWF_RESIDUAL) y += v;
    if (gr) {
      y = round_to(y, ty);  // oracle rounds the normalised value before gating
      y *= silu_e(ld_elem(gr, d, ty));
    }
    st_elem(yr, d, ty, y);
  }
}

// RoPE in place on q[B,S,NH,HD]; unit = one (b, s) row, all heads.
__device__ __forceinline__ void ew_rope(Ctx& c, const mk_op_t* op, int unit) {
  const int S = op->i[MK_EW_S], NH = op->i[MK_EW_H], D2 = op->i[MK_EW_D2], ty = op->i[MK_EW_T];
  const int esz = ty == MK_T_FP32 ? 4 : 2;
  const int s = unit % S;
  char* q = reinterpret_cast<char*>(op->p[MK_EW_P_X]) + unit * op->s[MK_EW_S_X] * esz;
  const void* cs = reinterpret_cast<const char*>(op->p[MK_EW_P_COS]) + s * op->s[MK_EW_S_COS] * esz;
  const void* sn = reinterpret_cast<const char*>(op->p[MK_EW_P_SIN]) + s * op->s[MK_EW_S_COS] * esz;
  for (int idx = c.lane; idx < NH * D2; idx += 32) {
    const int h = idx / D2, d = idx - h * D2;
    void* qh = q + h * op->s[MK_EW_S_X_H] * esz;
    const float q0 = ld_elem(qh, d, ty), q1 = ld_elem(qh, d + D2, ty);
    const float cv = ld_elem(cs, d, ty), sv = ld_elem(sn, d, ty);
    st_elem(qh, d, ty, q0 * cv - q1 * sv);
    st_elem(qh, d + D2, ty, q1 * cv + q0 * sv);
  }
}

// Per-head RMSNorm then RoPE, in place on q[M,H,D]; unit = (m, h).
__device__ __forceinline__ void ew_qknorm_rope(Ctx& c, const mk_op_t* op, int unit) {
  const int H = op->i[MK_EW_H], D = op->i[MK_EW_D], D2 = op->i[MK_EW_D2], ty = op->i[MK_EW_T];
  const int esz = ty == MK_T_FP32 ? 4 : 2;
  const float eps = op->f[MK_EW_F_EPS];
  const int m = unit / H, h = unit - m * H;
  char* q = reinterpret_cast<char*>(op->p[MK_EW_P_X]) + (m * op->s[MK_EW_S_X] + h * op->s[MK_EW_S_X_H]) * esz;
  const void* w = reinterpret_cast<const void*>(op->p[MK_EW_P_W]);
  const void* cs = reinterpret_cast<const char*>(op->p[MK_EW_P_COS]) + m * op->s[MK_EW_S_COS] * esz;
  const void* sn = reinterpret_cast<const char*>(op->p[MK_EW_P_SIN]) + m * op->s[MK_EW_S_COS] * esz;
  float sum = 0.f;
  for (int d = c.lane; d < D; d += 32) {
    const float v = ld_elem(q, d, ty);
    sum += v * v;
  }
  sum = warp_sum(sum);
  const float rstd = rsqrtf(sum / (float)D + eps);
  __syncwarp();
  // rotated part: pairs (d, d + D2); tail [2*D2, D) only normalised
  for (int d = c.lane; d < D2; d += 32) {
    const float n0 = round_to(ld_elem(q, d, ty) * rstd * ld_elem(w, d, ty), ty);
    const float n1 = round_to(ld_elem(q, d + D2, ty) * rstd * ld_elem(w, d + D2, ty), ty);
    const float cv = ld_elem(cs, d, ty), sv = ld_elem(sn, d, ty);
    st_elem(q, d, ty, n0 * cv - n1 * sv);
    st_elem(q, d + D2, ty, n1 * cv + n0 * sv);
  }
  for (int d = 2 * D2 + c.lane; d < D; d += 32) st_elem(q, d, ty, ld_elem(q, d, ty) * rstd * ld_elem(w, d, ty));
}

// GLU: y[.., d] = act(x[.., d]) * x[.., D + d]; unit = one row.
__device__ __forceinline__ void ew_glu(Ctx& c, const mk_op_t* op, int unit) {
  const int D = op->i[MK_EW_D], ty = op->i[MK_EW_T], act = op->i[MK_EW_ACT];
  const int esz = ty == MK_T_FP32 ? 4 : 2;
  const void* x = reinterpret_cast<const char*>(op->p[MK_EW_P_X]) + unit * op->s[MK_EW_S_X] * esz;
  void* y = reinterpret_cast<char*>(op->p[MK_EW_P_Y]) + unit * op->s[MK_EW_S_Y] * esz;
  for (int d = c.lane; d < D; d += 32) {
    float gv = ld_elem(x, d, ty);
    const float uv = ld_elem(x, D + d, ty);
    if (act == MK_TR_SILU)
      gv = silu_e(gv);
    else if (act == MK_TR_RELU)
      gv = fmaxf(gv, 0.f);
    st_elem(y, d, ty, gv * uv);
  }
}

// Add: y = x + w (second operand in the W slot); unit = one row.
__device__ __forceinline__ void ew_add(Ctx& c, const mk_op_t* op, int unit) {
  const int D = op->i[MK_EW_D], ty = op->i[MK_EW_T];
  const int esz = ty == MK_T_FP32 ? 4 : 2;
  const void* x = reinterpret_cast<const char*>(op->p[MK_EW_P_X]) + unit * op->s[MK_EW_S_X] * esz;
  const void* a = reinterpret_cast<const char*>(op->p[MK_EW_P_W]) + unit * op->s[MK_EW_S_W] * esz;
  void* y = reinterpret_cast<char*>(op->p[MK_EW_P_Y]) + unit * op->s[MK_EW_S_Y] * esz;
  for (int d = c.lane; d < D; d += 32) st_elem(y, d, ty, ld_elem(x, d, ty) + ld_elem(a, d, ty));
}

// Top-1 finalise: unpack keys[m] -> (value, index) and clear the keys so the
// next launch starts from zero.  One unit handles all rows.
__device__ __forceinline__ void ew_top1_final(Ctx& c, const mk_op_t* op, int unit) {
  const int rows = op->i[MK_EW_ROWS];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(op->p[MK_EW_P_X]);
  float* vals = reinterpret_cast<float*>(op->p[MK_EW_P_Y]);
  int32_t* idxs = reinterpret_cast<int32_t*>(op->p[MK_EW_P_W]);
  for (int m = c.lane; m < rows; m += 32) {
    const unsigned long long k = atomicExch(keys + m, 0ull);
    uint32_t b = (uint32_t)(k >> 32);
    b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
    if (vals) vals[m] = __uint_as_float(b);
    idxs[m] = (int32_t)(0xffffffffu - (uint32_t)(k & 0xffffffffull));
  }
  (void)unit;
  if (op->i[MK_EW_FLAGS] & MK_EWF_FEEDBACK) {
    // Feed the greedy token back: its embedding row becomes the next launch's input row, and
    // the device-resident cache position moves on.  Every other unit of this launch is complete
    // (this op waits for the whole LM head), so nothing still reads either of them.
    __syncwarp();
    const int D = op->i[MK_EW_D];
    const uint16_t* emb = reinterpret_cast<const uint16_t*>(op->p[MK_EW_P_RES_IN]);
    uint16_t* xin = reinterpret_cast<uint16_t*>(op->p[MK_EW_P_RES_OUT]);
    for (int m = 0; m < rows; ++m) {
      const int tok = *reinterpret_cast<volatile int32_t*>(idxs + m);
      const uint4* src = reinterpret_cast<const uint4*>(emb + (int64_t)tok * op->s[MK_EW_S_RI]);
      uint4* dst = reinterpret_cast<uint4*>(xin + (int64_t)m * op->s[MK_EW_S_RO]);
      for (int ch = c.lane; ch < D / 8; ch += 32) dst[ch] = src[ch];
    }
    int32_t* pos = reinterpret_cast<int32_t*>(op->p[MK_EW_P_GATE]);
    if (pos != nullptr && c.lane < c.pv->pos_count) pos[c.lane] += op->i[MK_EW_S];   // every sequence moves on
  }
}

}  // namespace mk
