// Split-KV flash decoding for one KV head per unit, and the log-sum-exp combine.
//
// A unit is (batch b, kv head, 16-row query tile, split).  The 16 rows of the
// tile enumerate (query position m, query head within the GQA group), so at
// decode (M = 1) one unit serves every query head that shares the KV head and
// each K/V byte is fetched once — the reference tiles per *query* head and
// re-reads each KV head `group` times (attention/flash_decoding.py:1192, 1324).
//
// K and V token rows arrive in a ring page by tiled TMA with the 128-byte
// swizzle, which makes ldmatrix bank-conflict free; scores and P·V
// run on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with an exp2 online
// softmax.  Partials follow the reference's contract: normalised fp32
// o_partial[B,H,SPLIT,M,D] and lse_partial[B,H,SPLIT,M] = max*scale + ln(sum)
// (attention/flash_decoding.py:1139-1172); the combine implements
// o = sum_s e^{lse_s-max} o_s / sum_s e^{lse_s-max} (:1858-1950).
#pragma once
#include "shell.cuh"

namespace mk {

struct AtUnit {
  int b, kvh, mt, sp;
  int t_begin, t_end;  // token range of the split
};

__device__ __forceinline__ AtUnit at_decode(const mk_op_t* op, int unit) {
  AtUnit u;
  const int S = op->i[MK_AT_SPLITS], MT = op->i[MK_AT_MT], HKV = op->i[MK_AT_HKV];
  u.sp = unit % S;
  int r = unit / S;
  u.mt = r % MT;
  r /= MT;
  u.kvh = r % HKV;
  u.b = r / HKV;
  const int ts = op->i[MK_AT_TS], N = op->i[MK_AT_N];
  u.t_begin = min(N, u.sp * ts);
  u.t_end = min(N, u.t_begin + ts);
  return u;
}
// The same from the instruction record, where mk_create has left the result
// of the divisions: row_a = first token, row_b = kv head | batch << 16,
// off_a = split, off_b = query tile.
__device__ __forceinline__ AtUnit at_decode_fast(const mk_op_t* op, const UnitArgs& a) {
  AtUnit u;
  const int rb = ins_field(a.mine->row_b, a.idx);
  u.t_begin = ins_field(a.mine->row_a, a.idx);
  u.sp = ins_field(a.mine->off_a, a.idx);
  u.mt = ins_field(a.mine->off_b, a.idx);
  u.kvh = rb & 0xffff;
  u.b = rb >> 16;
  u.t_end = u.t_begin + op->i[MK_AT_TS];   // the caller clips both to the window
  return u;
}

// Tokens per page for head dim D and a given page size: a K block and a V
// block of `tn` rows each; tn is a multiple of the consumer's inner block
// (64 tokens for D = 64, 32 for D = 128) and at most 64: a split of a few
// hundred tokens then spans several pages, which several consumer warps share.
__device__ __host__ __forceinline__ int at_page_tokens(int D, int page_bytes) {
  const int blk = (D == 64) ? 64 : 32;
  int tn = page_bytes / (4 * D);
  tn = (tn / blk) * blk;
  return tn > 64 ? 64 : tn;
}

// ---- loader -----------------------------------------------------------------------
// Page layout: a K tile followed by a V tile.  A tile is D/64 sub-tiles of
// [tn token rows][128 bytes] (64 head-dim values each), written by tiled TMA
// with the 128-byte swizzle: 16-byte chunk c of token row r sits at
// r*128 + ((c ^ (r & 7)) << 4), which is what ldmatrix wants (8 rows of a
// matrix hit 8 different bank groups).  Tokens past the end of the cache are
// zero-filled by TMA; tokens past the end of the split are masked by the
// consumer.  Called by loader lane 0 only.
__device__ __forceinline__ void at_load_issue(const void* tm_k, const void* tm_v, bool d128, int tn, int tok0, int kvh,
                                              int b, uint32_t page, uint32_t bar, uint64_t policy) {
  const uint32_t sub = (uint32_t)tn * 128u;
  const uint32_t tile = d128 ? 2u * sub : sub;
  mbar_expect_tx(bar, 2u * tile);
  tma_load_4d(page, tm_k, 0, kvh, tok0, b, bar, policy);
  if (d128) tma_load_4d(page + sub, tm_k, 64, kvh, tok0, b, bar, policy);
  tma_load_4d(page + tile, tm_v, 0, kvh, tok0, b, bar, policy);
  if (d128) tma_load_4d(page + tile + sub, tm_v, 64, kvh, tok0, b, bar, policy);
  mbar_arrive_n(bar, 32);
}

__device__ __forceinline__ uint32_t at_chunk_addr(uint32_t tile, int tn, int tok, int chunk) {
  return tile + (uint32_t)(chunk >> 3) * (uint32_t)tn * 128u + (uint32_t)tok * 128u +
         (uint32_t)(((chunk & 7) ^ (tok & 7)) << 4);
}

// ---- fused combine ----------------------------------------------------------------
__device__ __forceinline__ float ldcg_f(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ldcg_f4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Combine all splits of one (batch, kv head, query tile) group: the same sum
// as the combine op (weights e^{lse_s - max} / sum, splits added in order), for
// every query row of the tile at once.  A row is spread over D/8 lanes of 8
// output values each, so 32/(D/8) rows are in flight together and all of a
// pass's partial rows are requested in two batches.  The partials were written
// by other CTAs and fenced before their arrival was counted: they are read
// past L1.
template <int D>
__device__ __forceinline__ void at_combine_group(Ctx& c, const mk_op_t* op, const AtUnit& u) {
  constexpr int LPR = D / 8, RPP = 32 / LPR, UN = 9;
  const int M = op->i[MK_AT_M], H = op->i[MK_AT_H], HKV = op->i[MK_AT_HKV], S = op->i[MK_AT_SPLITS];
  const int G = op->i[MK_AT_GROUP];
  const float* opart = reinterpret_cast<const float*>(op->p[MK_AT_P_OPART]);
  const float* lpart = reinterpret_cast<const float*>(op->p[MK_AT_P_LSEPART]);
  float* lse_out = reinterpret_cast<float*>(op->p[MK_AT_P_LSE]);
  const int ot = op->i[MK_AT_O_T];
  // this warp's 2 KB of the split-K slot area (no matvec unit runs beside an attention op's units)
  float* scratch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.ctrl) + kCtrlStructBytes) + (c.warp - 1) * 512;
  const int rows = min(16, M * G - u.mt * 16);
  const int row = c.lane / LPR, dch = (c.lane % LPR) * 8;
#pragma unroll 1
  for (int r0 = 0; r0 < rows; r0 += RPP) {
    const int nr = min(RPP, rows - r0);
    const bool rv = row < nr;
    const int r = u.mt * 16 + r0 + (rv ? row : 0);
    const int m = M != 1 ? r / G : 0, h = u.kvh * G + (M != 1 ? r % G : r);
    const float* base = opart + ((((int64_t)u.b * H + h) * S) * M + m) * D + dch;
    const int64_t sstride = (int64_t)M * D;
    const float* ls = scratch + (rv ? row : 0) * S;
    float mx = -INFINITY, sum = 0.f, inv = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // One code path per batch of UN splits (kept rolled: this runs once per KV head and launch,
    // always from a cold instruction cache).  The first batch of partial rows is requested
    // together with the lse values: neither depends on the other, so they share one trip.
#pragma unroll 1
    for (int s0 = 0; s0 < S; s0 += UN) {
      float4 a[UN], b2[UN];
#pragma unroll
      for (int k = 0; k < UN; ++k) {
        a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        b2[k] = a[k];
        if (rv && s0 + k < S) {
          a[k] = ldcg_f4(base + (s0 + k) * sstride);
          b2[k] = ldcg_f4(base + (s0 + k) * sstride + 4);
        }
      }
      if (s0 == 0) {
        if (M == 1) {
          // one query token: the group's lse values are contiguous, (row, split) -> row * S + split
          const float* l0 = lpart + ((int64_t)u.b * H + (int64_t)u.kvh * G + u.mt * 16 + r0) * S;
          float lv[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) lv[q] = (c.lane + 32 * q < nr * S) ? ldcg_f(l0 + c.lane + 32 * q) : 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (c.lane + 32 * q < nr * S) scratch[c.lane + 32 * q] = lv[q];
        } else {
#pragma unroll 1
        for (int i = c.lane; i < nr * S; i += 32) {
          const int rr = i / S, s = i - rr * S, r2 = u.mt * 16 + r0 + rr;
          const int m2 = r2 / G, h2 = u.kvh * G + r2 % G;
          scratch[i] = ldcg_f(lpart + (((int64_t)u.b * H + h2) * S + s) * M + m2);
        }
        }
        __syncwarp();
        // The row's LPR lanes take the splits in turn: the maximum by shuffle (exact in any order), each
        // e^{lse_s - max} once, written over its lse value; the sum then adds them in split order.  (One
        // lane walking all S values waits for a shared-memory load and an exponential per step.)
        const int li = c.lane % LPR;
#pragma unroll 1
        for (int s = li; s < S; s += LPR) mx = fmaxf(mx, ls[s]);
#pragma unroll
        for (int o = 1; o < LPR; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (rv) {
#pragma unroll 1
          for (int s = li; s < S; s += LPR) scratch[row * S + s] = mx != -INFINITY ? __expf(ls[s] - mx) : 0.f;
        }
        __syncwarp();
#pragma unroll 1
        for (int s = 0; s < S; ++s) sum += ls[s];
        inv = sum > 0.f ? 1.f / sum : 0.f;
      } else {
        trace(c, TRC_AT_FETCHED, (uint32_t)r0);
      }
#pragma unroll
      for (int k = 0; k < UN; ++k) {
        if (s0 + k >= S) break;
        const float w = ls[s0 + k] * inv;
        acc[0] += w * a[k].x; acc[1] += w * a[k].y; acc[2] += w * a[k].z; acc[3] += w * a[k].w;
        acc[4] += w * b2[k].x; acc[5] += w * b2[k].y; acc[6] += w * b2[k].z; acc[7] += w * b2[k].w;
      }
    }
    if (rv) {
      const int64_t ooff = u.b * op->s[MK_AT_S_O_B] + m * op->s[MK_AT_S_O_M] + h * op->s[MK_AT_S_O_H] + dch;
      if (ot == MK_T_FP32) {
        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(op->p[MK_AT_P_O]) + ooff);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          w[i] = ot == MK_T_BF16 ? pack_bf16(acc[2 * i], acc[2 * i + 1]) : pack_f16(acc[2 * i], acc[2 * i + 1]);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(op->p[MK_AT_P_O]) + ooff) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (dch == 0 && lse_out) lse_out[((int64_t)u.b * H + h) * M + m] = (sum > 0.f) ? mx + __logf(sum) : -INFINITY;
    }
    __syncwarp();
  }
}

// ---- fused per-head RMSNorm + rotation of the new k row ------------------------------
// The row sits unrotated in the K tile of the page (and in the cache).  Lanes
// below D/16 take chunks l and l + D/16 (values d and d + D/2, the two halves a
// split-half rotation pairs); the finished row replaces the raw one in shared
// memory and in the cache.  Arithmetic as the stand-alone op: the normalised
// value is rounded to bf16 before the rotation, the rotated one once more.
__device__ __forceinline__ void at_unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16lo(w[i]);
    f[2 * i + 1] = bf16hi(w[i]);
  }
}
__device__ __forceinline__ uint4 at_pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
template <int D>
__device__ __forceinline__ void at_fix_k_row(Ctx& c, const mk_op_t* op, const AtUnit& u, uint32_t kpage, int tn, int row,
                                             int tok, int64_t tab_off) {
  constexpr int HALF = D / 16;
  const bool act = c.lane < HALF;
  const int l = act ? c.lane : 0;
  const uint32_t a0 = at_chunk_addr(kpage, tn, row, l), a1 = at_chunk_addr(kpage, tn, row, l + HALF);
  float fa[8], fb[8];
  at_unpack8(lds128_sync(a0), fa);
  at_unpack8(lds128_sync(a1), fb);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += fa[i] * fa[i] + fb[i] * fb[i];
  ss = warp_sum(act ? ss : 0.f);
  const float rstd = rsqrtf(ss / (float)D + op->f[MK_AT_F_EPS]);
  const uint16_t* nw = reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_KNW]);
  float wa[8], wb[8], cv[8], sv[8];
  at_unpack8(*reinterpret_cast<const uint4*>(nw + 8 * l), wa);
  at_unpack8(*reinterpret_cast<const uint4*>(nw + 8 * l + D / 2), wb);
  at_unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_COS]) + tab_off + 8 * l), cv);
  at_unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_SIN]) + tab_off + 8 * l), sv);
  float o0[8], o1[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float n0 = bf16_round(fa[i] * rstd * wa[i]), n1 = bf16_round(fb[i] * rstd * wb[i]);
    o0[i] = n0 * cv[i] - n1 * sv[i];
    o1[i] = n1 * cv[i] + n0 * sv[i];
  }
  if (act) {
    const uint4 p0 = at_pack8(o0), p1 = at_pack8(o1);
    sts128(a0, p0);
    sts128(a1, p1);
    uint16_t* k = reinterpret_cast<uint16_t*>(op->p[MK_AT_P_K]) + u.b * op->s[MK_AT_S_K_B] +
                  (int64_t)tok * op->s[MK_AT_S_K_N] + u.kvh * op->s[MK_AT_S_K_H];
    *reinterpret_cast<uint4*>(k + 8 * l) = p0;
    *reinterpret_cast<uint4*>(k + 8 * l + D / 2) = p1;
  }
  // the page goes back to the loader later: order these writes before its next TMA fill
  fence_proxy_async();
  __syncwarp();
}

// ---- consumer ---------------------------------------------------------------------
// The unit's pages (blocks of tn tokens) are dealt round-robin to `parts`
// consumer warps; each keeps its own online-softmax state (row max, row sum,
// unnormalised output).  A participant parks its state in the last page it
// consumed instead of handing that page back; the last one to arrive merges
// the states in participant order, writes the normalised partial and then
// releases everybody's parked page.  Returns true for the warp that finished
// the unit.
// QMODE 0: the fused q/k norm is compiled out (kernels for bf16-only programs); 1: decided per op.
template <int D, int QMODE>
__device__ __forceinline__ bool at_unit(Ctx& c, const mk_op_t* op, const UnitArgs& ua) {
  constexpr int KS = D / 16;   // k-steps of Q·K^T
  constexpr int ND = D / 8;    // n-tiles of the output
  constexpr int TN = (D == 64) ? 64 : 32;  // tokens processed per inner block
  constexpr int NS = TN / 8;   // score n-tiles per block
  const int part = ua.part;
  const uint32_t ord = ua.ord;
  const int parts = (ua.flags >> MK_LDF_SPLIT_SHIFT) & MK_LDF_SPLIT_MASK;
  AtUnit u = at_decode_fast(op, ua);
  const int g = c.lane >> 2, t = c.lane & 3;
  const int M = op->i[MK_AT_M], H = op->i[MK_AT_H], HKV = op->i[MK_AT_HKV];
  // the window: the scheduled length, or (device-resident position) every token up to this step's
  const bool dyn = op->i[MK_AT_DYNPOS] != 0;
  const int N = dyn ? min(op->i[MK_AT_N], c.ctrl->pos[u.b & 31] + M) : op->i[MK_AT_N];
  u.t_begin = min(u.t_begin, N);
  u.t_end = min(u.t_end, N);
  const int G = op->i[MK_AT_GROUP];
  const int S = op->i[MK_AT_SPLITS];
  const bool causal = op->i[MK_AT_CAUSAL] != 0;
  const float sc = op->f[MK_AT_F_SCALE];
  const float c2 = sc * 1.4426950408889634f;
  const int tn = at_page_tokens(D, c.pv->page_bytes);
  const uint32_t tile_bytes = (uint32_t)tn * (uint32_t)D * 2u;
  const int NPG = c.pv->n_pages;

  // rows of this thread: r0 = mt*16 + g, r1 = r0 + 8 -> (m, head)
  int rm[2], rh[2];
  bool rv[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = u.mt * 16 + g + 8 * e;
    rv[e] = r < M * G;
    // one token per sequence (decode): row r is head r of the group, no division
    rm[e] = (rv[e] && M != 1) ? r / G : 0;
    rh[e] = u.kvh * G + (rv[e] ? (M != 1 ? r % G : r) : 0);
  }
  // Q fragments (A operand), loaded straight from global.
  uint32_t qf[KS][4];
  {
    const uint16_t* q = reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_Q]) + u.b * op->s[MK_AT_S_Q_B];
    const uint16_t* q0 = q + rm[0] * op->s[MK_AT_S_Q_M] + rh[0] * op->s[MK_AT_S_Q_H];
    const uint16_t* q1 = q + rm[1] * op->s[MK_AT_S_Q_M] + rh[1] * op->s[MK_AT_S_Q_H];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int col = ks * 16 + 2 * t;
      qf[ks][0] = rv[0] ? *reinterpret_cast<const uint32_t*>(q0 + col) : 0u;
      qf[ks][1] = rv[1] ? *reinterpret_cast<const uint32_t*>(q1 + col) : 0u;
      qf[ks][2] = rv[0] ? *reinterpret_cast<const uint32_t*>(q0 + col + 8) : 0u;
      qf[ks][3] = rv[1] ? *reinterpret_cast<const uint32_t*>(q1 + col + 8) : 0u;
    }
  }
  const bool qknorm = QMODE == 0 ? false : op->i[MK_AT_QKNORM] != 0;
  if (qknorm) {
    // q arrives unrotated: per-head RMSNorm (rounded to bf16), then the split-half
    // rotation.  A row's D values sit in the four lanes of a quad; value d and its
    // partner d + D/2 are k-steps ks and ks + KS/2 of the same lane.
    const uint16_t* nw = reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_QNW]);
    // a device-resident position picks the table row (MK_AT_NEW_TOK then holds the row stride)
    const int64_t tab_off = dyn ? (int64_t)c.ctrl->pos[u.b & 31] * op->i[MK_AT_NEW_TOK] : 0;
    const uint16_t* cs = reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_COS]) + tab_off;
    const uint16_t* sn = reinterpret_cast<const uint16_t*>(op->p[MK_AT_P_SIN]) + tab_off;
    // the tables do not depend on q: request them first, so that they share q's round trip
    uint32_t tw0[KS / 2][2], tw1[KS / 2][2], tcs[KS / 2][2], tsn[KS / 2][2];
#pragma unroll
    for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int col = ks * 16 + 2 * t + 8 * h2;
        tw0[ks][h2] = *reinterpret_cast<const uint32_t*>(nw + col);
        tw1[ks][h2] = *reinterpret_cast<const uint32_t*>(nw + col + D / 2);
        tcs[ks][h2] = *reinterpret_cast<const uint32_t*>(cs + col);
        tsn[ks][h2] = *reinterpret_cast<const uint32_t*>(sn + col);
      }
    float ss[2] = {0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float lo = bf16lo(qf[ks][r]), hi = bf16hi(qf[ks][r]);
        ss[r & 1] += lo * lo + hi * hi;
      }
    float rstd[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 1);
      ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 2);
      rstd[e] = rsqrtf(ss[e] / (float)D + op->f[MK_AT_F_EPS]);
    }
#pragma unroll
    for (int ks = 0; ks < KS / 2; ++ks) {
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t w0 = tw0[ks][h2], w1 = tw1[ks][h2], cc = tcs[ks][h2], sc2 = tsn[ks][h2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t r0 = qf[ks][e + 2 * h2], r1 = qf[ks + KS / 2][e + 2 * h2];
          const float n0l = bf16_round(bf16lo(r0) * rstd[e] * bf16lo(w0)), n0h = bf16_round(bf16hi(r0) * rstd[e] * bf16hi(w0));
          const float n1l = bf16_round(bf16lo(r1) * rstd[e] * bf16lo(w1)), n1h = bf16_round(bf16hi(r1) * rstd[e] * bf16hi(w1));
          const float cl = bf16lo(cc), ch = bf16hi(cc), sl = bf16lo(sc2), sh = bf16hi(sc2);
          qf[ks][e + 2 * h2] = pack_bf16(n0l * cl - n1l * sl, n0h * ch - n1h * sh);
          qf[ks + KS / 2][e + 2 * h2] = pack_bf16(n1l * cl + n0l * sl, n1h * ch + n0h * sh);
        }
      }
    }
  }
  // causal limit per row: token index <= N - M + m
  int lim[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) lim[e] = causal ? (N - M + rm[e]) : (N - 1);

  float o[ND][4];
#pragma unroll
  for (int i = 0; i < ND; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY};
  float lrow[2] = {0.f, 0.f};   // per-lane partial row sums (summed over the quad at the end)

  const int np = ua.n_pages;
  RingPos rp = ua.rp;
  uint32_t park = 0;            // address of the page this warp keeps for its state
  for (int p = part; p < np; p += parts, ring_advance(rp, parts, NPG)) {
    uint32_t page;
    if (!page_acquire(c, rp, page)) return false;
    trace(c, TRC_PAGE_READY, rp.k * (uint32_t)NPG + rp.slot);
    const uint32_t kpage = page, vpage = page + tile_bytes;
    const int tp0 = u.t_begin + p * tn;
    if (qknorm) {
      const int nt = dyn ? c.ctrl->pos[u.b & 31] : op->i[MK_AT_NEW_TOK];
      if (nt >= tp0 && nt < tp0 + tn && nt < u.t_end)
        at_fix_k_row<D>(c, op, u, kpage, tn, nt - tp0, nt, dyn ? (int64_t)nt * op->i[MK_AT_NEW_TOK] : 0);
    }
    for (int blk = 0; blk * TN < tn; ++blk) {
      const int tb0 = tp0 + blk * TN;       // global token of column 0 of the block
      if (tb0 >= u.t_end) break;
      const int lt0 = blk * TN;             // token row inside the page
      float s[NS][4];
#pragma unroll
      for (int i = 0; i < NS; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
      // S = Q K^T
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int pr = 0; pr < NS / 2; ++pr) {
          const int mat = c.lane >> 3, r = c.lane & 7;
          const int tok = lt0 + pr * 16 + (mat >> 1) * 8 + r;
          const int chunk = 2 * ks + (mat & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(at_chunk_addr(kpage, tn, tok, chunk), b0, b1, b2, b3);
          mma_bf16(s[2 * pr], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
          mma_bf16(s[2 * pr + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
        }
      }
      // mask + row max
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < NS; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tb0 + i * 8 + 2 * t + (e & 1);
          const int row = e >> 1;
          if (tok >= u.t_end || tok > lim[row]) s[i][e] = -INFINITY;
          mx[row] = fmaxf(mx[row], s[i][e]);
        }
      }
      float corr[2], muse[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
        mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
        const float mnew = fmaxf(mrow[e], mx[e]);
        muse[e] = (mnew == -INFINITY) ? 0.f : mnew;
        corr[e] = fast_exp2((mrow[e] - muse[e]) * c2);
        mrow[e] = mnew;
        lrow[e] *= corr[e];
      }
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      // P = exp2(S*c2 - m*c2), packed as bf16 A fragments
      uint32_t pf[NS / 2][4];
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = e >> 1;
          pv[e] = fast_exp2(s[i][e] * c2 - muse[row] * c2);
          lrow[row] += pv[e];
        }
        pf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < NS / 2; ++kk) {
#pragma unroll
        for (int dp = 0; dp < ND / 2; ++dp) {
          const int mat = c.lane >> 3, r = c.lane & 7;
          const int tok = lt0 + kk * 16 + (mat & 1) * 8 + r;
          const int chunk = 2 * dp + (mat >> 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(at_chunk_addr(vpage, tn, tok, chunk), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b0, b1);
          mma_bf16(o[2 * dp + 1], pf[kk][0], pf[kk][1], pf[kk][2], pf[kk][3], b2, b3);
        }
      }
    }
    trace(c, TRC_PAGE_DONE, rp.k * (uint32_t)NPG + rp.slot);
    if (parts > 1 && p + parts >= np)
      park = page;              // the last page of this participant: keep it
    else
      page_release(c, rp);
  }

  if (parts > 1) {
    // park (o, m, l) in the kept page: 16-byte record (i*32 + lane) holds o[i][0..3], the last one (m, m, l, l)
    const int sets_log2 = __ffs(c.pv->mv_sets) - 1;                      // 1, 2 or 4 slot sets
    const uint32_t set = ord & (uint32_t)(c.pv->mv_sets - 1), gen = ord >> sets_log2;
    if (!wait_smem_ge(c, &c.ctrl->mv_done[set], gen, (int)ord)) return false;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ND; ++i)
      sts128(park + (uint32_t)(i * 32 + c.lane) * 16u,
             make_uint4(__float_as_uint(o[i][0]), __float_as_uint(o[i][1]), __float_as_uint(o[i][2]),
                        __float_as_uint(o[i][3])));
    sts128(park + (uint32_t)(ND * 32 + c.lane) * 16u,
           make_uint4(__float_as_uint(mrow[0]), __float_as_uint(mrow[1]), __float_as_uint(lrow[0]),
                      __float_as_uint(lrow[1])));
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
    // merge in participant order
#pragma unroll
    for (int i = 0; i < ND; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    mrow[0] = mrow[1] = -INFINITY;
    lrow[0] = lrow[1] = 0.f;
    // last page of participant j: the largest p = j (mod parts) below np — one division for all of them
    const int lq = (np - 1) / parts, lr = (np - 1) - lq * parts;
#pragma unroll 1
    for (int j = 0; j < parts; ++j) {
      const int pl = j + (j <= lr ? lq : lq - 1) * parts;
      RingPos rj = ua.rp0;
      ring_advance(rj, pl, NPG);
      const uint32_t src = c.pages_u32 + rj.slot * (uint32_t)c.pv->page_bytes;
      float wa[2], wb[2];
      // all of a participant's records are requested before the first is used
      const uint4 ml = lds128_sync(src + (uint32_t)(ND * 32 + c.lane) * 16u);
      uint4 v[ND];
#pragma unroll
      for (int i = 0; i < ND; ++i) v[i] = lds128_sync(src + (uint32_t)(i * 32 + c.lane) * 16u);
      const float mj[2] = {__uint_as_float(ml.x), __uint_as_float(ml.y)};
      const float lj[2] = {__uint_as_float(ml.z), __uint_as_float(ml.w)};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float mnew = fmaxf(mrow[e], mj[e]);
        const float muse = (mnew == -INFINITY) ? 0.f : mnew;
        wa[e] = fast_exp2((mrow[e] - muse) * c2);
        wb[e] = fast_exp2((mj[e] - muse) * c2);
        mrow[e] = mnew;
        lrow[e] = lrow[e] * wa[e] + lj[e] * wb[e];
      }
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        o[i][0] = o[i][0] * wa[0] + __uint_as_float(v[i].x) * wb[0];
        o[i][1] = o[i][1] * wa[0] + __uint_as_float(v[i].y) * wb[0];
        o[i][2] = o[i][2] * wa[1] + __uint_as_float(v[i].z) * wb[1];
        o[i][3] = o[i][3] * wa[1] + __uint_as_float(v[i].w) * wb[1];
      }
    }
    // hand the parked pages back (generic-proxy writes before the next TMA fill)
    __syncwarp();
    if (c.lane == 0) {
      fence_proxy_async();
      for (int j = 0; j < parts; ++j) {
        const int pl = j + (j <= lr ? lq : lq - 1) * parts;
        RingPos rj = ua.rp0;
        ring_advance(rj, pl, NPG);
        mbar_arrive(empty_bar(c, rj.slot));
        *reinterpret_cast<volatile uint32_t*>(&c.ctrl->released[rj.slot]) = rj.k + 1u;
      }
      c.ctrl->mv_arrive[set] = 0;
      __threadfence_block();
      *reinterpret_cast<volatile uint32_t*>(&c.ctrl->mv_done[set]) = gen + 1u;
    }
  }

  // finalise: normalised partial + lse
  trace(c, TRC_MV_REDUCED, ord);
  float* op_ = reinterpret_cast<float*>(op->p[MK_AT_P_OPART]);
  float* lp_ = reinterpret_cast<float*>(op->p[MK_AT_P_LSEPART]);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    float l = lrow[e];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (!rv[e]) continue;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float lse = l > 0.f ? mrow[e] * sc + __logf(l) : -INFINITY;
    const int64_t base = ((((int64_t)u.b * H + rh[e]) * S + u.sp) * M + rm[e]);
    float* dst = op_ + base * D;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
      float2 v = make_float2(o[i][2 * e] * inv, o[i][2 * e + 1] * inv);
      *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = v;
    }
    if (t == 0) lp_[base] = lse;
  }
  if (op->i[MK_AT_FUSE_COMBINE]) {
    // count this split in; whoever completes the group combines it
    __syncwarp();
    int last = 0;
    if (c.lane == 0) {
      int32_t* arrive = reinterpret_cast<int32_t*>(op->p[MK_AT_P_ARRIVE]) +
                        ((size_t)u.b * HKV + u.kvh) * op->i[MK_AT_MT] + u.mt;
      // one acq_rel atomic: releases this unit's partial (all lanes' stores, ordered by the
      // __syncwarp) and acquires the other splits' partials for the combine
      int32_t old;
      asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(arrive) : "memory");
      last = old == S - 1;
      if (last) *arrive = 0;   // ready for the next launch
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    trace(c, TRC_AT_COUNTED, (uint32_t)last);
    if (last) at_combine_group<D>(c, op, u);
  }
  return true;
}

template <int D, int QMODE>
__device__ __forceinline__ UnitResult at_unit_call(Ctx c, const mk_op_t* op, const UnitArgs& ua) {
  UnitResult r;
  r.signal = at_unit<D, QMODE>(c, op, ua);
  r.dead = c.dead;
  r.trace_n = c.trace_n;
  return r;
}

template <int FEAT>
__device__ __forceinline__ bool at_dispatch(Ctx& c, const mk_op_t* op, const UnitArgs& ua) {
  constexpr int QMODE = (FEAT & MK_F_QKNORM) ? 1 : 0;
  UnitResult r;
  if constexpr ((FEAT & MK_F_AT64) && (FEAT & MK_F_AT128)) {
    if (op->i[MK_AT_D] == 64)
      r = at_unit_call<64, QMODE>(c, op, ua);
    else
      r = at_unit_call<128, QMODE>(c, op, ua);
  } else if constexpr ((FEAT & MK_F_AT64) != 0) {
    r = at_unit_call<64, QMODE>(c, op, ua);
  } else {
    r = at_unit_call<128, QMODE>(c, op, ua);
  }
  c.dead = r.dead;
  c.trace_n = r.trace_n;
  return r.signal;
}

// Combine: one unit per (b, query head); all M rows.
__device__ __forceinline__ void at_combine_unit(Ctx& c, const mk_op_t* op, int unit) {
  const int H = op->i[MK_AT_H], M = op->i[MK_AT_M], D = op->i[MK_AT_D], S = op->i[MK_AT_SPLITS];
  const int b = unit / H, h = unit - b * H;
  const float* opart = reinterpret_cast<const float*>(op->p[MK_AT_P_OPART]);
  const float* lpart = reinterpret_cast<const float*>(op->p[MK_AT_P_LSEPART]);
  float* lse_out = reinterpret_cast<float*>(op->p[MK_AT_P_LSE]);
  const int ot = op->i[MK_AT_O_T];
  // Lane j of a chunk holds the weight of split c0 + j; the partial rows of
  // several splits are requested together so that their latencies overlap.
  constexpr int UN = 12;
  for (int m = 0; m < M; ++m) {
    const int64_t base = ((int64_t)b * H + h) * S;
    float mx = -INFINITY;
    for (int s = c.lane; s < S; s += 32) mx = fmaxf(mx, lpart[(base + s) * M + m]);
    mx = warp_max(mx);
    float sum = 0.f;
    if (mx != -INFINITY)
      for (int s = c.lane; s < S; s += 32) sum += __expf(lpart[(base + s) * M + m] - mx);
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    const int64_t ooff = b * op->s[MK_AT_S_O_B] + m * op->s[MK_AT_S_O_M] + h * op->s[MK_AT_S_O_H];
    for (int d0 = 0; d0 < D; d0 += 64) {
      const int d = d0 + c.lane * 2;
      const bool dv = d < D;
      float a0 = 0.f, a1 = 0.f;
      for (int c0 = 0; c0 < S && sum > 0.f; c0 += 32) {
        const int cnt = min(32, S - c0);
        const float wl = (c.lane < cnt) ? __expf(lpart[(base + c0 + c.lane) * M + m] - mx) * inv : 0.f;
        for (int j0 = 0; j0 < cnt; j0 += UN) {
          float2 v[UN];
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            v[u] = make_float2(0.f, 0.f);
            if (dv && j0 + u < cnt)
              v[u] = *reinterpret_cast<const float2*>(opart + ((base + c0 + j0 + u) * M + m) * D + d);
          }
#pragma unroll
          for (int u = 0; u < UN; ++u) {
            const float w = __shfl_sync(0xffffffffu, wl, (j0 + u) & 31);
            a0 += w * v[u].x;
            a1 += w * v[u].y;
          }
        }
      }
      if (!dv) continue;
      if (ot == MK_T_FP32) {
        float* o = reinterpret_cast<float*>(op->p[MK_AT_P_O]) + ooff + d;
        o[0] = a0;
        o[1] = a1;
      } else {
        uint32_t* o = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(op->p[MK_AT_P_O]) + ooff + d);
        *o = (ot == MK_T_BF16) ? pack_bf16(a0, a1) : pack_f16(a0, a1);
      }
    }
    if (c.lane == 0 && lse_out) lse_out[((int64_t)b * H + h) * M + m] = (sum > 0.f) ? mx + __logf(sum) : -INFINITY;
  }
}

}  // namespace mk
