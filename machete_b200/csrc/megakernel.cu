// The persistent decode megakernel and its C ABI.
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
// CTA meet, wait for the op's producers, copy the op record to shared memory
// and stage its activations (RMSNorm and residual add fused).
//
// Counterpart of the reference's ring loop (megakernel/replay_loops.py:27-824)
// and launch path (megakernel/megakernel.py:2163-2204).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "kernel.cuh"

namespace mk {

// ------------------------------------------------------------------ host side
static thread_local std::string g_err;

static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CUDA_TRY(expr)                                                                       \
  do {                                                                                       \
    cudaError_t e_ = (expr);                                                                 \
    if (e_ != cudaSuccess) return fail(-(int)e_ - 1000, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

static inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

constexpr int kMapsPerOp = 4;  // W0, W1, scales0, scales1

struct Layout {
  uint64_t state, counters, ops, instrs, ibegin, events, ebegin, waits, tmaps, total;
};

static Layout layout_of(const mk_program_t* p) {
  Layout l;
  uint64_t o = 0;
  l.state = o;
  o = align_up(o + sizeof(DeviceState), 256);
  l.counters = o;
  o = align_up(o + (uint64_t)(p->n_counters > 0 ? p->n_counters : 1) * 4, 256);
  l.ops = o;
  o = align_up(o + (uint64_t)p->n_ops * sizeof(mk_op_t), 256);
  l.instrs = o;
  o = align_up(o + (uint64_t)(p->n_instrs > 0 ? p->n_instrs : 1) * sizeof(mk_instr_t), 256);
  l.ibegin = o;
  o = align_up(o + (uint64_t)(p->n_ctas + 1) * 4, 256);
  l.events = o;
  o = align_up(o + (uint64_t)(p->n_events > 0 ? p->n_events : 1) * sizeof(mk_event_t), 256);
  l.ebegin = o;
  o = align_up(o + (uint64_t)(p->n_ctas + 1) * 4, 256);
  l.waits = o;
  o = align_up(o + (uint64_t)(p->n_waits > 0 ? p->n_waits : 1) * sizeof(mk_wait_t), 256);
  l.tmaps = o;
  o = align_up(o + (uint64_t)p->n_ops * kMapsPerOp * sizeof(CUtensorMap), 256);
  l.total = o;
  return l;
}

static bool aligned16(uint64_t p) { return (p & 15ull) == 0; }

// ---- tensor maps -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// A byte matrix of `rows` rows of `row_bytes` valid bytes (row stride `stride`)
// seen as 128-byte tiles: dims (128 bytes, rows, tiles); one box = 128 bytes x
// 8 rows x `box_tiles` tiles, written to shared memory tile after tile with
// the 128-byte swizzle.  Out-of-range rows and bytes read as zero.
static int encode_tile_map(CUtensorMap* out, uint64_t base, uint64_t rows, uint64_t row_bytes, uint64_t stride,
                           uint32_t box_tiles) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(-5, "cuTensorMapEncodeTiled is not available from this driver");
  if ((base & 15) || (stride & 15) || (row_bytes & 15) || rows == 0 || row_bytes == 0)
    return fail(-2, "tensor map: base, row stride and row length must be 16-byte multiples");
  const uint64_t tiles = (row_bytes + 127) / 128;
  // When a row is shorter than one tile the inner extent is the row itself;
  // otherwise rows are tiled in 128-byte steps and a ragged last tile is
  // covered by declaring the inner extent 128 (the excess bytes belong to the
  // same allocation only if row_bytes is a multiple of 128, which callers check).
  const cuuint64_t inner = row_bytes < 128 ? row_bytes : 128;
  cuuint64_t dims[3] = {inner, rows, tiles};
  cuuint64_t strides[2] = {stride, 128};
  cuuint32_t box[3] = {128, 8, box_tiles};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, reinterpret_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

static uint32_t mv_page_need(int wfmt, int Kc) {
  return wfmt >= MK_W_NVFP4_F16S32 ? 2u * (uint32_t)(Kc / 256) * 1024u + 2048u : 2u * (uint32_t)(Kc / 64) * 1024u;
}

// Build the descriptors of matvec op `op` into `maps` (host copies) and point
// the op record at their device addresses.
// K or V cache [B, N, HKV, D] (any strides with a contiguous head dim) as a
// 4-D map: box = 64 head-dim values x 1 head x tn tokens x 1 batch, swizzled.
static int encode_kv_map(CUtensorMap* out, uint64_t base, int D, int HKV, int N, int B, int64_t s_h, int64_t s_n,
                         int64_t s_b, uint32_t tn) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(-5, "cuTensorMapEncodeTiled is not available from this driver");
  if ((base & 15) || ((s_h * 2) & 15) || ((s_n * 2) & 15) || (B > 1 && ((s_b * 2) & 15)))
    return fail(-2, "attention: K/V base and head/token/batch strides must be 16-byte multiples");
  if (s_h <= 0 || s_n <= 0) return fail(-2, "attention: K/V strides must be positive");
  const uint64_t sb = (B > 1 && s_b > 0) ? (uint64_t)s_b * 2 : (uint64_t)s_n * 2 * (uint64_t)N;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)HKV, (cuuint64_t)N, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)s_h * 2, (cuuint64_t)s_n * 2, (cuuint64_t)((sb + 15) / 16 * 16)};
  cuuint32_t box[4] = {64, 1, tn, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, reinterpret_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled (K/V cache) failed with CUresult %d", (int)r);
  return 0;
}

static int build_op_maps(mk_op_t& op, CUtensorMap* maps, uint64_t dev_maps, int page_bytes) {
  if (op.opcode == MK_OP_ATTN_SPLIT || op.opcode == MK_OP_ATTN_COMBINE)
    op.i[MK_AT_GROUP] = op.i[MK_AT_H] / op.i[MK_AT_HKV];   // validated: H a positive multiple of HKV
  if (op.opcode == MK_OP_ATTN_SPLIT) {
    const int D = op.i[MK_AT_D];
    const uint32_t tn = (uint32_t)at_page_tokens(D, page_bytes);
    int rc = encode_kv_map(&maps[0], op.p[MK_AT_P_K], D, op.i[MK_AT_HKV], op.i[MK_AT_N], op.i[MK_AT_B],
                           op.s[MK_AT_S_K_H], op.s[MK_AT_S_K_N], op.s[MK_AT_S_K_B], tn);
    if (rc) return rc;
    return encode_kv_map(&maps[1], op.p[MK_AT_P_V], D, op.i[MK_AT_HKV], op.i[MK_AT_N], op.i[MK_AT_B],
                         op.s[MK_AT_S_V_H], op.s[MK_AT_S_V_N], op.s[MK_AT_S_V_B], tn);
  }
  if (op.opcode != MK_OP_MATVEC) return 0;
  const int wf = op.i[MK_MV_WFMT], K = op.i[MK_MV_K], Kc = op.i[MK_MV_KC];
  const bool fp4 = wf >= MK_W_NVFP4_F16S32;
  const bool pair = op.i[MK_MV_MODE] == MK_MV_PAIR;
  const uint64_t rows = (uint64_t)op.i[MK_MV_O];
  const uint64_t row_bytes = fp4 ? (uint64_t)K / 2 : (uint64_t)K * 2;
  const uint32_t box_tiles = fp4 ? (uint32_t)(Kc / 256) : (uint32_t)(Kc / 64);
  int rc = encode_tile_map(&maps[0], op.p[MK_MV_P_W0], rows, row_bytes, (uint64_t)op.s[MK_MV_S_WROW], box_tiles);
  if (rc) return rc;
  op.p[MK_MV_P_TM_W0] = dev_maps;
  if (pair) {
    rc = encode_tile_map(&maps[1], op.p[MK_MV_P_W1], rows, row_bytes, (uint64_t)op.s[MK_MV_S_WROW], box_tiles);
    if (rc) return rc;
    op.p[MK_MV_P_TM_W1] = dev_maps + sizeof(CUtensorMap);
  }
  if (fp4) {
    const uint64_t srow_bytes = (uint64_t)K / 16;
    rc = encode_tile_map(&maps[2], op.p[MK_MV_P_SC0], rows, srow_bytes, (uint64_t)op.s[MK_MV_S_SCROW], 1);
    if (rc) return rc;
    op.p[MK_MV_P_TM_SC0] = dev_maps + 2 * sizeof(CUtensorMap);
    if (pair) {
      rc = encode_tile_map(&maps[3], op.p[MK_MV_P_SC1], rows, srow_bytes, (uint64_t)op.s[MK_MV_S_SCROW], 1);
      if (rc) return rc;
      op.p[MK_MV_P_TM_SC1] = dev_maps + 3 * sizeof(CUtensorMap);
    }
  }
  return 0;
}

static int matvec_pages(const mk_op_t& op) {
  const int K = op.i[MK_MV_K], Kc = op.i[MK_MV_KC];
  return (K + Kc - 1) / Kc;
}
static int attn_pages(const mk_op_t& op, int unit, int page_bytes) {
  const int S = op.i[MK_AT_SPLITS];
  const int sp = unit % S;
  const int ts = op.i[MK_AT_TS], N = op.i[MK_AT_N];
  const int tb = std::min(N, sp * ts), te = std::min(N, tb + ts);
  const int tn = at_page_tokens(op.i[MK_AT_D], page_bytes);
  return (te - tb + tn - 1) / tn;
}

// Everything the device would otherwise derive per unit with divisions or
// op-table reads: the loader's tensor-map address, first rows and tiles per
// page, the participant count, and the finisher's output offsets.
static void fill_instr_fast_path(mk_instr_t& in, const mk_op_t& op, uint64_t dev_tmaps, int page_bytes, int n_ring_pages) {
  in.ld_maps = 0;
  in.ld_row_a = in.ld_row_b = in.ld_tiles = in.ld_flags = 0;
  in.out_off_a = in.out_off_b = 0;
  if (op.opcode == MK_OP_ATTN_SPLIT) {
    // unit -> (batch, kv head, query tile, split)
    const int S = op.i[MK_AT_SPLITS], MT = op.i[MK_AT_MT], HKV = op.i[MK_AT_HKV];
    const int sp = in.unit % S, mt = (in.unit / S) % MT, kvh = (in.unit / S / MT) % HKV, b = in.unit / S / MT / HKV;
    const int t_begin = std::min(op.i[MK_AT_N], sp * op.i[MK_AT_TS]);
    in.ld_maps = dev_tmaps + (uint64_t)in.op * kMapsPerOp * sizeof(CUtensorMap);
    in.ld_row_a = t_begin;
    in.ld_row_b = kvh | (b << 16);
    in.out_off_a = sp;
    in.out_off_b = mt;
    in.ld_tiles = at_page_tokens(op.i[MK_AT_D], page_bytes);
    // every participant keeps one ring page until the unit's states are merged:
    // leave at least two pages for the stream
    const int split = std::max(1, std::min(std::min((int)kConsumerWarps, in.n_pages), n_ring_pages - 2));
    in.ld_flags = MK_LDF_ATTN | (op.i[MK_AT_D] == 128 ? MK_LDF_D128 : 0) | (split << MK_LDF_SPLIT_SHIFT) |
                  (op.i[MK_AT_DYNPOS] ? MK_LDF_DYN : 0);
    if (in.n_pages == 0) in.ld_maps = 0;   // an empty split: nothing to load, one consumer writes the empty partial
    return;
  }
  if (op.opcode != MK_OP_MATVEC) return;
  const bool fp4 = op.i[MK_MV_WFMT] >= MK_W_NVFP4_F16S32;
  const int mode = op.i[MK_MV_MODE];
  in.ld_maps = dev_tmaps + (uint64_t)in.op * kMapsPerOp * sizeof(CUtensorMap);
  in.ld_tiles = fp4 ? op.i[MK_MV_KC] / 256 : op.i[MK_MV_KC] / 64;
  // consumers per unit: participant j takes pages j, j + split, ...; none idle
  int split = op.i[MK_MV_SPLIT];
  if (split <= 0 || split > kConsumerWarps) split = kConsumerWarps;
  split = std::min(split, std::max(1, in.n_pages));
  int chunk = 0;
  if (mode == MK_MV_PLAIN) {
    in.ld_row_a = in.unit * 16;
    in.ld_row_b = in.unit * 16 + 8;
  } else if (mode == MK_MV_PAIR) {
    in.ld_row_a = in.ld_row_b = in.unit * 8;
  } else {
    const int hd = op.i[MK_MV_HD], d2 = op.i[MK_MV_D2], upb = d2 / 8;
    const int h = in.unit / upb;
    chunk = in.unit - h * upb;
    in.ld_row_a = h * hd + chunk * 8;
    in.ld_row_b = in.ld_row_a + d2;
  }
  in.ld_flags = (fp4 ? MK_LDF_FP4 : 0) | (mode == MK_MV_PAIR ? MK_LDF_PAIR : 0) |
                (std::max(1, split) << MK_LDF_SPLIT_SHIFT) | ((chunk & MK_LDF_CHUNK_MASK) << MK_LDF_CHUNK_SHIFT);
  // output offsets of the two row groups (8 rows each never straddle a head: head dim % 8 == 0)
  const int hd = std::max(1, op.i[MK_MV_HD]);
  const int64_t sh = op.s[MK_MV_S_O_H];
  in.out_off_a = (int32_t)((int64_t)(in.ld_row_a / hd) * sh + in.ld_row_a % hd);
  in.out_off_b = (int32_t)((int64_t)(in.ld_row_b / hd) * sh + in.ld_row_b % hd);
}

static int validate_op(const mk_op_t& op, int idx, int page_bytes, int act_bytes) {
  if (op.opcode < 0 || op.opcode >= MK_OP__COUNT) return fail(-2, "op %d: unknown opcode %d", idx, op.opcode);
  if (op.n_units < 0) return fail(-2, "op %d: negative unit count", idx);
  if (op.opcode == MK_OP_MATVEC) {
    const int O = op.i[MK_MV_O], K = op.i[MK_MV_K], M = op.i[MK_MV_M], Kc = op.i[MK_MV_KC];
    const int wf = op.i[MK_MV_WFMT], mode = op.i[MK_MV_MODE];
    const bool fp4 = wf >= MK_W_NVFP4_F16S32;
    if (O <= 0 || K <= 0 || M <= 0 || op.i[MK_MV_S] <= 0) return fail(-2, "op %d: bad matvec dims", idx);
    if (M > 32) return fail(-2, "op %d: matvec supports at most 32 activation rows, got %d", idx, M);
    if (wf < 0 || wf > MK_W_NVFP4_E4M3S16) return fail(-2, "op %d: bad weight format", idx);
    if (fp4 ? (K % 256 != 0 || Kc % 256 != 0) : (K % 64 != 0 || Kc % 64 != 0))
      return fail(-2, "op %d: K=%d / Kc=%d must be multiples of %d", idx, K, Kc, fp4 ? 256 : 64);
    if (Kc <= 0 || (fp4 ? Kc > 2048 : Kc > 64 * 256))
      return fail(-2, "op %d: K slice %d out of range", idx, Kc);
    if (fp4 && Kc != (K < 2048 ? K : 2048))
      return fail(-2, "op %d: NVFP4 K slice must be min(K, 2048), got %d", idx, Kc);
    if (fp4 && K > 2048 && K % 2048 != 0)
      return fail(-2, "op %d: NVFP4 matvec needs K < 2048 or K %% 2048 == 0, got %d", idx, K);
    const uint64_t need = mv_page_need(wf, Kc);
    if (need > (uint64_t)page_bytes) return fail(-2, "op %d: K slice %d does not fit a %d-byte page", idx, Kc, page_bytes);
    if ((uint64_t)M * ((uint64_t)K * 2 + 64) > (uint64_t)act_bytes)
      return fail(-2, "op %d: %d x %d activations exceed the %d-byte staging buffer", idx, M, K, act_bytes);
    if (!aligned16(op.p[MK_MV_P_W0]) || !op.p[MK_MV_P_W0] || (op.s[MK_MV_S_WROW] & 15))
      return fail(-2, "op %d: weight pointer / row stride must be 16-byte aligned", idx);
    if (mode == MK_MV_PAIR && (!aligned16(op.p[MK_MV_P_W1]) || !op.p[MK_MV_P_W1]))
      return fail(-2, "op %d: second weight pointer missing or unaligned", idx);
    if (fp4) {
      if (!aligned16(op.p[MK_MV_P_SC0]) || !op.p[MK_MV_P_SC0] || (op.s[MK_MV_S_SCROW] & 15))
        return fail(-2, "op %d: scale pointer / row stride must be 16-byte aligned", idx);
      if (mode == MK_MV_PAIR && (!aligned16(op.p[MK_MV_P_SC1]) || !op.p[MK_MV_P_SC1]))
        return fail(-2, "op %d: second scale pointer missing or unaligned", idx);
    }
    if (!aligned16(op.p[MK_MV_P_X]) || !op.p[MK_MV_P_X] || (op.s[MK_MV_S_X_B] & 7) || (op.s[MK_MV_S_X_S] & 7))
      return fail(-2, "op %d: activation pointer / strides must be 16-byte aligned", idx);
    if (op.i[MK_MV_PRO] != MK_PRO_NONE && (!op.p[MK_MV_P_NORM_W] || !aligned16(op.p[MK_MV_P_NORM_W])))
      return fail(-2, "op %d: norm weight missing or unaligned", idx);
    if (op.i[MK_MV_PRO] == MK_PRO_ADD_RMS && op.p[MK_MV_P_RES_IN] &&
        (!aligned16(op.p[MK_MV_P_RES_IN]) || (op.s[MK_MV_S_RI_B] & 7) || (op.s[MK_MV_S_RI_S] & 7) ||
         (op.p[MK_MV_P_RES_OUT] && (!aligned16(op.p[MK_MV_P_RES_OUT]) || (op.s[MK_MV_S_RO_B] & 7) || (op.s[MK_MV_S_RO_S] & 7)))))
      return fail(-2, "op %d: residual pointers / strides must be 16-byte aligned", idx);
    if (!op.p[MK_MV_P_OUT]) return fail(-2, "op %d: output pointer missing", idx);
    if (op.i[MK_MV_HD] <= 0) return fail(-2, "op %d: head dim must be positive", idx);
    if (op.i[MK_MV_HD] % 8 != 0 && op.s[MK_MV_S_O_H] != op.i[MK_MV_HD])
      return fail(-2, "op %d: a strided head layout needs a head dim that is a multiple of 8", idx);
    int units;
    if (mode == MK_MV_PLAIN) {
      units = (O + 15) / 16;
    } else if (mode == MK_MV_PAIR) {
      units = (O + 7) / 8;
    } else if (mode == MK_MV_ROPE) {
      const int hd = op.i[MK_MV_HD], d2 = op.i[MK_MV_D2];
      if (d2 <= 0 || d2 % 8 != 0 || hd != 2 * d2 || O % hd != 0)
        return fail(-2, "op %d: rope mode needs head_dim == 2*D2, D2 %% 8 == 0, O %% head_dim == 0", idx);
      if (!op.p[MK_MV_P_COS] || !op.p[MK_MV_P_SIN]) return fail(-2, "op %d: cos/sin missing", idx);
      units = (O / hd) * (d2 / 8);
    } else {
      return fail(-2, "op %d: bad matvec mode", idx);
    }
    if (op.i[MK_MV_TR] == MK_TR_ROPE && mode != MK_MV_ROPE) return fail(-2, "op %d: rope transform needs rope mode", idx);
    if (op.i[MK_MV_TR] == MK_TR_SILU_MUL && mode != MK_MV_PAIR) return fail(-2, "op %d: silu-mul needs pair mode", idx);
    if (op.i[MK_MV_EPI] == MK_EPI_RESIDUAL && !op.p[MK_MV_P_EPI_RES]) return fail(-2, "op %d: epilogue residual missing", idx);
    if (op.n_units != units) return fail(-2, "op %d: expected %d units, got %d", idx, units, op.n_units);
  } else if (op.opcode == MK_OP_ATTN_SPLIT || op.opcode == MK_OP_ATTN_COMBINE) {
    const int D = op.i[MK_AT_D], H = op.i[MK_AT_H], HKV = op.i[MK_AT_HKV], M = op.i[MK_AT_M];
    if (D != 64 && D != 128) return fail(-2, "op %d: head dim %d unsupported (64 or 128)", idx, D);
    if (H <= 0 || HKV <= 0 || H % HKV != 0 || M <= 0 || op.i[MK_AT_B] <= 0 || op.i[MK_AT_SPLITS] <= 0 || op.i[MK_AT_N] < 0)
      return fail(-2, "op %d: bad attention dims", idx);
    if (!op.p[MK_AT_P_OPART] || !op.p[MK_AT_P_LSEPART] || (op.p[MK_AT_P_OPART] & 7))
      return fail(-2, "op %d: partial buffers missing", idx);
    if (op.opcode == MK_OP_ATTN_SPLIT) {
      const int G = H / HKV;
      if (op.i[MK_AT_MT] != (M * G + 15) / 16) return fail(-2, "op %d: bad query tile count", idx);
      if (op.i[MK_AT_TS] <= 0) return fail(-2, "op %d: tokens per split must be positive", idx);
      if ((int64_t)op.i[MK_AT_TS] * op.i[MK_AT_SPLITS] < op.i[MK_AT_N]) return fail(-2, "op %d: splits do not cover N", idx);
      if (at_page_tokens(D, page_bytes) <= 0) return fail(-2, "op %d: page too small for attention", idx);
      for (int k = MK_AT_P_Q; k <= MK_AT_P_V; ++k)
        if (!op.p[k] || !aligned16(op.p[k])) return fail(-2, "op %d: q/k/v pointer missing or unaligned", idx);
      for (int k = MK_AT_S_Q_B; k <= MK_AT_S_V_H; ++k)
        if (op.s[k] & 7) return fail(-2, "op %d: q/k/v strides must be multiples of 8 elements", idx);
      if (op.n_units != op.i[MK_AT_B] * HKV * op.i[MK_AT_MT] * op.i[MK_AT_SPLITS])
        return fail(-2, "op %d: bad unit count", idx);
      if (op.i[MK_AT_DYNPOS] && (M != 1 || op.i[MK_AT_CAUSAL]))
        return fail(-2, "op %d: a KV window that follows the cache position needs one token per sequence, non-causal", idx);
      if (op.i[MK_AT_QKNORM]) {
        if (M != 1 || op.i[MK_AT_MT] != 1) return fail(-2, "op %d: fused q/k norm needs one token per sequence and H/Hkv <= 16", idx);
        if (op.i[MK_AT_DYNPOS]) {
          if (op.i[MK_AT_NEW_TOK] < D / 2 || (op.i[MK_AT_NEW_TOK] & 7))
            return fail(-2, "op %d: with a device-resident position MK_AT_NEW_TOK is the cos / sin row stride (>= D/2, a multiple of 8)", idx);
        } else if (op.i[MK_AT_NEW_TOK] < 0 || op.i[MK_AT_NEW_TOK] >= op.i[MK_AT_N]) {
          return fail(-2, "op %d: new-token row outside the cache window", idx);
        }
        for (int k = MK_AT_P_QNW; k <= MK_AT_P_SIN; ++k)
          if (!op.p[k] || !aligned16(op.p[k])) return fail(-2, "op %d: fused q/k norm tables missing or unaligned", idx);
      }
    } else {
      if (!op.p[MK_AT_P_O] || (op.p[MK_AT_P_O] & 3)) return fail(-2, "op %d: output pointer missing or unaligned", idx);
      for (int k = MK_AT_S_O_B; k <= MK_AT_S_O_H; ++k)
        if (op.s[k] & 1) return fail(-2, "op %d: output strides must be even", idx);
      if (op.n_units != op.i[MK_AT_B] * H) return fail(-2, "op %d: bad unit count", idx);
    }
    if (op.opcode == MK_OP_ATTN_SPLIT && op.i[MK_AT_FUSE_COMBINE]) {
      if (!op.p[MK_AT_P_O] || (op.p[MK_AT_P_O] & 15) || !op.p[MK_AT_P_ARRIVE] || (op.p[MK_AT_P_ARRIVE] & 3))
        return fail(-2, "op %d: fused combine needs a 16-byte aligned output and the arrival counters", idx);
      if (op.i[MK_AT_SPLITS] > 128) return fail(-2, "op %d: fused combine handles at most 128 splits", idx);
      for (int k = MK_AT_S_O_B; k <= MK_AT_S_O_H; ++k)
        if (op.s[k] & 7) return fail(-2, "op %d: fused combine needs output strides that are multiples of 8", idx);
    }
  } else if (op.opcode >= MK_OP_RMSNORM && op.opcode <= MK_OP_ADD) {
    if (!op.p[MK_EW_P_X]) return fail(-2, "op %d: input pointer missing", idx);
    if (op.i[MK_EW_T] < 0 || op.i[MK_EW_T] > MK_T_FP32) return fail(-2, "op %d: bad element type", idx);
  } else if (op.opcode == MK_OP_TOP1_FINAL) {
    if (!op.p[MK_EW_P_X] || !op.p[MK_EW_P_W] || (op.p[MK_EW_P_X] & 7)) return fail(-2, "op %d: top-1 buffers missing", idx);
    if (op.i[MK_EW_FLAGS] & MK_EWF_FEEDBACK) {
      if (!op.p[MK_EW_P_RES_IN] || !op.p[MK_EW_P_RES_OUT] || ((op.p[MK_EW_P_RES_IN] | op.p[MK_EW_P_RES_OUT]) & 15) ||
          (op.i[MK_EW_D] & 7) || op.i[MK_EW_D] <= 0 || ((op.s[MK_EW_S_RI] | op.s[MK_EW_S_RO]) & 7) || (op.p[MK_EW_P_GATE] & 3))
        return fail(-2, "op %d: token feedback needs 16-byte aligned embedding and input rows of a multiple of 8 values", idx);
    }
  } else if (op.opcode == MK_OP_ALLREDUCE) {
    const int P = op.i[MK_AR_P], rank = op.i[MK_AR_RANK], n = op.i[MK_AR_N];
    if (P < 2 || P > MK_AR_MAX_RANKS || rank < 0 || rank >= P) return fail(-2, "op %d: bad all-reduce world %d / rank %d", idx, P, rank);
    if (!op.p[MK_AR_P_X] || !op.p[MK_AR_P_Y]) return fail(-2, "op %d: all-reduce input/output pointer missing", idx);
    for (int r = 0; r < P; ++r)
      if (!op.p[MK_AR_P_PEER0 + r] || (op.p[MK_AR_P_PEER0 + r] & 15)) return fail(-2, "op %d: peer buffer %d missing or unaligned", idx, r);
    if ((op.s[MK_AR_S_INBOX] & 15) || (op.s[MK_AR_S_FLAGS] & 3)) return fail(-2, "op %d: unaligned inbox/flag offsets", idx);
    if (op.i[MK_AR_MODE] == MK_AR_MAX_KEY) {
      if (n < 1 || n > 32 || op.n_units != 1) return fail(-2, "op %d: key all-reduce handles 1..32 rows in one unit", idx);
    } else {
      if (n < 8 || (n & 7) || op.n_units != (n + 255) / 256) return fail(-2, "op %d: bad all-reduce size %d", idx, n);
      if ((op.p[MK_AR_P_X] & 15) || (op.p[MK_AR_P_Y] & 15) || (op.p[MK_AR_P_RES] & 15)) return fail(-2, "op %d: all-reduce tensors must be 16-byte aligned", idx);
    }
  }
  return 0;
}

static int validate_program(const mk_program_t* p, int smem_optin, int num_sms, int* smem_bytes) {
  if (!p) return fail(-1, "null program");
  if (p->n_ops <= 0 || !p->ops) return fail(-1, "program has no ops");
  if (p->n_ctas <= 0 || p->n_ctas > 4096) return fail(-1, "bad grid size %d", p->n_ctas);
  if (num_sms > 0 && p->n_ctas > num_sms)
    return fail(-1, "grid of %d CTAs exceeds the %d multiprocessors: the CTAs of a launch wait on one another, so all must be resident", p->n_ctas, num_sms);
  if (p->n_pages < 2 || p->n_pages > kMaxPages) return fail(-1, "ring depth must be in [2, %d]", kMaxPages);
  if (p->page_bytes <= 0 || (p->page_bytes & 1023)) return fail(-1, "page size must be a positive multiple of 1024");
  if (p->act_bytes < 0 || (p->act_bytes & 1023)) return fail(-1, "activation buffer must be a multiple of 1024 bytes");
  if (!p->cta_instr_begin || !p->cta_event_begin) return fail(-1, "missing per-CTA offsets");
  if (p->n_instrs > 0 && !p->instrs) return fail(-1, "missing instruction table");
  if (p->n_events > 0 && !p->events) return fail(-1, "missing event table");
  if (p->n_waits > 0 && !p->waits) return fail(-1, "missing wait table");
  const int64_t smem = (int64_t)kCtrlBytes + p->act_bytes + (int64_t)p->n_pages * p->page_bytes;
  if (smem > smem_optin) return fail(-1, "program needs %lld bytes of shared memory, device offers %d", (long long)smem, smem_optin);
  *smem_bytes = (int)smem;
  for (int i = 0; i < p->n_ops; ++i) {
    const int rc = validate_op(p->ops[i], i, p->page_bytes, p->act_bytes);
    if (rc) return rc;
  }
  if (p->position == nullptr)
    for (int i = 0; i < p->n_ops; ++i) {
      const mk_op_t& op = p->ops[i];
      if ((op.opcode == MK_OP_MATVEC && op.i[MK_MV_DYNPOS]) || (op.opcode == MK_OP_ATTN_SPLIT && op.i[MK_AT_DYNPOS]))
        return fail(-2, "op %d follows a device-resident cache position, but the program has none (mk_program_t.position)", i);
    }
  if (p->position != nullptr && ((uint64_t)p->position & 3)) return fail(-1, "position scalar must be 4-byte aligned");
  if (p->position != nullptr && (p->position_count < 0 || p->position_count > 32))
    return fail(-1, "position_count must be 0 or 1 (one position for all rows) or the batch size, at most 32 (got %d)", p->position_count);
  if (p->position != nullptr && p->position_limit < 1)
    return fail(-1, "position_limit must be the cache length of the position-following ops (got %d)", p->position_limit);
  for (int i = 0; i < p->n_waits; ++i)
    if (p->waits[i].counter < 0 || p->waits[i].counter >= p->n_counters)
      return fail(-3, "wait %d: counter %d out of range", i, p->waits[i].counter);
  if (p->cta_instr_begin[0] != 0 || p->cta_instr_begin[p->n_ctas] != p->n_instrs)
    return fail(-3, "per-CTA instruction offsets do not span the table");
  if (p->cta_event_begin[0] != 0 || p->cta_event_begin[p->n_ctas] != p->n_events)
    return fail(-3, "per-CTA event offsets do not span the table");
  for (int cta = 0; cta < p->n_ctas; ++cta) {
    const int ib = p->cta_instr_begin[cta], ie = p->cta_instr_begin[cta + 1];
    const int eb = p->cta_event_begin[cta], ee = p->cta_event_begin[cta + 1];
    if (ie < ib || ee < eb) return fail(-3, "per-CTA offsets not monotonic at CTA %d", cta);
    for (int j = ib; j < ie; ++j) {
      const mk_instr_t& in = p->instrs[j];
      if (in.op < 0 || in.op >= p->n_ops) return fail(-3, "instr %d: op out of range", j);
      const mk_op_t& op = p->ops[in.op];
      if (in.unit < 0 || in.unit >= op.n_units) return fail(-3, "instr %d: unit %d out of range (op %d has %d)", j, in.unit, in.op, op.n_units);
      if (in.signal >= p->n_counters) return fail(-3, "instr %d: signal counter out of range", j);
      if (in.n_waits < 0 || in.wait_off < 0 || in.wait_off + in.n_waits > p->n_waits) return fail(-3, "instr %d: wait list out of range", j);
      if (in.n_lwaits < 0 || in.lwait_off < 0 || in.lwait_off + in.n_lwaits > p->n_waits) return fail(-3, "instr %d: loader wait list out of range", j);
      int pages = 0;
      if (op.opcode == MK_OP_MATVEC) pages = matvec_pages(op);
      else if (op.opcode == MK_OP_ATTN_SPLIT) pages = attn_pages(op, in.unit, p->page_bytes);
      if (in.n_pages != pages) return fail(-3, "instr %d: expected %d pages, got %d", j, pages, in.n_pages);
    }
    int last = -1;
    for (int e = eb; e < ee; ++e) {
      const mk_event_t& ev = p->events[e];
      if (ev.op < 0 || ev.op >= p->n_ops) return fail(-3, "event %d: op out of range", e);
      if (ev.pos < last || ev.pos < 0 || ev.pos > ie - ib) return fail(-3, "event %d: position out of order", e);
      if (ev.n_waits < 0 || ev.wait_off < 0 || ev.wait_off + ev.n_waits > p->n_waits) return fail(-3, "event %d: wait list out of range", e);
      last = ev.pos;
    }
  }
  return 0;
}

}  // namespace mk

// The kernel variants are compiled in groups, one translation unit per group
// (variants_*.cu), so that they build in parallel; each group hands out its
// table.  Variants differ in <activation-tile class, weight family, features>.
extern "C" const mk_variant* mk_variants_generic(int* n);
extern "C" const mk_variant* mk_variants_bf16(int* n);
extern "C" const mk_variant* mk_variants_bf16_wide(int* n);
extern "C" const mk_variant* mk_variants_fp4(int* n);
extern "C" const mk_variant* mk_variants_fp4_wide(int* n);
extern "C" const mk_variant* mk_variants_fp4_tp(int* n);
extern "C" const mk_variant* mk_variants_attn(int* n);

static const std::vector<mk_variant>& all_variants() {
  static const std::vector<mk_variant> v = [] {
    std::vector<mk_variant> out;
    typedef const mk_variant* (*group_fn)(int*);
    const group_fn groups[] = {mk_variants_generic, mk_variants_bf16,     mk_variants_bf16_wide,
                               mk_variants_fp4,     mk_variants_fp4_wide, mk_variants_fp4_tp,
                               mk_variants_attn};
    for (group_fn g : groups) {
      int n = 0;
      const mk_variant* t = g(&n);
      out.insert(out.end(), t, t + n);
    }
    return out;
  }();
  return v;
}

struct mk_handle_s {
  mk::ProgramView pv;
  mk_kernel_fn kernel;
  std::vector<int> op_ntc, op_wfc;   // per op: NT class and weight family (0 = not a matvec)
  std::vector<int> op_feat;          // per op: MK_F_* bits its unit handler needs
  int feat;                          // features of the kernel in use
  std::vector<mk_op_t> ops;          // host copy of the op records (as uploaded)
  std::vector<mk_instr_t> instrs;    // host copy of the instruction table (as uploaded)
  int n_ctas;
  int smem_bytes;
  int smem_optin;
  int device;
  int n_ops;
  uint8_t* ws;
  mk::Layout layout;
};

static void classify_op(const mk_op_t& op, int* ntc, int* wfc, int* feat) {
  *ntc = 0;
  *wfc = -1;
  *feat = 0;
  switch (op.opcode) {
    case MK_OP_ATTN_SPLIT:
      *feat = (op.i[MK_AT_D] == 64 ? mk::MK_F_AT64 : mk::MK_F_AT128) | (op.i[MK_AT_QKNORM] ? mk::MK_F_QKNORM : 0);
      return;
    case MK_OP_ATTN_COMBINE: *feat = mk::MK_F_COMBINE; return;
    case MK_OP_RMSNORM: case MK_OP_ROPE: case MK_OP_QKNORM_ROPE: case MK_OP_GLU: case MK_OP_ADD:
      *feat = mk::MK_F_EW;
      return;
    case MK_OP_TOP1_FINAL: *feat = mk::MK_F_TOP1; return;
    case MK_OP_ALLREDUCE: *feat = mk::MK_F_AR; return;
    case MK_OP_MATVEC: break;
    default: return;
  }
  const int m = op.i[MK_MV_M], wf = op.i[MK_MV_WFMT];
  *ntc = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
  *wfc = wf == MK_W_BF16 ? 0 : (wf >= MK_W_NVFP4_F16S32 ? 2 : 1);
  if (op.i[MK_MV_EPI] == MK_EPI_TOP1) *feat = mk::MK_F_TOP1;
}

// Pick the smallest kernel that covers the program: its matvec ops' tile class
// and weight family (one combination, else the generic matvec code) and the
// union of its ops' features.
static int select_kernel(mk_handle_s* h) {
  int ntc = -1, wfc = -2;
  bool mixed = false;
  int need = h->pv.trace != nullptr ? mk::MK_F_TRACE : 0;
  for (size_t i = 0; i < h->op_ntc.size(); ++i) {
    need |= h->op_feat[i];
    if (h->op_ntc[i] == 0) continue;
    if (ntc == -1) {
      ntc = h->op_ntc[i];
      wfc = h->op_wfc[i];
    } else if (ntc != h->op_ntc[i] || wfc != h->op_wfc[i]) {
      mixed = true;
    }
  }
  if (ntc == -1) {   // no matvec op at all: the variants built without matvec code
    wfc = 0;
  } else if (mixed || ntc <= 0 || wfc == 1) {   // fp16 weights run the generic matvec code
    ntc = 0;
    wfc = -1;
  }
  const mk_variant* best = nullptr;
  int best_cost = 1 << 30;
  for (const mk_variant& v : all_variants()) {
    if ((v.feat & need) != need) continue;
    const bool exact = v.ntc == ntc && v.wfc == wfc;
    if (!exact && !(v.ntc == 0 && v.wfc == -1)) continue;
    const int cost = __builtin_popcount((unsigned)v.feat) + (exact ? 0 : 100);
    if (cost < best_cost) {
      best_cost = cost;
      best = &v;
    }
  }
  if (!best) return mk::fail(-5, "no kernel variant covers this program (features 0x%x)", need);
  h->kernel = best->fn;
  h->feat = best->feat;
  h->pv.mv_sets = 4;
  for (int n : h->op_ntc)
    if (n > 0) h->pv.mv_sets = std::min(h->pv.mv_sets, n == 1 ? 4 : (n == 2 ? 2 : 1));
  // The dynamic shared-memory limit is a property of the kernel function, shared by
  // every handle that runs this variant: always raise it to the device's opt-in
  // maximum, so that a later, smaller program never lowers it under a live one.
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(h->kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, h->smem_optin);
  if (e != cudaSuccess) return mk::fail(-(int)e - 1000, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  return 0;
}

// Restores the caller's current device when an entry point returns.
struct DeviceScope {
  int prev = -1;
  ~DeviceScope() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

extern "C" {

int mk_abi_version(void) { return MK_ABI_VERSION; }

const char* mk_last_error(void) { return mk::g_err.c_str(); }

int mk_device_info(int device, int32_t* num_sms, int32_t* smem_optin, int32_t* cc_major, int32_t* cc_minor) {
  using namespace mk;
  int v = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
  if (num_sms) *num_sms = v;
  CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  if (smem_optin) *smem_optin = v;
  CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, device));
  if (cc_major) *cc_major = v;
  CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, device));
  if (cc_minor) *cc_minor = v;
  return 0;
}

uint64_t mk_workspace_bytes(const mk_program_t* prog) {
  if (!prog) return 0;
  return mk::layout_of(prog).total;
}

// Builds the program in `prog->workspace`.  With `stream_ordered` every clear
// and upload is queued on `stream` (the host buffers are pageable, so each
// copy is staged before its call returns) and the caller may launch on the
// same stream straight away; without it the copies are synchronous.
static int create_program(const mk_program_t* prog, mk_handle_t* out, bool stream_ordered, cudaStream_t stream) {
  using namespace mk;
  if (!out) return fail(-1, "null output handle");
  *out = nullptr;
  if (!prog) return fail(-1, "null program");
  DeviceScope scope;
  CUDA_TRY(cudaGetDevice(&scope.prev));
  CUDA_TRY(cudaSetDevice(prog->device));
  int smem_optin = 0, cc = 0, num_sms = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, prog->device));
  CUDA_TRY(cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, prog->device));
  CUDA_TRY(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, prog->device));
  if (cc != 10)
    return fail(-4, "device %d has compute capability %d.x; this library is built for sm_100a only", prog->device, cc);
  int smem_bytes = 0;
  int rc = validate_program(prog, smem_optin, num_sms, &smem_bytes);
  if (rc) return rc;
  const Layout l = layout_of(prog);
  if (!prog->workspace || prog->workspace_bytes < l.total || ((uint64_t)prog->workspace & 255))
    return fail(-1, "workspace must be 256-byte aligned device memory of at least %llu bytes", (unsigned long long)l.total);
  uint8_t* ws = reinterpret_cast<uint8_t*>(prog->workspace);
  auto clear = [&](void* dst, size_t n) {
    return stream_ordered ? cudaMemsetAsync(dst, 0, n, stream) : cudaMemset(dst, 0, n);
  };
  auto upload = [&](void* dst, const void* src, size_t n) {
    return stream_ordered ? cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, stream)
                          : cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice);
  };
  CUDA_TRY(clear(ws + l.state, l.ops - l.state));

  mk_handle_s* h = new mk_handle_s();
  struct Guard {
    mk_handle_s* h;
    ~Guard() { delete h; }
  } guard{h};
  {
    // tensor maps of the weight matrices, and op records that point at them
    h->ops.assign(prog->ops, prog->ops + prog->n_ops);
    std::vector<CUtensorMap> maps((size_t)prog->n_ops * kMapsPerOp);
    memset(maps.data(), 0, maps.size() * sizeof(CUtensorMap));
    for (int i = 0; i < prog->n_ops; ++i) {
      rc = build_op_maps(h->ops[i], &maps[(size_t)i * kMapsPerOp],
                         (uint64_t)(ws + l.tmaps) + (uint64_t)i * kMapsPerOp * sizeof(CUtensorMap), prog->page_bytes);
      if (rc) return rc;
    }
    CUDA_TRY(upload(ws + l.tmaps, maps.data(), maps.size() * sizeof(CUtensorMap)));
    CUDA_TRY(upload(ws + l.ops, h->ops.data(), h->ops.size() * sizeof(mk_op_t)));
  }
  if (prog->n_instrs) {
    // fill the fast path of every unit
    h->instrs.assign(prog->instrs, prog->instrs + prog->n_instrs);
    for (auto& in : h->instrs)
      fill_instr_fast_path(in, prog->ops[in.op], (uint64_t)(ws + l.tmaps), prog->page_bytes, prog->n_pages);
    CUDA_TRY(upload(ws + l.instrs, h->instrs.data(), h->instrs.size() * sizeof(mk_instr_t)));
  }
  CUDA_TRY(upload(ws + l.ibegin, prog->cta_instr_begin, (size_t)(prog->n_ctas + 1) * 4));
  if (prog->n_events) {
    // inline the head of every wait list into its event record
    std::vector<mk_event_t> events(prog->events, prog->events + prog->n_events);
    for (auto& ev : events)
      for (int k = 0; k < 4; ++k) {
        const bool have = k < ev.n_waits;
        ev.w_counter[k] = have ? prog->waits[ev.wait_off + k].counter : 0;
        ev.w_expected[k] = have ? prog->waits[ev.wait_off + k].expected : 0;
      }
    CUDA_TRY(upload(ws + l.events, events.data(), events.size() * sizeof(mk_event_t)));
  }
  CUDA_TRY(upload(ws + l.ebegin, prog->cta_event_begin, (size_t)(prog->n_ctas + 1) * 4));
  if (prog->n_waits) CUDA_TRY(upload(ws + l.waits, prog->waits, (size_t)prog->n_waits * sizeof(mk_wait_t)));

  h->pv.ops = reinterpret_cast<const mk_op_t*>(ws + l.ops);
  h->pv.instrs = reinterpret_cast<const mk_instr_t*>(ws + l.instrs);
  h->pv.cta_instr_begin = reinterpret_cast<const int32_t*>(ws + l.ibegin);
  h->pv.events = reinterpret_cast<const mk_event_t*>(ws + l.events);
  h->pv.cta_event_begin = reinterpret_cast<const int32_t*>(ws + l.ebegin);
  h->pv.waits = reinterpret_cast<const mk_wait_t*>(ws + l.waits);
  h->pv.counters = reinterpret_cast<int32_t*>(ws + l.counters);
  h->pv.state = reinterpret_cast<DeviceState*>(ws + l.state);
  h->pv.n_counters = prog->n_counters;
  h->pv.n_pages = prog->n_pages;
  h->pv.page_bytes = prog->page_bytes;
  h->pv.act_bytes = prog->act_bytes;
  h->pv.timeout_ns = (uint64_t)(prog->timeout_ms > 0 ? prog->timeout_ms : 1000) * 1000000ull;
  h->pv.trace = nullptr;
  h->pv.trace_cap = 0;
  h->pv.dyn_pos = prog->position;
  h->pv.pos_limit = prog->position_limit;
  h->pv.pos_count = prog->position_count > 0 ? prog->position_count : 1;
  h->n_ctas = prog->n_ctas;
  h->smem_bytes = smem_bytes;
  h->smem_optin = smem_optin;
  h->op_ntc.resize(prog->n_ops);
  h->op_wfc.resize(prog->n_ops);
  h->op_feat.resize(prog->n_ops);
  for (int i = 0; i < prog->n_ops; ++i) classify_op(prog->ops[i], &h->op_ntc[i], &h->op_wfc[i], &h->op_feat[i]);
  rc = select_kernel(h);
  if (rc) return rc;
  h->device = prog->device;
  h->n_ops = prog->n_ops;
  h->ws = ws;
  h->layout = l;
  guard.h = nullptr;
  *out = h;
  return 0;
}

int mk_create(const mk_program_t* prog, mk_handle_t* out) { return create_program(prog, out, false, nullptr); }

int mk_run(mk_handle_t h, void* cuda_stream) {
  using namespace mk;
  if (!h) return fail(-1, "null handle");
  void* args[] = {&h->pv};
  CUDA_TRY(cudaLaunchKernel(reinterpret_cast<const void*>(h->kernel), dim3(h->n_ctas), dim3(kThreads), args,
                            (size_t)h->smem_bytes, reinterpret_cast<cudaStream_t>(cuda_stream)));
  return 0;
}

int mk_status(mk_handle_t h, int32_t out[16]) {
  using namespace mk;
  if (!h || !out) return fail(-1, "null argument");
  CUDA_TRY(cudaMemcpy(out, h->ws + h->layout.state, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost));
  return 0;
}

int mk_set_trace(mk_handle_t h, void* buffer, uint64_t bytes, int32_t records_per_warp) {
  using namespace mk;
  if (!h) return fail(-1, "null handle");
  if (!buffer || records_per_warp <= 0) {
    h->pv.trace = nullptr;
    h->pv.trace_cap = 0;
    return select_kernel(h);
  }
  const uint64_t warps = (uint64_t)h->n_ctas * (kConsumerWarps + 1);
  const uint64_t need = warps * records_per_warp * sizeof(TraceRec) + warps * sizeof(int32_t);
  if (bytes < need || ((uint64_t)buffer & 15)) return fail(-1, "trace buffer needs %llu bytes, 16-byte aligned", (unsigned long long)need);
  if (records_per_warp < 8) return fail(-1, "a trace ring needs at least 8 records per warp");
  h->pv.trace = reinterpret_cast<TraceRec*>(buffer);
  h->pv.trace_cap = records_per_warp;
  return select_kernel(h);   // tracing is compiled into some kernel variants only
}

int mk_workspace_status(const void* workspace, int32_t out[16]) {
  using namespace mk;
  if (!workspace || !out) return fail(-1, "null argument");
  CUDA_TRY(cudaMemcpy(out, workspace, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost));
  return 0;
}

int mk_reset(mk_handle_t h, void* cuda_stream) {
  using namespace mk;
  if (!h) return fail(-1, "null handle");
  // Status, abort flag, the count of finished CTAs and the dependency counters
  // are cleared; the launch count is kept: the tensor-parallel exchange tags
  // its messages with it, and ranks stay in step only while every rank's count
  // advances once per launch.
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  uint8_t* base = h->ws + h->layout.state;
  CUDA_TRY(cudaMemsetAsync(base, 0, offsetof(DeviceState, launches), st));
  const size_t after = offsetof(DeviceState, launches) + sizeof(int32_t);
  CUDA_TRY(cudaMemsetAsync(base + after, 0, (h->layout.ops - h->layout.state) - after, st));
  return 0;
}

int mk_launch_count(mk_handle_t h, int32_t* out) {
  using namespace mk;
  if (!h || !out) return fail(-1, "null argument");
  CUDA_TRY(cudaMemcpy(out, h->ws + h->layout.state + offsetof(DeviceState, launches), sizeof(int32_t),
                      cudaMemcpyDeviceToHost));
  return 0;
}

int mk_set_launch_count(mk_handle_t h, int32_t count, void* cuda_stream) {
  using namespace mk;
  if (!h) return fail(-1, "null handle");
  if (count < 0) return fail(-1, "launch count must not be negative");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  CUDA_TRY(cudaMemcpyAsync(h->ws + h->layout.state + offsetof(DeviceState, launches), &count, sizeof(int32_t),
                           cudaMemcpyHostToDevice, st));
  CUDA_TRY(cudaStreamSynchronize(st));   // `count` lives on this stack frame
  return 0;
}

int mk_update_op(mk_handle_t h, int32_t op_index, const mk_op_t* op, void* cuda_stream) {
  using namespace mk;
  if (!h || !op) return fail(-1, "null argument");
  if (op_index < 0 || op_index >= h->n_ops) return fail(-1, "op index %d out of range", op_index);
  mk_op_t rec = *op;
  int rc = validate_op(rec, op_index, h->pv.page_bytes, h->pv.act_bytes);
  if (rc) return rc;
  if (rec.opcode != h->ops[op_index].opcode || rec.n_units != h->ops[op_index].n_units)
    return fail(-2, "op %d: an update may not change the opcode or the unit count (%d units scheduled, %d given)",
                op_index, h->ops[op_index].n_units, rec.n_units);
  // The record may carry new pointers: re-encode its tensor maps.
  CUtensorMap maps[kMapsPerOp];
  memset(maps, 0, sizeof(maps));
  uint8_t* dev_maps = h->ws + h->layout.tmaps + (size_t)op_index * kMapsPerOp * sizeof(CUtensorMap);
  rc = build_op_maps(rec, maps, (uint64_t)dev_maps, h->pv.page_bytes);
  if (rc) return rc;
  // Page counts and the per-unit fast path are derived from the record: recompute the
  // op's instruction rows and upload the span of the table that holds them.
  size_t lo = h->instrs.size(), hi = 0;
  for (size_t j = 0; j < h->instrs.size(); ++j) {
    mk_instr_t& in = h->instrs[j];
    if (in.op != op_index) continue;
    if (rec.opcode == MK_OP_MATVEC) in.n_pages = matvec_pages(rec);
    else if (rec.opcode == MK_OP_ATTN_SPLIT) in.n_pages = attn_pages(rec, in.unit, h->pv.page_bytes);
    fill_instr_fast_path(in, rec, (uint64_t)(h->ws + h->layout.tmaps), h->pv.page_bytes, h->pv.n_pages);
    lo = std::min(lo, j);
    hi = std::max(hi, j + 1);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  CUDA_TRY(cudaMemcpyAsync(dev_maps, maps, sizeof(maps), cudaMemcpyHostToDevice, st));
  CUDA_TRY(cudaMemcpyAsync(h->ws + h->layout.ops + (size_t)op_index * sizeof(mk_op_t), &rec, sizeof(mk_op_t),
                           cudaMemcpyHostToDevice, st));
  if (hi > lo)
    CUDA_TRY(cudaMemcpyAsync(h->ws + h->layout.instrs + lo * sizeof(mk_instr_t), h->instrs.data() + lo,
                             (hi - lo) * sizeof(mk_instr_t), cudaMemcpyHostToDevice, st));
  // the host buffers above must outlive the copies
  CUDA_TRY(cudaStreamSynchronize(st));
  h->ops[op_index] = rec;
  // a changed batch size or weight format may need another kernel variant
  classify_op(rec, &h->op_ntc[op_index], &h->op_wfc[op_index], &h->op_feat[op_index]);
  return select_kernel(h);
}

int mk_read_counters(mk_handle_t h, int32_t* out, int32_t n) {
  using namespace mk;
  if (!h || !out) return fail(-1, "null argument");
  if (n > h->pv.n_counters) n = h->pv.n_counters;
  if (n > 0) CUDA_TRY(cudaMemcpy(out, h->ws + h->layout.counters, (size_t)n * 4, cudaMemcpyDeviceToHost));
  return 0;
}

int mk_destroy(mk_handle_t h) {
  delete h;
  return 0;
}

}  // extern "C"

#include "standalone.inc"
#include "noalloc.inc"
