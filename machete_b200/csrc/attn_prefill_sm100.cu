// Prefill attention on the 5th-generation tensor cores: O = softmax(scale · Q Kᵀ) V for a block of
// query rows against a KV cache, bf16, causal or not, grouped-query heads.
//
// The decode megakernel's own attention op streams K/V once per KV head for a handful of query rows
// (mma.sync).  A prompt has hundreds of query rows per head, which is tensor-core work: this kernel
// takes the place of the reference's FlashAttentionSm100Op (src/machete/kernels/attention/
// sm_100.py:88-…, dispatch attention/__init__.py:16-130) as a launch of its own, so that a prompt can
// fill the KV cache the decode kernel then reads.
//
// One CTA = one (batch, query head, tile of 128 query rows); KV tiles of 64 tokens; two CTAs share an SM
// (<= 97 KB of shared memory and 256 tensor-memory columns each):
//
//   warp 0     TMA: Q once, then K and V tiles (both double-buffered, K one tile ahead of V) as
//              64-column boxes, 128-byte swizzle;
//   warp 1     tcgen05.mma issuer: S(j) = Q K(j)^T into one of two tensor-memory accumulators, one tile
//              ahead of the softmax, and O += P(j) V(j) with P read FROM TENSOR MEMORY (the M x K
//              operand) and V as the N operand in MN-major form (its head dimension is contiguous in
//              shared memory exactly as the cache stores it);
//   warps 2-5  one thread per query row (= tensor-memory lane): one tcgen05.ld of the row of S(j), mask,
//              maximum, P = exp2(scale * s - reference) with packed f32x2 arithmetic, running sum in
//              registers (no shuffles: a thread owns its row), P stored as bf16 pairs over the first half
//              of the accumulator it came from (tcgen05.st), O rescaled in tensor memory only when a row
//              maximum outgrew the exponent reference by 2^8; normalised bf16 store at the end.
//
// The row threads never wait for P V: while the tensor cores run P(j) V(j) and S(j + 2) they are already
// on tile j + 1, so the exponentials (the scarce unit: 16 per clock and SM) and the products overlap inside
// one CTA, and the second CTA of the SM fills what is left.
//
// Every wait is bounded; on expiry the CTA records a status, raises its abort flag, all roles fall
// through to the common exit and tensor memory is freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <type_traits>

#include "../../include/machete_b200.h"
#include "prims.cuh"

namespace mkp {

constexpr int kThreads = 192;
constexpr int kBM = 128;   // query rows per CTA
constexpr int kBN = 64;    // tokens per KV tile
constexpr uint32_t kBox = 128 * 64 * 2;   // one 128-row x 64-column bf16 box

struct Params {
  __nv_bfloat16* o;
  float* lse;            // [B, H, M] or null
  int32_t* status;
  int64_t o_sb, o_sh, o_sm;
  int B, H, Hkv, M, N, D;
  int causal;
  float scale_log2;      // scale * log2(e)
  uint64_t timeout_ns;
};

enum { PF_ST_TIMEOUT_EMPTY = 1, PF_ST_TIMEOUT_FULL = 2, PF_ST_TIMEOUT_S = 3, PF_ST_TIMEOUT_P = 4, PF_ST_TIMEOUT_O = 5 };

struct Shared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_ready[2], p_ready[2], pv_done[2];
  uint32_t tmem_base;
  int32_t abort_flag;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  // the M x K operand comes from tensor memory (lane = row, one 32-bit column = two bf16 along K)
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.ftz.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// one row of a 64-column accumulator; the wait is part of the statement so that nothing reads r before it
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {"
      "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Two fp32 operations per instruction (the packed f32x2 forms of sm_100): the softmax of one score costs the
// issue slots of half a multiply-add, one exp2, half an add and half a conversion.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// 2^x for two values on the FMA and integer pipes instead of the exp2 unit (16 results per clock and SM,
// the scarce unit at head dim 64): x = n + f with n = round(x) by the 1.5 * 2^23 addition, f in [-0.5, 0.5];
// 2^f by a cubic fitted here for the smallest maximal relative error (7.5e-5, far inside bf16's 2^-9), and
// n added to the exponent field.  x <= 8 by construction; below -126 it is clamped (the result, ~1e-38,
// rounds into nothing next to the row's maximum of at least 2^-8).
// Measured at 32 heads x 4096 x 4096: head dim 64, every third pair of scores on this path, 113 -> 109 us
// (every second: 114); head dim 128, where the tensor pipe is the bound, 131 -> 135 us: used at 64 only.
#ifndef MK_PF_POLY
#define MK_PF_POLY 3      /* head dim 64: every MK_PF_POLY-th pair of scores takes this path on unmasked tiles (0 = none) */
#endif
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& e0, float& e1) {
  float x0, x1;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(x2));
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  uint64_t xc, r, t, f, pl;
  asm("mov.b64 %0, {%1, %2};" : "=l"(xc) : "f"(x0), "f"(x1));
  const uint64_t magic = 0x4B4000004B400000ull, nmagic = 0xCB400000CB400000ull, neg1 = 0xBF800000BF800000ull;
  asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(xc), "l"(magic));
  asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(t) : "l"(r), "l"(nmagic));
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(f) : "l"(t), "l"(neg1), "l"(xc));
  // Horner: ((c3 f + c2) f + c1) f + c0
  const uint64_t c3 = 0x3D61FBB03D61FBB0ull, c2 = 0x3E786F0D3E786F0Dull, c1 = 0x3F31798D3F31798Dull, c0 = 0x3F7FFB493F7FFB49ull;
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(pl) : "l"(c3), "l"(f), "l"(c2));
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(pl) : "l"(pl), "l"(f), "l"(c1));
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(pl) : "l"(pl), "l"(f), "l"(c0));
  uint32_t p0, p1, r0, r1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(p0), "=r"(p1) : "l"(pl));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(r0), "=r"(r1) : "l"(r));
  e0 = __uint_as_float(p0 + (r0 << 23));
  e1 = __uint_as_float(p1 + (r1 << 23));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.ftz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// K-major bf16 tile of 128-byte swizzled rows (8-row groups 1024 bytes apart): Q, K and P.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major bf16 tile: V as stored, [token][64 head-dim values = 128 bytes], 128-byte swizzle.  Along K (tokens)
// the 8-row groups are 1024 bytes apart (stride offset); along N (head dim) the next 64 values are the next
// box, `next_box` bytes further (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t next_box) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((next_box >> 4) & 0x3FFF) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16, fp32 accumulate, bf16 operands, M = 128, N = n; b_mn = the N operand is MN-major.
__device__ __forceinline__ uint32_t idesc_bf16(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void give_up(const Params& p, Shared* sh, int code, int aux) {
  if (atomicCAS(&p.status[0], 0, code) == 0) {
    p.status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    p.status[2] = threadIdx.x >> 5;
    p.status[3] = aux;
  }
  atomicExch(&sh->abort_flag, 1);
  __threadfence();
}
__device__ __forceinline__ bool wait_bar(const Params& p, Shared* sh, uint32_t bar, uint32_t parity, int code, int aux) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mk::mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 255u) {
      if (*reinterpret_cast<volatile int32_t*>(&sh->abort_flag)) return false;
      const uint64_t now = mk::globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > p.timeout_ns) {
        give_up(p, sh, code, aux);
        return false;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const Params p) {
  constexpr int NB = D / 64;                       // 64-column boxes per row tile
  constexpr uint32_t kTile = NB * kBox;            // the 128 x D query tile
  constexpr uint32_t kKVBox = kBN * 64 * 2;        // one 64-token x 64-column box of K or V
  constexpr uint32_t kKVTile = NB * kKVBox;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = mk::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  // layout: Q | K0 | K1 | V0 | V1 | control
  const uint32_t q_s = base, k_s = q_s + kTile, v_s = k_s + 2 * kKVTile;
  Shared* sh = reinterpret_cast<Shared*>(smem + kTile + 4 * kKVTile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are handed out in the order x, y, z: the query tile is the slowest index and runs from the LAST tile
  // down, so that under a causal mask the tiles with the most KV tiles start first and the short ones fill the
  // tail (longest job first).
  const int mt = (int)(gridDim.z - 1 - blockIdx.z), h = blockIdx.x, b = blockIdx.y;
  const int kvh = h / (p.H / p.Hkv);
  const int m0 = mt * kBM;
  // tokens this query tile can see: all N, or (causal) up to the diagonal of its last row
  const int n_vis = p.causal ? min(p.N, p.N - p.M + m0 + kBM) : p.N;
  const int n_tiles = n_vis > 0 ? (n_vis + kBN - 1) / kBN : 0;
  // 256 tensor-memory columns and at most ~100 KB of shared memory per CTA, so that TWO CTAs share an SM.
  // Two S accumulators at columns [0, 64) / [64, 128) (P, as bf16 pairs, overwrites the first 32 columns of
  // the accumulator it was computed from), O at [128, 128 + D).
  constexpr uint32_t kOCol = 2 * kBN, kCols = 256;
  static_assert(kOCol + D <= kCols, "accumulators must fit the allocation");

  if (threadIdx.x == 0) {
    mk::mbar_init(mk::smem_u32(&sh->q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mk::mbar_init(mk::smem_u32(&sh->k_full[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->k_empty[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->v_full[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->v_empty[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->s_ready[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->p_ready[s]), 128);
      mk::mbar_init(mk::smem_u32(&sh->pv_done[s]), 1);
    }
    sh->abort_flag = 0;
    mk::fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(mk::smem_u32(&sh->tmem_base), kCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

  // Tile j uses slot j & 1 of every double-buffered resource; its barrier phase is (j >> 1) & 1.
  if (warp == 0) {
    if (lane == 0) {
      const uint32_t qb = mk::smem_u32(&sh->q_full);
      mk::mbar_arrive_expect_tx(qb, kTile);
      for (int x = 0; x < NB; ++x) tma_load_4d(q_s + x * kBox, &map_q, x * 64, m0, h, b, qb);
      auto load_kv = [&](int j, bool is_v) -> bool {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        uint64_t* empty = is_v ? &sh->v_empty[s] : &sh->k_empty[s];
        uint64_t* full = is_v ? &sh->v_full[s] : &sh->k_full[s];
        if (!wait_bar(p, sh, mk::smem_u32(empty), ph ^ 1u, PF_ST_TIMEOUT_EMPTY, j)) return false;
        const uint32_t fb = mk::smem_u32(full);
        mk::mbar_arrive_expect_tx(fb, kKVTile);
        const uint32_t dst = (is_v ? v_s : k_s) + (uint32_t)s * kKVTile;
        for (int x = 0; x < NB; ++x) tma_load_4d(dst + x * kKVBox, is_v ? &map_v : &map_k, x * 64, j * kBN, kvh, b, fb);
        return true;
      };
      // K runs one tile ahead of V: S(j + 1) is issued before P(j) V(j)
      bool pok = n_tiles > 0 ? load_kv(0, false) : true;
      for (int j = 0; j < n_tiles && pok; ++j) {
        if (j + 1 < n_tiles && !load_kv(j + 1, false)) break;
        if (!load_kv(j, true)) break;
      }
      if (*reinterpret_cast<volatile int32_t*>(&sh->abort_flag)) {
        // shared memory must outlive the copies in flight: a bounded wait for whatever was issued last
        const uint64_t t0 = mk::globaltimer_ns();
        while (mk::globaltimer_ns() - t0 < 20000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_s = idesc_bf16(kBN, false), id_o = idesc_bf16(D, true);
      bool ok = wait_bar(p, sh, mk::smem_u32(&sh->q_full), 0, PF_ST_TIMEOUT_FULL, -1);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!wait_bar(p, sh, mk::smem_u32(&sh->k_full[s]), (uint32_t)(j >> 1) & 1u, PF_ST_TIMEOUT_FULL, j)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t in_box = (uint32_t)(k & 3) * 32u;
          tc_mma(tmem + (uint32_t)s * kBN, desc_kmajor(q_s + (uint32_t)(k >> 2) * kBox + in_box),
                 desc_kmajor(k_s + s * kKVTile + (uint32_t)(k >> 2) * kKVBox + in_box), id_s, k > 0 ? 1u : 0u);
        }
        tc_commit(mk::smem_u32(&sh->s_ready[s]));
        tc_commit(mk::smem_u32(&sh->k_empty[s]));
        return true;
      };
      // Issue order S(0), S(1), P V(0), S(2), P V(1), S(3), ...  The tensor cores run the products in this
      // order, so S(j + 2) overwrites accumulator j & 1 only after P V(j) has read P(j) from it, and the
      // row threads find S(j + 1) finished while P V(j) is still running.
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        // O += P V once the row threads have written P (and rescaled O)
        ok = wait_bar(p, sh, mk::smem_u32(&sh->p_ready[s]), ph, PF_ST_TIMEOUT_P, j) &&
             wait_bar(p, sh, mk::smem_u32(&sh->v_full[s]), ph, PF_ST_TIMEOUT_FULL, j);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          // P: 16 tokens = 8 tensor-memory columns of bf16 pairs; V: MN-major, 16 tokens = 16 rows of 128 bytes
          const uint64_t dv = desc_mnmajor(v_s + (uint32_t)s * kKVTile + (uint32_t)k * 2048u, kKVBox);
          tc_mma_ts(tmem + kOCol, tmem + (uint32_t)s * kBN + (uint32_t)k * 8u, dv, id_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(mk::smem_u32(&sh->pv_done[s]));
        tc_commit(mk::smem_u32(&sh->v_empty[s]));
      }
    }
  } else {
    // row threads: warp w may touch tensor-memory lanes 32 * (w % 4) ..
    const int qd = warp & 3;
    const int row = qd * 32 + lane;                 // query row inside the tile = TMEM lane
    const int m = m0 + row;
    const int lim = p.causal ? (p.N - p.M + m) : (p.N - 1);   // last visible token of this row
    const uint32_t lane_addr = tmem + ((uint32_t)(qd * 32) << 16);
    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);
    float mx = -INFINITY, sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = wait_bar(p, sh, mk::smem_u32(&sh->s_ready[j & 1]), (uint32_t)(j >> 1) & 1u, PF_ST_TIMEOUT_S, j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // Only the tiles on the causal diagonal and the last one of a ragged cache need the per-score
      // mask: `open` is true (for the whole warp) everywhere else.
      const bool open = __all_sync(0xffffffffu, (j * kBN + kBN - 1 <= lim) && (j * kBN + kBN <= p.N));
      const uint32_t s_addr = lane_addr + (uint32_t)(j & 1) * kBN;
      uint32_t r[kBN];                               // this row of S, then of P (bf16 pairs in r[0 .. 32))
      tmem_ld64(s_addr, r);
      if (!open) {
#pragma unroll
        for (int i = 0; i < kBN; ++i) {
          const int tok = j * kBN + i;
          if (!(tok <= lim && tok < p.N)) r[i] = 0xff800000u;          // -inf: exp2 gives 0
        }
      }
      float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kBN; i += 8) {
#pragma unroll
        for (int u = 0; u < 4; ++u) t4[u] = max3(t4[u], __uint_as_float(r[i + 2 * u]), __uint_as_float(r[i + 2 * u + 1]));
      }
      const float tmax = max3(fmaxf(t4[0], t4[1]), t4[2], t4[3]) * p.scale_log2;   // the scale is positive
      // mx is the exponent reference in use, not the running maximum: it moves only when a maximum has grown
      // by more than 2^8 since it was set, so O is rescaled rarely (and no P exceeds 2^8).
      float alpha = 1.f;
      if (tmax > mx + 8.f) {                         // also the first visible tile (mx = -inf)
        alpha = exp2f(mx - tmax);                    // 0 when mx = -inf
        mx = tmax;
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O is free only after the previous P V has finished with it.  S(j) was issued after P V(j - 2), so
        // that phase of this barrier is behind us and the parity is unambiguous.
        ok = wait_bar(p, sh, mk::smem_u32(&sh->pv_done[(j - 1) & 1]), (uint32_t)((j - 1) >> 1) & 1u, PF_ST_TIMEOUT_O, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld32(lane_addr + kOCol + (uint32_t)c, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(lane_addr + kOCol + (uint32_t)c, o);
        }
      }
      sum *= alpha;
      const float muse = mx == -INFINITY ? 0.f : mx;
      const uint64_t ref2 = pack2(-muse, -muse);
      // P = exp2(s * scale - reference), two scores per multiply-add, add and conversion
      uint64_t tsum2 = pack2(0.f, 0.f);
      auto p_pass = [&](auto mixed) {
#pragma unroll
        for (int i = 0; i < kBN; i += 2) {
          const uint64_t x2 = fma2(pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, ref2);
          float e0, e1;
          if (decltype(mixed)::value && ((i >> 1) % (MK_PF_POLY > 0 ? MK_PF_POLY : 1)) == 0) {   // compile-time pattern
            exp2_poly2(x2, e0, e1);
          } else {
            float x0, x1;
            unpack2(x2, x0, x1);
            e0 = exp2f(x0);
            e1 = exp2f(x1);
          }
          const __nv_bfloat162 pk = __floats2bfloat162_rn(e0, e1);
          // the row sum is taken before the rounding to bf16 (an unbiased 2^-9 relative error per term)
          tsum2 = add2(tsum2, pack2(e0, e1));
          r[i >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
        }
      };
      // masked tiles keep the exp2 unit for every score: exp2(-inf) is exactly 0 there
      if (MK_PF_POLY > 0 && D == 64 && open)
        p_pass(std::true_type{});
      else
        p_pass(std::false_type{});
      float t0, t1;
      unpack2(tsum2, t0, t1);
      sum += t0 + t1;
      // P goes where its S came from: 64 bf16 = the first 32 columns of the accumulator
      tmem_st32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_wait_st();
      tc_fence_before();
      mk::mbar_arrive(mk::smem_u32(&sh->p_ready[j & 1]));
    }
    // epilogue: O / sum -> bf16
    if (ok && n_tiles > 0) {
      ok = wait_bar(p, sh, mk::smem_u32(&sh->pv_done[(n_tiles - 1) & 1]), (uint32_t)((n_tiles - 1) >> 1) & 1u,
                    PF_ST_TIMEOUT_O, n_tiles);
      ok = __all_sync(0xffffffffu, ok);
    }
    tc_fence_after();
    if (ok) {
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      __nv_bfloat16* dst = p.o + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)m * p.o_sm;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld32(lane_addr + kOCol + (uint32_t)c, o);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (m < p.M) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * u]) * inv,
                                                              __uint_as_float(o[i + 2 * u + 1]) * inv);
              w[u] = *reinterpret_cast<const uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (p.lse != nullptr && m < p.M)
        p.lse[((int64_t)b * p.H + h) * p.M + m] = sum > 0.f ? (mx + log2f(sum)) * 0.6931471805599453f : -INFINITY;
    }
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem, kCols);
}

static std::string g_err;
static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
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
// [batch][head][row][D] with element strides (s_b, s_h, s_r), D contiguous: dims (D, rows, heads, batch),
// one box = 64 columns x 128 rows of one head of one batch entry.
static int encode_rows_map(CUtensorMap* out, const void* base, int D, int rows, int heads, int batch, int64_t s_r,
                           int64_t s_h, int64_t s_b, int box_rows, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(-5, "cuTensorMapEncodeTiled is not available from this driver");
  if (((uint64_t)base & 15) || (s_r * 2) % 16 || (s_h * 2) % 16 || (s_b * 2) % 16 || s_r <= 0 || s_h <= 0 || s_b <= 0)
    return fail(-2, "mk_flash_prefill_bf16: %s must be 16-byte aligned with positive row / head / batch strides that are "
                    "multiples of 8 elements", what);
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)s_r * 2, (cuuint64_t)s_h * 2, (cuuint64_t)s_b * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled (%s) failed with CUresult %d", what, (int)r);
  return 0;
}

}  // namespace mkp

extern "C" {

const char* mk_flash_prefill_last_error(void) { return mkp::g_err.c_str(); }

int mk_flash_prefill_bf16(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Hkv, int M,
                          int N, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                          const int64_t v_strides[3], const int64_t o_strides[3], float scale, int causal,
                          void* workspace, uint64_t workspace_bytes, int timeout_ms, void* cuda_stream) {
  using namespace mkp;
  if (!q || !k || !v || !o || !workspace || !q_strides || !k_strides || !v_strides || !o_strides)
    return fail(-1, "mk_flash_prefill_bf16: null pointer");
  if (B < 1 || H < 1 || Hkv < 1 || M < 1 || N < 1 || H % Hkv)
    return fail(-2, "mk_flash_prefill_bf16: B, H, Hkv, M, N must be positive and H a multiple of Hkv");
  if (D != 64 && D != 128) return fail(-2, "mk_flash_prefill_bf16: head dim must be 64 or 128, got %d", D);
  if (B > 65535 || (M + 127) / 128 > 65535) return fail(-2, "mk_flash_prefill_bf16: at most 65535 batch entries and 65535 query tiles of 128 rows");
  if (causal && M > N) return fail(-2, "mk_flash_prefill_bf16: causal attention needs M <= N (the queries are the last M tokens)");
  if (workspace_bytes < 256 || ((uint64_t)workspace & 255)) return fail(-2, "mk_flash_prefill_bf16: workspace of 256 aligned bytes");
  if (((uint64_t)o & 15) || o_strides[2] % 8 || o_strides[1] % 8 || o_strides[0] % 8)
    return fail(-2, "mk_flash_prefill_bf16: o must be 16-byte aligned with strides that are multiples of 8 elements");
  int dev = 0, smem_optin = 0, cc = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(-1001, "cudaGetDevice failed");
  cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev);
  if (cc != 10) return fail(-6, "mk_flash_prefill_bf16 needs an sm_100 device (compute capability %d.x found)", cc);
  const int bn = kBN;                              // tokens per KV tile
  CUtensorMap mq, mkk, mv;
  int rc = encode_rows_map(&mq, q, D, M, H, B, q_strides[2], q_strides[1], q_strides[0], kBM, "q");
  if (rc) return rc;
  rc = encode_rows_map(&mkk, k, D, N, Hkv, B, k_strides[2], k_strides[1], k_strides[0], bn, "k");
  if (rc) return rc;
  rc = encode_rows_map(&mv, v, D, N, Hkv, B, v_strides[2], v_strides[1], v_strides[0], bn, "v");
  if (rc) return rc;
  const size_t tile = (size_t)(D / 64) * kBox, kv_tile = (size_t)(D / 64) * bn * 128;
  const size_t smem = 1024 + tile + 4 * kv_tile + sizeof(Shared);
  if ((int)smem > smem_optin) return fail(-4, "mk_flash_prefill_bf16: %zu bytes of shared memory needed, %d available", smem, smem_optin);
  Params p;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.status = reinterpret_cast<int32_t*>(workspace);
  p.o_sb = o_strides[0], p.o_sh = o_strides[1], p.o_sm = o_strides[2];
  p.B = B, p.H = H, p.Hkv = Hkv, p.M = M, p.N = N, p.D = D;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.timeout_ns = (uint64_t)(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull;
  const dim3 grid(H, B, (M + kBM - 1) / kBM);
  static bool attr64[64] = {}, attr128[64] = {};
  cudaError_t e = cudaSuccess;
  if (D == 64) {
    if (dev < 64 && !attr64[dev]) {
      e = cudaFuncSetAttribute(prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
      attr64[dev] = e == cudaSuccess;
    }
    if (e == cudaSuccess) prefill_kernel<64><<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(mq, mkk, mv, p);
  } else {
    if (dev < 64 && !attr128[dev]) {
      e = cudaFuncSetAttribute(prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin);
      attr128[dev] = e == cudaSuccess;
    }
    if (e == cudaSuccess) prefill_kernel<128><<<grid, kThreads, smem, reinterpret_cast<cudaStream_t>(cuda_stream)>>>(mq, mkk, mv, p);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-(int)e - 1000, "mk_flash_prefill_bf16 launch: %s", cudaGetErrorString(e));
  return 0;
}

int mk_flash_prefill_status(const void* workspace, int32_t out[4]) {
  if (!workspace || !out) return mkp::fail(-1, "mk_flash_prefill_status: null pointer");
  if (cudaDeviceSynchronize() != cudaSuccess) return mkp::fail(-1001, "mk_flash_prefill_status: device synchronise failed");
  if (cudaMemcpy(out, workspace, 16, cudaMemcpyDeviceToHost) != cudaSuccess)
    return mkp::fail(-1001, "mk_flash_prefill_status: copy failed");
  return 0;
}

}  // extern "C"
