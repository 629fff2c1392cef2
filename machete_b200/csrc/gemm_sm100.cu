// Small-M bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] · B[N,K]^T.
//
// The decode path's own matvec ops cover M <= 32 with mma.sync; from M = 64 up the
// work is worth a tcgen05 tile.  The problem is still weight-streaming bound
// (M <= 256 rows against an N x K weight), so the tile is laid out around the
// weight stream: the WEIGHT rows are the 128-row "M" operand of tcgen05.mma and the
// activation rows are its "N" operand (16..256 columns), i.e. the kernel computes
// C^T tile by tile.  One CTA owns 128 weight rows x one K range:
//
//   warp 0   TMA producer: per 64-wide K step one 128 x 64 weight box and one
//            Mpad x 64 activation box (128-byte swizzle) into a ring of stages;
//   warp 1   allocates tensor memory, issues tcgen05.mma (one thread), hands
//            stages back with tcgen05.commit;
//   warps 2-5 epilogue: tcgen05.ld of the fp32 accumulator (TMEM lane = weight
//            row, column = activation row) and bf16 stores.
//
// One SM cannot keep enough reads in flight to draw more than roughly 1/148 of the
// HBM bandwidth, so a weight with few 128-row tiles is also split along K: the CTAs
// of one output tile form a thread-block cluster, each leaves its fp32 partial tile
// in its own shared memory (the stage ring is free by then), and after a cluster
// barrier every CTA sums one slice of the rows over all peers through distributed
// shared memory and stores it.  No global workspace and no atomics are involved.
//
// Takes the place of the reference's GemmSm100Op (src/machete/kernels/gemm/
// gemm_sm100.py:56-658), which tiles (S, N) with a double-buffered K loop inside
// its interpreter; this one is a plain launch next to the decode megakernel.
//
// Every wait is bounded: a wait that runs out records a status, raises a CTA-wide
// abort flag, and all roles fall through to the common exit, where tensor memory
// is freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "../../include/machete_b200.h"
#include "prims.cuh"

namespace mkg {

constexpr int kThreads = 192;
constexpr int kTileN = 128;        // weight rows per CTA (the MMA's M)
constexpr int kTileK = 64;         // one 128-byte swizzle atom of bf16
constexpr int kMaxM = 256;         // activation rows per CTA (the MMA's N)
constexpr int kMaxStages = 8;
constexpr uint32_t kWBytes = kTileN * kTileK * 2;

struct Params {
  __nv_bfloat16* c;
  int32_t* status;       // [0] code, [1] cta, [2] role, [3] aux
  int64_t ldc;
  int M, N, K;
  int split_k, k_tiles;
  int stages;
  uint32_t ring_bytes;   // stages x stage bytes, or the fp32 partial tile if that is larger (split-K)
  int activation;        // applied to the fp32 sum before the bf16 store: 0 none, 1 relu, 2 silu
  int b_packed;          // the weight is stored K-tile-major: [K/64][N][64] (one box = 16 KB contiguous)
  int m_box;             // rows of one activation box (what one TMA copy delivers, whatever this CTA uses of it)
  uint64_t timeout_ns;
};

enum { GEMM_ST_OK = 0, GEMM_ST_TIMEOUT_EMPTY = 1, GEMM_ST_TIMEOUT_FULL = 2, GEMM_ST_TIMEOUT_ACC = 3 };

struct Shared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_ready;
  uint32_t tmem_base;
  int32_t abort_flag;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar), "l"(pol)
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `addr` (a shared address of this CTA) in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
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
// D[tmem] (+)= A[smem desc] x B[smem desc]^T, both operands K-major bf16, fp32 accumulate.
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 consecutive fp32 columns of this warp's 32 TMEM lanes: thread t gets lane t, columns c..c+31.
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

// Shared-memory matrix descriptor of a K-major bf16 tile stored as 128-byte rows with the
// 128-byte swizzle (what the TMA boxes above write): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                           // leading-dimension offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride between 8-row groups
  d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
  return d;
}
// kind::f16 instruction descriptor: fp32 accumulator, bf16 x bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
}

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return fmaxf(v, 0.f);
  if (act == 2) return v / (1.f + __expf(-v));
  return v;
}

__device__ __forceinline__ void give_up(const Params& p, Shared* sh, int code, int role, int aux) {
  if (atomicCAS(&p.status[0], 0, code) == 0) {
    p.status[1] = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    p.status[2] = role;
    p.status[3] = aux;
  }
  atomicExch(&sh->abort_flag, 1);
  __threadfence();
}
// One thread waits for an mbarrier phase; false = aborted or out of time (recorded).
__device__ __forceinline__ bool wait_bar(const Params& p, Shared* sh, uint32_t bar, uint32_t parity, int code, int role, int aux) {
  // The clock is read only after a batch of failed polls: reading the global timer costs about as
  // much as a whole K step, and almost every wait succeeds within a few polls.
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if (mk::mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 255u) {
      if (*reinterpret_cast<volatile int32_t*>(&sh->abort_flag)) return false;
      const uint64_t now = mk::globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > p.timeout_ns) {
        give_up(p, sh, code, role, aux);
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // stages first (1024-byte aligned for the swizzle), the control block after them
  const uint32_t raw = mk::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const int m0 = blockIdx.z * kMaxM;
  const int m_here = min(kMaxM, p.M - m0);
  const int mpad = (m_here + 15) & ~15;                       // the MMA's N: a multiple of 16
  const uint32_t a_bytes = (uint32_t)p.m_box * kTileK * 2;
  const uint32_t stage_bytes = (kWBytes + a_bytes + 1023u) & ~1023u;
  Shared* sh = reinterpret_cast<Shared*>(smem + p.ring_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kTileN;
  // this CTA's K steps
  const int per = (p.k_tiles + p.split_k - 1) / p.split_k;
  const int kt0 = blockIdx.y * per, kt1 = min(p.k_tiles, kt0 + per);
  const int n_steps = max(0, kt1 - kt0);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < mpad) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mk::mbar_init(mk::smem_u32(&sh->full[s]), 1);
      mk::mbar_init(mk::smem_u32(&sh->empty[s]), 1);
    }
    mk::mbar_init(mk::smem_u32(&sh->acc_ready), 1);
    sh->abort_flag = 0;
    mk::fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(mk::smem_u32(&sh->tmem_base), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = mk::l2_evict_first_policy();
      int issued = 0;
      for (int i = 0; i < n_steps; ++i, ++issued) {
        const int s = i % p.stages;
        const uint32_t it = (uint32_t)(i / p.stages);
        if (!wait_bar(p, sh, mk::smem_u32(&sh->empty[s]), (it & 1u) ^ 1u, GEMM_ST_TIMEOUT_EMPTY, 0, i)) break;
        const uint32_t dst = base + (uint32_t)s * stage_bytes;
        const uint32_t bar = mk::smem_u32(&sh->full[s]);
        mk::mbar_arrive_expect_tx(bar, kWBytes + a_bytes);
        if (p.b_packed)
          mk::tma_load_3d(dst, &map_b, 0, n0, kt0 + i, bar, pol);
        else
          tma_load_2d_hint(dst, &map_b, (kt0 + i) * kTileK, n0, bar, pol);
        tma_load_2d(dst + kWBytes, &map_a, (kt0 + i) * kTileK, m0, bar);
      }
      if (*reinterpret_cast<volatile int32_t*>(&sh->abort_flag)) {
        // shared memory must outlive the copies still in flight: wait (bounded) for the stages that
        // were issued but perhaps never consumed
        for (int i = max(0, issued - p.stages); i < issued; ++i) {
          const uint32_t bar = mk::smem_u32(&sh->full[i % p.stages]);
          const uint64_t t0 = mk::globaltimer_ns();
          while (!mk::mbar_try_wait(bar, (uint32_t)(i / p.stages) & 1u) && mk::globaltimer_ns() - t0 < p.timeout_ns) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(mpad);
      bool ok = true;
      for (int i = 0; i < n_steps && ok; ++i) {
        const int s = i % p.stages;
        const uint32_t it = (uint32_t)(i / p.stages);
        ok = wait_bar(p, sh, mk::smem_u32(&sh->full[s]), it & 1u, GEMM_ST_TIMEOUT_FULL, 1, i);
        if (!ok) break;
        tc_fence_after();
        const uint32_t w_addr = base + (uint32_t)s * stage_bytes;
        const uint64_t dw = smem_desc_sw128(w_addr), da = smem_desc_sw128(w_addr + kWBytes);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k)     // 16 bf16 = 32 bytes = 2 descriptor units per MMA
          tc_mma_bf16(tmem, dw + 2u * k, da + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(mk::smem_u32(&sh->empty[s]));   // the stage is free once these MMAs have read it
      }
      if (ok) tc_commit(mk::smem_u32(&sh->acc_ready));
    }
  } else {
    // epilogue warps 2..5: warp w may touch TMEM lanes 32 * (w % 4) ..
    const int q = warp & 3;
    bool ready = n_steps > 0 && wait_bar(p, sh, mk::smem_u32(&sh->acc_ready), 0, GEMM_ST_TIMEOUT_ACC, 2, warp);
    ready = __all_sync(0xffffffffu, ready);      // the tensor-memory loads below are warp-wide
    tc_fence_after();
    const int n = n0 + q * 32 + lane;
    const bool n_ok = n < p.N;
    // split-K: the partial tile goes to this CTA's shared memory as fp32 [activation row][128 weight rows]
    // (the stage ring is free: every copy was consumed before the accumulator was declared ready)
    float* part = reinterpret_cast<float*>(smem) + q * 32 + lane;
    for (int c = 0; c < mpad; c += 32) {
      uint32_t r[32];
      if (ready) {
        tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c, r);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;      // an empty K range (or an aborted CTA) adds nothing
      }
      if (p.split_k == 1) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int m = m0 + c + j;
          if (ready && n_ok && m < p.M)
            p.c[(int64_t)m * p.ldc + n] = __float2bfloat16_rn(apply_act(__uint_as_float(r[j]), p.activation));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c + j < mpad) part[(c + j) * kTileN] = __uint_as_float(r[j]);
      }
    }
    tc_fence_before();
  }
  __syncthreads();

  if (p.split_k > 1) {
    // The CTAs of this output tile are one cluster (its rank = the K split).  Each sums its slice of
    // the activation rows over every peer's partial tile and stores it.
    cluster_sync_all();
    const int rank = (int)cluster_ctarank();
    const int rows_per = (mpad + p.split_k - 1) / p.split_k;
    const int r_lo = rank * rows_per, r_hi = min(mpad, r_lo + rows_per);
    for (int idx = threadIdx.x; idx < (r_hi - r_lo) * (kTileN / 4); idx += kThreads) {
      const int ml = r_lo + idx / (kTileN / 4), nl = (idx % (kTileN / 4)) * 4;
      const uint32_t off = base + (uint32_t)(ml * kTileN + nl) * 4u;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int peer = 0; peer < p.split_k; ++peer) {
        const float4 v = ld_cluster_f4(peer_smem(off, (uint32_t)peer));
        acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
      }
      const int m = m0 + ml, n = n0 + nl;
      if (m < p.M) {
        __nv_bfloat16* dst = p.c + (int64_t)m * p.ldc + n;
        const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (n + e < p.N) dst[e] = __float2bfloat16_rn(apply_act(v[e], p.activation));
      }
    }
    cluster_sync_all();        // nobody leaves while a peer may still read its partial tile
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem, tmem_cols);
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
// A row-major bf16 matrix [rows, K] with row stride `ld` elements; one box = 64 K values x box_rows rows.
static int encode_bf16_map(CUtensorMap* out, const void* base, int rows, int K, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(-5, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

// The same matrix stored K-tile-major, [K/64][N][64]: dims (64, N, K/64), one box = 128 rows of one K tile,
// which is one contiguous 16 KB piece of memory.
static int encode_packed_map(CUtensorMap* out, const void* base, int N, int k_tiles) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(-5, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)kTileK, (cuuint64_t)N, (cuuint64_t)k_tiles};
  cuuint64_t strides[2] = {(cuuint64_t)kTileK * 2, (cuuint64_t)N * kTileK * 2};
  cuuint32_t box[3] = {(cuuint32_t)kTileK, (cuuint32_t)kTileN, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-5, "cuTensorMapEncodeTiled (packed weight) failed with CUresult %d", (int)r);
  return 0;
}

static int pick_split(int M, int N, int K, int sms) {
  const int tiles = ((N + kTileN - 1) / kTileN) * ((M + kMaxM - 1) / kMaxM);
  const int k_tiles = (K + kTileK - 1) / kTileK;
  int sk = sms / tiles;
  if (sk > 8) sk = 8;
  if (sk > k_tiles / 4) sk = k_tiles / 4;
  return sk < 1 ? 1 : sk;
}

struct Layout {
  uint64_t status_off, total;     // the workspace holds the status block only
};
static Layout layout_of(int, int) {
  Layout l;
  l.status_off = 0;
  l.total = 256;
  return l;
}

}  // namespace mkg

extern "C" {

const char* mk_gemm_last_error(void) { return mkg::g_err.c_str(); }

uint64_t mk_gemm_bf16_workspace_bytes(int M, int N, int K) {
  (void)K;
  if (M < 1 || N < 1) return 0;
  return mkg::layout_of(M, N).total;
}

}  // extern "C"

namespace mkg {
static int gemm_launch(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                       void* workspace, uint64_t workspace_bytes, int split_k, int timeout_ms, void* cuda_stream,
                       bool b_packed, int activation) {
  if (!a || !b || !c || !workspace) return fail(-1, "mk_gemm_bf16: null pointer");
  if (activation < 0 || activation > 2) return fail(-2, "mk_gemm_bf16: activation must be 0 (none), 1 (relu) or 2 (silu)");
  if (M < 1 || N < 1 || K < 1) return fail(-2, "mk_gemm_bf16: M, N, K must be positive (got %d, %d, %d)", M, N, K);
  if (K % 8 || lda % 8 || ldb % 8 || ((uint64_t)a & 15) || ((uint64_t)b & 15))
    return fail(-2, "mk_gemm_bf16: K and the row strides of A and B must be multiples of 8 elements, bases 16-byte aligned");
  if (lda < K || ldb < K || ldc < N) return fail(-2, "mk_gemm_bf16: a row stride is shorter than its row");
  if (((uint64_t)workspace & 255) != 0) return fail(-2, "mk_gemm_bf16: workspace must be 256-byte aligned");
  const Layout l = layout_of(M, N);
  if (workspace_bytes < l.total) return fail(-2, "mk_gemm_bf16: workspace of %llu bytes, need %llu",
                                             (unsigned long long)workspace_bytes, (unsigned long long)l.total);
  int dev = 0, sms = 0, smem_optin = 0, cc = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(-1001, "cudaGetDevice failed");
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev);
  if (cc != 10) return fail(-6, "mk_gemm_bf16 needs an sm_100 device (compute capability %d.x found)", cc);
  const int k_tiles = (K + kTileK - 1) / kTileK;
  if (split_k <= 0) split_k = pick_split(M, N, K, sms);
  if (split_k > k_tiles) split_k = k_tiles;
  if (split_k > 8) return fail(-2, "mk_gemm_bf16: split_k is at most 8 (one portable thread-block cluster)");
  const int m_box = ((M < kMaxM ? M : kMaxM) + 15) & ~15;
  CUtensorMap map_a, map_b;
  int rc = encode_bf16_map(&map_a, a, M, K, lda, m_box);
  if (rc) return rc;
  rc = b_packed ? encode_packed_map(&map_b, b, N, k_tiles) : encode_bf16_map(&map_b, b, N, K, ldb, kTileN);
  if (rc) return rc;
  const uint32_t stage_bytes = (kWBytes + (uint32_t)m_box * kTileK * 2 + 1023u) & ~1023u;
  int stages = (smem_optin - 2048) / (int)stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return fail(-4, "mk_gemm_bf16: shared memory holds fewer than two stages");
  const int per = (k_tiles + split_k - 1) / split_k;
  if (stages > per) stages = per < 2 ? 2 : per;
  uint32_t ring_bytes = (uint32_t)stages * stage_bytes;
  if (split_k > 1 && ring_bytes < (uint32_t)m_box * kTileN * 4u) ring_bytes = (uint32_t)m_box * kTileN * 4u;
  const size_t smem = 1024 + (size_t)ring_bytes + sizeof(Shared);
  static bool attr_set[64] = {};
  if (dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin) != cudaSuccess)
      return fail(-4, "mk_gemm_bf16: cannot raise the dynamic shared memory limit");
    attr_set[dev] = true;
  }
  Params p;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  p.c = reinterpret_cast<__nv_bfloat16*>(c);
  p.status = reinterpret_cast<int32_t*>(ws + l.status_off);
  p.ldc = ldc;
  p.M = M, p.N = N, p.K = K;
  p.split_k = split_k, p.k_tiles = k_tiles, p.stages = stages, p.m_box = m_box, p.b_packed = b_packed ? 1 : 0;
  p.ring_bytes = ring_bytes;
  p.activation = activation;
  p.timeout_ns = (uint64_t)(timeout_ms > 0 ? timeout_ms : 1000) * 1000000ull;
  const dim3 grid((N + kTileN - 1) / kTileN, split_k, (M + kMaxM - 1) / kMaxM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)split_k;      // the K splits of one output tile share a cluster
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = split_k > 1 ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel, map_a, map_b, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-(int)e - 1000, "mk_gemm_bf16 launch: %s", cudaGetErrorString(e));
  return 0;
}
}  // namespace mkg

extern "C" {

int mk_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                 void* workspace, uint64_t workspace_bytes, int split_k, int activation, int timeout_ms,
                 void* cuda_stream) {
  return mkg::gemm_launch(a, b, c, M, N, K, lda, ldb, ldc, workspace, workspace_bytes, split_k, timeout_ms, cuda_stream,
                          false, activation);
}

int mk_gemm_bf16_packed(const void* a, const void* b_packed, void* c, int M, int N, int K, int64_t lda, int64_t ldc,
                        void* workspace, uint64_t workspace_bytes, int split_k, int activation, int timeout_ms,
                        void* cuda_stream) {
  if (K % 64) return mkg::fail(-2, "mk_gemm_bf16_packed: K must be a multiple of 64 (the packer pads with zeros)");
  return mkg::gemm_launch(a, b_packed, c, M, N, K, lda, K, ldc, workspace, workspace_bytes, split_k, timeout_ms,
                          cuda_stream, true, activation);
}

int mk_gemm_bf16_status(const void* workspace, int32_t out[4]) {
  using namespace mkg;
  if (!workspace || !out) return fail(-1, "mk_gemm_bf16_status: null pointer");
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(-1001, "mk_gemm_bf16_status: device synchronise failed");
  if (cudaMemcpy(out, workspace, 16, cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(-1001, "mk_gemm_bf16_status: copy failed");
  return 0;
}

}  // extern "C"
