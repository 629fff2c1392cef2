/*
 * machete_b200 — C ABI of the B200 (sm_100a) decode megakernel library.
 *
 * The library is the native replacement for the device side of the
 * reference's `Megakernel` runtime (src/machete/megakernel/megakernel.py:285
 * `class Megakernel`, `.compile()` :1594, `.run()` :2183) and of the CuTe-DSL
 * op bodies it JIT-compiles.  Host code (Python via ctypes, or any C caller)
 * describes a decode step as a *program*: a table of op records, a per-CTA
 * instruction list, dependency-counter wait tables and op-entry events.  One
 * persistent kernel (one CTA per SM) executes the whole program per launch.
 *
 * Ownership: the caller owns every buffer.  `mk_create` copies the program
 * tables into a caller-provided device workspace; no entry point allocates or
 * frees device memory.
 *
 * Error model: every function returns 0 on success, a negative value for a
 * host-side error (bad argument, unsupported shape, CUDA error) with a
 * message available from `mk_last_error()`, and `mk_status` reports
 * device-side conditions (bounded waits that expired) after the caller has
 * synchronised the stream.
 */
#ifndef MACHETE_B200_H_
#define MACHETE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_ABI_VERSION 5

/* ---- opcodes ------------------------------------------------------------ */
enum {
  MK_OP_NOP = 0,
  /* y = epilogue(W · prologue(x)); replaces GemmOp (kernels/gemm/gemm.py:290)
   * at S<=32 rows and the decode matvec family
   * (kernels/decode_matvec/sm100.py:224-654, sm120.py NVFP4 variants). */
  MK_OP_MATVEC = 1,
  /* split-KV decode attention; replaces FlashDecodingSplitBSHDOp
   * (kernels/attention/flash_decoding.py:1175). */
  MK_OP_ATTN_SPLIT = 2,
  /* log-sum-exp combine; replaces FlashDecodingCombineBSHDOp (:1858). */
  MK_OP_ATTN_COMBINE = 3,
  /* RMSNormOp forward (kernels/rms_norm/rms_norm.py:162). */
  MK_OP_RMSNORM = 4,
  /* RopeOp forward (kernels/rope/rope.py:41). */
  MK_OP_ROPE = 5,
  /* QKNormRopeOp forward (kernels/qknorm_rope/qknorm_rope.py:47). */
  MK_OP_QKNORM_ROPE = 6,
  /* GLUOp / DirectGLUOp forward (kernels/glu/glu.py:316, :567). */
  MK_OP_GLU = 7,
  /* AddOp / ResidualAddSm100Op (kernels/activation/add.py:11,
   * kernels/decode_matvec/sm100.py:441). */
  MK_OP_ADD = 8,
  /* top-1 finalise: unpack per-row (max, argmax) keys; replaces
   * Llama1BReduceTop1PartialsSm120Op (kernels/llama1b/sm120.py:3464). */
  MK_OP_TOP1_FINAL = 9,
  /* one-shot all-reduce over peer-mapped inboxes (tensor parallel); replaces
   * GemmRowParallelOp's peer reduce-store and peer barriers
   * (kernels/gemm/gemm.py:1253-1363). */
  MK_OP_ALLREDUCE = 10,
  MK_OP__COUNT
};

/* matvec row-mapping modes (mk_op_t.i[MK_MV_MODE]) */
enum { MK_MV_PLAIN = 0, MK_MV_PAIR = 1, MK_MV_ROPE = 2 };
/* matvec prologues */
enum { MK_PRO_NONE = 0, MK_PRO_RMS = 1, MK_PRO_ADD_RMS = 2 };
/* matvec epilogues */
enum { MK_EPI_STORE = 0, MK_EPI_RESIDUAL = 1, MK_EPI_TOP1 = 2 };
/* matvec transforms applied to the accumulators before the epilogue */
enum { MK_TR_NONE = 0, MK_TR_ROPE = 1, MK_TR_SILU_MUL = 2, MK_TR_RELU = 3, MK_TR_SILU = 4 };
/* weight formats */
enum {
  MK_W_BF16 = 0,
  MK_W_FP16 = 1,
  /* e2m1 pairs per byte (low nibble first) + fp16 scale per 32 values:
   * the reference's format (quantization/nvfp4.py:3-9). */
  MK_W_NVFP4_F16S32 = 2,
  /* e2m1 + e4m3 scale per 16 values + one fp32 global scale. */
  MK_W_NVFP4_E4M3S16 = 3
};
/* element types of activations / outputs */
enum { MK_T_BF16 = 0, MK_T_FP16 = 1, MK_T_FP32 = 2 };

/* Indices into mk_op_t.i / .f / .p / .s for MK_OP_MATVEC. */
enum {
  MK_MV_O = 0, MK_MV_K, MK_MV_M, MK_MV_S, MK_MV_MODE, MK_MV_PRO, MK_MV_EPI,
  MK_MV_TR, MK_MV_HD, MK_MV_D2, MK_MV_POS, MK_MV_WFMT, MK_MV_KC, MK_MV_OUT_T,
  MK_MV_X_T, MK_MV_ROWS_PER_UNIT,
  /* consumer warps that share one unit: its K-slices (pages) are dealt to them
   * round-robin and the partial sums meet in shared memory.
   * 1 suits ops with many units per CTA, more suits ops with few.
   * 0 = one warp per page, up to all consumer warps. */
  MK_MV_SPLIT,
  /* MK_EPI_TOP1: added to the row index packed into the key (the first
   * vocabulary row of this rank's shard under tensor parallelism) */
  MK_MV_IDX0,
  /* The op follows the program's device-resident cache position p
   * (mk_program_t.position), a bit mask: MK_MV_DYN_TABLES = the RoPE tables
   * are read at row (s + p), so cos / sin point at row 0 of the full tables;
   * MK_MV_DYN_OUT = the output row offset becomes (s + POS + p) with POS 0
   * (a cache append: the output is the whole cache).  A projection into a
   * one-token buffer (q) sets the first bit only.  The reference bakes the
   * position into the schedule and re-schedules per token
   * (kernels/decode_matvec/sm100.py:116, 704-709). */
  MK_MV_DYNPOS
};
enum { MK_MV_DYN_TABLES = 1, MK_MV_DYN_OUT = 2 };
/* GSCALE / GSCALE1: fp32 global scale of W0 / of W1 (MK_MV_PAIR; block-scaled NVFP4 only) */
enum { MK_MV_F_EPS = 0, MK_MV_F_GSCALE = 1, MK_MV_F_GSCALE1 = 2 };
enum {
  MK_MV_P_W0 = 0, MK_MV_P_W1, MK_MV_P_X, MK_MV_P_RES_IN, MK_MV_P_NORM_W,
  MK_MV_P_RES_OUT, MK_MV_P_OUT, MK_MV_P_EPI_RES, MK_MV_P_COS, MK_MV_P_SIN,
  MK_MV_P_SC0, MK_MV_P_SC1,
  /* device addresses of the CUtensorMap descriptors of the weights / scales;
   * filled in by mk_create and mk_update_op, callers leave them zero */
  MK_MV_P_TM_W0, MK_MV_P_TM_W1, MK_MV_P_TM_SC0, MK_MV_P_TM_SC1
};
enum {
  MK_MV_S_WROW = 0,   /* weight row stride, bytes                         */
  MK_MV_S_X_B, MK_MV_S_X_S,           /* x strides, elements              */
  MK_MV_S_RI_B, MK_MV_S_RI_S,         /* residual_in (prologue)           */
  MK_MV_S_RO_B, MK_MV_S_RO_S,         /* residual_out (prologue)          */
  MK_MV_S_O_B, MK_MV_S_O_S, MK_MV_S_O_H, /* output (b, s, head) strides   */
  MK_MV_S_ER_B, MK_MV_S_ER_S,         /* epilogue residual                */
  MK_MV_S_COS,                        /* cos/sin row stride               */
  MK_MV_S_SCROW                       /* scale row stride, bytes          */
};

/* MK_OP_ATTN_SPLIT / MK_OP_ATTN_COMBINE */
enum {
  MK_AT_B = 0, MK_AT_M, MK_AT_H, MK_AT_HKV, MK_AT_D, MK_AT_N, MK_AT_SPLITS,
  MK_AT_CAUSAL, MK_AT_MT, MK_AT_TS /* tokens per split */, MK_AT_O_T,
  /* MK_OP_ATTN_SPLIT only: 1 = the unit that completes a (batch, kv head,
   * query tile) group also combines the group's splits into o / lse, so no
   * separate MK_OP_ATTN_COMBINE op (and no dependency stage) is needed */
  MK_AT_FUSE_COMBINE,
  /* MK_OP_ATTN_SPLIT only: 1 = q and the cache row MK_AT_NEW_TOK of k hold
   * UNROTATED projections; the op applies the per-head RMSNorm (weights
   * MK_AT_P_QNW / MK_AT_P_KNW, MK_AT_F_EPS, result rounded to bf16) and the
   * split-half rotation (row tables MK_AT_P_COS / MK_AT_P_SIN of D/2 values)
   * to q as it loads it, and to that k row in shared memory before use, and
   * writes the finished k row back to the cache.  Replaces the separate
   * QKNormRopeOp pass of the reference's Qwen schedule
   * (src/machete/kernels/qwen_3_5/sm120.py:2986-2994; numerics of
   * qknorm_rope/ref.py:10-39).  Needs M = 1 token per sequence, H/Hkv <= 16. */
  MK_AT_QKNORM,
  MK_AT_NEW_TOK,
  /* 1 = the KV window follows the device-resident cache position p: the op
   * attends to tokens [0, p + M); MK_AT_N is then the cache CAPACITY (tensor
   * maps, split bounds and the per-unit page limits derive from it; loader
   * and consumers compute the pages in use from p), and the new-token row of
   * the fused q/k norm is p: MK_AT_P_COS / MK_AT_P_SIN then point at the whole
   * tables and MK_AT_NEW_TOK holds their row stride in elements (row p is
   * used). */
  MK_AT_DYNPOS,
  /* query heads per KV head (H / Hkv): filled in by mk_create / mk_update_op, whatever the caller
   * leaves here, so that the kernel does not divide */
  MK_AT_GROUP
};
enum { MK_AT_F_SCALE = 0, MK_AT_F_EPS };
enum {
  MK_AT_P_Q = 0, MK_AT_P_K, MK_AT_P_V, MK_AT_P_OPART, MK_AT_P_LSEPART, MK_AT_P_O, MK_AT_P_LSE,
  /* fused combine: int32[B * Hkv * MT] arrival counters, zero before the first launch (the kernel leaves them zero) */
  MK_AT_P_ARRIVE,
  MK_AT_P_QNW, MK_AT_P_KNW, MK_AT_P_COS, MK_AT_P_SIN   /* MK_AT_QKNORM: bf16, 16-byte aligned */
};
enum {
  MK_AT_S_Q_B = 0, MK_AT_S_Q_M, MK_AT_S_Q_H,
  MK_AT_S_K_B, MK_AT_S_K_N, MK_AT_S_K_H,
  MK_AT_S_V_B, MK_AT_S_V_N, MK_AT_S_V_H,
  MK_AT_S_O_B, MK_AT_S_O_M, MK_AT_S_O_H
};

/* elementwise ops (RMSNORM, ROPE, QKNORM_ROPE, GLU, ADD): generic slots */
enum {
  MK_EW_ROWS = 0, MK_EW_D, MK_EW_S, MK_EW_H, MK_EW_D2, MK_EW_FLAGS, MK_EW_ACT,
  MK_EW_T, MK_EW_ROWS_PER_UNIT
};
enum { MK_EW_F_EPS = 0 };
enum { MK_EW_P_X = 0, MK_EW_P_Y, MK_EW_P_W, MK_EW_P_RES_IN, MK_EW_P_RES_OUT, MK_EW_P_GATE, MK_EW_P_COS, MK_EW_P_SIN };
enum { MK_EW_S_X = 0, MK_EW_S_Y, MK_EW_S_W, MK_EW_S_RI, MK_EW_S_RO, MK_EW_S_G, MK_EW_S_COS, MK_EW_S_X_H };
/* MK_EW_FLAGS bits */
enum { MK_EWF_RESIDUAL = 1, MK_EWF_GEMMA = 2, MK_EWF_FUSED_ADD = 4, MK_EWF_GATED = 8, MK_EWF_ROW_WEIGHT = 16,
       /* MK_OP_TOP1_FINAL: feed the greedy token back for the next launch — copy row
        * `token` of the embedding table p[MK_EW_P_RES_IN] (row stride s[MK_EW_S_RI],
        * MK_EW_D 16-bit values) into row m of p[MK_EW_P_RES_OUT] (row stride
        * s[MK_EW_S_RO]) and add MK_EW_S to the position scalar p[MK_EW_P_GATE] */
       MK_EWF_FEEDBACK = 32 };

/* MK_OP_ALLREDUCE: one-shot all-reduce over peer-mapped inboxes.  Every rank
 * runs the same op with its own MK_AR_RANK; p[MK_AR_P_PEER0 + r] is rank r's
 * symmetric buffer as mapped into this process (r = own rank included), and
 * s[] holds the byte offsets of the op's inbox and flag regions inside it. */
enum { MK_AR_N = 0 /* elements (sum) or rows (keys) */, MK_AR_P, MK_AR_RANK, MK_AR_MODE, MK_AR_X_T, MK_AR_Y_T,
       MK_AR_R_T, MK_AR_EPOCH_BASE };
enum { MK_AR_SUM = 0 /* y = sum_r x_r (+ residual) */, MK_AR_MAX_KEY = 1 /* y = max_r of 64-bit top-1 keys */ };
enum { MK_AR_P_X = 0, MK_AR_P_RES, MK_AR_P_Y, MK_AR_P_PEER0 /* .. MK_AR_P_PEER0 + 7 */ };
enum { MK_AR_S_INBOX = 0, MK_AR_S_FLAGS };
#define MK_AR_MAX_RANKS 8

/* A device-visible op record.  Field meaning depends on `opcode`; see the
 * index enums above.  The layout is fixed: 16 + 96 + 16 + 128 + 128 bytes. */
typedef struct mk_op {
  int32_t opcode;
  int32_t n_units;        /* work units                                      */
  int32_t act_key;        /* ops with equal non-zero key share staged input  */
  int32_t reserved;
  int32_t i[24];
  float f[4];
  uint64_t p[16];
  int64_t s[16];
} mk_op_t;

/* One work unit assigned to one CTA (executed by one consumer warp, or shared
 * page by page by several: see MK_LDF_SPLIT_SHIFT). */
typedef struct mk_instr {
  int32_t op;             /* index into the op table                         */
  int32_t unit;           /* unit index within the op                        */
  int32_t signal;         /* counter incremented on completion, -1 = none    */
  int32_t n_waits;        /* consumer-side waits (pairs in the wait table)   */
  int32_t wait_off;
  int32_t n_lwaits;       /* loader-side waits (before the unit's loads)     */
  int32_t lwait_off;
  int32_t n_pages;        /* ring pages the unit consumes                    */
  /* Fast path, filled in by mk_create (callers leave these zero): all the
   * loader warp needs to issue the unit's pages, and the row / output
   * offsets the finishing consumer needs, so that neither reads the op table
   * or divides on its critical path. */
  uint64_t ld_maps;       /* device address of the op's 4 tensor maps        */
  int32_t ld_tiles;       /* 128-byte K-tiles per page                       */
  int32_t ld_flags;       /* MK_LDF_*                                        */
  int32_t ld_row_a;       /* first weight row of virtual rows 0-7            */
  int32_t ld_row_b;       /* first weight row of virtual rows 8-15           */
  /* matvec: element offset of rows a / b inside one activation row's output
   * (head * head stride + dim); attention: split index / query tile */
  int32_t out_off_a;
  int32_t out_off_b;
} mk_instr_t;

/* bits 8-11 of ld_flags: consumer warps sharing the unit (from MK_MV_SPLIT);
 * bits 12-23: matvec RoPE units, index of the unit's 8-value chunk inside
 * the rotary half (dim = 8 * chunk + row). */
/* MK_LDF_ATTN marks a split-KV attention unit: ld_maps holds the K and V cache
 * maps, ld_row_a the first token, ld_row_b = kv head | batch << 16, ld_tiles
 * the tokens per page; MK_LDF_D128 = head dim 128 (two 64-wide sub-tiles). */
enum { MK_LDF_FP4 = 1, MK_LDF_PAIR = 2, MK_LDF_ATTN = 4, MK_LDF_D128 = 8,
       /* attention unit of an MK_AT_DYNPOS op: n_pages is the limit, the pages in use follow the position */
       MK_LDF_DYN = 16,
       MK_LDF_SPLIT_SHIFT = 8, MK_LDF_SPLIT_MASK = 15, MK_LDF_CHUNK_SHIFT = 12, MK_LDF_CHUNK_MASK = 4095 };

/* Op-entry event: before a CTA executes instruction `pos` of its list, all
 * of its consumer warps meet, wait for the listed counters and stage the
 * op's activations into shared memory. */
typedef struct mk_event {
  int32_t pos;
  int32_t op;
  int32_t n_waits;
  int32_t wait_off;
  int32_t flags;          /* MK_EVF_* */
  int32_t bulk_units;     /* with MK_EVF_BULK_SIGNAL: units of `op` on this CTA */
  /* filled in by mk_create (callers leave them zero): the first four
   * (counter, expected) pairs of the wait list, so that the poll that opens a
   * dependency stage starts without a table read */
  int32_t w_counter[4];
  int32_t w_expected[4];
  int32_t reserved[2];
} mk_event_t;

/* mk_event_t.flags
 * WRITE_RES_OUT: this CTA materialises residual_out = x + residual_in of the
 *   op's prologue in global memory (exactly one CTA per op does).
 * BULK_SIGNAL: the op's units on this CTA all signal the same counter; the CTA
 *   adds `bulk_units` to it once, after its last unit, instead of one
 *   device-scope release per unit. */
enum { MK_EVF_WRITE_RES_OUT = 1, MK_EVF_BULK_SIGNAL = 2 };

typedef struct mk_wait {
  int32_t counter;
  int32_t expected;       /* wait until counter >= expected                  */
} mk_wait_t;

/* Host-side program description handed to mk_create (all arrays in HOST
 * memory; mk_create copies them into the device workspace). */
typedef struct mk_program {
  int32_t n_ops;
  int32_t n_instrs;
  int32_t n_events;
  int32_t n_waits;
  int32_t n_counters;
  int32_t n_ctas;           /* persistent grid size                          */
  int32_t page_bytes;       /* shared-memory page stride                     */
  int32_t n_pages;          /* ring depth                                    */
  int32_t act_bytes;        /* staged-activation buffer size                 */
  int32_t timeout_ms;       /* bound of every device-side wait               */
  int32_t device;           /* CUDA device ordinal                           */
  int32_t flags;
  const mk_op_t* ops;
  const mk_instr_t* instrs;       /* grouped per CTA                         */
  const int32_t* cta_instr_begin; /* n_ctas + 1 offsets into instrs          */
  const mk_event_t* events;       /* grouped per CTA                         */
  const int32_t* cta_event_begin; /* n_ctas + 1 offsets into events          */
  const mk_wait_t* waits;
  void* workspace;                /* DEVICE memory, >= mk_workspace_bytes()  */
  uint64_t workspace_bytes;
  /* Optional device-resident cache position (one int32 in DEVICE memory, NULL =
   * none): ops scheduled with MK_MV_DYNPOS / MK_AT_DYNPOS read it at the start
   * of every launch, the feedback form of MK_OP_TOP1_FINAL advances it at the
   * end, so consecutive launches (or replays of one CUDA graph) decode
   * consecutive tokens with no host work in between. */
  const int32_t* position;
  /* With `position`: the first position the program's caches and tables do NOT
   * hold (the smallest cache length of its position-following ops).  A launch
   * that finds the position outside [0, position_limit) runs no op and ends
   * with device status 7; mk_create refuses a program with `position` set and
   * a limit < 1. */
  int32_t position_limit;
  /* Entries behind `position`: 0 or 1 = one position shared by every batch row,
   * else one int32 per batch row (<= 32): sequences of different lengths decode
   * side by side, each row reads and appends at its own position and attends to
   * its own window, and the feedback op advances every entry. */
  int32_t position_count;
} mk_program_t;

typedef struct mk_handle_s* mk_handle_t;

/* ABI version of the loaded library (MK_ABI_VERSION). */
int mk_abi_version(void);
/* Thread-local message describing the last host-side error. */
const char* mk_last_error(void);
/* Multiprocessor count and opt-in shared memory per block of `device`;
 * replaces the torch.cuda.get_device_properties queries in
 * megakernel/megakernel.py:523-569. */
int mk_device_info(int device, int32_t* num_sms, int32_t* smem_optin, int32_t* cc_major, int32_t* cc_minor);
/* Device workspace needed for `prog` (tables + counters + status block). */
uint64_t mk_workspace_bytes(const mk_program_t* prog);
/* Validate `prog`, upload its tables into prog->workspace, return a handle.
 * Replaces Megakernel.compile()'s metadata upload
 * (megakernel/megakernel.py:709-962); there is no JIT. */
int mk_create(const mk_program_t* prog, mk_handle_t* out);
/* Launch the persistent kernel on `cuda_stream` (a cudaStream_t; NULL = the
 * legacy default stream).  Asynchronous.  Counters are reset by the kernel
 * itself, so back-to-back launches and CUDA-graph replay are legal.
 * Replaces Megakernel.run() / launch_prepared (megakernel.py:2163-2204). */
int mk_run(mk_handle_t h, void* cuda_stream);
/* Copy the 16-word device status block to `out` (synchronises the device).
 * out[0] == 0 means no device-side error. */
int mk_status(mk_handle_t h, int32_t out[16]);
/* The same status block read straight from a workspace (it sits at offset
 * 0): for the standalone entry points, which hand out no handle. */
int mk_workspace_status(const void* workspace, int32_t out[16]);
/* Attach (or, with buffer == NULL, detach) a device buffer that the kernel
 * fills with 16-byte {globaltimer ns, code, arg} records, `records_per_warp`
 * per warp of every CTA (9 warps: loader first), followed by one int32 record
 * count per warp.  Needs n_ctas * 9 * (records_per_warp * 16 + 4) bytes.
 * Takes the place of the reference's cutedsl-trace lanes
 * (megakernel/tracing.py:51-153). */
int mk_set_trace(mk_handle_t h, void* buffer, uint64_t bytes, int32_t records_per_warp);
/* Clear status, abort flag and dependency counters after a device-side
 * error (Megakernel.wait() does this before it raises).  The launch count is
 * kept: the tensor-parallel exchange tags its messages with it.  Takes the
 * place of the per-run barriers.zero_() of the reference
 * (megakernel/megakernel.py:2149-2150). */
int mk_reset(mk_handle_t h, void* cuda_stream);
/* The number of launches this handle's workspace has completed, aborted ones
 * included (every CTA of an aborted launch still exits through the kernel's
 * end).  The in-kernel all-reduce of launch n uses message epoch
 * epoch_base + n + 1 on every rank, so ranks must agree on it: after one rank
 * missed or repeated a launch (a peer timeout, a restart) the group sets every
 * rank's count to the group maximum before launching again.  No counterpart in
 * the reference, which runs all ranks from one process
 * (megakernel/runtime_components.py:272-287). */
int mk_launch_count(mk_handle_t h, int32_t* out);
int mk_set_launch_count(mk_handle_t h, int32_t count, void* cuda_stream);
/* Replace op record `op_index` (new pointers, a new cache position, a longer
 * KV window).  The record is validated like mk_create does, the opcode and
 * unit count must stay, the op's tensor maps are re-encoded and the
 * instruction rows derived from the record (pages per unit, loader and
 * finisher fast path) are recomputed and uploaded.  Synchronises
 * `cuda_stream`.  The reference re-schedules and recompiles for a new
 * position (kernels/decode_matvec/sm100.py:116, 704-709). */
int mk_update_op(mk_handle_t h, int32_t op_index, const mk_op_t* op, void* cuda_stream);
/* Read back the dependency counters (n_counters words) — after a completed
 * run they are all zero; used by the tests' invariant checks. */
int mk_read_counters(mk_handle_t h, int32_t* out, int32_t n);
int mk_destroy(mk_handle_t h);

/* ---- standalone single-op entry points ----------------------------------
 * Each builds a one-op program in `workspace` (device memory, at least
 * mk_standalone_workspace_bytes() bytes) and launches it on `cuda_stream`.
 * They exist for profiling and for C callers that do not need a schedule. */
uint64_t mk_standalone_workspace_bytes(void);

/* y[M,O] = x[M,K] · W[O,K]^T, bf16 in/out, fp32 accumulate, M <= 32.
 * Replaces MatvecSm100Op (kernels/decode_matvec/sm100.py:386) and GemmOp at
 * decode sizes (kernels/gemm/gemm.py:290). */
int mk_matvec_bf16(const void* w, const void* x, void* y, int32_t M, int32_t O, int32_t K,
                   void* workspace, uint64_t workspace_bytes, void* cuda_stream);
/* Same with NVFP4 weights: `packed` [O,K/2] bytes, `scales` [O,K/group],
 * wfmt = MK_W_NVFP4_F16S32 or MK_W_NVFP4_E4M3S16.  Replaces
 * MatvecNvfp4Sm120Op (kernels/decode_matvec/sm120.py:1058). */
int mk_matvec_nvfp4(const void* packed, const void* scales, float global_scale, int32_t wfmt,
                    const void* x, void* y, int32_t M, int32_t O, int32_t K,
                    void* workspace, uint64_t workspace_bytes, void* cuda_stream);
/* Split-KV flash decoding + combine on contiguous BSHD tensors
 * q,o [B,M,H,D], k,v [B,N,Hkv,D] bf16; o_partial [B,H,splits,M,D] and
 * lse_partial [B,H,splits,M] fp32 scratch, lse [B,H,M] fp32.  Replaces
 * flash_decoding_schedule + run (kernels/attention/flash_decoding.py:1958). */
int mk_flash_decode(const void* q, const void* k, const void* v, void* o, void* lse,
                    void* o_partial, void* lse_partial,
                    int32_t B, int32_t M, int32_t H, int32_t Hkv, int32_t D, int32_t N,
                    int32_t splits, int32_t causal, float scale,
                    void* workspace, uint64_t workspace_bytes, void* cuda_stream);

/* The same computation for callers that cannot hand over scratch memory (a
 * plugin slot or custom-op hook that receives only its tensors, a loop that
 * must not touch the allocator).  No counterpart in the reference, whose
 * schedule() allocates the partials with torch.  The attention partials and
 * the program tables live in one fixed array inside the library's device
 * image (4 MiB + 1 MiB per device), so the call allocates nothing.
 *   - The first call on a device looks the array's address up (and may make
 *     the runtime load the module): make it before any stream capture.
 *   - Limits: B*H*splits*M partial rows must fit 4 MiB ((D+1)*4 bytes each,
 *     rounded to 256), and the work units (B*Hkv*ceil(M*H/Hkv/16)*splits +
 *     B*H) must fit the 1 MiB of tables; larger shapes are refused with a
 *     message, use mk_flash_decode for them.
 *   - The array is shared by all calls on a device and keeps its last
 *     contents; the call clears the part that must start at zero itself.
 *     Calls that overlap in time on one device race: serialise them.  Every
 *     clear and upload of a call is queued on `cuda_stream` ahead of its
 *     launch, so calls issued one after another on one stream need nothing
 *     more; calls on different streams need an event or a host
 *     synchronisation between them. */
int mk_flash_decode_noalloc(const void* q, const void* k, const void* v, void* o, void* lse,
                            int32_t B, int32_t M, int32_t H, int32_t Hkv, int32_t D, int32_t N,
                            int32_t splits, int32_t causal, float scale, void* cuda_stream);

/* Device status block of the last mk_flash_decode_noalloc call on the current
 * device (out[0] == 0: no bounded wait expired).  Synchronises the device.
 * No counterpart in the reference. */
int mk_flash_decode_noalloc_status(int32_t out[16]);

/* ---- small-M GEMM on tcgen05 tensor cores ------------------------------------
 * C[M,N] = A[M,K] x B[N,K]^T, bf16 operands (row strides lda / ldb / ldc in
 * elements, K contiguous), fp32 accumulation in tensor memory, bf16 output.
 * Replaces the reference's GemmSm100Op for the rows-per-launch range the decode
 * matvec ops do not cover (src/machete/kernels/gemm/gemm_sm100.py:56-658: a
 * (B,S,K), b (N,K), c (B,S,N); here B*S = M is flattened by the caller).  The
 * weight rows are the 128-row operand of tcgen05.mma and up to 256 activation
 * rows its N operand; more rows run as further CTAs along M.
 *   K, lda, ldb multiples of 8; a and b 16-byte aligned.
 *   workspace: mk_gemm_bf16_workspace_bytes(M, N, K) bytes of device memory
 *     (the device status block), 256-byte aligned, ZERO before its first use;
 *     it stays zero unless a wait ran out.
 *   split_k: CTAs that share one output tile's K range, at most 8 (0 = chosen
 *     so that the grid fills the device).  They form one thread-block cluster
 *     and add their fp32 partial tiles through distributed shared memory.
 *   activation: applied to the fp32 sum before the bf16 store, 0 = none, 1 = relu,
 *     2 = silu (the reference op's `activation=` keyword).
 *     timeout_ms bounds every device-side wait (0 = 1000).
 * Returns 0 or a negative code (mk_gemm_last_error); a device-side time-out
 * shows in mk_gemm_bf16_status (out[0] != 0: 1 stage-free, 2 stage-full,
 * 3 accumulator wait; [1] CTA, [2] role, [3] step), which synchronises. */
uint64_t mk_gemm_bf16_workspace_bytes(int M, int N, int K);
int mk_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                 void* workspace, uint64_t workspace_bytes, int split_k, int activation, int timeout_ms,
                 void* cuda_stream);
/* The same product with the weight stored K-tile-major: b_packed[K/64][N][64]
 * (tile kt holds columns kt*64 .. kt*64+63 of every row; K a multiple of 64,
 * zero-padded by the packer).  One 128-row x 64-column box is then ONE
 * contiguous 16 KB piece of memory instead of 128 pieces of 128 bytes one row
 * stride apart, which is what the copy engine streams fastest.  An offline
 * re-layout of inference weights, like the reference's per-KV-head interleaved
 * QKV weight (src/machete/kernels/llama1b/sm120.py:4330-4345). */
int mk_gemm_bf16_packed(const void* a, const void* b_packed, void* c, int M, int N, int K, int64_t lda, int64_t ldc,
                        void* workspace, uint64_t workspace_bytes, int split_k, int activation, int timeout_ms,
                        void* cuda_stream);
int mk_gemm_bf16_status(const void* workspace, int32_t out[4]);
const char* mk_gemm_last_error(void);

/* ---- prefill attention on tcgen05 tensor cores -----------------------------------
 * O = softmax(scale * Q K^T) V for M query rows per head against N cached tokens,
 * bf16, fp32 softmax and accumulation in tensor memory; grouped-query heads
 * (head h reads KV head h / (H / Hkv)); causal = the queries are the LAST M of
 * the N tokens (row m sees tokens 0 .. N - M + m).  Replaces the reference's
 * FlashAttentionSm100Op (src/machete/kernels/attention/sm_100.py:88,
 * attention/__init__.py:16-130) as a launch of its own: it lets a prompt fill
 * the KV cache that the decode kernel then reads.
 *   q [B][H][M][D], k / v [B][Hkv][N][D], o [B][H][M][D], each with element
 *   strides {batch, head, row} (so both the reference's (B,H,M,D) tensors and
 *   (B,N,Hkv,D) cache views fit), D = 64 or 128 contiguous, every stride a
 *   multiple of 8 elements, bases 16-byte aligned.  lse: [B][H][M] fp32 or NULL.
 *   workspace: 256 bytes of device memory, 256-byte aligned, ZERO before first
 *   use (the device status block; it stays zero unless a wait ran out).
 * Returns 0 or a negative code (mk_flash_prefill_last_error); a device-side
 * time-out shows in mk_flash_prefill_status (out[0] != 0), which synchronises. */
int mk_flash_prefill_bf16(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Hkv, int M,
                          int N, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                          const int64_t v_strides[3], const int64_t o_strides[3], float scale, int causal,
                          void* workspace, uint64_t workspace_bytes, int timeout_ms, void* cuda_stream);
int mk_flash_prefill_status(const void* workspace, int32_t out[4]);
const char* mk_flash_prefill_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MACHETE_B200_H_ */
