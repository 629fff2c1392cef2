"""ctypes binding of ``libmachete_b200.so`` (declared in ``include/machete_b200.h``).

There is no fallback: if the library cannot be loaded (or built with ``nvcc``
when it is missing), importing :func:`lib` raises ``RuntimeError``.  The
structures below mirror the C header field by field.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

import numpy as np

from . import build as _build

ABI_VERSION = 5
NUM_CONSUMER_WARPS = 7   # csrc/shell.cuh kConsumerWarps

# ---- enums (keep in sync with include/machete_b200.h) ------------------------
OP_NOP, OP_MATVEC, OP_ATTN_SPLIT, OP_ATTN_COMBINE, OP_RMSNORM, OP_ROPE, OP_QKNORM_ROPE, OP_GLU, OP_ADD, \
    OP_TOP1_FINAL, OP_ALLREDUCE = range(11)
MV_PLAIN, MV_PAIR, MV_ROPE = range(3)
PRO_NONE, PRO_RMS, PRO_ADD_RMS = range(3)
EPI_STORE, EPI_RESIDUAL, EPI_TOP1 = range(3)
TR_NONE, TR_ROPE, TR_SILU_MUL, TR_RELU, TR_SILU = range(5)
W_BF16, W_FP16, W_NVFP4_F16S32, W_NVFP4_E4M3S16 = range(4)
T_BF16, T_FP16, T_FP32 = range(3)

(MV_O, MV_K, MV_M, MV_S, MV_MODE, MV_PRO, MV_EPI, MV_TR, MV_HD, MV_D2, MV_POS, MV_WFMT, MV_KC, MV_OUT_T,
 MV_X_T, MV_ROWS_PER_UNIT, MV_SPLIT, MV_IDX0, MV_DYNPOS) = range(19)
MV_DYN_TABLES, MV_DYN_OUT = 1, 2
MV_F_EPS, MV_F_GSCALE, MV_F_GSCALE1 = range(3)
(MV_P_W0, MV_P_W1, MV_P_X, MV_P_RES_IN, MV_P_NORM_W, MV_P_RES_OUT, MV_P_OUT, MV_P_EPI_RES, MV_P_COS,
 MV_P_SIN, MV_P_SC0, MV_P_SC1) = range(12)
(MV_S_WROW, MV_S_X_B, MV_S_X_S, MV_S_RI_B, MV_S_RI_S, MV_S_RO_B, MV_S_RO_S, MV_S_O_B, MV_S_O_S, MV_S_O_H,
 MV_S_ER_B, MV_S_ER_S, MV_S_COS, MV_S_SCROW) = range(14)

(AT_B, AT_M, AT_H, AT_HKV, AT_D, AT_N, AT_SPLITS, AT_CAUSAL, AT_MT, AT_TS, AT_O_T, AT_FUSE_COMBINE, AT_QKNORM,
 AT_NEW_TOK, AT_DYNPOS, AT_GROUP) = range(16)      # AT_GROUP (H / Hkv) is filled in by the library
AT_F_SCALE, AT_F_EPS = 0, 1
(AT_P_Q, AT_P_K, AT_P_V, AT_P_OPART, AT_P_LSEPART, AT_P_O, AT_P_LSE, AT_P_ARRIVE, AT_P_QNW, AT_P_KNW, AT_P_COS,
 AT_P_SIN) = range(12)
(AT_S_Q_B, AT_S_Q_M, AT_S_Q_H, AT_S_K_B, AT_S_K_N, AT_S_K_H, AT_S_V_B, AT_S_V_N, AT_S_V_H, AT_S_O_B,
 AT_S_O_M, AT_S_O_H) = range(12)

(EW_ROWS, EW_D, EW_S, EW_H, EW_D2, EW_FLAGS, EW_ACT, EW_T, EW_ROWS_PER_UNIT) = range(9)
EW_F_EPS = 0
(EW_P_X, EW_P_Y, EW_P_W, EW_P_RES_IN, EW_P_RES_OUT, EW_P_GATE, EW_P_COS, EW_P_SIN) = range(8)
(EW_S_X, EW_S_Y, EW_S_W, EW_S_RI, EW_S_RO, EW_S_G, EW_S_COS, EW_S_X_H) = range(8)
(AR_N, AR_P, AR_RANK, AR_MODE, AR_X_T, AR_Y_T, AR_R_T, AR_EPOCH_BASE) = range(8)
AR_SUM, AR_MAX_KEY = 0, 1
(AR_P_X, AR_P_RES, AR_P_Y, AR_P_PEER0) = range(4)
AR_S_INBOX, AR_S_FLAGS = 0, 1
AR_MAX_RANKS = 8
EWF_RESIDUAL, EWF_GEMMA, EWF_FUSED_ADD, EWF_GATED, EWF_ROW_WEIGHT, EWF_FEEDBACK = 1, 2, 4, 8, 16, 32
EVF_WRITE_RES_OUT, EVF_BULK_SIGNAL = 1, 2

# Device status codes (csrc/shell.cuh).
STATUS_NAMES = {
    0: "ok",
    1: "dependency counter wait timed out",
    2: "page-full wait timed out",
    3: "page-empty wait timed out",
    4: "unknown opcode",
    5: "ring-slot turn wait timed out",
    6: "a peer rank's all-reduce flag never arrived",
    7: "the device-resident cache position is outside the caches (nothing ran)",
}


def workspace_status(workspace_ptr: int):
    """Status block of a standalone call's workspace (synchronises the device)."""
    out = (C.c_int32 * 16)()
    check(lib().mk_workspace_status(C.c_void_p(workspace_ptr), out), "mk_workspace_status")
    return list(out)

# numpy record layouts of the C structs
OP_DTYPE = np.dtype([
    ("opcode", "<i4"), ("n_units", "<i4"), ("act_key", "<i4"), ("reserved", "<i4"),
    ("i", "<i4", (24,)), ("f", "<f4", (4,)), ("p", "<u8", (16,)), ("s", "<i8", (16,)),
], align=False)
INSTR_DTYPE = np.dtype([
    ("op", "<i4"), ("unit", "<i4"), ("signal", "<i4"), ("n_waits", "<i4"), ("wait_off", "<i4"),
    ("n_lwaits", "<i4"), ("lwait_off", "<i4"), ("n_pages", "<i4"),
    # loader fast path: left zero here, filled in by mk_create
    ("ld_maps", "<u8"), ("ld_tiles", "<i4"), ("ld_flags", "<i4"), ("ld_row_a", "<i4"), ("ld_row_b", "<i4"),
    ("out_off_a", "<i4"), ("out_off_b", "<i4"),
])
EVENT_DTYPE = np.dtype([
    ("pos", "<i4"), ("op", "<i4"), ("n_waits", "<i4"), ("wait_off", "<i4"), ("flags", "<i4"),
    ("bulk_units", "<i4"),
    # inline copy of the first wait pairs: left zero here, filled in by mk_create
    ("w_counter", "<i4", (4,)), ("w_expected", "<i4", (4,)), ("reserved", "<i4", (2,)),
])
WAIT_DTYPE = np.dtype([("counter", "<i4"), ("expected", "<i4")])
assert OP_DTYPE.itemsize == 16 + 96 + 16 + 128 + 128
assert INSTR_DTYPE.itemsize == 64 and EVENT_DTYPE.itemsize == 64 and WAIT_DTYPE.itemsize == 8


class Program(C.Structure):
    _fields_ = [
        ("n_ops", C.c_int32), ("n_instrs", C.c_int32), ("n_events", C.c_int32), ("n_waits", C.c_int32),
        ("n_counters", C.c_int32), ("n_ctas", C.c_int32), ("page_bytes", C.c_int32), ("n_pages", C.c_int32),
        ("act_bytes", C.c_int32), ("timeout_ms", C.c_int32), ("device", C.c_int32), ("flags", C.c_int32),
        ("ops", C.c_void_p), ("instrs", C.c_void_p), ("cta_instr_begin", C.c_void_p),
        ("events", C.c_void_p), ("cta_event_begin", C.c_void_p), ("waits", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64), ("position", C.c_void_p), ("position_limit", C.c_int32), ("position_count", C.c_int32),
    ]


EXPORTS = [
    "mk_abi_version", "mk_last_error", "mk_device_info", "mk_workspace_bytes", "mk_create", "mk_run",
    "mk_status", "mk_workspace_status", "mk_set_trace", "mk_reset", "mk_launch_count", "mk_set_launch_count",
    "mk_update_op", "mk_read_counters", "mk_destroy",
    "mk_standalone_workspace_bytes", "mk_matvec_bf16", "mk_matvec_nvfp4", "mk_flash_decode",
    "mk_flash_decode_noalloc", "mk_flash_decode_noalloc_status",
    "mk_gemm_bf16_workspace_bytes", "mk_gemm_bf16", "mk_gemm_bf16_packed", "mk_gemm_bf16_status", "mk_gemm_last_error",
    "mk_flash_prefill_bf16", "mk_flash_prefill_status", "mk_flash_prefill_last_error",
]

_lib = None
_lock = threading.Lock()


def lib_path() -> Path:
    """The library file; ``MACHETE_B200_LIB`` names another build of it (same ABI)."""
    import os

    override = os.environ.get("MACHETE_B200_LIB")
    return Path(override) if override else _build.LIB_PATH


def lib() -> C.CDLL:
    """Load (building first if the file is missing) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            try:
                _build.build()
            except Exception as exc:  # noqa: BLE001
                raise RuntimeError(
                    f"machete_b200: native library {path} is missing and could not be built: {exc}"
                ) from exc
        try:
            handle = C.CDLL(str(path))
        except OSError as exc:
            raise RuntimeError(f"machete_b200: cannot load {path}: {exc}") from exc
        _declare(handle)
        if handle.mk_abi_version() != ABI_VERSION:
            raise RuntimeError(
                f"machete_b200: {path} has ABI {handle.mk_abi_version()}, Python side expects {ABI_VERSION}; rebuild"
            )
        _lib = handle
        return _lib


def _declare(h: C.CDLL) -> None:
    vp, i32, u64, f32 = C.c_void_p, C.c_int32, C.c_uint64, C.c_float
    h.mk_abi_version.restype = C.c_int
    h.mk_last_error.restype = C.c_char_p
    h.mk_device_info.argtypes = [C.c_int, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]
    h.mk_workspace_bytes.argtypes = [C.POINTER(Program)]
    h.mk_workspace_bytes.restype = u64
    h.mk_create.argtypes = [C.POINTER(Program), C.POINTER(vp)]
    h.mk_run.argtypes = [vp, vp]
    h.mk_status.argtypes = [vp, C.POINTER(i32)]
    h.mk_workspace_status.argtypes = [vp, C.POINTER(i32)]
    h.mk_set_trace.argtypes = [vp, vp, u64, i32]
    h.mk_set_trace.restype = C.c_int
    h.mk_reset.argtypes = [vp, vp]
    h.mk_launch_count.argtypes = [vp, C.POINTER(i32)]
    h.mk_set_launch_count.argtypes = [vp, i32, vp]
    h.mk_update_op.argtypes = [vp, i32, vp, vp]
    h.mk_read_counters.argtypes = [vp, C.POINTER(i32), i32]
    h.mk_destroy.argtypes = [vp]
    h.mk_standalone_workspace_bytes.restype = u64
    h.mk_matvec_bf16.argtypes = [vp, vp, vp, i32, i32, i32, vp, u64, vp]
    h.mk_matvec_nvfp4.argtypes = [vp, vp, f32, i32, vp, vp, i32, i32, i32, vp, u64, vp]
    h.mk_flash_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32,
                                  vp, u64, vp]
    h.mk_flash_decode_noalloc.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp]
    h.mk_flash_decode_noalloc.restype = C.c_int
    h.mk_flash_decode_noalloc_status.argtypes = [C.POINTER(i32)]
    h.mk_flash_decode_noalloc_status.restype = C.c_int
    i64 = C.c_int64
    h.mk_gemm_bf16_workspace_bytes.argtypes = [i32, i32, i32]
    h.mk_gemm_bf16_workspace_bytes.restype = u64
    h.mk_gemm_bf16.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, vp, u64, i32, i32, i32, vp]
    h.mk_gemm_bf16.restype = C.c_int
    h.mk_gemm_bf16_packed.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, vp, u64, i32, i32, i32, vp]
    h.mk_gemm_bf16_packed.restype = C.c_int
    h.mk_gemm_bf16_status.argtypes = [vp, C.POINTER(i32)]
    h.mk_gemm_bf16_status.restype = C.c_int
    h.mk_gemm_last_error.restype = C.c_char_p
    p64 = C.POINTER(C.c_int64)
    h.mk_flash_prefill_bf16.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, p64, p64, p64, p64, f32, i32,
                                        vp, u64, i32, vp]
    h.mk_flash_prefill_bf16.restype = C.c_int
    h.mk_flash_prefill_status.argtypes = [vp, C.POINTER(i32)]
    h.mk_flash_prefill_status.restype = C.c_int
    h.mk_flash_prefill_last_error.restype = C.c_char_p
    for name in ("mk_device_info", "mk_create", "mk_run", "mk_status", "mk_workspace_status", "mk_reset", "mk_update_op",
                 "mk_launch_count", "mk_set_launch_count",
                 "mk_read_counters", "mk_destroy", "mk_matvec_bf16", "mk_matvec_nvfp4", "mk_flash_decode"):
        getattr(h, name).restype = C.c_int


def last_error() -> str:
    return lib().mk_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Raise the reference's error types for a failed native call."""
    if rc == 0:
        return
    msg = f"{what}: {last_error()} (code {rc})"
    if rc in (-2, -3):
        raise ValueError(msg)
    raise RuntimeError(msg)


def device_info(device: int = 0) -> dict:
    sms, smem, major, minor = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
    check(lib().mk_device_info(device, C.byref(sms), C.byref(smem), C.byref(major), C.byref(minor)),
          "mk_device_info")
    return {"num_sms": sms.value, "smem_optin": smem.value, "cc": (major.value, minor.value)}
