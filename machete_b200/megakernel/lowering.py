"""Lowering targets: what an ``Op.lower()`` hands to the program builder.

A :class:`NativeOp` is one record of the device op table (``mk_op_t`` in
``include/machete_b200.h``) together with the facts the host scheduler needs:
how many work units it has, how many ring pages and bytes each unit streams,
which memory it reads and writes (for dependency inference), and how units
map to completion counters.

The reference derives the equivalent facts from ``reads``/``writes`` and tile
counts inside ``InstructionStreamBuilder`` (src/machete/megakernel/
scheduling.py:691-2424); here they are explicit because the native kernels
choose their own unit shapes, independent of the API-level tile sizes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native as N
from .ops import TensorMeta, tensor_meta_overlaps

_TORCH_TO_T = {torch.bfloat16: N.T_BF16, torch.float16: N.T_FP16, torch.float32: N.T_FP32}


def elem_type(t: torch.Tensor, what: str = "tensor") -> int:
    try:
        return _TORCH_TO_T[t.dtype]
    except KeyError:
        raise ValueError(f"{what}: dtype {t.dtype} is not supported by the native kernels") from None


def meta_of(t: torch.Tensor, name: str = "") -> TensorMeta:
    return TensorMeta(
        name=name, declared_dims=(), ndim=t.ndim, shape=tuple(t.shape), strides=tuple(t.stride()),
        dtype=None, is_contiguous=t.is_contiguous(), data_ptr=t.data_ptr(),
        storage_ptr=t.untyped_storage().data_ptr(), storage_offset=t.storage_offset(),
        element_size=t.element_size(),
    )


@dataclass
class Region:
    """A tensor view an op touches; ``loader`` marks reads issued by the loader warp."""

    meta: TensorMeta
    loader: bool = False
    act: bool = False   # an input of the op's staged activations
    # optional refinement: rows [lo, hi) along ``axis`` actually touched
    axis: Optional[int] = None
    lo: int = 0
    hi: int = 0

    def overlaps(self, other: "Region") -> bool:
        return tensor_meta_overlaps(self.meta, other.meta)


@dataclass
class NativeOp:
    """One device op record plus scheduling facts."""

    name: str
    opcode: int
    n_units: int
    i: Dict[int, int] = field(default_factory=dict)
    f: Dict[int, float] = field(default_factory=dict)
    p: Dict[int, int] = field(default_factory=dict)
    s: Dict[int, int] = field(default_factory=dict)
    reads: List[Region] = field(default_factory=list)
    writes: List[Region] = field(default_factory=list)
    # pages / HBM bytes per unit: a constant or one value per unit
    pages: object = 0
    unit_bytes: object = 0
    # activation-staging signature (matvec): ops with equal signature and the
    # same producers share the staged buffer
    act_sig: Optional[tuple] = None
    act_bytes: int = 0
    writes_res_out: bool = False
    # completion counters: unit -> group, one counter per group
    n_groups: int = 1
    unit_group: Optional[np.ndarray] = None
    # fine-grained dependencies: producer name-kind -> fn(consumer_unit) -> groups or None
    fine_dep: Optional[Callable[["NativeOp", "NativeOp"], Optional[List[List[int]]]]] = None
    # loader-side refinement: fn(producer, unit) -> bool, does this unit's load need the producer
    loader_dep_units: Optional[Callable[["NativeOp", int], bool]] = None
    page_need: int = 0     # bytes one page of this op needs (for ring sizing)
    keep: list = field(default_factory=list)  # tensors kept alive
    kind: str = ""         # free-form tag used by peephole rules and tests
    # an op that follows the device-resident cache position: first position its tensors do not hold
    pos_limit: Optional[int] = None
    # scratch that must be zero when a launch starts; the kernel leaves it zero unless a launch aborted
    zero_on_reset: list = field(default_factory=list)

    def record(self, act_key: int) -> np.void:
        rec = np.zeros((), dtype=N.OP_DTYPE)
        rec["opcode"] = self.opcode
        rec["n_units"] = self.n_units
        rec["act_key"] = act_key
        for k, v in self.i.items():
            rec["i"][k] = int(v)
        for k, v in self.f.items():
            rec["f"][k] = float(v)
        for k, v in self.p.items():
            rec["p"][k] = int(v)
        for k, v in self.s.items():
            rec["s"][k] = int(v)
        return rec

    def pages_of(self, unit: int) -> int:
        return int(self.pages[unit]) if hasattr(self.pages, "__len__") else int(self.pages)

    def bytes_of(self, unit: int) -> int:
        return int(self.unit_bytes[unit]) if hasattr(self.unit_bytes, "__len__") else int(self.unit_bytes)

    def group_of(self, unit: int) -> int:
        return int(self.unit_group[unit]) if self.unit_group is not None else 0

    def group_sizes(self) -> np.ndarray:
        if self.unit_group is None:
            return np.array([self.n_units], dtype=np.int64)
        return np.bincount(self.unit_group, minlength=self.n_groups).astype(np.int64)


@dataclass
class LowerCtx:
    """Device facts and tunables visible to ``Op.lower``."""

    num_sms: int
    page_bytes: int
    smem_optin: int
    kc_bf16: int = 1024
    kc_fp4: int = 2048
    fuse: bool = True
    # shortest bf16 K-slice to pick for ops with few units per CTA (0 = never shorten).  Off by default:
    # on B200 the extra pages cost more than the extra warps per unit gain (931 vs 916 us per Llama-1B step)
    small_op_kc: int = 0


# ---- helpers shared by the matvec-family lowerings ---------------------------------------
def bf16_page_need(kc: int) -> int:
    """Two halves of kc/64 swizzled 1 KB tiles (8 rows x 128 B) each."""
    return 2 * (kc // 64) * 1024


def fp4_page_need(kc: int) -> int:
    """Two halves of kc/256 packed tiles plus two 1 KB scale tiles."""
    return 2 * (kc // 256) * 1024 + 2048


def attn_page_tokens(D: int, page_bytes: int) -> int:
    blk = 64 if D == 64 else 32
    tn = page_bytes // (4 * D)
    tn = (tn // blk) * blk
    return min(tn, 64)     # short pages: more consumer warps share a split (csrc/op_attn.cuh)


def split_bs(t: torch.Tensor) -> Tuple[int, int, int, int]:
    """(B, S, stride_B, stride_S) of a (B, S, X) activation tensor."""
    if t.ndim != 3:
        raise ValueError(f"expected a (B, S, X) tensor, got shape {tuple(t.shape)}")
    if t.stride(-1) != 1:
        raise ValueError("activation tensors need a unit innermost stride")
    return int(t.shape[0]), int(t.shape[1]), int(t.stride(0)), int(t.stride(1))
