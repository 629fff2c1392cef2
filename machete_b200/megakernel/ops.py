"""Op protocol of the megakernel: declarations, ``schedule()`` and ``ScheduledOp``.

Host-side mirror of the reference's op protocol (src/machete/megakernel/ops.py:
``Op`` :1096, ``_process_op_declarations`` :881, ``_schedule_single`` :947,
``pack_config`` :675, ``TensorMeta`` :402, ``tensor_meta_overlaps`` :531,
``ScheduledOp`` :1373).  An op class declares its tensors as
``reads``/``writes`` dictionaries of ``name -> (dtype, dims)`` and the dims it
tiles over; ``schedule(**tensors)`` validates the tensors against the
declaration and captures pointers, shapes and strides.

What differs from the reference: there is no JIT, so an op has no
``load/compute/store`` bodies.  Instead every runnable op class implements
``lower(scheduled_op, ctx)``, which turns the scheduled op into records for
the precompiled sm_100a kernel (see ``machete_b200.megakernel.lowering``).
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass, field
from typing import Any, ClassVar, Dict, List, Optional, Tuple, Type

import torch

MAX_TILE_DIMS = 4
DEFAULT_PAGE_SIZE: int = 49152
"""Default ``page_size`` keyword of ``schedule()`` (bytes); kept for API parity."""

_SCHEDULING_STATIC_DIM_PREFIXES = ("barrier_", "pipeline_", "load_replay_")


# ---- dtype tokens -------------------------------------------------------------
class _DType:
    """Element-type token used in ``reads``/``writes`` declarations."""

    def __init__(self, name: str, width: int, torch_dtype):
        self.name, self.width, self.torch_dtype = name, width, torch_dtype

    def __repr__(self):
        return self.name


Float16 = _DType("Float16", 16, torch.float16)
BFloat16 = _DType("BFloat16", 16, torch.bfloat16)
Float32 = _DType("Float32", 32, torch.float32)
Int32 = _DType("Int32", 32, torch.int32)
Int64 = _DType("Int64", 64, torch.int64)
Uint8 = _DType("Uint8", 8, torch.uint8)
Float8E4M3 = _DType("Float8E4M3", 8, getattr(torch, "float8_e4m3fn", torch.uint8))

TORCH_TO_MK_DTYPE = {
    torch.float16: Float16,
    torch.bfloat16: BFloat16,
    torch.float32: Float32,
    torch.int32: Int32,
    torch.int64: Int64,
    torch.uint8: Uint8,
}
if hasattr(torch, "float8_e4m3fn"):
    TORCH_TO_MK_DTYPE[torch.float8_e4m3fn] = Float8E4M3
# name the reference exports (its values are CUTLASS dtypes)
TORCH_TO_CUTLASS_DTYPE = TORCH_TO_MK_DTYPE


def is_compile_static_dim(name: str) -> bool:
    """Scheduler-only ``static_dims`` keys never select device code."""
    return not name.startswith(_SCHEDULING_STATIC_DIM_PREFIXES)


def _resolve_dtype(declared, tensor_dtype):
    if declared is None:
        if tensor_dtype not in TORCH_TO_MK_DTYPE:
            raise ValueError(f"Unsupported tensor dtype: {tensor_dtype}")
        return TORCH_TO_MK_DTYPE[tensor_dtype]
    return declared


# ---- pipeline declarations (structural metadata only) --------------------------
@dataclass(frozen=True)
class PipelineSpec:
    """Page/semaphore budget an op asks of the shared-memory ring.

    Kept for declaration compatibility (reference ops.py:56-153); the native
    loader sizes its ring from the program, not from this contract.
    """

    page_count: int
    page_bytes: int = 0
    input_stages: int = 0
    output_stages: int = 0
    stage_pages: int = 1
    semaphore_count: int = 0
    scratch_bytes: int = 0

    def __post_init__(self):
        if self.page_count < 1:
            raise ValueError("PipelineSpec.page_count must be >= 1")
        for name in ("page_bytes", "input_stages", "output_stages", "semaphore_count", "scratch_bytes"):
            if getattr(self, name) < 0:
                raise ValueError(f"PipelineSpec.{name} must be non-negative")
        if self.stage_pages < 1:
            raise ValueError("PipelineSpec.stage_pages must be >= 1")

    @property
    def resource_bytes(self) -> int:
        return self.page_count * self.page_bytes + self.semaphore_count * 8 + self.scratch_bytes

    def with_overrides(self, **overrides) -> "PipelineSpec":
        values = {f: getattr(self, f) for f in (
            "page_count", "page_bytes", "input_stages", "output_stages", "stage_pages", "semaphore_count",
            "scratch_bytes")}
        values.update({k: v for k, v in overrides.items() if v is not None})
        return PipelineSpec(**values)

    @classmethod
    def streaming(cls, *, input_stages=3, output_stages=3, stage_pages=4, page_bytes=0, scratch_bytes=0):
        return cls(
            page_count=1 + input_stages * stage_pages,
            page_bytes=page_bytes,
            input_stages=input_stages,
            output_stages=output_stages,
            stage_pages=stage_pages,
            semaphore_count=1 + 2 * (input_stages + output_stages),
            scratch_bytes=scratch_bytes,
        )


# ---- tensor metadata and aliasing -----------------------------------------------
@dataclass
class TensorMeta:
    """Shape/stride/pointer snapshot of a tensor taken at ``schedule()`` time."""

    name: str
    declared_dims: Tuple[str, ...]
    ndim: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    dtype: Any
    is_contiguous: bool
    data_ptr: int
    storage_ptr: int
    storage_offset: int
    element_size: int = 2

    def byte_span(self) -> Tuple[int, int]:
        """Half-open absolute address range touched by the view."""
        if any(s == 0 for s in self.shape):
            return (self.data_ptr, self.data_ptr)
        hi = sum((n - 1) * abs(st) for n, st in zip(self.shape, self.strides)) + 1
        return (self.data_ptr, self.data_ptr + hi * self.element_size)


def _axis_starts(meta: TensorMeta) -> Optional[Tuple[int, ...]]:
    """Per-axis start indices of a view inside its storage lattice."""
    remaining = meta.storage_offset
    starts = []
    for axis, stride in enumerate(meta.strides):
        if stride <= 0:
            return None
        if axis == meta.ndim - 1:
            starts.append(remaining // stride if stride else 0)
            break
        starts.append(remaining // stride)
        remaining %= stride
    return tuple(starts)


def tensor_meta_overlaps(a: TensorMeta, b: TensorMeta) -> bool:
    """Do two captured views share any byte?

    Exact for views of one storage with identical strides (slices of a packed
    buffer are told apart axis by axis); otherwise the address spans decide,
    which can only over-report.
    """
    if a.data_ptr == b.data_ptr and min(a.byte_span()[1] - a.data_ptr, b.byte_span()[1] - b.data_ptr) > 0:
        return True
    a_lo, a_hi = a.byte_span()
    b_lo, b_hi = b.byte_span()
    if max(a_lo, b_lo) >= min(a_hi, b_hi):
        return False
    if (a.storage_ptr == b.storage_ptr and a.ndim == b.ndim and a.strides == b.strides
            and a.element_size == b.element_size):
        sa, sb = _axis_starts(a), _axis_starts(b)
        if sa is not None and sb is not None:
            return all(
                max(sa[i], sb[i]) < min(sa[i] + a.shape[i], sb[i] + b.shape[i]) for i in range(a.ndim)
            )
    return True


def last_dim_slice_region(full: TensorMeta, view: TensorMeta) -> Optional[Tuple[int, int, int]]:
    """``(start, length, full_length)`` if ``view`` is a last-dim slice of ``full``."""
    if full.storage_ptr != view.storage_ptr or full.ndim != view.ndim or full.ndim == 0:
        return None
    if full.strides != view.strides or full.shape[:-1] != view.shape[:-1]:
        return None
    sf, sv = _axis_starts(full), _axis_starts(view)
    if sf is None or sv is None or sf[:-1] != sv[:-1]:
        return None
    start = sv[-1] - sf[-1]
    if start < 0 or start + view.shape[-1] > full.shape[-1]:
        return None
    return start, view.shape[-1], full.shape[-1]


# ---- declaration processing --------------------------------------------------------
def _parse_dims(dims) -> List[str]:
    if isinstance(dims, (tuple, list)):
        return list(dims)
    if isinstance(dims, str):
        return [d.strip() for d in dims.split(",")]
    raise TypeError(f"dims must be tuple, list, or str, got {type(dims)}")


def _parse_tile_spec(tile) -> Tuple[str, ...]:
    if isinstance(tile, str):
        tile = (tile,)
    for item in tile:
        if not isinstance(item, str):
            raise ValueError(
                f"Invalid tile spec item: {item}. Expected dimension name string. "
                f"Tile sizes are passed at schedule() time via tile_sizes=."
            )
    return tuple(tile)


def _process_op_declarations(cls) -> None:
    tile = _parse_tile_spec(cls.tile)
    if len(tile) > MAX_TILE_DIMS:
        raise ValueError(f"Tile spec has {len(tile)} dims, max is {MAX_TILE_DIMS}")

    tensors: List[Tuple[str, Any, List[str]]] = []
    dims: List[Tuple[str, str, int]] = []
    seen_t, seen_d = set(), set()
    for decls in (cls.reads, cls.writes):
        for name, (dtype, dim_spec) in decls.items():
            if name in seen_t:
                continue
            seen_t.add(name)
            dlist = _parse_dims(dim_spec)
            tensors.append((name, dtype, dlist))
            for axis, d in enumerate(dlist):
                if d not in seen_d:
                    seen_d.add(d)
                    dims.append((d, name, axis))

    for d in tile:
        if d not in seen_d:
            raise ValueError(f"Tile dim '{d}' not found in any tensor shape declaration")

    overrides = set(getattr(cls, "dynamic_dims", ()))
    dynamic = {d for d, _, _ in dims if d not in tile} | overrides

    cls._UNIQUE_TENSORS = tensors
    cls._UNIQUE_DIMS = dims
    cls._TILE_DIM_NAMES = set(tile)
    cls._TILE_DIM_NAMES_ORDERED = tile
    cls._DYNAMIC_DIM_OVERRIDES = overrides
    cls._STATIC_DIM_NAMES = [d for d, _, _ in dims if d not in dynamic]
    cls.INPUTS = list(cls.reads.keys())
    cls.OUTPUTS = list(cls.writes.keys())
    cls.DIM_NAMES = {tile[i]: i for i in range(len(tile))}

    read_names, write_names = set(cls.reads), set(cls.writes)
    for attr, valid, kind in (
        ("tma_loads", read_names, "reads"), ("tma_compute_loads", read_names, "reads"),
        ("tma_stores", write_names, "writes"), ("tma_compute_stores", write_names, "writes"),
        ("tma_reduce_stores", write_names, "writes"), ("peer_stores", write_names, "writes"),
        ("peer_reduce_stores", write_names, "writes"),
    ):
        names = set(getattr(cls, attr, set()))
        for n in names:
            if n not in valid:
                raise ValueError(f"{attr} tensor '{n}' not found in {kind}")
        setattr(cls, "_" + attr.upper(), names)

    # config tensor layout: [ptr_lo, ptr_hi] per tensor, then the dynamic dims
    n_t = len(tensors)
    dyn = [(d, t, a) for d, t, a in dims if d in dynamic]
    cls._CONFIG_PTR_I64_INDEX = {name: i for i, (name, _, _) in enumerate(tensors)}
    cls._CONFIG_PTR_I32_OFFSET = {name: 2 * i for i, (name, _, _) in enumerate(tensors)}
    cls._CONFIG_DYNAMIC_I32_OFFSET = {d: 2 * n_t + j for j, (d, _, _) in enumerate(dyn)}
    config_size = 2 * n_t + len(dyn)

    def pack_config(**given):
        """Pointers (lo, hi words) and dynamic dims as an int32 tensor on the tensors' device."""
        first = next(iter(given.values()))
        words = [0] * config_size
        for i, (name, _, _) in enumerate(tensors):
            t = given.get(name)
            if t is None:  # optional tensor not supplied: null pointer
                continue
            if not (t.is_contiguous() or t.stride(-1) == 1):
                raise AssertionError(f"{name} must be contiguous or have unit innermost stride")
            lo, hi = struct.unpack("<2i", struct.pack("<Q", t.data_ptr()))
            words[2 * i], words[2 * i + 1] = lo, hi
        for j, (_, tname, axis) in enumerate(dyn):
            words[2 * n_t + j] = int(given[tname].shape[axis])
        return torch.tensor(words, dtype=torch.int32, device=first.device)

    cls.pack_config = staticmethod(pack_config)


# ---- the protocol ---------------------------------------------------------------------
class Op:
    """Base class of megakernel operations.

    Subclasses declare ``reads``, ``writes`` and ``tile`` and, to be runnable
    on the device, implement ``lower``.  A subclass without ``lower`` can
    still be scheduled (dependency inference treats it as a black box) but
    ``Megakernel`` refuses to build a program that contains it: there is no
    JIT that could compile a user-written body.
    """

    INPUTS: ClassVar[List[str]] = []
    OUTPUTS: ClassVar[List[str]] = []
    pipeline: ClassVar[Optional[PipelineSpec]] = None
    inline_phases: ClassVar[Tuple[str, ...]] = ()
    sync_compute_warps_after_tile: ClassVar[bool] = False
    uses_smem_page: ClassVar[bool] = True

    def __init__(self, **config):
        for key, value in config.items():
            setattr(self, key, value)

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if "reads" in cls.__dict__ or "writes" in cls.__dict__ or "tile" in cls.__dict__:
            if hasattr(cls, "reads") and hasattr(cls, "writes") and hasattr(cls, "tile"):
                _process_op_declarations(cls)

    # -- scheduling ---------------------------------------------------------------------
    @classmethod
    def _schedule_single(cls, tile_sizes=None, **tensors) -> "ScheduledOp":
        tile_sizes = dict(tile_sizes or {})
        unique_tensors, unique_dims = cls._UNIQUE_TENSORS, cls._UNIQUE_DIMS

        for name, _dtype, dims in unique_tensors:
            t = tensors.get(name)
            if t is not None and hasattr(t, "ndim") and t.ndim != len(dims):
                raise ValueError(
                    f"{cls.__name__}: tensor '{name}' declared as {len(dims)}D (dims={dims}) "
                    f"but got {t.ndim}D tensor with shape {tuple(t.shape)}"
                )

        dim_values: Dict[str, int] = {}
        for dim_name, tensor_name, axis in unique_dims:
            if tensor_name not in tensors:
                raise ValueError(f"{cls.__name__}: missing tensor '{tensor_name}'")
            dim_values[dim_name] = int(tensors[tensor_name].shape[axis])
        # every declared axis must agree with the first tensor that named the dim
        for name, _dtype, dims in unique_tensors:
            t = tensors.get(name)
            if t is None or not hasattr(t, "shape"):
                continue
            for axis, d in enumerate(dims):
                if int(t.shape[axis]) != dim_values[d]:
                    raise ValueError(
                        f"{cls.__name__}: dim '{d}' conflict: expected {dim_values[d]} but tensor "
                        f"'{name}' axis {axis} has {int(t.shape[axis])}"
                    )

        static_dims = {d: v for d, v in dim_values.items() if d not in cls._DYNAMIC_DIM_OVERRIDES}

        resolved, counts = {}, []
        for d in cls._TILE_DIM_NAMES_ORDERED:
            extent = dim_values[d]
            req = tile_sizes.get(d)
            if req is None:
                resolved[d] = extent
                counts.append(1)
            else:
                size = max(1, min(int(req), extent)) if extent > 0 else 1
                resolved[d] = size
                counts.append(max(1, (extent + size - 1) // size))

        tensor_dtypes, ptrs, refs, metas, strides = {}, {}, {}, {}, {}
        for name, t in tensors.items():
            if hasattr(t, "data_ptr"):
                ptrs[name] = t.data_ptr()
                refs[name] = t
        for name, declared, dims in unique_tensors:
            t = tensors.get(name)
            if t is None:
                continue
            if declared is None:
                tensor_dtypes[name] = _resolve_dtype(None, t.dtype)
            metas[name] = TensorMeta(
                name=name,
                declared_dims=tuple(dims),
                ndim=len(dims),
                shape=tuple(t.shape),
                strides=tuple(t.stride()),
                dtype=tensor_dtypes.get(name, declared),
                is_contiguous=t.is_contiguous(),
                data_ptr=t.data_ptr(),
                storage_ptr=t.untyped_storage().data_ptr(),
                storage_offset=t.storage_offset(),
                element_size=t.element_size(),
            )
            strides[name] = tuple(t.stride())

        return ScheduledOp(
            op_cls=cls,
            tile_counts=tuple(counts),
            config_data=cls.pack_config(**tensors),
            static_dims=static_dims,
            tensor_dtypes=tensor_dtypes,
            tensor_ptrs=ptrs,
            tensor_refs=refs,
            dim_names=cls.DIM_NAMES,
            tile_sizes=resolved,
            tensor_metas=metas,
            tensor_strides=strides,
        )

    @classmethod
    def schedule(cls, tile_sizes=None, **tensors) -> List["ScheduledOp"]:
        return [cls._schedule_single(tile_sizes=tile_sizes, **tensors)]

    @classmethod
    def gen_tensor_param_names(cls) -> List[str]:
        return [name for name, _, _ in cls._UNIQUE_TENSORS]

    # -- lowering -----------------------------------------------------------------------
    @classmethod
    def lower(cls, sop: "ScheduledOp", ctx) -> list:
        raise NotImplementedError(
            f"{cls.__name__} has no native sm_100a handler: this build runs one precompiled "
            f"persistent kernel and cannot JIT a user-defined compute() body"
        )

    # phase stubs kept so subclass code written against the reference imports cleanly
    def load(self, page_ptr) -> None:  # pragma: no cover - never executed
        pass

    def compute(self, page_ptr) -> None:  # pragma: no cover
        pass

    def store(self, page_ptr) -> None:  # pragma: no cover
        pass

    def communicate(self, page_ptr) -> None:  # pragma: no cover
        pass


def build_op_config(op: "ScheduledOp", kernel_config: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """Flatten a scheduled op into the attribute dict the reference hands to op instances."""
    config: Dict[str, Any] = dict(kernel_config or {})
    for d, size in (op.tile_sizes or {}).items():
        config[f"tile_size_{d}"] = size
    config.update({k: v for k, v in (op.static_dims or {}).items() if is_compile_static_dim(k)})
    for name, dtype, dims in getattr(op.op_cls, "_UNIQUE_TENSORS", []):
        resolved = (op.tensor_dtypes or {}).get(name, dtype)
        if resolved is not None:
            config.setdefault(f"{name}_dtype", resolved)
        if name in (op.tensor_strides or {}):
            for i, d in enumerate(dims):
                config[f"{name}_stride_{d}"] = op.tensor_strides[name][i]
    return config


@dataclass
class ScheduledOp:
    """An op class bound to concrete tensors and a tile grid."""

    op_cls: Type[Op]
    tile_counts: Tuple[int, ...] = (1,)
    params: Dict[str, Any] = field(default_factory=dict)
    dim_names: Dict[str, int] = None
    config_data: Any = None
    static_dims: Dict[str, Any] = field(default_factory=dict)
    tensor_dtypes: Dict[str, Any] = field(default_factory=dict)
    tile_sizes: Dict[str, int] = field(default_factory=dict)
    tensor_ptrs: Dict[str, int] = field(default_factory=dict)
    tensor_refs: Dict[str, Any] = field(default_factory=dict)
    tensor_metas: Dict[str, TensorMeta] = field(default_factory=dict)
    tensor_strides: Dict[str, Tuple[int, ...]] = field(default_factory=dict)
    dim_aliases: Dict[str, str] = field(default_factory=dict)

    def __post_init__(self):
        if self.dim_names is None:
            self.dim_names = getattr(self.op_cls, "DIM_NAMES", {})
        if len(self.tile_counts) > MAX_TILE_DIMS:
            raise ValueError(
                f"{self.op_cls.__name__} has {len(self.tile_counts)} tile dims, max supported is {MAX_TILE_DIMS}"
            )
        for count in self.tile_counts:
            if count < 1 or count > 0xFFFF:
                raise ValueError(f"{self.op_cls.__name__} tile counts must be in [1, 65535], got {count}")

    @property
    def ndims(self) -> int:
        return len(self.tile_counts)

    @property
    def total_tiles(self) -> int:
        return math.prod(self.tile_counts)

    def tiles_for_axis(self, axis: int) -> int:
        return self.tile_counts[axis] if axis < len(self.tile_counts) else 1


__all__ = [
    "MAX_TILE_DIMS", "DEFAULT_PAGE_SIZE", "TORCH_TO_CUTLASS_DTYPE", "TORCH_TO_MK_DTYPE",
    "Float16", "BFloat16", "Float32", "Int32", "Int64", "Uint8", "Float8E4M3",
    "PipelineSpec", "TensorMeta", "Op", "ScheduledOp", "build_op_config", "is_compile_static_dim",
    "tensor_meta_overlaps", "last_dim_slice_region",
]
