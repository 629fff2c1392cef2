"""Lowering helpers for the row-wise ops (``csrc/op_elementwise.cuh``)."""

from __future__ import annotations

import torch

from .. import _native as N
from ..megakernel.lowering import NativeOp, Region, elem_type, meta_of


def rows_view(t: torch.Tensor, name: str):
    """(rows, row_stride) of a (..., D) tensor whose leading dims collapse to one stride."""
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: needs a unit innermost stride")
    lead = t.shape[:-1]
    rows = 1
    for n in lead:
        rows *= int(n)
    if t.ndim == 1:
        return 1, int(t.shape[-1])
    # leading dims must be collapsible: stride[i] == stride[i+1] * shape[i+1]
    for i in range(t.ndim - 2):
        if lead[i] != 1 and t.stride(i) != t.stride(i + 1) * t.shape[i + 1]:
            raise ValueError(f"{name}: leading dimensions must be collapsible into rows (got strides {t.stride()})")
    return rows, int(t.stride(-2))


def ew_op(name: str, opcode: int, n_units: int, kind: str) -> NativeOp:
    op = NativeOp(name=name, opcode=opcode, n_units=n_units, kind=kind)
    op.unit_bytes = 0
    return op
