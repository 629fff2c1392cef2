"""Packed NVFP4 (E2M1) weight quantisation, two scale layouts.

``group_size=32`` with fp16 scales reproduces the reference's host quantiser
bit for bit (src/machete/quantization/nvfp4.py:78-122): two E2M1 codes per
byte, low nibble first; one fp16 scale per row and 32-value group,
``scale = amax / 6`` (1.0 for an all-zero group); codes from
``bucketize(|w / scale|, [.25, .75, 1.25, 1.75, 2.5, 3.5, 5])`` with the sign
in bit 3, the division using the *unrounded* fp32 scale.

``group_size=16`` with ``scale_dtype=torch.float8_e4m3fn`` is the NVIDIA
block-scaled layout: an e4m3 scale per 16 values plus one fp32 global scale
per tensor, ``global = amax_tensor / (448 * 6)``,
``block_scale = e4m3(amax_block / 6 / global)``; codes are taken against the
*decoded* ``block_scale * global`` so that dequantisation inverts them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_LUT = torch.tensor(list(E2M1_VALUES) + [-v for v in E2M1_VALUES], dtype=torch.float32)
_E2M1_THRESHOLDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32)
_E4M3 = getattr(torch, "float8_e4m3fn", None)


@dataclass(frozen=True)
class NVFP4Tensor:
    """Packed row-major NVFP4 matrix plus per-group scales (and a global scale)."""

    packed: torch.Tensor
    scales: torch.Tensor
    group_size: int = 32
    rows: Optional[int] = None
    cols: Optional[int] = None
    global_scale: float = 1.0

    def __post_init__(self):
        if self.packed.dtype != torch.uint8:
            raise TypeError(f"packed must be torch.uint8, got {self.packed.dtype}")
        if self.group_size == 32:
            if self.scales.dtype != torch.float16:
                raise TypeError(f"scales must be torch.float16, got {self.scales.dtype}")
        elif self.group_size == 16:
            if self.scales.element_size() != 1:
                raise TypeError(f"16-value groups use e4m3 scales, got {self.scales.dtype}")
        else:
            raise ValueError("group_size must be 32 (fp16 scales) or 16 (e4m3 scales)")
        if self.packed.dim() != 2 or self.scales.dim() != 2:
            raise ValueError("packed and scales must be rank-2 tensors")
        rows = self.packed.shape[0] if self.rows is None else self.rows
        cols = self.packed.shape[1] * 2 if self.cols is None else self.cols
        if rows != self.packed.shape[0]:
            raise ValueError("rows must match packed.shape[0]")
        if cols != self.packed.shape[1] * 2:
            raise ValueError("cols must equal packed.shape[1] * 2")
        if cols % self.group_size != 0:
            raise ValueError("cols must be divisible by group_size")
        expected = (rows, cols // self.group_size)
        if tuple(self.scales.shape) != expected:
            raise ValueError(f"scales shape must be {expected}, got {tuple(self.scales.shape)}")
        object.__setattr__(self, "rows", rows)
        object.__setattr__(self, "cols", cols)


def _check_weight(weight: torch.Tensor, group_size: int) -> None:
    if weight.dim() != 2:
        raise ValueError(f"weight must be rank-2, got shape {tuple(weight.shape)}")
    if weight.shape[1] % 2 != 0:
        raise ValueError("weight cols must be divisible by 2")
    if weight.shape[1] % group_size != 0:
        raise ValueError("weight cols must be divisible by group_size")
    if group_size % 2 != 0:
        raise ValueError("group_size must be even")
    if weight.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported weight dtype {weight.dtype}")


def _encode(normalized: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    thresholds = _E2M1_THRESHOLDS.to(normalized.device)
    codes = torch.bucketize(normalized.abs().contiguous(), thresholds).to(torch.uint8)
    codes = codes | ((normalized < 0).to(torch.uint8) << 3)
    codes = codes.reshape(rows, cols)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()


@torch.no_grad()
def quantize_nvfp4_weight(weight: torch.Tensor, group_size: int = 32, scale_dtype=None) -> NVFP4Tensor:
    """Quantise a ``(rows, cols)`` fp16/bf16/fp32 matrix to packed E2M1."""
    _check_weight(weight, group_size)
    rows, cols = weight.shape
    w = weight.float().reshape(rows, cols // group_size, group_size)
    amax = w.abs().amax(dim=-1)
    if scale_dtype is None:
        scale_dtype = torch.float16 if group_size == 32 else _E4M3
    if group_size == 32 and scale_dtype == torch.float16:
        scales_f = torch.where(amax > 0, amax / 6.0, torch.ones_like(amax))
        packed = _encode(w / scales_f.unsqueeze(-1), rows, cols)
        return NVFP4Tensor(packed, scales_f.to(torch.float16).contiguous(), group_size, rows, cols)
    if group_size == 16 and _E4M3 is not None and scale_dtype == _E4M3:
        tensor_amax = float(amax.max())
        global_scale = tensor_amax / (448.0 * 6.0) if tensor_amax > 0 else 1.0
        block = (amax / 6.0 / global_scale).clamp(max=448.0).to(_E4M3)
        decoded = block.float() * global_scale
        safe = torch.where(decoded > 0, decoded, torch.ones_like(decoded))
        packed = _encode(w / safe.unsqueeze(-1), rows, cols)
        return NVFP4Tensor(packed, block.contiguous(), group_size, rows, cols, global_scale)
    raise ValueError(f"unsupported NVFP4 layout: group_size={group_size}, scale_dtype={scale_dtype}")


@torch.no_grad()
def dequantize_nvfp4_weight(qweight: NVFP4Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Decode a packed NVFP4 matrix (validation / reference code)."""
    lut = _E2M1_LUT.to(qweight.packed.device)
    packed = qweight.packed
    codes = torch.empty((qweight.rows, qweight.cols), dtype=torch.long, device=packed.device)
    codes[:, 0::2] = (packed & 0x0F).long()
    codes[:, 1::2] = (packed >> 4).long()
    vals = lut[codes].reshape(qweight.rows, qweight.cols // qweight.group_size, qweight.group_size)
    scales = qweight.scales.float() * float(qweight.global_scale)
    return (vals * scales.unsqueeze(-1)).reshape(qweight.rows, qweight.cols).to(dtype)


__all__ = ["NVFP4Tensor", "quantize_nvfp4_weight", "dequantize_nvfp4_weight", "E2M1_VALUES"]
