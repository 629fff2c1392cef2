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

# magnitudes of the eight E2M1 codes; code | 8 is the negative of code
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# a magnitude takes the code of the nearest value; ties go down (strict comparison against the midpoints)
_MIDPOINTS = tuple((a + b) / 2 for a, b in zip(E2M1_VALUES[:-1], E2M1_VALUES[1:]))
_E4M3 = getattr(torch, "float8_e4m3fn", None)
_E4M3_MAX, _E2M1_MAX = 448.0, 6.0


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
        packed, scales, g = self.packed, self.scales, self.group_size
        if g not in (16, 32):
            raise ValueError("group_size must be 32 (fp16 scales) or 16 (e4m3 scales)")
        if packed.dtype != torch.uint8:
            raise TypeError(f"packed must be torch.uint8, got {packed.dtype}")
        if g == 32 and scales.dtype != torch.float16:
            raise TypeError(f"scales must be torch.float16, got {scales.dtype}")
        if g == 16 and scales.element_size() != 1:
            raise TypeError(f"16-value groups use e4m3 scales, got {scales.dtype}")
        if packed.dim() != 2 or scales.dim() != 2:
            raise ValueError("packed and scales must be rank-2 tensors")
        n_rows, n_cols = int(packed.shape[0]), 2 * int(packed.shape[1])
        if self.rows not in (None, n_rows):
            raise ValueError("rows must match packed.shape[0]")
        if self.cols not in (None, n_cols):
            raise ValueError("cols must equal packed.shape[1] * 2")
        if n_cols % g:
            raise ValueError("cols must be divisible by group_size")
        if tuple(scales.shape) != (n_rows, n_cols // g):
            raise ValueError(f"scales shape must be {(n_rows, n_cols // g)}, got {tuple(scales.shape)}")
        object.__setattr__(self, "rows", n_rows)
        object.__setattr__(self, "cols", n_cols)


def _codes(groups: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """E2M1 codes of ``groups / scale`` (``(rows, n_groups, g)`` against ``(rows, n_groups)``), packed
    two per byte with the even column in the low nibble."""
    x = groups / scale.unsqueeze(-1)
    mag = x.abs()
    code = torch.zeros(mag.shape, dtype=torch.uint8, device=mag.device)
    for mid in _MIDPOINTS:                      # = the number of midpoints strictly below the magnitude
        code += mag > mid
    code |= (x < 0).to(torch.uint8) << 3
    code = code.reshape(code.shape[0], -1)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()


@torch.no_grad()
def quantize_nvfp4_weight(weight: torch.Tensor, group_size: int = 32, scale_dtype=None) -> NVFP4Tensor:
    """Quantise a ``(rows, cols)`` fp16/bf16/fp32 matrix to packed E2M1."""
    if weight.dim() != 2:
        raise ValueError(f"weight must be rank-2, got shape {tuple(weight.shape)}")
    if weight.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"unsupported weight dtype {weight.dtype}")
    rows, cols = (int(v) for v in weight.shape)
    if group_size % 2:
        raise ValueError("group_size must be even")
    if cols % 2:
        raise ValueError("weight cols must be divisible by 2")
    if cols % group_size:
        raise ValueError("weight cols must be divisible by group_size")
    if scale_dtype is None:
        scale_dtype = torch.float16 if group_size == 32 else _E4M3
    groups = weight.float().reshape(rows, cols // group_size, group_size)
    peak = groups.abs().amax(dim=-1)
    one = torch.ones_like(peak)
    if (group_size, scale_dtype) == (32, torch.float16):
        # the division uses the unrounded fp32 scale; the stored scale is its fp16 rounding
        scale = torch.where(peak > 0, peak / _E2M1_MAX, one)
        return NVFP4Tensor(_codes(groups, scale), scale.to(torch.float16).contiguous(), group_size, rows, cols)
    if group_size == 16 and _E4M3 is not None and scale_dtype == _E4M3:
        top = float(peak.max())
        global_scale = top / (_E4M3_MAX * _E2M1_MAX) if top > 0 else 1.0
        stored = (peak / _E2M1_MAX / global_scale).clamp(max=_E4M3_MAX).to(_E4M3)
        # codes against the scale the kernel will see (the decoded e4m3 value times the global scale)
        seen = stored.float() * global_scale
        return NVFP4Tensor(_codes(groups, torch.where(seen > 0, seen, one)), stored.contiguous(), group_size, rows, cols,
                           global_scale)
    raise ValueError(f"unsupported NVFP4 layout: group_size={group_size}, scale_dtype={scale_dtype}")


@torch.no_grad()
def dequantize_nvfp4_weight(qweight: NVFP4Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Decode a packed NVFP4 matrix (validation / reference code)."""
    dev = qweight.packed.device
    nibbles = torch.stack((qweight.packed & 0x0F, qweight.packed >> 4), dim=-1).reshape(qweight.rows, qweight.cols)
    magnitude = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=dev)[(nibbles & 7).long()]
    value = torch.where((nibbles & 8) != 0, -magnitude, magnitude)
    scale = (qweight.scales.float() * float(qweight.global_scale)).repeat_interleave(qweight.group_size, dim=1)
    return (value * scale).to(dtype)


__all__ = ["NVFP4Tensor", "quantize_nvfp4_weight", "dequantize_nvfp4_weight", "E2M1_VALUES"]
