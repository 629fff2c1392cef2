"""The reference interpreter's instruction-row and barrier-formula formats.

This build's device loop reads its own tables (``mk_instr_t``, ``mk_event_t``); nothing here is
on its launch path.  The two formats below are how the reference's replay loop is fed
(src/machete/megakernel/scheduling.py:40-175, instruction_layout.py:1-12), and they are what a
tool needs in order to read a reference schedule dump, or to emit one from a program built here:

* a barrier formula names one dependency counter per tile:
  ``index = base + offset + sum(coeff[i] * (tile[i] // div[i]))``, with an ``expected`` signal
  count and an optional half-open guard on a linear tile index;
* an instruction row is five int32 words:
  ``[op | range_meta << 16, tile0 | tile1 << 16, tile2 | tile3 << 16, barrier row, range end]``
  where ``range_meta = (range_axis + 1) | (range_end_axis + 1) << 4`` (0 = a single tile) and an
  all-ones low half-word in word 0 ends a CTA's stream.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, List, Optional, Sequence, Tuple

from .ops import MAX_TILE_DIMS

INSTRUCTION_WORDS = 5
END_OF_STREAM = 0xFFFF


def _pad(tiles: Sequence[int]) -> Tuple[int, ...]:
    t = tuple(int(v) for v in tiles)
    if len(t) > MAX_TILE_DIMS:
        raise ValueError(f"Instruction tile rank exceeds {MAX_TILE_DIMS}")
    return t + (0,) * (MAX_TILE_DIMS - len(t))


def _i32(word: int) -> int:
    """The two's-complement int32 reading of an unsigned 32-bit word (rows live in int32 tensors)."""
    return word - (1 << 32) if word >= (1 << 31) else word


@dataclass
class BarrierFormula:
    """``index(tile) = base + offset + sum(coeffs[i] * (tile[i] // divs[i]))``; see the module docstring."""

    NO_GUARD: ClassVar[int] = 1 << 30          # a guard_max no tile index reaches

    base: int
    coeffs: Tuple[int, ...] = (0,) * MAX_TILE_DIMS
    divs: Tuple[int, ...] = (1,) * MAX_TILE_DIMS
    offset: int = 0
    expected: int = 1
    guard_min: int = 0
    guard_max: int = NO_GUARD
    guard_coeffs: Optional[Tuple[int, ...]] = None

    def compute_index(self, tiles: Sequence[int]) -> int:
        t = _pad(tiles)
        return self.base + self.offset + sum(c * (v // d) for c, v, d in zip(self.coeffs, t, self.divs))

    def is_guarded(self, tiles: Sequence[int]) -> bool:
        """Does the guard let this tile through?  The linear index uses ``guard_coeffs`` (default: ``coeffs``)."""
        t = _pad(tiles)
        gc = self.coeffs if self.guard_coeffs is None else self.guard_coeffs
        return self.guard_min <= sum(c * v for c, v in zip(gc, t)) < self.guard_max

    @property
    def has_guard(self) -> bool:
        return (self.guard_min, self.guard_max) != (0, self.NO_GUARD)


@dataclass
class TileInstruction:
    """One tile (or one range of tiles along ``range_axis``, ending before ``range_end``) of op ``op_idx``."""

    END_MARKER: ClassVar[int] = -1

    op_idx: int
    tiles: Tuple[int, ...]
    range_axis: int = -1
    range_end_axis: int = -1
    range_end: int = 0

    @classmethod
    def end_instruction(cls) -> "TileInstruction":
        return cls(cls.END_MARKER, (0,) * MAX_TILE_DIMS)

    @property
    def is_range(self) -> bool:
        return self.range_axis >= 0 and self.range_end_axis >= 0

    def pack(self, barrier_meta_idx: int = 0) -> List[int]:
        """The five int32 words of this instruction; ``barrier_meta_idx`` = its row in the wait / signal side tables."""
        if self.op_idx == self.END_MARKER:
            return [END_OF_STREAM, 0, 0, 0, 0]
        if not 0 <= self.op_idx < END_OF_STREAM:
            raise ValueError(f"Instruction op_idx must fit in uint16, got {self.op_idx}")
        if not 0 <= barrier_meta_idx < (1 << 31):
            raise ValueError(f"Instruction barrier_meta_idx must fit in int32, got {barrier_meta_idx}")
        t = _pad(self.tiles)
        for v in t:
            if not 0 <= v <= 0xFFFF:
                raise ValueError(f"Instruction tile coordinate must fit in uint16, got {v}")
        meta = 0
        if self.is_range:
            if self.range_axis >= MAX_TILE_DIMS:
                raise ValueError(f"range_axis must be < {MAX_TILE_DIMS}, got {self.range_axis}")
            if self.range_end_axis > 0xE:
                raise ValueError(f"range_end_axis must fit in 4 encoded bits, got {self.range_end_axis}")
            if not 0 <= self.range_end <= 0xFFFF:
                raise ValueError(f"range_end must fit in uint16, got {self.range_end}")
            meta = (self.range_axis + 1) | ((self.range_end_axis + 1) << 4)
        return [_i32(self.op_idx | (meta << 16)), _i32(t[0] | (t[1] << 16)), _i32(t[2] | (t[3] << 16)),
                barrier_meta_idx, self.range_end]

    @classmethod
    def unpack(cls, row: Sequence[int]) -> Tuple["TileInstruction", int]:
        """Inverse of :meth:`pack`: ``(instruction, barrier_meta_idx)``."""
        if len(row) != INSTRUCTION_WORDS:
            raise ValueError(f"an instruction row has {INSTRUCTION_WORDS} words, got {len(row)}")
        w0, w1, w2 = (int(v) & 0xFFFFFFFF for v in row[:3])
        if (w0 & 0xFFFF) == END_OF_STREAM:
            return cls.end_instruction(), 0
        meta = w0 >> 16
        tiles = (w1 & 0xFFFF, w1 >> 16, w2 & 0xFFFF, w2 >> 16)
        return cls(w0 & 0xFFFF, tiles, (meta & 0xF) - 1, ((meta >> 4) & 0xF) - 1 if meta else -1,
                   int(row[4])), int(row[3])

    def logical_tiles(self) -> List[Tuple[int, ...]]:
        """The tiles a (possibly range-owning) instruction covers, in order."""
        if self.op_idx == self.END_MARKER:
            return []
        t = list(_pad(self.tiles))
        if not self.is_range or self.range_end <= t[self.range_axis]:
            return [tuple(self.tiles)]
        out = []
        for v in range(t[self.range_axis], self.range_end):
            t[self.range_axis] = v
            out.append(tuple(t))
        return out


__all__ = ["INSTRUCTION_WORDS", "END_OF_STREAM", "BarrierFormula", "TileInstruction"]
