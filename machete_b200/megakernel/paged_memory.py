"""Shared-memory layout arithmetic of the reference's page ring, plus this build's own plan.

``NPageLayout`` and ``PipelinePageLayout`` restate the offsets the reference computes for its
ring kernel (src/machete/megakernel/paged_memory.py:270-545): callers and ops size their pages,
semaphores and scratch from these numbers (``Op.pipeline`` resources, ``Megakernel.smem_size``),
so the numbers are part of the host-side contract even though the device loop here lays its own
shared memory out differently.  ``NativeSmemPlan`` is that different layout: control block, staged
activations, then the TMA page ring of the persistent kernel in ``csrc/``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

MAX_PAGES = 16                 # pages (and work slots) the reference ring can address
IQ_DEPTH = 4                   # instruction-queue rows kept in shared memory
INSTRUCTION_ROW_BYTES = 5 * 4  # one reference instruction row: five int32 words

# reference flag words inside the 36-byte flags region (byte offsets; 0 and 8 are unused)
FLAG_DISPATCH_LOAD = 4
FLAG_PRODUCE_IDX = 16
FLAG_STORE_IDX = 20
FLAG_LOAD_DONE = 24
FLAG_DATA_RELEASE_IDX = 28
FLAG_DATA_PRODUCE_IDX = 32

B200_SMEM_OPTIN = 227 * 1024   # opt-in shared memory per CTA on sm_100


def _up(v: int, a: int) -> int:
    return -(-v // a) * a


@dataclass
class NPageLayout:
    """``[tile info 48 B x slots][flags 36 B][instruction queue 4 x 20 B][2 x slots mbarriers]``,
    rounded up to 128 B, then ``num_pages`` pages of ``page_size`` rounded up to 128 B each."""

    num_pages: int = 2
    page_size: int = 16384
    num_slots: Optional[int] = None

    _TILE_INFO_SIZE = 48
    _IQ_ENTRY_SIZE = INSTRUCTION_ROW_BYTES
    _FLAGS_SIZE = 36
    _MBARRIER_SIZE = 8

    def __post_init__(self):
        if self.num_slots is None:
            self.num_slots = self.num_pages
        for what, v in (("num_pages", self.num_pages), ("num_slots", self.num_slots)):
            if v < 1:
                raise ValueError(f"{what} must be >= 1, got {v}")
            if v > MAX_PAGES:
                raise ValueError(f"{what} must be <= {MAX_PAGES}, got {v}")
        self.ring_state_offset = 0
        self.flags_offset = self.num_slots * self._TILE_INFO_SIZE
        self.iq_offset = _up(self.flags_offset + self._FLAGS_SIZE, 8)
        self.mbarrier_offset = _up(self.iq_offset + IQ_DEPTH * self._IQ_ENTRY_SIZE, 8)
        self.scratch_size = _up(self.mbarrier_offset + 2 * self.num_slots * self._MBARRIER_SIZE, 128)
        self.aligned_page_size = _up(self.page_size, 128)
        self.pages_start = self.scratch_size
        self.total_size = self.pages_start + self.num_pages * self.aligned_page_size

    def work_notify_mbar_offset(self, slot_idx: int) -> int:
        return self.mbarrier_offset + slot_idx * self._MBARRIER_SIZE

    def compute_done_mbar_offset(self, slot_idx: int) -> int:
        return self.mbarrier_offset + (self.num_slots + slot_idx) * self._MBARRIER_SIZE

    def page_offset(self, page_idx: int) -> int:
        if not 0 <= page_idx < self.num_pages:
            raise IndexError(f"page {page_idx} out of range for {self.num_pages} pages")
        return self.pages_start + page_idx * self.aligned_page_size

    @classmethod
    def for_device(cls, page_size: int = 16384, max_smem: Optional[int] = None, min_pages: int = 2) -> "NPageLayout":
        """The most pages (at most 16) whose layout fits ``max_smem``; without a GPU the B200's
        227 KB opt-in limit stands in (the reference assumes 228 KB there)."""
        if max_smem is None:
            import torch

            if torch.cuda.is_available():
                max_smem = torch.cuda.get_device_properties(torch.cuda.current_device()).shared_memory_per_block_optin
            else:
                max_smem = B200_SMEM_OPTIN
        most = min((max_smem - (256 + MAX_PAGES * 4)) // _up(page_size, 128), MAX_PAGES)
        if most < min_pages:
            raise ValueError(f"Cannot fit {min_pages} pages of {page_size // 1024}KB in {max_smem // 1024}KB shared memory")
        for n in range(most, min_pages - 1, -1):
            layout = cls(num_pages=n, page_size=page_size)
            if layout.total_size <= max_smem:
                return layout
        return cls(num_pages=min_pages, page_size=page_size)


@dataclass(frozen=True)
class PipelinePageLayout:
    """Storage one op carves out of its page: ``[pages][semaphores, 8 B each][scratch]``."""

    page_count: int
    page_bytes: int
    semaphore_count: int = 0
    scratch_bytes: int = 0

    def __post_init__(self):
        if self.page_count < 1:
            raise ValueError("page_count must be >= 1")
        for what in ("page_bytes", "semaphore_count", "scratch_bytes"):
            if getattr(self, what) < 0:
                raise ValueError(f"{what} must be non-negative")

    pages_offset = 0

    @property
    def semaphores_offset(self) -> int:
        return _up(self.page_count * self.page_bytes, 8)

    @property
    def scratch_offset(self) -> int:
        return _up(self.semaphores_offset + self.semaphore_count * NPageLayout._MBARRIER_SIZE, 16)

    @property
    def total_size(self) -> int:
        return _up(self.scratch_offset + self.scratch_bytes, 128)

    @staticmethod
    def _check(what: str, idx: int, count: int) -> None:
        if not 0 <= idx < count:
            raise IndexError(f"{what} {idx} out of range for {count}")

    def page_offset(self, page_idx: int) -> int:
        self._check("pipeline page", page_idx, self.page_count)
        return page_idx * self.page_bytes

    def activation_page_offset(self) -> int:
        return self.page_offset(0)

    def weight_page_offset(self, *, input_stage: int, page_in_stage: int, input_stages: int, stage_pages: int) -> int:
        self._check("input_stage", input_stage, input_stages)
        self._check("page_in_stage", page_in_stage, stage_pages)
        return self.page_offset(1 + input_stage * stage_pages + page_in_stage)

    def semaphore_offset(self, sem_idx: int) -> int:
        self._check("pipeline semaphore", sem_idx, self.semaphore_count)
        return self.semaphores_offset + sem_idx * NPageLayout._MBARRIER_SIZE

    # semaphore numbering: activations | weights arrived | weights finished | outputs arrived | outputs finished
    @staticmethod
    def activations_arrived_sem() -> int:
        return 0

    @staticmethod
    def weights_arrived_sem(input_stage: int) -> int:
        return 1 + input_stage

    @staticmethod
    def weights_finished_sem(input_stages: int, input_stage: int) -> int:
        return 1 + input_stages + input_stage

    @staticmethod
    def outputs_arrived_sem(input_stages: int, output_stage: int) -> int:
        return 1 + 2 * input_stages + output_stage

    @staticmethod
    def outputs_finished_sem(input_stages: int, output_stages: int, output_stage: int) -> int:
        return 1 + 2 * input_stages + output_stages + output_stage

    def output_scratch_offset(self, *, output_stage: int, output_stages: int) -> int:
        self._check("output_stage", output_stage, output_stages)
        return self.scratch_offset + output_stage * (self.scratch_bytes // max(1, output_stages))


@dataclass(frozen=True)
class NativeSmemPlan:
    """Dynamic shared memory of this build's persistent kernel: ``[control block][staged
    activations][page ring]``.  ``Megakernel`` derives the page count from it."""

    ctrl_bytes: int
    act_bytes: int
    page_bytes: int
    smem_optin: int = B200_SMEM_OPTIN
    max_pages: int = 32

    @property
    def act_offset(self) -> int:
        return self.ctrl_bytes

    @property
    def pages_offset(self) -> int:
        return self.ctrl_bytes + _up(self.act_bytes, 1024)      # TMA-swizzled tiles want 1 KB alignment

    @property
    def num_pages(self) -> int:
        return max(0, min(self.max_pages, (self.smem_optin - self.pages_offset) // self.page_bytes))

    @property
    def total_size(self) -> int:
        return self.pages_offset + self.num_pages * self.page_bytes


__all__ = ["MAX_PAGES", "IQ_DEPTH", "INSTRUCTION_ROW_BYTES", "FLAG_DISPATCH_LOAD", "FLAG_PRODUCE_IDX", "FLAG_STORE_IDX",
           "FLAG_LOAD_DONE", "FLAG_DATA_RELEASE_IDX", "FLAG_DATA_PRODUCE_IDX", "NPageLayout", "PipelinePageLayout",
           "NativeSmemPlan", "B200_SMEM_OPTIN"]
