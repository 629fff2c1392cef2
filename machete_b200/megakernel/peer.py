"""Peer-mapped buffers for tensor-parallel ops inside the megakernel.

One process drives one GPU.  ``PeerBuffers`` is a *symmetric* allocation: every
rank of the group allocates the same number of bytes and maps every other
rank's allocation into its own address space, so a kernel on rank ``r`` can
store straight into rank ``q``'s memory over NVLink.  The all-reduce op
(``csrc/op_allreduce.cuh``) carves its inbox and flag regions out of it with
``alloc``; because every rank schedules the same ops in the same order, the
offsets agree without any exchange.

Takes the place of the reference's ``MegakernelConfig.peer_buffers`` /
``peer_barriers`` (src/machete/megakernel/megakernel.py:174-221), which hold
the device pointers of all ranks in ONE process; here the mapping comes from
``torch.distributed._symmetric_memory`` (CUDA IPC / fabric handles) and the
plumbing (rendezvous, barrier) from ``torch.distributed``.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import _native as N


class PeerBuffers:
    """A zero-initialised symmetric byte buffer plus a bump allocator over it.

    Args:
        nbytes: size of the allocation on every rank.
        group: ``torch.distributed`` process group (default: WORLD).
        device: CUDA device of this rank; ``None`` or a CPU device builds a
            table-only instance (offsets and fake non-null pointers) for host
            tests and dry runs.
    """

    def __init__(self, nbytes: int, group=None, device=None, rank: Optional[int] = None,
                 world_size: Optional[int] = None):
        import torch.distributed as dist

        if rank is None or world_size is None:
            if not dist.is_initialized():
                raise RuntimeError("PeerBuffers needs an initialised torch.distributed process group")
            group = group or dist.group.WORLD
            rank, world_size = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= world_size <= N.AR_MAX_RANKS:
            raise ValueError(f"tensor-parallel world size must be 2..{N.AR_MAX_RANKS}, got {world_size}")
        self.rank, self.world_size, self.group = int(rank), int(world_size), group
        self.nbytes = -(-int(nbytes) // 256) * 256
        self._cursor = 0
        self._generation = 0
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.device = dev
        if dev.type == "cuda":
            import torch.distributed._symmetric_memory as symm_mem

            self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=dev)
            self.buffer.zero_()
            handle = symm_mem.rendezvous(self.buffer, group.group_name if group is not None else None)
            self.ptrs: List[int] = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(dev)
            dist.barrier(group)          # every rank's flags are zero before anybody launches
        else:
            self.buffer = torch.zeros(self.nbytes, dtype=torch.uint8)
            base = self.buffer.data_ptr() & ~0xFF or 0x1000
            self.ptrs = [base + (r + 1) * (1 << 32) for r in range(world_size)]   # distinct, aligned, never used
            self.ptrs[self.rank] = self.buffer.data_ptr()

    @classmethod
    def local(cls, nbytes: int, rank: int, world_size: int, device) -> "PeerBuffers":
        """Every rank's buffer as a plain allocation on ONE device (no process group).

        The reference's same-device peer trick (tests/kernels/test_gemm_tp.py:80-113): it lets a
        single GPU lower and run a rank's program, e.g. to see the bounded wait for a peer that
        never writes give up with a status instead of hanging.
        """
        self = cls.__new__(cls)
        self.rank, self.world_size, self.group = int(rank), int(world_size), None
        self.nbytes = -(-int(nbytes) // 256) * 256
        self._cursor = 0
        self._generation = 0
        self.device = torch.device(device)
        self._locals = [torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device) for _ in range(world_size)]
        self.buffer = self._locals[self.rank]
        self.ptrs = [int(t.data_ptr()) for t in self._locals]
        return self

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes`` and return the offset (identical on every rank)."""
        off = -(-self._cursor // align) * align
        if off + nbytes > self.nbytes:
            raise ValueError(f"PeerBuffers exhausted: need {off + nbytes} bytes, have {self.nbytes}")
        self._cursor = off + int(nbytes)
        return off

    def next_epoch_base(self) -> int:
        """A fresh flag epoch base for one lowering of one op (same sequence on every rank).

        Flags written by an earlier program that used the same region are
        below every epoch of the new program (bases step by 2**22 launches).
        """
        self._generation += 1
        return (self._generation << 22) & 0x7FFFFFFF

    @staticmethod
    def bytes_for_model(batch_rows: int, hidden: int, num_layers: int, sums_per_layer: int = 2) -> int:
        """Enough for ``sums_per_layer`` sum all-reduces per layer (two: after the O and the down
        projection; more when the down projection runs as K-blocks) and the final key exchange."""
        per_sum = 2 * N.AR_MAX_RANKS * batch_rows * hidden * 8 + N.AR_MAX_RANKS * ((batch_rows * hidden + 255) // 256) * 4
        return (sums_per_layer * num_layers + 2) * (per_sum + 1024) + 65536
