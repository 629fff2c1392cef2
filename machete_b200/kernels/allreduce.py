"""Tensor-parallel exchange ops that run inside the megakernel.

``AllReduceSm100Op``: ``y = sum over ranks of x (+ residual_in)`` for the
partial outputs of a K-split (row-parallel) matvec — the O-projection and the
down projection under Megatron-style tensor parallelism.
``AllReduceTop1KeysSm100Op``: element-wise max of the ranks' 64-bit top-1 keys
after a vocabulary-split LM head.

Counterpart of the reference's ``GemmRowParallelOp`` peer reduce-store with
peer barriers (src/machete/kernels/gemm/gemm.py:1253-1363).  The device side
is ``csrc/op_allreduce.cuh``: a one-shot push over peer-mapped inboxes
(``megakernel/peer.py``), summed in rank order so all ranks agree bit for bit.
"""

from __future__ import annotations

import torch

from .. import _native as N
from ..megakernel.lowering import NativeOp, Region, elem_type, meta_of
from ..megakernel.ops import Int64, Op
from ..megakernel.peer import PeerBuffers


def _peer_fields(op: NativeOp, peers: PeerBuffers, n: int, elem: int, units: int, mode: int) -> None:
    half = -(-peers.world_size * n * elem // 16) * 16
    op.s = {N.AR_S_INBOX: peers.alloc(2 * half), N.AR_S_FLAGS: peers.alloc(peers.world_size * units * 4)}
    op.i.update({N.AR_N: n, N.AR_P: peers.world_size, N.AR_RANK: peers.rank, N.AR_MODE: mode,
                 N.AR_EPOCH_BASE: peers.next_epoch_base()})
    for r, ptr in enumerate(peers.ptrs):
        op.p[N.AR_P_PEER0 + r] = ptr
    op.keep.append(peers)


class AllReduceSm100Op(Op):
    """y = sum_r x_r (+ residual_in); x fp32 or 16-bit, y and residual_in 16-bit or fp32."""

    reads = {"x": (None, ("B", "S", "D")), "residual_in": (None, ("B", "S", "D"))}
    writes = {"y": (None, ("B", "S", "D"))}
    tile = ("B", "S")
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, peers: PeerBuffers = None, tile_sizes=None, **tensors):
        if peers is None:
            raise ValueError("AllReduceSm100Op.schedule needs peers=PeerBuffers(...)")
        x, y = tensors["x"], tensors["y"]
        res = tensors.get("residual_in")
        if res is None:
            tensors["residual_in"] = y        # declared input; the lowering sees that it is absent
        if not (x.is_contiguous() and y.is_contiguous()) or x.shape != y.shape:
            raise ValueError("AllReduceSm100Op: x and y must be contiguous (B, S, D) tensors of one shape")
        if x.numel() % 8:
            raise ValueError("AllReduceSm100Op: B*S*D must be a multiple of 8")
        if res is not None and (res.shape != y.shape or not res.is_contiguous()):
            raise ValueError("AllReduceSm100Op: residual_in must match y")
        op = cls._schedule_single(tile_sizes={"B": 1, "S": 1}, **tensors)
        op.static_dims["peers"] = peers
        op.static_dims["has_residual"] = res is not None
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        peers: PeerBuffers = sop.static_dims["peers"]
        x, y = t["x"], t["y"]
        n = x.numel()
        units = -(-n // 256)
        op = NativeOp(name=cls.__name__, opcode=N.OP_ALLREDUCE, n_units=units, kind="allreduce")
        op.i = {N.AR_X_T: elem_type(x, "x"), N.AR_Y_T: elem_type(y, "y"), N.AR_R_T: N.T_BF16}
        op.p = {N.AR_P_X: x.data_ptr(), N.AR_P_Y: y.data_ptr()}
        op.reads = [Region(meta_of(x, "x"))]
        op.keep = [x, y]
        if sop.static_dims.get("has_residual"):
            res = t["residual_in"]
            op.i[N.AR_R_T] = elem_type(res, "residual_in")
            op.p[N.AR_P_RES] = res.data_ptr()
            op.reads.append(Region(meta_of(res, "residual_in")))
            op.keep.append(res)
        op.writes = [Region(meta_of(y, "y"))]
        op.unit_bytes = 0
        _peer_fields(op, peers, n, 8, units, N.AR_SUM)
        return [op]


class AllReduceTop1KeysSm100Op(Op):
    """keys_out[b, s] = max over ranks of keys[b, s]; clears ``keys`` for the next launch."""

    reads = {"top_keys": (Int64, ("B", "S"))}
    writes = {"top_keys_out": (Int64, ("B", "S"))}
    tile = ("B",)
    dynamic_dims = ("B", "S")

    @classmethod
    def schedule(cls, peers: PeerBuffers = None, tile_sizes=None, **tensors):
        if peers is None:
            raise ValueError("AllReduceTop1KeysSm100Op.schedule needs peers=PeerBuffers(...)")
        keys, out = tensors["top_keys"], tensors["top_keys_out"]
        for k in (keys, out):
            if k.dtype != torch.int64 or not k.is_contiguous():
                raise ValueError("top-1 key tensors must be contiguous int64 (B, S)")
        if keys.numel() > 32:
            raise ValueError("the key exchange handles at most 32 rows")
        op = cls._schedule_single(tile_sizes={}, **tensors)
        op.static_dims["peers"] = peers
        return [op]

    @classmethod
    def lower(cls, sop, ctx):
        t = sop.tensor_refs
        peers: PeerBuffers = sop.static_dims["peers"]
        keys, out = t["top_keys"], t["top_keys_out"]
        op = NativeOp(name=cls.__name__, opcode=N.OP_ALLREDUCE, n_units=1, kind="allreduce_keys")
        op.p = {N.AR_P_X: keys.data_ptr(), N.AR_P_Y: out.data_ptr()}
        op.reads = [Region(meta_of(keys, "top_keys"))]
        op.writes = [Region(meta_of(keys, "top_keys")), Region(meta_of(out, "top_keys_out"))]
        op.keep = [keys, out]
        op.unit_bytes = 0
        _peer_fields(op, peers, keys.numel(), 8, 1, N.AR_MAX_KEY)
        return [op]


__all__ = ["AllReduceSm100Op", "AllReduceTop1KeysSm100Op", "PeerBuffers"]
