"""``GemmSm100Op``: ``C[B,S,N] = A[B,S,K] @ W[N,K]^T`` on the tcgen05 tensor cores.

API mirror of the reference's SM100 GEMM op (src/machete/kernels/gemm/gemm_sm100.py:56-658:
``reads a (B,S,K), b (N,K)``, ``writes c (B,S,N)``, ``schedule(tile_sizes=None, page_size, a=, b=,
c=)``).  There the op is a handler inside the interpreter; here it is a launch of its own
(``mk_gemm_bf16`` in ``csrc/gemm_sm100.cu``) next to the decode megakernel, which keeps the
mma.sync matvec units for up to 32 rows.  ``gemm_sm100(a, b, c)`` is the call; ``GemmSm100Op.schedule``
returns the scheduled-op record (tile grid, tensor metadata) and ``GemmSm100Op.launch`` runs it.
"""

from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from ... import _native as N
from ...megakernel.ops import DEFAULT_PAGE_SIZE, Op

TILE_N = 128     # weight rows per CTA
TILE_M = 256     # activation rows per CTA
TILE_K = 64

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = f"{what}: {N.lib().mk_gemm_last_error().decode('utf-8', 'replace')} (code {rc})"
    raise ValueError(msg) if rc in (-2, -3) else RuntimeError(msg)


def gemm_workspace(M: int, N_out: int, K: int, device) -> torch.Tensor:
    """A zeroed workspace for ``gemm_sm100`` (cached per device and size; the kernel leaves it zero)."""
    need = int(N.lib().mk_gemm_bf16_workspace_bytes(M, N_out, K))
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), need)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


class PackedWeight:
    """A weight stored K-tile-major, ``[K/64][N][64]`` (see :func:`gemm_pack_weight`)."""

    def __init__(self, data: torch.Tensor, n: int, k: int):
        self.data, self.n, self.k = data, int(n), int(k)

    @property
    def shape(self):
        return (self.n, self.k)


def gemm_pack_weight(b: torch.Tensor) -> PackedWeight:
    """Offline re-layout of an ``(N, K)`` bf16 weight for ``gemm_sm100``: K is cut into 64-column
    tiles (zero-padded) and each tile stores its 64 columns of every row contiguously, so one
    128-row box of the kernel is one contiguous 16 KB read."""
    if b.dim() != 2 or b.dtype != torch.bfloat16:
        raise ValueError("gemm_pack_weight: an (N, K) bfloat16 matrix is required")
    n, k = int(b.shape[0]), int(b.shape[1])
    kp = -(-k // TILE_K) * TILE_K
    src = b if kp == k else torch.nn.functional.pad(b, (0, kp - k))
    return PackedWeight(src.view(n, kp // TILE_K, TILE_K).permute(1, 0, 2).contiguous(), n, kp)


ACTIVATIONS = {None: 0, "relu": 1, "silu": 2}


def gemm_sm100(a: torch.Tensor, b, c: torch.Tensor, *, activation=None, split_k: int = 0, timeout_ms: int = 1000,
               workspace: Optional[torch.Tensor] = None, check_status: bool = False) -> torch.Tensor:
    """``c[..., N] = a[..., K] @ b[N, K]^T`` (bf16, fp32 accumulate) on the current stream.

    ``a`` and ``c`` may have any leading dims as long as their rows are equally spaced
    (``a.view(-1, K)`` must be a view).  ``check_status`` synchronises and raises if a device-side
    wait ran out.
    """
    if not (a.is_cuda and c.is_cuda):
        raise RuntimeError("gemm_sm100 runs on a CUDA device only; there is no CPU path")
    if activation not in ACTIVATIONS:
        raise ValueError(f"Unknown activation: {activation}")
    packed = isinstance(b, PackedWeight)
    bt = b.data if packed else b
    if not bt.is_cuda:
        raise RuntimeError("gemm_sm100 runs on a CUDA device only; there is no CPU path")
    if a.dtype != torch.bfloat16 or bt.dtype != torch.bfloat16 or c.dtype != torch.bfloat16:
        raise ValueError("gemm_sm100: a, b and c must be bfloat16")
    K, n_out = int(a.shape[-1]), int(b.shape[0])
    if (not packed and b.dim() != 2) or int(b.shape[1]) != K or int(c.shape[-1]) != n_out or a.shape[:-1] != c.shape[:-1]:
        raise ValueError(f"gemm_sm100: shapes a{tuple(a.shape)} b{tuple(b.shape)} c{tuple(c.shape)} do not match"
                         + (" (a packed weight pads K to a multiple of 64: pad the activations too)" if packed else ""))
    if a.stride(-1) != 1 or (not packed and b.stride(-1) != 1) or c.stride(-1) != 1:
        raise ValueError("gemm_sm100: K (a, b) and N (c) must be contiguous")
    a2, c2 = a.view(-1, K), c.view(-1, n_out)          # raises if the rows are not equally spaced
    M = int(a2.shape[0])
    ws = workspace if workspace is not None else gemm_workspace(M, n_out, K, a.device)
    base = (ws.data_ptr() + 255) // 256 * 256
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        if packed:
            _check(N.lib().mk_gemm_bf16_packed(a2.data_ptr(), bt.data_ptr(), c2.data_ptr(), M, n_out, K, a2.stride(0),
                                               c2.stride(0), base, ws.numel() - (base - ws.data_ptr()), int(split_k),
                                               ACTIVATIONS[activation], int(timeout_ms), C.c_void_p(stream)),
                   "mk_gemm_bf16_packed")
        else:
            _check(N.lib().mk_gemm_bf16(a2.data_ptr(), b.data_ptr(), c2.data_ptr(), M, n_out, K, a2.stride(0), b.stride(0),
                                        c2.stride(0), base, ws.numel() - (base - ws.data_ptr()), int(split_k),
                                        ACTIVATIONS[activation], int(timeout_ms), C.c_void_p(stream)), "mk_gemm_bf16")
        if check_status:
            st = (C.c_int32 * 4)()
            _check(N.lib().mk_gemm_bf16_status(C.c_void_p(base), st), "mk_gemm_bf16_status")
            if st[0] != 0:
                torch.cuda.synchronize(a.device)
                ws.zero_()
                raise RuntimeError(f"gemm_sm100 aborted: wait {st[0]} ran out (cta={st[1]}, role={st[2]}, step={st[3]})")
    return c


class GemmSm100Op(Op):
    """The reference's op declaration; execution is a launch of its own (see the module docstring)."""

    reads = {"a": (None, ("B", "S", "K")), "b": (None, ("N", "K"))}
    writes = {"c": (None, ("B", "S", "N"))}
    tile = ("B", "S", "N")
    dynamic_dims = ("B", "S")
    tma_loads = {"a", "b"}
    tma_stores = {"c"}

    @classmethod
    def schedule(cls, tile_sizes=None, page_size=DEFAULT_PAGE_SIZE, activation=None, **tensors):
        """``tile_sizes`` (``S`` in {64, 128, 256}, ``N``, ``K``) shape the scheduled-op record as in the
        reference; the kernel's own tile is fixed (128 weight rows x up to 256 activation rows x 64)."""
        if activation not in ACTIVATIONS:
            raise ValueError(f"Unknown activation: {activation}")
        ts = dict(tile_sizes or {})
        ts.setdefault("B", 1)
        ts.setdefault("S", TILE_M)
        ts.setdefault("N", TILE_N)
        tile_k = ts.pop("K", TILE_K)
        if ts["S"] not in (64, 128, 256):
            raise ValueError(f"GemmSm100Op: tile size S must be 64, 128 or 256, got {ts['S']}")
        op = cls._schedule_single(tile_sizes=ts, **tensors)
        op.static_dims["tile_K"] = tile_k
        op.static_dims["page_size"] = page_size
        if activation is not None:
            op.static_dims["activation"] = ACTIVATIONS[activation]
        op.params["activation"] = activation
        return [op]

    @classmethod
    def kernel_config(cls, ops):
        from ...megakernel import MegakernelConfig

        return MegakernelConfig(page_size=max(op.static_dims.get("page_size", DEFAULT_PAGE_SIZE) for op in ops))

    @classmethod
    def launch(cls, sop, **kw) -> torch.Tensor:
        t = sop.tensor_refs
        return gemm_sm100(t["a"], t["b"], t["c"], activation=sop.params.get("activation"), **kw)

    @classmethod
    def lower(cls, sop, ctx):
        raise NotImplementedError("GemmSm100Op runs as its own launch (GemmSm100Op.launch / gemm_sm100), "
                                  "not as an op of the decode megakernel; use GemmOp for up to 32 rows per pass")


__all__ = ["GemmSm100Op", "gemm_sm100", "gemm_workspace", "gemm_pack_weight", "PackedWeight", "TILE_M", "TILE_N", "TILE_K"]
