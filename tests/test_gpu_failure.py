"""Bounded device waits: a wait that can never be satisfied returns an error status, not a hang.

The failure is made on the host (a wait row whose ``expected`` count nobody
reaches); the kernel's waits give up after ``timeout_ms`` and every CTA exits
normally, so the context stays usable.
"""

import pytest
import torch

from machete_b200.kernels.decode_matvec import MatvecSm100Op
from machete_b200.megakernel import Megakernel, MegakernelConfig

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def test_unsatisfiable_wait_times_out_and_context_survives():
    a = torch.randn(1, 1, 256, device="cuda").to(BF)
    w = (torch.randn(256, 256, device="cuda") * 0.02).to(BF)
    mid = torch.zeros(1, 1, 256, dtype=BF, device="cuda")
    out = torch.zeros(1, 1, 256, dtype=BF, device="cuda")
    ops = MatvecSm100Op.schedule(a=a, weight=w, y=mid) + MatvecSm100Op.schedule(a=mid, weight=w, y=out)
    bad = Megakernel(ops, config=MegakernelConfig(timeout_ms=50, fuse=False))
    bad.program.waits["expected"][:] += 1000          # the producer has only 16 units
    with pytest.raises(RuntimeError, match="dependency counter wait timed out"):
        bad.run()
    # the same device context runs a correct program right afterwards
    good = Megakernel(ops, config=MegakernelConfig(fuse=False))
    good.run()
    want = (a.float().view(1, 256) @ w.float().t()).to(BF).float() @ w.float().t()
    assert float((out.float().view(1, 256) - want).abs().max()) < 2e-2
    # and the handle that failed was reset: it reports a clean status again
    assert bad.status()[0] == 0
