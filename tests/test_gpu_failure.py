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


def test_aborted_launch_leaves_no_stale_top1_keys():
    """The LM head packs (max, argmax) keys with atomicMax and the finalise op clears them.  When a
    launch aborts in between, the keys of that launch would leak into the next one's maxima; the reset
    after an abort zeroes every scratch buffer the kernel otherwise keeps at zero."""
    from machete_b200.kernels.decode_matvec.top1 import schedule_final_top1_sm100

    g = torch.Generator().manual_seed(3)
    hidden, vocab = 256, 512
    x = torch.randn(1, 1, hidden, generator=g).to(BF).cuda()
    r = torch.randn(1, 1, hidden, generator=g).to(BF).cuda()
    fn = torch.ones(hidden, dtype=BF, device="cuda")
    lm = (torch.randn(vocab, hidden, generator=g) * 0.05).to(BF).cuda()
    tv = torch.zeros(1, 1, device="cuda")
    ti = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    ops = schedule_final_top1_sm100(x=x, residual_in=r, final_norm=fn, lm_head=lm, top_values=tv, top_indices=ti, seq_len=1)
    keys = ops[0].tensor_refs["top_keys"]
    bad = Megakernel(ops, config=MegakernelConfig(timeout_ms=50))
    bad.program.waits["expected"][:] += 1000          # the finalise op never sees the head complete
    with pytest.raises(RuntimeError, match="timed out"):
        bad.run()
    assert int(keys.abs().max()) == 0                 # the head had written them; the reset cleared them
    good = Megakernel(ops)
    good.run()
    want = ((x.float() + r.float()) * torch.rsqrt(((x.float() + r.float()) ** 2).mean(-1, keepdim=True) + 1e-5)
            ).to(BF).float().view(1, hidden) @ lm.float().t()
    assert int(ti.item()) == int(want.argmax()) and int(keys.abs().max()) == 0
