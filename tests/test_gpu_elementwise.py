"""Row-wise ops on the GPU against the reference-generated golden fixtures."""

from pathlib import Path

import pytest
import torch

from machete_b200.kernels.activation import AddOp
from machete_b200.kernels.glu import GLUOp
from machete_b200.kernels.qknorm_rope import QKNormRopeOp
from machete_b200.kernels.rms_norm import RMSNormOp
from machete_b200.kernels.rope import RopeOp
from machete_b200.megakernel import Megakernel
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def cases():
    return torch.load(GOLD / "golden_ops.pt", weights_only=False)


def test_rmsnorm_variants(cases):
    n = 0
    for c in cases:
        if c["op"] != "rmsnorm":
            continue
        x, w = c["x"].cuda(), c["weight"].cuda()
        y = torch.empty_like(x)
        Megakernel(RMSNormOp.schedule(x=x, weight=w, y=y, residual=c["residual"], gemma=c["gemma"], eps=c["eps"])).run()
        assert_parity(y, c["y"], f"rmsnorm {x.dtype} residual={c['residual']} gemma={c['gemma']}")
        n += 1
    assert n == 12


def test_fused_add_and_gated_rmsnorm(cases):
    c = next(x for x in cases if x["op"] == "fused_add_rmsnorm")
    x, r, w = c["x"].cuda(), c["residual_in"].cuda(), c["weight"].cuda()
    y, ro = torch.empty_like(x), torch.empty_like(x)
    Megakernel(RMSNormOp.schedule(x=x, weight=w, y=y, residual_in=r, residual_out=ro, eps=c["eps"])).run()
    assert torch.equal(ro.cpu(), c["residual_out"])          # the rounded sum is exact
    assert_parity(y, c["y"], "fused add rmsnorm")
    # in place on the residual stream
    r2 = r.clone()
    Megakernel(RMSNormOp.schedule(x=x, weight=w, y=y, residual_in=r2, residual_out=r2, eps=c["eps"])).run()
    assert torch.equal(r2.cpu(), c["residual_out"])
    # the decode helper with the same contract (x, residual_in, norm_weight -> residual_out, y)
    from machete_b200.kernels.decode_matvec import RmsAddNormSm120Op

    y2, ro2 = torch.empty_like(x), torch.empty_like(x)
    Megakernel(RmsAddNormSm120Op.schedule(x=x, residual_in=r, norm_weight=w, residual_out=ro2, y=y2, eps=c["eps"])).run()
    assert torch.equal(ro2.cpu(), c["residual_out"])
    assert_parity(y2, c["y"], "RmsAddNormSm120Op")
    c = next(x for x in cases if x["op"] == "rmsnorm_gated")
    y = torch.empty_like(x)
    Megakernel(RMSNormOp.schedule(x=c["x"].cuda(), weight=c["weight"].cuda(), gate=c["gate"].cuda(), y=y,
                                  eps=c["eps"])).run()
    assert_parity(y, c["y"], "gated rmsnorm")


def test_rope_and_qknorm_rope(cases):
    for c in cases:
        if c["op"] == "rope":
            q = c["q"].cuda()
            Megakernel(RopeOp.schedule(q=q, cos=c["cos"].cuda(), sin=c["sin"].cuda())).run()
            assert_parity(q, c["y"], f"rope D={q.shape[-1]} D2={c['cos'].shape[1]}")
        elif c["op"] == "qknorm_rope":
            q = c["q"]
            B, S, H, D = q.shape
            # the op works on (M, H, D) rows with row m using cos[m]: run each batch element
            for b in range(B):
                qb = q[b].contiguous().cuda()
                Megakernel(QKNormRopeOp.schedule(q=qb, norm_weight=c["norm_weight"].cuda(), cos=c["cos"].cuda(),
                                                 sin=c["sin"].cuda(), eps=c["eps"])).run()
                assert_parity(qb, c["y"][b], f"qknorm_rope D={D}")


def test_glu_and_add(cases):
    for c in cases:
        if c["op"] != "glu":
            continue
        x = c["x"].cuda()
        y = torch.empty(*x.shape[:-1], x.shape[-1] // 2, dtype=x.dtype, device="cuda")
        Megakernel(GLUOp.schedule(x=x, y=y, activation=c["activation"])).run()
        assert_parity(y, c["y"], f"glu {c['activation']}")
    g = torch.Generator().manual_seed(0)
    a = torch.randn(2, 3, 130, generator=g).bfloat16().cuda()
    b = torch.randn(2, 3, 130, generator=g).bfloat16().cuda()
    y = torch.empty_like(a)
    Megakernel(AddOp.schedule(x=a, add=b, y=y)).run()
    assert torch.equal(y, (a.float() + b.float()).bfloat16())
