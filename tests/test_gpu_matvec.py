"""Weight-streaming matvec / small-M GEMM on the GPU against the fp32 oracle.

Parity bar for bf16 math: max-abs error <= 2e-2 and cosine >= 0.999 against
the fp32 oracle on the same seeded inputs (weights ~N(0, 0.02), activations
~N(0, 1)).
"""

import ctypes as C

import pytest
import torch

import oracle
from machete_b200 import _native as N
from machete_b200.kernels.decode_matvec import (MatvecNvfp4Sm120Op, MatvecResidualNvfp4Sm120Op, MatvecResidualSm100Op,
                                                MatvecSm100Op, RmsGateUpSiluNvfp4Sm120Op, RmsGateUpSiluSm100Op)
from machete_b200.kernels.gemm import GemmOp
from machete_b200.megakernel import Megakernel
from machete_b200.quantization import dequantize_nvfp4_weight, quantize_nvfp4_weight
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def seeded(M, O, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(BF)
    w = (torch.randn(O, K, generator=g) * 0.02).to(BF)
    return x, w


def workspace():
    n = int(N.lib().mk_standalone_workspace_bytes())
    return torch.empty(n, dtype=torch.uint8, device="cuda"), n


@pytest.mark.parametrize("M,O,K", [(1, 64, 256), (1, 4096, 4096), (4, 1000, 2048), (16, 1024, 1024),
                                   (32, 520, 512), (1, 14336, 4096), (8, 48, 8192)])
def test_standalone_matvec_bf16(M, O, K):
    x, w = seeded(M, O, K)
    xd, wd = x.cuda(), w.cuda()
    y = torch.full((M, O), float("nan"), dtype=BF, device="cuda")
    ws, n = workspace()
    rc = N.lib().mk_matvec_bf16(wd.data_ptr(), xd.data_ptr(), y.data_ptr(), M, O, K, ws.data_ptr(), n, None)
    N.check(rc, "mk_matvec_bf16")
    torch.cuda.synchronize()
    assert N.workspace_status(ws.data_ptr())[0] == 0, N.workspace_status(ws.data_ptr())[:6]
    assert_parity(y, oracle.matvec(x, w), f"matvec {M}x{O}x{K}")


def test_standalone_matvec_rejects_bad_shapes():
    ws, n = workspace()
    t = torch.zeros(64, dtype=BF, device="cuda")
    lib = N.lib()
    assert lib.mk_matvec_bf16(t.data_ptr(), t.data_ptr(), t.data_ptr(), 33, 16, 64, ws.data_ptr(), n, None) != 0
    assert lib.mk_matvec_bf16(t.data_ptr(), t.data_ptr(), t.data_ptr(), 1, 16, 48, ws.data_ptr(), n, None) != 0
    assert lib.mk_matvec_bf16(None, t.data_ptr(), t.data_ptr(), 1, 16, 64, ws.data_ptr(), n, None) != 0
    assert lib.mk_matvec_bf16(t.data_ptr(), t.data_ptr(), t.data_ptr(), 1, 16, 64, ws.data_ptr(), 128, None) != 0


@pytest.mark.parametrize("fmt", ["f16s32", "e4m3s16"])
@pytest.mark.parametrize("M,O,K", [(1, 256, 2048), (4, 1000, 4096), (16, 64, 256)])
def test_standalone_matvec_nvfp4(fmt, M, O, K):
    x, w = seeded(M, O, K, seed=1)
    if fmt == "f16s32":
        q = quantize_nvfp4_weight(w, group_size=32)
        wfmt = N.W_NVFP4_F16S32
    else:
        q = quantize_nvfp4_weight(w, group_size=16)
        wfmt = N.W_NVFP4_E4M3S16
    truth = x.float() @ dequantize_nvfp4_weight(q).t()
    pk, sc, xd = q.packed.cuda(), q.scales.cuda(), x.cuda()
    y = torch.full((M, O), float("nan"), dtype=BF, device="cuda")
    ws, n = workspace()
    rc = N.lib().mk_matvec_nvfp4(pk.data_ptr(), sc.data_ptr(), C.c_float(q.global_scale), wfmt, xd.data_ptr(),
                                 y.data_ptr(), M, O, K, ws.data_ptr(), n, None)
    N.check(rc, "mk_matvec_nvfp4")
    torch.cuda.synchronize()
    assert_parity(y, truth, f"nvfp4 {fmt} {M}x{O}x{K}")


@pytest.mark.parametrize("B,S,K,Nout,act", [(1, 16, 1024, 1024, None), (2, 4, 512, 384, "relu"), (1, 1, 4096, 4096, "silu"),
                                            (1, 48, 256, 128, None)])
def test_gemm_op(B, S, K, Nout, act):
    x, w = seeded(B * S, Nout, K, seed=2)
    a = x.view(B, S, K).cuda()
    b = w.cuda()
    c = torch.full((B, S, Nout), float("nan"), dtype=BF, device="cuda")
    Megakernel(GemmOp.schedule(a=a, b=b, c=c, activation=act)).run()
    want = oracle.matvec(x, w)
    if act == "relu":
        want = torch.relu(want)
    elif act == "silu":
        want = want * torch.sigmoid(want)
    assert_parity(c.view(B * S, Nout), want, f"GemmOp {B}x{S}x{K}x{Nout} {act}")


def test_strided_weight_and_residual_chain_matches_fused():
    """The reference's down projection: K-blocks of one weight accumulated in place (fused and unfused)."""
    g = torch.Generator().manual_seed(3)
    hid, inter = 256, 1024
    h = torch.randn(1, 1, inter, generator=g).to(BF).cuda()
    wd = (torch.randn(hid, inter, generator=g) * 0.02).to(BF).cuda()
    want = oracle.matvec(h.cpu().view(1, inter), wd.cpu())
    from machete_b200.megakernel import MegakernelConfig

    for fuse in (True, False):
        y = torch.full((1, 1, hid), float("nan"), dtype=BF, device="cuda")
        ops = []
        for blk in range(inter // hid):
            a_blk, w_blk = h[:, :, blk * hid:(blk + 1) * hid], wd[:, blk * hid:(blk + 1) * hid]
            if blk == 0:
                ops += MatvecSm100Op.schedule(a=a_blk, weight=w_blk, y=y)
            else:
                ops += MatvecResidualSm100Op.schedule(a=a_blk, weight=w_blk, residual_in=y, residual_out=y)
        mk = Megakernel(ops, config=MegakernelConfig(fuse=fuse))
        assert len(mk.native_ops) == (1 if fuse else 4)
        mk.run()
        assert_parity(y.view(1, hid), want, f"down-proj chain fuse={fuse}")
        assert (mk.read_counters() == 0).all()


def test_gate_up_silu_bf16_and_nvfp4():
    g = torch.Generator().manual_seed(4)
    hid, inter = 512, 1024
    x = torch.randn(2, 1, hid, generator=g).to(BF)
    nw = (1 + torch.randn(hid, generator=g) * 0.02).to(BF)
    wg = (torch.randn(inter, hid, generator=g) * 0.02).to(BF)
    wu = (torch.randn(inter, hid, generator=g) * 0.02).to(BF)
    y = torch.full((2, 1, inter), float("nan"), dtype=BF, device="cuda")
    Megakernel(RmsGateUpSiluSm100Op.schedule(x=x.cuda(), norm_weight=nw.cuda(), gate_weight=wg.cuda(),
                                             up_weight=wu.cuda(), y=y, eps=1e-5)).run()
    assert_parity(y, oracle.rms_gate_up_silu(x, nw, wg, wu, 1e-5), "gate/up bf16")
    for gs in (32, 16):
        qg, qu = quantize_nvfp4_weight(wg, gs), quantize_nvfp4_weight(wu, gs)
        # paired weights share one global scale in the kernel: re-quantise "up" against gate's scale range
        if gs == 16:
            both = quantize_nvfp4_weight(torch.cat([wg, wu]), gs)
            from machete_b200.quantization import NVFP4Tensor
            qg = NVFP4Tensor(both.packed[:inter].contiguous(), both.scales[:inter].contiguous(), gs, inter, hid,
                             both.global_scale)
            qu = NVFP4Tensor(both.packed[inter:].contiguous(), both.scales[inter:].contiguous(), gs, inter, hid,
                             both.global_scale)
        want = oracle.rms_gate_up_silu(x, nw, dequantize_nvfp4_weight(qg), dequantize_nvfp4_weight(qu), 1e-5)
        y.fill_(float("nan"))
        Megakernel(RmsGateUpSiluNvfp4Sm120Op.schedule(
            x=x.cuda(), norm_weight=nw.cuda(), gate_packed=qg.packed.cuda(), gate_scales=qg.scales.cuda(),
            up_packed=qu.packed.cuda(), up_scales=qu.scales.cuda(), y=y, eps=1e-5, group_size=gs,
            global_scale=qg.global_scale)).run()
        assert_parity(y, want, f"gate/up nvfp4 g{gs}")


def test_nvfp4_matvec_ops_with_residual():
    g = torch.Generator().manual_seed(5)
    a = torch.randn(1, 4, 1024, generator=g).to(BF)
    w = (torch.randn(768, 1024, generator=g) * 0.02).to(BF)
    res = torch.randn(1, 4, 768, generator=g).to(BF)
    q = quantize_nvfp4_weight(w, 32)
    deq = dequantize_nvfp4_weight(q)
    y = torch.full((1, 4, 768), float("nan"), dtype=BF, device="cuda")
    Megakernel(MatvecNvfp4Sm120Op.schedule(a=a.cuda(), weight_packed=q.packed.cuda(), weight_scales=q.scales.cuda(),
                                           y=y)).run()
    assert_parity(y, a.float() @ deq.t(), "MatvecNvfp4")
    r = res.cuda()
    Megakernel(MatvecResidualNvfp4Sm120Op.schedule(a=a.cuda(), weight_packed=q.packed.cuda(),
                                                   weight_scales=q.scales.cuda(), residual_in=r, residual_out=r)).run()
    assert_parity(r, a.float() @ deq.t() + res.float(), "MatvecResidualNvfp4")
