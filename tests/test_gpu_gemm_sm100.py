"""The tcgen05 GEMM tile against a plain fp32 PyTorch product of the same bf16 operands.

Tolerance: the kernel accumulates in fp32 and rounds once to bf16; the reference is computed in
fp32 (fp64 for the bar) from the same bf16 inputs and rounded the same way, so the two may differ by
the accumulation order only: |diff| <= one bf16 ulp of the result magnitude plus K * 2^-24 relative
fp32 accumulation noise.
"""

import pytest
import torch

from machete_b200.kernels.gemm import GemmSm100Op, gemm_sm100

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _ref(a, b):
    return (a.double().view(-1, a.shape[-1]) @ b.double().t())


def _check(a, b, c):
    want = _ref(a, b)
    got = c.double().view(-1, c.shape[-1])
    K = a.shape[-1]
    mag = (a.double().abs().view(-1, K) @ b.double().abs().t())
    bar = want.abs() * 2.0 ** -8 + mag * K * 2.0 ** -24 + 1e-30      # one bf16 rounding + fp32 accumulation
    bad = (got - want).abs() > bar
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} entries outside the bar; max diff {float((got - want).abs().max())}"


@pytest.mark.parametrize("M", [64, 128, 256])
@pytest.mark.parametrize("N_out,K", [(4096, 4096), (1024, 2048)])
def test_headline_shapes(M, N_out, K):
    g = torch.Generator(device="cuda").manual_seed(M + N_out)
    a = torch.randn(1, M, K, generator=g, device="cuda").to(BF)
    b = (torch.randn(N_out, K, generator=g, device="cuda") * 0.05).to(BF)
    c = torch.zeros(1, M, N_out, dtype=BF, device="cuda")
    gemm_sm100(a, b, c, check_status=True)
    _check(a, b, c)


@pytest.mark.parametrize("M,N_out,K,split", [(1, 128, 64, 1), (17, 200, 72, 1), (70, 130, 136, 2), (300, 384, 512, 0),
                                             (64, 256, 1024, 4), (96, 512, 4096, 8), (513, 128, 128, 1)])
def test_ragged_shapes_and_split_k(M, N_out, K, split):
    """Rows, columns and K that are not tile multiples (TMA zero-fills, the epilogue masks), every
    split-K path, and more than 256 rows (several CTAs along M)."""
    g = torch.Generator(device="cuda").manual_seed(7 * M + N_out + K)
    a = torch.randn(M, K, generator=g, device="cuda").to(BF)
    b = torch.randn(N_out, K, generator=g, device="cuda").to(BF)
    c = torch.full((M, N_out), 7.0, dtype=BF, device="cuda")
    gemm_sm100(a, b, c, split_k=split, check_status=True)
    _check(a, b, c)


def test_strided_operands_and_repeat_calls_share_one_workspace():
    g = torch.Generator(device="cuda").manual_seed(5)
    M, N_out, K = 128, 640, 1024
    a_full = torch.randn(M, K + 64, generator=g, device="cuda").to(BF)
    b_full = torch.randn(N_out, K + 8, generator=g, device="cuda").to(BF)
    c_full = torch.zeros(M, N_out + 32, dtype=BF, device="cuda")
    a, b, c = a_full[:, :K], b_full[:, :K], c_full[:, :N_out]
    for _ in range(3):           # the split-K workspace must come back zero after every call
        c_full.zero_()
        gemm_sm100(a, b, c, split_k=4, check_status=True)
        _check(a, b, c)
        assert float(c_full[:, N_out:].abs().max()) == 0.0           # nothing written past the N columns


def test_op_mirror_schedules_and_launches():
    a = torch.randn(2, 64, 256, device="cuda").to(BF)
    b = torch.randn(384, 256, device="cuda").to(BF)
    c = torch.zeros(2, 64, 384, dtype=BF, device="cuda")
    (sop,) = GemmSm100Op.schedule(a=a, b=b, c=c)
    assert sop.tile_counts == (2, 1, 3) and sop.static_dims["tile_K"] == 64
    GemmSm100Op.launch(sop, check_status=True)
    _check(a, b, c)
    # the reference's keywords: tile sizes shape the record, the activation is fused into the epilogue
    (s2,) = GemmSm100Op.schedule(a=a, b=b, c=c, tile_sizes={"S": 64, "N": 64, "K": 64}, activation="silu")
    assert s2.tile_counts == (2, 1, 6) and s2.static_dims["activation"] == 2
    GemmSm100Op.launch(s2, check_status=True)
    want = torch.nn.functional.silu(_ref(a, b))
    assert float((c.double().view(-1, 384) - want).abs().max()) <= float(want.abs().max()) * 2.0 ** -7
    gemm_sm100(a, b, c, activation="relu", split_k=2, check_status=True)
    assert float((c.double().view(-1, 384) - _ref(a, b).clamp_min(0)).abs().max()) <= float(want.abs().max()) * 2.0 ** -7
    with pytest.raises(ValueError):
        GemmSm100Op.schedule(a=a, b=b, c=c, activation="gelu")
    with pytest.raises(NotImplementedError):
        GemmSm100Op.lower(sop, None)


def test_bad_arguments_are_refused():
    a = torch.zeros(64, 100, dtype=BF, device="cuda")       # K not a multiple of 8
    b = torch.zeros(128, 100, dtype=BF, device="cuda")
    c = torch.zeros(64, 128, dtype=BF, device="cuda")
    with pytest.raises(ValueError):
        gemm_sm100(a, b, c)
    with pytest.raises(ValueError):
        gemm_sm100(a.float(), b, c)
    with pytest.raises(ValueError):
        gemm_sm100(torch.zeros(64, 128, dtype=BF, device="cuda"), b, c)
