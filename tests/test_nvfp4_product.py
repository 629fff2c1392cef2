"""The product's NVFP4 quantiser (machete_b200.quantization) is bit-exact, on the CPU.

Two layouts: the reference's (fp16 scale per 32 values) against the vectors its own quantiser
produced (tests/golden/golden_nvfp4.pt, written by tests/golden/make_golden.py), and the
block-scaled one (e4m3 scale per 16 values + fp32 global scale) against the oracle's restatement.
"""

from pathlib import Path

import pytest
import torch

import oracle
from machete_b200.quantization import NVFP4Tensor, dequantize_nvfp4_weight, quantize_nvfp4_weight

GOLD = Path(__file__).parent / "golden"


def test_reference_layout_matches_the_reference_quantiser_bit_for_bit():
    cases = torch.load(GOLD / "golden_nvfp4.pt", weights_only=False)
    assert len(cases) >= 3
    for c in cases:
        q = quantize_nvfp4_weight(c["weight"], group_size=c["group_size"])
        assert q.packed.dtype == torch.uint8 and q.scales.dtype == torch.float16
        assert torch.equal(q.packed, c["packed"]), "packed codes differ from the reference's"
        assert torch.equal(q.scales, c["scales"]), "scales differ from the reference's"
        assert torch.equal(dequantize_nvfp4_weight(q), c["dequant"]), "dequantised values differ"
        # the dataclass built from raw tensors decodes the same way
        again = NVFP4Tensor(c["packed"], c["scales"], c["group_size"])
        assert torch.equal(dequantize_nvfp4_weight(again), c["dequant"])


@pytest.mark.parametrize("rows,cols,seed,dtype", [(16, 512, 3, torch.float32), (48, 4096, 4, torch.bfloat16),
                                                  (7, 64, 5, torch.float16)])
def test_block_scaled_layout_matches_the_oracle_bit_for_bit(rows, cols, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(rows, cols, generator=g) * 0.02).to(dtype)
    w[0, :16] = 0                                       # an all-zero block
    w[1, 5] = w.abs().max() * 4                         # an outlier that sets the global scale
    q = quantize_nvfp4_weight(w, group_size=16)
    packed, scales, gs = oracle.quantize_nvfp4_e4m3(w)
    assert q.scales.dtype == torch.float8_e4m3fn and q.group_size == 16
    assert torch.equal(q.packed, packed)
    assert torch.equal(q.scales.view(torch.uint8), scales.view(torch.uint8))
    assert q.global_scale == gs
    assert torch.equal(dequantize_nvfp4_weight(q), oracle.dequantize_nvfp4(packed, scales, 16, gs))


def test_ties_and_sign_follow_bucketize():
    """A value exactly on a threshold takes the lower code (bucketize, right=False); the sign is bit 3."""
    vals = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0])   # amax 6 -> scale exactly 1: the thresholds themselves
    w = torch.cat([vals, -vals, torch.zeros(16)]).reshape(1, 32)
    q = quantize_nvfp4_weight(w, group_size=32)
    codes = torch.stack([q.packed[0] & 0xF, q.packed[0] >> 4], dim=1).reshape(-1)[:16].tolist()
    assert codes[:8] == [0, 1, 2, 3, 4, 5, 6, 7]
    assert codes[8:] == [8 | c for c in codes[:8]]
