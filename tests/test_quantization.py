"""FP8 wire-format reference: scale rules, corner rows, error bounds (reference: tests/test_s7.py:19-60)."""

import torch

from pcie_ep_b200 import dequantize_fp8_reference, fp8_roundtrip_reference, quantize_fp8_reference


def test_scale_rules():
    x = torch.zeros(4, 16, dtype=torch.bfloat16)
    x[1, 3] = 448.0
    x[2, 5] = -3.0
    x[3, 0] = 2.0 ** -130  # BF16 subnormal
    codes, scales = quantize_fp8_reference(x)
    assert scales[0] == 1.0                      # all-zero row
    assert scales[1] == 1.0                      # amax 448 -> scale 1
    assert torch.isclose(scales[2], torch.tensor(3.0 / 448.0))
    assert scales[3] == torch.finfo(torch.float32).tiny  # floored at the smallest normal
    assert torch.isfinite(scales.reciprocal()).all()
    back = dequantize_fp8_reference(codes, scales)
    assert back[1, 3] == 448.0 and back[2, 5] == -3.0
    assert not torch.count_nonzero(back[0])


def test_roundtrip_error_bound_and_outliers():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 512, generator=g)
    x[torch.rand(64, 512, generator=g) < 0.01] *= 50.0
    x = x.to(torch.bfloat16)
    back = fp8_roundtrip_reference(x).float()
    amax = x.float().abs().amax(dim=1, keepdim=True)
    # E4M3 has 3 mantissa bits: relative step 2^-3, half-step rounding, plus subnormal floor amax/448 * 2^-9
    bound = x.float().abs() * 2.0 ** -4 + amax / 448.0 * 2.0 ** -9 + 1e-30
    assert ((back - x.float()).abs() <= bound * 1.01 + back.abs() * 2.0 ** -8).all()


def test_shapes_and_type_checks():
    import pytest

    with pytest.raises(ValueError):
        quantize_fp8_reference(torch.zeros(4, dtype=torch.float32))
    with pytest.raises(ValueError):
        quantize_fp8_reference(torch.zeros(4, 4, dtype=torch.int32))
    with pytest.raises(ValueError):
        dequantize_fp8_reference(torch.zeros(4, 4), torch.ones(4))
    with pytest.raises(ValueError):
        dequantize_fp8_reference(torch.zeros(4, 4, dtype=torch.uint8), torch.ones(3))
    codes, scales = quantize_fp8_reference(torch.zeros(0, 8))
    assert codes.shape == (0, 8) and scales.shape == (0,)
