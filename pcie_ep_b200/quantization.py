"""PyTorch reference of the per-token FP8 (E4M3FN) wire format.

These functions are the oracle for the quantisation that the dispatch kernel
performs inside its send warps; they are never on the hot path.  The rules are
the reference's (``pcie_ep/quantization.py:14-44``): one FP32 scale per token,
``scale = amax / 448`` floored at the smallest normal FP32, an all-zero row uses
scale 1, the row is multiplied by the FP32 reciprocal of the scale, saturated
to +-448 and rounded to nearest even; decoding multiplies by the scale and
rounds to BF16.  Inputs must be finite.
"""

from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0


def quantize_fp8_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Return ``(codes uint8 [T,H], scales float32 [T])`` for a floating ``[T,H]`` tensor."""
    if x.ndim != 2 or not x.is_floating_point():
        raise ValueError("FP8 reference expects a floating [T,H] tensor")
    values = x.float()
    amax = values.abs().amax(dim=1) if values.shape[1] else values.new_zeros(values.shape[0])
    floor = torch.finfo(torch.float32).tiny
    scales = torch.where(amax == 0, torch.ones_like(amax), (amax / FP8_MAX).clamp_min(floor))
    normalized = (values * scales.reciprocal().unsqueeze(1)).clamp(-FP8_MAX, FP8_MAX)
    codes = normalized.to(torch.float8_e4m3fn).view(torch.uint8)
    return codes, scales


def dequantize_fp8_reference(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Decode wire bytes with the token scale and round to BF16."""
    if codes.dtype != torch.uint8 or codes.ndim != 2:
        raise ValueError("FP8 codes must be a uint8 [T,H] tensor")
    if scales.shape != codes.shape[:1] or scales.dtype != torch.float32:
        raise ValueError("FP8 scales must be FP32 [T]")
    return (codes.view(torch.float8_e4m3fn).float() * scales.unsqueeze(1)).to(torch.bfloat16)


def fp8_roundtrip_reference(x: torch.Tensor) -> torch.Tensor:
    """What a remote receiver sees for ``x``; local tokens bypass the wire format."""
    return dequantize_fp8_reference(*quantize_fp8_reference(x))
