"""PyTorch oracle of the per-token FP8 (E4M3FN) wire format.

Parity: ``pcie_ep/quantization.py:14-44`` of the reference (same three functions, bit-identical results).
The dispatch kernel quantises inside its send warps; these functions say what it must produce and are
never on the hot path.  Format: one FP32 scale per token, ``scale = amax / 448`` but never below the
smallest normal FP32 and exactly 1 for an all-zero row; a value is multiplied by the FP32 reciprocal of
the scale, clamped to +-448 and rounded to nearest even; decoding multiplies by the scale and rounds to
BF16.  Inputs must be finite.
"""

from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0


def quantize_fp8_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x`` floating ``[T, H]`` -> ``(codes uint8 [T, H], scales float32 [T])``."""
    if not (x.ndim == 2 and x.is_floating_point()):
        raise ValueError(f"expected a floating [tokens, hidden] tensor, got {x.dtype} with {x.ndim} dims")
    rows = x.to(torch.float32)
    peak = rows.abs().amax(dim=1) if rows.shape[1] > 0 else rows.new_zeros(rows.shape[0])
    smallest = torch.finfo(torch.float32).tiny
    scales = torch.where(peak == 0, torch.ones_like(peak), (peak / FP8_MAX).clamp_min(smallest))
    scaled = (rows * (1.0 / scales).unsqueeze(1)).clamp(min=-FP8_MAX, max=FP8_MAX)
    return scaled.to(torch.float8_e4m3fn).view(torch.uint8), scales


def dequantize_fp8_reference(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Wire bytes and token scales -> BF16 rows."""
    if not (codes.dtype == torch.uint8 and codes.ndim == 2):
        raise ValueError(f"codes: expected uint8 [tokens, hidden], got {codes.dtype} with {codes.ndim} dims")
    if not (scales.dtype == torch.float32 and tuple(scales.shape) == (codes.shape[0],)):
        raise ValueError(f"scales: expected float32 [{codes.shape[0]}], got {scales.dtype} {tuple(scales.shape)}")
    return (codes.view(torch.float8_e4m3fn).to(torch.float32) * scales.unsqueeze(1)).to(torch.bfloat16)


def fp8_roundtrip_reference(x: torch.Tensor) -> torch.Tensor:
    """What a remote receiver decodes for ``x`` (local tokens bypass the wire format unless rows stay FP8)."""
    codes, scales = quantize_fp8_reference(x)
    return dequantize_fp8_reference(codes, scales)
