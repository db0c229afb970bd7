"""Grouped expert FFN over the expanded dispatch layout.

``grouped_gemm`` multiplies, for every local expert ``e``, the rows
``[expert_offsets[e], expert_offsets[e] + expert_counts[e])`` of ``a`` with that expert's weight matrix,
reading offsets and counts on the device (no host synchronisation).  On a GPU it runs the hand-written
tcgen05/TMEM kernel (``csrc/kernels/expert_gemm.cu``); ``grouped_gemm_reference`` is the plain PyTorch
FP32 statement of the same operation used by the tests and by the CPU transport.

``grouped_swiglu_ffn`` is the expert FFN of a MoE layer: ``(silu(x W_gate^T) * (x W_up^T)) W_down^T``
with the SwiGLU fused into the first GEMM's epilogue.  The reference project has no expert compute
(``docs/pcie-ep/design.md:304``).
"""

from __future__ import annotations

from typing import Optional

import torch


def quantize_weights_fp8(w: torch.Tensor):
    """Per-output-channel E4M3 quantisation of expert weights ``[experts, n, k]``: returns ``(codes float8_e4m3fn,
    scales float32 [experts, n])`` with ``w ~= codes * scales[..., None]`` (scale = amax / 448, 1 for zero rows)."""
    codes = torch.empty(w.shape, dtype=torch.float8_e4m3fn, device=w.device)
    scales = torch.empty(w.shape[:2], dtype=torch.float32, device=w.device)
    for first in range(0, w.shape[0], 8):  # a few experts at a time: the FP32 temporaries stay small
        part = w[first:first + 8].float()
        amax = part.abs().amax(dim=2)
        scale = torch.where(amax == 0, torch.ones_like(amax), amax / 448.0)
        scales[first:first + 8] = scale
        codes[first:first + 8] = (part / scale.unsqueeze(2)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return codes, scales


def grouped_gemm_reference(a: torch.Tensor, w: torch.Tensor, expert_offsets: torch.Tensor, expert_counts: torch.Tensor,
                           swiglu: bool = False, a_scales: Optional[torch.Tensor] = None,
                           w_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
    """FP32 reference; rows outside every expert's valid range are zero.  FP8 operands are dequantised with
    their scales first (``a * a_scales[:, None]``, ``w * w_scales[..., None]``)."""
    if a_scales is not None:
        a = a.float() * a_scales.float().unsqueeze(1)
        w = w.float() * w_scales.float().unsqueeze(2)
    experts = w.shape[0]
    n = w.shape[1] // (2 if swiglu else 1)
    out = torch.zeros(a.shape[0], n, dtype=torch.float32, device=a.device)
    offsets = expert_offsets.tolist()
    counts = expert_counts.tolist()
    for e in range(experts):
        lo, cnt = offsets[e], counts[e]
        if cnt == 0:
            continue
        rows = a[lo:lo + cnt].float()
        full = rows @ w[e].float().t()
        if swiglu:
            gate, up = full[:, :n], full[:, n:]
            full = torch.nn.functional.silu(gate) * up
        out[lo:lo + cnt] = full
    return out


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, expert_offsets: torch.Tensor, expert_counts: torch.Tensor, *,
                 swiglu: bool = False, out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 a_scales: Optional[torch.Tensor] = None, w_scales: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[rows of e] = a[rows of e] @ w[e].T`` (with ``swiglu``: ``silu(gate) * up``, gate rows first in ``w[e]``).

    ``a`` is ``[rows, k]`` BF16, ``w`` ``[experts, n, k]`` (``[experts, 2n, k]`` with ``swiglu``); ``n`` must be a
    multiple of 128 and ``k`` of 64 on the GPU path.  Rows that belong to no expert are left untouched.
    ``status`` (int32 ``[4]``) is set non-zero by the kernel if one of its bounded waits expired.
    With ``float8_e4m3fn`` operands (``kind::f8f6f4`` MMA, ``k`` a multiple of 128) ``a_scales`` ``[rows]`` and
    ``w_scales`` ``[experts, n]`` are applied in the epilogue: per-row and per-output-channel scales factor out
    of the reduction, so this is exact with respect to the quantised operands.
    """
    n = w.shape[1] // (2 if swiglu else 1)
    if not a.is_cuda:
        result = grouped_gemm_reference(a, w, expert_offsets, expert_counts, swiglu, a_scales, w_scales)
        result = result.to(torch.bfloat16 if a_scales is not None else a.dtype)
        if out is not None:
            out.copy_(result)
            return out
        return result
    from .. import _C

    if out is None:
        out = torch.empty(a.shape[0], n, dtype=torch.bfloat16, device=a.device)
    if status is None:
        status = torch.zeros(4, dtype=torch.int32, device=a.device)
    _C.grouped_gemm(a, w, out, expert_offsets, expert_counts, status, swiglu, a_scales, w_scales, 0)
    return out


def grouped_swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, expert_offsets: torch.Tensor,
                       expert_counts: torch.Tensor, *, hidden_buffer: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Expert FFN on expanded rows: ``w_gate_up`` is ``[experts, 2*inter, hidden]`` (gate rows, then up rows),
    ``w_down`` ``[experts, hidden, inter]``.  Two launches; the activation between them is BF16."""
    h = grouped_gemm(x, w_gate_up, expert_offsets, expert_counts, swiglu=True, out=hidden_buffer, status=status)
    return grouped_gemm(h, w_down, expert_offsets, expert_counts, swiglu=False, out=out, status=status)
