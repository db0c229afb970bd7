"""One expert-parallel MoE layer: router -> dispatch -> grouped SwiGLU expert FFN -> weighted combine.

This is the "model" of the framework: the full round trip a transformer's MoE block performs, built
from the three native pieces (fused dispatch kernel, tcgen05 grouped GEMM, fused combine kernel).
The reference project stops at dispatch (no combine: ``pcie_ep/buffers/ep.py:461-462``; no expert
compute: ``docs/pcie-ep/design.md:304``), so this layer has no counterpart there; its expert
ownership and routing conventions are the reference's (rank r owns experts ``[r*E/P, (r+1)*E/P)``,
``topk_idx`` holds global expert ids, -1 marks an unused slot).

Nothing in ``forward`` synchronises with the host: the FFN reads ``expert_offsets`` / ``expert_counts``
on the device and all intermediate buffers are allocated once.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from ..ops.grouped_ffn import grouped_gemm, quantize_weights_fp8
from ..quantization import dequantize_fp8_reference, quantize_fp8_reference


class MoELayer:
    """Expert-parallel SwiGLU MoE layer bound to one ``EPBuffer``.

    Arguments:
        buffer: the EP buffer (any transport); fixes hidden size, top-k, expert count and rank.
        intermediate: expert FFN width.
        seed: weights are random-initialised N(0, 0.02) from this seed (per global expert, so that a
            multi-rank run and a single-process dense reference agree on every expert's weights).
        with_router: also create a router matrix ``[num_experts, hidden]``; without it ``forward`` needs
            ``topk_idx`` / ``topk_weights`` from the caller.
        weights: ``(w_gate_up [local experts, 2*intermediate, hidden], w_down [local experts, hidden, intermediate])``
            already on the device, used instead of drawing new ones (several layers or buffers sharing one set).
    """

    def __init__(self, buffer: Any, intermediate: int, *, seed: int = 0, with_router: bool = True,
                 dtype: torch.dtype = torch.bfloat16, weight_std: float = 0.02,
                 weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> None:
        self.buffer = buffer
        self.hidden = buffer.hidden
        self.intermediate = intermediate
        self.num_experts = buffer.num_experts
        self.num_topk = buffer.num_topk
        self.rank, self.num_ranks = buffer.rank_idx, buffer.num_ranks
        self.local_experts = self.num_experts // self.num_ranks
        self.device = torch.device("cuda", buffer.device) if buffer.on_gpu else torch.device("cpu")
        self.dtype = dtype if buffer.on_gpu else torch.float32
        first = self.rank * self.local_experts
        if weights is not None:
            self.w_gate_up, self.w_down = weights
            if tuple(self.w_gate_up.shape) != (self.local_experts, 2 * intermediate, self.hidden) or \
                    tuple(self.w_down.shape) != (self.local_experts, self.hidden, intermediate):
                raise ValueError("weights do not have the layer's shapes")
        else:
            w13, w2 = [], []
            for e in range(first, first + self.local_experts):
                g = torch.Generator().manual_seed(seed * 1_000_003 + e)
                w13.append(torch.randn(2 * intermediate, self.hidden, generator=g) * weight_std)
                w2.append(torch.randn(self.hidden, intermediate, generator=g) * weight_std)
            self.w_gate_up = torch.stack(w13).to(self.dtype).to(self.device).contiguous()
            self.w_down = torch.stack(w2).to(self.dtype).to(self.device).contiguous()
        self.router = None
        if with_router:
            g = torch.Generator().manual_seed(seed * 1_000_003 + 999_983)
            self.router = (torch.randn(self.num_experts, self.hidden, generator=g) * weight_std).to(self.dtype).to(self.device)
        # FP8 path: the dispatch delivers E4M3 rows + row scales (recv_dtype="fp8_e4m3"); the gate/up GEMM then
        # runs on kind::f8f6f4 with per-output-channel weight scales, the down projection stays BF16.
        self.fp8 = bool(buffer.on_gpu and getattr(buffer.config, "recv_dtype", "bf16") == "fp8_e4m3")
        self.w_gate_up_fp8 = self.w_gate_up_scales = None
        if self.fp8:
            codes, scales = quantize_weights_fp8(self.w_gate_up.float())
            self.w_gate_up_fp8, self.w_gate_up_scales = codes.to(self.device), scales.to(self.device)
        self.fused_combine = bool(getattr(buffer.config, "fused_expert_combine", False))
        self._hidden_rows: Optional[torch.Tensor] = None
        self._out_rows: Optional[torch.Tensor] = None
        self.gemm_status = torch.zeros(4, dtype=torch.int32, device=self.device) if buffer.on_gpu else None

    @staticmethod
    def expert_weights(seed: int, expert: int, hidden: int, intermediate: int, weight_std: float = 0.02):
        """The (gate_up, down) matrices of one global expert, as ``__init__`` draws them."""
        g = torch.Generator().manual_seed(seed * 1_000_003 + expert)
        w13 = torch.randn(2 * intermediate, hidden, generator=g) * weight_std
        w2 = torch.randn(hidden, intermediate, generator=g) * weight_std
        return w13, w2

    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Top-k softmax routing (library matmul: the router is not one of the fused hot paths)."""
        if self.router is None:
            raise RuntimeError("this layer was built without a router")
        logits = (x @ self.router.t()).float()
        top = torch.topk(logits, self.num_topk, dim=1)
        return top.indices.to(torch.int64).contiguous(), torch.softmax(top.values, dim=1).contiguous()

    def _buffers(self, rows: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._hidden_rows is None or self._hidden_rows.shape[0] != rows:
            self._hidden_rows = torch.empty(rows, self.intermediate, dtype=self.dtype, device=self.device)
            # the fused path never materialises the down projection's output
            self._out_rows = None if self.fused_combine else torch.empty(rows, self.hidden, dtype=self.dtype, device=self.device)
        return self._hidden_rows, self._out_rows

    def forward(self, x: torch.Tensor, topk_idx: Optional[torch.Tensor] = None,
                topk_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``y[t] = sum_k w[t,k] * FFN_{idx[t,k]}(x[t])`` for this rank's tokens ``x`` ``[T, hidden]``."""
        if topk_idx is None:
            topk_idx, topk_weights = self.route(x)
        recv_x, _, _, handle, _ = self.buffer.dispatch(x, topk_idx, topk_weights, do_expand=True)
        hidden_rows, out_rows = self._buffers(recv_x.shape[0])
        offsets, counts = handle.expert_offsets, handle.expert_counts
        if self.fp8:
            grouped_gemm(recv_x, self.w_gate_up_fp8, offsets, counts, swiglu=True, out=hidden_rows, status=self.gemm_status,
                         a_scales=handle._result["recv_x_scales"], w_scales=self.w_gate_up_scales)
        else:
            grouped_gemm(recv_x, self.w_gate_up, offsets, counts, swiglu=True, out=hidden_rows, status=self.gemm_status)
        if self.fused_combine:
            # down projection and combine in one pass: the GEMM epilogue writes weighted rows into the owners' memory
            combined, _, _ = self.buffer.fused_expert_combine(hidden_rows, self.w_down, handle)
            return combined
        grouped_gemm(hidden_rows, self.w_down, offsets, counts, swiglu=False, out=out_rows, status=self.gemm_status)
        combined, _, _ = self.buffer.combine(out_rows, handle)
        return combined

    __call__ = forward

    def check_errors(self) -> None:
        """Explicit diagnostic: dispatch/combine error words and the GEMM's wait status."""
        self.buffer.check_errors()
        if self.gemm_status is not None and int(self.gemm_status[0].item()) != 0:
            raise RuntimeError("grouped expert GEMM: a bounded wait expired")


def dense_moe_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, seed: int,
                        hidden: int, intermediate: int, weight_std: float = 0.02,
                        weight_dtype: torch.dtype = torch.bfloat16, fp8: bool = False) -> torch.Tensor:
    """Single-process FP32 evaluation of the same layer (weights rounded to ``weight_dtype`` like the layer's).
    ``fp8``: tokens and gate/up weights go through the same E4M3 quantisation as the FP8 path."""
    out = torch.zeros(x.shape[0], hidden, dtype=torch.float32)
    xf = x.float()
    if fp8:
        xf = (lambda c, s: c.view(torch.float8_e4m3fn).float() * s.unsqueeze(1))(*quantize_fp8_reference(x))
    for e in torch.unique(topk_idx[topk_idx >= 0]).tolist():
        w13, w2 = MoELayer.expert_weights(seed, e, hidden, intermediate, weight_std)
        w13, w2 = w13.to(weight_dtype).float(), w2.to(weight_dtype).float()
        if fp8:
            codes, scales = quantize_weights_fp8(w13.unsqueeze(0))
            w13 = (codes.float() * scales.unsqueeze(2))[0]
        tokens, slots = torch.nonzero(topk_idx == e, as_tuple=True)
        full = xf[tokens] @ w13.t()
        h = torch.nn.functional.silu(full[:, :intermediate]) * full[:, intermediate:]
        out.index_add_(0, tokens, (h @ w2.t()) * topk_weights[tokens, slots].unsqueeze(1))
    return out
