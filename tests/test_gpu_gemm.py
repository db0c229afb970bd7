"""tcgen05 grouped expert GEMM against a PyTorch FP32 reference: ragged expert sizes (including empty
experts, sizes that are not multiples of the 128-row tile, aligned gaps), plain and SwiGLU epilogues."""

import pytest
import torch

from pcie_ep_b200.ops.grouped_ffn import grouped_gemm, grouped_gemm_reference, grouped_swiglu_ffn, quantize_weights_fp8
from pcie_ep_b200.quantization import quantize_fp8_reference

pytestmark = pytest.mark.gpu


def _layout(counts, alignment=1):
    counts = torch.tensor(counts, dtype=torch.int32)
    padded = (counts + alignment - 1) // alignment * alignment
    offsets = torch.zeros(len(counts) + 1, dtype=torch.int32)
    offsets[1:] = padded.cumsum(0)
    return offsets, counts


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("n", [384, 512])  # plain GEMM: 128-column tiles / 256-column tiles
@pytest.mark.parametrize("counts,alignment", [([128], 1), ([5, 0, 300, 129, 1, 0, 77, 256], 1), ([40, 130, 0, 9], 16)])
def test_grouped_gemm_matches_reference(ext, swiglu, n, counts, alignment):
    torch.manual_seed(0)
    k = 256
    offsets, cnts = _layout(counts, alignment)
    rows = int(offsets[-1]) + 37  # spare capacity behind the last expert
    a = (torch.randn(rows, k) * 0.5).to(torch.bfloat16).cuda()
    w = (torch.randn(len(counts), (2 if swiglu else 1) * n, k) * 0.05).to(torch.bfloat16).cuda()
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    grouped_gemm(a, w, offsets.cuda(), cnts.cuda(), swiglu=swiglu, out=out, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    want = grouped_gemm_reference(a.cpu(), w.cpu(), offsets, cnts, swiglu)
    valid = torch.zeros(rows, dtype=torch.bool)
    for e, c in enumerate(counts):
        valid[int(offsets[e]):int(offsets[e]) + c] = True
    got = out.cpu().float()
    assert torch.allclose(got[valid], want[valid], rtol=2e-2, atol=2e-2), (got[valid] - want[valid]).abs().max()
    assert (got[~valid] == 7.0).all(), "rows outside every expert must not be written"


def test_swiglu_ffn_two_stage(ext):
    torch.manual_seed(1)
    hidden, inter = 512, 256
    offsets, cnts = _layout([200, 3, 0, 131])
    rows = int(offsets[-1])
    x = (torch.randn(rows, hidden) * 0.5).to(torch.bfloat16).cuda()
    w13 = (torch.randn(4, 2 * inter, hidden) * 0.03).to(torch.bfloat16).cuda()
    w2 = (torch.randn(4, hidden, inter) * 0.03).to(torch.bfloat16).cuda()
    y = grouped_swiglu_ffn(x, w13, w2, offsets.cuda(), cnts.cuda())
    torch.cuda.synchronize()
    h = grouped_gemm_reference(x.cpu(), w13.cpu(), offsets, cnts, True).to(torch.bfloat16)
    want = grouped_gemm_reference(h, w2.cpu(), offsets, cnts, False)
    assert torch.allclose(y.cpu().float(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_gemm_fp8_matches_dequantised_reference(ext, swiglu):
    """E4M3 operands on kind::f8f6f4 with per-row / per-channel scales in the epilogue: exact w.r.t. the
    quantised operands up to FP32 accumulation order and the BF16 output rounding."""
    torch.manual_seed(2)
    k, n = 512, 256
    counts = [70, 0, 200, 129, 3]
    offsets, cnts = _layout(counts)
    rows = int(offsets[-1]) + 11
    a = torch.randn(rows, k) * 0.7
    a[5] *= 40.0  # an outlier row gets its own scale
    codes, a_scales = quantize_fp8_reference(a)
    a8 = codes.view(torch.float8_e4m3fn)
    w = torch.randn(len(counts), (2 if swiglu else 1) * n, k) * 0.05
    w8, w_scales = quantize_weights_fp8(w)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    grouped_gemm(a8.cuda(), w8.cuda(), offsets.cuda(), cnts.cuda(), swiglu=swiglu, out=out, status=status,
                 a_scales=a_scales.cuda(), w_scales=w_scales.cuda())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    want = grouped_gemm_reference(a8, w8, offsets, cnts, swiglu, a_scales, w_scales)
    valid = torch.zeros(rows, dtype=torch.bool)
    for e, c in enumerate(counts):
        valid[int(offsets[e]):int(offsets[e]) + c] = True
    got = out.cpu().float()
    scale = float(want[valid].abs().max())
    assert torch.allclose(got[valid], want[valid], rtol=2e-2, atol=1e-2 * scale), (got[valid] - want[valid]).abs().max()
    assert (got[~valid] == 7.0).all()
