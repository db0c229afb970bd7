"""tcgen05 grouped expert GEMM against a PyTorch FP32 reference: ragged expert sizes (including empty
experts, sizes that are not multiples of the 128-row tile, aligned gaps), plain and SwiGLU epilogues."""

import pytest
import torch

from pcie_ep_b200.ops.grouped_ffn import grouped_gemm, grouped_gemm_reference, grouped_swiglu_ffn

pytestmark = pytest.mark.gpu


def _layout(counts, alignment=1):
    counts = torch.tensor(counts, dtype=torch.int32)
    padded = (counts + alignment - 1) // alignment * alignment
    offsets = torch.zeros(len(counts) + 1, dtype=torch.int32)
    offsets[1:] = padded.cumsum(0)
    return offsets, counts


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("counts,alignment", [([128], 1), ([5, 0, 300, 129, 1, 0, 77, 256], 1), ([40, 130, 0, 9], 16)])
def test_grouped_gemm_matches_reference(ext, swiglu, counts, alignment):
    torch.manual_seed(0)
    k, n = 256, 384
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
