"""CPU checks of two pieces whose kernels need a GPU: the view algebra of the 3-tap convolution (through the GEMM's fp32
statement) and the shape rules that pick a GEMM variant."""
import pytest
import torch
import torch.nn.functional as F

from levanter_b200.ops import conv1d as C
from levanter_b200.ops import gemm as G


@pytest.mark.parametrize("stride", [1, 2])
def test_three_tap_convolution_view_algebra(stride):
    torch.manual_seed(0)
    B, Ci, Co, T = 3, 8, 16, 10
    x = torch.randn(B, Ci, T).bfloat16()
    w = (torch.randn(Co, Ci, 3) * 0.2).bfloat16().requires_grad_()
    b = torch.randn(Co).bfloat16().requires_grad_()
    xp = C.pad_channels_last(x).requires_grad_()
    assert xp.shape == (B, T + 2, Ci) and float(xp[:, 0].abs().max()) == 0 and float(xp[:, -1].abs().max()) == 0
    out = C._Conv3.apply(xp, w, b, stride)  # [rows, Co]: the GEMM over the overlapping-row view (fp32 statement on a CPU)
    per, t_out = (T + 2) // stride, (T // 2 if stride == 2 else T)
    y = torch.as_strided(out, (B, t_out, Co), (per * Co, Co, 1))
    xr, wr, br = x.float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    ref = F.conv1d(xr, wr, br, stride=stride, padding=1).transpose(1, 2)
    assert (y.float() - ref).abs().max() < 0.03
    g = torch.randn_like(ref)
    y.backward(g.bfloat16())
    ref.backward(g)
    assert (w.grad.float() - wr.grad).abs().max() < 0.1
    assert (b.grad.float() - br.grad).abs().max() < 0.05
    assert (xp.grad[:, 1 : T + 1].float().transpose(1, 2) - xr.grad).abs().max() < 0.05


def test_convolution_entry_point_falls_back_off_the_gpu():
    x = torch.randn(2, 8, 12)
    w, b = torch.randn(4, 8, 3), torch.randn(4)
    xp = C.pad_channels_last(x)
    assert not C.kernel_ok(xp, w, 1)
    for stride in (1, 2):
        got = C.conv1d_k3(xp, w, b, stride)
        want = F.conv1d(x, w, b, stride=stride, padding=1).transpose(1, 2)
        assert torch.allclose(got, want, atol=1e-5)


def test_gemm_variant_by_shape():
    # one row block: always the weight-streaming kernel
    assert G._use_skinny(64, 4096) and G._use_skinny(128, 128256)
    # decode-size products with few 256 x 256 tiles and a K worth splitting: the pair kernel with K split
    assert G._use_pair_splitk(256, 4096, 4096) and G._use_pair_splitk(256, 4096, 14336) and G._use_pair_splitk(512, 4096, 4096)
    assert not G._use_pair_splitk(256, 28672, 4096)      # 112 tiles: every SM pair has work already
    assert not G._use_pair_splitk(256, 4096, 512)        # nothing to split
    assert not G._use_pair_splitk(16384, 4096, 4096)     # training shapes
    assert not G._use_skinny(256, 4096)                  # (the row-block streaming variant is opt-in)
