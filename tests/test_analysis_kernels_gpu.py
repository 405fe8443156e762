"""One-pass analysis kernels (tensor summary + histogram, entropy / top-2 gap of logits) against fp32 PyTorch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,dtype", [(1_000_003, torch.float32), (4096 * 333, torch.bfloat16), (17, torch.float32)])
def test_summary_and_histogram(n, dtype):
    from levanter_b200.ops import lib
    from levanter_b200.tracker.histogram import Histogram, sharded_histogram

    x = (torch.randn(n, device="cuda") * 3 + 1).to(dtype)
    n0 = lib.launch_count
    h = Histogram.from_array(x, num_bins=31)
    assert lib.launch_count - n0 == 3  # partial + final summary, bins
    xf = x.float().cpu()
    assert h.min == xf.min().item() and h.max == xf.max().item() and h.num == n
    assert abs(h.sum - xf.double().sum().item()) <= 1e-3 * xf.abs().double().sum().item()
    assert abs(h.sum_squares - (xf.double() ** 2).sum().item()) <= 1e-3 * (xf.double() ** 2).sum().item()
    want, edges = sharded_histogram(xf, bins=31, range=(h.min, h.max), reduce=False)  # the PyTorch statement, on the CPU
    got = torch.from_numpy(h.bucket_counts)
    assert got.sum().item() == n
    # an element within rounding of an edge may fall on either side
    assert (got - want).abs().sum().item() <= max(2, n // 100_000)
    np.testing.assert_allclose(h.bucket_limits, edges.numpy(), rtol=1e-6, atol=1e-6)


def test_constant_tensor_lands_in_one_bin():
    from levanter_b200.tracker.histogram import Histogram

    h = Histogram.from_array(torch.full((1000,), 2.5, device="cuda"), num_bins=8)
    assert h.min == h.max == 2.5 and h.bucket_counts[0] == 1000 and h.bucket_counts.sum() == 1000


@pytest.mark.parametrize("rows,V,dtype", [(64, 32000, torch.bfloat16), (7, 50257, torch.float32), (5, 1003, torch.bfloat16), (3, 2, torch.float32)])
def test_entropy_top2_matches_fp32(rows, V, dtype):
    from levanter_b200.analysis.entropy import entropy_from_logits, top2_gap_from_logits
    from levanter_b200.ops.analysis_kernels import entropy_top2, entropy_top2_reference

    z = (torch.randn(rows, V, device="cuda") * 4).to(dtype)
    z[0, 0] = z[0, V - 1] = 30.0  # a tie for the top: gap 0
    if V > 100:
        z[1, 10:20] = -float("inf")  # masked entries
    ent, gap, lse = entropy_top2(z)
    ent_ref, gap_ref, lse_ref = entropy_top2_reference(z.cpu())
    torch.testing.assert_close(ent.cpu(), ent_ref, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(lse.cpu(), lse_ref, atol=2e-3, rtol=1e-4)
    torch.testing.assert_close(gap.cpu(), gap_ref, atol=0, rtol=0)
    assert gap[0].item() == 0.0
    torch.testing.assert_close(entropy_from_logits(z.view(rows, 1, V)).cpu(), ent_ref.view(rows, 1), atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(top2_gap_from_logits(z).cpu(), gap_ref, atol=0, rtol=0)
