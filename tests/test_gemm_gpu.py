"""tcgen05 GEMM against a PyTorch fp32 reference of the same op."""
import pytest
import torch

from levanter_b200.ops import gemm as G
from levanter_b200.ops import lib

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * 0.5).to(torch.bfloat16)


def _check(c, ref, K):
    """Per-element bound: the rounding of the output type relative to each element plus an accumulation term that grows with
    sqrt(K) (operands have standard deviation 0.5, so a product has 0.25); a wrong low-magnitude column cannot hide behind the
    largest element of the matrix."""
    c, ref = c.float(), ref.float()
    tol = 2.0 ** -7 * ref.abs() + 2e-5 * (K ** 0.5) + 1e-6
    bad = (c - ref).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} elements off; worst {((c - ref).abs() - tol).max().item():.3e} beyond its bound"


def _check_f32(c, ref, K):
    c, ref = c.float(), ref.float()
    tol = 1e-5 * ref.abs() + 2e-5 * (K ** 0.5) + 1e-6
    bad = (c - ref).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} elements off; worst {((c - ref).abs() - tol).max().item():.3e} beyond its bound"


@pytest.mark.parametrize("M,N,K", [(8192, 11008, 4096), (8192, 32000, 4096)])
def test_gemm_training_shapes_forward(M, N, K):
    torch.manual_seed(3)
    a, b = _rand(M, K), _rand(N, K)
    c = G.gemm(a, b)
    torch.cuda.synchronize()
    lib.check_status()
    for r0 in range(0, M, 2048):  # the fp32 oracle in slabs (a whole fp32 copy of the 32000-column product is 1 GB)
        _check(c[r0:r0 + 2048], a[r0:r0 + 2048].float() @ b.float().t(), K)


def test_gemm_training_shape_weight_gradient_accumulates_in_fp32():
    """dW[N, K] += dY[T, N]^T X[T, K] with T = 8192 tokens, both operands read MN-major, twice into the same fp32 buffer."""
    torch.manual_seed(4)
    T, N, K = 8192, 4096, 4096
    dy, x = _rand(T, N), _rand(T, K)
    acc = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    G.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    G.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
    torch.cuda.synchronize()
    lib.check_status()
    _check_f32(acc, 2.0 * (dy.float().t() @ x.float()), 2 * T)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 264, 200), (1000, 136, 72), (77, 96, 512), (2048, 4096, 1024)])
def test_gemm_matches_fp32(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    if a_mn and (M % 8):
        pytest.skip("MN-major A needs M % 8 == 0 (row stride multiple of 16 bytes)")
    if b_mn and (N % 8):
        pytest.skip("MN-major B needs N % 8 == 0")
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    c = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    lib.check_status()
    ref = G.gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _check(c, ref, K)


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 300, 520, 328
    a, b = _rand(M, K), _rand(N, K)
    bias = _rand(N)
    res = _rand(M, N)
    c = G.gemm(a, b, bias=bias, residual=res, alpha=0.5)
    ref = G.gemm_reference(a, b, bias=bias, residual=res, alpha=0.5, out_dtype=torch.float32)
    _check(c, ref, K)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc0 = acc.clone()
    G.gemm(a, b, out=acc, accumulate=True)
    ref = acc0 + a.float() @ b.float().t()
    _check(acc, ref, K)
    lib.check_status()


def test_linear_autograd():
    torch.manual_seed(2)
    x = _rand(4, 96, 256).requires_grad_()
    w = _rand(384, 256).requires_grad_()
    bias = _rand(384).requires_grad_()
    y = G.linear(x, w, bias)
    g = _rand(4, 96, 384)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    br = bias.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _check(y, yr, 256)
    _check(x.grad, xr.grad, 384)
    _check(w.grad, wr.grad, 384)
    _check(bias.grad, br.grad, 384)
    lib.check_status()


def test_gemm_deterministic():
    a, b = _rand(512, 512), _rand(768, 512)
    c1 = G.gemm(a, b).clone()
    c2 = G.gemm(a, b)
    assert torch.equal(c1, c2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 384), (1024, 128, 2048)])
@pytest.mark.parametrize("a_dt,b_dt", [("e4m3", "e4m3"), ("e5m2", "e4m3")])
def test_fp8_gemm_matches_dequantised_reference(M, N, K, a_dt, b_dt):
    from levanter_b200.ops.fp8 import E4M3, E5M2, fp8_gemm, quantize

    dts = {"e4m3": E4M3, "e5m2": E5M2}
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(N, K, device="cuda")
    aq, sa = quantize(a, dts[a_dt])
    bq, sb = quantize(b, dts[b_dt])
    got = fp8_gemm(aq, bq, sa * sb, out_dtype=torch.float32)
    want = (aq.float() @ bq.float().t()) * (sa * sb)
    torch.cuda.synchronize()
    lib.check_status()
    assert (got - want).abs().max() <= 1e-3 * want.abs().max()
    acc = torch.ones(M, N, device="cuda")
    fp8_gemm(aq, bq, sa * sb, out=acc, accumulate=True)
    assert (acc - 1 - want).abs().max() <= 1e-3 * want.abs().max()


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (1, 6144, 1024), (128, 14336, 512), (17, 136, 200), (100, 32768, 256), (8, 40, 64)])
def test_single_row_block_shapes_use_the_streaming_kernel(M, N, K):
    """M <= 128 (decode, small batches) goes to the weight-streaming kernel: partial A boxes, deep B ring, tiles of 32 to 128 columns."""
    torch.manual_seed(2)
    a, b = _rand(M, K), _rand(N, K)
    bias = _rand(N)
    c = G.gemm(a, b, bias=bias)
    torch.cuda.synchronize()
    lib.check_status()
    ref = a.float() @ b.float().t() + bias.float()
    _check(c, ref, K)
    # residual and fp32 output through the same kernel; rows beyond M of the 128-row MMA must not leak anywhere
    res = _rand(M, N)
    guard = torch.full((M + 8, N), 7.0, device="cuda")
    G.gemm(a, b, residual=res, out=guard[:M])
    torch.cuda.synchronize()
    lib.check_status()
    _check(guard[:M], a.float() @ b.float().t() + res.float(), K)
    assert bool((guard[M:] == 7.0).all())


@pytest.mark.parametrize("M,N,K", [(256, 4096, 4096), (200, 1024, 14336), (512, 6144, 1024), (300, 136, 200), (129, 4096, 512)])
@pytest.mark.parametrize("mode", ["splitk", "stream"])
def test_a_few_row_blocks_with_a_narrow_output(M, N, K, mode, monkeypatch):
    """128 < M <= 512 with few 256-column tiles.  "splitk": the pair kernel with K split over several CTA pairs per tile and
    the partials summed by a second kernel; "stream": the weight-streaming kernel with row blocks of 128 sharing each tile
    of B.  The last row block is partial in both."""
    monkeypatch.setattr(G, "SPLITK_MODE", mode)
    assert G._use_skinny(M, N) == (mode == "stream")
    torch.manual_seed(3)
    a, b = _rand(M, K), _rand(N, K)
    bias = _rand(N)
    c = G.gemm(a, b, bias=bias)
    torch.cuda.synchronize()
    lib.check_status()
    _check(c, a.float() @ b.float().t() + bias.float(), K)
    res = _rand(M, N)
    guard = torch.full((M + 8, N), 7.0, device="cuda")
    G.gemm(a, b, residual=res, out=guard[:M])
    torch.cuda.synchronize()
    lib.check_status()
    _check(guard[:M], a.float() @ b.float().t() + res.float(), K)
    assert bool((guard[M:] == 7.0).all())
    c2 = G.gemm(a, b, bias=bias)
    assert torch.equal(c, c2)  # split-K partials are summed in a fixed order
