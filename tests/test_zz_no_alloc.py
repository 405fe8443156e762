"""The allocation-free sum-of-squares entry point, called as a C symbol, against the regular entry point.

The file name sorts last on purpose: it must pass on its own and after every other GPU test has used the library."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from levanter_b200.ops import lib

    cdll = lib.load()
    f = cdll.lvb_sumsq_noalloc
    f.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    f.restype = ctypes.c_int
    cdll.lvb_sumsq_noalloc_last_error.restype = ctypes.c_char_p
    cdll.lvb_sumsq_noalloc_max_elems.restype = ctypes.c_longlong
    return cdll, f


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_sumsq_matches_regular_entry_point_twice(dtype):
    from levanter_b200.ops import lib, optim_kernels

    cdll, f = _bind()
    torch.manual_seed(0)
    stream = lib.stream_ptr()
    # two calls in a row on different sizes: the second must not see partial sums of the first (larger) one
    for n in (3_000_001, 12_345):
        x = torch.randn(n, device="cuda", dtype=torch.float32).to(dtype)
        want = optim_kernels.sumsq(x)
        out = torch.full((1,), 7.0, device="cuda", dtype=torch.float32)
        rc = f(x.data_ptr(), n, int(dtype == torch.bfloat16), out.data_ptr(), 0, stream)
        assert rc == 0, cdll.lvb_sumsq_noalloc_last_error()
        torch.cuda.synchronize()
        assert out.item() == want.item()  # same kernels, same grid, fixed reduction order: bitwise equal
        ref = x.float().double().pow(2).sum().item()
        assert abs(out.item() - ref) <= 1e-4 * ref
        # accumulate adds to what is there
        rc = f(x.data_ptr(), n, int(dtype == torch.bfloat16), out.data_ptr(), 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert abs(out.item() - 2 * want.item()) <= 1e-6 * abs(want.item())


def test_noalloc_sumsq_does_not_allocate_and_rejects_bad_sizes():
    from levanter_b200.ops import lib

    cdll, f = _bind()
    x = torch.ones(4096, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert f(x.data_ptr(), 4096, 0, out.data_ptr(), 0, lib.stream_ptr()) == 0  # set-up call
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert f(x.data_ptr(), 4096, 0, out.data_ptr(), 0, lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert out.item() == 4096.0
    too_big = cdll.lvb_sumsq_noalloc_max_elems() + 1
    assert f(x.data_ptr(), too_big, 0, out.data_ptr(), 0, lib.stream_ptr()) == -4
    assert b"exceeds the maximum" in cdll.lvb_sumsq_noalloc_last_error()
    assert f(x.data_ptr(), 0, 0, out.data_ptr(), 0, lib.stream_ptr()) == -1
    assert f(0, 16, 0, out.data_ptr(), 0, lib.stream_ptr()) == -1
