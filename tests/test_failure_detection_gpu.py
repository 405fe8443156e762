"""The time-out path of a device-side wait, without any fault: a flag that nothing sets makes the bounded wait run out; the
kernel reports it through its result and the library's status word, and the CUDA context keeps working."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_context_stays_usable():
    from levanter_b200.ops import lib
    from levanter_b200.parallel.symm import wait_for_flag

    lib.clear_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    reached, last, waited = wait_for_flag(flag, 1, limit_seconds=0.2)
    assert not reached and last == 0 and 0.2 <= waited < 1.0
    with pytest.raises(lib.KernelStatusError, match="flag wait timed out"):
        lib.check_status()
    lib.check_status()  # the status word was cleared by the raise above
    # the context is alive: ordinary work still runs, and a flag that is set is seen at once
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0
    flag.fill_(3)
    reached, last, waited = wait_for_flag(flag, 3, limit_seconds=0.2)
    assert reached and last == 3 and waited < 0.1
    lib.check_status()
