"""The run-out path of the bounded device waits, exercised without stalling any product kernel: a self-test kernel
built from the same wait helper waits (for about a millisecond) on an mbarrier that nothing arrives on.  The wait
must give up, record where it gave up in the status word, release the CTA's other waiter through the abort flag, and
the kernel must return with the context intact (nothing traps, nothing faults)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_through_the_status_word_and_the_kernel_returns():
    from alpha_moe_b200 import capi
    assert capi.read_status(reset=True)[0] == 0
    res = torch.full((2,), 7, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    capi.selftest_wait_timeout(2_000_000, 33, 5, res.data_ptr(), torch.cuda.current_stream().cuda_stream)
    t1.record()
    torch.cuda.synchronize()                       # returns: the kernel did not hang
    assert res.tolist() == [0, 0]                  # both waits gave up: the first on its limit, the second on the abort flag
    assert 0.3 < t0.elapsed_time(t1) < 100.0       # about 2M cycles, far below the product's one-second limit
    code, block, where, it = capi.read_status(reset=True)
    assert (code, block, where, it) == (1, 0, 33, 5)
    assert capi.read_status()[0] == 0              # reading with reset cleared it
    # the context is still usable: an ordinary launch of the library works afterwards
    from oracle import moe_oracle as orc
    from tests.harness import check_close, run_capi
    case = orc.make_case(8, 512, 128, 16, 2, seed=0)
    check_close(run_capi(case, 16), orc.run_oracle(case, 16), tag="after the self-test")


def test_selftest_rejects_limits_that_would_stall_the_gpu():
    from alpha_moe_b200 import capi
    res = torch.zeros(2, dtype=torch.int32, device="cuda")
    for bad in (0, 999, 2_000_000_000):
        with pytest.raises(capi.AlphaMoeError):
            capi.selftest_wait_timeout(bad, 1, 1, res.data_ptr())
    with pytest.raises(capi.AlphaMoeError):
        capi.selftest_wait_timeout(10000, 1, 1, 0)
