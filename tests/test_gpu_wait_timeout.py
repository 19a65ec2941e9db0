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


@pytest.mark.parametrize("which", ["barrier", "exchange_sum", "allreduce", "reduce_scatter"])
def test_cross_gpu_wait_runs_out_when_a_rank_never_arrives(which):
    """The tensor-parallel exchange kernels wait for the other ranks through flag words in peer-mapped memory.  Here
    "rank 1" is a flag array that nothing ever writes (one GPU, no second process): rank 0's wait must run out after
    the given few milliseconds, record {1, rank 0, 90 or 100 + the missing rank, epoch} and return; nothing hangs,
    and `result` is left alone."""
    from alpha_moe_b200 import capi
    assert capi.read_status(reset=True)[0] == 0
    n = 4096
    bufs = [torch.ones(n, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    result = torch.full((n,), 7.0, dtype=torch.bfloat16, device="cuda")
    bp, fp = [b.data_ptr() for b in bufs], [f.data_ptr() for f in flags]
    st = torch.cuda.current_stream().cuda_stream
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    if which == "barrier":
        capi.tp_barrier(fp, 0, 5, st)
    elif which == "exchange_sum":
        capi.tp_exchange_sum(bp, result.data_ptr(), 0, n, 0, fp, 0, 5, st)
    elif which == "allreduce":
        capi.tp_allreduce(bp, n, fp, 0, 5, st)
    else:
        capi.tp_reduce_scatter(bp, n, fp, 0, 5, st)
    t1.record()
    torch.cuda.synchronize()
    assert 2.0 < t0.elapsed_time(t1) < 200.0            # about the 5 ms limit (twice for the two-phase all-reduce)
    code, rank, where, epoch = capi.read_status(reset=True)
    assert code == 1 and rank == 0 and where in (91, 101) and epoch >= 1
    if which == "exchange_sum":
        assert (result == 7.0).all()                     # not written after a run-out wait
    # rank 0 did announce itself to "rank 1": once, and once more for the all-reduce's second phase
    assert int(flags[1][0]) == (2 if which in ("allreduce", "reduce_scatter") else 1)
