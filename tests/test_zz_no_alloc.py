"""The block-schedule entry point that allocates nothing (built-in scratch array) must give exactly
what the workspace-taking entry point gives.  Some hosts of this library cannot allocate device
memory at the call site - they run under a graph capture, with a frozen pool, or are only ever handed
buffers - so this variant keeps its scratch inside the library.  Collected last on purpose: a run that
stops at the first failure has then already covered every other test.  Works in a fresh process too."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(ids, block, e):
    from alpha_moe_b200 import capi
    dev = ids.device
    numel = ids.numel()
    total = numel + e * (block - 1)
    nb = (total + block - 1) // block

    def outputs():
        return (torch.full((total,), -7, dtype=torch.int32, device=dev),
                torch.full((nb,), -7, dtype=torch.int32, device=dev),
                torch.full((1,), -7, dtype=torch.int32, device=dev))
    ref = outputs()
    ws = torch.empty(max(capi.align_workspace_bytes(numel, e), 4), dtype=torch.uint8, device=dev)
    capi.moe_align_block_size(ids.data_ptr(), numel, e, block, ref[0].data_ptr(), ref[1].data_ptr(),
                              ref[2].data_ptr(), ws.data_ptr(), 0)
    got = outputs()                      # allocated before the call under test, which itself allocates nothing
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    capi.moe_align_block_size_noalloc(ids.data_ptr(), numel, e, block, got[0].data_ptr(), got[1].data_ptr(),
                                      got[2].data_ptr(), 0)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    return ref, got


def test_noalloc_schedule_equals_workspace_schedule_on_two_calls_in_a_row():
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(21)
    # first call: many chunks (fills the built-in scratch); second: fewer chunks and other sizes, so
    # stale contents of the shared array from the first call are still lying around
    for m, e, k, block in ((8192, 257, 9, 64), (700, 37, 9, 16)):
        ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(m)]).to(torch.int32).to(dev)
        ref, got = _run_both(ids, block, e)
        for a, b, name in zip(got, ref, ("sorted_token_ids", "expert_ids", "num_tokens_post_padded")):
            assert torch.equal(a, b), name
        assert int(got[2]) % block == 0 and int(got[2]) >= m * k


def test_noalloc_rejects_what_does_not_fit():
    from alpha_moe_b200 import capi
    dev = torch.device("cuda:0")
    e, numel = 1024, 70 * 1024                       # 70 chunks x 1024 experts > 65536 scratch entries
    ids = torch.zeros(numel, dtype=torch.int32, device=dev)
    out = torch.empty(numel + e * 15, dtype=torch.int32, device=dev)
    with pytest.raises(capi.AlphaMoeError, match="built-in scratch"):
        capi.moe_align_block_size_noalloc(ids.data_ptr(), numel, e, 16, out.data_ptr(), out.data_ptr(),
                                          out.data_ptr(), 0)
