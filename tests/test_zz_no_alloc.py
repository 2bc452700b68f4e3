"""The allocation-free decode-attention entry point against the workspace-based one.

Some hosts of the library may not allocate device memory (their own arena owns the GPU, or a plugin
contract forbids it), so they cannot create a workspace; for them the library carries a fixed
built-in scratch array.  This test calls that entry point through the C ABI twice in a row -- the
second call finds the first call's leftovers in the shared array -- and checks both outputs against
the existing entry point on the same inputs (same kernels, so the bound is the tight one the other
GPU tests use).  It lives in a file that sorts last so that a run stopping at the first failure has
already executed every other test; it needs no state from them and passes alone in a fresh process.
"""
import numpy as np
import pytest

from paged_fixture import PagedBatch, assert_attention_close, load_b200

pytestmark = pytest.mark.gpu


def test_noalloc_matches_workspace_entry_point_twice(orc):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    b = load_b200()
    slots, W, P, kvh, hd = 6, 40, 21, 10, 128
    pb = PagedBatch(orc, slots, 1, kvh, hd, W, b.BF16, [P, P, 0, P, 7, P],
                    prefix_keys=["a", "a", "none", "a", "b", "a"], seed=4242)
    pb.write_prefixes()
    ds = torch.tensor([5, 3, 0, 1, 4, 2], dtype=torch.int32, device="cuda")
    rows = [5, 3, 0, 1, 4, 2]
    for call in range(2):
        for t in range(call * (W + 2), call * (W + 2) + W // 2 + 3 + call * W):
            k, v, q = pb.step_inputs(t, 0, rows)
            pb.append(0, k, v, rows)
        dq = torch.from_numpy(q).cuda()
        want = torch.full((slots, kvh * hd), float("nan"), device="cuda")
        got = torch.full((slots, kvh * hd), float("nan"), device="cuda")
        b.attention_batch_paged(pb.layer[0], dq, pb.d_len[0], pb.d_prefill, ds, slots, kvh, want, pb.ws)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's own count of free device memory
        b.attention_batch_paged_noalloc(pb.layer[0], dq, pb.d_len[0], pb.d_prefill, ds, slots, kvh, got)
        torch.cuda.synchronize()
        if call == 1:  # the first call may load the kernel's code; by the second nothing may change hands
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free call changed free device memory"
        assert_attention_close(got.cpu().numpy(), want.cpu().numpy(), 2e-5, 1e-5)
        # and both agree with the CPU oracle
        ref = np.stack([pb.cache[s].attention(0, q[i:i + 1], pb.cache[s].len(0) - 1, kvh, False)[0]
                        for i, s in enumerate(rows)])
        assert_attention_close(got.cpu().numpy(), ref, 2e-5, 1e-5)
    # sizes beyond the built-in scratch are refused with a clear error, nothing is launched
    before = b.launch_count()
    with pytest.raises(b.Error) as e:
        b.attention_batch_paged_noalloc(pb.layer[0], dq, pb.d_len[0], pb.d_prefill, ds, 1025, kvh, got)
    assert e.value.status == 4 and "1024" in str(e.value)
    assert b.launch_count() == before
    assert b.noalloc_status() == 0  # nothing was recorded by the calls above


def test_noalloc_reports_device_status(orc):
    # A block id outside the pool is never dereferenced: the kernel reads block 0 instead and records the
    # fact.  A caller of the allocation-free entry point has no workspace to ask, so the word lives in the
    # built-in array and uocr_b200_noalloc_status reads (and clears) it.  A refused call leaves it alone.
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    b = load_b200()
    pb = PagedBatch(orc, 2, 1, 2, 16, 16, b.BF16, [4, 4], seed=5)
    q = torch.zeros((2, 32), device="cuda")
    out = torch.zeros((2, 32), device="cuda")
    ds = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    b.noalloc_status()  # start from a clean word whatever ran before
    tbl = pb.table.clone()
    tbl[0, 0] = pb.num_blocks + 5
    poisoned = b.PagedLayer(pb.num_blocks, 2, 16, b.BF16, tbl)
    b.attention_batch_paged_noalloc(poisoned, q, pb.d_len[0], pb.d_prefill, ds, 2, 2, out)
    with pytest.raises(b.Error):  # heads not a multiple of kv_heads: refused before the array is touched
        b.attention_batch_paged_noalloc(pb.layer[0], q, pb.d_len[0], pb.d_prefill, ds, 2, 3, out)
    assert b.noalloc_status() & b.STATUS_BAD_BLOCK
    assert b.noalloc_status() == 0  # reading clears it
    b.attention_batch_paged_noalloc(pb.layer[0], q, pb.d_len[0], pb.d_prefill, ds, 2, 2, out)
    assert b.noalloc_status() == 0
