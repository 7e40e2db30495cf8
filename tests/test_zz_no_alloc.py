"""The allocation-free sort entry point (``bolt_moe_sort_ck_static``).

Some callers of this library cannot allocate device memory at the point where they
sort tokens -- an engine that handed the whole device heap to its own pools at
start-up, or a foreign-language binding with no device allocator.  For them the
library carries the sort's scratch inside its own image.  This test drives that
entry point through the C ABI exactly as such a caller would (inputs and outputs
only) and requires its outputs to equal those of the workspace-taking entry point
bit for bit, on two calls in a row, because the second call finds the first call's
leftovers in the shared scratch.  The file name keeps it last in collection order.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort_both(lib, ptr, tokens, experts, topk, unit, seed, use_mask):
    from boltops_b200 import _cabi
    rng = np.random.default_rng(seed)
    ids = np.argsort(rng.random((tokens, experts)), axis=1)[:, :topk].astype(np.int32)
    wts = rng.random((tokens, topk), dtype=np.float32)
    d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(wts).cuda()
    d_mask = None
    if use_mask:
        mask = np.ones(experts, np.int32)
        mask[2::5] = 0
        d_mask = torch.from_numpy(mask).cuda()
    cap = tokens * topk + experts * unit - topk
    cap_alloc = (cap + unit - 1) // unit * unit
    stream = torch.cuda.current_stream().cuda_stream

    def outputs():
        return (torch.full((cap_alloc,), -7, dtype=torch.int32, device="cuda"),
                torch.full((cap_alloc,), -7.0, dtype=torch.float32, device="cuda"),
                torch.full((cap_alloc // unit,), -7, dtype=torch.int32, device="cuda"),
                torch.full((2 * experts,), -7, dtype=torch.int32, device="cuda"),
                torch.full((1,), -7, dtype=torch.int32, device="cuda"))

    ref = outputs()
    ws_bytes = lib.bolt_moe_sort_workspace_bytes(tokens, topk, experts)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    _cabi.check(lib.bolt_moe_sort_ck(ptr(d_ids), ptr(d_w), ptr(d_mask), tokens, topk, experts, unit,
                                     *(ptr(x) for x in ref), None, None, None, 0, None, 0, ptr(ws), ws_bytes,
                                     stream))
    got = outputs()
    _cabi.check(lib.bolt_moe_sort_ck_static(ptr(d_ids), ptr(d_w), ptr(d_mask), tokens, topk,
                                            experts, unit, *(ptr(x) for x in got), stream))
    torch.cuda.synchronize()
    n = int(ref[4].item())
    assert int(got[4].item()) == n and n > 0
    assert torch.equal(got[0][:n], ref[0][:n])
    assert torch.equal(got[1][:n].view(torch.int32), ref[1][:n].view(torch.int32))
    assert torch.equal(got[2][: n // unit], ref[2][: n // unit])
    assert torch.equal(got[3], ref[3])


def test_static_scratch_sort_matches_workspace_sort_twice_in_a_row():
    from boltops_b200 import _cabi
    lib = _cabi.load()
    ptr = _cabi.ptr
    assert lib.bolt_moe_sort_static_scratch_bytes() == 1 << 20
    # two multi-block problems back to back (the second reuses dirty scratch), then a
    # single-block one, then a masked one
    _sort_both(lib, ptr, 4096, 256, 8, 128, seed=1, use_mask=False)
    _sort_both(lib, ptr, 3000, 128, 8, 128, seed=2, use_mask=False)
    _sort_both(lib, ptr, 64, 8, 2, 128, seed=3, use_mask=False)
    _sort_both(lib, ptr, 9000, 64, 6, 32, seed=4, use_mask=True)


def test_static_scratch_sort_rejects_oversized_requests():
    from boltops_b200 import _cabi
    lib = _cabi.load()
    tokens, topk, experts = 8192, 8, 4096          # needs ~2 MiB of scratch
    assert lib.bolt_moe_sort_workspace_bytes(tokens, topk, experts) > (1 << 20)
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.bolt_moe_sort_ck_static(_cabi.ptr(dummy), _cabi.ptr(dummy), None, tokens, topk,
                                     experts, 128, _cabi.ptr(dummy), _cabi.ptr(dummy),
                                     _cabi.ptr(dummy), _cabi.ptr(dummy), _cabi.ptr(dummy), None)
    assert rc == 1                                  # BOLT_ERR_INVALID, nothing launched
    assert b"scratch" in lib.bolt_last_error()
    torch.cuda.synchronize()
