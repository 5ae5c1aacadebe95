"""The allocation-free gather entry point (apt_gather_rows_static) against the
workspace-taking one (apt_gather_rows), through the C ABI.

Some callers may not call cudaMalloc at all — a server that planned all of its
device memory up front, a latency-critical loop, a process whose allocator is
locked after start-up. For them the library keeps the gather's scratch in a
fixed device array. This test checks that the two entry points return the
same bytes on two calls in a row (the second one smaller, so that what the
first call left in the shared scratch would show if it were not cleared), and
that an oversized request is refused. The file name makes pytest collect it
last.
"""
import ctypes

import numpy as np
import pytest
import torch

from apt_b200 import _lib
from apt_b200._lib import check, lib

pytestmark = pytest.mark.gpu


def _tables(n, dim, rng):
    feats = torch.from_numpy(rng.standard_normal((n, dim)).astype(np.float32))
    cached = torch.from_numpy(rng.permutation(n)[: n // 3].astype(np.int64))
    pos = -torch.arange(n, dtype=torch.int64) - 2           # row i of the host table
    pos[cached] = torch.arange(cached.numel())                # cached rows point into the device table
    return feats.pin_memory(), feats[cached].contiguous().cuda(), pos.cuda()


def _with_workspace(ids, pos, dev_t, uva_t, status):
    n, rb = ids.numel(), dev_t.shape[1] * 4
    out = torch.empty((n, dev_t.shape[1]), device="cuda")
    nbytes = lib.apt_gather_workspace_bytes(n)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    check(lib.apt_gather_rows(ids.data_ptr(), n, None, pos.data_ptr(), pos.numel(), dev_t.data_ptr(), dev_t.shape[0], rb,
                              uva_t.data_ptr(), uva_t.shape[0], rb, 0, out.data_ptr(), ws.data_ptr(), nbytes,
                              status.data_ptr(), None))
    return out


def _static(ids, pos, dev_t, uva_t, status):
    n, rb = ids.numel(), dev_t.shape[1] * 4
    out = torch.empty((n, dev_t.shape[1]), device="cuda")
    check(lib.apt_gather_rows_static(ids.data_ptr(), n, pos.data_ptr(), pos.numel(), dev_t.data_ptr(),
                                     dev_t.shape[0], rb, uva_t.data_ptr(), uva_t.shape[0], rb, 0, out.data_ptr(),
                                     status.data_ptr(), None))
    return out


def test_static_gather_matches_workspace_gather_twice():
    rng = np.random.default_rng(123)
    n, dim = 20000, 128
    uva_t, dev_t, pos = _tables(n, dim, rng)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rows in (50000, 777):   # the second call reuses the scratch the first one filled
        ids = torch.from_numpy(rng.integers(0, n, rows).astype(np.int64)).cuda()
        want = _with_workspace(ids, pos, dev_t, uva_t, status)
        got = _static(ids, pos, dev_t, uva_t, status)
        torch.cuda.synchronize()
        assert torch.equal(got, want)                        # byte copies: exact
        assert torch.equal(got.cpu(), uva_t[ids.cpu()])
    assert int(status.item()) == 0


def test_static_gather_allocates_nothing():
    # the point of the entry point: once the library's device image is loaded (first call), a call
    # changes neither the free device memory nor what PyTorch's allocator holds
    rng = np.random.default_rng(5)
    n, dim, rows = 5000, 64, 30000
    uva_t, dev_t, pos = _tables(n, dim, rng)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ids = torch.from_numpy(rng.integers(0, n, rows).astype(np.int64)).cuda()
    out = torch.empty((rows, dim), device="cuda")
    rb = dim * 4

    def call():
        check(lib.apt_gather_rows_static(ids.data_ptr(), rows, pos.data_ptr(), pos.numel(), dev_t.data_ptr(),
                                         dev_t.shape[0], rb, uva_t.data_ptr(), uva_t.shape[0], rb, 0, out.data_ptr(),
                                         status.data_ptr(), None))
        torch.cuda.synchronize()

    call()                                   # loads the device image if this process has not yet
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before and torch.cuda.memory_reserved() == reserved_before
    assert torch.equal(out.cpu(), uva_t[ids.cpu()]) and int(status.item()) == 0


def test_static_gather_refuses_more_rows_than_its_scratch_holds():
    limit = lib.apt_gather_static_max_rows()
    assert limit == 1 << 20
    st = lib.apt_gather_rows_static(None, limit + 1, None, 10, None, 0, 16, None, 0, 16, 0, None, None, None)
    assert st == _lib.APT_ERR_CAPACITY
    assert b"exceed the built-in scratch" in lib.apt_last_error()
