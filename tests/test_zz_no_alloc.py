"""GPU test of haste_targets_bucket_noalloc, the bucketing entry point for callers that cannot allocate device
memory (its per-group counters live in a fixed array inside the library instead of a caller-provided scratch
buffer).  Called through the C ABI twice in a row with different inputs — the second call finds the first call's
leftovers in the shared array — and compared with haste_targets_bucket: the CSR offsets must be identical and
every group must hold the same set of entries (the order inside a group is unspecified for both)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bucket_both(lib, coo, label0, L, G):
    NG = (L + G - 1) // G
    nnz = coo.shape[0]
    st = torch.cuda.current_stream().cuda_stream
    out = []
    for noalloc in (False, True):
        ptr = torch.full((NG + 1,), -1, dtype=torch.int32, device="cuda")
        ent = torch.full((max(nnz, 1),), -1, dtype=torch.int32, device="cuda")
        if noalloc:
            rc = lib.haste_targets_bucket_noalloc(coo.data_ptr(), nnz, label0, L, G, ptr.data_ptr(), ent.data_ptr(), st)
        else:
            scratch = torch.zeros(NG, dtype=torch.int32, device="cuda")
            rc = lib.haste_targets_bucket(coo.data_ptr(), nnz, label0, L, G, ptr.data_ptr(), ent.data_ptr(), scratch.data_ptr(), st)
        assert rc == 0, lib.haste_last_error_string().decode()
        torch.cuda.synchronize()
        out.append((ptr.cpu().numpy(), ent.cpu().numpy().view(np.uint32)))
    return out


def test_noalloc_bucket_matches_allocating_entry_point():
    from haste_b200 import _lib
    lib = _lib.lib
    rs = np.random.RandomState(0)
    # two calls in a row: a large problem first, then a smaller one that reuses (and must re-clear) the array
    for B, L, G, nnz, label0 in ((512, 670091, 128, 2816, 0), (64, 9000, 32, 1500, 4096)):
        rows = rs.randint(0, B, nnz)
        cols = rs.randint(0, L + 2 * label0, nnz)          # some labels fall outside [label0, label0+L)
        coo = torch.tensor(np.stack([rows, cols], 1), dtype=torch.int32, device="cuda")
        (p0, e0), (p1, e1) = _bucket_both(lib, coo, label0, L, G)
        assert np.array_equal(p0, p1)
        NG = (L + G - 1) // G
        n = int(p0[NG])
        assert n == int(((cols >= label0) & (cols < label0 + L)).sum())
        for g in np.nonzero(np.diff(p0))[0]:
            assert sorted(e0[p0[g]:p0[g + 1]]) == sorted(e1[p1[g]:p1[g + 1]])


def test_noalloc_bucket_rejects_too_many_groups():
    from haste_b200 import _lib
    coo = torch.zeros(1, 2, dtype=torch.int32, device="cuda")
    ptr = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = _lib.lib.haste_targets_bucket_noalloc(coo.data_ptr(), 1, 0, 65537 * 16, 16, ptr.data_ptr(), coo.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_TOO_LARGE and "65536" in _lib.last_error()
