"""srf_sample_offsets_static: the scan for callers that may not allocate device memory (its scratch is a
fixed array inside the library).  Called through the C-ABI twice in a row and compared with
srf_sample_offsets, which keeps its scratch in a context buffer.  Integer work: results must be identical.
This file sorts last on purpose, so a run that stops at the first failure has already run everything else."""
import ctypes as C

import numpy as np
import pytest

from sphericalrf_b200 import abi

from helpers import make_renderer, small_scene

pytestmark = pytest.mark.gpu


def test_static_scratch_scan_matches_context_scan_twice(built_lib):
    import torch
    dev = torch.device("cuda", 0)
    sc = small_scene(kind="blobs", width=16, height=8)
    r = make_renderer(sc)                       # only the comparison entry point needs a context
    rng = np.random.default_rng(11)
    err = C.create_string_buffer(256)
    for n in (1, 2047, 2048, 2049, 300_001, 5_000_000):      # two calls in a row, and then some, sharing the array
        counts_h = rng.integers(0, 3000, size=n, dtype=np.uint32)
        counts = torch.from_numpy(counts_h.astype(np.int32)).to(dev)
        want = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        got = torch.full((n + 1,), -1, dtype=torch.int64, device=dev)
        assert built_lib.srf_sample_offsets(r.ctx, counts.data_ptr(), n, want.data_ptr(), None) == abi.OK
        st = built_lib.srf_sample_offsets_static(0, counts.data_ptr(), n, got.data_ptr(), None, err, 256)
        assert st == abi.OK, err.value
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        ref = np.concatenate([[0], np.cumsum(counts_h.astype(np.int64))])
        assert np.array_equal(got.cpu().numpy(), ref)
    # beyond the stated maximum: refused with a clear message, nothing launched
    st = built_lib.srf_sample_offsets_static(0, counts.data_ptr(), (1 << 25) + 1, got.data_ptr(), None, err, 256)
    assert st == abi.ERR_CAPACITY and b"33554432" in err.value
