"""evb_hist_rows_noalloc: the histogram entry point for callers that must not allocate device memory.

Some users of this library cannot call cudaMalloc while they run: a service that promised its host framework
to stay inside a fixed memory pool, a plug-in called between the capture-safe phases of a larger pipeline, or
code that must avoid the device-wide synchronisation an allocation implies.  For them the library offers one
entry point whose work memory is a fixed block inside the library image.  This test calls it through the C ABI
twice in a row (different problems, so the second call sees the first call's leftovers in the shared block) and
checks each result against the allocating entry point `evb_hist_rows`, with the tolerance used by the other
histogram tests (1e-5 of the bound of sum|contribution| per bin), and against a float64 numpy histogram.

The file name sorts last on purpose: with `pytest -x` every other test has already run when this one starts.
"""
import numpy as np
import pytest

from tests.hist_rows_util import assert_hist_close, call, make_inputs, reference_hist

pytestmark = pytest.mark.gpu

PROBLEMS = [(60_000, 100, 64, 3, 45_000, 11), (20_000, 28, 32, 2, 20_000, 12)]


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(pkg):
    import torch
    from evotrees_b200 import _lib
    lib = _lib.lib()
    for n, nfeats, nbins, nch, nrows, seed in PROBLEMS:           # two calls in a row on the same GPU
        x, g, rows = make_inputs(n, nfeats, nbins, nch, nrows, seed)
        rc_a, want = call(lib.evb_hist_rows, torch, x, g, rows, nfeats, nbins, nch)
        _lib.check(rc_a)
        rc_b, got = call(lib.evb_hist_rows_noalloc, torch, x, g, rows, nfeats, nbins, nch)
        _lib.check(rc_b)
        assert_hist_close(got, want, g)                            # against the existing entry point
        assert_hist_close(got, reference_hist(x, g, rows, nfeats, nbins, nch), g)
    # same problem again: the block still holds the previous call's partial images
    n, nfeats, nbins, nch, nrows, seed = PROBLEMS[0]
    x, g, rows = make_inputs(n, nfeats, nbins, nch, nrows, seed)
    rc, again = call(lib.evb_hist_rows_noalloc, torch, x, g, rows, nfeats, nbins, nch)
    _lib.check(rc)
    assert_hist_close(again, reference_hist(x, g, rows, nfeats, nbins, nch), g)


def test_noalloc_leaves_the_free_device_memory_untouched(pkg):
    """The promise itself: with the inputs and the output already on the device, a call changes nothing about the free
    device memory -- neither while it runs (nothing it could have allocated is left behind) nor afterwards."""
    import ctypes as C
    import torch
    from evotrees_b200 import _lib
    lib = _lib.lib()
    n, nfeats, nbins, nch, nrows, seed = PROBLEMS[1]
    x, g, rows = make_inputs(n, nfeats, nbins, nch, nrows, seed)
    dev = torch.device("cuda", 0)
    xd, gd = torch.from_numpy(x).to(dev), torch.from_numpy(g).to(dev)
    rd = torch.from_numpy(rows.view(np.int32)).to(dev)
    out = torch.zeros((nfeats, nch, nbins), dtype=torch.float64, device=dev)

    def run():
        return lib.evb_hist_rows_noalloc(C.c_int32(0), C.c_void_p(0), C.c_void_p(xd.data_ptr()), C.c_int64(n), C.c_int32(nfeats),
                                         C.c_int32(x.shape[1]), C.c_int32(nbins), C.c_void_p(gd.data_ptr()), C.c_int32(nch),
                                         C.c_void_p(rd.data_ptr()), C.c_int64(rows.size), C.c_void_p(out.data_ptr()))

    _lib.check(run())                       # first call on the device (address look-up, kernel attributes)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0]
    _lib.check(run())
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_before


def test_noalloc_rejects_sizes_beyond_its_block(pkg):
    import torch
    from evotrees_b200 import _lib
    x, g, rows = make_inputs(64, 1025, 4, 1, 10, seed=3)            # 1025 features > the built-in limit of 1024
    rc, _ = call(_lib.lib().evb_hist_rows_noalloc, torch, x, g, rows, 1025, 4, 1)
    assert rc == -7
    assert "limit" in _lib.lib().evb_last_error().decode()
