"""The histogram kernel through its stand-alone C entry point, against a float64 numpy histogram."""
import numpy as np
import pytest

from tests.hist_rows_util import assert_hist_close, call, make_inputs, reference_hist

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,nfeats,nbins,nch,nrows", [(50_000, 100, 64, 3, 50_000), (30_000, 28, 32, 2, 7_001),
                                                       (10_000, 130, 255, 4, 3_333), (5_000, 5, 2, 1, 1), (4_096, 33, 17, 3, 0)])
def test_hist_rows_matches_numpy(pkg, n, nfeats, nbins, nch, nrows):
    import torch
    from evotrees_b200 import _lib
    x, g, rows = make_inputs(n, nfeats, nbins, nch, nrows, seed=n + nfeats)
    rc, got = call(_lib.lib().evb_hist_rows, torch, x, g, rows, nfeats, nbins, nch)
    _lib.check(rc)
    assert_hist_close(got, reference_hist(x, g, rows, nfeats, nbins, nch), g)


def test_hist_rows_rejects_bad_arguments(pkg):
    import torch
    from evotrees_b200 import _lib
    x, g, rows = make_inputs(1000, 10, 16, 3, 100, seed=1)
    rc, _ = call(_lib.lib().evb_hist_rows, torch, x, g, rows, 10, 300, 3)       # nbins > 255
    assert rc == -1
    rc, _ = call(_lib.lib().evb_hist_rows, torch, x, g, rows, 10, 16, 5)        # nch > 4
    assert rc == -1
