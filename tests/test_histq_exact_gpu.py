"""The fixed-point histogram path (mse, one target, all features): every histogram of the tree must be EXACTLY the sum
of the quantised gradients q = rint(g * 2^s) of the node's rows times 2^-s -- for built nodes (integer partial sums),
for siblings (parent - built child in f64, exact for multiples of 2^-s) and on any number of row pieces.  The check is
bit-for-bit on float64, for unit weights (row count riding in the low word) and with weights (four words)."""
import math
import os

import numpy as np
import pytest

from tests.parity import make_regression

pytestmark = pytest.mark.gpu


def _quantise(v: np.ndarray, bits: int):
    m = float(np.abs(v).max())
    _, e = math.frexp(m)
    sc = np.float32(2.0 ** (bits - e))
    q = np.rint((v.astype(np.float32) * sc).astype(np.float32)).astype(np.int64)   # __float2int_rn: half to even
    return q, 2.0 ** (e - bits)


def _depth(n):
    return int(n).bit_length()


@pytest.mark.parametrize("weighted", [False, True])
# shapes: the headline's 3 full units + a 4-feature unit; two units with a short second one and several sub-piece flushes per
# CTA; one short unit with 255 bins; more than 128 features (several CTA groups per row range); more rows than 148 pieces of
# 2^17 rows can hold (the row ranges are doubled)
@pytest.mark.parametrize("nobs,nfeats,nbins,depth", [(60_000, 100, 64, 6), (300_000, 37, 32, 5), (5_000, 9, 255, 4),
                                                     (40_000, 150, 16, 4), (20_000_000, 4, 8, 3)])
def test_histograms_are_exact_sums_of_quantised_gradients(pkg, nobs, nfeats, nbins, depth, weighted):
    from evotrees_b200 import _lib
    from evotrees_b200.fit import init_target
    x, y = make_regression(nobs, nfeats, seed=nobs % 97)
    rng = np.random.default_rng(7)
    params = pkg.EvoTreeRegressor(loss="mse", nrounds=1, max_depth=depth, nbins=nbins, eta=0.3, min_weight=1.0)
    edges, _, _ = pkg.get_edges(x, nbins, rng)
    x_bin = pkg.binarize(x, edges, 0)
    K, yd, ycols, mu, _, _ = init_target("mse", y, None)
    w = rng.uniform(0.25, 3.0, nobs).astype(np.float32) if weighted else None
    flags = _lib.FLAG_FULL_PARTITION | _lib.FLAG_KEEP_ALL_HIST
    cache = pkg.init_core_binned(params, x_bin, yd, ycols, K, mu, w, None, None, 0, flags)
    try:
        js = np.arange(1, nfeats + 1, dtype=np.uint32)
        t = pkg.grow_tree(cache, params, None, js, update_grads=True)
        nid = cache.nidx(from_partition=True).astype(np.int64)
        # first-round gradients as the device computes them (float32): g = 2 (p - y) w
        w32 = np.ones(nobs, np.float32) if w is None else w
        g = (np.float32(2.0) * (np.float32(mu[0]) - yd.astype(np.float32))).astype(np.float32) * w32
        # unweighted: the registers-direct kernel quantises to 24 bits (26 when asked to, or when the staged kernel runs)
        qb = 26 if os.environ.get("EVB_HIST_Q2") == "0" or os.environ.get("EVB_Q2_QBITS") == "26" else 24
        qg, ginv = _quantise(g, 29 if weighted else qb)
        if weighted:
            qw, winv = _quantise(w32, 29)
        else:
            qw, winv = np.ones(nobs, np.int64), 1.0
        nn = t.feat.size
        checked = 0
        for n in range(1, 2 ** (depth - 1)):
            if n != 1 and not t.split[(n >> 1) - 1]:
                continue                                   # not a node of this tree
            d = _depth(n)
            rows = np.nonzero((nid >> (np.vectorize(_depth)(nid) - d).clip(0)) == n)[0] if n > 1 else np.arange(nobs)
            rows = rows[np.vectorize(_depth)(nid[rows]) >= d]
            if rows.size == 0:
                continue
            hg = cache.hist(n, nfeats, nbins)              # [feature, bin, (g, h, w)]
            for f in sorted({0, nfeats // 2, nfeats - 1}):
                b = x_bin[rows, f].astype(np.int64) - 1
                sg = np.zeros(nbins, np.int64); np.add.at(sg, b, qg[rows])
                sw = np.zeros(nbins, np.int64); np.add.at(sw, b, qw[rows])
                if weighted and nbins > 128:
                    # four word planes of 257 bin rows do not fit beside the rings: the float kernel runs instead
                    tol = 1e-5 * float(np.abs(g).max()) * np.maximum(1, np.bincount(b, minlength=nbins))
                    assert (np.abs(hg[f, :, 0] - sg.astype(np.float64) * ginv) <= tol).all(), (n, f, "g (float kernel)")
                    continue
                assert np.array_equal(hg[f, :, 0], sg.astype(np.float64) * ginv), (n, f, "g")
                assert np.array_equal(hg[f, :, 2], sw.astype(np.float64) * winv), (n, f, "w")
                assert np.array_equal(hg[f, :, 1], 2.0 * sw.astype(np.float64) * winv), (n, f, "h = 2w")
            checked += 1
        assert checked >= 3 and nn == 2 ** depth - 1
    finally:
        cache.close()


def test_float_kernel_is_used_with_a_column_sample(pkg):
    """With colsample < 1 the unit's bins are not adjacent bytes: the float kernel runs and the model still trains."""
    x, y = make_regression(20_000, 20, seed=5)
    m = pkg.fit(pkg.EvoTreeRegressor(loss="mse", nrounds=5, max_depth=4, nbins=32, colsample=0.5, eta=0.3), x_train=x, y_train=y)
    p = np.asarray(m(x)).reshape(x.shape[0], -1)[:, 0]
    assert np.mean((p - y) ** 2) < np.var(y)
