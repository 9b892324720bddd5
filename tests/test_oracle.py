"""CPU oracle against everything the reference's own tests pin for this path, plus self-consistency checks.

Known-answer / finite-difference checks follow test/metrics.jl:134-232 (MLE gradients, Fisher information,
softplus round trip, inverse link, softmax gradient) and test/predict-leaf-idx.jl:25-73 (traversal rule and
leaf invariants).  Statistical thresholds follow test/core.jl (eval MSE must beat the bias model by > 75 %).
"""
import math

import numpy as np
import pytest


def _dbl4(orc, loc, sr, y):
    import ctypes as C
    out = (C.c_double * 4)()
    orc.lib().orc_gaussian_grad_hess64(C.c_double(loc), C.c_double(sr), C.c_double(y), out)
    return list(out)


def gaussian_lpdf(y, loc, scale):
    return -(math.log(scale) + (y - loc) ** 2 / (2 * scale ** 2))


def test_softplus_roundtrip(orc):
    for scale in (2.0, 0.5, 1.0):
        sr = orc.lib().orc_invsoftplus64(scale)
        assert orc.lib().orc_softplus64(sr) == pytest.approx(scale, rel=1e-12)


def test_gaussian_mle_gradients_match_finite_differences(orc):
    loc, scale, h = 0.5, 2.0, 1e-6
    sr = orc.lib().orc_invsoftplus64(scale)
    sp = orc.lib().orc_softplus64

    def metric(lc, raw, y):
        return gaussian_lpdf(y, lc, sp(raw))

    for y in (1.5, 4.0, -3.0):
        g1, g2, h1, h2 = _dbl4(orc, loc, sr, y)
        dloc = (metric(loc + h, sr, y) - metric(loc - h, sr, y)) / (2 * h)
        draw = (metric(loc, sr + h, y) - metric(loc, sr - h, y)) / (2 * h)
        assert dloc == pytest.approx(-g1, abs=1e-5)
        assert draw == pytest.approx(-g2, abs=1e-5)
    # Fisher information: independent of the residual, positive
    ds = orc.lib().orc_sigmoid64(sr)
    ref = _dbl4(orc, loc, sr, loc)[2:]
    assert ref[0] == pytest.approx(1 / scale ** 2)
    assert ref[1] == pytest.approx(2 * (ds / scale) ** 2)
    assert ref[0] > 0 and ref[1] > 0
    for y in (1.5, 4.0, -3.0):
        assert _dbl4(orc, loc, sr, y)[2:] == ref


def test_inverse_link(orc):
    # Julia: pred = Float32[0.0 1.0; -2.0 0.5] (K x nobs); here rows are observations
    pred = np.array([[0.0, -2.0], [1.0, 0.5]], np.float32)
    p = orc.Params(loss="gaussian_mle", K=2)
    orc.link(p, pred)
    assert pred[:, 0].tolist() == [0.0, 1.0]
    sp = np.array([orc.lib().orc_softplus(float(v)) for v in (-2.0, 0.5)], np.float32)
    np.testing.assert_allclose(pred[:, 1], sp, rtol=1e-6)
    assert not np.allclose(pred[:, 1], np.exp(np.array([-2.0, 0.5], np.float32)))
    pl = np.array([[0.3], [-4.0]], np.float32)
    orc.link(orc.Params(loss="logloss", K=1), pl)
    np.testing.assert_allclose(pl[:, 0], 1 / (1 + np.exp(-np.array([0.3, -4.0]))), rtol=1e-6)
    ps = np.array([[2.0, 1.0, 0.0]], np.float32)
    orc.link(orc.Params(loss="mlogloss", K=3), ps)
    np.testing.assert_allclose(ps[0], np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum(), rtol=1e-6)


def test_softmax_gradient_and_hessian(orc):
    import ctypes as C

    def loss(p, k):
        return math.log(sum(math.exp(v) for v in p)) - p[k]

    target = 1  # the reference's target = 2 (1-based)
    for p in ([0.0, 0.0, 0.0], [2.0, 1.0, 0.0], [1.0, -0.5, 0.3], [-1.0, -1.0, 2.0]):
        isum = sum(math.exp(v) for v in p)
        h = 1e-5
        for k in range(len(p)):
            out = (C.c_double * 2)()
            orc.lib().orc_mlogloss_grad_hess64(C.c_double(p[k]), C.c_double(isum), C.c_int(k == target), out)
            pp, pm = list(p), list(p)
            pp[k] += h
            pm[k] -= h
            assert out[0] == pytest.approx((loss(pp, target) - loss(pm, target)) / (2 * h), abs=1e-5)
            assert out[1] == pytest.approx((loss(pp, target) - 2 * loss(p, target) + loss(pm, target)) / h ** 2, abs=1e-4)


def test_update_grads_formulas(orc):
    rng = np.random.default_rng(0)
    n = 257
    w = rng.uniform(0.5, 2, n).astype(np.float32)
    # mse / logloss
    for loss in ("mse", "logloss"):
        p = orc.Params(loss=loss, K=1)
        pred = rng.normal(size=(n, 1)).astype(np.float32)
        y = rng.random(n).astype(np.float32)
        g = np.zeros((n, 3), np.float32)
        g[:, 2] = w
        orc.update_grads(p, pred, y, g)
        if loss == "mse":
            np.testing.assert_array_equal(g[:, 0], (np.float32(2) * (pred[:, 0] - y)) * w)
            np.testing.assert_array_equal(g[:, 1], np.float32(2) * w)
        else:
            s = 1 / (1 + np.exp(-pred[:, 0].astype(np.float64)))
            np.testing.assert_allclose(g[:, 0], (s - y) * w, rtol=2e-6, atol=1e-7)
            np.testing.assert_allclose(g[:, 1], s * (1 - s) * w, rtol=2e-6, atol=1e-7)
    # softmax
    K = 4
    p = orc.Params(loss="mlogloss", K=K)
    pred = rng.normal(size=(n, K)).astype(np.float32)
    y = rng.integers(1, K + 1, n).astype(np.uint32)
    g = np.zeros((n, 2 * K + 1), np.float32)
    g[:, -1] = w
    orc.update_grads(p, pred, y, g)
    e = np.exp(pred.astype(np.float64))
    prob = e / e.sum(axis=1, keepdims=True)
    onehot = np.eye(K)[y - 1]
    np.testing.assert_allclose(g[:, :K], (prob - onehot) * w[:, None], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(g[:, K:2 * K], prob * (1 - prob) * w[:, None], rtol=1e-5, atol=1e-6)
    # gaussian: layout g_mu, g_phi, h_mu, h_phi, w
    p = orc.Params(loss="gaussian_mle", K=2)
    pred = rng.normal(size=(n, 2)).astype(np.float32)
    y = rng.normal(size=n).astype(np.float32)
    g = np.zeros((n, 5), np.float32)
    g[:, -1] = w
    orc.update_grads(p, pred, y, g)
    for i in range(0, n, 37):
        ref = _dbl4(orc, float(pred[i, 0]), float(pred[i, 1]), float(y[i]))
        np.testing.assert_allclose(g[i, :4], np.array(ref) * w[i], rtol=2e-5, atol=1e-6)


def _python_traverse(t, xb_row, feattypes=None):
    nid = 1
    while t.split[nid - 1]:
        f = int(t.feat[nid - 1]) - 1
        num = True if feattypes is None else bool(feattypes[f])
        cond = xb_row[f] <= t.cond_bin[nid - 1] if num else xb_row[f] == t.cond_bin[nid - 1]
        nid = (nid << 1) + (0 if cond else 1)
    return nid


def _fit_oracle(orc, loss="mse", n=3000, f=5, depth=4, rounds=5, nbins=16, seed=1, **kw):
    rng = np.random.default_rng(seed)
    x = rng.random((n, f))
    y = (np.sin(x[:, 0] * 6) + x[:, 1] * x[:, 2] + 0.05 * rng.normal(size=n)).astype(np.float32)
    if loss == "logloss":
        y = (y > np.median(y)).astype(np.float32)
    edges = orc.get_edges(x, nbins, rng)
    xb = orc.binarize(x, edges)
    p = orc.Params(loss=loss, K=2 if loss == "gaussian_mle" else 1, nbins=nbins, max_depth=depth, **kw)
    b = orc.Booster(p, xb, y)
    js = np.arange(1, f + 1, dtype=np.uint32)
    last = None
    for _ in range(rounds):
        last = b.round(None, 255, js, want_hist=True)
    return b, xb, y, last


def test_leaf_index_invariants(orc):
    b, xb, y, (t, nidx, hist, nsum) = _fit_oracle(orc)
    leaf = orc.leaf_idx(xb, t)
    assert np.array_equal(leaf, nidx)                       # partition and traversal agree
    for i in range(0, xb.shape[0], 97):
        assert leaf[i] == _python_traverse(t, xb[i])         # independent traversal: nid = nid << 1 + !cond
    assert not t.split[leaf - 1].any()                       # leaves are non-split nodes
    pred = np.zeros((xb.shape[0], 1), np.float32)
    orc.predict_tree(b.p, xb, t, pred)
    for l in np.unique(leaf):                                # rows of one leaf share one prediction
        assert np.unique(pred[leaf == l]).size == 1
    # a stump (max_depth = 1) sends every row to node 1
    p1 = orc.Params(max_depth=1, nbins=16)
    b1 = orc.Booster(p1, xb, y)
    t1, n1, _, _ = b1.round(None, 255, np.arange(1, 6, dtype=np.uint32))
    assert t1.feat.size == 1 and not t1.split[0] and (n1 == 1).all()


def test_histograms_and_subtraction(orc):
    b, xb, y, (t, nidx, hist, nsum) = _fit_oracle(orc, depth=3, rounds=1)
    g = b.grad.astype(np.float64)
    # the gradients that built the tree are the pre-round ones: recompute them from the bias
    p = b.p
    pred0 = np.tile(b.mu, (xb.shape[0], 1)).astype(np.float32)
    g0 = b.grad.copy()
    orc.update_grads(p, pred0, y, g0)
    for j in range(xb.shape[1]):
        for c in range(3):
            ref = np.bincount(xb[:, j].astype(np.int64) - 1, weights=g0[:, c].astype(np.float64), minlength=p.nbins)
            np.testing.assert_allclose(hist[0, j, :, c], ref, rtol=1e-12, atol=1e-9)
    assert t.split[0]
    np.testing.assert_allclose(hist[0], hist[1] + hist[2], rtol=1e-10, atol=1e-9)   # parent = left + right
    np.testing.assert_allclose(nsum[0], nsum[1] + nsum[2], rtol=1e-12, atol=1e-9)
    np.testing.assert_allclose(nsum[0], g0.astype(np.float64).sum(axis=0), rtol=1e-12)
    # split condition: left child holds exactly the rows with bin <= cond_bin
    f0, cb = int(t.feat[0]) - 1, int(t.cond_bin[0])
    assert (xb[:, f0] <= cb).sum() == round(nsum[1, 2])


@pytest.mark.parametrize("loss", ["mse", "logloss", "gaussian_mle"])
def test_training_beats_the_bias_model(orc, loss):
    b, xb, y, _ = _fit_oracle(orc, loss=loss, n=4000, depth=5, rounds=60, eta=0.2)
    mu = np.tile(b.mu, (y.size, 1)).astype(np.float32)
    pred = b.pred.copy()
    orc.link(b.p, pred)
    orc.link(b.p, mu)
    mse0, mse1 = np.mean((mu[:, 0] - y) ** 2), np.mean((pred[:, 0] - y) ** 2)
    assert mse1 < 0.25 * mse0, (mse0, mse1)


def test_softmax_training(orc):
    rng = np.random.default_rng(3)
    n, f, K = 3000, 6, 3
    x = rng.normal(size=(n, f))
    y = (x[:, :K] + 0.3 * rng.gumbel(size=(n, K))).argmax(axis=1).astype(np.uint32) + 1
    xb = orc.binarize(x, orc.get_edges(x, 16, rng))
    p = orc.Params(loss="mlogloss", K=K, nbins=16, max_depth=4, eta=0.3)
    b = orc.Booster(p, xb, y)
    for _ in range(30):
        b.round(None, 255, np.arange(1, f + 1, dtype=np.uint32))
    assert np.isfinite(b.pred).all() and b.pred.max() <= 0 and b.pred.min() >= -15   # predict! keeps logits in [-15, 0]
    assert (b.pred.argmax(axis=1) + 1 == y).mean() > 0.8


def test_binning(orc):
    rng = np.random.default_rng(5)
    for dt in (np.float32, np.float64):
        x = rng.normal(size=(5000, 4)).astype(dt)
        e = orc.get_edges(x, 32, rng)
        assert e.dtype == dt and e.shape == (4, 31) and (np.diff(e, axis=1) >= 0).all()
        np.testing.assert_allclose(e, np.quantile(x.astype(np.float64), np.arange(1, 32) / 32, axis=0, method="linear").T,
                                   rtol=1e-5, atol=1e-6)
        xb = orc.binarize(x, e)
        ref = np.stack([np.searchsorted(e[j], x[:, j], side="left") for j in range(4)], 1) + 1
        assert xb.dtype == np.uint8 and np.array_equal(xb, ref) and xb.min() >= 1 and xb.max() <= 32
    # ties and exact hits: searchsortedfirst puts x == edge into the edge's own bin
    e = np.array([[1.0, 2.0, 2.0, 3.0]], np.float64)
    x = np.array([[0.5], [1.0], [2.0], [2.5], [3.0], [9.0]])
    assert orc.binarize(x, e)[:, 0].tolist() == [1, 1, 2, 4, 4, 5]


def test_row_sampling_and_constraints(orc):
    b, xb, y, _ = _fit_oracle(orc, rounds=1)
    rng = np.random.default_rng(9)
    mask = rng.integers(0, 256, xb.shape[0], dtype=np.uint8)
    t, nidx, _, nsum = b.round(mask, 128, np.array([1, 3, 5], np.uint32))
    assert ((nidx > 0) == (mask <= 128)).all()                                   # src/subsample.jl:21
    assert set(np.unique(t.feat)) <= {0, 1, 3, 5}                                # only sampled columns split
    assert round(nsum[0, 2]) == (mask <= 128).sum()
    # min_weight is a strict bound on both children (src/fit-utils.jl:419)
    p = orc.Params(nbins=16, max_depth=6, min_weight=200.0)
    bb = orc.Booster(p, xb, y)
    t2, _, _, ns2 = bb.round(None, 255, np.arange(1, 6, dtype=np.uint32))
    assert (ns2[t2.w != 0][:, 2] > 200).all()
    # monotone constraint +1 on feature 2: left leaf value < right leaf value wherever feature 2 splits
    mono = np.array([0, 1, 0, 0, 0], np.int32)
    bm = orc.Booster(orc.Params(nbins=16, max_depth=5), xb, y, monotone=mono)
    tm, _, _, nsm = bm.round(None, 255, np.arange(1, 6, dtype=np.uint32))
    for n in np.nonzero(tm.split)[0] + 1:
        if tm.feat[n - 1] == 2:
            pl = -0.1 * nsm[2 * n - 1, 0] / (nsm[2 * n - 1, 1] + 1.0)
            pr = -0.1 * nsm[2 * n, 0] / (nsm[2 * n, 1] + 1.0)
            assert pl < pr


def test_eval_metrics_against_float64_formulas(orc):
    """The metric restatement against the closed forms of src/metrics.jl:1-110 evaluated in float64."""
    rng = np.random.default_rng(11)
    n = 5000
    w = rng.uniform(0.5, 2.0, n).astype(np.float32)
    p = rng.normal(0, 1.5, (n, 1)).astype(np.float32)
    y = rng.normal(0, 1, n).astype(np.float32)
    p64, y64, w64 = p[:, 0].astype(np.float64), y.astype(np.float64), w.astype(np.float64)
    assert np.isclose(orc.eval_metric("mse", p, y, w), np.sum(w64 * (p64 - y64) ** 2) / w64.sum(), rtol=1e-6)
    assert np.isclose(orc.eval_metric("rmse", p, y, w), np.sqrt(np.sum(w64 * (p64 - y64) ** 2) / w64.sum()), rtol=1e-6)
    assert np.isclose(orc.eval_metric("mae", p, y), np.mean(np.abs(p64 - y64)), rtol=1e-6)
    yb = (rng.random(n) < 0.3).astype(np.float32)
    s = 1 / (1 + np.exp(-p64))
    assert np.isclose(orc.eval_metric("logloss", p, yb, w), np.sum(w64 * -(yb * np.log(s) + (1 - yb) * np.log(1 - s))) / w64.sum(), rtol=1e-5)
    K = 4
    pm = rng.normal(0, 1, (n, K)).astype(np.float32)
    yc = rng.integers(1, K + 1, n).astype(np.uint32)
    lse = np.log(np.exp(pm.astype(np.float64)).sum(axis=1))
    assert np.isclose(orc.eval_metric("mlogloss", pm, yc, w), np.sum(w64 * (lse - pm[np.arange(n), yc - 1])) / w64.sum(), rtol=1e-5)
    pg = np.stack([rng.normal(0, 1, n), rng.normal(0, 1, n)], axis=1).astype(np.float32)
    sc = np.log1p(np.exp(pg[:, 1].astype(np.float64)))
    ref = np.sum(w64 * -(np.log(sc) + (y64 - pg[:, 0]) ** 2 / (2 * sc ** 2))) / w64.sum()
    assert np.isclose(orc.eval_metric("gaussian_mle", pg, y, w), ref, rtol=1e-5)
    # matrix target: mean over the K columns (src/metrics.jl:43-47)
    p2 = rng.normal(0, 1, (n, 3)).astype(np.float32)
    y2 = rng.normal(0, 1, (n, 3)).astype(np.float32)
    assert np.isclose(orc.eval_metric("mse", p2, y2), np.mean((p2.astype(np.float64) - y2) ** 2), rtol=1e-6)


def test_log_link_and_logistic_gradients_against_finite_differences(orc):
    """poisson / gamma / tweedie / logistic_mle gradients of the oracle (src/loss.jl:59-76, 207-217) against central
    differences of the losses they derive from, as the reference's test/metrics.jl does for the MLE losses; the
    hessians of the log-link losses against the derivative of the gradient."""
    rng = np.random.default_rng(3)
    n = 400
    p64 = rng.normal(0.2, 0.7, n)
    y = np.exp(rng.normal(0.0, 0.6, n)).astype(np.float32)

    def grads(loss, pred, yy, K=1):
        par = orc.Params(loss=loss, K=K)
        g = np.zeros((pred.shape[0], 2 * K + 1), np.float32)
        g[:, -1] = 1.0
        orc.update_grads(par, np.ascontiguousarray(pred, np.float32), yy, g)
        return g.astype(np.float64)

    losses = {
        "poisson": lambda p, yy: np.exp(p) - yy * p,
        "gamma": lambda p, yy: 2 * (p + yy / np.exp(p)),
        "tweedie": lambda p, yy: 2 * (np.exp(p) ** 0.5 / 0.5 - yy * np.exp(p) ** -0.5 / -0.5),
    }
    h = 1e-4
    for name, f in losses.items():
        g = grads(name, p64.reshape(-1, 1), y)
        fd = (f(p64 + h, y.astype(np.float64)) - f(p64 - h, y.astype(np.float64))) / (2 * h)
        assert np.allclose(g[:, 0], fd, rtol=2e-4, atol=2e-4), name
        fd2 = (f(p64 + h, y) - 2 * f(p64, y) + f(p64 - h, y)) / h ** 2
        assert np.allclose(g[:, 1], fd2, rtol=5e-3, atol=5e-3), name + " hessian"

    # logistic: nll = log(s) + z + 2 log(1 + exp(-z)), z = (y - loc) / s, s = softplus(raw)
    loc, raw = rng.normal(0, 1, n), rng.normal(0.3, 0.6, n)
    yl = rng.normal(0, 1.5, n).astype(np.float32)

    def nll(lc, rw):
        s = np.log1p(np.exp(rw))
        z = (yl - lc) / s
        return np.log(s) + z + 2 * np.log1p(np.exp(-z))

    g = grads("logistic_mle", np.stack([loc, raw], axis=1), yl, K=2)
    assert np.allclose(g[:, 0], (nll(loc + h, raw) - nll(loc - h, raw)) / (2 * h), rtol=2e-3, atol=2e-4)
    assert np.allclose(g[:, 1], (nll(loc, raw + h) - nll(loc, raw - h)) / (2 * h), rtol=2e-3, atol=2e-4)
    # Fisher information of Logistic(loc, s): 1 / (3 s^2) and (pi^2 + 3) / (9 s^2) (chain rule with dscale)
    s = np.log1p(np.exp(raw))
    ds = 1 / (1 + np.exp(-raw))
    assert np.allclose(g[:, 2], 1 / (3 * s ** 2), rtol=1e-5)
    assert np.allclose(g[:, 3], (np.pi ** 2 + 3) / 9 * (ds / s) ** 2, rtol=1e-5)


def test_deviance_metrics_against_float64_formulas(orc):
    rng = np.random.default_rng(8)
    n = 3000
    p = rng.normal(0.1, 0.5, (n, 1)).astype(np.float32)
    y = np.exp(rng.normal(0, 0.5, n)).astype(np.float32)
    w = rng.uniform(0.5, 2.0, n).astype(np.float32)
    pr, y64, w64 = np.exp(p[:, 0].astype(np.float64)), y.astype(np.float64), w.astype(np.float64)
    ref = {"poisson": 2 * (y64 * np.log(y64 / pr) + pr - y64), "gamma": 2 * (np.log(pr / y64) + y64 / pr - 1),
           "tweedie": 2 * (y64 ** 0.5 / -0.5 / 0.5 - y64 * pr ** -0.5 / -0.5 + pr ** 0.5 / 0.5)}
    for name, v in ref.items():
        assert np.isclose(orc.eval_metric(name, p, y, w), np.sum(w64 * v) / w64.sum(), rtol=2e-4, atol=1e-6), name
    pg = np.stack([rng.normal(0, 1, n), rng.normal(0, 1, n)], axis=1).astype(np.float32)
    s = np.log1p(np.exp(pg[:, 1].astype(np.float64)))
    az = np.abs((y64 - pg[:, 0]) / s)
    assert np.isclose(orc.eval_metric("logistic_mle", pg, y, w), np.sum(w64 * (-np.log(s) - az - 2 * np.log1p(np.exp(-az)))) / w64.sum(), rtol=1e-5)


def test_mae_and_credibility_trees_by_hand(orc):
    """A two-bin, one-feature problem small enough to evaluate by hand: the oracle must split where the formulas of
    src/split.jl:2-4, 119-141 say and give the leaves of src/predict.jl:211-218, 250-257."""
    x_bin = np.asfortranarray(np.array([[1], [1], [1], [2], [2], [2], [2], [2]], np.uint8))
    y = np.array([1.0, 2.0, 3.0, 7.0, 8.0, 9.0, 10.0, 11.0], np.float32)
    n = y.size
    for loss in ("mae", "cred_var", "cred_std"):
        p = orc.Params(loss=loss, K=1, nbins=2, max_depth=2, eta=1.0, lambda_=0.0, L2=0.0, min_weight=0.5)
        # categorical feature: both bins are candidates (a numeric one only scans bins 1..nbins-1, which is the same here)
        grad = np.zeros((n, 3), np.float32)
        grad[:, 2] = 1.0
        pred = np.full((n, 1), y.mean(), np.float32)
        orc.update_grads(p, pred, y, grad)
        t, nidx, _, _ = orc.grow_tree(p, x_bin, grad, np.arange(1, n + 1, dtype=np.uint32), np.array([1], np.uint32))
        assert t.split[0] and t.feat[0] == 1 and t.cond_bin[0] == 1
        d = y - y.mean()
        left, right = d[:3], d[3:]
        # eta = 1, lambda = L2 = 0: both leaf formulas reduce to the mean residual of the leaf
        assert np.allclose(t.pred[1, 0], left.mean(), rtol=1e-6) and np.allclose(t.pred[2, 0], right.mean(), rtol=1e-6)
        if loss == "mae":
            gain = abs(left.mean()) * 3 + abs(right.mean()) * 5          # parent mean residual is 0, node gain is 0
        else:
            def cred(v):
                m1, m2, w = v.sum(), (v ** 2).sum(), v.size
                vhm = (m1 / w) ** 2
                evpv = max(np.finfo(np.float64).eps, m2 / w - vhm)
                z = vhm / (vhm + evpv) if loss == "cred_var" else np.sqrt(vhm) / (np.sqrt(vhm) + np.sqrt(evpv))
                return z * abs(m1)
            gain = cred(left.astype(np.float64)) + cred(right.astype(np.float64)) - cred(d.astype(np.float64))
        assert np.isclose(t.gain[0], gain, rtol=1e-4), (loss, t.gain[0], gain)


def test_quantile_leaves_by_hand(orc):
    """One split, two leaves: the leaf values must be numpy's (type-7) quantile of the residuals of each side."""
    x_bin = np.asfortranarray(np.array([[1]] * 5 + [[2]] * 6, np.uint8))
    y = np.array([1.0, 2.0, 4.0, 8.0, 3.0, 20.0, 30.0, 25.0, 21.0, 40.0, 22.0], np.float32)
    n = y.size
    for alpha in (0.25, 0.5, 0.9):
        p = orc.Params(loss="quantile", K=1, nbins=2, max_depth=2, eta=1.0, lambda_=0.0, L2=0.0, min_weight=0.5, alpha=alpha)
        grad = np.zeros((n, 3), np.float32)
        grad[:, 2] = 1.0
        pred = np.full((n, 1), y.mean(), np.float32)
        orc.update_grads(p, pred, y, grad)
        d = y - np.float32(y.mean())
        assert np.array_equal(grad[:, 1], d) and np.allclose(grad[:, 0], np.where(d > 0, alpha, alpha - 1))
        t, _, _, _ = orc.grow_tree(p, x_bin, grad, np.arange(1, n + 1, dtype=np.uint32), np.array([1], np.uint32))
        assert t.split[0] and t.cond_bin[0] == 1
        assert np.isclose(t.pred[1, 0], np.quantile(d[:5].astype(np.float64), alpha), rtol=1e-6)
        assert np.isclose(t.pred[2, 0], np.quantile(d[5:].astype(np.float64), alpha), rtol=1e-6)


def test_oblivious_tree_levels_by_hand(orc):
    """grow_otree! (src/fit.jl:147-263): one (feature, bin) per depth = first maximum of the gains summed over the
    depth's nodes, candidates that are not eligible or not positive in any node dropped; checked against a numpy
    restatement on the oracle's own histograms.  test/oblivious.jl:28-146 pins the same learner by loss thresholds."""
    from tests.parity import _gain_of
    b, xb, y, (t, nidx, hist, nsum) = _fit_oracle(orc, depth=4, rounds=3, tree_type=1, min_weight=20.0)
    p = b.p
    B, F = p.nbins, xb.shape[1]
    assert np.array_equal(orc.leaf_idx(xb, t), nidx)
    for d in range(1, p.max_depth):
        nodes = list(range(2 ** (d - 1), 2 ** d))
        if not t.split[nodes[0] - 1]:
            assert not any(t.split[n - 1] for n in range(nodes[0], t.split.size + 1))
            break
        assert all(t.split[n - 1] for n in nodes)
        assert len({(int(t.feat[n - 1]), int(t.cond_bin[n - 1])) for n in nodes}) == 1
        tot = np.zeros((F, B))
        ok = np.ones((F, B), bool)
        for n in nodes:
            for j in range(F):
                wl = np.cumsum(hist[n - 1, j, :, 2])
                for bin1 in range(1, B):
                    g = 0.0
                    if wl[bin1 - 1] > p.min_weight and nsum[n - 1, 2] - wl[bin1 - 1] > p.min_weight:
                        g = _gain_of(p, hist[n - 1], nsum[n - 1], j, bin1)
                    tot[j, bin1 - 1] += g
                    ok[j, bin1 - 1] &= g > 0
        tot = np.where(ok, tot, 0.0)
        j, bi = np.unravel_index(np.argmax(tot), tot.shape)       # row-major over (feature, bin) = the reference's order
        assert (int(t.feat[nodes[0] - 1]), int(t.cond_bin[nodes[0] - 1])) == (j + 1, bi + 1)
        np.testing.assert_allclose(t.gain[nodes[0] - 1], tot[j, bi], rtol=1e-6)
    assert t.split[0] and t.split[1] and t.split[2]               # the data supports at least two shared levels


def test_oblivious_training_beats_the_bias_model(orc):
    b, xb, y, _ = _fit_oracle(orc, depth=5, rounds=40, nbins=32, tree_type=1)   # test/oblivious.jl: eval loss thresholds
    pred = b.pred[:, 0]
    assert np.mean((pred - y) ** 2) < 0.25 * np.mean((y.mean() - y) ** 2)
