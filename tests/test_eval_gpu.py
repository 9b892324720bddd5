"""Evaluation data tracked on the device (`evb_eval_attach` / `evb_eval_sums` behind `fit(...; x_eval, y_eval)`):
the logged metric of every iteration against the oracle's `predict!` + metric on the same trees, early stopping as
in the reference's test/core.jl:59-103, and class encoding of the evaluation target as in test/metrics.jl:95-135."""
import numpy as np
import pytest

from tests.parity import make_regression, oracle_params

pytestmark = pytest.mark.gpu

RTOL = 1e-5  # float32 per-row values (expf / logf of two math libraries), float64 sums


def _oracle_log(orc, m, op, metric, x_eval, y_eval, w_eval=None, pred0=None, alpha=0.5):
    """Metric after the bias tree and after every further tree, from the oracle's traversal and metric."""
    xb = orc.binarize(x_eval, m.info["edges"])
    ft = m.info["feattypes"].astype(np.uint8)
    pred = np.zeros((x_eval.shape[0], m.K), np.float32) if pred0 is None else pred0.astype(np.float32).copy()
    out = []
    for t in m.trees:
        ot = orc.Tree(t.feat, t.cond_bin, t.w, t.gain, t.pred, t.split.astype(np.uint8))
        orc.predict_tree(op, xb, ot, pred, ft)
        out.append(orc.eval_metric(metric, pred, y_eval, w_eval, alpha))
    return np.array(out), pred


def _data(loss, n, seed):
    x, y = make_regression(n, 8, seed=seed)
    if loss == "logloss":
        y = (y > np.median(y)).astype(np.float32)
    if loss == "mlogloss":
        y = np.digitize(y, np.quantile(y, [0.3, 0.6])).astype(np.int64)
    if loss in ("poisson", "gamma", "tweedie"):
        y = np.exp(0.5 * (y - y.mean()) / y.std()).astype(np.float32)      # positive target for the log link
    return x, y


CASES = [("mse", "mse", "EvoTreeRegressor"), ("mse", "rmse", "EvoTreeRegressor"), ("mse", "mae", "EvoTreeRegressor"),
         ("logloss", "logloss", "EvoTreeRegressor"), ("mlogloss", "mlogloss", "EvoTreeClassifier"),
         ("gaussian_mle", "gaussian_mle", "EvoTreeMLE"), ("poisson", "poisson", "EvoTreeRegressor"),
         ("gamma", "gamma", "EvoTreeRegressor"), ("tweedie", "tweedie", "EvoTreeRegressor"),
         ("logistic_mle", "logistic_mle", "EvoTreeMLE"), ("gaussian_mle", "logistic_mle", "EvoTreeMLE"),
         ("quantile", "quantile", "EvoTreeRegressor")]


@pytest.mark.parametrize("loss,metric,learner", CASES)
def test_logged_metric_matches_oracle(pkg, orc, loss, metric, learner):
    x, y = _data(loss, 30_000, 3)
    tr, ev = slice(0, 22_000), slice(22_000, None)
    w_eval = np.random.default_rng(1).uniform(0.5, 2.0, 8_000).astype(np.float32)
    params = getattr(pkg, learner)(loss=loss, metric=metric, nrounds=8, eta=0.3, max_depth=5, nbins=32, alpha=0.3)
    m = pkg.fit(params, x_train=x[tr], y_train=y[tr], x_eval=x[ev], y_eval=y[ev], w_eval=w_eval)
    lg = m.info["logger"]
    assert lg["iter"] == list(range(9)) and lg["nrounds"] == 8 and lg["name"] == metric
    op = oracle_params(orc, params, m.K)
    y_or = y[ev] if loss != "mlogloss" else (np.searchsorted(m.info["target_levels"], y[ev]) + 1).astype(np.uint32)
    ref, _ = _oracle_log(orc, m, op, metric, x[ev], y_or, w_eval, alpha=0.3)
    np.testing.assert_allclose(np.array(lg["metrics"]), ref, rtol=RTOL)
    # the metric moves in the right direction on data drawn from the training distribution
    better = lg["metrics"][-1] > lg["metrics"][0] if lg["maximise"] else lg["metrics"][-1] < lg["metrics"][0]
    assert better and lg["maximise"] == (metric in ("gaussian_mle", "logistic_mle"))


def test_eval_predictions_and_offset(pkg, orc):
    """Evaluation predictions on the device equal the oracle's, offsets included (src/callback.jl:110-118)."""
    F = pkg
    x, y = _data("logloss", 12_000, 9)
    tr, ev = slice(0, 9_000), slice(9_000, None)
    rng = np.random.default_rng(2)
    off_tr = rng.uniform(0.2, 0.8, 9_000).astype(np.float32)
    off_ev = rng.uniform(0.2, 0.8, 3_000).astype(np.float32)
    params = pkg.EvoTreeRegressor(loss="logloss", nrounds=5, eta=0.5, max_depth=4, nbins=16)
    m, cache = F.init_core(params, x[tr], y[tr], offset_train=off_tr)
    cb = F.CallBack(params, m, cache, x[ev], y[ev], offset_eval=off_ev)
    logger = F.init_logger(params.metric, False, params.early_stopping_rounds)
    cb(logger, 0)
    for i in range(1, 6):
        F.grow_evotree(m, cache, params)
        cb(logger, i)
    op = oracle_params(orc, params, m.K)
    p0 = np.log(off_ev / (1 - off_ev)).astype(np.float32).reshape(-1, 1)
    ref, pred = _oracle_log(orc, m, op, "logloss", x[ev], y[ev], None, p0)
    np.testing.assert_allclose(np.array(logger["metrics"]), ref, rtol=RTOL)
    np.testing.assert_allclose(cb.pred(), pred, rtol=1e-6, atol=1e-6)
    # detaching stops the tracking; the handle keeps boosting
    cb.detach()
    F.grow_evotree(m, cache, params)
    with pytest.raises(pkg.EvbError, match="no evaluation data"):
        cb.last()
    cache.close()


def test_pipelined_logger_equals_sequential(pkg):
    """The host-one-tree-ahead loop logs the same metrics as the strictly sequential loop."""
    x, y = _data("mse", 20_000, 4)
    tr, ev = slice(0, 15_000), slice(15_000, None)
    kw = dict(nrounds=12, eta=0.2, max_depth=5, nbins=32, rowsample=0.7, colsample=0.6)
    m_pipe = pkg.fit(pkg.EvoTreeRegressor(**kw), x_train=x[tr], y_train=y[tr], x_eval=x[ev], y_eval=y[ev])
    m_seq = pkg.fit(pkg.EvoTreeRegressor(early_stopping_rounds=12, **kw), x_train=x[tr], y_train=y[tr], x_eval=x[ev], y_eval=y[ev])
    assert len(m_pipe.trees) == len(m_seq.trees) == 13
    assert m_pipe.info["logger"]["metrics"] == m_seq.info["logger"]["metrics"]
    for a, b in zip(m_pipe.trees, m_seq.trees):
        assert np.array_equal(a.feat, b.feat) and np.array_equal(a.pred, b.pred)


def test_early_stopping_tolerance(pkg):
    """Mirror of the reference's "MSE early stopping tolerance" test (test/core.jl:59-103) on seeded synthetic data."""
    rng = np.random.default_rng(321)
    n = 1_000
    x = rng.normal(size=(n, 1))
    y = x[:, 0] + 0.1 * rng.normal(size=n)
    idx = rng.permutation(n)
    tr, ev = idx[:800], idx[800:]
    kw = dict(loss="mse", nrounds=50, early_stopping_rounds=5, eta=0.05, seed=123)
    fit = lambda p: pkg.fit(p, x_train=x[tr], y_train=y[tr], x_eval=x[ev], y_eval=y[ev])
    m_strict = fit(pkg.EvoTreeRegressor(early_stopping_tolerance=0.0, **kw))
    m_tol = fit(pkg.EvoTreeRegressor(early_stopping_tolerance=0.01, **kw))
    m_default = fit(pkg.EvoTreeRegressor(**kw))
    assert len(m_tol.trees) < len(m_strict.trees)
    assert len(m_strict.trees) == 51
    assert m_tol.info["logger"]["iter_since_best"] >= 5
    assert m_tol.info["logger"]["best_iter"] < m_strict.info["logger"]["best_iter"]
    assert len(m_default.trees) == len(m_strict.trees)
    assert np.array_equal(m_default(x[ev]), m_strict(x[ev]))
    # a stopped model holds exactly the trees that were logged
    assert len(m_tol.trees) == m_tol.info["logger"]["nrounds"] + 1 == m_tol.info["nrounds"] + 1


def test_eval_class_encoding(pkg):
    """Mirror of test/metrics.jl:95-135: the evaluation target is encoded against the training levels, also when
    the evaluation fold lacks some classes, and an unseen level is rejected."""
    rng = np.random.default_rng(1)
    nobs = 4_000
    x = rng.random((nobs, 3))
    z = 2 * x[:, 0] - x[:, 1]
    y = np.where(z < -0.3, 1, np.where(z < 0.5, 2, 3))

    def true_mlogloss(m, xe, ye):
        p = m(xe)
        col = np.searchsorted(m.info["target_levels"], ye)
        return float(np.mean(-np.log(np.maximum(p[np.arange(ye.size), col].astype(np.float64), 1e-15))))

    first = np.arange(2_000)
    for ie in (np.arange(1_500), first[y[:2_000] != 1], first[y[:2_000] == 3]):
        m = pkg.fit(pkg.EvoTreeClassifier(nrounds=20, max_depth=4, eta=0.1), x_train=x, y_train=y, x_eval=x[ie], y_eval=y[ie])
        assert np.isclose(m.info["logger"]["metrics"][-1], true_mlogloss(m, x[ie], y[ie]), rtol=1e-4)
    tr = np.nonzero(y != 3)[0]
    with pytest.raises(ValueError, match="absent from `y_train`"):
        pkg.fit(pkg.EvoTreeClassifier(nrounds=5, max_depth=3), x_train=x[tr], y_train=y[tr], x_eval=x, y_eval=y)


def test_eval_attach_argument_checks(pkg):
    import ctypes as C
    from evotrees_b200 import _lib
    F = pkg
    x, y = _data("mse", 2_000, 1)
    params = pkg.EvoTreeRegressor(nrounds=1, max_depth=3, nbins=16)
    m, cache = F.init_core(params, x, y)
    xb = pkg.binarize(x, m.info["edges"])
    sums = (C.c_double * 2)()
    y32 = y.astype(np.float32)
    rc = _lib.lib().evb_eval_attach(cache.handle, C.c_int64(2_000), _lib.ptr(xb), _lib.ptr(y32), None, None, None, C.c_int32(3), sums)
    assert rc == -1 and b"not defined for loss" in _lib.lib().evb_last_error()
    rc = _lib.lib().evb_eval_sums(cache.handle, sums)
    assert rc == -1
    cb = F.CallBack(params, m, cache, x, y)
    with pytest.raises(pkg.EvbError, match="already attached"):
        F.CallBack(params, m, cache, x, y)
    assert np.isclose(cb.initial, float(np.mean((y32 - y32.mean()) ** 2)), rtol=1e-5)
    cache.close()
