"""Inference through the C ABI (`evb_predict_x`: device binarize + traversal of all trees + link, and `evb_predict`
on binned input) against the oracle's `predict!` / `predict_leaf_idx!` / link applied tree by tree."""
import numpy as np
import pytest

from tests.parity import make_regression, oracle_params

pytestmark = pytest.mark.gpu


def _oracle_predict(orc, m, op, x, ntree_limit=None, link=True):
    xb = orc.binarize(x, m.info["edges"])
    n = len(m.trees) if ntree_limit is None else ntree_limit
    pred = np.zeros((x.shape[0], m.K), np.float32)
    leaves = np.zeros((x.shape[0], n), np.uint32)
    for i, t in enumerate(m.trees[:n]):
        nn = t.feat.size
        ot = orc.Tree(t.feat, t.cond_bin, t.w, t.gain, t.pred, t.split.astype(np.uint8))
        orc.predict_tree(op, xb, ot, pred, m.info["feattypes"].astype(np.uint8))
        leaves[:, i] = orc.leaf_idx(xb, ot, m.info["feattypes"].astype(np.uint8))
        assert nn >= 1
    if link:
        orc.link(op, pred)
    return pred, leaves


CASES = [("mse", "EvoTreeRegressor", dict(max_depth=5, nbins=32)), ("logloss", "EvoTreeRegressor", dict(max_depth=4, nbins=16)),
         ("mlogloss", "EvoTreeClassifier", dict(max_depth=4, nbins=16)), ("gaussian_mle", "EvoTreeMLE", dict(max_depth=4, nbins=32)),
         ("poisson", "EvoTreeRegressor", dict(max_depth=4, nbins=16)), ("gamma", "EvoTreeRegressor", dict(max_depth=4, nbins=16)),
         ("tweedie", "EvoTreeRegressor", dict(max_depth=4, nbins=16)), ("logistic_mle", "EvoTreeMLE", dict(max_depth=4, nbins=32))]


@pytest.mark.parametrize("loss,learner,kw", CASES)
def test_predict_matches_oracle(pkg, orc, loss, learner, kw):
    x, y = make_regression(20_000, 9, seed=hash(loss) % 1000)
    if loss == "logloss":
        y = (y > np.median(y)).astype(np.float32)
    if loss == "mlogloss":
        y = np.digitize(y, np.quantile(y, [0.3, 0.6])).astype(np.int64)
    if loss in ("poisson", "gamma", "tweedie"):
        y = np.exp(0.5 * (y - y.mean()) / y.std()).astype(np.float32)      # positive target for the log link
    params = getattr(pkg, learner)(loss=loss, nrounds=6, eta=0.3, **kw)
    m = pkg.fit(params, x_train=x, y_train=y)
    assert len(m.trees) == 7 and m.info["nrounds"] == 6
    op = oracle_params(orc, params, m.K)
    xt, _ = make_regression(7_777, 9, seed=5)
    want, leaves = _oracle_predict(orc, m, op, xt)
    for xin in (np.ascontiguousarray(xt), np.asfortranarray(xt), xt.astype(np.float64)):
        got = pkg.predict(m, xin)
        np.testing.assert_allclose(got.reshape(want.shape), want, rtol=1e-5, atol=1e-6)
    assert np.array_equal(pkg.predict_leaf_idx(m, xt), leaves)                       # bit-exact leaf ids
    w3, l3 = _oracle_predict(orc, m, op, xt, ntree_limit=3)
    np.testing.assert_allclose(pkg.predict(m, xt, ntree_limit=3).reshape(w3.shape), w3, rtol=1e-5, atol=1e-6)
    assert np.array_equal(pkg.predict_leaf_idx(m, xt, ntree_limit=3), l3)
    # binned entry point gives the same numbers as the raw one
    xb = pkg.binarize(xt, m.info["edges"])
    assert np.array_equal(xb, orc.binarize(xt, m.info["edges"]))
    np.testing.assert_allclose(pkg.predict_binned(m, xb), pkg.predict(m, xt).reshape(want.shape), rtol=0, atol=0)
    with pytest.raises(ValueError):
        pkg.predict(m, xt, ntree_limit=99)


def test_bias_only_model_and_empty_input(pkg, orc):
    x, y = make_regression(500, 4, seed=2)
    m = pkg.fit(pkg.EvoTreeRegressor(nrounds=0, max_depth=3, nbins=8), x_train=x, y_train=y)
    assert len(m.trees) == 1
    p = pkg.predict(m, x)
    np.testing.assert_allclose(p, np.full(500, np.float32(y.mean())), rtol=1e-6)
    assert pkg.predict(m, x[:0]).shape == (0,)


def test_training_predictions_equal_inference(pkg):
    """The predictions kept by the training cache equal what inference returns for the training rows."""
    x, y = make_regression(30_000, 12, seed=8)
    params = pkg.EvoTreeRegressor(nrounds=10, max_depth=6, nbins=64, eta=0.2, rowsample=0.6, colsample=0.7)
    m, cache = pkg.fit(params, x_train=x, y_train=y, return_cache=True)
    try:
        np.testing.assert_allclose(cache.pred()[:, 0], pkg.predict(m, x), rtol=1e-5, atol=1e-5)
    finally:
        cache.close()
    assert np.mean((pkg.predict(m, x) - y) ** 2) < 0.5 * np.var(y)


def test_pipelined_rounds_equal_sequential_rounds(pkg):
    """`grow_rounds` (host one tree ahead, per-tree CUDA graph replay) grows exactly the trees that one
    `grow_evotree` call per round grows."""
    x, y = make_regression(40_000, 15, seed=13)
    params = pkg.EvoTreeRegressor(nrounds=8, max_depth=6, nbins=32, eta=0.2, rowsample=0.8, colsample=0.8)
    m1, c1 = pkg.init_core(params, x, y)
    m2, c2 = pkg.init_core(params, x, y)
    try:
        pkg.grow_rounds(m1, c1, params, 8)
        for _ in range(8):
            pkg.grow_evotree(m2, c2, params)
        assert len(m1.trees) == len(m2.trees) == 9
        for t1, t2 in zip(m1.trees, m2.trees):
            assert np.array_equal(t1.feat, t2.feat) and np.array_equal(t1.cond_bin, t2.cond_bin)
            assert np.array_equal(t1.pred, t2.pred) and np.array_equal(t1.gain, t2.gain)
        assert np.array_equal(c1.pred(), c2.pred())
        # a third tree cannot be started while two are in flight
        mask, js = pkg.sample_round(c1, params)
        pkg.grow_tree_begin(c1, params, mask, js, True)
        pkg.grow_tree_begin(c1, params, mask, js, True)
        with pytest.raises(pkg.EvbError):
            pkg.grow_tree_begin(c1, params, mask, js, True)
        pkg.grow_tree_end(c1, params)
        pkg.grow_tree_end(c1, params)
    finally:
        c1.close()
        c2.close()
