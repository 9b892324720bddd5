"""GPU parity tests: the CUDA library (through its C ABI) against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest

from tests.parity import lockstep_check, make_regression

pytestmark = pytest.mark.gpu


def _softmax_data(n, f, k, seed=5):
    rng = np.random.default_rng(seed)
    x = rng.normal(size=(n, f)).astype(np.float32)
    W = rng.normal(size=(f, k))
    logits = x @ W + rng.gumbel(size=(n, k))
    return x, logits.argmax(axis=1).astype(np.int64)


def test_mse_small_config(pkg, orc):
    """The reference benchmark's smallest shape (100k x 10, depth 6, 32 bins), a few rounds in lock-step."""
    x, y = make_regression(100_000, 10, dtype=np.float64)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=4, max_depth=6, nbins=32, eta=0.1)
    s = lockstep_check(pkg, orc, p, x, y, rounds=4)
    assert s["splits"] > 50 and s["diverged"] == 0, s


def test_mse_row_col_sampling(pkg, orc):
    """Regression with 100 features and row / column sampling, scaled down in rows: 100 features, rowsample / colsample 0.5, 64 bins."""
    x, y = make_regression(60_000, 100, seed=3, dtype=np.float64)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=3, max_depth=6, nbins=64, eta=0.05, rowsample=0.5, colsample=0.5)
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 30, s


def test_mse_deep_headline_shape(pkg, orc):
    """Headline shape scaled down in rows: 100 features, depth 11, 64 bins."""
    x, y = make_regression(200_000, 100, seed=11)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=2, max_depth=11, nbins=64)
    s = lockstep_check(pkg, orc, p, x, y, rounds=2)
    assert s["splits"] > 500, s


def test_logloss(pkg, orc):
    x, y = make_regression(50_000, 20, seed=9)
    yb = (y > np.median(y)).astype(np.float32)
    p = pkg.EvoTreeRegressor(loss="logloss", nrounds=3, max_depth=5, nbins=32, eta=0.3)
    lockstep_check(pkg, orc, p, x, yb, rounds=3)


def test_softmax(pkg, orc):
    """Five-class softmax shape scaled down in rows: 28 features, 5 classes, depth 8, 64 bins."""
    x, y = _softmax_data(80_000, 28, 5)
    p = pkg.EvoTreeClassifier(nrounds=3, max_depth=8, nbins=64, eta=0.2)
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 100, s


def test_gaussian_mle(pkg, orc):
    """Gaussian maximum-likelihood shape scaled down in rows: 50 features, depth 7, 32 bins, min_weight 8."""
    rng = np.random.default_rng(17)
    n, f = 80_000, 50
    x = rng.random((n, f)).astype(np.float32)
    y = (x @ rng.normal(size=f) + np.exp(0.5 * x[:, 0]) * rng.normal(size=n)).astype(np.float32)
    p = pkg.EvoTreeMLE(nrounds=3, max_depth=7, nbins=32, eta=0.2)
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 50, s


def _positive_target(n, f, seed, kind):
    """Count / positive targets with a log-linear mean, the shapes the log-link losses are meant for."""
    rng = np.random.default_rng(seed)
    x = rng.random((n, f)).astype(np.float32)
    mu = np.exp(0.3 + x[:, :4] @ np.array([0.8, -0.6, 0.4, 0.3]))
    if kind == "poisson":
        y = rng.poisson(mu)
    elif kind == "gamma":
        y = rng.gamma(2.0, mu / 2.0) + 1e-3
    else:  # tweedie: compound poisson-gamma with exact zeros
        cnt = rng.poisson(mu)
        y = np.array([rng.gamma(2.0, 0.5, c).sum() if c > 0 else 0.0 for c in cnt])
    return x, y.astype(np.float32)


@pytest.mark.parametrize("loss", ["poisson", "gamma", "tweedie"])
def test_log_link_losses(pkg, orc, loss):
    """poisson / gamma / tweedie (src/loss.jl:59-76): gradients, log-mean bias, trees and predictions in lock-step."""
    x, y = _positive_target(40_000, 12, seed=31, kind=loss)
    p = pkg.EvoTreeRegressor(loss=loss, nrounds=3, max_depth=5, nbins=32, eta=0.3)
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 20, s


def test_evotreecount_is_poisson(pkg, orc):
    x, y = _positive_target(20_000, 8, seed=4, kind="poisson")
    p = pkg.EvoTreeCount(nrounds=2, max_depth=4, nbins=16, eta=0.3)
    assert p.loss == "poisson" and p.metric == "poisson"
    lockstep_check(pkg, orc, p, x, y, rounds=2)


def test_logistic_mle(pkg, orc):
    """Two-parameter logistic likelihood (src/loss.jl:207-217): same shape as the gaussian case."""
    rng = np.random.default_rng(23)
    n, f = 60_000, 20
    x = rng.random((n, f)).astype(np.float32)
    y = (x @ rng.normal(size=f) + np.exp(0.5 * x[:, 0]) * rng.logistic(size=n)).astype(np.float32)
    p = pkg.EvoTreeMLE(loss="logistic_mle", nrounds=3, max_depth=6, nbins=32, eta=0.2)
    assert p.metric == "logistic_mle" and pkg.EvoTreeMLE(loss="logistic").loss == "logistic_mle"
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 30, s


@pytest.mark.parametrize("loss", ["mae", "cred_var", "cred_std"])
def test_losses_with_their_own_gain_and_leaf(pkg, orc, loss):
    """mae and the credibility losses: split gain and leaf value of their own (src/split.jl:2-4, 119-141,
    src/predict.jl:211-222, 250-262), with a monotone constraint so that their pred_scalar is exercised too."""
    x, y = make_regression(40_000, 10, seed=41)
    y = y + 2.0                                         # a non-zero mean: the credibility terms depend on it
    p = pkg.EvoTreeRegressor(loss=loss, nrounds=3, max_depth=5, nbins=32, eta=0.3, L2=1.0, lambda_=0.1,
                             monotone_constraints={1: 1, 2: -1})
    assert p.metric == ("mae" if loss != "mae" else "mae")
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 10, s


@pytest.mark.parametrize("alpha,rowsample", [(0.5, 1.0), (0.1, 1.0), (0.9, 0.6)])
def test_quantile_loss(pkg, orc, alpha, rowsample):
    """Quantile loss (src/loss.jl:93-98, src/predict.jl:264-272): the gain of mae, leaf values = alpha-quantile of the
    residuals of the leaf's sampled rows, found on the device by a radix selection and by a sort in the oracle."""
    x, y = make_regression(30_000, 8, seed=int(alpha * 100))
    p = pkg.EvoTreeRegressor(loss="quantile", alpha=alpha, nrounds=3, max_depth=5, nbins=32, eta=0.5, rowsample=rowsample, L2=0.5)
    assert p.metric == "quantile"
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 10, s


def test_multiquantile_loss(pkg, orc):
    """One target, one output row per quantile (src/loss.jl:160-172, src/predict.jl:274-281): three selections per tree."""
    x, y = make_regression(30_000, 8, seed=77)
    p = pkg.EvoTreeRegressor(loss="multiquantile", alphas=(0.2, 0.5, 0.85), nrounds=3, max_depth=5, nbins=32, eta=0.5, L2=0.5)
    assert p.metric == "multiquantile"
    s = lockstep_check(pkg, orc, p, x, y, rounds=3)
    assert s["splits"] > 10, s
    m = pkg.fit(pkg.EvoTreeRegressor(loss="multiquantile", alphas=(0.2, 0.8), nrounds=30, max_depth=4, nbins=32, eta=0.3), x_train=x, y_train=y)
    q = m(x)
    assert q.shape == (30_000, 2) and abs(float(np.mean(y <= q[:, 0])) - 0.2) < 0.04 and abs(float(np.mean(y <= q[:, 1])) - 0.8) < 0.04


def test_quantile_model_covers_its_quantile(pkg):
    rng = np.random.default_rng(6)
    x = rng.random((40_000, 5)).astype(np.float32)
    y = (2 * x[:, 0] + (0.2 + x[:, 1]) * rng.normal(size=40_000)).astype(np.float32)
    for alpha in (0.2, 0.8):
        m = pkg.fit(pkg.EvoTreeRegressor(loss="quantile", alpha=alpha, nrounds=40, max_depth=5, nbins=32, eta=0.2), x_train=x, y_train=y)
        assert abs(float(np.mean(y <= m(x))) - alpha) < 0.03


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_shallow_depths(pkg, orc, depth):
    x, y = make_regression(5_000, 7, seed=depth)
    p = pkg.EvoTreeRegressor(nrounds=3, max_depth=depth, nbins=16)
    lockstep_check(pkg, orc, p, x, y, rounds=3)


@pytest.mark.parametrize("nbins,nfeats", [(2, 3), (255, 5), (100, 33), (64, 130), (17, 64)])
def test_bin_and_feature_edge_sizes(pkg, orc, nbins, nfeats):
    x, y = make_regression(20_000, nfeats, seed=nbins)
    p = pkg.EvoTreeRegressor(nrounds=2, max_depth=5, nbins=nbins)
    lockstep_check(pkg, orc, p, x, y, rounds=2)


def test_weights_and_regularisation(pkg, orc):
    x, y = make_regression(30_000, 12, seed=21)
    w = np.random.default_rng(1).uniform(0.5, 3.0, size=y.size).astype(np.float32)
    p = pkg.EvoTreeRegressor(nrounds=3, max_depth=6, nbins=32, lambda_=0.5, L2=2.0, gamma=0.1, min_weight=20.0)
    lockstep_check(pkg, orc, p, x, y, rounds=3, w=w)


def test_monotone_constraints(pkg, orc):
    x, y = make_regression(30_000, 6, seed=31)
    p = pkg.EvoTreeRegressor(nrounds=3, max_depth=5, nbins=32, monotone_constraints={1: 1, 2: -1, 4: 1})
    lockstep_check(pkg, orc, p, x, y, rounds=3)


def test_categorical_features(pkg, orc):
    """feattypes = false uses the `==` rule in the split scan, the partition and the traversal."""
    rng = np.random.default_rng(41)
    n, f, nb = 30_000, 6, 12
    x_bin = np.asfortranarray(rng.integers(1, nb + 1, size=(n, f)).astype(np.uint8))
    eff = rng.normal(size=(f, nb + 1))
    y = sum(eff[j][x_bin[:, j]] for j in range(f)).astype(np.float32) + 0.1 * rng.normal(size=n).astype(np.float32)
    ft = np.array([0, 1, 0, 1, 0, 0], np.uint8)
    p = pkg.EvoTreeRegressor(nrounds=3, max_depth=5, nbins=nb)
    lockstep_check(pkg, orc, p, None, y, rounds=3, feattypes=ft, x_bin=x_bin)


def test_bagging(pkg, orc):
    x, y = make_regression(20_000, 9, seed=51)
    p = pkg.EvoTreeRegressor(nrounds=2, max_depth=4, nbins=32, bagging_size=3, rowsample=0.7)
    s = lockstep_check(pkg, orc, p, x, y, rounds=2)
    assert s["trees"] == 6


def test_tiny_and_ragged_inputs(pkg, orc):
    for n in (1, 2, 31, 33, 2049):
        x, y = make_regression(n, 3, seed=n)
        p = pkg.EvoTreeRegressor(nrounds=2, max_depth=4, nbins=8, min_weight=0.0)
        lockstep_check(pkg, orc, p, x, y, rounds=2)


def test_empty_subsample_is_an_error(pkg):
    """`no subsample observation` (src/subsample.jl:36, test/core.jl:510-530)."""
    x, y = make_regression(50, 3)
    p = pkg.EvoTreeRegressor(nrounds=1, max_depth=3, nbins=8, rowsample=1e-9)
    with pytest.raises(pkg.EvbError, match="no subsample"):
        pkg.fit(p, x_train=x, y_train=y)


def test_bad_bins_rejected(pkg):
    x_bin = np.asfortranarray(np.full((100, 3), 9, np.uint8))
    p = pkg.EvoTreeRegressor(nrounds=1, max_depth=3, nbins=8)
    with pytest.raises(pkg.EvbError, match="outside 1..nbins"):
        pkg.init_core_binned(p, x_bin, np.zeros(100, np.float32), 1, 1, np.zeros(1, np.float32))


def test_multi_target_mse(pkg, orc):
    """Matrix target (K = 3): for mse only g_1..g_K and w are accumulated, the hessians are rebuilt from w."""
    x, y = make_regression(30_000, 11, seed=61)
    rng = np.random.default_rng(2)
    Y = np.stack([y, -0.5 * y + 0.1 * rng.normal(size=y.size), np.sin(3 * x[:, 0])], axis=1).astype(np.float32)
    p = pkg.EvoTreeRegressor(nrounds=3, max_depth=5, nbins=32, eta=0.3)
    s = lockstep_check(pkg, orc, p, x, Y, rounds=3)
    assert s["splits"] > 30, s


def test_multi_target_logloss(pkg, orc):
    """K = 2 logistic targets: five channels in two channel groups."""
    x, y = make_regression(30_000, 40, seed=62)
    Y = np.stack([(y > np.median(y)), (x[:, 1] + x[:, 2] > 1.0)], axis=1).astype(np.float32)
    p = pkg.EvoTreeRegressor(loss="logloss", nrounds=3, max_depth=5, nbins=64, eta=0.3)
    lockstep_check(pkg, orc, p, x, Y, rounds=3)


def test_softmax_many_classes(pkg, orc):
    """12 classes: 25 channels in seven channel groups, several unit groups per CTA."""
    rng = np.random.default_rng(63)
    n, f, k = 40_000, 20, 12
    x = rng.normal(size=(n, f)).astype(np.float32)
    y = (x @ rng.normal(size=(f, k)) + rng.gumbel(size=(n, k))).argmax(axis=1).astype(np.int64)
    p = pkg.EvoTreeClassifier(nrounds=2, max_depth=5, nbins=32, eta=0.3)
    s = lockstep_check(pkg, orc, p, x, y, rounds=2)
    assert s["splits"] > 20, s


# ---- oblivious trees (tree_type = :oblivious, grow_otree!, src/fit.jl:147-263; test/oblivious.jl) -----------------
def test_oblivious_mse_lockstep(pkg, orc):
    """One (feature, bin) per depth: the same trees as the oracle, node for node (fixed-point histogram kernel)."""
    x, y = make_regression(60_000, 12, seed=21, dtype=np.float64)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=4, max_depth=6, nbins=32, eta=0.2, tree_type="oblivious")
    s = lockstep_check(pkg, orc, p, x, y, rounds=4)
    assert s["splits"] >= 4 * 31 and s["diverged"] == 0, s


def test_oblivious_sampling_and_weights(pkg, orc):
    x, y = make_regression(50_000, 40, seed=22)
    w = np.random.default_rng(3).uniform(0.5, 2.0, size=x.shape[0]).astype(np.float32)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=3, max_depth=5, nbins=64, eta=0.1, rowsample=0.6, colsample=0.5,
                             tree_type="oblivious", min_weight=10.0)
    s = lockstep_check(pkg, orc, p, x, y, rounds=3, w=w)
    assert s["splits"] >= 3 * 7 and s["diverged"] == 0, s


def test_oblivious_logloss_monotone(pkg, orc):
    x, y = make_regression(40_000, 10, seed=23)
    yb = (y > np.median(y)).astype(np.float32)
    p = pkg.EvoTreeRegressor(loss="logloss", nrounds=3, max_depth=5, nbins=32, eta=0.3, tree_type="oblivious",
                             monotone_constraints={1: 1, 2: -1})
    s = lockstep_check(pkg, orc, p, x, yb, rounds=3)
    assert s["diverged"] == 0, s


def test_oblivious_softmax_and_mae(pkg, orc):
    x, yc = _softmax_data(40_000, 12, 3)
    s = lockstep_check(pkg, orc, pkg.EvoTreeClassifier(nrounds=2, max_depth=5, nbins=32, eta=0.2, tree_type="oblivious"), x, yc, rounds=2)
    assert s["splits"] >= 2 * 7 and s["diverged"] == 0, s
    x, y = make_regression(30_000, 8, seed=24)
    s = lockstep_check(pkg, orc, pkg.EvoTreeRegressor(loss="mae", nrounds=2, max_depth=4, nbins=32, tree_type="oblivious"), x, y, rounds=2)
    assert s["diverged"] == 0, s


def test_oblivious_fit_through_the_graph_path(pkg, orc):
    """`fit` (CUDA-graph replay, pipelined trees): every depth of every tree shares one split; same trees as the
    oracle's booster on the same bins; the model beats the bias model (test/oblivious.jl thresholds)."""
    x, y = make_regression(50_000, 10, seed=25)
    p = pkg.EvoTreeRegressor(loss="mse", nrounds=30, max_depth=5, nbins=32, eta=0.2, tree_type="oblivious")
    m = pkg.fit(p, x_train=x, y_train=y)
    assert len(m.trees) == 31
    for t in m.trees[1:]:
        for d in range(1, 5):
            nodes = range(2 ** (d - 1), 2 ** d)
            if t.split[2 ** (d - 1) - 1]:
                assert len({(int(t.feat[n - 1]), int(t.cond_bin[n - 1])) for n in nodes}) == 1
            else:
                assert not any(t.split[n - 1] for n in nodes)
    pred = np.asarray(m(x)).reshape(x.shape[0], -1)[:, 0]
    assert np.mean((pred - y) ** 2) < 0.25 * np.var(y)
    rng = np.random.default_rng(p.seed)
    edges, _, _ = pkg.get_edges(x, p.nbins, rng)
    xb = orc.binarize(x, edges)
    b = orc.Booster(orc.Params(loss="mse", nbins=32, max_depth=5, eta=0.2, tree_type=1), xb, y.astype(np.float32))
    js = np.arange(1, 11, dtype=np.uint32)
    same = 0
    for r in range(5):
        to = b.round(None, 255, js)[0]
        tg = m.trees[r + 1]
        same += int(np.array_equal(to.feat, tg.feat) and np.array_equal(to.cond_bin, tg.cond_bin))
    assert same == 5
