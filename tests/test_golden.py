"""Committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py):
the oracle must keep reproducing them (CPU), and the CUDA library must match them (GPU)."""
import os

import numpy as np
import pytest

from tests.conftest import ROOT
from tests.golden.make_golden import CASES, ROUNDS

GOLD = os.path.join(ROOT, "tests", "golden")


def _load(loss):
    return np.load(os.path.join(GOLD, f"{loss}.npz"))


@pytest.mark.parametrize("loss", list(CASES))
def test_oracle_reproduces_golden(orc, loss):
    c, g = CASES[loss], _load(loss)
    p = orc.Params(loss=loss, K=c["K"], nbins=c["nbins"], max_depth=c["depth"], eta=c["eta"], min_weight=c.get("min_weight", 1.0))
    b = orc.Booster(p, np.asfortranarray(g["x_bin"]), g["y"], g["w"])
    np.testing.assert_allclose(b.mu, g["mu"], rtol=1e-6)
    for r in range(ROUNDS):
        mask = g[f"mask{r}"]
        t, nidx, _, _ = b.round(mask if mask.size else None, int(g["mask_cond"]), g[f"js{r}"])
        assert np.array_equal(t.feat, g[f"feat{r}"]) and np.array_equal(t.cond_bin, g[f"cond_bin{r}"])
        assert np.array_equal(t.split, g[f"split{r}"]) and np.array_equal(nidx, g[f"nidx{r}"])
        np.testing.assert_allclose(t.gain, g[f"gain{r}"], rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(t.pred, g[f"leaf{r}"], rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(b.pred, g[f"pred{r}"], rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("loss", list(CASES))
def test_library_matches_golden(pkg, loss):
    from evotrees_b200 import _lib
    c, g = CASES[loss], _load(loss)
    learner = {"mlogloss": pkg.EvoTreeClassifier, "gaussian_mle": pkg.EvoTreeMLE}.get(loss, pkg.EvoTreeRegressor)
    params = learner(loss=loss, nrounds=ROUNDS, max_depth=c["depth"], nbins=c["nbins"], eta=c["eta"],
                     min_weight=c.get("min_weight", 1.0), rowsample=c["rowsample"], colsample=c["colsample"])
    x_bin = np.asfortranarray(g["x_bin"])
    cache = pkg.init_core_binned(params, x_bin, g["y"], 1, c["K"], g["mu"], g["w"], None, None, 0, _lib.FLAG_FULL_PARTITION)
    try:
        for r in range(ROUNDS):
            mask = g[f"mask{r}"]
            t = pkg.grow_tree(cache, params, mask if mask.size else None, g[f"js{r}"], True)
            # bit-exact: structure and row -> node ids
            assert np.array_equal(t.feat, g[f"feat{r}"]) and np.array_equal(t.cond_bin, g[f"cond_bin{r}"])
            assert np.array_equal(t.split.astype(np.uint8), g[f"split{r}"])
            assert np.array_equal(cache.nidx(from_partition=True), g[f"nidx{r}"])
            # 1e-5 relative: gains, node weights, leaf values, predictions
            np.testing.assert_allclose(t.gain, g[f"gain{r}"], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(t.w, g[f"w{r}"], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(t.pred, g[f"leaf{r}"], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(cache.pred(), g[f"pred{r}"], rtol=1e-5, atol=1e-5)
    finally:
        cache.close()
