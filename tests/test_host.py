"""Host-side logic and the shape of the C ABI (no GPU needed)."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from tests.conftest import ROOT, has_gpu


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "evb.h")).read()
    return sorted(set(re.findall(r"EVB_API\s+[\w\s\*]+?\b(evb_\w+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol(pkg):
    from evotrees_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 18 and "evb_grow_tree" in names
    lib = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/evb.h but not exported"
    assert sorted(_lib.EXPORTS) == names
    assert lib.evb_version() >= 1


def test_struct_layouts_match_the_header(pkg):
    from evotrees_b200 import _lib
    src = '#include <stdio.h>\n#include "evb.h"\nint main(void){printf("%zu %zu %d\\n", sizeof(evb_params), sizeof(evb_timings), EVB_NTIMERS);return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", os.path.join(d, "t")], check=True)
        out = subprocess.run([os.path.join(d, "t")], capture_output=True, text=True, check=True).stdout.split()
    assert int(out[0]) == C.sizeof(_lib.EvbParams)
    assert int(out[1]) == C.sizeof(_lib.EvbTimings)
    assert int(out[2]) == _lib.NTIMERS == len(_lib.TIMER_NAMES)


def test_learner_defaults_and_validation(pkg):
    r = pkg.EvoTreeRegressor()
    assert (r.loss, r.nrounds, r.max_depth, r.nbins, r.eta, r.L2, r.min_weight, r.rowsample, r.seed) == \
        ("mse", 100, 6, 64, 0.1, 1.0, 1.0, 1.0, 123)                     # src/learners.jl:28-50
    assert pkg.EvoTreeMLE().min_weight == 8.0 and pkg.EvoTreeMLE().loss == "gaussian_mle"
    assert pkg.EvoTreeClassifier().loss == "mlogloss"
    assert pkg.EvoTreeRegressor(loss="linear").loss == "mse"
    for bad in (dict(nbins=1), dict(nbins=256), dict(max_depth=0), dict(rowsample=0.0), dict(colsample=1.5), dict(eta=-1),
                dict(loss="nope"), dict(tree_type="ternary"), dict(device="cpu"), dict(gamma=-1.0)):
        with pytest.raises(ValueError):
            pkg.EvoTreeRegressor(**bad)


def test_get_edges_equals_the_oracle_restatement(pkg, orc):
    for dt in (np.float32, np.float64):
        x = np.random.default_rng(1).normal(size=(70_000, 3)).astype(dt)   # > 1000 * nbins rows: sampling path
        e1, fb, ft = pkg.get_edges(x, 64, np.random.default_rng(7))
        e2 = orc.get_edges(x, 64, np.random.default_rng(7))
        assert e1.dtype == dt and np.array_equal(e1, e2)
        assert (fb == 64).all() and ft.all()
        e3, _, _ = pkg.get_edges(x[:100], 8, np.random.default_rng(7))
        assert np.array_equal(e3, orc.get_edges(x[:100], 8, np.random.default_rng(7)))
        e4, _, _ = pkg.get_edges(x[:100], 2, np.random.default_rng(7))      # one edge -> the sample minimum (src/fit-utils.jl:17-19)
        assert np.array_equal(e4, orc.get_edges(x[:100], 2, np.random.default_rng(7))) and np.array_equal(e4[:, 0], x[:100].min(axis=0))


def test_init_target(pkg, orc):
    from evotrees_b200.fit import init_target
    rng = np.random.default_rng(2)
    y = rng.normal(size=1000)
    K, yd, ycols, mu, lv, _ = init_target("mse", y, None)
    assert (K, ycols, yd.dtype) == (1, 1, np.float32) and mu[0] == pytest.approx(y.mean(), rel=1e-5)
    K, yd, ycols, mu, lv, _ = init_target("gaussian_mle", y, None)
    assert K == 2 and mu[1] == pytest.approx(orc.lib().orc_invsoftplus64(float(np.std(y.astype(np.float32), ddof=1))), rel=1e-5)
    yb = (y > 0).astype(np.float64)
    K, yd, ycols, mu, lv, _ = init_target("logloss", yb, None)
    assert mu[0] == pytest.approx(np.log(yb.mean() / (1 - yb.mean())), rel=1e-5)
    labels = np.array(["b", "a", "c", "a", "b", "a"])
    K, yd, ycols, mu, lv, _ = init_target("mlogloss", labels, None)
    assert K == 3 and lv.tolist() == ["a", "b", "c"] and yd.tolist() == [2, 1, 3, 1, 2, 1] and mu.max() == 0
    with pytest.raises(ValueError):
        init_target("mlogloss", np.array(["a", "a"]), None)
    with pytest.raises(ValueError):
        init_target("logloss", np.array([0.0, 2.0]), None)
    # oracle and product agree on the bias
    for loss, yy in (("mse", y), ("logloss", yb), ("gaussian_mle", y)):
        K, yd, _, mu, _, _ = init_target(loss, yy, None)
        np.testing.assert_allclose(mu, orc.init_pred(orc.Params(loss=loss, K=K), yd), rtol=1e-5)


def test_tree_packing_for_inference(pkg):
    from evotrees_b200.model import _pack
    m = pkg.EvoTree("mse", 1, [pkg.Tree.bias(np.array([0.5], np.float32)), pkg.Tree.empty(3, 1)], {})
    m.trees[1].split[0] = 1
    m.trees[1].feat[0] = 2
    nn, feat, cb, sp, lp = _pack(m, 2)
    assert nn == 7 and feat.shape == (2, 7) and lp[0, 0, 0] == 0.5 and sp[0].sum() == 0 and feat[1, 0] == 2
    with pytest.raises(ValueError):
        pkg.predict(m, np.zeros((1, 2)), ntree_limit=5)


def test_shard_bounds(pkg):
    from evotrees_b200.dist import shard_bounds
    for n, w in ((10, 3), (7, 8), (10_000_000, 8), (1, 2)):
        b = [shard_bounds(n, w, r) for r in range(w)]
        assert b[0][0] == 0 and b[-1][1] == n and all(b[i][1] == b[i + 1][0] for i in range(w - 1))


def test_logger_matches_oracle_rule(pkg, orc):
    """`update_logger!` + the stopping rule (src/callback.jl:146-164, src/fit.jl:429) on random metric sequences."""
    F = pkg
    rng = np.random.default_rng(5)
    for metric in ("mse", "gaussian_mle"):
        for tol in (0.0, 0.05):
            seq = np.cumsum(rng.normal(0.0 if metric == "mse" else 0.01, 0.1, 60))
            lg = F.init_logger(metric, F.IS_MAXIMISE[metric], 4, tol)
            ol = orc.Logger(metric, 4, tol)
            for it, v in enumerate(seq):
                F.update_logger(lg, it, float(v))
                stop = ol.update(it, float(v))
                assert (lg["iter_since_best"] >= lg["early_stopping_rounds"]) == stop
                assert (lg["best_iter"], lg["best_metric"], lg["iter_since_best"]) == (ol.best_iter, ol.best_metric, ol.iter_since_best)
                if stop:
                    break
            assert lg["nrounds"] == lg["iter"][-1] and lg["metrics"] == ol.metrics


def test_logger_hand_case(pkg):
    F = pkg
    lg = F.init_logger("mse", False, 2, 0.1)
    for it, v in enumerate([1.0, 0.8, 0.75, 0.72, 0.5]):   # 0.75 and 0.72 do not beat 0.8 - 0.1
        F.update_logger(lg, it, v)
        if lg["iter_since_best"] >= 2:
            break
    assert lg["best_iter"] == 1 and lg["best_metric"] == 0.8 and lg["iter"] == [0, 1, 2, 3] and lg["iter_since_best"] == 2


def test_eval_levelcode(pkg):
    F = pkg
    lv = np.array([2, 5, 9])
    assert F.eval_levelcode(np.array([9, 2, 2, 5]), lv).tolist() == [3, 1, 1, 2]
    assert F.eval_levelcode(np.array([9, 9]), lv).tolist() == [3, 3]          # an eval fold without some classes
    with pytest.raises(ValueError, match="absent from `y_train`"):
        F.eval_levelcode(np.array([2, 7, 11]), lv)


def test_metric_defaults_and_validation(pkg):
    assert pkg.EvoTreeRegressor().metric == "mse" and pkg.EvoTreeRegressor(loss="logloss").metric == "logloss"
    assert pkg.EvoTreeRegressor(metric="rmse").metric == "rmse"
    assert pkg.EvoTreeClassifier().metric == "mlogloss" and pkg.EvoTreeMLE().metric == "gaussian_mle"
    with pytest.raises(ValueError, match="Invalid metric"):
        pkg.EvoTreeClassifier(metric="mse")
    with pytest.raises(ValueError, match="early_stopping_tolerance"):
        pkg.EvoTreeRegressor(early_stopping_tolerance=-1.0)


@pytest.mark.skipif(has_gpu(), reason="checks the behaviour of a machine without a GPU")
def test_no_gpu_fails_loudly(pkg):
    x = np.random.default_rng(0).random((50, 3)).astype(np.float32)
    with pytest.raises(pkg.EvbError, match="no CPU fallback"):
        pkg.fit(pkg.EvoTreeRegressor(nrounds=1), x_train=x, y_train=x[:, 0])
    with pytest.raises(pkg.EvbError, match="no CPU fallback"):
        pkg.binarize(x, np.zeros((3, 7), np.float32))


def test_julia_glue_loss_codes_match_the_header_and_the_python_binding(pkg):
    """The Julia glue is not executed here (no Julia runtime), so its loss table is checked as text: every loss symbol it
    maps must carry the code of include/evb.h's enum and of the ctypes binding, and the model-type lookup must go through
    the reference's own symbol -> type table instead of a name transformation."""
    import re
    from evotrees_b200 import _lib
    src = open(os.path.join(ROOT, "evotrees.jl_b200", "julia", "EvoTreesB200Ext.jl")).read()
    table = src[src.index("const LOSS_CODE = Dict("):]
    table = table[:table.index(")\n") + 1]
    julia = {m.group(1): int(m.group(2)) for m in re.finditer(r":(\w+)\s*=>\s*(\d+)", table)}
    assert julia == _lib.LOSS_CODES
    header = open(os.path.join(ROOT, "include", "evb.h")).read()
    enum = header[header.index("enum evb_loss {"):]
    enum = enum[:enum.index("};")]
    codes = {m.group(1).lower(): int(m.group(2)) for m in re.finditer(r"EVB_(\w+)\s*=\s*(\d+)", enum)}
    assert codes == julia
    assert "LOSS_TYPE_CODE = Dict(T => LOSS_CODE[s] for (s, T) in _loss2type_dict)" in src
    assert "lowercase(" not in src and "LOSS_TYPE_CODE[L]" in src
