"""Host side of the row-sharded path with two gloo ranks on CPU: shard bounds, bias from sufficient statistics,
broadcast of edges, and the additivity that the device path relies on (histograms and child row counts of the
shards sum to those of the whole data set, so every rank takes the same split and build/subtract decisions)."""
import os
import sys

import numpy as np
import pytest

from tests.conftest import ROOT


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as g
    g.load_package()
    from evotrees_b200.dist import Comm, shard_bounds
    from evotrees_b200.fit import init_target
    from oracle import evo_oracle as orc
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Comm(dist)
    rng = np.random.default_rng(11)
    n, f, nbins = 5001, 4, 16
    x = rng.random((n, f))
    y = (x @ np.array([1.0, -2.0, 0.5, 0.0]) + 0.1 * rng.normal(size=n)).astype(np.float32)
    lo, hi = shard_bounds(n, world, rank)
    xs, ys = x[lo:hi], y[lo:hi]
    # edges come from rank 0 and are identical everywhere
    edges = orc.get_edges(xs, nbins, np.random.default_rng(1)) if rank == 0 else np.zeros((f, nbins - 1))
    edges = comm.broadcast_host(edges)
    out = {"edges": edges}
    for loss in ("mse", "gaussian_mle", "logloss", "mlogloss"):
        yy = ys if loss in ("mse", "gaussian_mle") else (ys > 0).astype(np.float32)
        if loss == "mlogloss":
            yy = (ys > 0).astype(np.int64) + (ys > 1).astype(np.int64)
        K, yd, _, mu_local, _, _ = init_target(loss, yy, None)
        out["mu_" + loss] = comm.allreduce_bias(loss, yd, mu_local, K)
    # shard histograms of the root sum to the global histogram; so do the child row counts of a split
    xb = orc.binarize(xs, edges)
    g = (2 * (ys.mean() - ys)).astype(np.float64)
    h = np.stack([np.bincount(xb[:, j].astype(np.int64) - 1, weights=g, minlength=nbins) for j in range(f)])
    out["hist"] = comm.allreduce_sum(h)
    out["nleft"] = comm.allreduce_sum(np.array([(xb[:, 0] <= 7).sum()]))
    # evaluation shards: every rank holds the metric sums of its rows, the logged metric is the ratio of the added sums
    from evotrees_b200.fit import metric_from_sums, allreduce_bias_losses
    w = rng.uniform(0.5, 2.0, n).astype(np.float32)[lo:hi]
    p = (ys + 0.3).astype(np.float32)
    sums = (float(np.sum(w.astype(np.float64) * (p.astype(np.float64) - ys) ** 2)), float(w.astype(np.float64).sum()))
    out["eval_mse"] = np.array([metric_from_sums("mse", sums, comm), metric_from_sums("rmse", sums, comm)])
    for loss in allreduce_bias_losses:
        yy = np.abs(ys) + 0.1
        K, yd, _, mu_local, _, _ = init_target(loss, yy, None, (0.1, 0.5, 0.9))
        out["mu_" + loss] = comm.allreduce_bias(loss, yd, mu_local, K, (0.1, 0.5, 0.9))
    # uneven shards (5001 rows over 2 ranks), row and column sampling: every rank must draw the same `js` in every round,
    # because the ranks' histograms are added slot by slot; the row masks are per rank
    from evotrees_b200.fit import Cache, make_rngs, sample_round
    import evotrees_b200 as pkg
    params = pkg.EvoTreeRegressor(loss="mse", rowsample=0.5, colsample=0.5, seed=77)
    c = Cache()
    c.nobs, c.nfeats, c.njs, c.use_mask = hi - lo, 40, 20, True
    c.rng, c.rng_js = make_rngs(params.seed, rank)
    draws = [sample_round(c, params) for _ in range(6)]
    assert all(m.size == hi - lo for m, _ in draws)
    out["js_rounds"] = np.stack([js for _, js in draws])
    np.savez(os.path.join(tmp, f"r{rank}.npz"), **out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_host_plumbing(tmp_path, orc, pkg):
    import torch.multiprocessing as mp
    from evotrees_b200.fit import init_target
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), f"ranks disagree on {k}"
    rng = np.random.default_rng(11)
    n, f, nbins = 5001, 4, 16
    x = rng.random((n, f))
    y = (x @ np.array([1.0, -2.0, 0.5, 0.0]) + 0.1 * rng.normal(size=n)).astype(np.float32)
    K, yd, _, mu, _, _ = init_target("mse", y, None)
    assert r0["js_rounds"].shape == (6, 20) and len({tuple(r) for r in r0["js_rounds"]}) > 1   # equal on both ranks (above), not constant
    np.testing.assert_allclose(r0["mu_mse"], mu, rtol=1e-6)
    K, yd, _, mu, _, _ = init_target("gaussian_mle", y, None)
    np.testing.assert_allclose(r0["mu_gaussian_mle"], mu, rtol=1e-5)
    K, yd, _, mu, _, _ = init_target("logloss", (y > 0).astype(np.float32), None)
    np.testing.assert_allclose(r0["mu_logloss"], mu, rtol=1e-5)
    K, yd, _, mu, _, _ = init_target("mlogloss", (y > 0).astype(np.int64) + (y > 1).astype(np.int64), None)
    np.testing.assert_allclose(r0["mu_mlogloss"], mu, rtol=1e-5, atol=1e-6)
    xb = orc.binarize(x, r0["edges"])
    per = -(-n // 2)
    gfull = np.concatenate([2 * (y[:per].mean() - y[:per]), 2 * (y[per:].mean() - y[per:])]).astype(np.float64)
    hfull = np.stack([np.bincount(xb[:, j].astype(np.int64) - 1, weights=gfull, minlength=nbins) for j in range(f)])
    np.testing.assert_allclose(r0["hist"], hfull, rtol=1e-12, atol=1e-9)
    assert int(r0["nleft"][0]) == int((xb[:, 0] <= 7).sum())
    w = rng.uniform(0.5, 2.0, n).astype(np.float32).astype(np.float64)
    mse = np.sum(w * 0.09) / w.sum()
    np.testing.assert_allclose(r0["eval_mse"], [mse, np.sqrt(mse)], rtol=1e-5)
    from evotrees_b200.fit import allreduce_bias_losses
    for loss in allreduce_bias_losses:   # the bias of the added losses from per-shard statistics == the bias of the whole
        K, yd, _, mu, _, _ = init_target(loss, np.abs(y) + 0.1, None, (0.1, 0.5, 0.9))
        np.testing.assert_allclose(r0["mu_" + loss], mu, rtol=1e-5, atol=1e-6)
