"""Parity harness: drives the CUDA library and the CPU oracle on the same inputs, tree by tree.

In lock-step mode the oracle restarts every round from the library's own predictions, so one near-tied
split that goes the other way cannot compound over rounds: each tree is judged on its own inputs.
Tolerances (stated once, used everywhere):
  * binning, row->node ids, leaf ids, split feature / bin: bit-exact;
  * histograms: |gpu - oracle| <= 1e-5 * (upper bound of sum |contribution| of the bin at the root);
  * node sums: 1e-5 relative plus the histogram bound (1e-5 x max|g| x rows of the node);
  * predictions and gradients: 1e-5 relative (+ 1e-6 absolute: float32 outputs);
  * gains and leaf values: 1e-5 of the magnitudes they are made of (a gain is children's terms minus the parent's term)
    plus what the allowed error of the node sums does to them (`_gain_tol`, `_leaf_tol`);
  * a split may differ from the oracle's only if, by the oracle's own histogram, the gain of the library's
    choice is within 1e-5 relative of the oracle's best gain (near tie); descendants of such a node and the
    rest of that round's row ids are then not compared.
"""
from __future__ import annotations

import numpy as np

RTOL = 1e-5


def oracle_params(orc, params, K):
    return orc.Params(loss=params.loss, K=K, nbins=params.nbins, max_depth=params.max_depth,
                      bagging_size=params.bagging_size, eta=params.eta, lambda_=params.lambda_, L2=params.L2,
                      gamma=params.gamma, min_weight=params.min_weight, alpha=params.alpha, alphas=tuple(params.alphas),
                      tree_type=1 if getattr(params, "tree_type", "binary") == "oblivious" else 0)


def _gain_of(op, hist_node, nsum_node, feat0, bin1, numeric=True):
    """Split gain of (feature, bin) at a node from the oracle's histogram [nfeats, B, C] (src/split.jl)."""
    C = nsum_node.size
    K = (C - 1) // 2
    h = hist_node[feat0]
    sl = h[:bin1].sum(axis=0) if numeric else h[bin1 - 1]
    eps = np.finfo(np.float64).eps

    def term(g, hh, w):
        return g * g / max(eps, hh + op.lambda_ * w + op.L2) / 2.0

    wl, wr = sl[C - 1], nsum_node[C - 1] - sl[C - 1]
    if op.loss in ("mae", "quantile", "multiquantile"):   # src/split.jl:2, 119-130
        wp = nsum_node[C - 1]
        dl, dr = max(eps, 1 + op.lambda_ + op.L2 / wl), max(eps, 1 + op.lambda_ + op.L2 / wr)
        return sum(abs(sl[k] / wl - nsum_node[k] / wp) * wl / dl + abs((nsum_node[k] - sl[k]) / wr - nsum_node[k] / wp) * wr / dr
                   for k in range(K))
    if op.loss in ("cred_var", "cred_std"):      # src/split.jl:3-4, 70-78, 132-141
        def cred(m1, m2, w):
            vhm = (m1 / w) ** 2
            evpv = max(eps, m2 / w - vhm)
            z = vhm / (vhm + evpv) if op.loss == "cred_var" else np.sqrt(vhm) / (np.sqrt(vhm) + np.sqrt(evpv))
            return z * abs(m1) / (1 + op.L2 / w)
        gp = sum(cred(nsum_node[k], nsum_node[K + k], nsum_node[C - 1]) for k in range(K))
        return sum(cred(sl[k], sl[K + k], wl) + cred(nsum_node[k] - sl[k], nsum_node[K + k] - sl[K + k], wr) for k in range(K)) - gp
    gp = sum(term(nsum_node[k], nsum_node[K + k], nsum_node[C - 1]) for k in range(K))
    g = sum(term(sl[k], sl[K + k], wl) + term(nsum_node[k] - sl[k], nsum_node[K + k] - sl[K + k], wr) for k in range(K))
    return g - gp


SUM_SLACK = 1.0   # multiplies the bound of `_sum_err`; see lockstep_check(float_sum_slack=)


def _sum_err(op, nsum_node, gmax):
    """Absolute error allowed on a node's gradient sums: 1e-5 x max|g| x (rows of the node), channel by channel -- the same
    bound the histogram comparison uses.  It covers the float32 partial sums of the float histogram kernel (whose
    error grows with the sum of |g| of the rows, not with the possibly much smaller |sum of g|); the fixed-point path is
    exact to 2^-26 of max|g| and stays far inside it."""
    C = nsum_node.size
    return SUM_SLACK * RTOL * np.asarray(gmax, np.float64)[:C] * float(nsum_node[C - 1])


def _gain_tol(op, gain, nsum_node, gmax):
    """A gain is children's terms minus the parent's term, each term G^2 / (2 D): the tolerance is 1e-5 of the terms
    (children = gain + parent, plus the parent) plus what the allowed error of the sums does to a term, |G| dG / D."""
    C = nsum_node.size
    K = (C - 1) // 2
    eps = np.finfo(np.float64).eps
    w = float(nsum_node[C - 1])
    if op.loss in ("mae", "quantile", "multiquantile", "cred_var", "cred_std"):
        scale = abs(gain) + float(np.abs(nsum_node[:K]).sum())
        return RTOL * scale + (float(_sum_err(op, nsum_node, gmax)[:K].sum()) if gmax is not None else 0.0) + 1e-6
    d = [max(eps, nsum_node[K + k] + op.lambda_ * w + op.L2) for k in range(K)]
    scale = abs(gain) + 2.0 * float(sum(nsum_node[k] ** 2 / d[k] / 2.0 for k in range(K)))
    extra = 0.0
    if gmax is not None:
        e = _sum_err(op, nsum_node, gmax)
        extra = float(sum(2.0 * abs(nsum_node[k]) * e[k] / d[k] for k in range(K)))   # parent + children: twice |G| dG / D
    return RTOL * scale + extra + 1e-6


def _leaf_tol(op, leaf, nsum_node, gmax, k):
    """Leaf k = -eta G_k / D_k: 1e-5 relative + 1e-6 (float32 output) + eta dG / D for the allowed error of the sum."""
    C = nsum_node.size
    K = (C - 1) // 2
    tol = RTOL * abs(float(leaf)) + 1e-6
    if gmax is not None and op.loss not in ("mae", "quantile", "multiquantile", "cred_var", "cred_std"):
        w = float(nsum_node[C - 1])
        if op.loss in ("gaussian_mle", "logistic_mle"):   # channels g_mu, g_phi, h_mu, h_phi (one target)
            hk = nsum_node[K + k]
        else:
            hk = nsum_node[K + k]
        d = max(np.finfo(np.float64).eps, hk + op.lambda_ * w + op.L2)
        tol += op.eta / op.bagging_size * float(_sum_err(op, nsum_node, gmax)[k]) / d
    return tol


def compare_tree(op, tg, to, ohist, onsum, feattypes=None, gmax=None):
    """Node-by-node comparison.  Returns (n_compared, diverged_nodes)."""
    nn = to.feat.size
    skip = np.zeros(nn + 1, bool)
    diverged = []
    compared = 0
    for n in range(1, nn + 1):
        if skip[n]:
            if 2 * n + 1 <= nn:
                skip[2 * n] = skip[2 * n + 1] = True
            continue
        sg, so = bool(tg.split[n - 1]), bool(to.split[n - 1])
        reached = to.w[n - 1] != 0 or tg.w[n - 1] != 0 or n == 1
        if not reached:
            assert not sg and not so
            continue
        compared += 1
        np.testing.assert_allclose(tg.w[n - 1], to.w[n - 1], rtol=RTOL, atol=1e-6, err_msg=f"node weight {n}")
        same = sg == so and (not sg or (tg.feat[n - 1] == to.feat[n - 1] and tg.cond_bin[n - 1] == to.cond_bin[n - 1]))
        if same:
            if sg:
                tol = _gain_tol(op, float(to.gain[n - 1]), onsum[n - 1], gmax)
                assert abs(float(tg.gain[n - 1]) - float(to.gain[n - 1])) <= tol, f"gain {n}: {tg.gain[n - 1]} vs {to.gain[n - 1]} (allowed {tol})"
            else:
                for k in range(to.pred.shape[1]):
                    tol = _leaf_tol(op, to.pred[n - 1, k], onsum[n - 1], gmax, k)
                    assert abs(float(tg.pred[n - 1, k]) - float(to.pred[n - 1, k])) <= tol, f"leaf {n}[{k}]: {tg.pred[n - 1]} vs {to.pred[n - 1]} (allowed {tol})"
            continue
        # structural difference: only acceptable as a near tie by the oracle's own numbers
        assert op.tree_type == 0, f"oblivious tree differs at node {n} (the level's split is a sum over nodes: no per-node tie rule)"
        assert ohist is not None, f"tree differs at node {n} and no oracle histogram to arbitrate"
        best = float(to.gain[n - 1]) if so else op.gamma
        if sg:
            f0 = int(tg.feat[n - 1]) - 1
            num = True if feattypes is None else bool(feattypes[f0])
            alt = _gain_of(op, ohist[n - 1], onsum[n - 1], f0, int(tg.cond_bin[n - 1]), num)
        else:
            alt = op.gamma
        scale = max(abs(best), abs(alt), 1e-12)
        assert abs(best - alt) <= RTOL * scale, (
            f"node {n}: library split (feat {tg.feat[n-1]}, bin {tg.cond_bin[n-1]}, split={sg}) has oracle gain {alt}, "
            f"oracle best (feat {to.feat[n-1]}, bin {to.cond_bin[n-1]}, split={so}) {best}")
        diverged.append(n)
        if 2 * n + 1 <= nn:
            skip[2 * n] = skip[2 * n + 1] = True
    return compared, diverged


def compare_hist(hg, ho, gmax, wmin, wroot):
    """hg, ho [njs, B, C].  The library accumulates float32 partial sums and gets half of the nodes by
    parent - sibling subtraction, so its absolute error in a bin is set by the bin's population in the
    ancestor where the chain of subtractions started (at most the root).  Bound used:
    sum|contribution| <= gmax[c] * (root w_bin / wmin)."""
    wbin = wroot[:, :, -1:]
    atol = RTOL * gmax[None, None, :] * (wbin / wmin) + 1e-12
    err = np.abs(hg - ho)
    bad = err > atol
    assert not bad.any(), f"histogram mismatch: max err {err.max()} (allowed {atol[bad].min()}) at {np.argwhere(bad)[:5]}"
    return float((err / np.maximum(atol, 1e-300)).max())


def lockstep_check(pkg, orc, params, x, y, rounds, w=None, feattypes=None, x_bin=None, check_hist=True,
                   max_diverged_frac=0.02, device=0, hist_nodes=None, float_sum_slack=1.0):
    """Grow `rounds` boosting rounds on the GPU; after each tree, rebuild the same tree with the oracle from
    the library's own pre-round state and compare everything.  Returns summary statistics.
    `float_sum_slack` widens the allowed error of the node sums (and what follows from them: gains, leaves) for the
    float histogram kernel on millions of rows, whose float32 partial sums -- inherited through parent - sibling
    subtractions -- reach a few 1e-5 of max|g| x rows there; the fixed-point path never needs it."""
    global SUM_SLACK
    SUM_SLACK = float(float_sum_slack)
    from evotrees_b200 import _lib
    from evotrees_b200.fit import init_target

    rng = np.random.default_rng(params.seed)
    if x_bin is None:
        edges, _, _ = pkg.get_edges(x, params.nbins, rng)
        x_bin = pkg.binarize(x, edges, device)
        xb_cpu = orc.binarize(x, edges)
        assert np.array_equal(x_bin, xb_cpu), "device binarize differs from the oracle"
    nobs, nfeats = x_bin.shape
    K, yd, ycols, mu, _, _ = init_target(params.loss, y, None, params.alphas)
    op = oracle_params(orc, params, K)
    flags = _lib.FLAG_FULL_PARTITION | _lib.FLAG_KEEP_ALL_HIST | _lib.FLAG_TIMING
    cache = pkg.init_core_binned(params, x_bin, yd, ycols, K, mu, w, None, feattypes, device, flags)
    C = 2 * K + 1
    grad = np.zeros((nobs, C), np.float32)
    grad[:, -1] = 1.0 if w is None else w
    wmin = float(grad[:, -1].min())
    pred_prev = np.tile(mu, (nobs, 1)).astype(np.float32)
    stats = {"rounds": 0, "trees": 0, "nodes_compared": 0, "diverged": 0, "hist_worst": 0.0, "splits": 0}
    try:
        for r in range(rounds):
            orc.update_grads(op, pred_prev, yd, grad)
            for b in range(params.bagging_size):
                mask, js = pkg.sample_round(cache, params)
                tg = pkg.grow_tree(cache, params, mask, js, update_grads=(b == 0))
                is_ = (np.arange(1, nobs + 1, dtype=np.uint32) if mask is None
                       else (np.nonzero(mask <= cache.mask_cond)[0] + 1).astype(np.uint32))
                to, onidx, ohist, onsum = orc.grow_tree(op, x_bin, grad, is_, js, feattypes,
                                                        _mono(params, nfeats), want_hist=True)
                ncmp, div = compare_tree(op, tg, to, ohist, onsum, feattypes, gmax=np.abs(grad).max(axis=0).astype(np.float64))
                stats["nodes_compared"] += ncmp
                stats["diverged"] += len(div)
                stats["splits"] += int(tg.split.sum())
                stats["trees"] += 1
                if check_hist:
                    gmax = np.abs(grad).max(axis=0).astype(np.float64)
                    j0 = js.astype(np.int64) - 1
                    nkeep = 2 ** (params.max_depth - 1) if params.max_depth > 1 else 1
                    dead = _descendants(div, to.feat.size)
                    for n in range(1, nkeep if hist_nodes is None else min(nkeep, hist_nodes)):
                        if to.split[n - 1] or tg.split[n - 1] or n == 1:
                            if n in dead or (to.w[n - 1] == 0 and n != 1):
                                continue
                            hg = cache.hist(n, js.size, params.nbins)
                            stats["hist_worst"] = max(stats["hist_worst"], compare_hist(hg, ohist[n - 1][j0], gmax, wmin, ohist[0][j0]))
                if not div:
                    assert np.array_equal(cache.nidx(from_partition=True), onidx), "row->node ids from the partition differ"
                    leaf = orc.leaf_idx(x_bin, to, feattypes)
                    assert np.array_equal(cache.nidx(from_partition=False), leaf), "leaf ids from the traversal differ"
                    # float32 partial sums: the absolute error scales with sum|g| <= gmax * (root rows)
                    gs, os_ = cache.node_sums()[to.w != 0], onsum[to.w != 0]
                    atol = RTOL * np.abs(grad).max(axis=0).astype(np.float64) * (onsum[0, -1] / wmin)
                    assert (np.abs(gs - os_) <= RTOL * np.abs(os_) + atol[None, :]).all(), "node sums"
                # the library's own tree, applied by the oracle's predict!, must reproduce the library's predictions
                orc_tree = orc.Tree(tg.feat, tg.cond_bin, tg.w, tg.gain, tg.pred, tg.split.astype(np.uint8))
                orc.predict_tree(op, x_bin, orc_tree, pred_prev, feattypes)
                pg = cache.pred()
                np.testing.assert_allclose(pg, pred_prev, rtol=RTOL, atol=1e-6, err_msg="training predictions")
                pred_prev = pg
            # gradients of the next round were produced inside the last evb_grow_tree of this round
            gnext = grad.copy()
            orc.update_grads(op, pred_prev, yd, gnext)
            np.testing.assert_allclose(cache.grads(), gnext, rtol=RTOL, atol=1e-6, err_msg="gradients")
            stats["rounds"] += 1
        assert stats["diverged"] <= max(1, max_diverged_frac * stats["nodes_compared"]), f"too many near-tie divergences: {stats}"
        stats["timings"] = cache.timings()
    finally:
        cache.close()
    return stats


def _mono(params, nfeats):
    if not params.monotone_constraints:
        return None
    mono = np.zeros(nfeats, np.int32)
    for k, v in params.monotone_constraints.items():
        mono[int(k) - 1] = int(v)
    return mono


def _descendants(nodes, nn):
    out = set()
    stack = list(nodes)
    while stack:
        n = stack.pop()
        for c in (2 * n, 2 * n + 1):
            if c <= nn and c not in out:
                out.add(c)
                stack.append(c)
    return out


def make_regression(n, f, seed=123, dtype=np.float32):
    rng = np.random.default_rng(seed)
    x = rng.random((n, f)).astype(dtype)
    beta = rng.normal(size=f)
    y = (x.astype(np.float64) @ beta + 0.1 * rng.normal(size=n)).astype(np.float32)
    return x, y
