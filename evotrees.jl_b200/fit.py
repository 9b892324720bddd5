"""Training driver mirroring `init_core` / `grow_evotree!` / `fit` of the reference's GPU extension
(ext/EvoTreesKernelAbstractionsExt/init.jl:1-151, ext/.../fit.jl:1-21, src/fit.jl:388-437).

The host keeps what the reference keeps on the host: the RNG (row mask bytes, column sample), the quantile
edges, the initial bias and the `Tree` containers.  Everything else happens behind `evb_grow_tree`.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib
from .binning import binarize, get_edges
from .learners import EvoTypes
from .model import EvoTree, Tree


def _logit(x):
    return np.log(x / (1 - x))


def _invsoftplus(x):
    return x + math.log(-math.expm1(-x))  # src/loss.jl:266-268


def init_target(loss: str, y_train: np.ndarray, offset, alphas=(0.1, 0.5, 0.9)):
    """`_init_target` (src/init.jl:10-146) for the losses of this path.
    Returns K, y (device dtype), ycols, mu float32 [K], target_levels, offset (link space)."""
    levels = None
    if loss in ("mse", "logloss", "poisson", "gamma", "tweedie", "mae", "cred_var", "cred_std", "quantile"):
        y = np.ascontiguousarray(y_train, np.float32)
        ycols = 1 if y.ndim == 1 else y.shape[1]
        K = ycols
        m = y.reshape(y.shape[0], -1).mean(axis=0, dtype=np.float32)
        if loss == "logloss":
            if y.min() < 0 or y.max() > 1:
                raise ValueError("logloss targets must lie in [0, 1]")
            mu = _logit(m).astype(np.float32)
            if offset is not None:
                offset = _logit(offset)
        elif loss in ("poisson", "gamma", "tweedie"):          # log link (src/init.jl:31-42)
            mu = np.log(m).astype(np.float32)
            if offset is not None:
                offset = np.log(offset)
        else:
            mu = m.astype(np.float32)
    elif loss == "multiquantile":                             # src/init.jl:99-103: one target, one row per quantile
        y = np.ascontiguousarray(y_train, np.float32)
        if y.ndim != 1:
            raise ValueError("multiquantile takes a vector target")
        ycols, K = 1, len(alphas)
        mu = np.quantile(y.astype(np.float64), alphas).astype(np.float32)
    elif loss == "mlogloss":
        yt = np.asarray(y_train)
        if yt.ndim != 1 or not (np.issubdtype(yt.dtype, np.integer) or yt.dtype == bool or yt.dtype.kind in "US"):
            raise ValueError(f"Invalid target eltype: {yt.dtype}")
        levels, codes = np.unique(yt, return_inverse=True)
        K = int(levels.size)
        if K < 2:
            raise ValueError(f"Classification requires a target with at least 2 levels, got {K}")
        y = (codes + 1).astype(np.uint32)
        ycols = 1
        prop = np.bincount(codes, minlength=K) / codes.size
        mu = np.log(prop).astype(np.float32)
        mu -= mu.max()
        if offset is not None:
            offset = np.log(offset)
    elif loss in ("gaussian_mle", "logistic_mle"):
        y = np.ascontiguousarray(y_train, np.float32)
        ycols = 1 if y.ndim == 1 else y.shape[1]
        K = 2 * ycols
        y2 = y.reshape(y.shape[0], -1)
        mu = np.empty(K, np.float32)
        sd_factor = math.sqrt(3.0) / math.pi if loss == "logistic_mle" else 1.0   # src/init.jl:86, 95
        for t in range(ycols):
            mu[2 * t] = y2[:, t].mean(dtype=np.float32)
            mu[2 * t + 1] = _invsoftplus(float(np.std(y2[:, t].astype(np.float64), ddof=1)) * sd_factor)
        if offset is not None:
            offset = np.array(offset, np.float32, copy=True)
            offset[:, 1::2] = [[_invsoftplus(float(v)) for v in row] for row in offset[:, 1::2]]
    else:
        raise ValueError(loss)
    return K, y, ycols, mu.astype(np.float32), levels, offset


class Cache:
    """Training cache: owns the device handle (counterpart of `CacheBaseGPU`,
    ext/EvoTreesKernelAbstractionsExt/structs.jl).  It survives `fit` so that boosting can be resumed
    (the reference's MLJ `update`, src/MLJ.jl:38-57)."""

    def __init__(self):
        self.handle = C.c_void_p()
        self.rng = None
        self.nobs = self.nfeats = 0
        self.njs = 0
        self.mask_cond = 255
        self.use_mask = False
        self.K = 1
        self.nn = 0
        self.feature_names = None

    def close(self):
        if self.handle:
            _lib.lib().evb_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # read-backs used by the parity tests
    def pred(self):
        out = np.empty((self.nobs, self.K), np.float32)
        _lib.check(_lib.lib().evb_get_pred(self.handle, _lib.ptr(out)))
        return out

    def grads(self):
        out = np.empty((self.nobs, 2 * self.K + 1), np.float32)
        _lib.check(_lib.lib().evb_get_grads(self.handle, _lib.ptr(out)))
        return out

    def nidx(self, from_partition: bool = False):
        out = np.empty(self.nobs, np.uint32)
        _lib.check(_lib.lib().evb_get_nidx(self.handle, _lib.ptr(out), C.c_int32(1 if from_partition else 0)))
        return out

    def hist(self, node: int, njs: int, nbins: int):
        out = np.empty((njs, nbins, 2 * self.K + 1), np.float64)  # == Julia [C, B, njs]
        _lib.check(_lib.lib().evb_get_hist(self.handle, C.c_int32(node), _lib.ptr(out)))
        return out

    def node_sums(self):
        out = np.empty((self.nn, 2 * self.K + 1), np.float64)
        _lib.check(_lib.lib().evb_get_node_sums(self.handle, _lib.ptr(out)))
        return out

    def timings(self) -> dict:
        t = _lib.EvbTimings()
        _lib.check(_lib.lib().evb_get_timings(self.handle, C.byref(t)))
        return {"ms": {n: t.ms[i] for i, n in enumerate(_lib.TIMER_NAMES)},
                "launches": {n: t.launches[i] for i, n in enumerate(_lib.TIMER_NAMES)},
                "hist_rows": t.hist_rows, "hist_nodes": t.hist_nodes, "trees": t.trees}

    def stream(self) -> int:
        """cudaStream_t of the handle as an integer (e.g. for torch.cuda.ExternalStream)."""
        out = C.c_void_p()
        _lib.check(_lib.lib().evb_get_stream(self.handle, C.byref(out)))
        return out.value or 0

    def set_timing(self, on: bool):
        _lib.check(_lib.lib().evb_set_timing(self.handle, C.c_int32(1 if on else 0)))

    def reset_timings(self):
        _lib.check(_lib.lib().evb_reset_timings(self.handle))


def make_rngs(seed: int, rank: int = 0):
    """Generators of one rank: row masks come from a per-rank stream; the column sample from a stream of its own that
    depends on the seed only, so that every rank of a sharded fit draws the same `js` whatever its shard size is
    (the library sums the ranks' histograms slot by slot)."""
    return np.random.default_rng([seed, rank]), np.random.default_rng([seed, 0x6A73])


def make_params(params: EvoTypes, K: int, device: int, flags: int = 0) -> _lib.EvbParams:
    return _lib.EvbParams(_lib.LOSS_CODES[params.loss], K, params.nbins, params.max_depth, params.bagging_size,
                          1 if params.tree_type == "oblivious" else 0, params.eta, params.lambda_, params.L2, params.gamma, params.min_weight, device, flags, params.alpha,
                          (C.c_double * 8)(*(list(params.alphas) + [0.0] * 8)[:8]))


def init_core_binned(params: EvoTypes, x_bin: np.ndarray, y, ycols: int, K: int, mu: np.ndarray, w=None, pred0=None,
                     feattypes=None, device: int = 0, flags: int = 0, comm=None, x_raw=None, edges=None) -> Cache:
    """Creates the device handle from an already binned matrix (uint8, Fortran order, values 1..nbins), or -- with
    `x_raw` (float32 / float64, Fortran order) and `edges` [nfeats, nbins - 1] -- from the raw features, which are then
    binarized on the device (`evb_create_x`)."""
    if x_raw is None:
        assert x_bin.dtype == np.uint8 and x_bin.flags.f_contiguous
        nobs, nfeats = x_bin.shape
    else:
        assert x_raw.dtype in (np.float32, np.float64) and x_raw.flags.f_contiguous
        nobs, nfeats = x_raw.shape
    cache = Cache()
    cache.nobs, cache.nfeats, cache.K, cache.nn = nobs, nfeats, K, 2 ** params.max_depth - 1
    cache.njs = math.ceil(params.colsample * nfeats)            # src/init.jl:181
    cache.mask_cond = int(np.uint8(round(255 * params.rowsample)))  # src/subsample.jl:9
    cache.use_mask = params.rowsample < 1.0
    cache.rng, cache.rng_js = make_rngs(params.seed, 0 if comm is None else comm.rank)
    mono = np.zeros(nfeats, np.int32)
    for k, v in params.monotone_constraints.items():
        mono[int(k) - 1] = int(v)
    ft = None if feattypes is None else np.ascontiguousarray(feattypes, np.uint8)
    w32 = None if w is None else np.ascontiguousarray(w, np.float32)
    if w32 is not None and (w32.size != nobs or w32.min() <= 0):
        raise ValueError("weights must be positive and of length nobs")   # src/init.jl:165
    p0 = None if pred0 is None else np.ascontiguousarray(pred0, np.float32)
    cp = make_params(params, K, device, flags)
    ydt = _lib.EVB_U32 if params.loss == "mlogloss" else _lib.EVB_F32
    mu32 = np.ascontiguousarray(mu, np.float32)
    if x_raw is None:
        _lib.check(_lib.lib().evb_create(C.byref(cache.handle), C.byref(cp), C.c_int64(nobs), C.c_int32(nfeats), _lib.ptr(x_bin),
                                         _lib.ptr(y), C.c_int32(ydt), C.c_int32(ycols), _lib.ptr(w32), _lib.ptr(p0), _lib.ptr(mu32),
                                         _lib.ptr(ft), _lib.ptr(mono)))
    else:
        e = np.ascontiguousarray(edges, dtype=x_raw.dtype)  # [nfeats, nedges] C order == [nedges x nfeats] column-major
        xdt = _lib.EVB_F32 if x_raw.dtype == np.float32 else _lib.EVB_F64
        try:
            _lib.check(_lib.lib().evb_create_x(C.byref(cache.handle), C.byref(cp), C.c_int64(nobs), C.c_int32(nfeats), _lib.ptr(x_raw),
                                               C.c_int32(xdt), _lib.ptr(e), C.c_int32(e.shape[1]), _lib.ptr(y), C.c_int32(ydt),
                                               C.c_int32(ycols), _lib.ptr(w32), _lib.ptr(p0), _lib.ptr(mu32), _lib.ptr(ft), _lib.ptr(mono)))
        except _lib.EvbError as err:
            if "NaN" in str(err):
                raise ValueError("missing / NaN feature values are not supported") from err   # test/missings.jl
            raise
    if comm is not None:
        comm.attach(cache)
    return cache


def init_core(params: EvoTypes, x_train: np.ndarray, y_train, w_train=None, offset_train=None, feature_names=None,
              device: int = 0, flags: int = 0, comm=None):
    """`init_core(params, ::Type{<:GPU}, ...)`: edges + binarize + target / bias initialisation + device cache.
    Returns (EvoTree, Cache).  With `comm` (multi-GPU) `x_train` / `y_train` are this rank's row shard and
    the edges and the bias are computed from rank 0's shard and broadcast."""
    x_train = np.asarray(x_train)
    if x_train.dtype not in (np.float32, np.float64):
        x_train = x_train.astype(np.float64)
    x_train = np.asfortranarray(x_train)      # a Julia Matrix is column-major; no copy when it already is
    nobs, nfeats = x_train.shape
    rng = np.random.default_rng(params.seed)
    edges, featbins, feattypes = get_edges(x_train, params.nbins, rng)
    if np.isnan(edges).any():                 # the device check below covers the rows the sample did not see
        raise ValueError("missing / NaN feature values are not supported")   # test/missings.jl
    offset = None if offset_train is None else np.array(offset_train, np.float32, copy=True).reshape(nobs, -1)
    K, y, ycols, mu, levels, offset = init_target(params.loss, y_train, offset, params.alphas)
    if comm is not None:
        edges, mu = comm.broadcast_host(edges), comm.allreduce_bias(params.loss, y, mu, K, params.alphas)
    pred0 = None
    if offset is not None:
        mu = np.zeros_like(mu)                                               # src/init.jl:164
        pred0 = np.ascontiguousarray(np.broadcast_to(mu, (nobs, K)) + offset, np.float32)
    # `binarize(x_train; edges)` runs on the device inside evb_create_x: raw features up, bins never down
    cache = init_core_binned(params, None, y, ycols, K, mu, w_train, pred0, feattypes, device, flags, comm, x_raw=x_train, edges=edges)
    names = [f"feat_{i + 1}" for i in range(nfeats)] if feature_names is None else [str(s) for s in feature_names]
    if len(names) != nfeats:
        raise ValueError("feature_names must have one entry per column of x_train")
    cache.feature_names = names
    info = {"nrounds": 0, "feature_names": names, "target_levels": levels, "edges": edges, "featbins": featbins,
            "feattypes": feattypes}
    m = EvoTree(params.loss, K, [Tree.bias(mu)], info)
    return m, cache


def sample_round(cache: Cache, params: EvoTypes):
    """Row mask bytes and the ascending column sample of one bag (src/subsample.jl:7, src/fit.jl:16).
    The mask is only drawn when rowsample < 1: with rowsample == 1 every byte passes `mask <= 255`."""
    mask = cache.rng.integers(0, 256, size=cache.nobs, dtype=np.uint8) if cache.use_mask else None
    if cache.njs >= cache.nfeats:
        js = np.arange(1, cache.nfeats + 1, dtype=np.uint32)
    else:
        js = (np.sort(cache.rng_js.choice(cache.nfeats, size=cache.njs, replace=False)) + 1).astype(np.uint32)
    return mask, js


def grow_tree(cache: Cache, params: EvoTypes, mask, js, update_grads: bool) -> Tree:
    """One `evb_grow_tree` call; returns the tree with the reference's `Tree` layout."""
    t = Tree.empty(params.max_depth, cache.K)
    js = np.ascontiguousarray(js, np.uint32)
    _lib.check(_lib.lib().evb_grow_tree(cache.handle, _lib.ptr(mask), C.c_uint8(cache.mask_cond), _lib.ptr(js),
                                        C.c_int32(js.size), C.c_int32(1 if update_grads else 0), _lib.ptr(t.feat),
                                        _lib.ptr(t.cond_bin), _lib.ptr(t.w), _lib.ptr(t.gain), _lib.ptr(t.pred), _lib.ptr(t.split)))
    return t


def grow_tree_begin(cache: Cache, params: EvoTypes, mask, js, update_grads: bool) -> None:
    """Enqueues one tree (`evb_grow_tree_begin`); collect it with `grow_tree_end`.  Up to two trees may be in flight,
    so the host can prepare tree t+1 while the GPU grows tree t."""
    js = np.ascontiguousarray(js, np.uint32)
    _lib.check(_lib.lib().evb_grow_tree_begin(cache.handle, _lib.ptr(mask), C.c_uint8(cache.mask_cond), _lib.ptr(js),
                                              C.c_int32(js.size), C.c_int32(1 if update_grads else 0)))


def grow_tree_end(cache: Cache, params: EvoTypes) -> Tree:
    t = Tree.empty(params.max_depth, cache.K)
    _lib.check(_lib.lib().evb_grow_tree_end(cache.handle, _lib.ptr(t.feat), _lib.ptr(t.cond_bin), _lib.ptr(t.w), _lib.ptr(t.gain),
                                            _lib.ptr(t.pred), _lib.ptr(t.split)))
    return t


def grow_rounds(m: EvoTree, cache: Cache, params: EvoTypes, nrounds: int, on_tree=None) -> None:
    """`nrounds` boosting rounds with the host one tree ahead of the GPU (same trees as calling `grow_evotree`
    `nrounds` times).  `on_tree(i)` is called after the i-th tree of this call has been collected."""
    in_flight = collected = 0

    def collect():
        nonlocal in_flight, collected
        m.trees.append(grow_tree_end(cache, params))
        in_flight -= 1
        collected += 1
        if on_tree is not None:
            on_tree(collected)

    try:
        for _ in range(nrounds):
            for b in range(params.bagging_size):
                mask, js = sample_round(cache, params)
                grow_tree_begin(cache, params, mask, js, update_grads=(b == 0))
                in_flight += 1
                if in_flight == 2:
                    collect()
            m.info["nrounds"] += 1
    finally:
        while in_flight > 0:
            collect()


def grow_evotree(m: EvoTree, cache: Cache, params: EvoTypes) -> None:
    """`grow_evotree!(m, cache, params)`: one boosting round = bagging_size trees."""
    for b in range(params.bagging_size):
        mask, js = sample_round(cache, params)
        m.trees.append(grow_tree(cache, params, mask, js, update_grads=(b == 0)))
    m.info["nrounds"] += 1


IS_MAXIMISE = {"mse": False, "rmse": False, "mae": False, "logloss": False, "mlogloss": False, "poisson": False,
               "gamma": False, "tweedie": False, "quantile": False, "multiquantile": False, "gaussian_mle": True,
               "logistic_mle": True}   # src/metrics.jl:194-205


def init_logger(metric: str, maximise: bool, early_stopping_rounds: int, early_stopping_tolerance: float = 0.0) -> dict:
    """`init_logger` (src/callback.jl:130-144)."""
    return {"name": str(metric), "maximise": maximise, "early_stopping_rounds": early_stopping_rounds,
            "early_stopping_tolerance": early_stopping_tolerance, "nrounds": 0, "iter": [], "metrics": [],
            "iter_since_best": 0, "best_iter": 0, "best_metric": 0.0}


def update_logger(logger: dict, it: int, metric: float) -> None:
    """`update_logger!` (src/callback.jl:146-164)."""
    logger["nrounds"] = it
    logger["iter"].append(it)
    logger["metrics"].append(metric)
    if it == 0:
        logger["best_metric"] = metric
        return
    tol = logger["early_stopping_tolerance"]
    improved = metric > logger["best_metric"] + tol if logger["maximise"] else metric < logger["best_metric"] - tol
    if improved:
        logger["best_metric"] = metric
        logger["best_iter"] = it
        logger["iter_since_best"] = 0
    else:
        logger["iter_since_best"] += logger["iter"][-1] - logger["iter"][-2]


def eval_levelcode(y_eval, target_levels) -> np.ndarray:
    """Class codes 1..K of `y_eval` against the levels the model was trained on (src/callback.jl:11-19)."""
    y_eval = np.asarray(y_eval)
    levels = np.asarray(target_levels)
    pos = np.searchsorted(levels, y_eval)
    pos = np.clip(pos, 0, levels.size - 1)
    bad = levels[pos] != y_eval
    if bad.any():
        raise ValueError(f"`y_eval` contains levels absent from `y_train`: {np.unique(y_eval[bad]).tolist()}. "
                         f"Training levels are {levels.tolist()}.")
    return (pos + 1).astype(np.uint32)


# losses whose bias the sharded path derives from per-shard sums (`Comm.allreduce_bias`) besides the four original ones
allreduce_bias_losses = ("poisson", "gamma", "tweedie", "logistic_mle", "mae", "cred_var", "cred_std", "quantile", "multiquantile")


def metric_from_sums(metric: str, sums, comm=None) -> float:
    """Metric from the two sums that `evb_eval_attach` / `evb_eval_sums` return for this rank's evaluation shard
    (sum of w * value, sum of w): the sums are added over the ranks first, then divided (`sqrt` for rmse)."""
    s = np.array([sums[0], sums[1]], np.float64)
    if comm is not None:
        s = comm.allreduce_sum(s)
    v = float(s[0] / s[1])
    return math.sqrt(v) if metric == "rmse" else v


class CallBack:
    """`CallBack(params, m, x_eval, y_eval, device; w_eval, offset_eval)` (src/callback.jl:82-121): the evaluation
    data is binarized with the model's edges and handed to the training handle (`evb_eval_attach`), which from then
    on applies every grown tree to the evaluation predictions and re-evaluates the metric on the device.  Calling
    the object after a tree has been collected logs that tree's metric (`(cb::CallBack)(logger, iter, tree)`,
    src/callback.jl:123-128).  With `comm` every rank holds a shard of the evaluation rows and the sums are added
    over the ranks.  Deviation: with bagging_size > 1 the reference adds only the last tree of a round to the
    evaluation predictions; here all trees of the round are added, so they equal `m(x_eval)` in link space."""

    def __init__(self, params: EvoTypes, m: EvoTree, cache: Cache, x_eval, y_eval, w_eval=None, offset_eval=None,
                 device: int = 0, comm=None):
        x_eval = np.asarray(x_eval)
        if x_eval.dtype not in (np.float32, np.float64):
            x_eval = x_eval.astype(np.float64)
        nobs = x_eval.shape[0]
        if x_eval.ndim != 2 or x_eval.shape[1] != cache.nfeats:
            raise ValueError("x_eval must have the columns of x_train")
        edges = m.info["edges"]
        x_bin = binarize(x_eval.astype(edges.dtype, copy=False), edges, device)
        loss, K = params.loss, m.K
        if loss == "mlogloss":
            y = eval_levelcode(y_eval, m.info["target_levels"])
        else:
            y = np.ascontiguousarray(y_eval, np.float32)
        if y.shape[0] != nobs:
            raise ValueError("y_eval must have one entry per row of x_eval")
        w = None if w_eval is None else np.ascontiguousarray(w_eval, np.float32)
        pred0 = None
        if offset_eval is not None:                                  # src/callback.jl:110-118
            off = np.array(offset_eval, np.float32, copy=True).reshape(nobs, -1)
            if loss == "logloss":
                off = _logit(off)
            elif loss in ("mlogloss", "poisson", "gamma", "tweedie"):
                off = np.log(off)
            elif loss in ("gaussian_mle", "logistic_mle"):
                off[:, 1::2] = [[_invsoftplus(float(v)) for v in row] for row in off[:, 1::2]]
            pred0 = np.ascontiguousarray(np.broadcast_to(off, (nobs, K)), np.float32)
        self.metric = params.metric
        self.cache, self.comm = cache, comm
        bias = np.ascontiguousarray(m.trees[-1].pred[0], np.float32)  # cb(logger, 0, m.trees[end]), src/fit.jl:416
        sums = (C.c_double * 2)()
        _lib.check(_lib.lib().evb_eval_attach(cache.handle, C.c_int64(nobs), _lib.ptr(x_bin), _lib.ptr(y), _lib.ptr(w),
                                              _lib.ptr(pred0), _lib.ptr(bias), C.c_int32(_lib.METRIC_CODES[self.metric]), sums))
        self.nobs = nobs
        self.initial = self._metric(sums)

    def _metric(self, sums) -> float:
        return metric_from_sums(self.metric, sums, self.comm)

    def last(self) -> float:
        """Metric after the tree collected last by `grow_tree` / `grow_tree_end`."""
        sums = (C.c_double * 2)()
        _lib.check(_lib.lib().evb_eval_sums(self.cache.handle, sums))
        return self._metric(sums)

    def pred(self) -> np.ndarray:
        out = np.empty((self.nobs, self.cache.K), np.float32)
        _lib.check(_lib.lib().evb_eval_get_pred(self.cache.handle, _lib.ptr(out)))
        return out

    def __call__(self, logger: dict, it: int) -> None:
        update_logger(logger, it, self.initial if it == 0 else self.last())

    def detach(self) -> None:
        _lib.check(_lib.lib().evb_eval_detach(self.cache.handle))


def fit(params: EvoTypes, *, x_train, y_train, w_train=None, offset_train=None, x_eval=None, y_eval=None, w_eval=None,
        offset_eval=None, feature_names=None, device: int = 0, return_cache: bool = False, comm=None, **_ignored):
    """`fit(params; x_train, y_train, w_train, offset_train, x_eval, y_eval, w_eval, offset_eval, feature_names)`
    (src/fit.jl:388-437).  With evaluation data the metric of every round is logged in `m.info["logger"]` and
    boosting stops once `early_stopping_rounds` rounds passed without improvement."""
    m, cache = init_core(params, x_train, y_train, w_train, offset_train, feature_names, device, comm=comm)
    if (x_eval is None) != (y_eval is None):
        import warnings
        warnings.warn("To track eval metric in logger, both `x_eval` and `y_eval` must be provided.")
    logger = cb = None
    if x_eval is not None and y_eval is not None:
        cb = CallBack(params, m, cache, x_eval, y_eval, w_eval, offset_eval, device, comm)
        logger = init_logger(params.metric, IS_MAXIMISE[params.metric], params.early_stopping_rounds,
                             params.early_stopping_tolerance)
        cb(logger, 0)
    if logger is None:
        grow_rounds(m, cache, params, params.nrounds)
    elif params.early_stopping_rounds > params.nrounds and params.bagging_size == 1:
        # early stopping cannot trigger: keep the host one tree ahead and log each tree as it is collected
        grow_rounds(m, cache, params, params.nrounds, on_tree=lambda i: cb(logger, i))
    else:
        for i in range(1, params.nrounds + 1):
            grow_evotree(m, cache, params)
            cb(logger, i)
            if logger["iter_since_best"] >= logger["early_stopping_rounds"]:
                break
    m.info["logger"] = logger
    if return_cache:
        return m, cache
    cache.close()
    return m
