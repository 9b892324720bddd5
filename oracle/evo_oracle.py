"""ctypes front end of the CPU oracle (oracle/evo_oracle.c) plus the numpy restatement of binning.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU-baseline
leg.  The shipped package never imports this module.

Parity pinning: see the header of evo_oracle.c.  `get_edges` below restates `Statistics.quantile`
(type 7, Julia stdlib, not vendored in the reference tree) as called at src/fit-utils.jl:16; the
reference holds no golden vector for it, so it is unpinned as well.  The row sample that the reference
draws with `StatsBase.sample(rng, ...)` (src/fit-utils.jl:10) is replaced by a numpy draw: the oracle
and the library under test are always fed the *same* edges / masks / column samples, which is what
parity is defined on.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libevo_oracle.so")

LOSSES = {"mse": 0, "logloss": 1, "mlogloss": 2, "gaussian_mle": 3, "poisson": 4, "gamma": 5, "tweedie": 6, "logistic_mle": 7,
          "mae": 8, "cred_var": 9, "cred_std": 10, "quantile": 11, "multiquantile": 12}


class OrcParams(C.Structure):
    _fields_ = [
        ("loss", C.c_int32), ("K", C.c_int32), ("nbins", C.c_int32), ("max_depth", C.c_int32),
        ("bagging_size", C.c_int32), ("tree_type", C.c_int32),
        ("eta", C.c_double), ("lambda_", C.c_double), ("L2", C.c_double), ("gamma", C.c_double),
        ("min_weight", C.c_double), ("alpha", C.c_double), ("alphas", C.c_double * 8),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to this file (gcc only)."""
    src = os.path.join(_HERE, "evo_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "CC=gcc"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_sigmoid.restype = C.c_float
        _lib.orc_sigmoid.argtypes = [C.c_float]
        _lib.orc_softplus.restype = C.c_float
        _lib.orc_softplus.argtypes = [C.c_float]
        for f in ("orc_softplus64", "orc_invsoftplus64", "orc_sigmoid64"):
            getattr(_lib, f).restype = C.c_double
            getattr(_lib, f).argtypes = [C.c_double]
        _lib.orc_gaussian_grad_hess64.argtypes = [C.c_double, C.c_double, C.c_double, C.POINTER(C.c_double)]
        _lib.orc_mlogloss_grad_hess64.argtypes = [C.c_double, C.c_double, C.c_int, C.POINTER(C.c_double)]
        _lib.orc_grow_tree.restype = C.c_int
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


@dataclass
class Params:
    loss: str = "mse"
    K: int = 1
    nbins: int = 64
    max_depth: int = 6
    bagging_size: int = 1
    eta: float = 0.1
    lambda_: float = 0.0
    L2: float = 1.0
    gamma: float = 0.0
    min_weight: float = 1.0
    alpha: float = 0.5
    alphas: tuple = (0.1, 0.5, 0.9)
    tree_type: int = 0   # 0 binary, 1 oblivious (grow_otree!, src/fit.jl:147-263)

    def c(self) -> OrcParams:
        al = (C.c_double * 8)(*(list(self.alphas) + [0.0] * 8)[:8])
        return OrcParams(LOSSES[self.loss], self.K, self.nbins, self.max_depth, self.bagging_size, self.tree_type,
                         self.eta, self.lambda_, self.L2, self.gamma, self.min_weight, self.alpha, al)


@dataclass
class Tree:
    """Same fields as the reference's `Tree{L,K}` (src/structs.jl:77-84), 1-based feat/cond_bin."""
    feat: np.ndarray      # int64 [nn]
    cond_bin: np.ndarray  # uint8 [nn]
    w: np.ndarray         # float32 [nn]
    gain: np.ndarray      # float32 [nn]
    pred: np.ndarray      # float32 [nn, K]  (row n = Julia's pred[:, n])
    split: np.ndarray     # uint8 [nn]


# ----------------------------------------------------------------------------- binning
def quantile_type7(sorted_v: np.ndarray, p: float):
    """Statistics._quantile with alpha = beta = 1 on an already sorted vector."""
    n = sorted_v.shape[0]
    aleph = float(np.float64(n) * np.float64(p) + np.float64(1.0 - p))  # fma(n, p, 1 - p)
    j = min(max(int(aleph), 1), n - 1) if n > 1 else 1
    g = min(max(aleph - j, 0.0), 1.0)
    if n == 1:
        a = b = sorted_v[0]
    else:
        a, b = sorted_v[j - 1], sorted_v[j]
    rtol = np.sqrt(np.finfo(sorted_v.dtype).eps)
    a64, b64 = np.float64(a), np.float64(b)
    if np.isfinite(a64) and np.isfinite(b64) and abs(a64 - b64) <= rtol * max(abs(a64), abs(b64)):
        return a64 + g * (b64 - a64)
    return (1.0 - g) * a64 + g * b64


def get_edges(x: np.ndarray, nbins: int, rng: np.random.Generator) -> np.ndarray:
    """Matrix method of `get_edges` (src/fit-utils.jl:7-24): nbins-1 quantile edges per feature,
    from at most 1000*nbins sampled rows, stored with the element type of `x`.
    Returns edges [nfeats, nbins-1]."""
    nobs = x.shape[0]
    ns = min(nobs, 1000 * nbins)
    idx = np.sort(rng.choice(nobs, size=ns, replace=False)) if ns < nobs else np.arange(nobs)
    edges = np.empty((x.shape[1], nbins - 1), dtype=x.dtype)
    for j in range(x.shape[1]):
        v = np.sort(x[idx, j])
        for b in range(1, nbins):
            edges[j, b - 1] = quantile_type7(v, b / nbins)
        if nbins == 2:      # `length(edges[j]) == 1` -> the sample minimum (src/fit-utils.jl:17-19)
            edges[j, 0] = v[0]
    return edges


def binarize(x: np.ndarray, edges: np.ndarray) -> np.ndarray:
    """`binarize` (src/fit-utils.jl:66-72) through the C oracle.  x [nobs, nfeats] any order;
    returns x_bin uint8 [nobs, nfeats] in Fortran (Julia) order."""
    xf = np.asfortranarray(x)
    nobs, nfeats = xf.shape
    out = np.zeros((nobs, nfeats), dtype=np.uint8, order="F")
    e = np.ascontiguousarray(edges, dtype=xf.dtype)
    fn = lib().orc_binarize_f32 if xf.dtype == np.float32 else lib().orc_binarize_f64
    fn(C.c_int64(nobs), C.c_int32(nfeats), _p(xf), _p(e), C.c_int32(e.shape[1]), _p(out))
    return out


# ----------------------------------------------------------------------------- training pieces
def update_grads(p: Params, pred: np.ndarray, y: np.ndarray, grad: np.ndarray) -> None:
    """In place on grad [nobs, C] (row i = Julia's grad[:, i]); the last column holds w."""
    nobs = pred.shape[0]
    cp = p.c()
    lib().orc_update_grads(C.byref(cp), C.c_int64(nobs), _p(pred), _p(y), _p(grad))


def grow_tree(p: Params, x_bin: np.ndarray, grad: np.ndarray, is_: np.ndarray, js: np.ndarray,
              feattypes: np.ndarray | None = None, monotone: np.ndarray | None = None,
              want_hist: bool = False, x_bin_T: np.ndarray | None = None):
    """One `grow_tree!` (src/fit.jl:45-143).  x_bin uint8 Fortran [nobs, nfeats]; is_/js 1-based uint32.
    Returns (Tree, nidx uint32 [nobs], hist or None, nsum [nn, C])."""
    assert x_bin.flags.f_contiguous and x_bin.dtype == np.uint8
    nobs, nfeats = x_bin.shape
    K, Cc = p.K, 2 * p.K + 1
    nn = 2 ** p.max_depth - 1
    t = Tree(np.zeros(nn, np.int64), np.zeros(nn, np.uint8), np.zeros(nn, np.float32), np.zeros(nn, np.float32),
             np.zeros((nn, K), np.float32), np.zeros(nn, np.uint8))
    nidx = np.zeros(nobs, np.uint32)
    hist = np.zeros((nn, nfeats, p.nbins, Cc), np.float64) if want_hist else None
    nsum = np.zeros((nn, Cc), np.float64)
    is_ = np.ascontiguousarray(is_, np.uint32)
    js = np.ascontiguousarray(js, np.uint32)
    ft = None if feattypes is None else np.ascontiguousarray(feattypes, np.uint8)
    mo = None if monotone is None else np.ascontiguousarray(monotone, np.int32)
    cp = p.c()
    rc = lib().orc_grow_tree(C.byref(cp), C.c_int64(nobs), C.c_int32(nfeats), _p(x_bin), _p(x_bin_T), _p(grad),
                             _p(is_), C.c_int64(is_.size), _p(js), C.c_int32(js.size), _p(ft), _p(mo),
                             _p(t.feat), _p(t.cond_bin), _p(t.w), _p(t.gain), _p(t.pred), _p(t.split),
                             _p(nidx), _p(hist), _p(nsum))
    if rc != 0:
        raise ValueError(f"orc_grow_tree failed: {rc}")
    return t, nidx, hist, nsum


def predict_tree(p: Params, x_bin: np.ndarray, t: Tree, pred: np.ndarray, feattypes=None) -> None:
    """`predict!(pred, tree, x_bin, feattypes)` in place, with the loss-specific clamps."""
    ft = None if feattypes is None else np.ascontiguousarray(feattypes, np.uint8)
    lib().orc_predict_tree(C.c_int32(LOSSES[p.loss]), C.c_int32(p.K), C.c_int64(x_bin.shape[0]), _p(x_bin), _p(ft),
                           _p(t.feat), _p(t.cond_bin), _p(t.split), _p(t.pred), _p(pred))


def leaf_idx(x_bin: np.ndarray, t: Tree, feattypes=None) -> np.ndarray:
    out = np.zeros(x_bin.shape[0], np.uint32)
    ft = None if feattypes is None else np.ascontiguousarray(feattypes, np.uint8)
    lib().orc_leaf_idx(C.c_int64(x_bin.shape[0]), _p(x_bin), _p(ft), _p(t.feat), _p(t.cond_bin), _p(t.split), _p(out))
    return out


def link(p: Params, pred: np.ndarray) -> None:
    lib().orc_link(C.c_int32(LOSSES[p.loss]), C.c_int32(p.K), C.c_int64(pred.shape[0]), _p(pred))


def init_pred(p: Params, y: np.ndarray) -> np.ndarray:
    """Initial bias mu per loss, `_init_target` (src/init.jl:19-145), returned as float32 [K]."""
    if p.loss in ("mse", "mae", "cred_var", "cred_std", "quantile"):
        return np.array([np.mean(y.astype(np.float32), dtype=np.float32)], np.float32)
    if p.loss == "logloss":
        m = np.float32(np.mean(y.astype(np.float32), dtype=np.float32))
        return np.array([np.log(m / (np.float32(1) - m))], np.float32)
    if p.loss == "mlogloss":
        cnt = np.bincount(y.astype(np.int64) - 1, minlength=p.K).astype(np.float64)
        mu = np.log(cnt / cnt.sum()).astype(np.float32)
        return (mu - mu.max()).astype(np.float32)
    if p.loss in ("poisson", "gamma", "tweedie"):
        return np.array([np.log(np.mean(y.astype(np.float32), dtype=np.float32))], np.float32)
    if p.loss in ("gaussian_mle", "logistic_mle"):
        y32 = y.astype(np.float32)
        sd = np.float32(np.std(y32.astype(np.float64), ddof=1))
        if p.loss == "logistic_mle":
            sd = np.float32(sd * np.sqrt(3.0) / np.pi)   # src/init.jl:86
        return np.array([np.mean(y32, dtype=np.float32), lib().orc_invsoftplus64(float(sd))], np.float32)
    raise ValueError(p.loss)


METRICS = {"mse": 0, "rmse": 0, "mae": 1, "logloss": 2, "mlogloss": 3, "gaussian_mle": 4, "poisson": 5, "gamma": 6, "tweedie": 7,
           "logistic_mle": 8, "quantile": 9, "multiquantile": 10}
IS_MAXIMISE = {"mse": False, "rmse": False, "mae": False, "logloss": False, "mlogloss": False, "gaussian_mle": True,
               "poisson": False, "gamma": False, "tweedie": False, "logistic_mle": True, "quantile": False, "multiquantile": False}


def eval_metric(metric: str, pred: np.ndarray, y: np.ndarray, w: np.ndarray | None = None, alpha: float = 0.5, alphas=(0.1, 0.5, 0.9)) -> float:
    """Metric functions of src/metrics.jl:31-116 on link-space predictions `pred` [nobs, K] (float32)."""
    pred = np.ascontiguousarray(pred, np.float32)
    nobs, K = pred.shape
    y = np.ascontiguousarray(y, np.uint32 if metric == "mlogloss" else np.float32)
    ycols = 1 if y.ndim == 1 else y.shape[1]
    w32 = None if w is None else np.ascontiguousarray(w, np.float32)
    ev = np.empty(nobs, np.float32)
    out = (C.c_double * 2)()
    lib().orc_eval_metric(C.c_int32(METRICS[metric]), C.c_int32(K), C.c_int64(nobs), _p(pred), _p(y), C.c_int32(ycols),
                          _p(w32), _p(ev), out, C.c_double(alpha), (C.c_double * 8)(*(list(alphas) + [0.0] * 8)[:8]))
    v = out[0] / out[1]
    return float(np.sqrt(v)) if metric == "rmse" else float(v)


class Logger:
    """`init_logger` / `update_logger!` (src/callback.jl:130-164) and the stopping rule of `fit` (src/fit.jl:429)."""

    def __init__(self, metric: str, early_stopping_rounds: int, early_stopping_tolerance: float = 0.0):
        self.maximise = IS_MAXIMISE[metric]
        self.rounds, self.tol = early_stopping_rounds, early_stopping_tolerance
        self.iter, self.metrics = [], []
        self.iter_since_best = self.best_iter = 0
        self.best_metric = 0.0

    def update(self, it: int, metric: float) -> bool:
        """Logs one iteration; True when boosting has to stop."""
        self.iter.append(it)
        self.metrics.append(metric)
        if it == 0:
            self.best_metric = metric
            return False
        better = metric > self.best_metric + self.tol if self.maximise else metric < self.best_metric - self.tol
        if better:
            self.best_metric, self.best_iter, self.iter_since_best = metric, it, 0
        else:
            self.iter_since_best += self.iter[-1] - self.iter[-2]
        return self.iter_since_best >= self.rounds


def num_threads() -> int:
    return lib().orc_num_threads()


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on, whatever OMP_NUM_THREADS says."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().orc_set_num_threads(C.c_int(n))
    return num_threads()


class Booster:
    """Boosting loop of `grow_evotree!` (src/fit.jl:6-42) on top of the C pieces.  The caller supplies
    the per-tree row mask / column sample so that both sides of a parity test consume the same draws."""

    def __init__(self, p: Params, x_bin: np.ndarray, y: np.ndarray, w: np.ndarray | None = None,
                 feattypes=None, monotone=None, use_x_bin_T: bool = False):
        self.p, self.x_bin, self.y = p, x_bin, y
        nobs = x_bin.shape[0]
        self.feattypes, self.monotone = feattypes, monotone
        self.x_bin_T = np.ascontiguousarray(x_bin) if use_x_bin_T else None  # C order [nobs, nfeats] == Julia [nfeats, nobs]
        Cc = 2 * p.K + 1
        self.grad = np.zeros((nobs, Cc), np.float32)
        self.grad[:, -1] = 1.0 if w is None else w
        mu = init_pred(p, y)
        self.mu = mu
        self.pred = np.tile(mu, (nobs, 1)).astype(np.float32)
        self.trees: list[Tree] = []

    def round(self, mask: np.ndarray | None, mask_cond: int, js: np.ndarray, want_hist=False):
        p = self.p
        update_grads(p, self.pred, self.y, self.grad)
        nobs = self.x_bin.shape[0]
        if mask is None:
            is_ = np.arange(1, nobs + 1, dtype=np.uint32)
        else:
            is_ = (np.nonzero(mask <= mask_cond)[0] + 1).astype(np.uint32)   # src/subsample.jl:6-38
        t, nidx, hist, nsum = grow_tree(p, self.x_bin, self.grad, is_, js, self.feattypes, self.monotone, want_hist,
                                        self.x_bin_T)
        self.trees.append(t)
        predict_tree(p, self.x_bin, t, self.pred, self.feattypes)
        return t, nidx, hist, nsum
