"""`Tree` / `EvoTree` containers with the reference's field layout (src/structs.jl:77-138) and inference."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from .binning import binarize


@dataclass
class Tree:
    """Heap-indexed complete binary tree of 2^depth - 1 nodes (the bias tree has one node).
    feat / cond_bin are 1-based, 0 = no split, exactly as in the reference."""
    feat: np.ndarray      # int64 [nn]
    cond_bin: np.ndarray  # uint8 [nn]
    w: np.ndarray         # float32 [nn]
    gain: np.ndarray      # float32 [nn]
    pred: np.ndarray      # float32 [nn, K]; row n is the reference's pred[:, n]
    split: np.ndarray     # bool [nn]

    @staticmethod
    def empty(depth: int, K: int) -> "Tree":
        nn = 2 ** depth - 1
        return Tree(np.zeros(nn, np.int64), np.zeros(nn, np.uint8), np.zeros(nn, np.float32), np.zeros(nn, np.float32),
                    np.zeros((nn, K), np.float32), np.zeros(nn, np.uint8))

    @staticmethod
    def bias(mu: np.ndarray) -> "Tree":
        t = Tree.empty(1, mu.size)
        t.pred[0, :] = mu
        return t


@dataclass
class EvoTree:
    loss: str
    K: int
    trees: list = field(default_factory=list)
    info: dict = field(default_factory=dict)

    def __call__(self, x, ntree_limit: int | None = None, device: int = 0):
        return predict(self, x, ntree_limit=ntree_limit, device=device)


def _pack(m: EvoTree, ntree_limit: int):
    nn = max(t.feat.size for t in m.trees[:ntree_limit])
    K = m.K
    feat = np.zeros((ntree_limit, nn), np.int64)
    cb = np.zeros((ntree_limit, nn), np.uint8)
    sp = np.zeros((ntree_limit, nn), np.uint8)
    lp = np.zeros((ntree_limit, nn, K), np.float32)
    for i, t in enumerate(m.trees[:ntree_limit]):
        k = t.feat.size
        feat[i, :k], cb[i, :k], sp[i, :k], lp[i, :k] = t.feat, t.cond_bin, t.split, t.pred
    return nn, feat, cb, sp, lp


def _run(m: EvoTree, x, ntree_limit, device, apply_link: bool, want_leaf: bool):
    ntrees = len(m.trees)
    ntree_limit = ntrees if ntree_limit is None else ntree_limit
    if ntree_limit > ntrees:
        raise ValueError(f"ntree_limit is larger than number of trees {ntrees}.")
    x = np.asarray(x)
    x_bin = binarize(x, m.info["edges"], device)
    nobs, nfeats = x_bin.shape
    nn, feat, cb, sp, lp = _pack(m, ntree_limit)
    out = np.empty((nobs, m.K), np.float32, order="F")
    leaf = np.empty((nobs, ntree_limit), np.uint32, order="F") if want_leaf else None
    ft = np.ascontiguousarray(m.info["feattypes"], np.uint8)
    _lib.check(_lib.lib().evb_predict(C.c_int32(device), C.c_int32(_lib.LOSS_CODES[m.loss]), C.c_int32(m.K),
                                      C.c_int32(ntree_limit), C.c_int32(nn), _lib.ptr(feat), _lib.ptr(cb), _lib.ptr(sp),
                                      _lib.ptr(lp), _lib.ptr(x_bin), C.c_int64(nobs), C.c_int32(nfeats), _lib.ptr(ft),
                                      C.c_int32(1 if apply_link else 0), _lib.ptr(out), _lib.ptr(leaf)))
    return out, leaf


def predict(m: EvoTree, x, ntree_limit: int | None = None, device: int = 0) -> np.ndarray:
    """`predict(m, data; ntree_limit, device=:gpu)` (src/predict.jl:93-96): sums the trees and applies the
    loss's inverse link.  Returns [nobs] when K == 1, else [nobs, K]."""
    out, _ = _run(m, x, ntree_limit, device, True, False)
    return out[:, 0].copy() if m.K == 1 else out


def predict_leaf_idx(m: EvoTree, x, ntree_limit: int | None = None, device: int = 0) -> np.ndarray:
    """`predict_leaf_idx(m, data; ntree_limit)` (src/predict.jl:173-185): uint32 [nobs, ntree_limit]."""
    _, leaf = _run(m, x, ntree_limit, device, False, True)
    return leaf
