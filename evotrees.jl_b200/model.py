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


def _run(m: EvoTree, x, ntree_limit, device, apply_link: bool, want_leaf: bool, stats: dict | None = None):
    """Binarize on the device and apply the trees in one call (`evb_predict_x`).  `x` may be C- or Fortran-ordered:
    no host-side transpose is made."""
    ntrees = len(m.trees)
    ntree_limit = ntrees if ntree_limit is None else ntree_limit
    if ntree_limit > ntrees:
        raise ValueError(f"ntree_limit is larger than number of trees {ntrees}.")
    x = np.asarray(x)
    if x.dtype not in (np.float32, np.float64):
        x = x.astype(np.float64)
    row_major = 1 if (x.flags.c_contiguous and not x.flags.f_contiguous) else 0
    if not (x.flags.c_contiguous or x.flags.f_contiguous):
        x = np.asfortranarray(x)
    nobs, nfeats = x.shape
    edges = np.ascontiguousarray(m.info["edges"], dtype=x.dtype)   # [nfeats, nedges] C order == [nedges x nfeats] column-major
    nn, feat, cb, sp, lp = _pack(m, ntree_limit)
    out = np.empty((nobs, m.K), np.float32, order="F")
    leaf = np.empty((nobs, ntree_limit), np.uint32, order="F") if want_leaf else None
    ft = np.ascontiguousarray(m.info["feattypes"], np.uint8)
    kms = C.c_double(0.0)
    _lib.check(_lib.lib().evb_predict_x(C.c_int32(device), C.c_int32(_lib.LOSS_CODES[m.loss]), C.c_int32(m.K),
                                        C.c_int32(ntree_limit), C.c_int32(nn), _lib.ptr(feat), _lib.ptr(cb), _lib.ptr(sp),
                                        _lib.ptr(lp), _lib.ptr(x), C.c_int32(_lib.EVB_F32 if x.dtype == np.float32 else _lib.EVB_F64),
                                        C.c_int32(row_major), _lib.ptr(edges), C.c_int32(edges.shape[1]), C.c_int64(nobs),
                                        C.c_int32(nfeats), _lib.ptr(ft), C.c_int32(1 if apply_link else 0), _lib.ptr(out),
                                        _lib.ptr(leaf), C.byref(kms)))
    if stats is not None:
        stats["kernel_ms"] = kms.value
    return out, leaf


def predict_binned(m: EvoTree, x_bin: np.ndarray, ntree_limit: int | None = None, device: int = 0, apply_link: bool = True):
    """Inference from an already binned matrix (uint8, Fortran order) through `evb_predict`."""
    ntree_limit = len(m.trees) if ntree_limit is None else ntree_limit
    nobs, nfeats = x_bin.shape
    nn, feat, cb, sp, lp = _pack(m, ntree_limit)
    out = np.empty((nobs, m.K), np.float32, order="F")
    ft = np.ascontiguousarray(m.info["feattypes"], np.uint8)
    _lib.check(_lib.lib().evb_predict(C.c_int32(device), C.c_int32(_lib.LOSS_CODES[m.loss]), C.c_int32(m.K),
                                      C.c_int32(ntree_limit), C.c_int32(nn), _lib.ptr(feat), _lib.ptr(cb), _lib.ptr(sp),
                                      _lib.ptr(lp), _lib.ptr(x_bin), C.c_int64(nobs), C.c_int32(nfeats), _lib.ptr(ft),
                                      C.c_int32(1 if apply_link else 0), _lib.ptr(out), None))
    return out


def predict(m: EvoTree, x, ntree_limit: int | None = None, device: int = 0, stats: dict | None = None) -> np.ndarray:
    """`predict(m, data; ntree_limit, device=:gpu)` (src/predict.jl:93-96): sums the trees and applies the
    loss's inverse link.  Returns [nobs] when K == 1, else [nobs, K]."""
    out, _ = _run(m, x, ntree_limit, device, True, False, stats)
    return out[:, 0].copy() if m.K == 1 else out


def predict_leaf_idx(m: EvoTree, x, ntree_limit: int | None = None, device: int = 0) -> np.ndarray:
    """`predict_leaf_idx(m, data; ntree_limit)` (src/predict.jl:173-185): uint32 [nobs, ntree_limit]."""
    _, leaf = _run(m, x, ntree_limit, device, False, True)
    return leaf
