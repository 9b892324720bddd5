"""Quantile edges on the host and `binarize` on the device.

`get_edges` mirrors the Matrix method of the reference (src/fit-utils.jl:7-24), which also runs on the host
in the reference's GPU path (ext/EvoTreesKernelAbstractionsExt/init.jl:3-6).  `binarize`
(src/fit-utils.jl:66-72) runs on the GPU through `evb_binarize`.
"""
from __future__ import annotations

import ctypes as C

import os

import numpy as np

from . import _lib


def _edge_threads() -> int:
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(16, n))


def get_edges(x: np.ndarray, nbins: int, rng: np.random.Generator):
    """Returns (edges [nfeats, nbins-1] of x.dtype, featbins uint8 [nfeats], feattypes bool [nfeats]).

    Per feature: type-7 quantiles at (1:nbins-1)/nbins of at most 1000*nbins sampled rows (drawn without
    replacement, ascending), computed in float64 and stored with the element type of `x`."""
    nobs, nfeats = x.shape
    ns = min(nobs, 1000 * nbins)
    idx = np.sort(rng.choice(nobs, size=ns, replace=False)) if ns < nobs else slice(None)
    p = np.arange(1, nbins, dtype=np.float64) / nbins
    aleph = ns * p + (1.0 - p)
    j = np.clip(np.trunc(aleph).astype(np.int64), 1, max(ns - 1, 1))
    g = np.clip(aleph - j, 0.0, 1.0)
    rtol = np.sqrt(np.finfo(x.dtype).eps)
    edges = np.empty((nfeats, nbins - 1), dtype=x.dtype)

    def one(f):
        v = np.sort(x[idx, f]).astype(np.float64)
        if ns == 1:
            a = b = np.full(nbins - 1, v[0])
        else:
            a, b = v[j - 1], v[j]
        close = np.isfinite(a) & np.isfinite(b) & (np.abs(a - b) <= rtol * np.maximum(np.abs(a), np.abs(b)))
        edges[f] = np.where(close, a + g * (b - a), (1.0 - g) * a + g * b).astype(x.dtype)
        if nbins == 2:      # a single edge is replaced by the sample minimum (src/fit-utils.jl:17-19)
            edges[f, 0] = v[0]

    # the reference runs this loop under `@threads` (src/fit-utils.jl:15); the gather and the sort release the GIL
    nthreads = min(nfeats, _edge_threads()) if ns * nfeats >= 1 << 18 else 1
    if nthreads > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(nthreads) as pool:
            list(pool.map(one, range(nfeats)))
    else:
        for f in range(nfeats):
            one(f)
    featbins = np.full(nfeats, nbins, dtype=np.uint8)
    feattypes = np.ones(nfeats, dtype=bool)
    return edges, featbins, feattypes


def binarize(x: np.ndarray, edges: np.ndarray, device: int = 0) -> np.ndarray:
    """x [nobs, nfeats] float32/float64 -> x_bin uint8 [nobs, nfeats] (Fortran order), computed on the GPU."""
    if x.dtype not in (np.float32, np.float64):
        x = x.astype(np.float64)
    xf = np.asfortranarray(x)
    nobs, nfeats = xf.shape
    e = np.ascontiguousarray(edges, dtype=xf.dtype)  # [nfeats, nedges] C order == [nedges x nfeats] column-major
    out = np.empty((nobs, nfeats), dtype=np.uint8, order="F")
    dt = _lib.EVB_F32 if xf.dtype == np.float32 else _lib.EVB_F64
    _lib.check(_lib.lib().evb_binarize(C.c_int32(device), _lib.ptr(xf), C.c_int32(dt), C.c_int64(nobs), C.c_int32(nfeats),
                                       _lib.ptr(e), C.c_int32(e.shape[1]), _lib.ptr(out)))
    return out
