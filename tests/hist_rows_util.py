"""Helpers for the tests of the stand-alone histogram entry points (device buffers come from torch)."""
import ctypes as C

import numpy as np


def make_inputs(n, nfeats, nbins, nch, nrows, seed):
    rng = np.random.default_rng(seed)
    rs = (nfeats + 31) // 32 * 32
    x = np.zeros((n, rs), np.uint8)
    x[:, :nfeats] = rng.integers(1, nbins + 1, size=(n, nfeats), dtype=np.uint8)
    g = np.zeros((n, 4), np.float32)
    g[:, :nch] = rng.normal(size=(n, nch)).astype(np.float32)
    g[:, nch - 1] = 1.0  # last channel = unit weights, gives the bin populations
    rows = np.sort(rng.choice(n, size=nrows, replace=False)).astype(np.uint32)
    return x, g, rows


def reference_hist(x, g, rows, nfeats, nbins, nch):
    """float64 histogram [nfeats, nch, nbins] by numpy, rows added in ascending order like `_hist!`."""
    out = np.zeros((nfeats, nch, nbins), np.float64)
    xr, gr = x[rows], g[rows].astype(np.float64)
    for f in range(nfeats):
        for c in range(nch):
            out[f, c] = np.bincount(xr[:, f].astype(np.int64) - 1, weights=gr[:, c], minlength=nbins)
    return out


def call(fn, torch, x, g, rows, nfeats, nbins, nch, device=0):
    dev = torch.device("cuda", device)
    xd = torch.from_numpy(x).to(dev)
    gd = torch.from_numpy(g).to(dev)
    rd = torch.from_numpy(rows.view(np.int32)).to(dev) if rows.size else torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.full((nfeats, nch, nbins), float("nan"), dtype=torch.float64, device=dev)
    torch.cuda.synchronize()
    rc = fn(C.c_int32(device), C.c_void_p(0), C.c_void_p(xd.data_ptr()), C.c_int64(x.shape[0]), C.c_int32(nfeats),
            C.c_int32(x.shape[1]), C.c_int32(nbins), C.c_void_p(gd.data_ptr()), C.c_int32(nch), C.c_void_p(rd.data_ptr()),
            C.c_int64(rows.size), C.c_void_p(out.data_ptr()))
    torch.cuda.synchronize()
    return rc, out.cpu().numpy()


def assert_hist_close(got, want, g, rtol=1e-5):
    """|got - want| <= rtol * max|g_c| * population of the bin (the bound of sum |contribution|)."""
    pop = want[:, -1:, :]
    gmax = np.abs(g).max(axis=0)[: want.shape[1]].astype(np.float64)
    atol = rtol * gmax[None, :, None] * pop + 1e-12
    err = np.abs(got - want)
    assert np.isfinite(got).all(), "output holds non-finite values"
    assert (err <= atol).all(), f"max err {err.max()} vs allowed {atol[err > atol].min()}"
