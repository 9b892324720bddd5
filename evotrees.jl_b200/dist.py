"""Row sharding over several GPUs: one process per GPU, `torch.distributed` for the host-side plumbing.

The device-side exchange (per-level histogram sum, child row counts) happens inside libevotrees_b200.so
over NCCL; this module only distributes the NCCL id, the quantile edges and the initial bias.  The
reference has no multi-GPU path.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


def shard_bounds(nobs: int, world: int, rank: int):
    """Contiguous row block of `rank`: ceil(nobs / world) rows per rank, the last ranks may get fewer."""
    per = -(-nobs // world)
    lo = min(nobs, rank * per)
    return lo, min(nobs, lo + per)


class Comm:
    """Wraps an initialised torch.distributed process group (nccl on GPUs, gloo in CPU tests)."""

    def __init__(self, dist, device=None):
        self.dist = dist
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self.device = device  # torch device for collectives (None = CPU tensors, gloo)
        import os
        self.p2p = os.environ.get("EVB_P2P", "1") != "0"

    def _tensor(self, a: np.ndarray):
        import torch
        t = torch.from_numpy(np.ascontiguousarray(a))
        return t.to(self.device) if self.device is not None else t

    def broadcast_host(self, a: np.ndarray, src: int = 0) -> np.ndarray:
        t = self._tensor(a)
        self.dist.broadcast(t, src=src)
        return t.cpu().numpy()

    def allgather_host(self, a: np.ndarray) -> np.ndarray:
        """[world, *a.shape] with rank q's array in row q."""
        import torch
        t = self._tensor(a)
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return np.stack([o.cpu().numpy() for o in out])

    def allreduce_sum(self, a: np.ndarray) -> np.ndarray:
        t = self._tensor(np.asarray(a, np.float64))
        self.dist.all_reduce(t)
        return t.cpu().numpy()

    def allreduce_bias(self, loss: str, y: np.ndarray, mu_local: np.ndarray, K: int, alphas=None) -> np.ndarray:
        """Initial bias of the whole data set from per-shard sufficient statistics
        (same formulas as `_init_target`, src/init.jl:19-145)."""
        from .fit import _invsoftplus, _logit
        if loss in ("mse", "logloss", "poisson", "gamma", "tweedie", "mae", "cred_var", "cred_std", "quantile"):
            y2 = y.reshape(y.shape[0], -1).astype(np.float64)
            s = self.allreduce_sum(np.concatenate([y2.sum(axis=0), [y2.shape[0]]]))
            m = s[:-1] / s[-1]
            return (_logit(m) if loss == "logloss" else np.log(m) if loss in ("poisson", "gamma", "tweedie") else m).astype(np.float32)
        if loss == "mlogloss":
            cnt = self.allreduce_sum(np.bincount(y.astype(np.int64) - 1, minlength=K))
            mu = np.log(cnt / cnt.sum()).astype(np.float32)
            return mu - mu.max()
        if loss in ("gaussian_mle", "logistic_mle"):
            y2 = y.reshape(y.shape[0], -1).astype(np.float64)
            s = self.allreduce_sum(np.concatenate([y2.sum(axis=0), (y2 ** 2).sum(axis=0), [y2.shape[0]]]))
            n, Y = s[-1], y2.shape[1]
            mean = s[:Y] / n
            var = (s[Y:2 * Y] - n * mean ** 2) / (n - 1)
            mu = np.empty(2 * Y, np.float32)
            mu[0::2] = mean
            f = np.sqrt(3.0) / np.pi if loss == "logistic_mle" else 1.0
            mu[1::2] = [_invsoftplus(float(np.sqrt(v)) * f) for v in var]
            return mu
        if loss == "multiquantile":
            # quantiles of the whole target (src/init.jl:99-103): the shards' targets are gathered on every rank
            # (4 bytes per row, once per fit), padded to the longest shard
            sizes = self.allgather_host(np.array([y.shape[0]], np.int64))[:, 0]
            pad = np.full(int(sizes.max()), np.nan, np.float32)
            pad[: y.shape[0]] = np.asarray(y, np.float32).reshape(-1)
            allv = self.allgather_host(pad)
            yy = np.concatenate([allv[q, : int(sizes[q])] for q in range(self.world)]).astype(np.float64)
            return np.quantile(yy, list(alphas)).astype(np.float32)
        raise ValueError(loss)

    def attach(self, cache) -> None:
        """Creates the NCCL communicator of the handle (rank 0 draws the id, everybody receives it)."""
        ident = np.zeros(128, np.uint8)
        if self.rank == 0:
            _lib.check(_lib.lib().evb_comm_unique_id(_lib.ptr(ident)))
        ident = self.broadcast_host(ident)
        _lib.check(_lib.lib().evb_comm_init(cache.handle, _lib.ptr(ident), C.c_int32(self.rank), C.c_int32(self.world)))
        if self.p2p and 2 <= self.world <= 8:
            # peer access: exchange the CUDA IPC handles so that the split scan can read the other ranks' histograms;
            # it is used only if every rank could map every other rank, otherwise all ranks stay on NCCL
            blob = np.zeros(256, np.uint8)
            ok = 1.0
            try:
                _lib.check(_lib.lib().evb_comm_ipc_export(cache.handle, _lib.ptr(blob)))
            except _lib.EvbError:
                ok = 0.0
            blobs = np.ascontiguousarray(self.allgather_host(blob))
            if ok:
                try:
                    _lib.check(_lib.lib().evb_comm_ipc_import(cache.handle, _lib.ptr(blobs)))
                except _lib.EvbError:
                    ok = 0.0
            if self.allreduce_sum(np.array([ok]))[0] < self.world:
                _lib.check(_lib.lib().evb_comm_ipc_import(cache.handle, None))
            self.dist.barrier()
