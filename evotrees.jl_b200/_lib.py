"""ctypes binding of libevotrees_b200.so (C ABI: include/evb.h).

There is no CPU path behind these calls: if the shared library is missing or no B200 is visible the
functions raise `EvbError`.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libevotrees_b200.so")

EVB_F32, EVB_U32, EVB_F64 = 0, 1, 2
LOSS_CODES = {"mse": 0, "logloss": 1, "mlogloss": 2, "gaussian_mle": 3, "poisson": 4, "gamma": 5, "tweedie": 6, "logistic_mle": 7,
              "mae": 8, "cred_var": 9, "cred_std": 10, "quantile": 11, "multiquantile": 12}
METRIC_CODES = {"mse": 0, "rmse": 0, "mae": 1, "logloss": 2, "mlogloss": 3, "gaussian_mle": 4, "poisson": 5, "gamma": 6, "tweedie": 7,
                "logistic_mle": 8, "quantile": 9, "multiquantile": 10}  # rmse = sqrt of the mse sums
FLAG_TIMING, FLAG_FULL_PARTITION, FLAG_KEEP_ALL_HIST = 1, 2, 4
NTIMERS = 12
TIMER_NAMES = ["grads", "rows_init", "hist", "hist_reduce", "allreduce", "scan", "partition", "plan", "finalize",
               "d2h", "h2d", "tree_total"]

EXPORTS = ["evb_last_error", "evb_version", "evb_create", "evb_create_x", "evb_destroy", "evb_comm_unique_id", "evb_comm_init", "evb_comm_ipc_export", "evb_comm_ipc_import",
           "evb_grow_tree", "evb_grow_tree_begin", "evb_grow_tree_end", "evb_eval_attach", "evb_eval_sums", "evb_eval_get_pred", "evb_eval_detach", "evb_test_peer_timeout", "evb_set_timing", "evb_get_pred", "evb_get_grads", "evb_get_nidx", "evb_get_hist", "evb_get_node_sums",
           "evb_get_stream", "evb_get_timings", "evb_reset_timings", "evb_predict", "evb_predict_x", "evb_binarize", "evb_hist_rows", "evb_hist_rows_noalloc", "evb_trim_cache"]


class EvbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[evb {code}] {msg}")
        self.code = code


class EvbParams(C.Structure):
    _fields_ = [("loss", C.c_int32), ("K", C.c_int32), ("nbins", C.c_int32), ("max_depth", C.c_int32),
                ("bagging_size", C.c_int32), ("tree_type", C.c_int32),
                ("eta", C.c_double), ("lambda_", C.c_double), ("L2", C.c_double), ("gamma", C.c_double),
                ("min_weight", C.c_double), ("device", C.c_int32), ("flags", C.c_uint32), ("alpha", C.c_double), ("alphas", C.c_double * 8)]


class EvbTimings(C.Structure):
    _fields_ = [("ms", C.c_double * NTIMERS), ("launches", C.c_int64 * NTIMERS), ("hist_rows", C.c_int64),
                ("hist_nodes", C.c_int64), ("trees", C.c_int64)]


_lib = None


def lib() -> C.CDLL:
    """Load the CUDA library; it is built in-tree by `build.py` (nvcc, sm_100a)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EvbError(-2, f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.evb_last_error.restype = C.c_char_p
        for name in EXPORTS:
            if name not in ("evb_last_error", "evb_destroy"):
                getattr(_lib, name).restype = C.c_int32
        _lib.evb_destroy.restype = None
    return _lib


def trim_cache(device: int = 0) -> None:
    """Hands the device blocks, pinned buffers, streams and events that the library keeps for reuse back to the driver."""
    check(lib().evb_trim_cache(C.c_int32(device)))


def check(rc: int) -> None:
    if rc != 0:
        raise EvbError(rc, lib().evb_last_error().decode("utf-8", "replace"))


def ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)
