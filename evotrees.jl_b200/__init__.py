"""B200-native device path for EvoTrees: training (`fit`) and inference (`m(x)`) behind the reference's API.

Drop-in scope: what `ext/EvoTreesCUDAExt` provides in the reference.  The compute lives in
libevotrees_b200.so (hand-written sm_100a CUDA, C ABI in include/evb.h); this package is the host-side
mirror of the reference's operator interface.
"""
from .learners import EvoTreeClassifier, EvoTreeCount, EvoTreeMLE, EvoTreeRegressor, EvoTypes
from .model import EvoTree, Tree, predict, predict_binned, predict_leaf_idx
from .fit import (IS_MAXIMISE, CallBack, eval_levelcode, init_logger, update_logger, Cache, fit, grow_evotree, grow_rounds, grow_tree, grow_tree_begin, grow_tree_end, init_core,
                  init_core_binned, sample_round)
from .binning import binarize, get_edges
from ._lib import EvbError, trim_cache

__all__ = ["trim_cache", "EvoTreeRegressor", "EvoTreeClassifier", "EvoTreeMLE", "EvoTreeCount", "EvoTypes", "EvoTree", "Tree", "predict",
           "predict_leaf_idx", "predict_binned", "fit", "init_core", "init_core_binned", "grow_evotree", "grow_tree", "grow_tree_begin", "grow_tree_end", "grow_rounds", "sample_round",
           "Cache", "CallBack", "init_logger", "update_logger", "eval_levelcode", "IS_MAXIMISE", "binarize", "get_edges", "EvbError"]
