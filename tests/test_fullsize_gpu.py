"""Lock-step parity against the CPU oracle at the full row counts of the benchmark configurations (the shapes that
`bench.py` times), one or two boosting rounds each: bit-exact binning, split features / bins, row -> node ids and leaf
ids; node sums, gains, leaf values, predictions and next-round gradients within the tolerances of tests/parity.py.
Histograms are compared at these sizes for the first nodes only (reading every node back would dominate the run)."""
import numpy as np
import pytest

import bench
from tests.parity import lockstep_check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("workload,rounds", [("headline_10Mx100_d11", 1), ("cfg2_1Mx100_d6", 2), ("cfg4_2Mx28_softmax_d8", 1),
                                             ("cfg5_5Mx50_gaussian_d7", 1), ("cfg1_100kx10_d6", 3)])
def test_lockstep_at_benchmark_size(pkg, orc, workload, rounds):
    w = bench.WORKLOADS[workload]
    orc.use_all_cores()
    x, y = bench.make_shard(w, w["rows"], 0, 1)
    params = bench.make_params(pkg, w, nrounds=rounds)
    # mse runs the fixed-point kernel (exact sums); the other losses run the float kernel, whose float32 partial sums
    # need ten times the bound at these row counts
    stats = lockstep_check(pkg, orc, params, x, y, rounds=rounds, check_hist=w["rows"] <= 1_000_000, hist_nodes=8,
                           float_sum_slack=1.0 if w["loss"] == "mse" else 10.0)
    assert stats["trees"] == rounds and stats["splits"] >= rounds * (2 ** (w["depth"] - 2))
    assert stats["diverged"] <= max(1, stats["nodes_compared"] // 500), stats
