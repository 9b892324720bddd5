"""Benchmark of the EvoTrees training hot path on B200.

Metric: seconds per 200 boosting rounds, mse, 10M x 100 Float32 features, depth 11, 64 bins,
rows sharded over --gpus GPUs (strong scaling).  A "step" is one boosting round over synthetic data of that
shape (uniform features, y = x.beta + 0.1 N(0,1); the reference's benchmark data is synthetic too,
benchmarks/regressor.jl:47-48).

  python bench.py --gpus N --steps K --warmup W            # this library
  python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference's CPU path (oracle)

Prints one JSON line (rank 0).  `value` = device-resident boosting loop (x_bin already in HBM), `e2e` = the
same metric through the public API from host buffers (init + upload inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (rows, feats, depth, nbins, eta, rowsample, colsample)
    "headline_10Mx100_d11": (10_000_000, 100, 11, 64, 0.1, 1.0, 1.0),
    "cfg2_1Mx100_d6": (1_000_000, 100, 6, 64, 0.05, 0.5, 0.5),
    "cfg1_100kx10_d6": (100_000, 10, 6, 32, 0.1, 1.0, 1.0),
}
ROUNDS_PER_JOB = 200


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="headline_10Mx100_d11", choices=list(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the number of rows (for quick checks)")
    ap.add_argument("--tree-type", default="binary", choices=["binary", "oblivious"], help="not the headline: side measurements")
    ap.add_argument("--cpu-rounds", type=int, default=2, help="rounds of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def make_shard(rows_total, feats, rank, world, seed=123):
    """Rows [lo, hi) of the synthetic matrix; every rank draws its own block from a rank-specific stream."""
    per = -(-rows_total // world)
    lo, hi = min(rows_total, rank * per), min(rows_total, (rank + 1) * per)
    rng = np.random.default_rng([seed, rank])
    beta = np.random.default_rng(seed).normal(size=feats).astype(np.float32)
    n = hi - lo
    x = np.empty((n, feats), np.float32, order="F")
    for j in range(feats):
        x[:, j] = rng.random(n, dtype=np.float32)
    y = x @ beta + 0.1 * rng.standard_normal(n, dtype=np.float32)
    return x, y.astype(np.float32)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(x_bin, y, depth, nbins, eta, rounds, tree_type=0):
    """Times the oracle (C + OpenMP restatement of the reference's CPU path) on the full matrix for a few rounds."""
    from oracle import evo_oracle as orc
    p = orc.Params(loss="mse", K=1, nbins=nbins, max_depth=depth, eta=eta, tree_type=tree_type)
    b = orc.Booster(p, x_bin, y, use_x_bin_T=True)
    js = np.arange(1, x_bin.shape[1] + 1, dtype=np.uint32)
    b.round(None, 255, js)  # warm-up round (page faults, thread pool)
    t0 = time.perf_counter()
    for _ in range(rounds):
        b.round(None, 255, js)
    dt = (time.perf_counter() - t0) / rounds
    return dt, orc.num_threads()


def run_reference(args):
    """Reference arm: the reference is Julia and no Julia runtime exists in this image, so the CPU restatement of
    its CPU path (oracle/) is timed instead, with all host threads, on the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows, feats, depth, nbins, eta, _, _ = WORKLOADS[args.workload]
    rows = args.rows or rows
    from oracle import evo_oracle as orc
    x, y = make_shard(rows, feats, 0, 1)
    rng = np.random.default_rng(123)
    edges = orc.get_edges(x[: min(rows, 1000 * nbins)], nbins, rng)
    x_bin = orc.binarize(x, edges)
    del x
    p = orc.Params(loss="mse", K=1, nbins=nbins, max_depth=depth, eta=eta, tree_type=int(args.tree_type == "oblivious"))
    b = orc.Booster(p, x_bin, y, use_x_bin_T=True)
    js = np.arange(1, feats + 1, dtype=np.uint32)
    steps = max(1, min(args.steps, 8))      # bounded sample: every step is one full boosting round on all rows
    for _ in range(min(args.warmup, 1)):
        b.round(None, 255, js)
    t0 = time.perf_counter()
    for _ in range(steps):
        b.round(None, 255, js)
    ms = (time.perf_counter() - t0) / steps * 1e3
    val = ms * ROUNDS_PER_JOB / 1e3
    sample = f"{steps} full boosting rounds on all {rows} rows (of {ROUNDS_PER_JOB}), scaled linearly"
    out = {"impl": "reference", "metric": "train_seconds_per_200_rounds", "value": val, "unit": "s", "n_gpus": args.gpus,
           "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
           "vs_baseline": None, "dtype": "f32 gradients, f64 histograms", "data": "synthetic",
           "config": {"workload": args.workload, "rows": rows, "feats": feats, "max_depth": depth, "nbins": nbins, "loss": "mse"},
           "cpu_baseline": {"value": val, "unit": "s", "cores": orc.num_threads(), "kind": "port", "sample": sample},
           "e2e": {"value": val, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "note": "reference Julia runtime unavailable: C/OpenMP restatement of the reference CPU path timed instead"}
    print(json.dumps(out), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g
    pkg = g.load_package()
    from evotrees_b200 import _lib
    from evotrees_b200.dist import Comm
    from evotrees_b200.fit import init_core_binned, init_target

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback")
    torch.cuda.set_device(local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        comm = Comm(dist, torch.device("cuda", local))

    rows, feats, depth, nbins, eta, rowsample, colsample = WORKLOADS[args.workload]
    rows = args.rows or rows
    params = pkg.EvoTreeRegressor(loss="mse", nrounds=ROUNDS_PER_JOB, max_depth=depth, nbins=nbins, eta=eta,
                                  rowsample=rowsample, colsample=colsample, tree_type=args.tree_type)
    x, y = make_shard(rows, feats, rank, world)
    nloc = x.shape[0]

    # ---- host side of init: edges (rank 0's sample, broadcast), bias, device binarize --------------------
    t_init0 = time.perf_counter()
    rng = np.random.default_rng(params.seed)
    edges, _, feattypes = pkg.get_edges(x, nbins, rng)
    K, yd, ycols, mu, _, _ = init_target("mse", y, None)
    if comm is not None:
        edges = comm.broadcast_host(edges)
        mu = comm.allreduce_bias("mse", yd, mu, K)
    t_edges = time.perf_counter() - t_init0
    t0 = time.perf_counter()
    x_bin = pkg.binarize(x, edges, local)
    t_binarize = time.perf_counter() - t0
    del x
    x_bin_pinned = torch.empty((feats, nloc), dtype=torch.uint8).pin_memory()   # column-major [nloc x feats]
    xb_host = x_bin_pinned.numpy().T
    xb_host[...] = x_bin
    assert xb_host.flags.f_contiguous

    def create():
        return init_core_binned(params, xb_host, yd, ycols, K, mu, None, None, feattypes, local, 0, comm)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident loop: `value` --------------------------------------------------------------------
    def run_rounds(cache, k, keep=None):
        """k boosting rounds, the host one tree ahead of the GPU (how `fit` drives the library)."""
        in_flight = 0
        for _ in range(k):
            mask, js = pkg.sample_round(cache, params)
            pkg.grow_tree_begin(cache, params, mask, js, True)
            in_flight += 1
            if in_flight == 2:
                t = pkg.grow_tree_end(cache, params)
                in_flight -= 1
                if keep is not None:
                    keep.append(t)
        while in_flight:
            t = pkg.grow_tree_end(cache, params)
            in_flight -= 1
            if keep is not None:
                keep.append(t)

    cache = create()
    ext = torch.cuda.ExternalStream(cache.stream(), device=torch.device("cuda", local))
    run_rounds(cache, args.warmup)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    run_rounds(cache, args.steps)
    e1.record(ext)
    sync_all()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps
    if world > 1:
        t = torch.tensor([ms_step], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
    # Per-kernel CUDA events cannot be read back from graph replays, so the kernel breakdown (and the histogram
    # kernel's launch durations for the roofline) comes from an instrumented pass of the same number of rounds on
    # the same handle, right after the timed region.
    cache.set_timing(True)
    cache.reset_timings()
    for _ in range(args.steps):
        mask, js = pkg.sample_round(cache, params)
        pkg.grow_tree(cache, params, mask, js, True)
    tm = cache.timings()
    cache.close()

    # ---- end to end through the public C-ABI path from host buffers: `e2e` --------------------------------
    e2e = None
    inference = None
    if not args.no_e2e:
        sync_all()
        t0 = time.perf_counter()
        cache2 = create()                                   # H2D of x_bin / y inside the timed region
        t_create = time.perf_counter() - t0
        nn = 2 ** depth - 1
        # the first round is timed on its own: it carries one-off costs (first gradients, lazy NCCL channel set-up)
        # that must not be multiplied when the loop is scaled to 200 rounds
        t0 = time.perf_counter()
        mask, js = pkg.sample_round(cache2, params)
        pkg.grow_tree(cache2, params, mask, js, True)
        torch.cuda.synchronize()
        t_first = time.perf_counter() - t0
        t0 = time.perf_counter()
        grown = []
        run_rounds(cache2, args.steps, grown)               # every round returns its tree arrays to the host (D2H)
        torch.cuda.synchronize()
        t_loop = time.perf_counter() - t0
        cache2.close()
        if world == 1 and grown:
            # inference (`m(x)` on binned input): a model of ROUNDS_PER_JOB trees + the bias tree, made by repeating the
            # trees just grown (the cost of a tree does not depend on which boosting round it comes from), applied to
            # all rows from the host matrix: H2D of x_bin, traversal of every tree, D2H of the predictions
            from evotrees_b200.model import EvoTree, Tree
            trees = [Tree.bias(mu)] + [grown[i % len(grown)] for i in range(ROUNDS_PER_JOB)]
            model = EvoTree("mse", K, trees, {"feattypes": np.ones(feats, bool) if feattypes is None else feattypes})
            pkg.predict_binned(model, xb_host[:1000], device=local)          # warm-up
            t0 = time.perf_counter()
            pkg.predict_binned(model, xb_host, device=local)
            t_pred = time.perf_counter() - t0
            inference = {"rows_per_s": nloc / t_pred, "seconds": t_pred, "rows": nloc, "trees": len(trees),
                         "input": "host x_bin (uint8): H2D, traversal of all trees, D2H of the predictions inside the timed region"}
        e2e_s = t_create + t_first + t_loop / args.steps * (ROUNDS_PER_JOB - 1)
        if world > 1:
            t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        h2d = (nloc * feats + nloc * 4) / ROUNDS_PER_JOB + feats * 4 + (nloc if rowsample < 1 else 0)
        d2h = nn * (4 + 4 + 4 + 4 + 4 + 1 + 1) + 24 * (depth + 2) + 16
        e2e = {"value": e2e_s, "unit": "s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "init_upload_s": t_create, "first_round_s": t_first, "loop_s_per_199": t_loop / args.steps * (ROUNDS_PER_JOB - 1),
               "host_edges_s": t_edges, "device_binarize_from_host_s": t_binarize}

    if rank == 0:
        C = 3
        F = int(np.ceil(colsample * feats))
        hist_ms = tm["ms"]["hist"]
        hist_launches = tm["launches"]["hist"]
        # algorithmic bytes of the histogram kernel: rows x (F bin bytes + C gradient floats + 4-byte row id)
        # + one float image [F x nbins x C] per built node
        alg = tm["hist_rows"] * (F + 4 * C + 4) + tm["hist_nodes"] * F * nbins * C * 4
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = alg / (hist_ms * 1e-3) / 1e9 if hist_ms > 0 else None
        launches = sum(v for k, v in tm["launches"].items() if k not in ("d2h", "h2d", "tree_total", "allreduce"))
        out = {
            "metric": "train_seconds_per_200_rounds", "value": ms_step * ROUNDS_PER_JOB / 1e3, "unit": "s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 gradients, exact 32-bit fixed-point partial sums in shared memory, f64 histograms and split scan", "data": "synthetic",
            "config": {"workload": args.workload, "rows": rows, "feats": feats, "max_depth": depth, "nbins": nbins, "loss": "mse", "tree_type": args.tree_type,
                       "eta": eta, "rowsample": rowsample, "colsample": colsample, "rows_per_gpu": nloc,
                       "l2_policy": "inputs larger than L2 (x_bin shard %.0f MB)" % (nloc * 128 / 1e6)},
            "roofline": {"bound": "hbm", "kernel": "k_histq", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None,
                         # DRAM bytes per launch: 145 B per streamed row, measured with ncu on a 2M-row case of this
                         # workload (dram__bytes_read + write: 306.5 MB for the 2M rows of the root launch = 153 B per
                         # row, 127.0 MB for the 0.98M rows of the level-2 launch = 130 B per row) and scaled by the
                         # rows per launch
                         "traffic": (145.0 * tm["hist_rows"] / max(1, hist_launches)) if args.workload == "headline_10Mx100_d11" else None,
                         "peak_source": "MEASURED_PEAKS.json hbm_gbs" if peaks else "fallback 6650",
                         "hist_ms_per_launch": hist_ms / max(1, hist_launches), "hist_launches": hist_launches,
                         "measured_in": "instrumented pass (CUDA events around every launch) of the same rounds right after the timed region",
                         "alg_bytes_per_launch": alg / max(1, hist_launches)},
            "kernel_ms_per_step": {k: v / args.steps for k, v in tm["ms"].items()},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "e2e": e2e,
            "inference": inference,
        }
        if not args.no_cpu_baseline and world == 1:
            try:
                dt, cores = cpu_baseline(np.asfortranarray(xb_host), y, depth, nbins, eta, args.cpu_rounds, int(args.tree_type == "oblivious"))
                out["cpu_baseline"] = {"value": dt * ROUNDS_PER_JOB, "unit": "s", "cores": cores, "kind": "port",
                                       "sample": f"{args.cpu_rounds} full boosting rounds on all {rows} rows (of {ROUNDS_PER_JOB}), scaled linearly"}
            except Exception as e:  # the baseline is reported, never required
                out["cpu_baseline"] = {"value": None, "unit": "s", "cores": None, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
