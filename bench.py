"""Benchmark of the EvoTrees training / inference hot path on B200.

Metric: seconds per 200 boosting rounds.  Default workload = the headline of the reference's benchmark table: mse,
10M x 100 Float32 features, depth 11, 64 bins, rows sharded over --gpus GPUs (strong scaling).  A "step" is one boosting
round over synthetic data of that shape (the reference's own benchmark data is synthetic too, benchmarks/regressor.jl).
The other configurations of the benchmark list are selectable with --workload.

  python bench.py --gpus N --steps K --warmup W            # this library
  python bench.py --impl reference --steps K --warmup W    # CPU restatement of the reference's CPU path (oracle)

Prints one JSON line (rank 0):
  value      device time of K boosting rounds scaled to 200, the training data already resident in HBM
  e2e        wall time of the public call `fit(params, x_train=, y_train=)` for all 200 rounds from an ordinary
             (pageable) Float32 host matrix: quantile edges on the host, upload + binarize on the device, boosting loop,
             every tree read back -- whatever --steps says
  roofline   the histogram kernel: algorithmic bytes / its summed CUDA-event time, against the measured HBM copy peak
  inference  `m(x)` from raw host features (upload, device binarize, all 201 trees, predictions back), rows sharded
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
    "headline_10Mx100_d11": dict(rows=10_000_000, feats=100, depth=11, nbins=64, eta=0.1, rowsample=1.0, colsample=1.0,
                                 loss="mse", data="uniform_linear"),
    "cfg2_1Mx100_d6": dict(rows=1_000_000, feats=100, depth=6, nbins=64, eta=0.05, rowsample=0.5, colsample=0.5,
                           loss="mse", data="uniform_linear"),
    "cfg1_100kx10_d6": dict(rows=100_000, feats=10, depth=6, nbins=32, eta=0.1, rowsample=1.0, colsample=1.0,
                            loss="mse", data="uniform_linear"),
    "cfg4_2Mx28_softmax_d8": dict(rows=2_000_000, feats=28, depth=8, nbins=64, eta=0.1, rowsample=1.0, colsample=1.0,
                                  loss="mlogloss", classes=5, data="normal_softmax"),
    "cfg5_5Mx50_gaussian_d7": dict(rows=5_000_000, feats=50, depth=7, nbins=32, eta=0.1, rowsample=1.0, colsample=1.0,
                                   loss="gaussian_mle", data="uniform_hetero", predict_rows=10_000_000),
}
ROUNDS_PER_JOB = 200


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="headline_10Mx100_d11", choices=list(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the number of rows (for quick checks and profiler captures)")
    ap.add_argument("--tree-type", default="binary", choices=["binary", "oblivious"], help="not the headline: side measurements")
    ap.add_argument("--cpu-rounds", type=int, default=2, help="rounds of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-inference", action="store_true")
    return ap.parse_args()


def make_shard(w, rows_total, rank, world, seed=123):
    """Rows [lo, hi) of the synthetic data set of workload `w`: x float32 [n, feats] in column-major order (what a Julia
    Matrix is) and the target.  Every rank draws its own block from a rank-specific stream."""
    feats = w["feats"]
    per = -(-rows_total // world)
    lo, hi = min(rows_total, rank * per), min(rows_total, (rank + 1) * per)
    n = hi - lo
    rng = np.random.default_rng([seed, rank])
    par = np.random.default_rng(seed)
    x = np.empty((n, feats), np.float32, order="F")
    if w["data"] == "normal_softmax":        # x ~ N(0,1), label = argmax(x W + Gumbel(0,1))
        W = par.normal(size=(feats, w["classes"])).astype(np.float32)
        for j in range(feats):
            x[:, j] = rng.standard_normal(n, dtype=np.float32)
        logits = x @ W
        logits -= np.log(-np.log(rng.random(logits.shape, dtype=np.float32) * np.float32(0.999998) + np.float32(1e-6)))
        return x, np.argmax(logits, axis=1).astype(np.int64)
    beta = par.normal(size=feats).astype(np.float32)
    for j in range(feats):
        x[:, j] = rng.random(n, dtype=np.float32)
    noise = rng.standard_normal(n, dtype=np.float32)
    if w["data"] == "uniform_hetero":        # y = x.beta + exp(0.5 x_1) N(0,1)
        y = x @ beta + np.exp(np.float32(0.5) * x[:, 0]) * noise
    else:                                    # y = x.beta + 0.1 N(0,1)
        y = x @ beta + np.float32(0.1) * noise
    return x, y.astype(np.float32)


def make_params(pkg, w, tree_type="binary", nrounds=ROUNDS_PER_JOB):
    kw = dict(nrounds=nrounds, max_depth=w["depth"], nbins=w["nbins"], eta=w["eta"], rowsample=w["rowsample"],
              colsample=w["colsample"], tree_type=tree_type)
    if w["loss"] == "mlogloss":
        return pkg.EvoTreeClassifier(**kw)
    if w["loss"] == "gaussian_mle":
        return pkg.EvoTreeMLE(loss="gaussian_mle", **kw)      # min_weight = 8, the learner's default
    return pkg.EvoTreeRegressor(loss=w["loss"], **kw)


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


def oracle_setup(w, x, y, tree_type=0):
    """CPU restatement of the reference's CPU path on the whole matrix: returns (booster, seconds of get_edges + binarize,
    threads).  All host cores are used whatever OMP_NUM_THREADS says (torch.distributed.run exports 1)."""
    from oracle import evo_oracle as orc
    cores = orc.use_all_cores()
    t0 = time.perf_counter()
    rng = np.random.default_rng(123)
    edges = orc.get_edges(x, w["nbins"], rng)
    x_bin = orc.binarize(x, edges)
    t_init = time.perf_counter() - t0
    if w["loss"] == "mlogloss":
        K, yd = w["classes"], (y + 1).astype(np.uint32)
    elif w["loss"] == "gaussian_mle":
        K, yd = 2, y
    else:
        K, yd = 1, y
    p = orc.Params(loss=w["loss"], K=K, nbins=w["nbins"], max_depth=w["depth"], eta=w["eta"], tree_type=tree_type,
                   min_weight=8.0 if w["loss"] == "gaussian_mle" else 1.0)
    b = orc.Booster(p, x_bin, yd, use_x_bin_T=True)
    return b, t_init, cores


def oracle_rounds(w, b, rounds, seed=123):
    """Seconds per boosting round of the oracle, row / column sampling of the workload included."""
    nobs, feats = b.x_bin.shape
    rng = np.random.default_rng(seed)
    njs = int(np.ceil(w["colsample"] * feats))
    cond = int(np.uint8(round(255 * w["rowsample"])))

    def one():
        mask = rng.integers(0, 256, size=nobs, dtype=np.uint8) if w["rowsample"] < 1 else None
        js = (np.arange(1, feats + 1) if njs >= feats else np.sort(rng.choice(feats, njs, replace=False)) + 1).astype(np.uint32)
        b.round(mask, cond, js)

    one()  # warm-up round (page faults, thread pool)
    t0 = time.perf_counter()
    for _ in range(rounds):
        one()
    return (time.perf_counter() - t0) / rounds


def run_reference(args):
    """Reference arm: the reference is Julia and no Julia runtime exists in this image, so the CPU restatement of its CPU
    path (oracle/) is timed instead, with all host cores, on the same workload.  `value` is the boosting loop (a bounded
    sample of full rounds on all rows, scaled to 200), `e2e` adds the oracle's get_edges + binarize."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    rows = args.rows or w["rows"]
    x, y = make_shard(w, rows, 0, 1)
    b, t_init, cores = oracle_setup(w, x, y, int(args.tree_type == "oblivious"))
    del x
    steps = max(1, min(args.steps, 8))      # bounded sample: every step is one full boosting round on all rows
    sec = oracle_rounds(w, b, steps)
    val = sec * ROUNDS_PER_JOB
    sample = f"{steps} full boosting rounds on all {rows} rows (of {ROUNDS_PER_JOB}), scaled linearly"
    out = {"impl": "reference", "metric": "train_seconds_per_200_rounds", "value": val, "unit": "s", "n_gpus": args.gpus,
           "steps": steps, "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": False, "scaling": "strong",
           "vs_baseline": None, "dtype": "f32 gradients, f64 histograms", "data": "synthetic",
           "config": {"workload": args.workload, "rows": rows, "feats": w["feats"], "max_depth": w["depth"], "nbins": w["nbins"], "loss": w["loss"]},
           "cpu_baseline": {"value": val, "unit": "s", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": val + t_init, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "init_s": t_init,
                   "init": "get_edges + binarize of the oracle on the host"},
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
    from evotrees_b200.dist import Comm

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

    w = WORKLOADS[args.workload]
    rows = args.rows or w["rows"]
    feats, depth, nbins = w["feats"], w["depth"], w["nbins"]
    K = {"mse": 1, "mlogloss": w.get("classes", 0), "gaussian_mle": 2}[w["loss"]]
    C = 2 * K + 1
    params = make_params(pkg, w, args.tree_type)
    x, y = make_shard(w, rows, rank, world)       # ordinary (pageable) host memory
    nloc = x.shape[0]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return float(v)
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident loop: `value` --------------------------------------------------------------------
    def run_rounds(cache, k):
        """k boosting rounds, the host one tree ahead of the GPU (how `fit` drives the library)."""
        in_flight = 0
        for _ in range(k):
            mask, js = pkg.sample_round(cache, params)
            pkg.grow_tree_begin(cache, params, mask, js, True)
            in_flight += 1
            if in_flight == 2:
                pkg.grow_tree_end(cache, params)
                in_flight -= 1
        while in_flight:
            pkg.grow_tree_end(cache, params)
            in_flight -= 1

    _, cache = pkg.init_core(params, x, y, device=local, comm=comm)
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
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop() if rank == 0 else None
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

    # ---- end to end through the public call: `e2e` ---------------------------------------------------------
    e2e = None
    inference = None
    model = None
    nn = 2 ** depth - 1
    if not args.no_e2e:
        sync_all()
        t0 = time.perf_counter()
        model = pkg.fit(params, x_train=x, y_train=y, device=local, comm=comm)   # all ROUNDS_PER_JOB rounds, from raw host features
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        assert len(model.trees) == ROUNDS_PER_JOB + 1
        h2d = (nloc * feats * 4 + nloc * 4) / ROUNDS_PER_JOB + feats * 4 + (nloc if w["rowsample"] < 1 else 0)
        d2h = nn * (4 + 4 + 4 + 4 * K + 4 + 1 + 1) + 24 * (depth + 2) + 32
        e2e = {"value": e2e_s, "unit": "s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "rounds": ROUNDS_PER_JOB,
               "call": "fit(params, x_train=, y_train=): edges on the host, raw Float32 features from pageable memory, binarize on the device, "
                       "all 200 rounds, every tree read back"}
    if model is not None and not args.no_inference:
        # `m(x)` from raw host features, rows sharded over the ranks (no collective): the training shard, or fresh rows
        # where the workload asks for them
        if w.get("predict_rows"):
            xp, _ = make_shard(w, w["predict_rows"] if not args.rows else args.rows, rank, world, seed=321)
        else:
            xp = x
        pkg.predict(model, xp[:1000], device=local)          # warm-up
        times, kms = [], []
        for _ in range(5):
            sync_all()
            st = {}
            t0 = time.perf_counter()
            pkg.predict(model, xp, device=local, stats=st)
            times.append(time.perf_counter() - t0)
            kms.append(st.get("kernel_ms", 0.0))
        t_med = max_over_ranks(float(np.median(times)))
        k_med = max_over_ranks(float(np.median(kms)))
        rows_all = xp.shape[0] * world if world > 1 else xp.shape[0]
        inference = {"rows_per_s": rows_all / t_med, "seconds": t_med, "rows": rows_all, "trees": len(model.trees), "repeats": 5,
                     "kernel_ms": k_med, "alg_bytes": int(xp.shape[0] * (feats + 4 * K)),
                     "input": "raw Float32 host features (pageable): H2D, device binarize, all trees, D2H of the predictions inside the timed region; "
                              "median of 5, max over ranks"}

    if rank == 0:
        F = int(np.ceil(w["colsample"] * feats))
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
        traffic = None
        if args.workload == "headline_10Mx100_d11" and hist_launches:
            # DRAM bytes per launch from an ncu capture of a 2M-row case of this workload (dram__bytes_read + write): 110 B
            # per row for the root launch (rows are contiguous: 96 + 8 + 4 bytes), 158 B per row below the root (gathered
            # rows: whole 64-byte DRAM bursts), scaled by the rows of a launch
            root_rows = nloc * tm["trees"]
            traffic = (110.0 * root_rows + 158.0 * max(0, tm["hist_rows"] - root_rows)) / hist_launches
        if inference is not None:
            inference["hbm_frac_kernels"] = (inference["alg_bytes"] / (inference["kernel_ms"] * 1e-3) / 1e9 / peak) if inference["kernel_ms"] else None
        out = {
            "metric": "train_seconds_per_200_rounds", "value": ms_step * ROUNDS_PER_JOB / 1e3, "unit": "s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": ("f32 gradients, exact 24-bit fixed-point sums (u32 reductions in shared memory, 64-bit accumulators), f64 split scan"
                      if w["loss"] == "mse" else "f32 gradients, f32 partial sums in shared memory, f64 histograms and split scan"),
            "data": "synthetic",
            "config": {"workload": args.workload, "rows": rows, "feats": feats, "max_depth": depth, "nbins": nbins, "loss": w["loss"], "tree_type": args.tree_type,
                       "eta": w["eta"], "rowsample": w["rowsample"], "colsample": w["colsample"], "rows_per_gpu": nloc,
                       "l2_policy": "inputs larger than L2 (bins of the shard: %.0f MB)" % (nloc * (feats + 8) / 1e6)},
            "roofline": {"bound": "hbm", "kernel": "k_histq2" if w["loss"] == "mse" else "k_hist", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": traffic,
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
                b, t_init, cores = oracle_setup(w, x, y, int(args.tree_type == "oblivious"))
                sec = oracle_rounds(w, b, args.cpu_rounds)
                out["cpu_baseline"] = {"value": sec * ROUNDS_PER_JOB, "unit": "s", "cores": cores, "kind": "port", "init_s": t_init,
                                       "sample": f"{args.cpu_rounds} full boosting rounds on all {rows} rows (of {ROUNDS_PER_JOB}), scaled linearly"}
            except Exception as e:  # the baseline is reported, never required
                out["cpu_baseline"] = {"value": None, "unit": "s", "cores": None, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
