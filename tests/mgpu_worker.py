"""Worker of tests/test_multigpu_gpu.py, launched once per GPU by torch.distributed.run.

Every rank builds the same synthetic data set, keeps its contiguous block of rows, and grows the same trees
through the row-sharded path (NCCL sums inside the library).  Rank 0 then repeats the fit on one GPU with all
rows and stores both results."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(out_path):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as g
    pkg = g.load_package()
    from evotrees_b200.dist import Comm, shard_bounds
    from evotrees_b200.fit import init_target
    from oracle import evo_oracle as orc

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Comm(dist, torch.device("cuda", local))
    results = {}
    # cases 4 and 6 grow oblivious trees, over peer access and over the NCCL sums
    for case, (loss, n, f, depth, nbins, rowsample, tree_type) in enumerate([
            ("mse", 60_001, 20, 7, 32, 1.0, "binary"), ("mse", 40_000, 9, 5, 16, 0.6, "binary"),
            ("gaussian_mle", 30_000, 12, 5, 32, 1.0, "binary"), ("mlogloss", 30_000, 8, 5, 16, 1.0, "binary"),
            ("mse", 50_000, 10, 5, 32, 1.0, "oblivious"),
            # quantile leaves: the ranks add the digit counts of the selection, so the leaves are those of one GPU
            ("quantile", 40_001, 8, 4, 32, 0.7, "binary"), ("mse", 30_000, 10, 5, 32, 1.0, "oblivious_nccl")]):
        p2p_default = comm.p2p
        comm.p2p = p2p_default and not tree_type.endswith("_nccl")
        tree_type = tree_type.split("_")[0]
        rng = np.random.default_rng(100 + case)
        x = rng.random((n, f)).astype(np.float32)
        raw = x @ rng.normal(size=f) + 0.2 * rng.normal(size=n)
        y = raw.astype(np.float32) if loss != "mlogloss" else np.digitize(raw, np.quantile(raw, [0.3, 0.7])).astype(np.int64)
        learner = {"mlogloss": pkg.EvoTreeClassifier, "gaussian_mle": pkg.EvoTreeMLE}.get(loss, pkg.EvoTreeRegressor)
        params = learner(loss=loss, nrounds=3, max_depth=depth, nbins=nbins, eta=0.3, rowsample=rowsample, tree_type=tree_type)
        edges = orc.get_edges(x, nbins, np.random.default_rng(1))
        x_bin = orc.binarize(x, edges)
        K, yd, ycols, mu, _, _ = init_target(loss, y, None)
        lo, hi = shard_bounds(n, world, rank)
        mrng = np.random.default_rng(5)
        masks = [mrng.integers(0, 256, n, dtype=np.uint8) if rowsample < 1 else None for _ in range(3)]
        js = np.arange(1, f + 1, dtype=np.uint32)

        def run(xb, yy, sl, cm):
            cache = pkg.init_core_binned(params, np.asfortranarray(xb), yy, ycols, K, mu, None, None, None, local, 0, cm)
            trees = []
            for r in range(3):
                m = None if masks[r] is None else np.ascontiguousarray(masks[r][sl])
                trees.append(pkg.grow_tree(cache, params, m, js, True))
            pred = cache.pred()
            cache.close()
            return trees, pred

        trees_s, pred_s = run(x_bin[lo:hi], yd[lo:hi], slice(lo, hi), comm)
        gathered = [None] * world
        dist.all_gather_object(gathered, pred_s)
        if rank == 0:
            trees_1, pred_1 = run(x_bin, yd, slice(0, n), None)
            for r in range(3):
                for name in ("feat", "cond_bin", "split", "gain", "pred", "w"):
                    results[f"c{case}_s_{name}{r}"] = getattr(trees_s[r], name)
                    results[f"c{case}_1_{name}{r}"] = getattr(trees_1[r], name)
            results[f"c{case}_s_pred"] = np.concatenate(gathered)
            results[f"c{case}_1_pred"] = pred_1
        comm.p2p = p2p_default
        dist.barrier()
    if rank == 0:
        np.savez(out_path, **results)
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
