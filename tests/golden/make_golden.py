"""Generates the golden fixtures of tests/golden/ with the CPU oracle.

    python tests/golden/make_golden.py

No Julia runtime exists in the build image, so these vectors come from the C restatement of the reference
(oracle/evo_oracle.c), not from the reference itself; they freeze the oracle's behaviour so that a change
in either the oracle or the CUDA library shows up as a diff against committed numbers.  Each file holds the
binned inputs, the per-round row masks / column samples, every tree of three boosting rounds and the final
predictions for one loss.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import evo_oracle as orc  # noqa: E402

CASES = {
    "mse": dict(K=1, depth=4, nbins=16, rowsample=0.7, colsample=0.75, eta=0.3),
    "logloss": dict(K=1, depth=3, nbins=8, rowsample=1.0, colsample=1.0, eta=0.5),
    "mlogloss": dict(K=3, depth=3, nbins=12, rowsample=1.0, colsample=1.0, eta=0.5),
    "gaussian_mle": dict(K=2, depth=3, nbins=16, rowsample=1.0, colsample=1.0, eta=0.3, min_weight=8.0),
}
ROUNDS, N, F = 3, 1500, 6


def make_case(loss, c, seed):
    rng = np.random.default_rng(seed)
    x = rng.random((N, F)).astype(np.float32)
    raw = np.sin(5 * x[:, 0]) + x[:, 1] * x[:, 2] - x[:, 3] + 0.05 * rng.normal(size=N)
    if loss == "mse":
        y = raw.astype(np.float32)
    elif loss == "logloss":
        y = (raw > np.median(raw)).astype(np.float32)
    elif loss == "mlogloss":
        y = (np.digitize(raw, np.quantile(raw, [1 / 3, 2 / 3])) + 1).astype(np.uint32)
    else:
        y = (raw + np.exp(0.5 * x[:, 0]) * rng.normal(size=N)).astype(np.float32)
    w = rng.uniform(0.5, 2.0, N).astype(np.float32)
    edges = orc.get_edges(x, c["nbins"], rng)
    x_bin = orc.binarize(x, edges)
    p = orc.Params(loss=loss, K=c["K"], nbins=c["nbins"], max_depth=c["depth"], eta=c["eta"], min_weight=c.get("min_weight", 1.0))
    b = orc.Booster(p, x_bin, y, w)
    njs = int(np.ceil(c["colsample"] * F))
    cond = int(np.uint8(round(255 * c["rowsample"])))
    out = dict(x_bin=x_bin, y=y, w=w, mu=b.mu, mask_cond=np.array(cond), pred0=b.pred.copy())
    for r in range(ROUNDS):
        mask = rng.integers(0, 256, N, dtype=np.uint8) if c["rowsample"] < 1 else np.zeros(0, np.uint8)
        js = (np.sort(rng.choice(F, njs, replace=False)) + 1).astype(np.uint32)
        t, nidx, _, nsum = b.round(mask if mask.size else None, cond, js)
        out.update({f"mask{r}": mask, f"js{r}": js, f"feat{r}": t.feat, f"cond_bin{r}": t.cond_bin, f"split{r}": t.split,
                    f"gain{r}": t.gain, f"w{r}": t.w, f"leaf{r}": t.pred, f"nidx{r}": nidx, f"pred{r}": b.pred.copy()})
    return out


if __name__ == "__main__":
    for i, (loss, c) in enumerate(CASES.items()):
        np.savez_compressed(os.path.join(HERE, f"{loss}.npz"), **make_case(loss, c, 100 + i))
        print("wrote", loss)
