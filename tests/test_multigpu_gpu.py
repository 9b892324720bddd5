"""Row-sharded training on 2, 4 and 8 GPUs (peer-access histogram sums inside the split scan, or NCCL sums) against the
same fit on one GPU: same trees, same predictions.  Cases the box has too few GPUs for are skipped."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.conftest import ROOT

pytestmark = pytest.mark.gpu


def _ngpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_sharded_fit_equals_one_gpu(tmp_path, nproc):
    if _ngpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    out = tmp_path / "mgpu.npz"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + os.getpid() % 1000), os.path.join(ROOT, "tests", "mgpu_worker.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    z = np.load(out)
    for case in range(7):
        for rr in range(3):
            k = f"c{case}_"
            assert np.array_equal(z[k + f"s_feat{rr}"], z[k + f"1_feat{rr}"]), (case, rr)
            assert np.array_equal(z[k + f"s_cond_bin{rr}"], z[k + f"1_cond_bin{rr}"])
            assert np.array_equal(z[k + f"s_split{rr}"], z[k + f"1_split{rr}"])
            np.testing.assert_allclose(z[k + f"s_gain{rr}"], z[k + f"1_gain{rr}"], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(z[k + f"s_pred{rr}"], z[k + f"1_pred{rr}"], rtol=1e-5, atol=1e-6)
            np.testing.assert_allclose(z[k + f"s_w{rr}"], z[k + f"1_w{rr}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(z[k + "s_pred"], z[k + "1_pred"], rtol=1e-5, atol=1e-5)
