"""Error paths of the C ABI that never fault or hang a GPU: a handle used by two host threads at once, a bounded wait
for a peer that runs out, out-of-order calls of the peer-access set-up, and a device allocation that fails in the middle
of evb_create (injected on the host)."""
import ctypes as C
import os
import threading
import time

import numpy as np
import pytest

from tests.parity import make_regression

pytestmark = pytest.mark.gpu


def _cache(pkg, n=200_000, f=20, depth=8, **kw):
    from evotrees_b200.fit import init_target
    x, y = make_regression(n, f, seed=3)
    params = pkg.EvoTreeRegressor(loss="mse", nrounds=1, max_depth=depth, nbins=32, **kw)
    rng = np.random.default_rng(1)
    edges, _, _ = pkg.get_edges(x, 32, rng)
    K, yd, ycols, mu, _, _ = init_target("mse", y, None)
    cache = pkg.init_core_binned(params, None, yd, ycols, K, mu, x_raw=np.asfortranarray(x), edges=edges)
    return cache, params


def test_handle_in_use_by_another_thread_reports_busy(pkg):
    from evotrees_b200 import _lib
    cache, params = _cache(pkg)
    js = np.arange(1, cache.nfeats + 1, dtype=np.uint32)
    codes, stop = [], threading.Event()

    def poke():                      # a second host thread keeps asking the same handle for its timings
        t = _lib.EvbTimings()
        while not stop.is_set():
            codes.append(_lib.lib().evb_get_timings(cache.handle, C.byref(t)))
            time.sleep(1e-4)         # a tree takes milliseconds: ten looks per tree are plenty

    def grow():                      # the owner may itself meet the other thread inside the handle: it just calls again
        for _ in range(2000):
            try:
                return pkg.grow_tree(cache, params, None, js, True)
            except _lib.EvbError as e:
                if e.code != -6:
                    raise
                time.sleep(5e-4)
        raise AssertionError("the handle stayed busy")

    th = threading.Thread(target=poke)
    th.start()
    try:
        for _ in range(30):
            grow()                                                # each call holds the handle for a few milliseconds
    finally:
        stop.set()
        th.join()
    assert set(codes) <= {0, -6}, set(codes)
    assert -6 in codes, "the second thread never saw EVB_ERR_BUSY"
    assert pkg.grow_tree(cache, params, None, js, True).split[0]   # the handle works as before
    cache.close()


def test_bounded_wait_for_a_silent_peer_runs_out(pkg):
    from evotrees_b200 import _lib
    cache, params = _cache(pkg, n=20_000)
    rc = _lib.lib().evb_test_peer_timeout(cache.handle, C.c_int32(20_000))      # about 2 ms of polling
    assert rc == -5, rc                                                           # EVB_ERR_DEVICE
    assert "wait for the other ranks expired" in _lib.lib().evb_last_error().decode()
    js = np.arange(1, cache.nfeats + 1, dtype=np.uint32)
    assert pkg.grow_tree(cache, params, None, js, True).split[0]                 # the handle is still usable
    assert _lib.lib().evb_test_peer_timeout(cache.handle, C.c_int32(0)) == -1     # argument check
    cache.close()


def test_peer_access_setup_out_of_order(pkg):
    from evotrees_b200 import _lib
    lib = _lib.lib()
    cache, _ = _cache(pkg, n=20_000)
    blob = np.zeros(256, np.uint8)
    assert lib.evb_comm_ipc_export(cache.handle, _lib.ptr(blob)) == -1           # no evb_comm_init before
    assert "evb_comm_init" in lib.evb_last_error().decode()
    assert lib.evb_comm_ipc_import(cache.handle, _lib.ptr(np.zeros(512, np.uint8))) == -1   # import before export
    assert lib.evb_comm_ipc_import(cache.handle, None) == 0                      # "no peer access": always allowed
    ident = np.zeros(128, np.uint8)
    assert lib.evb_comm_init(cache.handle, _lib.ptr(ident), C.c_int32(3), C.c_int32(2)) == -1   # rank outside the world
    assert lib.evb_comm_init(cache.handle, None, C.c_int32(0), C.c_int32(2)) == -1              # null id
    cache.close()


@pytest.mark.parametrize("kth", [1, 5, 17, 30])
def test_failed_allocation_inside_create_frees_everything(pkg, kth):
    import torch
    from evotrees_b200 import _lib
    cache, _ = _cache(pkg, n=50_000)        # warm-up: context, pinned staging ring, kernel attributes
    cache.close()
    assert _lib.lib().evb_trim_cache(C.c_int32(0)) == 0     # released blocks are kept for reuse: hand them back first
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0]
    os.environ["EVB_TEST_FAIL_ALLOC"] = str(kth)
    try:
        with pytest.raises(_lib.EvbError) as ei:
            _cache(pkg, n=50_000)
        assert ei.value.code == -2 and "out of memory" in str(ei.value).lower()
    finally:
        del os.environ["EVB_TEST_FAIL_ALLOC"]
    assert _lib.lib().evb_trim_cache(C.c_int32(0)) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_before, "a failed evb_create left device memory behind"
    cache, params = _cache(pkg, n=50_000)   # and the next create works
    js = np.arange(1, cache.nfeats + 1, dtype=np.uint32)
    assert pkg.grow_tree(cache, params, None, js, True).split[0]
    cache.close()


def test_released_blocks_are_reused_and_trimmed(pkg):
    """evb_destroy keeps the device blocks; an equal evb_create takes them back (no growth), evb_trim_cache returns them."""
    import torch
    from evotrees_b200 import _lib
    lib = _lib.lib()
    cache, _ = _cache(pkg, n=200_000)
    cache.close()
    assert lib.evb_trim_cache(C.c_int32(0)) == 0
    torch.cuda.synchronize()
    free_empty = torch.cuda.mem_get_info(0)[0]
    cache, params = _cache(pkg, n=200_000)
    torch.cuda.synchronize()
    free_live = torch.cuda.mem_get_info(0)[0]
    assert free_live < free_empty
    cache.close()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_live          # nothing went back to the driver
    cache, params = _cache(pkg, n=200_000)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_live          # and nothing new was taken
    js = np.arange(1, cache.nfeats + 1, dtype=np.uint32)
    t1 = pkg.grow_tree(cache, params, None, js, True)
    cache.close()
    cache, params = _cache(pkg, n=200_000)                     # reused blocks hold the old handle's data: same tree all the same
    t2 = pkg.grow_tree(cache, params, None, js, True)
    assert np.array_equal(t1.feat, t2.feat) and np.array_equal(t1.cond_bin, t2.cond_bin) and np.array_equal(t1.pred, t2.pred)
    cache.close()
    assert lib.evb_trim_cache(C.c_int32(0)) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_empty
    assert lib.evb_trim_cache(C.c_int32(99)) == -1
