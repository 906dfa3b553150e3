"""GPU parity of the Gated DeltaNet core with checkpoints and of the rollback, bit-exact against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


def _check(c):
    from tests import gpu_util as G

    ref = cases.gdn_oracle(c)
    got = G.run_gdn(c)
    T = c["T"]
    assert np.array_equal(got["y32"].view(np.uint32), ref["y32"].view(np.uint32)), "gated output"
    assert np.array_equal(got["yq"], ref["yq"]), "q8_1 output"
    assert np.array_equal(got["S"].view(np.uint32), ref["S"].view(np.uint32)), "state"
    if T > 1:
        assert np.array_equal(got["snap"][: T - 1].view(np.uint32), ref["snap"][: T - 1].view(np.uint32)), "checkpoints"
        assert np.array_equal(got["hsnap"][: T - 1], ref["hsnap"][: T - 1]), "history variants"
    assert np.array_equal(got["hist"], ref["hist"]), "conv history"
    assert not got["scratch_tail"].any(), "per-head counters left at zero"
    return ref, got


def test_gdn_small():
    _check(cases.gdn_case(T=16, nk=2, nv=6, seed=31))


def test_gdn_rows_1_2_5():
    for T in (1, 2, 5):
        _check(cases.gdn_case(T=T, nk=2, nv=4, seed=32 + T))


def test_gdn_benchmark_shape_with_rollback():
    """16 key heads, 48 value heads, T = 16 with 15 checkpoints; then the rollback to a prefix n drawn from 1..16 through
    fnx_copy_many, compared with the oracle's rollback; n = T copies nothing."""
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    c = cases.gdn_case(T=16, nk=16, nv=48, seed=35)
    ref, got = _check(c)
    t, snap, hsnap = got["dev"]
    rng = np.random.default_rng(36)
    ch = c["ch"]
    for n in sorted(set(rng.integers(1, 17, 4).tolist() + [16])):
        S, hist = ref["S"].copy(), ref["hist"].copy()
        cases.O.gdn_rollback(S, hist, ref["snap"], ref["hsnap"], c["ctl"], 16, 48, 16, n)
        dS, dh = G.dev(got["S"]), G.dev(got["hist"])
        if n < 16:
            jobs = (L.CopyJob * 2)(L.CopyJob(dS.data_ptr(), snap[n - 1].data_ptr(), 48 * 128 * 128 * 4),
                                   L.CopyJob(dh[0].data_ptr(), hsnap[n - 1].data_ptr(), 3 * ch * 4))
            import torch

            dj = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8).to(G.DEV)
            L.call("fnx_copy_many", dj.data_ptr(), 2, L.stream())
        G.sync()
        assert np.array_equal(G.host(dS), S) and np.array_equal(G.host(dh), hist), n
