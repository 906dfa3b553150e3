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


def _lanes_run(cs, T, with_snap):
    """Several sequences through one launch: lane s's rows are window rows s T .. s T + T - 1 (weights shared, taken
    from the first case)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    c0, nseg = cs[0], len(cs)
    nk, nv, ch = c0["nk"], c0["nv"], c0["ch"]
    qkvz, ab = G.dev(np.concatenate([c["qkvz"] for c in cs])), G.dev(np.concatenate([c["ab"] for c in cs]))
    w = {k: G.dev(c0[k]) for k in ("convw", "dt", "a", "nw", "vmap")}
    S, hist, ctl = [G.dev(c["S"]) for c in cs], [G.dev(c["hist"]) for c in cs], [G.dev(c["ctl"]) for c in cs]
    ptrs = lambda ts: G.dev(np.array([t.data_ptr() for t in ts], np.uint64))
    pS, ph, pc = ptrs(S), ptrs(hist), ptrs(ctl)
    rows = nseg * T
    yq = G.zeros(rows * (nv * 128 // 32) * 36, torch.uint8)
    scratch = G.zeros(L.load().fnx_gdn_scratch_floats(nv))
    if with_snap:
        row0 = G.dev(np.arange(nseg, dtype=np.int32) * T)
        snap, hsnap = G.zeros((rows, nv, 128, 128)), G.zeros((rows, 3, ch))
        gl = L.GdnLanes(pS.data_ptr(), ph.data_ptr(), pc.data_ptr(), row0.data_ptr(), snap.data_ptr(), hsnap.data_ptr())
        L.call("fnx_gdn_core_segs", qkvz.data_ptr(), ab.data_ptr(), w["convw"].data_ptr(), w["dt"].data_ptr(), w["a"].data_ptr(),
               w["nw"].data_ptr(), yq.data_ptr(), scratch.data_ptr(), nk, nv, w["vmap"].data_ptr(), C.byref(gl), nseg, T, c0["eps"], L.stream())
    else:
        snap = hsnap = None
        gl = L.GdnLanes(pS.data_ptr(), ph.data_ptr(), pc.data_ptr(), None, None, None)
        L.call("fnx_gdn_core_lanes", qkvz.data_ptr(), ab.data_ptr(), w["convw"].data_ptr(), w["dt"].data_ptr(), w["a"].data_ptr(),
               w["nw"].data_ptr(), yq.data_ptr(), scratch.data_ptr(), nk, nv, w["vmap"].data_ptr(), C.byref(gl), nseg, c0["eps"], L.stream())
    G.sync()
    return {"S": [G.host(t) for t in S], "hist": [G.host(t) for t in hist], "yq": G.host(yq).reshape(rows, -1),
            "snap": G.host(snap) if with_snap else None, "hsnap": G.host(hsnap) if with_snap else None}


def _lane_cases(nseg, T, nk, nv, seed):
    cs = [cases.gdn_case(T=T, nk=nk, nv=nv, seed=seed + s) for s in range(nseg)]
    for s, c in enumerate(cs):   # one layer's weights; every lane its own state, history, position and parity
        for k in ("convw", "dt", "a", "nw", "vmap"):
            c[k] = cs[0][k]
        c["ctl"] = np.array([100 * s + 7, 4 + s], np.int32)
    return cs


def test_gdn_segments_of_several_sequences():
    """Three sequences x 5 rows in one launch: each lane's outputs, state, history and checkpoints as a window of 5 rows
    on that lane alone gives them (batched lanes = alone)."""
    T, cs = 5, _lane_cases(3, 5, 2, 6, seed=70)
    got = _lanes_run(cs, T, with_snap=True)
    for s, c in enumerate(cs):
        ref = cases.gdn_oracle(c)
        assert np.array_equal(got["yq"][s * T:(s + 1) * T], ref["yq"]), s
        assert np.array_equal(got["S"][s].view(np.uint32), ref["S"].view(np.uint32)), s
        assert np.array_equal(got["hist"][s], ref["hist"]), s
        assert np.array_equal(got["snap"][s * T:s * T + T - 1].view(np.uint32), ref["snap"][:T - 1].view(np.uint32)), s
        assert np.array_equal(got["hsnap"][s * T:s * T + T - 1], ref["hsnap"][:T - 1]), s


def test_gdn_one_row_per_lane():
    """Six lanes, one row each (a batched decode step)."""
    cs = _lane_cases(6, 1, 2, 4, seed=80)
    got = _lanes_run(cs, 1, with_snap=False)
    for s, c in enumerate(cs):
        ref = cases.gdn_oracle(c)
        assert np.array_equal(got["yq"][s:s + 1], ref["yq"]), s
        assert np.array_equal(got["S"][s].view(np.uint32), ref["S"].view(np.uint32)), s
        assert np.array_equal(got["hist"][s], ref["hist"]), s


def test_gdn_log_and_replay_equal_the_checkpoints():
    """The window without checkpoints: fnx_gdn_core_log leaves the state as it was and gives the same output rows and conv
    history as fnx_gdn_core; fnx_gdn_replay of the first n rows gives, bit for bit, the checkpoint after row n - 1 (n < T) and
    the final state (n = T).  At the benchmark's head counts and at a small ragged shape."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    for nk, nv, T, seed in ((16, 48, 16, 37), (2, 6, 5, 38)):
        c = cases.gdn_case(T=T, nk=nk, nv=nv, seed=seed)
        ref = cases.gdn_oracle(c)
        t = {k: G.dev(c[k]) for k in ("qkvz", "ab", "hist", "convw", "dt", "a", "nw", "S", "vmap", "ctl")}
        yq = G.zeros(T * (nv * 128 // 32) * 36, torch.uint8)
        scratch = G.zeros(L.load().fnx_gdn_scratch_floats(nv))
        log = G.zeros(L.load().fnx_gdn_log_floats(nk, nv))
        hsnap = G.zeros((16, 3, c["ch"]))
        L.call("fnx_gdn_core_log", t["qkvz"].data_ptr(), t["ab"].data_ptr(), t["hist"].data_ptr(), t["convw"].data_ptr(), t["dt"].data_ptr(),
               t["a"].data_ptr(), t["nw"].data_ptr(), t["S"].data_ptr(), yq.data_ptr(), t["ctl"].data_ptr(), scratch.data_ptr(), log.data_ptr(),
               hsnap.data_ptr(), nk, nv, t["vmap"].data_ptr(), T, c["eps"], L.stream())
        G.sync()
        assert np.array_equal(G.host(yq).reshape(T, -1), ref["yq"]), "q8_1 output"
        assert np.array_equal(G.host(t["S"]), c["S"]), "the state is left as it was"
        assert np.array_equal(G.host(t["hist"]), ref["hist"]) and np.array_equal(G.host(hsnap)[: T - 1], ref["hsnap"][: T - 1])
        for n in range(1, T + 1):
            dS = G.dev(c["S"])
            job = L.GdnReplay(dS.data_ptr(), log.data_ptr(), t["vmap"].data_ptr(), nk, nv, 0, n)
            dj = torch.frombuffer(bytearray(bytes(job)), dtype=torch.uint8).to(G.DEV)
            L.call("fnx_gdn_replay", dj.data_ptr(), 1, nv, L.stream())
            G.sync()
            want = ref["S"] if n == T else ref["snap"][n - 1]
            assert np.array_equal(G.host(dS).view(np.uint32), want.view(np.uint32)), (nk, nv, n)
