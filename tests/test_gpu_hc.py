"""GPU parity of the hyper-connection write and read (reference src/hc.cuh, src/kernels.cu:1493-1503) against the CPU
oracle, bit for bit: the streams after the folded write, the mixed row, its q8_1 copy and the inject values."""
import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,n,hc,lr,fold,inject", [(16, 3072, 4, 320, True, True), (16, 2560, 4, 320, True, True), (3, 1024, 2, 64, False, False),
                                                   (1, 512, 4, 32, True, False), (7, 1536, 3, 96, False, True)])
def test_hc_read(T, n, hc, lr, fold, inject):
    import oracle.binding as O
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    c = cases.hc_case(T, n, hc, lr, seed=70 + T, fold=fold, inject=inject)
    R_ref = c["R"].copy()
    mixed, inj, q8 = O.hc_read(R_ref, c["w_norm"], c["down"], c["up"], c["eps"], c["bo"], c["inj_prev"], c["w_inj"], want_q8=True)
    st = L.stream()
    R = G.dev(c["R"])
    dq, dd, uq, ud = G.dev(c["down"][0]), G.dev(c["down"][1]), G.dev(c["up"][0]), G.dev(c["up"][1])
    wn = G.dev(c["w_norm"])
    bo = G.dev(c["bo"]) if fold else None
    ip = G.dev(c["inj_prev"]) if fold else None
    wi = G.dev(c["w_inj"]) if inject else None
    d_mixed, d_inj = G.zeros((T, n)), G.zeros((T, hc))
    d_q8 = G.dev(np.zeros((T, n // 32 * 36), np.uint8))
    scratch = G.zeros(L.load().fnx_hc_scratch_floats(T, n, hc, lr))
    ptr = lambda t: t.data_ptr() if t is not None else None
    for _ in range(2):   # a second read of the same streams must not depend on what the first left in the scratch
        R.copy_(G.dev(c["R"]))
        L.call("fnx_hc_read", R.data_ptr(), ptr(bo), ptr(ip), wn.data_ptr(), L.Q8S(dq.data_ptr(), dd.data_ptr()), L.Q8S(uq.data_ptr(), ud.data_ptr()),
               ptr(wi), c["eps"], d_mixed.data_ptr(), d_inj.data_ptr() if inject else None, scratch.data_ptr(), d_q8.data_ptr(), T, n, hc, lr, st)
        G.sync()
        assert np.array_equal(G.host(R).view(np.uint32), R_ref.view(np.uint32)), "streams after the folded write"
        assert np.array_equal(G.host(d_mixed).view(np.uint32), mixed.view(np.uint32)), "mixed"
        assert np.array_equal(G.host(d_q8, np.uint8), q8), "mixed as q8_1"
        if inject:
            assert np.array_equal(G.host(d_inj).view(np.uint32), inj.view(np.uint32)), "inject"


def test_hc_write():
    import oracle.binding as O
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    c = cases.hc_case(5, 1024, 4, 32, seed=3)
    ref = c["R"].copy()
    O.hc_write(ref, c["bo"], c["inj_prev"])
    R, bo, inj = G.dev(c["R"]), G.dev(c["bo"]), G.dev(c["inj_prev"])
    L.call("fnx_hc_write", R.data_ptr(), bo.data_ptr(), inj.data_ptr(), 5, 1024, 4, L.stream())
    G.sync()
    assert np.array_equal(G.host(R).view(np.uint32), ref.view(np.uint32))


def test_hc_read_timing(capsys):
    """Device time of the read at the benchmark's width (T = 16, four streams of 3072, low rank 320), CUDA events over 50
    back-to-back reads after warm-up; printed, and held only to a loose bound (three dependent launches of a few
    microseconds each)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    T, n, hc, lr = 16, 3072, 4, 320
    c = cases.hc_case(T, n, hc, lr, seed=5)
    st = L.stream()
    R, wn = G.dev(c["R"]), G.dev(c["w_norm"])
    dq, dd, uq, ud = G.dev(c["down"][0]), G.dev(c["down"][1]), G.dev(c["up"][0]), G.dev(c["up"][1])
    bo, ip, wi = G.dev(c["bo"]), G.dev(c["inj_prev"]), G.dev(c["w_inj"])
    mixed, inj = G.zeros((T, n)), G.zeros((T, hc))
    q8 = G.dev(np.zeros((T, n // 32 * 36), np.uint8))
    scratch = G.zeros(L.load().fnx_hc_scratch_floats(T, n, hc, lr))

    def read():
        L.call("fnx_hc_read", R.data_ptr(), bo.data_ptr(), ip.data_ptr(), wn.data_ptr(), L.Q8S(dq.data_ptr(), dd.data_ptr()),
               L.Q8S(uq.data_ptr(), ud.data_ptr()), wi.data_ptr(), c["eps"], mixed.data_ptr(), inj.data_ptr(), scratch.data_ptr(), q8.data_ptr(), T, n,
               hc, lr, st)

    for _ in range(5):
        read()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(torch.cuda.current_stream())
    for _ in range(50):
        read()
    e1.record(torch.cuda.current_stream())
    G.sync()
    us = e0.elapsed_time(e1) * 1e3 / 50
    weights = 2 * lr * hc * n * 34 / 32 + hc * hc * n * 2   # down + up (split Q8_0) + inject rows (bf16)
    with capsys.disabled():
        print("\nhc_read T=16, 4 x 3072, low rank 320: %.1f us per read (three launches), %.2f MB of weights, %.0f GB/s" % (us, weights / 1e6, weights / us / 1e3))
    assert us < 200
