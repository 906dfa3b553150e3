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
