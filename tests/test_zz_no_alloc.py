"""The down projection without a caller-supplied scratch buffer (fnx_moe_down_noalloc): for hosts that cannot allocate
device memory, the pairs' quantised h is kept in an array inside the library.  Its output must have the bits of
fnx_moe_down's on the same inputs, call after call, and a request beyond the array is refused with a clear text."""
import ctypes as C

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


def test_down_without_caller_scratch_matches_down():
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(91)
    w = cases.moe_weights(n=512, nexp=32, ffs=256, seed=17)
    n, nexp, ffs, topk = 512, 32, 256, 10
    edn, keep = G.experts_q6p(w["dn_planes"], n, ffs)
    st = L.stream()
    for call, T in enumerate((16, 5)):   # two calls in a row, of different sizes: the second finds the first one's bytes there
        x = rng.standard_normal((T, n)).astype(np.float32)
        ref = cases.moe_oracle(w, x, topk)
        P = T * topk
        gu, jobs = G.dev(ref["gu"]), G.dev(ref["jobs_dn"])
        njobs = G.dev(np.array([ref["njobs"], 0], np.int32))
        hq = G.zeros(L.load().fnx_moe_h_bytes(P, ffs), torch.uint8)
        part_a, part_b = G.zeros((P, n)), G.zeros((P, n))
        L.call("fnx_moe_down", C.byref(edn), jobs.data_ptr(), njobs.data_ptr(), P, gu.data_ptr(), P, hq.data_ptr(), part_a.data_ptr(), st)
        L.call("fnx_moe_down_noalloc", C.byref(edn), jobs.data_ptr(), njobs.data_ptr(), P, gu.data_ptr(), P, part_b.data_ptr(), st)
        G.sync()
        a, b = G.host(part_a), G.host(part_b)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), "call %d" % call
        assert np.array_equal(b.view(np.uint32), ref["part"].view(np.uint32)), "call %d against the oracle" % call
    big = L.Experts(L.Q6_K, n, 4096, None, None, None, None, 0, 0)
    with pytest.raises(L.FnxError, match="the built-in array holds"):
        L.call("fnx_moe_down_noalloc", C.byref(big), None, None, 160, None, 160, None, st)
