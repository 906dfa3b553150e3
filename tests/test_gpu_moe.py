"""GPU parity of the routed-expert FFN half against the CPU oracle through the C ABI: bit-exact router indices,
weights, jobs, gate|up, down, shared expert and combine on seeded cases (small, ragged, and the benchmark's shapes)."""
import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def _check(w, x, topk):
    from tests import gpu_util as G

    ref = cases.moe_oracle(w, x, topk)
    got = G.run_moe(w, x, topk)
    T = x.shape[0]
    assert np.array_equal(got["xq"], ref["xq"]), "q8_1 activations"
    assert np.array_equal(_bits(got["logits"]), _bits(ref["logits"])), "router logits"
    assert np.array_equal(got["topi"], ref["topi"]), "router indices"
    assert np.array_equal(_bits(got["topw"]), _bits(ref["topw"])), "router weights"
    assert got["njobs"] == ref["njobs"]
    nj = ref["njobs"]
    for name in ("jobs_gu", "jobs_dn"):
        g, r = got[name][:nj], ref[name][:nj]
        assert np.array_equal(g["w"], r["w"]) and np.array_equal(g["n"], r["n"]), name
        for j in range(nj):
            k = r["n"][j]
            assert np.array_equal(g["y"][j][:k], r["y"][j][:k]) and np.array_equal(g["out"][j][:k], r["out"][j][:k]), name
    assert np.array_equal(_bits(got["gu"]), _bits(ref["gu"])), "gate|up"
    assert np.array_equal(_bits(got["part"]), _bits(ref["part"])), "down"
    assert np.array_equal(_bits(got["sh_gu"]), _bits(ref["sh_gu"])), "shared gate|up"
    assert np.array_equal(_bits(got["sh"]), _bits(ref["sh"])), "shared down"
    assert np.array_equal(_bits(got["out"]), _bits(ref["out"])), "combine"
    assert got["counter"][:4].view(np.uint32)[0] == 0, "router block counter left at zero"
    return got


def test_moe_small_T16():
    rng = np.random.default_rng(21)
    w = cases.moe_weights(n=512, nexp=64, ffs=256, seed=1)
    _check(w, rng.standard_normal((16, 512)).astype(np.float32), topk=10)


def test_moe_single_row_and_ties():
    rng = np.random.default_rng(22)
    w = cases.moe_weights(n=1024, nexp=32, ffs=96, seed=2)   # ff width 96: the 8-GPU slice of 768
    w["router"][9] = w["router"][4]                          # tied logits: the lower index first
    _check(w, rng.standard_normal((1, 1024)).astype(np.float32), topk=10)
    x = rng.standard_normal((5, 1024)).astype(np.float32)
    x[3] = x[1]                                              # two rows routed alike: jobs of several rows
    x[2] = 0                                                 # an all-zero row: zero scales
    _check(w, x, topk=10)


def test_moe_all_rows_one_expert_set():
    """Every row identical: ten jobs of 16 rows each, the largest job shape."""
    rng = np.random.default_rng(23)
    w = cases.moe_weights(n=512, nexp=32, ffs=128, seed=3)
    x = np.repeat(rng.standard_normal((1, 512)).astype(np.float32), 16, axis=0)
    got = _check(w, x, topk=10)
    assert got["njobs"] == 10 and set(got["jobs_gu"]["n"][:10].tolist()) == {16}


def test_moe_benchmark_shape_hidden_3072():
    """Hidden 3072, FF 768, top-10 + shared, T = 16 as the benchmark's MoE layer, with 32 experts to keep the CPU side
    short (the expert count only changes which matrices are read)."""
    rng = np.random.default_rng(24)
    w = cases.moe_weights(n=3072, nexp=32, ffs=768, seed=4)
    _check(w, rng.standard_normal((16, 3072)).astype(np.float32), topk=10)


def test_moe_benchmark_shape_slices_of_four_and_eight_gpus():
    """The benchmark's hidden width with the FF slices a GPU of 4 or 8 holds (192 and 96 of 768): gate|up then takes two rows
    a lane group instead of four."""
    rng = np.random.default_rng(25)
    for ffs in (192, 96):
        w = cases.moe_weights(n=3072, nexp=32, ffs=ffs, seed=40 + ffs)
        x = rng.standard_normal((16, 3072)).astype(np.float32)
        x[5] = x[2]
        _check(w, x, topk=10)


def test_moe_q8_0_experts():
    """The all-Q8_0 configuration's routed experts: gate|up in the dense row-dot order, down in 32-column units; small and
    ragged shapes (FF slice 96), one row, tied routing, rows routed alike, and a job of 16 rows."""
    rng = np.random.default_rng(25)
    w = cases.moe_weights_q8(n=1024, nexp=32, ffs=96, seed=5)
    w["router"][9] = w["router"][4]
    _check(w, rng.standard_normal((1, 1024)).astype(np.float32), topk=10)
    x = rng.standard_normal((16, 1024)).astype(np.float32)
    x[3] = x[1]
    x[2] = 0
    _check(w, x, topk=10)
    w = cases.moe_weights_q8(n=512, nexp=32, ffs=128, seed=6)
    got = _check(w, np.repeat(rng.standard_normal((1, 512)).astype(np.float32), 16, axis=0), topk=10)
    assert got["njobs"] == 10


def test_moe_q8_0_experts_benchmark_shape():
    rng = np.random.default_rng(26)
    w = cases.moe_weights_q8(n=3072, nexp=32, ffs=768, seed=7)
    _check(w, rng.standard_normal((16, 3072)).astype(np.float32), topk=10)


def test_mmvq_is_the_job_matvec():
    """mmvq over a job list: the same entry as the experts' gate|up for the types it takes, refused for the others."""
    import ctypes as C

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(29)
    w = cases.moe_weights(n=512, nexp=16, ffs=128, seed=9)
    x = rng.standard_normal((7, 512)).astype(np.float32)
    ref = cases.moe_oracle(w, x, topk=4)
    nj, P = ref["njobs"], 7 * 4
    ex, keep = G.experts_q4k(w["gu_q4k"], 256, 512)
    dj, dn = G.dev(ref["jobs_gu"].view(np.uint8).reshape(-1)), G.dev(np.array([nj, 0], np.int32))
    dxq, out = G.dev(ref["xq"]), G.zeros((P, 256))
    L.call("fnx_mmvq", C.byref(ex), dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), out.data_ptr(), 256, L.stream())
    G.sync()
    assert np.array_equal(_bits(G.host(out)), _bits(ref["gu"]))
    assert L.load().fnx_mmvq(C.byref(ex), dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), out.data_ptr(), 300, L.stream()) != 0
    e6, keep6 = G.experts_q6p(w["dn_planes"], 512, 128)
    assert L.load().fnx_mmvq(C.byref(e6), dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), out.data_ptr(), 512, L.stream()) != 0
