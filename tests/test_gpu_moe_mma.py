"""GPU parity of the routed experts over many rows (the prompt path's jobs of up to 64 rows, tcgen05 tensor cores)
against the CPU oracle through the C ABI: the f16 weights bit for bit (read back through one-hot rows), the sums to a
stated bound on fp32 summation error, SwiGLU to f16 bit for bit."""
import ctypes as C

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


def _f16_bits(a):
    return np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)


def _run(entry, experts, jobs, x16, nout):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    st = L.stream()
    dj = G.dev(jobs.view(np.uint8).reshape(-1))
    nj = G.dev(np.array([len(jobs), 0], np.int32))
    dx = G.dev(x16)
    out = torch.full((nout, experts.nrows), float("nan"), device="cuda")
    L.call(entry, C.byref(experts), dj.data_ptr(), nj.data_ptr(), len(jobs) + 3, dx.data_ptr(), out.data_ptr(), st)   # spare grid rows do nothing
    G.sync()
    assert L.load().fnx_device_fault() == 0
    return G.host(out)


def _close(got, ref, mag, n):
    """fp32 sums of exact products in an unstated order, one partial sum per 16 columns: each step may lose one fp32 unit
    in the last place of the running magnitude, so |got - ref| <= (n / 16 + 8) 2^-23 sum|products|."""
    bound = (n / 16 + 8) * 2.0 ** -23 * mag + 1e-30
    err = np.abs(got.astype(np.float64) - ref)
    assert np.isfinite(got).all()
    assert (err <= bound).all(), (float((err / bound).max()), float(err.max()))


def _experts(w, which):
    from tests import gpu_util as G

    n, ffs = w["n"], w["ffs"]
    if w.get("experts") == "q8_0":
        return G.experts_q8(w["gu_q8"], 2 * ffs, n) if which == "gu" else G.experts_q8(w["dn_q8"], n, ffs)
    return G.experts_q4k(w["gu_q4k"], 2 * ffs, n) if which == "gu" else G.experts_q6p(w["dn_planes"], n, ffs)


def _weights16(w, which):
    """The oracle's f16 weights [experts * rows][cols]."""
    from oracle import binding as O

    n, ffs, nexp = w["n"], w["ffs"], w["nexp"]
    if w.get("experts") == "q8_0":
        q, d = w["gu_q8"] if which == "gu" else w["dn_q8"]
        return O.mma_weights_q8(q, d)
    if which == "gu":
        return O.mma_weights_q4k(w["gu_q4k"], nexp * 2 * ffs, n)
    return O.mma_weights_q6p(w["dn_planes"], nexp * n, ffs)


@pytest.mark.parametrize("kind", ["q4k", "q8_0"])
def test_f16_weights_bit_exact_through_one_hot_rows(kind):
    """Row s of a job is the unit vector of column 64 j + s: the job's output is 64 columns of the expert's f16 weights,
    each sum a single non-zero product, so the dequantisation is read back bit for bit."""
    n, ffs, nexp = 512, 256, 3
    w = (cases.moe_weights if kind == "q4k" else cases.moe_weights_q8)(n=n, nexp=nexp, ffs=ffs, seed=31)
    from oracle import binding as O

    for which, cols, rows in (("gu", n, 2 * ffs), ("dn", ffs, n)):
        x = np.zeros((cols, cols), np.float16)
        x[np.arange(cols), np.arange(cols)] = 1
        jobs = np.zeros(nexp * cols // 64, O.BIGJOB_DTYPE)
        for e in range(nexp):
            for j in range(cols // 64):
                jb = jobs[e * (cols // 64) + j]
                jb["w"], jb["n"] = e, 64
                jb["y"][:] = np.arange(64) + 64 * j
                jb["out"][:] = e * cols + jb["y"]
        ex, keep = _experts(w, which)
        got = _run("fnx_moe_gate_up_mma" if which == "gu" else "fnx_moe_down_mma", ex, jobs, x.view(np.uint16), nexp * cols)
        ref = _weights16(w, which).view(np.float16).reshape(nexp, rows, cols).transpose(0, 2, 1).reshape(nexp * cols, rows)
        assert np.array_equal(got.astype(np.float32).view(np.uint32), ref.astype(np.float32).view(np.uint32)), which


@pytest.mark.parametrize("kind,n,ffs,nexp,ntok,topk", [("q4k", 512, 256, 8, 150, 4), ("q8_0", 1024, 96, 6, 70, 3), ("q4k", 3072, 768, 4, 150, 2),
                                                      ("q4k", 256, 64, 5, 1, 2), ("q8_0", 256, 64, 2, 330, 2)])
def test_gate_up_swiglu_down(kind, n, ffs, nexp, ntok, topk):
    """gate|up -> SwiGLU -> down over jobs of 1 to 64 rows (ragged job sizes, row tiles past the matrix's last row, FF slice
    96; experts with one, two and six jobs: consecutive jobs of an expert are taken in pairs), each step against the
    oracle fed with the GPU's previous step."""
    from oracle import binding as O

    w = (cases.moe_weights if kind == "q4k" else cases.moe_weights_q8)(n=n, nexp=nexp, ffs=ffs, seed=32)
    jobs, P = cases.big_jobs(ntok, nexp, topk, seed=33)
    rng = np.random.default_rng(34)
    x16 = _f16_bits(rng.standard_normal((ntok, n)))
    ex, keep = _experts(w, "gu")
    gu = _run("fnx_moe_gate_up_mma", ex, jobs, x16, P)
    ref, mag = O.moe_mma(_weights16(w, "gu"), jobs, len(jobs), x16, 2 * ffs, P)
    _close(gu, ref, mag, n)

    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    dgu, h16 = G.dev(gu), torch.zeros((P, ffs), dtype=torch.int16, device="cuda")
    L.call("fnx_swiglu_h16", dgu.data_ptr(), ffs, P, h16.data_ptr(), L.stream())
    G.sync()
    h = G.host(h16, np.uint16)
    assert np.array_equal(h, O.swiglu_h16(gu, ffs)), "h = f16(silu(gate) * up)"

    dn_jobs = jobs.copy()
    for jb in dn_jobs:   # the down jobs read the pairs' h rows
        jb["y"][:jb["n"]] = jb["out"][:jb["n"]]
    ex, keep2 = _experts(w, "dn")
    part = _run("fnx_moe_down_mma", ex, dn_jobs, h, P)
    ref, mag = O.moe_mma(_weights16(w, "dn"), dn_jobs, len(dn_jobs), h, n, P)
    _close(part, ref, mag, ffs)
