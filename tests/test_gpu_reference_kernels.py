"""The reference's own CUDA kernels, run here: its src/kernels.cu compiled unmodified for sm_100a (oracle/Makefile
`refgpu`, its own -O3 --use_fast_math flags, behind oracle/ref_kernels_shim.cu) beside this library's kernels and the
CPU oracle on the same seeded inputs, at the reference's compile-time shapes (hidden 2560, 512 experts top-10, FF 640 as
the slice of one card of two, 24 query / 2 KV heads of 256, 48 value heads).

What it pins: the oracle's statements of the router, the Q4_K gate|up, the split-Q8_0 dense product, the Gated DeltaNet
core, the attention scan, argmax and the top-64 against the reference's binary.  Integer results (picks, jobs, argmax, the
64 candidates, int8 activations up to the stated count of last-place ties) must be equal; floating-point results are held
to the reference's own fast-math slack, stated per check: the reference divides by approximation and takes __expf /
rsqrtf, this library and the oracle use IEEE operations in the same order.

The launchers that wait on a peer GPU or on a grid-wide barrier (ring_sum, the attention merge, hc_read) are not run.
The last test prints both sides' kernel times (CUDA events, same inputs)."""
import ctypes as C

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu
O = cases.O


@pytest.fixture(scope="module")
def ref():
    from oracle import refgpu

    if not refgpu.available():
        pytest.skip("oracle/_ref/libref_kernels.so is not built (make -C oracle -j8 refgpu REF=<reference tree>)")
    refgpu.load()
    return refgpu


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def _q4k_random(rng, nexp, rows, n):
    """Random Q4_K super-blocks with finite f16 d / dmin: [nexp][rows * n / 256 * 144] bytes."""
    b = rng.integers(0, 256, size=(nexp, rows * (n // 256), 144), dtype=np.uint8)
    d = (rng.random((nexp, rows * (n // 256))) * 2e-3 + 5e-4).astype(np.float16).view(np.uint16)
    dm = (rng.random((nexp, rows * (n // 256))) * 2e-3 + 5e-4).astype(np.float16).view(np.uint16)
    b[..., 0], b[..., 1] = d & 255, d >> 8
    b[..., 2], b[..., 3] = dm & 255, dm >> 8
    return b.reshape(nexp, -1)


def _moe_case(sh, seed=61, nexp=None):
    rng = np.random.default_rng(seed)
    n, nexp, ffs = sh["N"], nexp or sh["NEXP"], sh["FF"] // sh["NCARD"]
    W = (rng.standard_normal((sh["NEXP"] + 1, n)) * 0.02).astype(np.float32)
    x = rng.standard_normal((16, n)).astype(np.float32)
    return W, x, _q4k_random(rng, nexp, 2 * ffs, n), ffs


def test_shapes_are_the_reference_models(ref):
    sh = ref.shapes()
    assert (sh["N"], sh["NEXP"], sh["TOPK"], sh["FF"], sh["NQH"], sh["NKVH"], sh["HD"], sh["MAXT"]) == (2560, 512, 10, 640, 24, 2, 256, 16), sh


def test_quantize_router_and_gate_up(ref):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    sh = ref.shapes()
    n, nexp, topk, T = sh["N"], sh["NEXP"], sh["TOPK"], 16
    W, x, gu_w, ffs = _moe_case(sh)
    st = L.stream()
    dW, dx = G.dev(W), G.dev(x)
    # ---- q8_1: the reference divides by approximation, so a value within an ulp of a rounding boundary may land on the
    # other side: at most 1 in 1000 int8 values off by one, every f16 scale within one f16 ulp
    xq_o = O.quantize_q8_1(x)
    xq_r = G.zeros(T * (n // 32) * 36, torch.uint8)
    ref.call("ref_quantize_q8_1", dx.data_ptr(), xq_r.data_ptr(), n, T, st)
    G.sync()
    a, b = G.host(xq_r).reshape(T, n // 32, 36), xq_o.reshape(T, n // 32, 36)
    dq = np.abs(a[..., 4:].view(np.int8).astype(int) - b[..., 4:].view(np.int8).astype(int))
    assert dq.max() <= 1 and (dq != 0).mean() <= 1e-3, (dq.max(), (dq != 0).mean())
    da, db = a[..., :2].copy().view(np.float16).astype(np.float64), b[..., :2].copy().view(np.float16).astype(np.float64)
    assert np.all(np.abs(da - db) <= np.abs(db) * 2.0 ** -10)
    # ---- router: picks, weights and jobs of the reference's kernel = the oracle's (logits to 1e-5 of the row's largest:
    # the compiler may fuse the reference's chunk sums differently)
    r_logits, r_topi, r_topw, r_jgu, r_jdn, r_nj = O.router_route(W, x, topk)
    P = T * topk
    logits, topi, topw = G.zeros((T, nexp + 1)), G.zeros((T, topk), torch.int32), G.zeros((T, topk))
    jgu, jdn, njobs = G.zeros(P * 136, torch.uint8), G.zeros(P * 136, torch.uint8), G.zeros(2, torch.int32)
    ref.call("ref_router_route", dW.data_ptr(), dx.data_ptr(), logits.data_ptr(), T, topi.data_ptr(), topw.data_ptr(), jgu.data_ptr(), jdn.data_ptr(),
             njobs.data_ptr(), st)
    G.sync()
    lg = G.host(logits)
    assert np.allclose(lg, r_logits, rtol=0, atol=1e-5 * np.abs(r_logits).max())
    assert np.array_equal(G.host(topi), r_topi), "the reference's picks differ from the oracle's"
    assert np.allclose(G.host(topw), r_topw, rtol=1e-5, atol=1e-7)
    assert int(G.host(njobs)[0]) == r_nj
    got = G.host(jgu).view(O.JOB_DTYPE)
    assert np.array_equal(got["w"][:r_nj], r_jgu["w"][:r_nj]) and np.array_equal(got["n"][:r_nj], r_jgu["n"][:r_nj])
    for j in range(r_nj):   # a job's rows: the reference fills them in atomic order, the oracle in pair order: the same set
        k = r_jgu["n"][j]
        assert sorted(got["out"][j][:k].tolist()) == sorted(r_jgu["out"][j][:k].tolist())
    # ---- Q4_K gate|up over the oracle's jobs and q8_1 rows: reference vs oracle to 2e-6 of the row's magnitude; this
    # library = the oracle bit for bit
    gu_o = O.moe_gate_up_q4k(gu_w, gu_w.shape[1], r_jgu, r_nj, xq_o, n, 2 * ffs, P)
    dgw, dj, dn, dxq = G.dev(gu_w), G.dev(r_jgu.view(np.uint8).reshape(-1)), G.dev(np.array([r_nj, 0], np.int32)), G.dev(xq_o)
    gu_r, gu_m = G.zeros((P, 2 * ffs)), G.zeros((P, 2 * ffs))
    ref.call("ref_moe_gate_up_q4k", dgw.data_ptr(), gu_w.shape[1], 2 * ffs, n, dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), gu_r.data_ptr(), st)
    ex = L.Experts(L.Q4_K, 2 * ffs, n, dgw.data_ptr(), None, None, None, gu_w.shape[1], 0)
    L.call("fnx_moe_gate_up", C.byref(ex), dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), gu_m.data_ptr(), st)
    G.sync()
    assert np.array_equal(_bits(G.host(gu_m)), _bits(gu_o)), "this library's gate|up differs from the oracle"
    scale = np.abs(gu_o).max()
    assert np.allclose(G.host(gu_r), gu_o, rtol=0, atol=2e-6 * scale), float(np.abs(G.host(gu_r) - gu_o).max() / scale)


def test_dense_q8_0_product_bit_equal(ref):
    """The split-Q8_0 row dot has no division and no transcendental: the reference's kernel, this library's and the
    oracle give the same bits."""
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    sh = ref.shapes()
    rng = np.random.default_rng(62)
    rows, cols = 4100, sh["N"]
    wq = rng.integers(-127, 128, size=(rows, cols), dtype=np.int8)
    wd = (rng.random((rows, cols // 32), dtype=np.float32) * 2e-4 + 1e-4).astype(np.float16).view(np.uint16)
    for T in (1, 5, 16):
        yq = O.quantize_q8_1(rng.standard_normal((T, cols)).astype(np.float32))
        want = O.q8s_gemv(wq, wd, yq, T)
        w, keep = G.q8s((wq, wd))
        dy, out_r, out_m = G.dev(yq), G.zeros((T, rows)), G.zeros((T, rows))
        ref.call("ref_q8s_gemv", keep[0].data_ptr(), keep[1].data_ptr(), rows, cols, dy.data_ptr(), out_r.data_ptr(), rows, T, L.stream())
        L.call("fnx_q8s_gemv", w, rows, cols, dy.data_ptr(), out_m.data_ptr(), rows, T, L.stream())
        G.sync()
        assert np.array_equal(_bits(G.host(out_m)), _bits(want))
        assert np.array_equal(_bits(G.host(out_r)), _bits(want)), "the reference's dense kernel differs from the oracle (T = %d)" % T


def test_gdn_core(ref):
    """One card's Gated DeltaNet heads over a 16-row window: the reference's kernel against the oracle.  Its decay,
    sigmoid and norms go through __expf / rsqrtf: state, checkpoints and outputs to 2e-5 of their largest value, the
    quantised output rows within one step."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    sh = ref.shapes()
    nv, nk = sh["NVH"] // sh["NCARD"], sh["NKH"] // sh["NCARD"]
    c = cases.gdn_case(T=16, nk=nk, nv=nv, seed=63)
    want, mine = cases.gdn_oracle(c), G.run_gdn(c)
    assert np.array_equal(_bits(mine["S"]), _bits(want["S"])) and np.array_equal(mine["yq"], want["yq"])
    t = {k: G.dev(c[k]) for k in ("qkvz", "ab", "hist", "convw", "dt", "a", "nw", "S", "vmap", "ctl")}
    T, ch = 16, c["ch"]
    yq, y32 = G.zeros(T * (nv * 128 // 32) * 36, torch.uint8), G.zeros((T, nv * 128))
    scratch = G.zeros(ref.load().ref_gdn_scratch_floats(nv))
    snap, hsnap = G.zeros((T - 1, nv, 128, 128)), G.zeros((16, 3, ch))
    ref.call("ref_gdn_core", t["qkvz"].data_ptr(), t["ab"].data_ptr(), t["hist"].data_ptr(), t["convw"].data_ptr(), t["dt"].data_ptr(),
             t["a"].data_ptr(), t["nw"].data_ptr(), t["S"].data_ptr(), yq.data_ptr(), t["ctl"].data_ptr(), scratch.data_ptr(), snap.data_ptr(),
             hsnap.data_ptr(), nk, nv, t["vmap"].data_ptr(), T, c["eps"], L.stream(), y32.data_ptr())
    G.sync()
    for name, got, exp in (("S", G.host(t["S"]), want["S"]), ("snap", G.host(snap), want["snap"]), ("y32", G.host(y32), want["y32"])):
        assert np.allclose(got, exp, rtol=0, atol=2e-5 * np.abs(exp).max()), (name, float(np.abs(got - exp).max() / np.abs(exp).max()))
    assert np.array_equal(G.host(hsnap)[:T - 1], want["hsnap"][:T - 1]), "conv history checkpoints are copies: equal"
    assert np.array_equal(G.host(t["hist"]), want["hist"])
    a, b = G.host(yq).reshape(T, -1, 36), want["yq"].reshape(T, -1, 36)
    dq = np.abs(a[..., 4:].view(np.int8).astype(int) - b[..., 4:].view(np.int8).astype(int))
    assert dq.max() <= 1 and (dq != 0).mean() <= 0.02, (dq.max(), (dq != 0).mean())


def test_attention_scan_runs(ref):
    """The reference's scan (k_attn_part through attn_part_lanes: card 0 of 2, paged f16 K/V) against this library's scan
    in the same order of sums, run by run: accumulators to 1e-4 of the run's largest, maxima to 1e-5, normalisers to 1e-4
    (the reference's __expf)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    sh = ref.shapes()
    nq, nkv, hd, ncard, T, rpp = sh["NQH"], sh["NKVH"], sh["HD"], sh["NCARD"], 16, 64
    c = cases.attn_case(T=T, ctx=6001, nq=nq, nkv=nkv, hd=hd, ncard=ncard, seed=64)
    r = cases.attn_oracle(c)
    rows = (r["kc"][0].shape[0] + rpp - 1) // rpp * rpp
    kc, vc = np.zeros((rows, nkv, hd), np.uint16), np.zeros((rows, nkv, hd), np.uint16)
    kc[:r["kc"][0].shape[0]], vc[:r["vc"][0].shape[0]] = r["kc"][0], r["vc"][0]
    dq, dkc, dvc = G.dev(r["qg"]), G.dev(kc), G.dev(vc)
    pt = torch.arange(rows // rpp, dtype=torch.int32, device=G.DEV)
    pos = torch.tensor([c["pos0"] + t for t in range(T)], dtype=torch.int32, device=G.DEV)
    pos_p = torch.tensor([pos[t:t + 1].data_ptr() for t in range(T)], dtype=torch.int64, device=G.DEV)
    pt_p = torch.tensor([pt.data_ptr()] * T, dtype=torch.int64, device=G.DEV)
    page = rpp * nkv * hd
    sc_r = G.zeros(ref.load().ref_attn_scratch_floats())
    ref.call("ref_attn_part_lanes", dq.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), page, rpp, pos_p.data_ptr(), pt_p.data_ptr(), T, sc_r.data_ptr(), 0,
             L.stream())
    sc_m, part = G.zeros(L.load().fnx_attn_scratch_floats(nq, hd, T)), G.zeros((T, nq, hd + 2))
    L.call("fnx_attn_part_lanes", dq.data_ptr(), dkc.data_ptr(), dvc.data_ptr(), L.KvPages(None, page, rpp, 0), L.LaneRows(pos_p.data_ptr(), pt_p.data_ptr()),
           part.data_ptr(), 0, ncard, T, nq, nkv, hd, sc_m.data_ptr(), L.stream())
    G.sync()
    assert np.array_equal(_bits(G.host(part)), _bits(r["part"][0])), "this library's scan differs from the oracle"
    nacc = T * nq * 16 * hd
    acc_r, acc_m = G.host(sc_r)[:nacc].reshape(T, nq, 16, hd), G.host(sc_m)[:nacc].reshape(T, nq, 16, hd)
    off = ref.load().ref_attn_mz_offset()
    mz_r, mz_m = G.host(sc_r)[off:off + T * nq * 32].reshape(T, nq, 16, 2), G.host(sc_m)[nacc:nacc + T * nq * 32].reshape(T, nq, 16, 2)
    assert np.array_equal(np.isinf(mz_r[..., 0]), np.isinf(mz_m[..., 0]))
    live = ~np.isinf(mz_m[..., 0])
    assert live.all(), "every run holds positions at this context"
    assert np.allclose(mz_r[..., 0], mz_m[..., 0], rtol=0, atol=1e-5 * np.abs(mz_m[..., 0]).max())
    assert np.allclose(mz_r[..., 1], mz_m[..., 1], rtol=1e-4)
    assert np.allclose(acc_r, acc_m, rtol=0, atol=1e-4 * np.abs(acc_m).max()), float(np.abs(acc_r - acc_m).max() / np.abs(acc_m).max())


def test_argmax_and_top64_equal(ref):
    """Compare-and-select only: the reference's kernels, this library's and the oracle agree on every tie scenario of the
    reference's own top-64 test (tools/topk_test.cu:110-163)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G
    from tests.test_oracle_path import _tie_cases, pack_pens

    for name, rows, pens, v0 in _tie_cases():
        logits = np.stack(rows)
        T, n = logits.shape
        tok, cnt, pn, par = pack_pens(pens)
        want_l = logits.copy()
        wv, wi, _ = O.top_tokens(want_l, v0, tok, cnt, pn, par)
        av, ai, _ = O.argmax(logits, v0)
        for side in ("ref", "ours"):
            dl, err = G.dev(logits), G.zeros(1, torch.int32)
            keys, bv, bi = G.zeros(32, torch.int64), G.zeros(T), G.zeros(T, torch.int32)
            ov, oi = G.zeros((T, 64)), G.zeros((T, 64), torch.int32)
            dt, dc, dn, dp = G.dev(tok), G.dev(cnt), G.dev(pn), G.dev(par)
            a1 = (dl.data_ptr(), n, T, v0, bv.data_ptr(), bi.data_ptr(), keys.data_ptr(), err.data_ptr(), L.stream())
            a2 = (dl.data_ptr(), n, T, v0, dt.data_ptr(), dc.data_ptr(), dn.data_ptr(), tok.shape[1], dp.data_ptr(), ov.data_ptr(), oi.data_ptr(),
                  err.data_ptr(), L.stream())
            if side == "ref":
                ref.call("ref_argmax", *a1)
                ref.call("ref_top_tokens", *a2)
            else:
                L.call("fnx_argmax", *a1)
                L.call("fnx_top_tokens", *a2)
            G.sync()
            assert np.array_equal(G.host(bi), ai) and np.array_equal(_bits(G.host(bv)), _bits(av)), (side, name)
            assert np.array_equal(G.host(oi), wi) and np.array_equal(_bits(G.host(ov)), _bits(wv)), (side, name)
            assert np.array_equal(_bits(G.host(dl)), _bits(want_l)), (side, name)


def test_kernel_times_side_by_side(ref, capsys):
    """Both sides' kernels on the same inputs, CUDA events, median of 20 launches after 3 (weights larger than L2 where the
    kernel streams weights).  Printed, not asserted: a same-GPU anchor for this library's kernels."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    sh = ref.shapes()
    n, nexp, topk, T = sh["N"], sh["NEXP"], sh["TOPK"], 16
    W, x, gu_w, ffs = _moe_case(sh, seed=65)
    st = L.stream()
    P = T * topk
    dW, dx = G.dev(W), G.dev(x)
    xq = O.quantize_q8_1(x)
    _, _, _, jgu, _, nj = O.router_route(W, x, topk)
    dgw, dj, dn, dxq = G.dev(gu_w), G.dev(jgu.view(np.uint8).reshape(-1)), G.dev(np.array([nj, 0], np.int32)), G.dev(xq)
    out = G.zeros((P, 2 * ffs))
    logits, topi, topw = G.zeros((T, nexp + 1)), G.zeros((T, topk), torch.int32), G.zeros((T, topk))
    j1, j2, njb, rs = G.zeros(P * 136, torch.uint8), G.zeros(P * 136, torch.uint8), G.zeros(2, torch.int32), G.zeros(16, torch.uint8)
    ex = L.Experts(L.Q4_K, 2 * ffs, n, dgw.data_ptr(), None, None, None, gu_w.shape[1], 0)
    rng = np.random.default_rng(66)
    rows = 65536
    wq = torch.randint(-127, 128, (rows, n), dtype=torch.int8, device=G.DEV)
    wd = torch.full((rows, n // 32), 0.0002, dtype=torch.float16, device=G.DEV).view(torch.int16)
    dout = G.zeros((T, rows))
    nv, nk = sh["NVH"] // sh["NCARD"], sh["NKH"] // sh["NCARD"]
    c = cases.gdn_case(T=16, nk=nk, nv=nv, seed=67)
    g = {k: G.dev(c[k]) for k in ("qkvz", "ab", "hist", "convw", "dt", "a", "nw", "S", "vmap", "ctl")}
    yq, snap, hsnap = G.zeros(T * (nv * 4) * 36, torch.uint8), G.zeros((T - 1, nv, 128, 128)), G.zeros((16, 3, c["ch"]))
    sc_r, sc_m = G.zeros(ref.load().ref_gdn_scratch_floats(nv)), G.zeros(L.load().fnx_gdn_scratch_floats(nv))
    gargs = lambda sc: (g["qkvz"].data_ptr(), g["ab"].data_ptr(), g["hist"].data_ptr(), g["convw"].data_ptr(), g["dt"].data_ptr(), g["a"].data_ptr(),   # noqa: E731
                        g["nw"].data_ptr(), g["S"].data_ptr(), yq.data_ptr(), g["ctl"].data_ptr(), sc.data_ptr(), snap.data_ptr(), hsnap.data_ptr(), nk, nv,
                        g["vmap"].data_ptr(), T, c["eps"], st, None)
    lg = G.dev((rng.standard_normal((T, 75968)) * 3).astype(np.float32))
    ov, oi, err = G.zeros((T, 64)), G.zeros((T, 64), torch.int32), G.zeros(1, torch.int32)
    ptk, pn, pp = G.zeros((T, 1), torch.int32), G.zeros(T, torch.int32), G.dev(np.tile(np.array([1, 0, 0], np.float32), (T, 1)))
    targs = (lg.data_ptr(), 75968, T, 0, ptk.data_ptr(), ptk.data_ptr(), pn.data_ptr(), 1, pp.data_ptr(), ov.data_ptr(), oi.data_ptr(), err.data_ptr(), st)   # no penalties: zero counts

    def med(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(20):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return sorted(ts)[10]

    rowsout = []
    rowsout.append(("router_route (513 x %d, T 16)" % n,
                    med(lambda: ref.call("ref_router_route", dW.data_ptr(), dx.data_ptr(), logits.data_ptr(), T, topi.data_ptr(), topw.data_ptr(),
                                         j1.data_ptr(), j2.data_ptr(), njb.data_ptr(), st)),
                    med(lambda: L.call("fnx_router_route", dW.data_ptr(), dx.data_ptr(), logits.data_ptr(), T, n, nexp, topk, topi.data_ptr(),
                                       topw.data_ptr(), j1.data_ptr(), j2.data_ptr(), njb.data_ptr(), rs.data_ptr(), st))))
    rowsout.append(("moe gate|up Q4_K (%d jobs, 640 x %d each)" % (nj, n),
                    med(lambda: ref.call("ref_moe_gate_up_q4k", dgw.data_ptr(), gu_w.shape[1], 2 * ffs, n, dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(),
                                         out.data_ptr(), st)),
                    med(lambda: L.call("fnx_moe_gate_up", C.byref(ex), dj.data_ptr(), dn.data_ptr(), P, dxq.data_ptr(), out.data_ptr(), st))))
    rowsout.append(("dense Q8_0 (%d x %d, T 16)" % (rows, n),
                    med(lambda: ref.call("ref_q8s_gemv", wq.data_ptr(), wd.data_ptr(), rows, n, dxq.data_ptr(), dout.data_ptr(), rows, T, st)),
                    med(lambda: L.call("fnx_q8s_gemv", L.Q8S(wq.data_ptr(), wd.data_ptr()), rows, n, dxq.data_ptr(), dout.data_ptr(), rows, T, st))))
    rowsout.append(("gdn_core (%d value heads, T 16)" % nv, med(lambda: ref.call("ref_gdn_core", *gargs(sc_r))), med(lambda: L.call("fnx_gdn_core", *gargs(sc_m)))))
    rowsout.append(("top-64 (16 x 75968)", med(lambda: ref.call("ref_top_tokens", *targs)), med(lambda: L.call("fnx_top_tokens", *targs))))
    with capsys.disabled():
        print("\nkernel | reference's kernel on this GPU (us) | this library (us) | ratio")
        for name, a, b in rowsout:
            print("%s | %.1f | %.1f | %.2fx" % (name, a, b, a / b))
