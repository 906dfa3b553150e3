"""GPU parity of the position-split attention against the CPU oracle: prep + append bit-exact (norm, rotary, f16
rounding, placement), the exact-order scan and the merges bit-exact, for one GPU and for the partials of several."""
import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu


def _run(c, entry="fnx_attn_partial_exact", known_rows=False):
    """known_rows: the cache is handed over with its row count (FnxKvPages.cap), which lets the tensor-core scan fetch K/V
    by tensor loads; 70 rows of NaNs are put after the case's rows, inside the count, to stand for stale memory."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    T, nq, nkv, hd, ncard = c["T"], c["nq"], c["nkv"], c["hd"], c["ncard"]
    st = L.stream()
    pos0 = G.dev(np.array([c["pos0"]], np.int32))
    parts = G.zeros((ncard, T, nq, hd + 2))
    res = {"kc": [], "vc": []}
    for card in range(ncard):
        qg, k, v = G.dev(c["qg"]), G.dev(c["k"]), G.dev(c["v"])
        qn, kn = G.dev(c["qn"]), G.dev(c["kn"])
        hk, hv = c["kc"][card], c["vc"][card]
        if known_rows:
            stale = np.full((70,) + hk.shape[1:], 0x7E00, np.uint16)
            hk, hv = np.concatenate([hk, stale]), np.concatenate([hv, stale])
        kc, vc = G.dev(hk), G.dev(hv)
        g = L.KvPages(None, 0, 0, hk.shape[0] if known_rows else 0, 0)
        if c.get("q8_rows"):
            g = L.KvPages(None, 0, 0, c["q8_rows"], 1)
        L.call("fnx_attn_prep_append", qg.data_ptr(), k.data_ptr(), v.data_ptr(), qn.data_ptr(), kn.data_ptr(), kc.data_ptr(),
               vc.data_ptr(), g, card, ncard, T, pos0.data_ptr(), c["eps"], L.Rope(c["rope_base"], 64), nq, nkv, hd, st)
        scratch = G.zeros(L.load().fnx_attn_scratch_floats(nq, hd, T))
        L.call(entry, qg.data_ptr(), kc.data_ptr(), vc.data_ptr(), g, parts[card].data_ptr(), card, ncard, T,
               pos0.data_ptr(), nq, nkv, hd, scratch.data_ptr(), st)
        res["kc"].append(G.host(kc, np.uint16)[:c["kc"][card].shape[0]])
        res["vc"].append(G.host(vc, np.uint16)[:c["vc"][card].shape[0]])
        res["qg"], res["k"] = qg, k
    own = nq // ncard
    outs = [G.zeros((T, own, hd)) for _ in range(ncard)]
    for card in range(ncard):   # each GPU merges the partials for the heads it owns
        L.call("fnx_attn_finish", parts.data_ptr(), ncard, card, res["qg"].data_ptr(), outs[card].data_ptr(), T, nq, card * own, own, hd, st)
    G.sync()
    out = torch.cat(outs, dim=1)
    res["qg"], res["k"] = G.host(res["qg"]), G.host(res["k"])
    res["part"], res["out"] = G.host(parts), G.host(out)
    return res


@pytest.mark.parametrize("T,ctx,ncard,hd", [(16, 1000, 1, 256), (3, 5, 1, 256), (16, 2077, 2, 256), (5, 515, 4, 128), (1, 0, 1, 256)])
def test_attention_exact(T, ctx, ncard, hd):
    c = cases.attn_case(T=T, ctx=ctx, nq=8 if hd == 128 else 24, nkv=2 if hd == 128 else 4, hd=hd, ncard=ncard, seed=50 + T)
    ref = cases.attn_oracle(c)
    got = _run(c)
    assert np.array_equal(got["qg"].view(np.uint32), ref["qg"].view(np.uint32)), "q norm + rotary"
    assert np.array_equal(got["k"].view(np.uint32), ref["k"].view(np.uint32)), "k norm + rotary"
    for card in range(ncard):
        assert np.array_equal(got["kc"][card], ref["kc"][card]) and np.array_equal(got["vc"][card], ref["vc"][card]), "append"
        assert np.array_equal(got["part"][card].view(np.uint32), ref["part"][card].view(np.uint32)), "partials"
    assert np.array_equal(got["out"].view(np.uint32), ref["out"].view(np.uint32)), "merged, gated output"


@pytest.mark.parametrize("T,ctx,ncard,hd", [(16, 1000, 1, 256), (3, 5, 1, 256), (16, 2077, 2, 256), (5, 515, 4, 128), (1, 0, 1, 256)])
def test_attention_int8_kv(T, ctx, ncard, hd):
    """int8 K/V rows (reference kv_q8: groups of 32 with an f16 scale): the appended rows' bytes and scales, the partials of
    the exact-order scan over them and the merged output, bit for bit against the oracle; fnx_attn_partial hands an int8
    cache to the same scan."""
    c = cases.attn_case_q8(cases.attn_case(T=T, ctx=ctx, nq=8 if hd == 128 else 24, nkv=2 if hd == 128 else 4, hd=hd, ncard=ncard, seed=50 + T))
    ref = cases.attn_oracle(c)
    for entry in ("fnx_attn_partial_exact", "fnx_attn_partial"):
        got = _run(c, entry)
        for card in range(ncard):
            assert np.array_equal(got["kc"][card], ref["kc"][card]) and np.array_equal(got["vc"][card], ref["vc"][card]), "append"
            assert np.array_equal(got["part"][card].view(np.uint32), ref["part"][card].view(np.uint32)), "partials"
        assert np.array_equal(got["out"].view(np.uint32), ref["out"].view(np.uint32)), "merged, gated output"


@pytest.mark.parametrize("T,ctx,ncard,hd", [(16, 3000, 1, 256), (16, 70, 1, 256), (7, 1500, 2, 256), (5, 515, 4, 128), (1, 0, 1, 256),
                                            (16, 40000, 1, 256), (2, 262144, 1, 256), (3, 70000, 8, 256)])
@pytest.mark.parametrize("known_rows", [False, True])
def test_attention_fast_scan(T, ctx, ncard, hd, known_rows):
    """The one-pass tensor-core scan against the oracle: the same partial format and merge, values equal to f32 rounding
    (its sums run in another order; queries and weights enter the f16 MMAs as high + low halves).  Both ways of fetching
    K/V: a warp's asynchronous copies (row count unknown) and tensor loads (row count given, stale NaN rows after the
    newest position)."""
    c = cases.attn_case(T=T, ctx=ctx, nq=8 if hd == 128 else 24, nkv=2 if hd == 128 else 4, hd=hd, ncard=ncard, seed=60 + T)
    ref = cases.attn_oracle(c)
    got = _run(c, "fnx_attn_partial", known_rows)
    assert np.isfinite(got["out"]).all()
    err = np.abs(got["out"] - ref["out"])
    assert np.allclose(got["out"], ref["out"], rtol=3e-5, atol=2e-6), (err.max(), np.abs(ref["out"]).max())
    for card in range(ncard):   # the normalisers of the partials agree too
        zr, zg = ref["part"][card][..., hd + 1], got["part"][card][..., hd + 1]
        mr, mg = ref["part"][card][..., hd], got["part"][card][..., hd]
        assert np.allclose(zg * np.exp(mg - mr), zr, rtol=1e-4)


@pytest.mark.parametrize("T,ctx,ramp", [(16, 3000, 8.0), (16, 700, 20.0), (3, 5000, 12.0)])
@pytest.mark.parametrize("known_rows", [False, True])
def test_attention_fast_scan_rising_scores(T, ctx, ramp, known_rows):
    """Keys that grow along the cache: every row's largest score rises by far more than the scan's rescaling threshold
    between the first and the last chunk, so the accumulated output is rescaled several times on the way."""
    c = cases.attn_case(T=T, ctx=ctx, seed=90 + T, ramp=ramp)
    ref = cases.attn_oracle(c)
    got = _run(c, "fnx_attn_partial", known_rows)
    assert np.isfinite(got["out"]).all()
    assert (ref["part"][0][..., 256] > 16).all(), "the case does not reach the rescaling path"
    # scores reach 30 to 70 here, where one f32 rounding of a score moves its weight by 4e-6 relative: the bound is
    # stated against the largest output, 2e-5 of it
    err, top = np.abs(got["out"] - ref["out"]), np.abs(ref["out"]).max()
    assert err.max() <= 2e-5 * top, (err.max(), top)


def test_attention_rows_of_several_sequences():
    """A batched window: six rows of three sequences (2 + 1 + 3), each row at its lane's position on its lane's pages of one
    paged pool; every row's partial as the exact scan of that lane alone gives it."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    nq, nkv, hd, rpp = 24, 4, 256, 64   # local rows per page
    lanes = [(2, 300, 71), (1, 37, 72), (3, 1000, 73)]
    cs = [cases.attn_case(T=T, ctx=ctx, seed=seed) for T, ctx, seed in lanes]
    refs = [cases.attn_oracle(c) for c in cs]
    npages = [(r["kc"][0].shape[0] + rpp - 1) // rpp for r in refs]
    rng = np.random.default_rng(74)
    phys = rng.permutation(sum(npages) + 3)   # a few pages stay unused
    pool_k = np.zeros((len(phys), rpp, nkv, hd), np.uint16)
    pool_v = np.zeros_like(pool_k)
    pts, at = [], 0
    for r, n in zip(refs, npages):
        pt = phys[at:at + n].astype(np.int32)
        at += n
        for j, pg in enumerate(pt):
            rows = r["kc"][0][j * rpp:(j + 1) * rpp]
            pool_k[pg, :len(rows)], pool_v[pg, :len(rows)] = rows, r["vc"][0][j * rpp:(j + 1) * rpp]
        pts.append(G.dev(pt))
    kc, vc = G.dev(pool_k), G.dev(pool_v)
    qg = G.dev(np.concatenate([r["qg"] for r in refs]))
    T = sum(T for T, _, _ in lanes)
    pos = [G.dev(np.array([ctx + i], np.int32)) for (Tl, ctx, _) in lanes for i in range(Tl)]
    row_pt = [pts[l] for l, (Tl, _, _) in enumerate(lanes) for _ in range(Tl)]
    ppos = G.dev(np.array([t.data_ptr() for t in pos], np.uint64))
    ppt = G.dev(np.array([t.data_ptr() for t in row_pt], np.uint64))
    g = L.KvPages(None, rpp * nkv * hd, rpp, 0)
    part = G.zeros((T, nq, hd + 2))
    scratch = G.zeros(L.load().fnx_attn_scratch_floats(nq, hd, T))
    L.call("fnx_attn_part_lanes", qg.data_ptr(), kc.data_ptr(), vc.data_ptr(), g, L.LaneRows(ppos.data_ptr(), ppt.data_ptr()), part.data_ptr(),
           0, 1, T, nq, nkv, hd, scratch.data_ptr(), L.stream())
    G.sync()
    ref = np.concatenate([r["part"][0] for r in refs])
    assert np.array_equal(G.host(part).view(np.uint32), ref.view(np.uint32))


def test_attention_scan_timings(capsys):
    """Device times of the three scans of one layer at the benchmark's shape (T = 16, 24 / 4 heads of 256, 32 768 positions on
    one GPU): the tcgen05 scan over f16 rows, the exact-order scan over f16 rows and over int8 rows.  Printed; no bound
    beyond finishing."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    T, ctx, nq, nkv, hd = 16, 32768, 24, 4, 256
    rows = ctx + 64
    g = torch.Generator(device=G.DEV).manual_seed(3)
    qg = torch.randn((T, nq, 2 * hd), generator=g, device=G.DEV)
    kc = torch.randn((rows, nkv, hd), generator=g, device=G.DEV).half().view(torch.int16)
    vc = torch.randn((rows, nkv, hd), generator=g, device=G.DEV).half().view(torch.int16)
    halves = L.load().fnx_kvq_halves(rows, nkv, hd)
    kq = torch.randint(-127, 127, (halves,), generator=g, device=G.DEV, dtype=torch.int16)
    vq = torch.randint(-127, 127, (halves,), generator=g, device=G.DEV, dtype=torch.int16)
    kq[rows * nkv * hd // 2:] = 0x1C00   # the scales: f16 2^-8
    vq[rows * nkv * hd // 2:] = 0x1C00
    pos0 = G.dev(np.array([ctx], np.int32))
    part = G.zeros((T, nq, hd + 2))
    scratch = G.zeros(L.load().fnx_attn_scratch_floats(nq, hd, T))
    st = L.stream()
    out = []
    for name, entry, k, v, pages in (("tcgen05 scan, f16 rows", "fnx_attn_partial", kc, vc, L.KvPages(None, 0, 0, rows, 0)),
                                     ("exact-order scan, f16 rows", "fnx_attn_partial_exact", kc, vc, L.KvPages(None, 0, 0, rows, 0)),
                                     ("exact-order scan, int8 rows", "fnx_attn_partial_exact", kq, vq, L.KvPages(None, 0, 0, rows, 1))):
        def run():
            L.call(entry, qg.data_ptr(), k.data_ptr(), v.data_ptr(), pages, part.data_ptr(), 0, 1, T, pos0.data_ptr(), nq, nkv, hd, scratch.data_ptr(), st)
        for _ in range(2):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream())
        for _ in range(5):
            run()
        e1.record(torch.cuda.current_stream())
        G.sync()
        assert torch.isfinite(part).all()
        out.append("%s: %.1f us" % (name, e0.elapsed_time(e1) * 1e3 / 5))
    with capsys.disabled():
        print("\nattention scans at 32 768 positions: " + "; ".join(out))
