"""The oracle's algorithms pinned without a GPU against independent statements: the routing against a sort-based
restatement (as the reference's host routing, tools/kbench.cu:59-96), the top-64 against a full sort on the
reference's own adversarial tie cases (tools/topk_test.cu:110-163), the ring's addition order against the analytic
all-reduce (tools/s27_ring_test.cu:131-168), acceptance against the reference's own object code (fixture), and
size-independent properties of the DeltaNet rollback and the position-split attention."""
import os

import numpy as np

from tests import cases

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_routing_indices_weights_jobs(oracle):
    rng = np.random.default_rng(5)
    T, n, nexp, topk = 16, 512, 64, 10
    W = (rng.standard_normal((nexp + 1, n)) * 0.02).astype(np.float32)
    x = rng.standard_normal((T, n)).astype(np.float32)
    W[7] = W[3]   # exact logit ties: the lower index must win
    logits, topi, topw, gu, dn, nj = oracle.router_route(W, x, topk)
    assert np.allclose(logits, x @ W.T, rtol=1e-4, atol=1e-5)
    for t in range(T):
        order = sorted(range(nexp), key=lambda i: (-logits[t, i], i))[:topk]
        assert topi[t].tolist() == order
        e = np.exp(logits[t, order].astype(np.float64) - logits[t, order[0]])
        assert np.allclose(topw[t], e / e.sum(), rtol=1e-6)
    # jobs: distinct experts in first-pick order, rows in pair order, every pair exactly once
    flat = topi.reshape(-1).tolist()
    first_order = list(dict.fromkeys(flat))
    assert nj == len(first_order)
    assert [int(j["w"]) for j in gu[:nj]] == first_order
    seen = []
    for j in gu[:nj]:
        pairs = j["out"][: j["n"]].tolist()
        assert pairs == sorted(pairs) and all(flat[p] == j["w"] for p in pairs)
        assert j["y"][: j["n"]].tolist() == [p // topk for p in pairs]
        seen += pairs
    assert sorted(seen) == list(range(T * topk))
    assert np.array_equal(gu["out"], dn["out"]) and np.array_equal(dn["y"], dn["out"])


def _topk_ref(row, v0):
    idx = np.lexsort((np.arange(row.size), -row.astype(np.float64)))[:64]
    return row[idx], idx + v0


def _tie_cases():
    N, V0 = 82944, 82944
    rng = np.random.default_rng(7)
    none = ([], [], (1.0, 0.0, 0.0))
    rnd = lambda: (rng.standard_normal(N) * 3).astype(np.float32)  # noqa: E731
    yield "random", [rnd(), rnd(), rnd()], [none] * 3, V0
    yield "all equal", [np.full(N, 1.5, np.float32)], [none], V0
    yield "all zero", [np.zeros(N, np.float32)], [none], V0
    r = np.full(N, -5.0, np.float32)
    r[[k * 7919 % N for k in range(10)]] = 9.0 + np.arange(10)
    r[[(k * 104729 + 13) % N for k in range(300)]] = 2.0
    yield "300 tied at the threshold", [r], [none], V0
    r = np.full(N, -1.0, np.float32)
    r[[(k * 31 + 5) % N for k in range(5000)]] = 0.25
    r[[(k * 1299709 + 3) % N for k in range(63)]] = 4.0 + 0.01 * np.arange(63, dtype=np.float32)
    yield "63 above, 5000 tied", [r], [none], V0
    r = np.full(N, -2.0, np.float32)
    for c in range(40):
        r[1024 * (c + 1) - 4: 1024 * (c + 1) + 4] = 1.0
    yield "ties straddling chunks", [r], [none], V0
    r = np.full(N, -3.0, np.float32)
    r[[k * 97 for k in range(400)]] = 3.0
    r[[k * 97 + 50 for k in range(300)]] = 2.0
    yield "penalties making a wide tie", [r], [([V0 + k * 97 for k in range(400)], [1] * 400, (1.0, 0.0, 1.0))], V0
    yield "mixed rows", [rnd(), np.full(N, 7.0, np.float32), rnd()], [none] * 3, V0


def pack_pens(pens):
    stride = max(1, max(len(p[0]) for p in pens))
    T = len(pens)
    tok = np.zeros((T, stride), np.int32)
    cnt = np.zeros((T, stride), np.int32)
    n = np.zeros(T, np.int32)
    par = np.zeros((T, 3), np.float32)
    for t, (tk, ct, pr) in enumerate(pens):
        tok[t, : len(tk)] = tk
        cnt[t, : len(ct)] = ct
        n[t] = len(tk)
        par[t] = pr
    return tok, cnt, n, par


def apply_pens(row, v0, pen):
    row = row.copy()
    tk, ct, (rep, fr, pr) = pen
    for t, c in zip(tk, ct):
        j = t - v0
        if 0 <= j < row.size and c > 0:
            l = row[j]
            l = np.float32(l * np.float32(rep)) if l <= 0 else np.float32(l / np.float32(rep))
            row[j] = np.float32(np.float32(l - np.float32(np.float32(c) * np.float32(fr))) - np.float32(pr))
    return row


def test_top64_exact_on_tie_cases(oracle):
    for name, rows, pens, v0 in _tie_cases():
        logits = np.stack(rows)
        tok, cnt, n, par = pack_pens(pens)
        ov, oi, err = oracle.top_tokens(logits.copy(), v0, tok, cnt, n, par)
        assert err == 0
        for t, row in enumerate(rows):
            rv, ri = _topk_ref(apply_pens(row, v0, pens[t]), v0)
            assert np.array_equal(ov[t], rv) and np.array_equal(oi[t], ri), name


def test_argmax_ties_and_merge(oracle):
    rng = np.random.default_rng(8)
    logits = rng.standard_normal((4, 1000)).astype(np.float32)
    logits[1, [17, 400]] = 9.0
    logits[2] = -0.0
    bv, bi, err = oracle.argmax(logits, v0=100)
    assert err == 0 and bi.tolist() == [int(np.argmax(logits[0])) + 100, 117, 100, int(np.argmax(logits[3])) + 100]
    logits[3, 5] = np.inf
    assert oracle.argmax(logits)[2] == 16
    # slices: the lower slice wins a tie
    v = np.array([[1.0, 3.0], [1.0, 3.0], [0.5, 2.0]], np.float32)
    i = np.array([[10, 11], [20, 21], [30, 31]], np.int32)
    assert oracle.argmax_merge(v, i).tolist() == [10, 11]


def test_ring_order_analytic(oracle):
    """x_c = (c + 1)(i % 97 + t) / 64 summed over n ranks is n(n+1)/2 x exactly in fp32 (tools/s27_ring_test.cu)."""
    for n in (2, 3, 4, 8):
        T, N = 5, 3072
        i = np.arange(N, dtype=np.float32)[None, :] % 97 + np.arange(T, dtype=np.float32)[:, None]
        xs = [((c + 1) * i / 64).astype(np.float32) for c in range(n)]
        out = oracle.ring_sum(xs)
        assert np.array_equal(out, (n * (n + 1) / 2 * i / 64).astype(np.float32))
    # the order itself: chunk c starts at rank c
    rng = np.random.default_rng(9)
    xs = [rng.standard_normal((2, 64)).astype(np.float32) for _ in range(4)]
    out = oracle.ring_sum(xs)
    for c in range(4):
        sl = slice(2 * (c * 32 // 4), 2 * ((c + 1) * 32 // 4))
        exp = xs[c][:, sl]
        for s in range(1, 4):
            exp = exp + xs[(c + s) % 4][:, sl]
        assert np.array_equal(out[:, sl], exp)


def test_acceptance_matches_reference_fixture(oracle):
    g = np.load(os.path.join(GOLD, "accept.npz"))
    rng = oracle.mt_new(int(g["unif_seed"]))
    assert np.array_equal(np.array([oracle.mt_unif(rng) for _ in range(4096)]), g["unif"])
    for c in range(g["rows"].shape[0]):
        temp, top_p, min_p, top_k = g["samp"][c]
        kw = dict(temperature=float(temp), top_p=float(top_p), min_p=float(min_p), top_k=int(top_k))
        for t in range(16):
            ids, p = oracle.make_dist(g["cand_v"][c, t], g["cand_i"][c, t], **kw)
            n = g["dist_n"][c, t]
            assert len(ids) == n and np.array_equal(ids, g["dist_ids"][c, t, :n]) and np.array_equal(p, g["dist_p"][c, t, :n])
        n, toks = oracle.accept_sampled(g["rows"][c], g["cand_v"][c], g["cand_i"][c], oracle.mt_new(int(g["seeds"][c])), **kw)
        assert n == g["n_out"][c] and np.array_equal(toks, g["toks"][c, :n])
    assert len(set(g["n_out"].tolist())) > 3   # the fixture covers early, middle and full acceptance


def test_greedy_acceptance(oracle):
    assert oracle.accept_greedy([5, 1, 2, 3], [1, 2, 9, 4]) == 3
    assert oracle.accept_greedy([5, 1, 2, 3], [7, 2, 3, 4]) == 1
    assert oracle.accept_greedy([5, 1, 2, 3], [1, 2, 3, 4]) == 4
    assert oracle.accept_greedy([5], [1]) == 1


def test_gdn_window_splits_and_rollback(oracle):
    """A window of T rows leaves the state and outputs of two windows of n and T - n rows (each row's arithmetic does
    not depend on the window it is in), and rolling back to n rows restores exactly the state and conv history that a
    window of n rows leaves."""
    T, n = 6, 4
    c = cases.gdn_case(T, nk=2, nv=4, seed=11)
    full = cases.gdn_oracle(c)
    a = dict(c, qkvz=c["qkvz"][:n].copy(), ab=c["ab"][:n].copy(), T=n)
    ra = cases.gdn_oracle(a)
    assert np.array_equal(ra["yq"], full["yq"][:n]) and np.array_equal(ra["S"], full["snap"][n - 1])
    b = dict(c, qkvz=c["qkvz"][n:].copy(), ab=c["ab"][n:].copy(), T=T - n, S=ra["S"], hist=ra["hist"], ctl=np.array([1004, 6], np.int32))
    rb = cases.gdn_oracle(b)
    assert np.array_equal(rb["yq"], full["yq"][n:]) and np.array_equal(rb["S"], full["S"])
    S, hist = full["S"].copy(), full["hist"].copy()
    oracle.gdn_rollback(S, hist, full["snap"], full["hsnap"], c["ctl"], 2, 4, T, n)
    assert np.array_equal(S, ra["S"]) and np.array_equal(hist[0], ra["hist"][0])   # parity 1 read, half 0 written
    # against a plain float64 statement of the delta rule for one head and row
    k = full  # noqa: F841


def test_gdn_against_float64_recurrence(oracle):
    T, nk, nv = 3, 1, 2
    c = cases.gdn_case(T, nk, nv, seed=12)
    r = cases.gdn_oracle(c)
    ch = c["ch"]
    hin = c["hist"][1].astype(np.float64)
    seq = np.concatenate([hin, c["qkvz"][:, :ch].astype(np.float64)])
    conv = np.stack([(seq[t:t + 4] * c["convw"].T.astype(np.float64)).sum(0) for t in range(T)])
    conv = conv / (1 + np.exp(-conv))
    S = c["S"].astype(np.float64).copy()
    for lv in range(nv):
        for t in range(T):
            q, k = conv[t, :128], conv[t, 128:256]
            q, k = q / np.sqrt((q * q).sum() + 1e-6), k / np.sqrt((k * k).sum() + 1e-6)
            v = conv[t, 256 + lv * 128: 256 + (lv + 1) * 128]
            g = np.exp(-np.log1p(np.exp(float(c["ab"][t, lv]))))
            beta = 1 / (1 + np.exp(-float(c["ab"][t, nv + lv])))
            kv = S[lv].T @ k
            delta = (v - g * kv) * beta
            S[lv] = g * S[lv] + np.outer(k, delta)
            o = S[lv].T @ q / np.sqrt(128)
            z = c["qkvz"][t, ch + lv * 128: ch + (lv + 1) * 128].astype(np.float64)
            y = o / np.sqrt((o * o).mean() + 1e-6) * c["nw"] / (1 + np.exp(-z))
            assert np.allclose(r["y32"][t, lv * 128:(lv + 1) * 128], y, rtol=2e-4, atol=2e-5)
    assert np.allclose(r["S"], S, rtol=1e-4, atol=1e-5)


def test_attention_position_split_matches_single(oracle):
    """The merge of the per-GPU partials equals one GPU's attention over all positions (to rounding), and both equal a
    float64 softmax attention; appended K/V rows land where the placement rule says."""
    base = cases.attn_case(T=3, ctx=203, nq=4, nkv=2, hd=128, ncard=1, seed=13)
    one = cases.attn_oracle(base)
    for ncard in (2, 4):
        c = cases.attn_case(T=3, ctx=203, nq=4, nkv=2, hd=128, ncard=ncard, seed=13)
        r = cases.attn_oracle(c)
        assert np.allclose(r["out"], one["out"], rtol=2e-4, atol=2e-5)
        for card in range(ncard):
            for t in range(3):
                p = 203 + t
                if (p // 4) % ncard == card:
                    row = (p // 4 // ncard) * 4 + p % 4
                    assert np.array_equal(r["kc"][card][row].view(np.float16), r["k"][t].astype(np.float16))
    qg, kc, vc = one["qg"].astype(np.float64), one["kc"][0].view(np.float16).astype(np.float64), one["vc"][0].view(np.float16).astype(np.float64)
    for t in range(3):
        for h in range(4):
            L = 203 + t + 1
            s = kc[:L, h // 2] @ qg[t, h, :128] / np.sqrt(128)
            w = np.exp(s - s.max())
            o = (w[:, None] * vc[:L, h // 2]).sum(0) / w.sum() / (1 + np.exp(-qg[t, h, 128:]))
            assert np.allclose(one["out"][t, h], o, rtol=2e-4, atol=2e-5)


def test_attention_int8_kv(oracle):
    """int8 K/V rows (reference kv_q8): the oracle's append writes the bytes numpy's statement of the quantiser gives, the
    scan over them equals a float64 softmax attention over the values the cache holds, and its result stays within the
    quantisation error of the f16 cache's."""
    T, ctx, nq, nkv, hd = 3, 203, 4, 2, 128
    for ncard in (1, 2):
        c16 = cases.attn_case(T=T, ctx=ctx, nq=nq, nkv=nkv, hd=hd, ncard=ncard, seed=13)
        c8 = cases.attn_case_q8(c16)
        r16, r8 = cases.attn_oracle(c16), cases.attn_oracle(c8)
        rows = c8["q8_rows"]
        for card in range(ncard):
            # the appended rows: quantised from the normed, rotated k and from v as numpy quantises them
            want_k, want_v = c8["kc"][card].copy(), c8["vc"][card].copy()
            for t in range(T):
                p = ctx + t
                if (p // 4) % ncard != card:
                    continue
                row = (p // 4 // ncard) * 4 + p % 4
                for want, src in ((want_k, r8["k"][t]), (want_v, c8["v"][t])):
                    one = cases.kv_q8_rows(src[None])
                    n = nkv * hd
                    want[row * n // 2:(row + 1) * n // 2] = one[:n // 2]
                    want[rows * n // 2 + row * n // 32:rows * n // 2 + (row + 1) * n // 32] = one[n // 2:]
            assert np.array_equal(r8["kc"][card], want_k) and np.array_equal(r8["vc"][card], want_v)
        assert np.abs(r8["out"] - r16["out"]).max() < 0.05 and not np.array_equal(r8["out"], r16["out"])
        if ncard == 1:
            kc = cases.kv_q8_values(r8["kc"][0], rows, nkv, hd).astype(np.float64)
            vc = cases.kv_q8_values(r8["vc"][0], rows, nkv, hd).astype(np.float64)
            qg = r8["qg"].astype(np.float64)
            for t in range(T):
                for h in range(nq):
                    L = ctx + t + 1
                    s = kc[:L, h // 2] @ qg[t, h, :hd] / np.sqrt(hd)
                    w = np.exp(s - s.max())
                    o = (w[:, None] * vc[:L, h // 2]).sum(0) / w.sum() / (1 + np.exp(-qg[t, h, hd:]))
                    assert np.allclose(r8["out"][t, h], o, rtol=2e-4, atol=2e-5)


def test_moe_layer_against_dequantised_float64(oracle):
    """The quantised FFN half equals, to quantisation error of the activations, the float64 product of the dequantised
    weights (the kind of check the reference's moe_mma_bench makes, tools/moe_mma_bench.cu:198-224)."""
    rng = np.random.default_rng(14)
    n, nexp, ffs, T = 512, 32, 256, 4
    w = cases.moe_weights(n, nexp, ffs, seed=3)
    x = rng.standard_normal((T, n)).astype(np.float32)
    r = cases.moe_oracle(w, x, topk=4)
    gu_w = oracle.dequant(w["gu_q4k"].reshape(-1), "q4k").reshape(nexp, 2 * ffs, n).astype(np.float64)
    dn_w = oracle.dequant(w["dn_q6k"].reshape(-1), "q6k").reshape(nexp, n, w["dn_src_cols"])[:, :, w["dn_c0"]:w["dn_c0"] + ffs].astype(np.float64)
    for t in range(T):
        acc = np.zeros(n)
        for k in range(4):
            e = r["topi"][t, k]
            g = gu_w[e] @ x[t].astype(np.float64)
            assert np.allclose(r["gu"][t * 4 + k], g, atol=0.02 * np.abs(g).max() + 1e-3)
            h = g[:ffs] / (1 + np.exp(-g[:ffs])) * g[ffs:]
            d = dn_w[e] @ h
            assert np.allclose(r["part"][t * 4 + k], d, atol=0.03 * np.abs(d).max() + 1e-4)
            acc += r["topw"][t, k] * r["part"][t * 4 + k]
        acc += r["sh"][t] / (1 + np.exp(-r["logits"][t, nexp]))
        assert np.allclose(r["out"][t], acc, rtol=1e-4, atol=1e-5)


def test_hyper_connections_against_float64(oracle):
    """The hyper-connection write and read: the oracle against a float64 statement of the same mixing with the same int8
    roundings of xs and lo (taken from a first float64 pass), to f32 rounding."""
    c = cases.hc_case(T=3, n=1024, hc=4, lr=64, seed=21)
    T, n, hc, lr = c["T"], c["n"], c["hc"], c["lr"]
    R = c["R"].copy()
    oracle.hc_write(R, c["bo"], c["inj_prev"])
    g = 2.0 / (1.0 + np.exp(-c["inj_prev"].astype(np.float64) / hc))
    want = c["R"].astype(np.float64) + c["bo"].astype(np.float64)[:, None, :] * g[:, :, None]
    assert np.allclose(R, want, rtol=1e-6, atol=1e-6)
    R2 = c["R"].copy()
    mixed, inject, q8 = oracle.hc_read(R2, c["w_norm"], c["down"], c["up"], c["eps"], c["bo"], c["inj_prev"], c["w_inj"], want_q8=True)
    assert np.allclose(R2, want, rtol=1e-6, atol=1e-6), "the folded write"
    assert np.array_equal(q8, oracle.quantize_q8_1(mixed))
    # float64 restatement
    Rp = R2.astype(np.float64).reshape(T, hc * n)
    xs = Rp * c["w_norm"]
    rs = 1.0 / np.sqrt((R2.astype(np.float64) ** 2).mean(-1) + c["eps"])                # [T][hc]
    xb = xs.reshape(T, -1, 32)
    xd = np.abs(xb).max(-1) / 127
    xq = np.round(xb / np.where(xd == 0, 1, xd)[..., None])
    dw = c["down"][0].astype(np.float64).reshape(lr, -1, 32) * c["down"][1].view(np.float16).astype(np.float64)[..., None]
    xdq = (xq * xd[..., None]).reshape(T, hc, n)
    lo_pre = np.einsum("rcn,tcn,tc->tr", dw.reshape(lr, hc, n), xdq, rs) / hc
    lo = lo_pre / (1 + np.exp(-lo_pre))
    lb = lo.reshape(T, -1, 32)
    ld = np.abs(lb).max(-1) / 127
    lq = np.round(lb / ld[..., None]) * ld[..., None]
    uw = c["up"][0].astype(np.float64).reshape(hc * n, -1, 32) * c["up"][1].view(np.float16).astype(np.float64)[..., None]
    gate = 1 / (1 + np.exp(-(uw.reshape(hc * n, lr) @ lq.reshape(T, lr).T).T))          # [T][hc n]
    xn = (xs.reshape(T, hc, n) * rs[..., None]).reshape(T, hc * n)
    ref = (gate * xn).reshape(T, hc, n).mean(1)
    # a rounding of xs or lo that falls the other way in float64 moves one code by one step: compare in the bulk
    err = np.abs(mixed - ref)
    assert np.median(err) < 2e-5 and np.quantile(err, 0.99) < 5e-3, (np.median(err), err.max())
    wi = (c["w_inj"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    inj = np.einsum("jcn,tcn,tc->tj", wi.reshape(hc, hc, n), xs.reshape(T, hc, n), rs)
    assert np.allclose(inject, inj, rtol=1e-4, atol=1e-4)


def test_block_selection_against_float64(oracle):
    """The indexer's restatement against plain float64 numpy: projection, normed query heads, pooled keys and scores to
    rounding; the selection as the `top` highest scores, this GPU's blocks of them ascending, then the row's tail; a scan over
    a list naming every owned position equals the scan without a list."""
    from tests import cases

    O = oracle
    T, pos0, top, ncard = 16, 201, 8, 2
    c = cases.qsa_case(T, pos0, 256, top, seed=11)
    r = [cases.qsa_oracle(c, card, ncard) for card in range(ncard)]
    bf = lambda w: (w.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    y64 = c["x"].astype(np.float64) @ np.concatenate([bf(c["wq"]), bf(c["wk"])]).T
    assert np.allclose(r[0]["y"], y64, rtol=1e-4, atol=1e-4)
    q = r[0]["q"].astype(np.float64)
    want_norm = np.sqrt((c["qn"].astype(np.float64) ** 2 * (y64[:, :512].reshape(T, 4, 128) ** 2)
                         / (y64[:, :512].reshape(T, 4, 128) ** 2).mean(-1, keepdims=True)).sum(-1))
    assert np.allclose(np.linalg.norm(q, axis=-1), want_norm, rtol=1e-4)      # the rotation keeps the normed head's length
    pooled = r[0]["pooled"].view(np.float16).astype(np.float64)
    for t in range(T):
        p = pos0 + t
        nv, tail = (p + 1) // 4, (p + 1) % 4
        s64 = np.maximum(q[t] @ pooled[:nv].T, 0).sum(0) / np.sqrt(128.0)
        assert np.allclose(r[0]["scores"][t, :nv], s64, rtol=1e-4, atol=1e-4)
        sel = np.sort(np.argsort(-r[0]["scores"][t, :nv], kind="stable")[:top])   # stable: the lower block among equals
        for card in range(ncard):
            mine = sel[sel % ncard == card]
            cells = ((mine // ncard)[:, None] * 4 + np.arange(4)).reshape(-1)
            if (p // 4) % ncard == card:
                cells = np.concatenate([cells, (p // 4 // ncard) * 4 + np.arange(tail)])
            assert r[card]["n_cells"][t] == len(cells) and np.array_equal(r[card]["cells"][t, :len(cells)], cells)
    dense = cases.qsa_oracle(cases.qsa_case(4, 9, 256, top, seed=2))
    assert (dense["n_cells"] == -1).all()
    a = cases.attn_case(T=4, ctx=300, nq=8, nkv=2, hd=128, ncard=2, seed=3)
    ref = cases.attn_oracle(a)
    own = [O.kv_owned(300 + t, 1, 2) for t in range(4)]
    cells = np.zeros((4, max(own)), np.int32)
    cells[:] = np.arange(max(own))
    part = O.attn_partial_cells(ref["qg"], ref["kc"][1], ref["vc"][1], 1, 2, 300, 8, 2, cells, np.array(own, np.int32), 128)
    assert np.array_equal(part.view(np.uint32), ref["part"][1].view(np.uint32))


def test_block_selection_edges(oracle):
    """Edges of the selection: exactly `top` visible blocks is still dense and one more selects; a window that starts inside
    a block pools it from the ring's earlier rows and its own; every GPU's cells together are the selection, each block once;
    equal scores keep the lower blocks."""
    from tests import cases

    O = oracle
    top = 8
    c = cases.qsa_case(8, 4 * top - 4, 256, top, seed=5)          # rows at positions 28 .. 35: 7, 7, 7, 8, 8, 8, 8, 9 visible blocks
    r = cases.qsa_oracle(c)
    assert list(r["n_cells"][:7]) == [-1] * 7 and r["n_cells"][7] == 4 * top   # position 35 completes block 8: nine visible, no tail
    # pooling across the window's start: position 30 and 31 in the window, 28 and 29 from the ring
    c = cases.qsa_case(4, 30, 256, top, seed=6)
    r = cases.qsa_oracle(c)
    y = r["y"][:, 512:]
    raw = [c["ring"][28 % 64].view(np.float16).astype(np.float32), c["ring"][29 % 64].view(np.float16).astype(np.float32),
           y[0].astype(np.float16).astype(np.float32), y[1].astype(np.float16).astype(np.float32)]
    mean = (((raw[0] + raw[1]) + raw[2]) + raw[3]) * np.float32(0.25)
    got = r["pooled"][7].view(np.float16).astype(np.float64)
    want = mean.astype(np.float64) / np.sqrt((mean.astype(np.float64) ** 2).mean() + 1e-6) * c["kn"]
    assert np.allclose(np.linalg.norm(got), np.linalg.norm(want), rtol=2e-3)          # the rotation keeps the length
    assert np.allclose(got[64:], want[64:], rtol=2e-3, atol=2e-3)                      # dimensions past the rotary are the normed mean
    # the GPUs' cells together
    c = cases.qsa_case(6, 801, 256, top, seed=7, ties=True)
    parts = [cases.qsa_oracle(c, card, 4) for card in range(4)]
    for t in range(6):
        p = 801 + t
        nv = (p + 1) // 4
        blocks = []
        for card, r in enumerate(parts):
            cells = r["cells"][t, :r["n_cells"][t]]
            full = cells[:len(cells) // 4 * 4].reshape(-1, 4) if (p // 4) % 4 != card else cells[:len(cells) - (p + 1) % 4].reshape(-1, 4)
            assert (full == full[:, :1] + np.arange(4)).all()
            blocks += [int(b) // 4 * 4 + card for b in full[:, 0]]                    # local block -> global block
        s = parts[0]["scores"][t, :nv]
        assert len(blocks) == top and len(set(blocks)) == top
        thr = np.sort(s)[::-1][top - 1]
        kept = sorted(blocks)
        assert all(s[b] >= thr for b in kept)
        ties = [b for b in range(nv) if s[b] == thr]
        kept_ties = [b for b in kept if s[b] == thr]
        assert kept_ties == ties[:len(kept_ties)]                                       # the lower blocks among equals
