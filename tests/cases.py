"""Seeded synthetic cases of the verify window and their evaluation by the CPU oracle (test infrastructure).

Shapes follow the benchmark configurations: one MoE FFN layer (T rows, hidden n, nexp experts, top-k + shared expert,
Q4_K gate|up, Q6_K down, Q8_0 shared expert), one Gated DeltaNet layer with rollback, position-split attention.
"""
import numpy as np

from oracle import binding as O


# ---------------------------------------------------------------- MoE layer
def moe_weights(n, nexp, ffs, seed=0, sigma=0.02):
    """ffs not a multiple of 256 (an FF slice of a wider expert, as one GPU of several holds): the down matrix is cut
    out of a 256-column-aligned Q6_K matrix at column 64."""
    rng = np.random.default_rng(seed)
    w = {"n": n, "nexp": nexp, "ffs": ffs}
    src_cols = ffs if ffs % 256 == 0 else (64 + ffs + 255) // 256 * 256
    c0 = 0 if ffs % 256 == 0 else 64
    w["router"] = (rng.standard_normal((nexp + 1, n)) * sigma).astype(np.float32)
    gu = (rng.standard_normal((nexp, 2 * ffs, n)) * sigma).astype(np.float32)
    w["gu_q4k"] = O.quantize_q4k(gu).reshape(nexp, 2 * ffs * (n // 256) * 144)
    dn = (rng.standard_normal((nexp, n, src_cols)) * sigma).astype(np.float32)
    w["dn_q6k"] = O.quantize_q6k(dn).reshape(nexp, n * (src_cols // 256) * 210)
    w["dn_src_cols"], w["dn_c0"] = src_cols, c0
    planes = [O.q6k_to_planes(w["dn_q6k"][e], n, src_cols, c0, ffs) for e in range(nexp)]
    w["dn_planes"] = tuple(np.stack([p[i] for p in planes]) for i in range(4))
    sgu = (rng.standard_normal((2 * ffs, n)) * sigma).astype(np.float32)
    sdn = (rng.standard_normal((n, ffs)) * sigma).astype(np.float32)
    w["sh_gu"] = O.q8_0_to_split(O.quantize_q8_0(sgu), 2 * ffs, n)
    w["sh_dn"] = O.q8_0_to_split(O.quantize_q8_0(sdn), n, ffs)
    return w


def moe_weights_q8(n, nexp, ffs, seed=0, sigma=0.02):
    """The same layer with the routed experts in split Q8_0 (the all-Q8_0 configuration): gate|up [nexp][2 ffs][n] and
    down [nexp][n][ffs] as int8 planes + f16 block scales."""
    rng = np.random.default_rng(seed)
    w = {"n": n, "nexp": nexp, "ffs": ffs, "experts": "q8_0"}
    w["router"] = (rng.standard_normal((nexp + 1, n)) * sigma).astype(np.float32)
    gu = (rng.standard_normal((nexp * 2 * ffs, n)) * sigma).astype(np.float32)
    q, d = O.q8_0_to_split(O.quantize_q8_0(gu), nexp * 2 * ffs, n)
    w["gu_q8"] = (q.reshape(nexp, 2 * ffs, n), d.reshape(nexp, 2 * ffs, n // 32))
    dn = (rng.standard_normal((nexp * n, ffs)) * sigma).astype(np.float32)
    q, d = O.q8_0_to_split(O.quantize_q8_0(dn), nexp * n, ffs)
    w["dn_q8"] = (q.reshape(nexp, n, ffs), d.reshape(nexp, n, ffs // 32))
    sgu = (rng.standard_normal((2 * ffs, n)) * sigma).astype(np.float32)
    sdn = (rng.standard_normal((n, ffs)) * sigma).astype(np.float32)
    w["sh_gu"] = O.q8_0_to_split(O.quantize_q8_0(sgu), 2 * ffs, n)
    w["sh_dn"] = O.q8_0_to_split(O.quantize_q8_0(sdn), n, ffs)
    return w


def big_jobs(ntok, nexp, topk, seed=0, cap=64):
    """The prompt path's jobs: every token picks topk distinct experts, pair p = t topk + k; an expert's pairs in pair
    order, cut into jobs of at most `cap` rows (reference src/kernels.hpp:25-32).  Returns (jobs, pairs)."""
    rng = np.random.default_rng(seed)
    picks = np.argsort(rng.random((ntok, nexp)), axis=1)[:, :topk]
    order = np.argsort(picks.reshape(-1), kind="stable")   # pairs grouped by expert, in pair order inside an expert
    experts = picks.reshape(-1)[order]
    jobs, start = [], 0
    while start < len(order):
        e = experts[start]
        end = start + int(np.searchsorted(experts[start:], e, side="right"))
        for i in range(start, end, cap):
            jobs.append((e, order[i:min(i + cap, end)]))
        start = end
    out = np.zeros(len(jobs), O.BIGJOB_DTYPE)
    for j, (e, pairs) in enumerate(jobs):
        out[j]["w"], out[j]["n"] = e, len(pairs)
        out[j]["y"][:len(pairs)], out[j]["out"][:len(pairs)] = pairs // topk, pairs
    return out, ntok * topk


def moe_oracle(w, x, topk=10):
    """The whole FFN half on the CPU oracle; returns every intermediate."""
    n, ffs = w["n"], w["ffs"]
    T = x.shape[0]
    r = {}
    r["xq"] = O.quantize_q8_1(x)
    r["logits"], r["topi"], r["topw"], r["jobs_gu"], r["jobs_dn"], r["njobs"] = O.router_route(w["router"], x, topk)
    if w.get("experts") == "q8_0":
        r["gu"] = O.moe_gate_up_q8(w["gu_q8"][0], w["gu_q8"][1], r["jobs_gu"], r["njobs"], r["xq"], T, T * topk)
        r["part"] = O.moe_down_q8(w["dn_q8"][0], w["dn_q8"][1], r["jobs_dn"], r["njobs"], r["gu"], T * topk)
    else:
        r["gu"] = O.moe_gate_up_q4k(w["gu_q4k"], w["gu_q4k"].shape[1], r["jobs_gu"], r["njobs"], r["xq"], n, 2 * ffs, T * topk)
        r["part"] = O.moe_down_q6p(w["dn_planes"], r["jobs_dn"], r["njobs"], r["gu"], n, ffs, T * topk)
    r["sh_gu"], r["sh"] = O.shared_expert(w["sh_gu"][0], w["sh_gu"][1], w["sh_dn"][0], w["sh_dn"][1], r["xq"], T)
    r["out"] = O.moe_combine(r["part"], r["topw"], r["sh"], r["logits"], T, n, topk)
    return r


# ---------------------------------------------------------------- Gated DeltaNet layer
def gdn_case(T, nk, nv, seed=0):
    """q/k/v/z rows, gates and state with the distributions of the benchmark configuration: state N(0, 0.1), q/k/v
    N(0, 1) before the conv (the core L2-normalises q and k itself), beta = sigmoid(N(0, 1)), decay = exp(-softplus(N(0,
    1))) through a = -1, dt = 0; conv width 4."""
    rng = np.random.default_rng(seed)
    ch = (2 * nk + nv) * 128
    c = {"T": T, "nk": nk, "nv": nv, "ch": ch}
    c["qkvz"] = rng.standard_normal((T, ch + nv * 128)).astype(np.float32)
    c["ab"] = rng.standard_normal((T, 2 * nv)).astype(np.float32)
    c["hist"] = rng.standard_normal((2, 3, ch)).astype(np.float32)
    c["convw"] = (rng.standard_normal((ch, 4)) * 0.5).astype(np.float32)
    c["dt"] = np.zeros(nv, np.float32)
    c["a"] = -np.ones(nv, np.float32)
    c["nw"] = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    c["S"] = (rng.standard_normal((nv, 128, 128)) * 0.1).astype(np.float32)
    vpk = nv // nk
    vmap = np.zeros(nv, np.int32)
    for lv in range(nv):   # value heads in key-head order; the first value head of a key head writes its history
        vmap[lv] = (lv // vpk) | ((1 if lv % vpk == 0 else 0) << 8)
    c["vmap"] = vmap
    c["ctl"] = np.array([1000, 5], np.int32)   # position, tag (odd: history parity 1)
    c["eps"] = 1e-6
    return c


def gdn_oracle(c):
    S, hist = c["S"].copy(), c["hist"].copy()
    yq, y32, snap, hsnap = O.gdn_core(c["qkvz"], c["ab"], hist, c["convw"], c["dt"], c["a"], c["nw"], S, c["ctl"], c["nk"], c["nv"],
                                      c["vmap"], c["eps"])
    return {"S": S, "hist": hist, "yq": yq, "y32": y32, "snap": snap, "hsnap": hsnap}


# ---------------------------------------------------------------- attention
def attn_case(T, ctx, nq=24, nkv=4, hd=256, ncard=1, seed=0, ramp=None):
    """A K/V cache of ctx positions N(0, 1) rounded to f16, split by position over ncard GPUs, and a window of T rows at
    positions ctx .. ctx + T - 1.  With `ramp` the cached keys grow from 0.5x at position 0 to ramp x at the last one, so
    that a row's largest score keeps rising along the scan."""
    rng = np.random.default_rng(seed)
    c = {"T": T, "ctx": ctx, "nq": nq, "nkv": nkv, "hd": hd, "ncard": ncard, "pos0": ctx}
    c["qg"] = rng.standard_normal((T, nq, 2 * hd)).astype(np.float32)
    c["k"] = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    c["v"] = rng.standard_normal((T, nkv, hd)).astype(np.float32)
    c["qn"] = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    c["kn"] = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    rows = ((ctx + T + 3) // 4 + ncard - 1) // ncard * 4
    full_k = rng.standard_normal((ctx, nkv, hd))
    if ramp is not None:
        full_k *= np.linspace(0.5, ramp, ctx)[:, None, None]
    full_k = full_k.astype(np.float16)
    full_v = rng.standard_normal((ctx, nkv, hd)).astype(np.float16)
    c["kc"], c["vc"] = [], []
    for card in range(ncard):
        kc = np.zeros((rows, nkv, hd), np.float16)
        vc = np.zeros((rows, nkv, hd), np.float16)
        p = np.arange(ctx)
        mine = (p // 4) % ncard == card
        at = (p // 4 // ncard) * 4 + p % 4
        kc[at[mine]], vc[at[mine]] = full_k[mine], full_v[mine]
        c["kc"].append(kc.view(np.uint16))
        c["vc"].append(vc.view(np.uint16))
    c["eps"] = 1e-6
    c["rope_base"] = 1e7
    return c


def kv_q8_rows(x):
    """Rows [rows][nkv][hd] (any float type) as an int8 cache: groups of 32 with d = max |x| / 127, q = round-half-away(x / d),
    f16 d (reference src/kernels.cu:1561-1566), laid out as one page: the int8 rows, then the rows' scales; returned as
    the uint16 words the entry points take."""
    rows = x.shape[0]
    g = x.astype(np.float32).reshape(rows, -1, 32)
    d = (np.abs(g).max(-1) / np.float32(127)).astype(np.float32)
    inv = np.where(d != 0, np.float32(1) / np.where(d != 0, d, np.float32(1)), np.float32(0)).astype(np.float32)
    y = g * inv[..., None]
    q = (np.sign(y) * np.floor(np.abs(y) + np.float32(0.5))).astype(np.int8)
    return np.concatenate([q.reshape(-1).view(np.uint16), d.astype(np.float16).reshape(-1).view(np.uint16)])


def kv_q8_values(words, rows, nkv, hd):
    """The f32 values an int8 cache holds: [rows][nkv][hd]."""
    n = rows * nkv * hd
    q = words[:n // 2].view(np.int8).astype(np.float32).reshape(rows, -1, 32)
    d = words[n // 2:n // 2 + n // 32].view(np.float16).astype(np.float32).reshape(rows, -1)
    return (q * d[..., None]).reshape(rows, nkv, hd)


def attn_case_q8(c):
    """The same case with int8 K/V caches (the cached rows quantised as the append would have)."""
    c = dict(c)
    c["q8_rows"] = c["kc"][0].shape[0]
    c["kc"] = [kv_q8_rows(k.view(np.float16)) for k in c["kc"]]
    c["vc"] = [kv_q8_rows(v.view(np.float16)) for v in c["vc"]]
    return c


def attn_oracle(c):
    """Runs prep + append + partials + merge per GPU on copies; returns qg/k after prep, the caches, partials, out."""
    T, nq, nkv, hd, ncard = c["T"], c["nq"], c["nkv"], c["hd"], c["ncard"]
    r = {"kc": [], "vc": [], "part": []}
    q8 = c.get("q8_rows", 0)
    for card in range(ncard):
        qg, k = c["qg"].copy(), c["k"].copy()
        kc, vc = c["kc"][card].copy(), c["vc"][card].copy()
        O.attn_prep_append(qg, k, c["v"], c["qn"], c["kn"], kc, vc, card, ncard, c["pos0"], c["eps"], c["rope_base"], nq, nkv, hd,
                           q8_rows=q8)
        r["qg"], r["k"] = qg, k
        r["kc"].append(kc)
        r["vc"].append(vc)
        r["part"].append(O.attn_partial(qg, kc, vc, card, ncard, c["pos0"], nq, nkv, hd, q8_rows=q8))
    r["out"] = O.attn_merge(r["part"], r["qg"], nq, hd)
    return r


# ---------------------------------------------------------------- logits comparison (the reference's exactness bar)
def kl_top64(ref, new):
    """Per-row KL(ref || new) over the union of both rows' 64 highest logits, a token outside a side's 64 taking that
    side's 64th logit, probabilities from each side's full-row log-sum-exp (reference tools/fnx_run.cpp:244-288)."""
    out = []
    for a, b in zip(ref.astype(np.float64), new.astype(np.float64)):
        ia, ib = np.argsort(-a, kind="stable")[:64], np.argsort(-b, kind="stable")[:64]
        union = np.union1d(ia, ib)
        la = a.max() + np.log(np.exp(a - a.max()).sum())
        lb = b.max() + np.log(np.exp(b - b.max()).sum())
        va = np.where(np.isin(union, ia), a[union], a[ia[-1]]) - la
        vb = np.where(np.isin(union, ib), b[union], b[ib[-1]]) - lb
        out.append(float(np.sum(np.exp(va) * (va - vb))))
    return np.array(out)


# ---------------------------------------------------------------- hyper-connections
def hc_case(T, n, hc, lr, seed, fold=True, inject=True):
    """Residual streams R [T][hc][n], the norm weights, split Q8_0 down [lr][hc n] and up [hc n][lr] (random int8 codes
    and f16 scales), bf16 inject rows, and the previous half's output and inject values when its write is folded in."""
    rng = np.random.default_rng(seed)
    D = n * hc
    c = {"T": T, "n": n, "hc": hc, "lr": lr, "eps": 1e-6}
    c["R"] = rng.standard_normal((T, hc, n)).astype(np.float32)
    c["w_norm"] = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    c["down"] = (rng.integers(-127, 128, (lr, D), dtype=np.int8), (0.02 * rng.random((lr, D // 32)) / 127).astype(np.float16).view(np.uint16))
    c["up"] = (rng.integers(-127, 128, (D, lr), dtype=np.int8), (0.3 * rng.random((D, lr // 32)) / 127).astype(np.float16).view(np.uint16))
    c["w_inj"] = (rng.standard_normal((hc, D)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16) if inject else None
    c["bo"] = rng.standard_normal((T, n)).astype(np.float32) if fold else None
    c["inj_prev"] = rng.standard_normal((T, hc)).astype(np.float32) if fold else None
    return c


# ---------------------------------------------------------------- the attention layers' block selection
def bf16_bits(a):
    """float array -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def qsa_case(T, pos0, n=256, top=8, seed=0, ties=False, ring_rows=64):
    """Indexer weights (bf16), a window of T rows at positions pos0 .. pos0 + T - 1, a ring holding raw keys of earlier
    positions and the pooled keys of the pos0 / 4 blocks completed before the window.  ties: the blocks' keys are drawn
    from 20 distinct ones, so that many scores are equal and the rule among equals (the lower block first) decides."""
    rng = np.random.default_rng(seed)
    c = {"T": T, "pos0": pos0, "n": n, "top": top, "eps": 1e-6, "rope_base": 1e7}
    c["wq"] = bf16_bits(0.05 * rng.standard_normal((512, n)))
    c["wk"] = bf16_bits(0.05 * rng.standard_normal((128, n)))
    c["x"] = rng.standard_normal((T, n)).astype(np.float32)
    c["qn"] = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    c["kn"] = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    c["ring"] = rng.standard_normal((ring_rows, 128)).astype(np.float16).view(np.uint16)
    c["max_pools"] = (pos0 + T) // 4 + 8
    pooled = rng.standard_normal((c["max_pools"], 128)).astype(np.float16)
    if ties:
        pooled = pooled[rng.integers(0, 20, c["max_pools"])]
    pooled[pos0 // 4:] = 0
    c["pooled"] = pooled.view(np.uint16)
    return c


def qsa_oracle(c, card=0, ncard=1):
    y = O.qsa_proj(c["wq"], c["wk"], c["x"])
    ring, pooled = c["ring"].copy(), c["pooled"].copy()
    q = O.qsa_index(y, c["qn"], c["kn"], ring, pooled, c["pos0"], c["eps"], c["rope_base"], ncard)
    pos = np.arange(c["pos0"], c["pos0"] + c["T"], dtype=np.int32)
    scores, cells, n_cells = O.qsa_select(q, pooled, pos, c["top"], c["max_pools"], card, ncard)
    return {"y": y, "ring": ring, "pooled": pooled, "q": q, "scores": scores, "cells": cells, "n_cells": n_cells}
