"""Generates the committed golden fixtures under tests/golden/ (run where the reference tree and the `gguf` Python
package are present; the fixtures then travel with the repository).

  dequant.npz   random GGUF blocks of Q4_K / Q6_K / Q8_0 and their dequantisation by the `gguf` package (third-party
                black box pinning the block formats)
  accept.npz    candidate lists, sampling settings and seeds with the outputs of the reference's own make_dist / draw
                (johnfink8/sfnx src/session.cpp, compiled unmodified into oracle/_ref/libref_accept.so) and of the
                acceptance loop around them, plus the unit uniforms of std::mt19937_64
  lookup.npz    token histories with draft budgets and required first drafts, and the n-gram lookup drafts the reference's
                own lookup_drafts (src/session.cpp:377-394, the same object code) returns for them

Usage: make -C oracle ref && python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import binding as O  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def dequant_fixture():
    import gguf
    from gguf import quants

    rng = np.random.default_rng(20240)
    out = {}
    for kind, bsz, t, scale_hi in [("q4k", 144, gguf.GGMLQuantizationType.Q4_K, (1, 3)),
                                   ("q6k", 210, gguf.GGMLQuantizationType.Q6_K, (209,)),
                                   ("q8_0", 34, gguf.GGMLQuantizationType.Q8_0, (1,))]:
        b = rng.integers(0, 256, (96, bsz), dtype=np.uint8)
        for hi in scale_hi:   # keep the f16 scales finite and small
            b[:, hi] &= 0x3F
        # and blocks made by quantising N(0, 0.02) values
        x = (rng.standard_normal(32 * (256 if bsz != 34 else 32)) * 0.02).astype(np.float32)
        qb = {"q4k": O.quantize_q4k, "q6k": O.quantize_q6k, "q8_0": O.quantize_q8_0}[kind](x).reshape(-1, bsz)
        blocks = np.concatenate([b, qb]).reshape(-1)
        out[kind + "_blocks"] = blocks
        out[kind + "_values"] = quants.dequantize(blocks, t).reshape(-1).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "dequant.npz"), **out)


def accept_fixture():
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_accept.so"))
    rng = np.random.default_rng(777)
    ncase, T = 64, 16
    cand_v = np.zeros((ncase, T, 64), np.float32)
    cand_i = np.zeros((ncase, T, 64), np.int32)
    rows = np.zeros((ncase, T), np.int32)
    samp = np.zeros((ncase, 4), np.float64)   # temperature, top_p, min_p, top_k
    seeds = rng.integers(0, 2**62, ncase).astype(np.uint64)
    n_out = np.zeros(ncase, np.int32)
    toks = np.zeros((ncase, T), np.int32)
    dist_n = np.zeros((ncase, T), np.int32)
    dist_ids = np.zeros((ncase, T, 64), np.int32)
    dist_p = np.zeros((ncase, T, 64), np.float64)
    for c in range(ncase):
        temp = float(rng.choice([1.0, 0.6, 1.3]))
        top_p = float(rng.choice([1.0, 0.95, 0.5]))
        min_p = float(rng.choice([0.0, 0.05]))
        top_k = int(rng.choice([0, 8, 40]))
        samp[c] = [temp, top_p, min_p, top_k]
        s = O.Sampling(temp, top_p, min_p, top_k)
        spread = float(rng.choice([0.5, 3.0]))
        for t in range(T):
            v = np.sort((rng.standard_normal(64) * spread).astype(np.float32))[::-1]
            if rng.random() < 0.2:
                v[3:6] = v[3]   # ties
            cand_v[c, t] = v
            cand_i[c, t] = rng.permutation(151936)[:64]
            n = C.c_int()
            ref.ref_make_dist(O.P(cand_v[c, t]), O.P(cand_i[c, t]), 64, C.byref(s), C.byref(n), O.P(dist_ids[c, t]), O.P(dist_p[c, t]))
            dist_n[c, t] = n.value
        rows[c, 0] = rng.integers(0, 151936)
        for t in range(1, T):   # drafts: mostly the row's likeliest candidates, sometimes not a candidate at all
            r = rng.random()
            rows[c, t] = cand_i[c, t - 1, 0] if r < 0.6 else cand_i[c, t - 1, rng.integers(0, 64)] if r < 0.9 else 7
        n_out[c] = ref.ref_accept_sampled(O.P(rows[c]), T, O.P(cand_v[c]), O.P(cand_i[c]), C.byref(s), C.c_ulonglong(int(seeds[c])), 0,
                                          O.P(toks[c]), None)
    u = np.zeros(4096)
    ref.ref_uniforms(C.c_ulonglong(424242), 4096, O.P(u))
    np.savez_compressed(os.path.join(OUT, "accept.npz"), cand_v=cand_v, cand_i=cand_i, rows=rows, samp=samp, seeds=seeds, n_out=n_out,
                        toks=toks, dist_n=dist_n, dist_ids=dist_ids, dist_p=dist_p, unif_seed=np.uint64(424242), unif=u)


def lookup_fixture():
    """Contexts over small alphabets (so that trigrams repeat), with copied runs, image cells and contexts that end in the
    middle of a repeat; for each a draft budget lk and a required first draft d1: the reference's own lookup_drafts."""
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_accept.so"))
    rng = np.random.default_rng(4242)
    ncase, maxn = 400, 96
    ctx = np.zeros((ncase, maxn), np.int32)
    n = np.zeros(ncase, np.int32)
    lk = np.zeros(ncase, np.int32)
    d1 = np.zeros(ncase, np.int32)
    cnt = np.zeros(ncase, np.int32)
    out = np.zeros((ncase, 16), np.int32)
    for c in range(ncase):
        n[c] = rng.integers(0, maxn + 1)
        seq = rng.integers(0, int(rng.choice([2, 3, 5, 50])), maxn).astype(np.int32)
        if n[c] > 24 and rng.random() < 0.6:   # a copied run: the tail repeats an earlier stretch
            L = int(rng.integers(4, 12))
            src = int(rng.integers(0, n[c] - 2 * L))
            seq[n[c] - L:n[c]] = seq[src:src + L]
        if rng.random() < 0.2 and n[c] > 8:
            seq[rng.integers(0, n[c])] = (1 << 30) + 5   # an image cell somewhere
        ctx[c] = seq
        lk[c] = rng.integers(0, 16)
        d1[c] = -1 if rng.random() < 0.5 else rng.integers(0, 5)
        cnt[c] = ref.ref_lookup_drafts(O.P(ctx[c]), int(n[c]), int(lk[c]), int(d1[c]), O.P(out[c]))
    assert (cnt > 0).sum() > 60, "too few cases with drafts"
    np.savez_compressed(os.path.join(OUT, "lookup.npz"), ctx=ctx, n=n, lk=lk, d1=d1, cnt=cnt, out=out)


if __name__ == "__main__":
    dequant_fixture()
    accept_fixture()
    lookup_fixture()
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))
