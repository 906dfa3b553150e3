"""n-gram lookup drafts: the oracle's statement and the library's host function against the outputs of the reference's own
lookup_drafts (src/session.cpp:377-394, compiled unmodified: tests/golden/lookup.npz, made by tests/golden/make_golden.py).
Host code only: no GPU is needed."""
import ctypes as C
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lookup.npz")


def _cases():
    g = np.load(GOLD)
    for c in range(len(g["n"])):
        yield g["ctx"][c][: g["n"][c]].copy(), int(g["lk"][c]), int(g["d1"][c]), g["out"][c][: g["cnt"][c]].tolist()


def test_oracle_lookup_matches_the_reference(oracle):
    hits = 0
    for ctx, lk, d1, want in _cases():
        assert oracle.lookup_drafts(ctx, lk, d1).tolist() == want, (ctx.tolist(), lk, d1)
        hits += bool(want)
    assert hits > 60


def test_library_lookup_matches_the_reference(fnx):
    lib = fnx.load()
    for ctx, lk, d1, want in _cases():
        out = (C.c_int * 16)()
        arr = (C.c_int * max(1, len(ctx)))(*ctx.tolist())
        n = lib.fnx_lookup_drafts(arr, len(ctx), lk, d1, 1 << 30, out)
        assert n >= 0 and list(out[:n]) == want, (ctx.tolist(), lk, d1)
    assert lib.fnx_lookup_drafts(None, 5, 3, -1, 1 << 30, None) < 0   # refused, not dereferenced
