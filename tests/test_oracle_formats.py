"""The oracle's block formats and exact math, pinned without a GPU: dequantisation against the committed fixture made
with the `gguf` package, the quantisers' round trip, the device-layout repacks, and the math against libm."""
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_dequant_matches_gguf_fixture(oracle):
    g = np.load(os.path.join(GOLD, "dequant.npz"))
    for kind in ("q4k", "q6k", "q8_0"):
        mine = oracle.dequant(g[kind + "_blocks"], kind)
        assert np.array_equal(mine.view(np.uint32), g[kind + "_values"].view(np.uint32)), kind


def test_quantisers_round_trip(oracle):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(256 * 40) * 0.02).astype(np.float32)
    for kind, fn, tol in (("q4k", oracle.quantize_q4k, 0.12), ("q6k", oracle.quantize_q6k, 0.03), ("q8_0", oracle.quantize_q8_0, 0.01)):
        y = oracle.dequant(fn(x), kind)
        assert np.sqrt(np.mean((y - x) ** 2)) / 0.02 < tol, kind
    assert np.all(oracle.dequant(oracle.quantize_q4k(np.zeros(256, np.float32)), "q4k") == 0)
    assert np.all(oracle.dequant(oracle.quantize_q6k(np.zeros(256, np.float32)), "q6k") == 0)


def test_q8_0_split_layout(oracle):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((6, 96)) * 0.02).astype(np.float32)
    b = oracle.quantize_q8_0(x)
    q, d = oracle.q8_0_to_split(b, 6, 96)
    vals = q.astype(np.float32).reshape(6, 3, 32) * d.view(np.float16).astype(np.float32)[:, :, None]
    assert np.array_equal(vals.reshape(-1), oracle.dequant(b, "q8_0"))


def test_q6k_units_hold_the_same_values(oracle):
    """The 32-column regrouping of Q6_K dequantises to the GGUF block's values, whole and for a column slice."""
    rng = np.random.default_rng(3)
    rows, cols = 5, 768
    x = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    b = oracle.quantize_q6k(x)
    ref = oracle.dequant(b, "q6k").reshape(rows, cols)
    for c0, n in ((0, cols), (96, 96), (672, 96), (384, 384)):
        QL, QH, SC, D = oracle.q6k_to_planes(b, rows, cols, c0, n)
        assert QL.nbytes + QH.nbytes + SC.nbytes + D.nbytes == rows * (n // 32) * 28
        codes = np.zeros((rows, n // 32, 32), np.int32)
        for i in range(32):
            lo = (QL[:, :, i] & 15) if i < 16 else (QL[:, :, i - 16] >> 4)
            w, bb = i // 4, i % 4
            hi = (QH[:, :, (w // 4) * 4 + bb] >> (2 * (w % 4))) & 3
            codes[:, :, i] = lo.astype(np.int32) | (hi.astype(np.int32) << 4)
        d = D.view(np.float16).astype(np.float32)
        sc = np.repeat(SC.astype(np.float32), 16, axis=2)
        vals = (d[:, :, None] * sc) * (codes - 32).astype(np.float32)
        assert np.array_equal(vals.reshape(rows, n), ref[:, c0:c0 + n])


def test_q8_1_rounding(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 128)).astype(np.float32)
    x[1, 32:64] = 0
    q = oracle.quantize_q8_1(x).reshape(3, 4, 36)
    d = q[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    s = q[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    qs = q[:, :, 4:].view(np.int8).astype(np.float32)
    xb = x.reshape(3, 4, 32)
    amax = np.abs(xb).max(-1)
    assert np.array_equal(d, (amax / np.float32(127)).astype(np.float16).astype(np.float32))
    assert np.all(qs[1, 1] == 0) and d[1, 1] == 0
    assert np.abs(qs).max() == 127
    assert np.allclose(s, xb.sum(-1), rtol=2e-3, atol=2e-3)
    assert np.max(np.abs(qs * (amax / 127)[..., None] - xb)) <= (amax / 127).max() * 0.5001


def test_exact_math_close_to_libm(oracle):
    x = np.linspace(-85.9, 87.9, 200001).astype(np.float32)
    r = np.exp(x.astype(np.float64))
    assert np.max(np.abs(oracle.math_probe(0, x) - r) / r) < 2e-7
    assert oracle.math_probe(0, np.array([-100, 100], np.float32)).tolist() == [0.0, np.inf]
    y = np.logspace(-10, 8.5, 50001).astype(np.float32)
    r = np.log1p(y.astype(np.float64))
    assert np.max(np.abs(oracle.math_probe(1, y) - r) / r) < 5e-7
    x = np.linspace(-30, 30, 20001).astype(np.float32)
    assert np.max(np.abs(oracle.math_probe(2, x) - 1 / (1 + np.exp(-x.astype(np.float64))))) < 2e-7
    th = np.linspace(0, 3e5, 300001).astype(np.float32)
    assert np.max(np.abs(oracle.math_probe(5, th) - np.sin(th.astype(np.float64)))) < 1e-7
    assert np.max(np.abs(oracle.math_probe(6, th) - np.cos(th.astype(np.float64)))) < 1e-7
    assert oracle.math_probe(4, np.array([256.0], np.float32))[0] == 0.0625
