"""The oracle of the prompt path's experts, pinned without a GPU: its one-rounding conversion to f16, its f16 weights
against the (gguf-pinned) f32 dequantisation, and its sums against numpy."""
import numpy as np


def test_double_to_f16_rounds_once(oracle):
    """numpy converts float64 to float16 with one rounding to nearest even; so must the oracle, ties and values a hair off
    a tie included (the cases a detour through float32 gets wrong)."""
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(20000) * 10.0 ** rng.integers(-6, 4, 20000),
                        np.float64(np.float16(rng.standard_normal(2000))) * (1 + 2.0 ** -11),                       # exact ties
                        np.float64(np.float16(rng.standard_normal(2000))) * (1 + 2.0 ** -11) * (1 + 2.0 ** -40),    # a hair above
                        np.float64(np.float16(rng.standard_normal(2000))) * (1 + 2.0 ** -11) * (1 - 2.0 ** -40),    # a hair below
                        np.array([0.0, -0.0, 65504.0, 65519.9, 5.96e-8, 2.9e-8, 3.1e-8, 6.0e-5, -6.1e-5])])
    lib = oracle.lib()
    got = np.array([lib.orc_d2h(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, x.astype(np.float16).view(np.uint16))


def test_f16_weights_are_the_f32_dequantisation_rounded(oracle):
    rng = np.random.default_rng(6)
    rows, n = 24, 512
    x = (rng.standard_normal((rows, n)) * 0.02).astype(np.float32)
    # Q8_0: q * d is exact in f32, so the f16 weight is that value rounded once
    q, d = oracle.q8_0_to_split(oracle.quantize_q8_0(x), rows, n)
    w = oracle.mma_weights_q8(q, d).view(np.float16)
    ref = (q.astype(np.float32).reshape(rows, n // 32, 32) * d.view(np.float16).astype(np.float32)[:, :, None]).reshape(rows, n)
    assert np.array_equal(w.view(np.uint16), ref.astype(np.float16).view(np.uint16))
    # Q4_K: scale and min are rounded to f16 before the fused step: within an f16 unit in the last place of the larger
    # term of (d sc) q - dmin m (the reference's own bound, src/moe_mma.cuh:56-60)
    b = oracle.quantize_q4k(x)
    w = oracle.mma_weights_q4k(b, rows, n).view(np.float16).astype(np.float64)
    f32 = oracle.dequant(b, "q4k").reshape(rows, n).astype(np.float64)
    scale = np.abs(f32).reshape(rows, n // 32, 32).max(axis=2, keepdims=True)   # at least the larger term's size over the sub-block
    err = np.abs(w - f32).reshape(rows, n // 32, 32)
    assert (err <= 2.0 ** -9 * np.maximum(scale, 1e-8) + 2.0 ** -24).all(), float((err / np.maximum(scale, 1e-8)).max())
    # Q6_K units: (d sc) rounded to f16, then one product
    b6 = oracle.quantize_q6k(x)
    planes = oracle.q6k_to_planes(b6, rows, n)
    w = oracle.mma_weights_q6p(planes, rows, n).view(np.float16).astype(np.float64)
    f32 = oracle.dequant(b6, "q6k").reshape(rows, n).astype(np.float64)
    assert (np.abs(w - f32) <= 2.0 ** -10 * np.abs(f32) + 2.0 ** -24).all()


def test_sums_in_double(oracle):
    rng = np.random.default_rng(7)
    nexp, rows, n = 3, 10, 64
    w = rng.standard_normal((nexp * rows, n)).astype(np.float16)
    x = rng.standard_normal((5, n)).astype(np.float16)
    jobs = np.zeros(2, oracle.BIGJOB_DTYPE)
    jobs[0]["w"], jobs[0]["n"] = 2, 3
    jobs[0]["y"][:3], jobs[0]["out"][:3] = [4, 0, 1], [0, 1, 2]
    jobs[1]["w"], jobs[1]["n"] = 0, 1
    jobs[1]["y"][:1], jobs[1]["out"][:1] = [2], [3]
    out, mag = oracle.moe_mma(w.view(np.uint16), jobs, 2, x.view(np.uint16), rows, 4)
    W, X = w.astype(np.float64).reshape(nexp, rows, n), x.astype(np.float64)
    assert np.allclose(out[:3], X[[4, 0, 1]] @ W[2].T, rtol=1e-13, atol=1e-13)
    assert np.allclose(out[3], X[2] @ W[0].T, rtol=1e-13, atol=1e-13)
    assert np.allclose(mag[3], np.abs(X[2]) @ np.abs(W[0]).T, rtol=1e-13)
    g = rng.standard_normal((4, 2 * 96)).astype(np.float32)
    h = oracle.swiglu_h16(g, 96).view(np.float16).astype(np.float64)
    ref = g[:, :96].astype(np.float64) / (1 + np.exp(-g[:, :96].astype(np.float64))) * g[:, 96:]
    assert np.allclose(h, ref, rtol=2e-3, atol=1e-6)
