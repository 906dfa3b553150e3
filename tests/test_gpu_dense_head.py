"""GPU parity of the dense Q8_0 projections, the f32 GEMV, RMS norm, argmax and the exact top-64, and of the device
math against the oracle's, bit-exact through the C ABI."""
import numpy as np
import pytest

from tests import cases
from tests.test_oracle_path import _tie_cases, pack_pens

pytestmark = pytest.mark.gpu


def test_device_math_bit_exact(oracle):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(40)
    probes = {0: np.concatenate([np.linspace(-90, 90, 100001), rng.standard_normal(50000) * 10]),
              1: np.concatenate([np.logspace(-12, 8.6, 100001), [0.0]]),
              2: np.linspace(-40, 40, 100001), 3: np.linspace(-40, 40, 100001),
              4: np.logspace(-8, 8, 100001), 5: np.linspace(0, 1.2e6, 200001), 6: np.linspace(0, 1.2e6, 200001),
              7: rng.standard_normal(100000) * 100}
    for op, x in probes.items():
        x = x.astype(np.float32)
        dx = G.dev(x)
        dy = torch.zeros_like(dx)
        L.call("fnx_math_probe", op, dx.data_ptr(), dy.data_ptr(), x.size, L.stream())
        G.sync()
        assert np.array_equal(G.host(dy).view(np.uint32), oracle.math_probe(op, x).view(np.uint32)), op


def _q8s_case(rows, cols, T, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    wq, wd = cases.O.q8_0_to_split(cases.O.quantize_q8_0(w), rows, cols)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    return wq, wd, cases.O.quantize_q8_1(x)


@pytest.mark.parametrize("rows,cols,T", [(100, 512, 1), (257, 768, 3), (1000, 3072, 16), (4133, 3072, 7), (96, 6144, 16)])
def test_q8s_gemv(rows, cols, T):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    wq, wd, yq = _q8s_case(rows, cols, T, rows + T)
    ref = cases.O.q8s_gemv(wq, wd, yq, T)
    w, keep = G.q8s((wq, wd))
    dy = G.dev(yq)
    out = G.zeros((T, rows))
    L.call("fnx_q8s_gemv", w, rows, cols, dy.data_ptr(), out.data_ptr(), rows, T, L.stream())
    G.sync()
    assert np.array_equal(G.host(out).view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("rows,cols,T", [(16384, 3072, 16), (8200, 1024, 5), (40000, 2560, 1), (9000, 256, 16)])
def test_q8s_gemv_blocks_tensor_cores(rows, cols, T):
    """The tcgen05 dense kernel: bit-equal to the oracle's statement of its order of sums (blocks in ascending order), equal
    to the reference-order product to fp32 rounding of the sum, over ragged row counts (a last tile past the matrix), one
    to sixteen window rows and several widths; no bounded wait ran out."""
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(rows + T)
    wq = rng.integers(-127, 128, size=(rows, cols), dtype=np.int8)
    wd = (rng.random((rows, cols // 32), dtype=np.float32) * 2e-4 + 1e-4).astype(np.float16).view(np.uint16)
    yq = cases.O.quantize_q8_1(rng.standard_normal((T, cols)).astype(np.float32))
    want = cases.O.q8s_gemv_blocks(wq, wd, yq, T)
    w, keep = G.q8s((wq, wd))
    dy, out = G.dev(yq), G.zeros((T, rows))
    for _ in range(2):   # twice: the barriers' phases start afresh with every launch
        out.zero_()
        L.call("fnx_q8s_gemv_blocks", w, rows, cols, dy.data_ptr(), out.data_ptr(), rows, T, L.stream())
        G.sync()
        assert L.load().fnx_device_fault() == 0
        assert np.array_equal(G.host(out).view(np.uint32), want.view(np.uint32))
    ref = cases.O.q8s_gemv(wq, wd, yq, T)
    assert np.allclose(want, ref, rtol=0, atol=4e-6 * np.abs(ref).max())
    assert L.load().fnx_q8s_gemv_blocks(w, 100, cols, dy.data_ptr(), out.data_ptr(), rows, T, L.stream()) != 0   # too few rows: refused


def test_q8s_gemv_f32_pair(oracle):
    """The quantised projection and the small f32 one behind one call (the DeltaNet layer's qkvz and alpha|beta): each
    output as its own entry point gives it."""
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rows, cols, T, rf = 4100, 3072, 16, 96
    wq, wd, yq = _q8s_case(rows, cols, T, 77)
    rng = np.random.default_rng(78)
    W = (rng.standard_normal((rf, cols)) * 0.02).astype(np.float32)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    w, keep = G.q8s((wq, wd))
    dy, dW, dx, out, yf = G.dev(yq), G.dev(W), G.dev(x), G.zeros((T, rows)), G.zeros((T, rf))
    L.call("fnx_q8s_gemv_f32", w, rows, cols, dy.data_ptr(), out.data_ptr(), dW.data_ptr(), dx.data_ptr(), yf.data_ptr(), rf, T, L.stream())
    G.sync()
    assert np.array_equal(G.host(out).view(np.uint32), cases.O.q8s_gemv(wq, wd, yq, T).view(np.uint32))
    assert np.array_equal(G.host(yf).view(np.uint32), oracle.gemv_f32(W, x, 4).view(np.uint32))


def test_gemv_f32_and_rms_norm(oracle):
    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(41)
    W = (rng.standard_normal((96, 3072)) * 0.02).astype(np.float32)
    x = rng.standard_normal((16, 3072)).astype(np.float32)
    dW, dx, y = G.dev(W), G.dev(x), G.zeros((16, 96))
    L.call("fnx_gemv_f32", dW.data_ptr(), dx.data_ptr(), y.data_ptr(), 96, 3072, 16, L.stream())
    G.sync()
    assert np.array_equal(G.host(y).view(np.uint32), oracle.gemv_f32(W, x, 4).view(np.uint32))
    # norm with the residual add folded in and the q8_1 copy
    add = rng.standard_normal((16, 3072)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(3072)).astype(np.float32)
    import torch

    dadd, dwn, yn = G.dev(add), G.dev(wn), G.zeros((16, 3072))
    q = G.zeros(16 * 96 * 36, torch.uint8)
    L.call("fnx_rms_norm_rows", dx.data_ptr(), dadd.data_ptr(), dwn.data_ptr(), yn.data_ptr(), q.data_ptr(), 16, 3072, 1e-6, L.stream())
    G.sync()
    x2 = x + add
    ref = oracle.rms_norm_rows(x2, wn, 1e-6)
    assert np.array_equal(G.host(dx), x2)
    assert np.array_equal(G.host(yn).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(G.host(q).reshape(16, -1), oracle.quantize_q8_1(ref))


def test_argmax_and_top64(oracle):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    for name, rows, pens, v0 in _tie_cases():
        logits = np.stack(rows)
        T, n = logits.shape
        tok, cnt, pn, par = pack_pens(pens)
        ref_l = logits.copy()
        rv, ri, _ = oracle.top_tokens(ref_l, v0, tok, cnt, pn, par)
        dl = G.dev(logits)
        keys, err = G.zeros(32, torch.int64), G.zeros(1, torch.int32)
        bv, bi = G.zeros(T), G.zeros(T, torch.int32)
        L.call("fnx_argmax", dl.data_ptr(), n, T, v0, bv.data_ptr(), bi.data_ptr(), keys.data_ptr(), err.data_ptr(), L.stream())
        ov, oi = G.zeros((T, 64)), G.zeros((T, 64), torch.int32)
        dt, dc, dn, dp = G.dev(tok), G.dev(cnt), G.dev(pn), G.dev(par)
        L.call("fnx_top_tokens", dl.data_ptr(), n, T, v0, dt.data_ptr(), dc.data_ptr(), dn.data_ptr(), tok.shape[1], dp.data_ptr(),
               ov.data_ptr(), oi.data_ptr(), err.data_ptr(), L.stream())
        G.sync()
        av, ai, _ = oracle.argmax(logits, v0)
        assert np.array_equal(G.host(bi), ai) and np.array_equal(G.host(bv), av), name
        assert np.array_equal(G.host(oi), ri) and np.array_equal(G.host(ov), rv), name
        assert np.array_equal(G.host(dl), ref_l), name   # penalties applied in place
        assert int(G.host(err)[0]) == 0 and not G.host(keys).any()
    bad = np.zeros((2, 4096), np.float32)
    bad[1, 77] = np.nan
    dl, err = G.dev(bad), G.zeros(1, torch.int32)
    keys, bv, bi = G.zeros(32, torch.int64), G.zeros(2), G.zeros(2, torch.int32)
    L.call("fnx_argmax", dl.data_ptr(), 4096, 2, 0, bv.data_ptr(), bi.data_ptr(), keys.data_ptr(), err.data_ptr(), L.stream())
    G.sync()
    assert int(G.host(err)[0]) == 16


@pytest.mark.gpu
def test_l2_prefetch_changes_nothing():
    """fnx_l2_prefetch (reference src/kernels.hpp:364 l2_prefetch) is a hint: any range, aligned or not, leaves the bytes as
    they were and raises no error; an empty range is accepted."""
    import torch
    from sfnx_b200 import lib
    x = torch.randint(0, 255, (5 * 1024 * 1024 + 77,), dtype=torch.uint8, device="cuda")
    ref = x.clone()
    st = torch.cuda.current_stream().cuda_stream
    for off, n in [(0, x.numel()), (3, 100), (16, 32768), (5, 1 << 20), (0, 0)]:
        lib.call("fnx_l2_prefetch", x.data_ptr() + off, n, st)
    torch.cuda.synchronize()
    assert torch.equal(x, ref)
