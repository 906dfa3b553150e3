"""CPU ORACLE - test infrastructure, not product code.

ctypes binding of liboracle.so (the plain-C restatement of the reference's verify-window arithmetic) with numpy
arrays.  Only tests, the smoke check and the bench's CPU-baseline leg import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

MAXT = 16
TOPK_N = 64


class Job(C.Structure):
    _fields_ = [("w", C.c_int), ("n", C.c_int), ("y", C.c_int * MAXT), ("out", C.c_int * MAXT)]


JOB_DTYPE = np.dtype([("w", "<i4"), ("n", "<i4"), ("y", "<i4", (MAXT,)), ("out", "<i4", (MAXT,))])


PF_JOB = 64
BIGJOB_DTYPE = np.dtype([("w", "<i4"), ("n", "<i4"), ("y", "<i4", (PF_JOB,)), ("out", "<i4", (PF_JOB,))])


class KvPages(C.Structure):
    _fields_ = [("pt", C.c_void_p), ("page", C.c_size_t), ("rows", C.c_int), ("cap", C.c_int), ("q8", C.c_int)]


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("top_k", C.c_int)]


class Mt(C.Structure):
    _fields_ = [("mt", C.c_uint64 * 312), ("idx", C.c_int)]


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file (gcc, a second or two)."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".c", ".h"))]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        _LIB = C.CDLL(so)
        _LIB.orc_q8s_row_dot.restype = C.c_float
        _LIB.orc_d2h.restype = C.c_uint16
        _LIB.orc_d2h.argtypes = [C.c_double]
        _LIB.orc_mt_unif.restype = C.c_double
        _LIB.orc_mt_next.restype = C.c_uint64
        _LIB.orc_argmax.restype = C.c_uint
        _LIB.orc_top_tokens.restype = C.c_uint
    return _LIB


def P(a):
    """Pointer to a numpy array's data (None passes NULL).  The array must be C-contiguous."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle binding: array must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------- formats
Q4K_B, Q6K_B, Q80_B, Q81_B = 144, 210, 34, 36


def quantize_q4k(x):
    x = _f32(x)
    out = np.zeros(x.size // 256 * Q4K_B, np.uint8)
    lib().orc_quantize_q4k(P(x), P(out), C.c_size_t(x.size // 256))
    return out


def quantize_q6k(x):
    x = _f32(x)
    out = np.zeros(x.size // 256 * Q6K_B, np.uint8)
    lib().orc_quantize_q6k(P(x), P(out), C.c_size_t(x.size // 256))
    return out


def quantize_q8_0(x):
    x = _f32(x)
    out = np.zeros(x.size // 32 * Q80_B, np.uint8)
    lib().orc_quantize_q8_0(P(x), P(out), C.c_size_t(x.size // 32))
    return out


def dequant(blocks, kind):
    fn, bsz, vals = {"q4k": ("orc_dequant_q4k", Q4K_B, 256), "q6k": ("orc_dequant_q6k", Q6K_B, 256),
                     "q8_0": ("orc_dequant_q8_0", Q80_B, 32)}[kind]
    nb = blocks.size // bsz
    out = np.zeros(nb * vals, np.float32)
    getattr(lib(), fn)(P(blocks), P(out), C.c_size_t(nb))
    return out


def q8_0_to_split(blocks, rows, cols):
    q = np.zeros((rows, cols), np.int8)
    d = np.zeros((rows, cols // 32), np.uint16)
    lib().orc_q8_0_to_split(P(blocks), P(q), P(d), C.c_size_t(rows), C.c_size_t(cols))
    return q, d


def q6k_to_planes(blocks, rows, src_cols, c0=0, cols=None):
    cols = src_cols if cols is None else cols
    nu = cols // 32
    QL = np.zeros((rows, nu, 16), np.uint8)
    QH = np.zeros((rows, nu, 8), np.uint8)
    SC = np.zeros((rows, nu, 2), np.int8)
    D = np.zeros((rows, nu), np.uint16)
    lib().orc_q6k_to_planes(P(blocks), C.c_size_t(rows), C.c_size_t(src_cols), C.c_size_t(c0), C.c_size_t(cols), P(QL), P(QH),
                            P(SC), P(D))
    return QL, QH, SC, D


def quantize_q8_1(x):
    x = _f32(x)
    rows, n = x.shape
    out = np.zeros((rows, n // 32 * Q81_B), np.uint8)
    lib().orc_quantize_q8_1(P(x), P(out), n, rows)
    return out


def math_probe(op, x):
    x = _f32(x)
    y = np.zeros_like(x)
    lib().orc_math_probe(op, P(x), P(y), C.c_size_t(x.size))
    return y


# ---------------------------------------------------------------- MoE
def gemv_f32(W, x, parts):
    W, x = _f32(W), _f32(x)
    rows, n = W.shape
    T = x.shape[0]
    y = np.zeros((T, rows), np.float32)
    lib().orc_gemv_f32(P(W), P(x), P(y), rows, n, T, parts, rows)
    return y


def router_route(W, x, topk=10):
    W, x = _f32(W), _f32(x)
    L, n = W.shape
    T = x.shape[0]
    logits = np.zeros((T, L), np.float32)
    topi = np.zeros((T, topk), np.int32)
    topw = np.zeros((T, topk), np.float32)
    gu = np.zeros(T * topk, JOB_DTYPE)
    dn = np.zeros(T * topk, JOB_DTYPE)
    nj = np.zeros(2, np.int32)
    lib().orc_router_route(P(W), P(x), P(logits), T, n, L - 1, topk, P(topi), P(topw), P(gu), P(dn), P(nj))
    return logits, topi, topw, gu, dn, int(nj[0])


def moe_gate_up_q4k(A, sa, jobs, njobs, xq, n, nrows, nout):
    gu = np.zeros((nout, nrows), np.float32)
    lib().orc_moe_gate_up_q4k(P(A), C.c_size_t(sa), P(jobs), njobs, P(xq), P(gu), n, nrows)
    return gu


def q8s_gemv(wq, wd, yq, T):
    rows, cols = wq.shape
    out = np.zeros((T, rows), np.float32)
    lib().orc_q8s_gemv(P(wq), P(wd), rows, cols, P(yq), P(out), rows, T)
    return out


def q8s_gemv_blocks(wq, wd, yq, T):
    """The dense product with its sums in block order (this library's tensor-core kernel's order, not the reference's)."""
    rows, cols = wq.shape
    out = np.zeros((T, rows), np.float32)
    lib().orc_q8s_gemv_blocks(P(wq), P(wd), rows, cols, P(yq), P(out), rows, T)
    return out


def moe_gate_up_q8(wq, wd, jobs, njobs, xq, T, nout):
    nexp, nrows, n = wq.shape
    gu = np.zeros((nout, nrows), np.float32)
    lib().orc_moe_gate_up_q8(P(wq), C.c_size_t(nrows * n), P(wd), C.c_size_t(nrows * n // 32), P(jobs), njobs, P(xq), T, P(gu),
                             n, nrows)
    return gu


def moe_down_q6p(planes, jobs, njobs, gu, nrows, ffs, nout):
    QL, QH, SC, D = planes  # [nexp][rows][nu][..]
    part = np.zeros((nout, nrows), np.float32)
    lib().orc_moe_down_q6p(P(QL), P(QH), P(SC), P(D), C.c_size_t(nrows * (ffs // 32)), P(jobs), njobs, P(_f32(gu)), P(part), nrows,
                           ffs)
    return part


def moe_down_q8(wq, wd, jobs, njobs, gu, nout):
    nexp, nrows, ffs = wq.shape
    part = np.zeros((nout, nrows), np.float32)
    lib().orc_moe_down_q8(P(wq), C.c_size_t(nrows * ffs), P(wd), C.c_size_t(nrows * ffs // 32), P(jobs), njobs, P(_f32(gu)),
                          P(part), nrows, ffs)
    return part


def mma_weights_q4k(A, rows, n):
    """f16 weights (bit patterns) of `rows` Q4_K rows of n columns, several experts stacked as rows."""
    w = np.zeros((rows, n), np.uint16)
    lib().orc_mma_weights_q4k(P(A), rows, n, P(w))
    return w


def mma_weights_q8(wq, wd):
    rows, n = wq.reshape(-1, wq.shape[-1]).shape
    w = np.zeros((rows, n), np.uint16)
    lib().orc_mma_weights_q8(P(wq), P(wd), rows, n, P(w))
    return w


def mma_weights_q6p(planes, rows, n):
    QL, QH, SC, D = planes
    w = np.zeros((rows, n), np.uint16)
    lib().orc_mma_weights_q6p(P(QL), P(QH), P(SC), P(D), rows, n, P(w))
    return w


def moe_mma(w, jobs, njobs, x, nrows, nout):
    """w: f16 bits [experts * nrows][n]; x: f16 bits [rows][n]; returns (sums, sums of |products|) as float64 [nout][nrows]."""
    n = w.shape[-1]
    out = np.zeros((nout, nrows), np.float64)
    mag = np.zeros((nout, nrows), np.float64)
    lib().orc_moe_mma(P(w), P(jobs), njobs, P(x), nrows, n, P(out), P(mag))
    return out, mag


def swiglu_h16(gu, ffs):
    gu = _f32(gu)
    h = np.zeros((gu.shape[0], ffs), np.uint16)
    lib().orc_swiglu_h16(P(gu), ffs, gu.shape[0], P(h))
    return h


def shared_expert(guq, gud, dnq, dnd, xq, T):
    n = guq.shape[1]
    ffs = guq.shape[0] // 2
    sh_gu = np.zeros((T, 2 * ffs), np.float32)
    out = np.zeros((T, n), np.float32)
    lib().orc_shared_expert(P(guq), P(gud), P(dnq), P(dnd), P(xq), T, n, ffs, P(sh_gu), P(out))
    return sh_gu, out


def moe_combine(part, topw, sh, logits, T, n, topk=10):
    out = np.zeros((T, n), np.float32)
    L = logits.shape[1]
    lib().orc_moe_combine(P(_f32(part)), P(_f32(topw)), P(_f32(sh)), P(_f32(logits)), L, L - 1, P(out), T, n, topk)
    return out


def rms_norm_rows(x, w, eps):
    x, w = _f32(x), _f32(w)
    y = np.zeros_like(x)
    lib().orc_rms_norm_rows(P(x), P(w), P(y), x.shape[0], x.shape[1], C.c_float(eps))
    return y


# ---------------------------------------------------------------- Gated DeltaNet
def gdn_core(qkvz, ab, hist, convw, dt, a, nw, S, ctl, nk, nv, vmap, eps, want_y32=True):
    """Runs the core in place on hist and S (pass copies).  Returns yq, y32, snap, hsnap."""
    T = qkvz.shape[0]
    ch = (2 * nk + nv) * 128
    yq = np.zeros((T, nv * 128 // 32 * Q81_B), np.uint8)
    y32 = np.zeros((T, nv * 128), np.float32) if want_y32 else None
    snap = np.zeros((max(T - 1, 1), nv, 128, 128), np.float32)
    hsnap = np.zeros((MAXT, 3, ch), np.float32)
    lib().orc_gdn_core(P(qkvz), P(ab), P(hist), P(convw), P(dt), P(a), P(nw), P(S), P(yq), P(ctl), P(snap), P(hsnap), nk, nv,
                       P(vmap), T, C.c_float(eps), P(y32))
    return yq, y32, snap, hsnap


def gdn_rollback(S, hist, snap, hsnap, ctl, nk, nv, T, n):
    lib().orc_gdn_rollback(P(S), P(hist), P(snap), P(hsnap), P(ctl), nk, nv, T, n)


# ---------------------------------------------------------------- attention
def kv_owned(p, card, ncard):
    return lib().orc_kv_owned(p, card, ncard)


def rope_freqs(base, nrot):
    f = np.zeros(nrot // 2, np.float32)
    lib().orc_rope_freqs(C.c_float(base), nrot, P(f))
    return f


def attn_prep_append(qg, k, v, qn, kn, kc, vc, card, ncard, pos0, eps, base, nq, nkv, hd=256, nrot=64, q8_rows=0):
    """q8_rows > 0: kc / vc are int8 caches of that many rows (uint16 arrays of kvq_halves(rows) halves)."""
    T = qg.shape[0]
    g = KvPages(None, 0, 0, q8_rows, 1 if q8_rows else 0)
    lib().orc_attn_prep_append(P(qg), P(k), P(v), P(qn), P(kn), P(kc), P(vc), C.byref(g), card, ncard, T, pos0, C.c_float(eps),
                               C.c_float(base), nq, nkv, hd, nrot)


def kvq_halves(rows, nkv, hd):
    return rows * nkv * hd // 2 + rows * nkv * hd // 32


def attn_partial(qg, kc, vc, card, ncard, pos0, nq, nkv, hd=256, q8_rows=0):
    T = qg.shape[0]
    part = np.zeros((T, nq, hd + 2), np.float32)
    g = KvPages(None, 0, 0, q8_rows, 1 if q8_rows else 0)
    lib().orc_attn_partial(P(qg), P(kc), P(vc), C.byref(g), P(part), card, ncard, T, pos0, nq, nkv, hd)
    return part


def attn_partial_cells(qg, kc, vc, card, ncard, pos0, nq, nkv, cells, n_cells, hd=256, q8_rows=0):
    """cells [T][maxsel] int32, n_cells [T] int32 (-1: the row attends every owned position)."""
    T = qg.shape[0]
    part = np.zeros((T, nq, hd + 2), np.float32)
    g = KvPages(None, 0, 0, q8_rows, 1 if q8_rows else 0)
    lib().orc_attn_partial_cells(P(qg), P(kc), P(vc), C.byref(g), P(part), card, ncard, T, pos0, nq, nkv, hd, P(cells), P(n_cells),
                                 cells.shape[1])
    return part


# ---------------------------------------------------------------- the attention layers' block selection
QSA_DIM, QSA_HEADS, QSA_POOL = 128, 4, 4


def _pages(pt, page, rows):
    return KvPages(pt.ctypes.data_as(C.POINTER(C.c_int)) if pt is not None else None, page, rows, 0, 0)


def qsa_proj(wq, wk, x):
    """wq [512][n], wk [128][n] bf16 bit patterns (uint16); x [T][n] f32 -> y [T][640]."""
    T, n = x.shape
    y = np.zeros((T, QSA_HEADS * QSA_DIM + QSA_DIM), np.float32)
    lib().orc_qsa_proj(P(wq), P(wk), P(x), P(y), T, n)
    return y


def qsa_index(y, qn, kn, ring, pooled, pos0, eps, base, ncard=1, pt=None, page=0, rows=0):
    """ring [ring_rows][128], pooled: uint16 (f16 bits), both updated in place; returns q [T][4][128]."""
    T = y.shape[0]
    q = np.zeros((T, QSA_HEADS, QSA_DIM), np.float32)
    g = _pages(pt, page, rows)
    lib().orc_qsa_index(P(y), P(qn), P(kn), P(ring), ring.shape[0], P(pooled), C.byref(g), ncard, P(q), pos0, T, C.c_float(eps),
                        C.c_float(base))
    return q


def qsa_select(q, pooled, pos, top, max_pools, card=0, ncard=1, pt=None, page=0, rows=0):
    """pos [T] int32: every row's position.  Returns (scores [T][max_pools], cells [T][4 top + 3], n_cells [T])."""
    T = q.shape[0]
    scores = np.zeros((T, max_pools), np.float32)
    cells = np.zeros((T, top * QSA_POOL + QSA_POOL - 1), np.int32)
    n_cells = np.zeros(T, np.int32)
    g = _pages(pt, page, rows)
    pos = np.ascontiguousarray(pos, np.int32)
    lib().orc_qsa_select(P(q), P(pooled), C.byref(g), P(scores), P(cells), P(n_cells), max_pools, P(pos), None, T, card, ncard, top)
    return scores, cells, n_cells


def attn_merge(parts, qg, nq, hd=256):
    T = qg.shape[0]
    out = np.zeros((T, nq, hd), np.float32)
    arr = (C.c_void_p * len(parts))(*[p.ctypes.data for p in parts])
    lib().orc_attn_merge(arr, P(qg), P(out), len(parts), T, nq, hd)
    return out


# ---------------------------------------------------------------- hyper-connections
def hc_write(R, bo, inj):
    """R [T][hc][n] += bo [T][n] * 2 sigmoid(inj [T][hc] / hc), in place."""
    T, hc, n = R.shape
    lib().orc_hc_write(P(R), P(_f32(bo)), P(_f32(inj)), T, n, hc)


def hc_read(R, w_norm, down, up, eps, bo_prev=None, inj_prev=None, w_inj=None, want_q8=False):
    """The read (R updated in place when bo_prev is given).  down = (int8 [lr][hc n], f16 bits [lr][hc n / 32]),
    up = (int8 [hc n][lr], f16 bits [hc n][lr / 32]), w_inj bf16 bits [hc][hc n] or None.  Returns mixed [T][n],
    inject [T][hc] (None without w_inj), q8_1 rows of mixed (None unless asked)."""
    T, hc, n = R.shape
    lr = down[0].shape[0]
    mixed = np.zeros((T, n), np.float32)
    inject = np.zeros((T, hc), np.float32) if w_inj is not None else None
    q8 = np.zeros((T, n // 32 * Q81_B), np.uint8) if want_q8 else None
    lib().orc_hc_read(P(R), P(bo_prev), P(inj_prev), P(w_norm), P(down[0]), P(down[1]), P(up[0]), P(up[1]), P(w_inj), C.c_float(eps), P(mixed),
                      P(inject), P(q8), T, n, hc, lr)
    return mixed, inject, q8


# ---------------------------------------------------------------- head and acceptance
def argmax(logits, v0=0):
    logits = _f32(logits)
    T, rows = logits.shape
    bv = np.zeros(T, np.float32)
    bi = np.zeros(T, np.int32)
    err = lib().orc_argmax(P(logits), rows, T, v0, P(bv), P(bi))
    return bv, bi, err


def argmax_merge(best_v, best_i):
    nslice, T = best_v.shape
    out = np.zeros(T, np.int32)
    lib().orc_argmax_merge(P(_f32(best_v)), P(np.ascontiguousarray(best_i, np.int32)), nslice, T, P(out))
    return out


def top_tokens(logits, v0, pen_tok, pen_cnt, pen_n, pen_par):
    """logits is modified in place (the penalties), as the reference's kernel does."""
    T, n = logits.shape
    stride = pen_tok.shape[1] if pen_tok.ndim == 2 else 1
    ov = np.zeros((T, TOPK_N), np.float32)
    oi = np.zeros((T, TOPK_N), np.int32)
    err = lib().orc_top_tokens(P(logits), n, T, v0, P(pen_tok), P(pen_cnt), P(pen_n), stride, P(pen_par), P(ov), P(oi))
    return ov, oi, err


def top_merge(vs, is_):
    nslice, T, _ = vs.shape
    ov = np.zeros((T, TOPK_N), np.float32)
    oi = np.zeros((T, TOPK_N), np.int32)
    lib().orc_top_merge(P(_f32(vs)), P(np.ascontiguousarray(is_, np.int32)), nslice, T, P(ov), P(oi))
    return ov, oi


def make_dist(cv, ci, temperature=1.0, top_p=1.0, min_p=0.0, top_k=0):
    s = Sampling(temperature, top_p, min_p, top_k)
    n = C.c_int(0)
    ids = np.zeros(TOPK_N, np.int32)
    p = np.zeros(TOPK_N, np.float64)
    lib().orc_make_dist(P(_f32(cv)), P(np.ascontiguousarray(ci, np.int32)), len(cv), C.byref(s), C.byref(n), P(ids), P(p))
    return ids[: n.value].copy(), p[: n.value].copy()


def mt_new(seed):
    g = Mt()
    lib().orc_mt_seed(C.byref(g), C.c_uint64(seed))
    return g


def mt_unif(g):
    return lib().orc_mt_unif(C.byref(g))


def lookup_drafts(ctx, lk, d1=-1, image_tok=1 << 30):
    ctx = np.ascontiguousarray(ctx, np.int32)
    out = np.zeros(max(lk, 1), np.int32)
    n = lib().orc_lookup_drafts(P(ctx), len(ctx), lk, d1, image_tok, P(out))
    return out[:n].copy()


def accept_greedy(rows, out):
    rows = np.ascontiguousarray(rows, np.int32)
    out = np.ascontiguousarray(out, np.int32)
    return lib().orc_accept_greedy(P(rows), P(out), len(rows))


def accept_sampled(rows, cand_v, cand_i, rng, temperature=1.0, top_p=1.0, min_p=0.0, top_k=0):
    rows = np.ascontiguousarray(rows, np.int32)
    s = Sampling(temperature, top_p, min_p, top_k)
    o = np.zeros(len(rows), np.int32)
    n = lib().orc_accept_sampled(P(rows), len(rows), P(_f32(cand_v)), P(np.ascontiguousarray(cand_i, np.int32)), C.byref(s),
                                 C.byref(rng), P(o))
    return n, o[:n].copy()


def ring_sum(xs):
    nrank = len(xs)
    T, row_len = xs[0].shape
    out = np.zeros((T, row_len), np.float32)
    arr = (C.c_void_p * nrank)(*[x.ctypes.data for x in xs])
    lib().orc_ring_sum(arr, P(out), nrank, T, row_len)
    return out
