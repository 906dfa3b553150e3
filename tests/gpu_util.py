"""Helpers of the GPU parity tests: numpy <-> device tensors and thin wrappers over the C ABI (test infrastructure)."""
import ctypes as C

import numpy as np
import torch

from sfnx_b200 import lib as L

DEV = "cuda:0"


def dev(a):
    """numpy array -> device tensor of the same bytes (uint16 goes over as int16)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    if a.dtype.fields is not None:   # structured (jobs)
        return torch.from_numpy(a.view(np.uint8)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def host(t, dtype=None):
    a = t.detach().cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def zeros(shape, dtype=torch.float32):
    return torch.zeros(shape, dtype=dtype, device=DEV)


def sync():
    torch.cuda.synchronize()


def q8s(qd):
    """(int8 plane, uint16 scales) numpy pair -> (FnxQ8S, keepalive tensors)."""
    q, d = dev(qd[0]), dev(qd[1])
    return L.Q8S(q.data_ptr(), d.data_ptr()), (q, d)


def experts_q4k(blocks, nrows, ncols):
    """[nexp][bytes] Q4_K rows -> FnxExperts."""
    t = dev(blocks)
    e = L.Experts(L.Q4_K, nrows, ncols, t.data_ptr(), None, None, None, blocks.shape[1], 0)
    return e, (t,)


def experts_q6p(planes, nrows, ffs):
    QL, QH, SC, D = (dev(p) for p in planes)
    e = L.Experts(L.Q6_K, nrows, ffs, QL.data_ptr(), QH.data_ptr(), SC.data_ptr(), D.data_ptr(), nrows * (ffs // 32), 0)
    return e, (QL, QH, SC, D)


def experts_q8(planes, nrows, ncols):
    """([nexp][nrows][ncols] int8, [nexp][nrows][ncols / 32] f16 bits) -> FnxExperts of type Q8_0."""
    q, d = dev(planes[0]), dev(planes[1])
    e = L.Experts(L.Q8_0, nrows, ncols, q.data_ptr(), d.data_ptr(), None, None, nrows * ncols, nrows * (ncols // 32) * 2)
    return e, (q, d)


def run_moe(w, x, topk=10, keep=None):
    """The FFN half through the C ABI on device copies of the case's weights; returns intermediates as numpy."""
    n, nexp, ffs = w["n"], w["nexp"], w["ffs"]
    T, P = x.shape[0], x.shape[0] * topk
    st = L.stream()
    dx = dev(x)
    xq = zeros(T * (n // 32) * 36, torch.uint8)
    L.call("fnx_quantize_q8_1", dx.data_ptr(), xq.data_ptr(), n, T, st)
    router = dev(w["router"])
    logits, topi, topw = zeros((T, nexp + 1)), zeros((T, topk), torch.int32), zeros((T, topk))
    jgu, jdn = zeros(P * 136, torch.uint8), zeros(P * 136, torch.uint8)
    njobs, scratch = zeros(2, torch.int32), zeros(16, torch.uint8)
    L.call("fnx_router_route", router.data_ptr(), dx.data_ptr(), logits.data_ptr(), T, n, nexp, topk, topi.data_ptr(), topw.data_ptr(),
           jgu.data_ptr(), jdn.data_ptr(), njobs.data_ptr(), scratch.data_ptr(), st)
    if w.get("experts") == "q8_0":
        egu, k1 = experts_q8(w["gu_q8"], 2 * ffs, n)
        edn, k2 = experts_q8(w["dn_q8"], n, ffs)
    else:
        egu, k1 = experts_q4k(w["gu_q4k"], 2 * ffs, n)
        edn, k2 = experts_q6p(w["dn_planes"], n, ffs)
    gu = zeros((P, 2 * ffs))
    L.call("fnx_moe_gate_up", C.byref(egu), jgu.data_ptr(), njobs.data_ptr(), P, xq.data_ptr(), gu.data_ptr(), st)
    hq = zeros(L.load().fnx_moe_h_bytes(P, ffs), torch.uint8)
    part = zeros((P, n))
    L.call("fnx_moe_down", C.byref(edn), jdn.data_ptr(), njobs.data_ptr(), P, gu.data_ptr(), P, hq.data_ptr(), part.data_ptr(), st)
    sgu, k3 = q8s(w["sh_gu"])
    sdn, k4 = q8s(w["sh_dn"])
    sh_gu, sh = zeros((T, 2 * ffs)), zeros((T, n))
    shq = zeros(L.load().fnx_moe_h_bytes(T, ffs), torch.uint8)
    L.call("fnx_shared_expert", sgu, sdn, xq.data_ptr(), T, n, ffs, sh_gu.data_ptr(), shq.data_ptr(), sh.data_ptr(), st)
    out = zeros((T, n))
    L.call("fnx_moe_combine", part.data_ptr(), topw.data_ptr(), sh.data_ptr(), logits.data_ptr(), nexp, out.data_ptr(), T, n, topk, st)
    sync()
    from oracle.binding import JOB_DTYPE

    nj = int(host(njobs)[0])
    return {"xq": host(xq).reshape(T, -1), "logits": host(logits), "topi": host(topi), "topw": host(topw), "njobs": nj,
            "jobs_gu": host(jgu).view(JOB_DTYPE), "jobs_dn": host(jdn).view(JOB_DTYPE), "gu": host(gu), "part": host(part),
            "sh_gu": host(sh_gu), "sh": host(sh), "out": host(out), "counter": host(scratch)}


def run_gdn(c, want_y32=True):
    T, nk, nv, ch = c["T"], c["nk"], c["nv"], c["ch"]
    st = L.stream()
    t = {k: dev(c[k]) for k in ("qkvz", "ab", "hist", "convw", "dt", "a", "nw", "S", "vmap", "ctl")}
    yq = zeros(T * (nv * 128 // 32) * 36, torch.uint8)
    y32 = zeros((T, nv * 128)) if want_y32 else None
    scratch = zeros(L.load().fnx_gdn_scratch_floats(nv))
    snap = zeros((max(T - 1, 1), nv, 128, 128))
    hsnap = zeros((16, 3, ch))
    L.call("fnx_gdn_core", t["qkvz"].data_ptr(), t["ab"].data_ptr(), t["hist"].data_ptr(), t["convw"].data_ptr(), t["dt"].data_ptr(),
           t["a"].data_ptr(), t["nw"].data_ptr(), t["S"].data_ptr(), yq.data_ptr(), t["ctl"].data_ptr(), scratch.data_ptr(),
           snap.data_ptr(), hsnap.data_ptr(), nk, nv, t["vmap"].data_ptr(), T, c["eps"], st, L.ptr(y32))
    sync()
    return {"S": host(t["S"]), "hist": host(t["hist"]), "yq": host(yq).reshape(T, -1), "y32": host(y32) if want_y32 else None,
            "snap": host(snap), "hsnap": host(hsnap), "scratch_tail": host(scratch)[-nv:], "dev": (t, snap, hsnap)}
