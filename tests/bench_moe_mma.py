"""Times the routed experts of the prompt path (jobs of up to 64 rows of one expert on the tcgen05 tensor cores):
`python -m tests.bench_moe_mma [--tokens 4096] [--experts 512] [--type q4k|q8_0]`.

The counterpart of the reference's tools/moe_mma_bench.cu (random experts of the real shapes, 4,096 tokens): seeded
synthetic weights generated on the GPU, every token routed to top-k distinct experts, an expert's pairs cut into jobs of
at most 64 rows.  Prints one JSON line: milliseconds per launch (CUDA events, median), weight bytes and FLOPs per second
for gate|up, SwiGLU and down.  Weights of 512 experts (1.4 GB and up) are far larger than L2, so launches run back to back.
"""
import argparse
import ctypes as C
import json

import numpy as np

from sfnx_b200 import lib as L

PF_JOB = 64
BIGJOB_DTYPE = np.dtype([("w", "<i4"), ("n", "<i4"), ("y", "<i4", (PF_JOB,)), ("out", "<i4", (PF_JOB,))])


def big_jobs(ntok, nexp, topk, seed=0, cap=PF_JOB):
    """Every token picks topk distinct experts, pair p = t topk + k; an expert's pairs in pair order, cut into jobs of at
    most `cap` rows (reference src/kernels.hpp:25-32).  Returns (jobs, pairs)."""
    rng = np.random.default_rng(seed)
    picks = np.argsort(rng.random((ntok, nexp)), axis=1)[:, :topk]
    order = np.argsort(picks.reshape(-1), kind="stable")   # pairs grouped by expert, in pair order inside an expert
    experts = picks.reshape(-1)[order]
    jobs = []
    start = 0
    while start < len(order):
        e = experts[start]
        end = start + int(np.searchsorted(experts[start:], e, side="right"))
        for i in range(start, end, cap):
            jobs.append((e, order[i:min(i + cap, end)]))
        start = end
    out = np.zeros(len(jobs), BIGJOB_DTYPE)
    for j, (e, pairs) in enumerate(jobs):
        out[j]["w"], out[j]["n"] = e, len(pairs)
        out[j]["y"][:len(pairs)], out[j]["out"][:len(pairs)] = pairs // topk, pairs
    return out, ntok * topk


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=512)
    ap.add_argument("--topk", type=int, default=10)
    ap.add_argument("--hidden", type=int, default=3072)
    ap.add_argument("--ff", type=int, default=768)
    ap.add_argument("--type", default="q4k", choices=["q4k", "q8_0"], help="q4k: Q4_K gate|up + Q6_K down; q8_0: both Q8_0")
    ap.add_argument("--reps", type=int, default=20)
    a = ap.parse_args()
    n, ffs, nexp = a.hidden, a.ff, a.experts
    st = L.stream()
    jobs, P = big_jobs(a.tokens, nexp, a.topk, seed=1)
    down_jobs = jobs.copy()
    for jb in down_jobs:   # the down jobs read the pairs' h rows
        jb["y"][:jb["n"]] = jb["out"][:jb["n"]]
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x).view(np.uint8).reshape(-1).copy()).cuda()
    dj, djd = dev(jobs), dev(down_jobs)
    nj = torch.tensor([len(jobs), 0], dtype=torch.int32, device="cuda")
    keep = []
    if a.type == "q4k":
        gub = 2 * ffs * (n // 256) * 144
        wgu = torch.empty(nexp * gub, dtype=torch.uint8, device="cuda")
        L.call("fnx_synth_quant", L.Q4_K, wgu.data_ptr(), nexp * 2 * ffs * n, 0.02, 1, st)
        egu = L.Experts(L.Q4_K, 2 * ffs, n, wgu.data_ptr(), None, None, None, gub, 0)
        gu_bytes = nexp * gub
        src_cols = (ffs + 255) // 256 * 256
        blocks = torch.empty(nexp * n * (src_cols // 256) * 210, dtype=torch.uint8, device="cuda")
        L.call("fnx_synth_quant", L.Q6_K, blocks.data_ptr(), nexp * n * src_cols, 0.02, 2, st)
        units = nexp * n * (ffs // 32)
        planes = [torch.empty(units * k, dtype=torch.uint8, device="cuda") for k in (16, 8, 2, 2)]
        L.call("fnx_repack_q6k_units", blocks.data_ptr(), nexp * n, src_cols, 0, ffs, *[p.data_ptr() for p in planes], st)
        edn = L.Experts(L.Q6_K, n, ffs, *[p.data_ptr() for p in planes], n * (ffs // 32), 0)
        dn_bytes = units * 28
        keep += [wgu, planes]
        del blocks
    else:
        def q8(rows, cols, seed):
            b = torch.empty(nexp * rows * (cols // 32) * 34, dtype=torch.uint8, device="cuda")
            L.call("fnx_synth_quant", L.Q8_0, b.data_ptr(), nexp * rows * cols, 0.02, seed, st)
            q = torch.empty(nexp * rows * cols, dtype=torch.int8, device="cuda")
            d = torch.empty(nexp * rows * (cols // 32), dtype=torch.int16, device="cuda")
            L.call("fnx_repack_q8_0_split", b.data_ptr(), q.data_ptr(), d.data_ptr(), nexp * rows, cols, st)
            keep.extend([q, d])
            return L.Experts(L.Q8_0, rows, cols, q.data_ptr(), d.data_ptr(), None, None, rows * cols, rows * (cols // 32) * 2)
        egu, edn = q8(2 * ffs, n, 1), q8(n, ffs, 2)
        gu_bytes, dn_bytes = nexp * 2 * ffs * n * 34 // 32, nexp * n * ffs * 34 // 32
    x = torch.randn(a.tokens, n, device="cuda").half()
    gu = torch.zeros(P, 2 * ffs, device="cuda")
    h16 = torch.zeros(P, ffs, dtype=torch.int16, device="cuda")
    part = torch.zeros(P, n, device="cuda")
    steps = [
        ("gate_up", lambda: L.call("fnx_moe_gate_up_mma", C.byref(egu), dj.data_ptr(), nj.data_ptr(), len(jobs), x.data_ptr(), gu.data_ptr(), st),
         gu_bytes, 2.0 * P * 2 * ffs * n),
        ("swiglu_h16", lambda: L.call("fnx_swiglu_h16", gu.data_ptr(), ffs, P, h16.data_ptr(), st), P * ffs * 10, 0.0),
        ("down", lambda: L.call("fnx_moe_down_mma", C.byref(edn), djd.data_ptr(), nj.data_ptr(), len(jobs), h16.data_ptr(), part.data_ptr(), st),
         dn_bytes, 2.0 * P * n * ffs),
    ]
    res = {"workload": f"{a.tokens} tokens, top-{a.topk} of {nexp} experts, hidden {n}, ff {ffs}, {a.type}", "jobs": int(len(jobs)), "pairs": int(P)}
    stream = torch.cuda.current_stream()
    for name, f, nbytes, flops in steps:
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            f()
            e1.record(stream)
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts))
        res[name] = {"ms": round(ms, 4), "weight_GBps": round(nbytes / ms / 1e6, 1), "TFLOPps": round(flops / ms / 1e9, 1)}
    res["device_fault"] = int(L.load().fnx_device_fault())
    print(json.dumps(res))


if __name__ == "__main__":
    main()
