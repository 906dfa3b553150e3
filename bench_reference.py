"""The CPU arm of the benchmark: the verify window's arithmetic on the host cores.

The reference (johnfink8/sfnx) has no CPU implementation of this path and its CUDA kernels need an un-vendored
dependency to compile, so what is timed is the CPU oracle (oracle/, a plain-C restatement of the reference's kernel
arithmetic, OpenMP over experts / heads / vocabulary rows): kind "port".  A step is a bounded sample of one window of the
benchmark's workload: one FFN half, one DeltaNet mixer, one attention mixer at the configured context and the head, each
on seeded synthetic tensors of the workload's shapes and formats made with numpy (the timed arithmetic does not depend on
the values: every block is read and every product taken whatever the bits); the window's time is the sum scaled by the
layer counts.  Nothing here touches a GPU or the CUDA library.
"""
import json
import os
import time

T = 16


def _cores():
    return len(os.sched_getaffinity(0))


def _use_all_cores():
    """OpenMP reads its thread count when the oracle library is loaded: launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1 to their children, which would time one core; use the process's affinity mask instead."""
    os.environ["OMP_NUM_THREADS"] = str(_cores())


def synthetic_pieces(shape, ctx, seed=0, nexp_pool=160):
    """Seeded tensors of one layer of each kind at the workload's shapes.  The routed experts are a pool of `nexp_pool`
    matrices (a window touches about 120 - 140 distinct experts of the 512; the router's picks are folded into the pool)."""
    import numpy as np

    from oracle import binding as O

    rng = np.random.default_rng([seed, 3])
    n, ff, nq, nkv, hd = shape.n, shape.ff, shape.nq, shape.nkv, shape.hd
    f16 = lambda lo, hi, size: (rng.random(size, dtype=np.float32) * (hi - lo) + lo).astype(np.float16).view(np.uint16)   # noqa: E731

    def q8s(rows, cols):
        return rng.integers(-127, 128, size=(rows, cols), dtype=np.int8), f16(1e-4, 3e-4, (rows, cols // 32))

    p = {"x": rng.standard_normal((T, n)).astype(np.float32), "router": (rng.standard_normal((shape.nexp + 1, n)) * 0.02).astype(np.float32)}
    if shape.experts == "q4k":
        gu = rng.integers(0, 256, size=(nexp_pool, 2 * ff * (n // 256), 144), dtype=np.uint8)
        gu[:, :, 0:2] = np.frombuffer(np.float16(2e-4).tobytes(), np.uint8)   # d, dmin: finite f16 values
        gu[:, :, 2:4] = np.frombuffer(np.float16(1e-4).tobytes(), np.uint8)
        p["gu"] = gu.reshape(nexp_pool, -1)
        nu = ff // 32
        p["dn"] = (rng.integers(0, 256, size=(nexp_pool, n, nu, 16), dtype=np.uint8), rng.integers(0, 256, size=(nexp_pool, n, nu, 8), dtype=np.uint8),
                   rng.integers(-32, 32, size=(nexp_pool, n, nu, 2), dtype=np.int8), f16(1e-5, 3e-5, (nexp_pool, n, nu)))
    else:
        q, d = q8s(nexp_pool * 2 * ff, n)
        p["gu"] = (q.reshape(nexp_pool, 2 * ff, n), d.reshape(nexp_pool, 2 * ff, n // 32))
        q, d = q8s(nexp_pool * n, ff)
        p["dn"] = (q.reshape(nexp_pool, n, ff), d.reshape(nexp_pool, n, ff // 32))
    p["sh_gu"], p["sh_dn"] = q8s(2 * ff, n), q8s(n, ff)
    nk, nv = shape.nkh, shape.nvh
    ch = (2 * nk + nv) * 128
    p["qkvz"], p["ssm_out"] = q8s(ch + nv * 128, n), q8s(n, nv * 128)
    p["ab"] = (rng.standard_normal((2 * nv, n)) * 0.02).astype(np.float32)
    p["S"] = (rng.standard_normal((nv, 128, 128)) * 0.1).astype(np.float32)
    p["hist"] = rng.standard_normal((2, 3, ch)).astype(np.float32)
    p["conv"] = (rng.standard_normal((ch, 4)) * 0.5).astype(np.float32)
    vpk = nv // nk
    p["vmap"] = np.array([(v // vpk) | ((1 if v % vpk == 0 else 0) << 8) for v in range(nv)], np.int32)
    p["wq"], p["wk"], p["wv"], p["wo"] = q8s(nq * hd * 2, n), q8s(nkv * hd, n), q8s(nkv * hd, n), q8s(n, nq * hd)
    rows = (ctx + 64 + 3) // 4 * 4
    p["kc"] = rng.standard_normal((rows, nkv, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    p["vc"] = rng.standard_normal((rows, nkv, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
    p["head"] = q8s(shape.vocab, n)
    p["pool"] = nexp_pool
    O.build()
    return p


def sample(p, shape, ctx):
    """Times one layer of each kind on the CPU oracle.  Returns seconds per piece."""
    import numpy as np

    from oracle import binding as O

    n, topk, ff = shape.n, shape.topk, shape.ff
    x, t = p["x"], {}
    t0 = time.perf_counter()
    xq = O.quantize_q8_1(x)
    logits, topi, topw, jgu, jdn, nj = O.router_route(p["router"], x, topk)
    t["router"] = time.perf_counter() - t0
    for j in range(nj):   # the picked experts' matrices come from the pool
        jgu[j]["w"] = jdn[j]["w"] = j % p["pool"]
    t0 = time.perf_counter()
    if shape.experts == "q4k":
        gu = O.moe_gate_up_q4k(p["gu"], p["gu"].shape[1], jgu, nj, xq, n, 2 * ff, T * topk)
        part = O.moe_down_q6p(p["dn"], jdn, nj, gu, n, ff, T * topk)
    else:
        gu = O.moe_gate_up_q8(p["gu"][0], p["gu"][1], jgu, nj, xq, T, T * topk)
        part = O.moe_down_q8(p["dn"][0], p["dn"][1], jdn, nj, gu, T * topk)
    _, sh = O.shared_expert(p["sh_gu"][0], p["sh_gu"][1], p["sh_dn"][0], p["sh_dn"][1], xq, T)
    O.moe_combine(part, topw, sh, logits, T, n, topk)
    t["experts"] = time.perf_counter() - t0
    nk, nv = shape.nkh, shape.nvh
    S, hist = p["S"].copy(), p["hist"].copy()
    t0 = time.perf_counter()
    qkvz = O.q8s_gemv(p["qkvz"][0], p["qkvz"][1], xq, T)
    ab = O.gemv_f32(p["ab"], x, 4)
    yq, _, _, _ = O.gdn_core(qkvz, ab, hist, p["conv"], np.zeros(nv, np.float32), -np.ones(nv, np.float32), np.ones(128, np.float32), S,
                             np.array([ctx, 1], np.int32), nk, nv, p["vmap"], shape.eps, want_y32=False)
    O.q8s_gemv(p["ssm_out"][0], p["ssm_out"][1], yq, T)
    t["gdn_layer"] = time.perf_counter() - t0
    ones = np.ones(shape.hd, np.float32)
    t0 = time.perf_counter()
    qg = O.q8s_gemv(p["wq"][0], p["wq"][1], xq, T).reshape(T, shape.nq, 2 * shape.hd)
    k = O.q8s_gemv(p["wk"][0], p["wk"][1], xq, T).reshape(T, shape.nkv, shape.hd)
    v = O.q8s_gemv(p["wv"][0], p["wv"][1], xq, T).reshape(T, shape.nkv, shape.hd)
    O.attn_prep_append(qg, k, v, ones, ones, p["kc"], p["vc"], 0, 1, ctx, shape.eps, shape.rope_base, shape.nq, shape.nkv, shape.hd, shape.nrot)
    part = O.attn_partial(qg, p["kc"], p["vc"], 0, 1, ctx, shape.nq, shape.nkv, shape.hd)
    att = O.attn_merge([part], qg, shape.nq, shape.hd)
    O.q8s_gemv(p["wo"][0], p["wo"][1], O.quantize_q8_1(att.reshape(T, -1)), T)
    t["attn_layer"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    lg = O.q8s_gemv(p["head"][0], p["head"][1], xq, T)
    O.argmax(lg)
    t["head"] = time.perf_counter() - t0
    t["distinct_experts"] = nj
    return t


def window_seconds(t, kinds):
    return len(kinds) * (t["router"] + t["experts"]) + kinds.count(0) * t["gdn_layer"] + kinds.count(1) * t["attn_layer"] + t["head"]


SAMPLE = ("CPU oracle (C + OpenMP) on one FFN half, one DeltaNet mixer, one attention mixer at the workload's context and the head, on numpy-made "
          "tensors of the workload's shapes; window time = sum scaled by the layer counts")


def cpu_baseline(wl, shape, accepted_per_step):
    """The `cpu_baseline` object of this arm's line: one sample on this host's cores, the same numerator as the GPU's."""
    _use_all_cores()
    p = synthetic_pieces(shape, wl["ctx"])
    t = sample(p, shape, wl["ctx"])
    w = window_seconds(t, shape.kinds) * wl["nseq"]
    return {"value": round(accepted_per_step / w, 4), "unit": "tok/s", "cores": _cores(), "kind": "port", "sample": SAMPLE + ", once",
            "window_s": round(w, 3), "pieces_s": {k: round(v, 4) for k, v in t.items()}}


def main(args, rank, wl, emit=print):
    """`bench.py --impl reference`: rank 0 alone runs (the other ranks exit 0 without work)."""
    if rank != 0:
        return 0
    _use_all_cores()
    import bench
    from sfnx_b200.shapes import StackShape

    shape = StackShape(kinds=wl["kinds"], ctx=wl["ctx"], nexp=args.experts, vocab=args.vocab, experts=wl["experts"])
    p = synthetic_pieces(shape, wl["ctx"], seed=args.seed)
    repeats = args.repeats or (max(1, min(10, -(-200 // max(1, args.steps)))) if wl["name"] == "cfg2" else 1)
    nsteps = args.warmup + args.steps * repeats
    if wl["sampled"]:
        accepted, numerator = float(wl["nseq"]), "1 token per window and sequence (what rejection sampling emits at the least)"
    else:   # the numerator of the GPU arm: decided by the same Bernoulli draws
        _, n = bench.accepted_from_draws(args.seed, nsteps * wl["nseq"])
        accepted = sum(n[args.warmup * wl["nseq"]:]) / (args.steps * repeats)
        numerator = "mean accepted tokens per step of the same %d windows the GPU arm times (1 + leading true Bernoulli draws)" % (args.steps * repeats)
    times = []
    for i in range(args.warmup + args.steps):
        t = sample(p, shape, wl["ctx"])
        if i >= args.warmup:
            times.append(window_seconds(t, shape.kinds) * wl["nseq"])
    times.sort()
    w = times[len(times) // 2]
    val = round(accepted / w, 4)
    emit(json.dumps({
        "impl": "reference", "metric": bench.METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(w * 1e3, 2), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": bench.DTYPE, "data": "synthetic", "config": bench.workload_config(wl, shape, max(1, args.gpus)),
        "accepted_per_step": round(accepted, 3), "timing": {"statistic": "median step", "numerator": numerator},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": _cores(), "kind": "port", "sample": "each step: " + SAMPLE},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0
