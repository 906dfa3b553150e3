"""The CPU arm of the benchmark: the verify window's arithmetic on the host cores.

The reference (johnfink8/sfnx) has no CPU implementation of this path and its CUDA kernels need an un-vendored
dependency to compile, so what is timed is the CPU oracle (oracle/, a plain-C restatement of the reference's kernel
arithmetic, OpenMP over experts / heads / vocabulary rows): kind "port".  A step is a bounded sample of one window of the
benchmark's workload: one FFN half, one DeltaNet mixer, one attention mixer at the configured context and the head,
each on the synthetic stack's own tensors; the window's time is the sum scaled by the layer counts.
"""
import json
import os
import time


def _np(t, dtype=None):
    a = t.detach().cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def _sample(stack, shape, seed=0):
    """Times one layer of each kind on the CPU oracle.  Returns seconds per piece."""
    import numpy as np

    from oracle import binding as O

    O.build()
    rng = np.random.default_rng(seed)
    T, n, topk = 16, shape.n, shape.topk
    kinds = shape.kinds
    lg, la = kinds.index(0), kinds.index(1)
    x = rng.standard_normal((T, n)).astype(np.float32)
    t = {}
    # ---- FFN half of layer lg (its own router, so the picks are the model's; only the picked experts are fetched)
    router = _np(stack.named[(lg, "router")])
    t0 = time.perf_counter()
    xq = O.quantize_q8_1(x)
    logits, topi, topw, jgu, jdn, nj = O.router_route(router, x, topk)
    t["router"] = time.perf_counter() - t0
    experts = [int(j["w"]) for j in jgu[:nj]]
    idx = stack.named[(lg, "gate_up")].new_tensor(experts, dtype=__import__("torch").long)
    gu_w = _np(stack.named[(lg, "gate_up")][idx])
    planes = tuple(_np(p[idx]) for p in stack.named[(lg, "down")])
    planes = (planes[0], planes[1], planes[2].view(np.int8), planes[3].view(np.uint16))
    for j in range(nj):
        jgu[j]["w"] = jdn[j]["w"] = j
    sgu = tuple(_np(a) for a in stack.named[(lg, "sh_gate_up")])
    sdn = tuple(_np(a) for a in stack.named[(lg, "sh_down")])
    t0 = time.perf_counter()
    gu = O.moe_gate_up_q4k(gu_w, gu_w.shape[1], jgu, nj, xq, n, 2 * stack.ffs, T * topk)
    part = O.moe_down_q6p(planes, jdn, nj, gu, n, stack.ffs, T * topk)
    _, sh = O.shared_expert(sgu[0], sgu[1].view(np.uint16), sdn[0], sdn[1].view(np.uint16), xq, T)
    O.moe_combine(part, topw, sh, logits, T, n, topk)
    t["experts"] = time.perf_counter() - t0
    # ---- DeltaNet mixer of layer lg
    qkvz_w = tuple(_np(a) for a in stack.named[(lg, "qkvz")])
    out_w = tuple(_np(a) for a in stack.named[(lg, "ssm_out")])
    ab_w = _np(stack.named[(lg, "ab")])
    S, hist = _np(stack.named[(lg, "S")]).copy(), _np(stack.named[(lg, "hist")]).copy()
    conv, vmap = _np(stack.named[(lg, "conv")]), _np(stack.named[(lg, "vmap")])
    nk, nv = stack.nk, stack.nv
    t0 = time.perf_counter()
    qkvz = O.q8s_gemv(qkvz_w[0], qkvz_w[1].view(np.uint16), xq, T)
    ab = O.gemv_f32(ab_w, x, 4)
    yq, _, _, _ = O.gdn_core(qkvz, ab, hist, conv, np.zeros(nv, np.float32), -np.ones(nv, np.float32), np.ones(128, np.float32), S,
                             np.array([shape.ctx, 1], np.int32), nk, nv, vmap, shape.eps, want_y32=False)
    O.q8s_gemv(out_w[0], out_w[1].view(np.uint16), yq, T)
    t["gdn_layer"] = time.perf_counter() - t0
    # ---- attention mixer of layer la
    wq, wk, wv, wo = (tuple(_np(a) for a in stack.named[(la, k)]) for k in ("wq", "wk", "wv", "wo"))
    kc, vc = _np(stack.named[(la, "kc")], np.uint16).copy(), _np(stack.named[(la, "vc")], np.uint16).copy()
    ones = np.ones(shape.hd, np.float32)
    t0 = time.perf_counter()
    qg = O.q8s_gemv(wq[0], wq[1].view(np.uint16), xq, T).reshape(T, shape.nq, 2 * shape.hd)
    k = O.q8s_gemv(wk[0], wk[1].view(np.uint16), xq, T).reshape(T, shape.nkv, shape.hd)
    v = O.q8s_gemv(wv[0], wv[1].view(np.uint16), xq, T).reshape(T, shape.nkv, shape.hd)
    O.attn_prep_append(qg, k, v, ones, ones, kc, vc, stack.card, stack.ncard, shape.ctx, shape.eps, shape.rope_base, shape.nq, shape.nkv,
                       shape.hd, shape.nrot)
    part = O.attn_partial(qg, kc, vc, stack.card, stack.ncard, shape.ctx, shape.nq, shape.nkv, shape.hd)
    att = O.attn_merge([part], qg, shape.nq, shape.hd)
    aq = O.quantize_q8_1(att.reshape(T, -1))
    O.q8s_gemv(wo[0], wo[1].view(np.uint16), aq, T)
    t["attn_layer"] = time.perf_counter() - t0
    # ---- head
    hw = tuple(_np(a) for a in stack.named[(len(kinds), "output")])
    t0 = time.perf_counter()
    logits = O.q8s_gemv(hw[0], hw[1].view(np.uint16), xq, T)
    O.argmax(logits)
    t["head"] = time.perf_counter() - t0
    return t


def window_seconds(t, kinds):
    return len(kinds) * (t["router"] + t["experts"]) + kinds.count(0) * t["gdn_layer"] + kinds.count(1) * t["attn_layer"] + t["head"]


def cpu_baseline(stack, runner, step, shape, accepted_per_window):
    cores = len(os.sched_getaffinity(0))
    t = _sample(stack, shape)
    w = window_seconds(t, shape.kinds)
    return {"value": round(accepted_per_window / w, 4), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": "CPU oracle (C + OpenMP) on one FFN half, one DeltaNet mixer, one attention mixer (ctx %d) and the head of the same "
                      "stack, once each; window time = sum scaled by the layer counts (%d FFN, %d DeltaNet, %d attention)" %
                      (shape.ctx, len(shape.kinds), shape.kinds.count(0), shape.kinds.count(1)),
            "window_s": round(w, 3), "pieces_s": {k: round(v, 4) for k, v in t.items()}}


def main(args, rank, world, emit=print, workload_config=None):
    """`bench.py --impl reference`: rank 0 alone runs (the other ranks exit 0 without work)."""
    if rank != 0:
        return 0
    import torch

    from sfnx_b200.window import StackShape, SyntheticStack

    kinds = [1 if (i % 4) == 3 else 0 for i in range(args.layers)]
    full = StackShape(kinds=kinds, ctx=args.ctx)
    # a two-layer stack (one DeltaNet, one attention) holds every tensor the sample reads; the inputs are generated on
    # the device and copied to the host, the timed arithmetic runs on the host cores only
    small = StackShape(kinds=[0, 1], ctx=args.ctx)
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    stack = SyntheticStack(small, ncard=1, card=0, seed=args.seed)
    cores = len(os.sched_getaffinity(0))
    accepted = 1 + sum(0.8 ** k for k in range(1, 16))   # expected tokens per window under Bernoulli(0.8) drafts
    times = []
    for i in range(args.warmup + args.steps):
        t = _sample(stack, small, seed=i)
        if i >= args.warmup:
            times.append(window_seconds(t, full.kinds))
    w = sum(times) / len(times)
    val = round(accepted / w, 4)
    emit(json.dumps({
        "impl": "reference", "metric": "accepted tok/s @ draft len 16", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(w * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int4/int6/int8 dot products, f32 accumulate", "data": "synthetic",
        "config": workload_config(full, kinds, args.ctx, max(1, args.gpus)),
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": "each step: CPU oracle on one FFN half, one DeltaNet mixer, one attention mixer and the head, scaled "
                                   "by the layer counts"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
    return 0
