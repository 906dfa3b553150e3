"""Verify-window benchmark: accepted tok/s at draft length 16 on N B200s, with the roofline of the dominant kernel and
the CPU oracle timed beside it.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Workload (N = 1): the 8-layer synthetic stack (6 Gated DeltaNet + 2 attention layers, every layer with the 512-expert
top-10 + shared-expert FFN in Q4_K/Q6_K, Q8_0 dense projections and head), batch 1, 32 768-token fp16 K/V context, one
window of 16 rows (the last committed token + 15 drafts) per step, greedy prefix acceptance, rollback of the rejected
rows.  Drafts are uniform over the vocabulary, overwritten with the greedy continuation where a Bernoulli(0.8) draw per
position is true; they are prepared before the timed region (the draft model is not part of the measured path) and the
timed region replays the recorded windows from the saved initial state.  N > 1: the same model split across the GPUs
(experts by FF width, DeltaNet by value heads, K/V by position, vocabulary by ranges) with NCCL all-reduce / all-gather
between the stages: strong scaling.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=8, help="stack depth (8 = the benchmark configuration)")
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--experts", type=int, default=512, help="routed experts (512 = the benchmark configuration; fewer for small profiling runs)")
    ap.add_argument("--vocab", type=int, default=151936, help="vocabulary (151936 = the benchmark configuration)")
    ap.add_argument("--expert-type", default="q4k", choices=["q4k", "q8_0"],
                    help="routed experts: q4k (Q4_K gate|up + Q6_K down, the benchmark configuration) or q8_0 (the all-Q8_0 configuration)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="enqueue every window call by call instead of replaying a CUDA graph")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx = int(f[1])
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(shape, distinct_experts, ctx):
    """Bytes a window must move once (weights, K/V, state + checkpoints, logits), per kernel family, whole model."""
    n, ff = shape.n, shape.ff
    q8 = lambda r, c: r * c * 34 // 32  # noqa: E731
    gu = 2 * ff * (n // 256) * 144 if shape.experts == "q4k" else q8(2 * ff, n)
    dn = n * (ff // 256) * 210 if shape.experts == "q4k" else q8(n, ff)
    state = shape.nvh * 128 * 128 * 4
    b = {"moe_gate_up": gu, "moe_down": dn, "router": (shape.nexp + 1) * n * 4, "shared": q8(2 * ff, n) + q8(n, ff),
         "gdn_core": 17 * state, "qkvz": q8((2 * shape.nkh + 2 * shape.nvh) * 128, n), "ssm_out": q8(n, shape.nvh * 128),
         "wq": q8(shape.nq * shape.hd * 2, n), "wkv": 2 * q8(shape.nkv * shape.hd, n), "wo": q8(n, shape.nq * shape.hd),
         "attn_kv": ctx * shape.nkv * shape.hd * 2 * 2, "head": q8(shape.vocab, n) + 16 * shape.vocab * 4}
    return b


def workload_config(shape, kinds, ctx, world):
    """The `config` object of the result line: the same for this arm and for the CPU arm."""
    b = algorithmic_bytes(shape, 0, ctx)
    experts_all = shape.nexp * (b["moe_gate_up"] + b["moe_down"])
    resident = (len(kinds) * (experts_all + b["router"] + b["shared"]) + kinds.count(0) * (b["qkvz"] + b["ssm_out"] + b["gdn_core"]) +
                kinds.count(1) * (b["wq"] + b["wkv"] + b["wo"] + b["attn_kv"]) + b["head"])
    d_exp = shape.nexp * (1.0 - (1.0 - shape.topk / shape.nexp) ** 16)   # expected distinct experts of 16 rows
    window = (len(kinds) * (d_exp * (b["moe_gate_up"] + b["moe_down"]) + b["router"] + b["shared"]) +
              kinds.count(0) * (b["qkvz"] + b["ssm_out"] + b["gdn_core"]) + kinds.count(1) * (b["wq"] + b["wkv"] + b["wo"] + b["attn_kv"]) + b["head"])
    return {"workload": "cfg2: %d-layer stack (%d DeltaNet + %d attention), batch 1, ctx %d, T=16 rows (1 committed + 15 drafts), "
                        "greedy acceptance, Bernoulli(0.8) drafts" % (len(kinds), kinds.count(0), kinds.count(1), ctx),
            "hidden": shape.n, "experts": shape.nexp, "expert_type": shape.experts, "topk": shape.topk, "ff": shape.ff, "vocab": shape.vocab,
            "l2": "inputs larger than L2, no flush: %.1f GB of weights, state and K/V resident, about %.1f GB of them read per window "
                  "(126 MB of L2)" % (resident / 1e9, window / 1e9),
            "parallelism": "tp%d (FF blocks / value heads / KV positions / vocabulary)" % world}


_REAL_STDOUT = None


def emit(line):
    """The result line, on the process's original stdout."""
    os.write(_REAL_STDOUT if _REAL_STDOUT is not None else 1, (line + "\n").encode())


def main():
    args = parse()
    import numpy as np
    import torch
    import torch.distributed as dist

    # stdout carries the one JSON line and nothing else: whatever libraries print there (NCCL's version line) goes to
    # stderr, and the line is written to the saved descriptor at the end
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        import bench_reference

        return bench_reference.main(args, rank, world, emit, workload_config)
    assert world == args.gpus, "launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus)
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    from sfnx_b200 import lib as L
    from sfnx_b200.window import StackShape, SyntheticStack, WindowRunner

    L.load()
    kinds = [1 if (i % 4) == 3 else 0 for i in range(args.layers)]
    T = L.MAXT
    shape = StackShape(kinds=kinds, ctx=args.ctx, kv_slack=(args.warmup + args.steps + 2) * T, nexp=args.experts, vocab=args.vocab,
                       experts=args.expert_type)
    t_build = time.time()
    stack = SyntheticStack(shape, ncard=world, card=rank, seed=args.seed, device="cuda:%d" % local)
    runner = WindowRunner(stack, T, group=group, graph=not args.no_graph)
    t_build = time.time() - t_build
    lib = L.load()

    # ---- drafting pass (untimed): the rows of every step, recorded
    rng = np.random.default_rng(args.seed + 1)
    state0 = stack.save_state()
    nsteps = args.warmup + args.steps
    rec, pos, tag, x = [], args.ctx, 1, int(rng.integers(0, shape.vocab))
    out_c = (C.c_int * T)()
    rows_c = (C.c_int * T)()
    for s in range(nsteps):
        draws = rng.random(T - 1) < 0.8
        rows = [x] + [int(v) for v in rng.integers(0, shape.vocab, T - 1)]
        saved = stack.save_state()
        for _ in range(T):   # rows[j + 1] = the greedy token after row j wherever the leading draws are true
            out = runner.window(rows, pos, tag)
            stack.load_state(saved)
            changed = False
            for j in range(T - 1):
                if not draws[j]:
                    break
                if rows[j + 1] != out[j]:
                    rows[j + 1] = out[j]
                    changed = True
                    break
            if not changed:
                break
        out = runner.window(rows, pos, tag)
        rows_c[:], out_c[:] = rows, out
        n = lib.fnx_accept_greedy(rows_c, out_c, T)
        runner.commit(n, tag)
        rec.append((rows, pos, tag, n, out))
        pos, tag, x = pos + n, tag + 1, out[n - 1]
    torch.cuda.synchronize()
    accepted = sum(r[3] for r in rec[args.warmup:])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- device-timed replay: ids and (position, tag) of every step already in HBM, no host read-back
    d_ids = torch.tensor([r[0] for r in rec], dtype=torch.int32, device=stack.dev)
    d_ctl = torch.tensor([[r[1], r[2]] for r in rec], dtype=torch.int32, device=stack.dev)
    clocks = ClockSampler(local)

    def device_step(i):
        with torch.cuda.stream(runner.stream):
            runner.ids[:T].copy_(d_ids[i], non_blocking=True)
            runner.ctl_in.copy_(d_ctl[i], non_blocking=True)
            runner.launch()
        runner.commit(rec[i][3], rec[i][2])

    stack.load_state(state0)
    clocks.start()
    for i in range(args.warmup):
        device_step(i)
    barrier()
    lib.fnx_window_kernel_count(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(runner.stream)
    for i in range(args.warmup, nsteps):
        device_step(i)
    e1.record(runner.stream)
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))

    # ---- end-to-end replay through the runner's public call: host token ids in, host argmax tokens out, acceptance on
    # the host, rollback
    stack.load_state(state0)
    for i in range(args.warmup):
        out = runner.window(rec[i][0], rec[i][1], rec[i][2])
        runner.commit(rec[i][3], rec[i][2])
    barrier()
    t0 = time.perf_counter()
    e2e_accepted = 0
    for i in range(args.warmup, nsteps):
        rows, p, tg, n_rec, out_rec = rec[i]
        out = runner.window(rows, p, tg)
        rows_c[:], out_c[:] = rows, out
        n = lib.fnx_accept_greedy(rows_c, out_c, T)
        runner.commit(n, tg)
        e2e_accepted += n
        assert n == n_rec and out[:n] == out_rec[:n], "replay diverged from the recorded windows at step %d" % i
    barrier()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    clk = clocks.stop()

    # ---- per-kernel timing of the same windows enqueued call by call (no graph): CUDA events around every C ABI call
    stack.load_state(state0)
    eager = WindowRunner(stack, T, group=group, graph=False)
    per = {}
    ntr = min(8, args.steps)
    for i in range(args.warmup, args.warmup + ntr):
        rows, p, tg, n_rec, _ = rec[i]
        eager.h_ids[:T] = torch.as_tensor(rows, dtype=torch.int32)
        eager.h_ctl[0], eager.h_ctl[1] = p, tg
        with torch.cuda.stream(eager.stream):
            eager.ids.copy_(eager.h_ids, non_blocking=True)
            eager.ctl_in.copy_(eager.h_ctl, non_blocking=True)
        eager.stream.synchronize()
        lib.fnx_trace_begin()
        eager.launch()
        eager.stream.synchronize()
        ms, lay, names = (C.c_float * 4096)(), (C.c_int * 4096)(), (C.c_char_p * 4096)()
        k = lib.fnx_trace_end(ms, lay, names, 4096)
        for j in range(k):
            per.setdefault(names[j].decode(), []).append(ms[j])
        # distinct experts of this window's layers: read the job counts back (the last layer's is left in the workspace)
        eager.commit(n_rec, tg)
    torch.cuda.synchronize()
    kernels_per_window = lib.fnx_window_kernel_count(1) // max(1, ntr)

    # distinct experts per layer, measured on one window: run stage by stage and read njobs
    # (E[D] = 512 (1 - (1 - 10/512)^16) = 138.6 for independent uniform picks)
    algo = algorithmic_bytes(shape, 0, args.ctx)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    D = distinct_experts(stack, runner, rec[args.warmup], T)
    gu_ms = float(np.mean(per["moe_gate_up"])) if "moe_gate_up" in per else None
    gu_bytes = D * algo["moe_gate_up"] / world
    roof = None
    if gu_ms:
        ach = gu_bytes / (gu_ms * 1e-3) / 1e9
        roof = {"kernel": "k_moe_gu_q4k" if shape.experts == "q4k" else "k_moe_gu_q8", "bound": "hbm", "achieved": round(ach, 1), "peak": peak_gbs, "unit": "GB/s",
                # dram read + write bytes of one launch: ncu on a 128-expert case measured 1.00 x the algorithmic bytes
                # read (each selected expert's rows once) + the output rows written; scaled to this launch by D
                "frac": round(ach / peak_gbs, 4), "traffic": int(gu_bytes + T * shape.topk * 2 * (shape.ff // world) * 4),
                "peak_source": "measured" if peaks else "fallback",
                "bytes_per_launch": int(gu_bytes), "us_per_launch": round(gu_ms * 1e3, 2), "distinct_experts": D}
    breakdown = {k: round(float(np.mean(v)) * 1e3, 2) for k, v in sorted(per.items())}

    result = {
        "metric": "accepted tok/s @ draft len 16", "value": round(accepted / (dev_ms * 1e-3), 2), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int4/int6/int8 dot products, f32 accumulate", "data": "synthetic",
        "config": workload_config(shape, kinds, args.ctx, world),
        "accepted_per_window": round(accepted / args.steps, 3),
        "e2e": {"value": round(e2e_accepted / (e2e_ms * 1e-3), 2), "unit": "tok/s", "ms_per_step": round(e2e_ms / args.steps, 4),
                "h2d_bytes_per_step": runner.h2d_bytes + runner.job_bytes, "d2h_bytes_per_step": runner.d2h_bytes},
        "gpu_launches": int(kernels_per_window * args.steps), "kernels_per_window": int(kernels_per_window),
        "clocks": clk, "roofline": roof, "kernel_us": breakdown, "build_s": round(t_build, 1),
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline and shape.experts == "q4k":
        import bench_reference

        result["cpu_baseline"] = bench_reference.cpu_baseline(stack, runner, rec[args.warmup], shape, accepted / args.steps)
    if rank == 0:
        emit(json.dumps(result))
    sys.stdout.flush()
    if world > 1:
        # leave without tearing the communicator down: its destruction can wait for ever on the captured graphs' kernels
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


def distinct_experts(stack, runner, step, T):
    """Mean number of distinct routed experts per layer in one recorded window (the job counts, read back per layer)."""
    import torch

    from sfnx_b200 import lib as L

    rows, pos, tag, n_rec, _ = step
    saved = stack.save_state()
    eager = runner
    counts = []
    with torch.cuda.stream(runner.stream):
        runner.ids[:T].copy_(torch.tensor(rows, dtype=torch.int32, device=stack.dev))
        runner.ctl_in.copy_(torch.tensor([pos, tag], dtype=torch.int32, device=stack.dev))
        runner.ctl.copy_(runner.ctl_in)
        st = torch.cuda.current_stream().cuda_stream
        L.call("fnx_embed_rows", stack.embed.data_ptr(), runner.ids.data_ptr(), runner.x.data_ptr(), T, stack.shape.n, st)
        # the job count lives at a fixed place of the workspace; find it through the layout: run every stage and read it
        # after each FFN stage (kind 1 of `after` follows both mixer and FFN stages, so read after every stage)
        import ctypes as C

        nj_prev = None
        for i in range(runner.nstages):
            L.call("fnx_window_stage", C.byref(stack.cfg), stack.layers, C.byref(stack.head), stack.ws.data_ptr(), T, i, st)
            if stack.ncard > 1:
                if runner.after[i] == 1:
                    runner.dist.all_reduce(runner.bo, group=runner.group)
                elif runner.after[i] == 2:
                    per = runner.partials.numel() // stack.ncard
                    runner.dist.all_gather_into_tensor(runner.partials, runner.partials[stack.card * per:(stack.card + 1) * per],
                                                       group=runner.group)
            nj = int(stack.buf(9, torch.int32, 2)[0].item())
            if nj != nj_prev or True:
                counts.append(nj)
            nj_prev = nj
    torch.cuda.synchronize()
    stack.load_state(saved)
    # njobs changes only at FFN stages; keep the value seen right after each FFN stage
    ffn = []
    s = 0
    for l, kind in enumerate(stack.shape.kinds):
        s += 2 if kind == 1 else 1
        ffn.append(counts[s])
        s += 1
    return sum(ffn) / len(ffn)


if __name__ == "__main__":
    main()
