"""The multi-GPU path's host logic on CPU: the partition rule against the reference's written-out two- and three-card
tables (src/card_split.hpp:31-39), and two gloo ranks that split the vocabulary, the K/V positions and the FF width the
way the GPUs do and exchange with the same collectives (all-reduce of partial sums, all-gather of attention partials and
of per-rank argmax), checked against the unsplit oracle."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import cases


def test_partition_rule_matches_reference_tables(fnx):
    lib = fnx.load()
    # the reference's shapes: 16 key heads, 48 value heads, FF 640
    K3 = [(0, 6), (5, 6), (10, 6)]
    V3 = [[0, 1, 2, 3, 4, 5, 16, 17, 18, 19, 20, 32, 33, 34, 35, 36], [6, 7, 8, 9, 10, 21, 22, 23, 24, 25, 26, 37, 38, 39, 40, 41],
          [11, 12, 13, 14, 15, 27, 28, 29, 30, 31, 42, 43, 44, 45, 46, 47]]
    F3 = [(0, 224), (224, 448), (448, 640)]
    K2 = [(0, 8), (8, 8)]
    V2 = [[0, 1, 2, 3, 4, 5, 6, 7, 16, 17, 18, 19, 20, 21, 22, 23, 32, 33, 34, 35, 36, 37, 38, 39],
          [8, 9, 10, 11, 12, 13, 14, 15, 24, 25, 26, 27, 28, 29, 30, 31, 40, 41, 42, 43, 44, 45, 46, 47]]
    F2 = [(0, 320), (320, 640)]
    for n, K, V, F in ((3, K3, V3, F3), (2, K2, V2, F2)):
        for c in range(n):
            assert (lib.fnx_khead_first(16, 48, n, c), lib.fnx_khead_count(16, 48, n, c)) == K[c]
            assert [v for v in range(48) if lib.fnx_vhead_card(16, 48, n, v) == c] == V[c]
            assert (lib.fnx_ff_lo(640, n, c), lib.fnx_ff_lo(640, n, c + 1)) == F[c]
    # the benchmark's FF 768 over 2 / 4 / 8 GPUs: 384 / 192 / 96 each, every value head on one GPU beside its key head
    for n in (2, 4, 8):
        assert [lib.fnx_ff_lo(768, n, c + 1) - lib.fnx_ff_lo(768, n, c) for c in range(n)] == [768 // n] * n
        for c in range(n):
            mine = [v for v in range(48) if lib.fnx_vhead_card(16, 48, n, v) == c]
            assert len(mine) == 48 // n
            k0, kc = lib.fnx_khead_first(16, 48, n, c), lib.fnx_khead_count(16, 48, n, c)
            assert all(k0 <= v % 16 < k0 + kc for v in mine)


def _rank(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import binding as O
        from sfnx_b200.window import merge_best, vocab_slice

        rng = np.random.default_rng(3)   # the same inputs on every rank
        T, vocab = 5, 1003
        logits = rng.standard_normal((T, vocab)).astype(np.float32)
        logits[1, [10, 700]] = 9.0   # a tie across the slices: the lower rank's token
        v0, rows = vocab_slice(vocab, world, rank)
        bv, bi, _ = O.argmax(np.ascontiguousarray(logits[:, v0:v0 + rows]), v0)
        allv = [torch.zeros(T) for _ in range(world)]
        alli = [torch.zeros(T, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(allv, torch.from_numpy(bv))
        dist.all_gather(alli, torch.from_numpy(bi))
        got = merge_best(torch.stack(allv), torch.stack(alli))
        want = [int(np.flatnonzero(r == r.max())[0]) for r in logits]
        assert got == want, (got, want)
        # attention: this rank's positions only, partials gathered, merged for the heads it owns
        c = cases.attn_case(T=3, ctx=77, nq=4, nkv=2, hd=128, ncard=world, seed=4)
        qg, k = c["qg"].copy(), c["k"].copy()
        kc, vc = c["kc"][rank].copy(), c["vc"][rank].copy()
        O.attn_prep_append(qg, k, c["v"], c["qn"], c["kn"], kc, vc, rank, world, c["pos0"], c["eps"], c["rope_base"], 4, 2, 128)
        part = torch.from_numpy(O.attn_partial(qg, kc, vc, rank, world, c["pos0"], 4, 2, 128))
        parts = [torch.zeros_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        out = O.attn_merge([p.numpy() for p in parts], qg, 4, 128)
        ref = cases.attn_oracle(c)["out"]
        own = 4 // world
        assert np.array_equal(out[:, rank * own:(rank + 1) * own], ref[:, rank * own:(rank + 1) * own])
        # experts split by FF width: the ranks' partial down outputs sum to the unsplit layer's (to f32 rounding)
        x = rng.standard_normal((4, 512)).astype(np.float32)
        full = cases.moe_weights(n=512, nexp=32, ffs=256, seed=9)
        ref_moe = cases.moe_oracle(full, x, 4)
        ff0, ffs = 128 * rank, 128
        w = dict(full, ffs=ffs)
        rb = 512 // 256 * 144
        w["gu_q4k"] = np.ascontiguousarray(full["gu_q4k"].reshape(32, 2, 256, rb)[:, :, ff0:ff0 + ffs].reshape(32, -1))
        planes = [O.q6k_to_planes(full["dn_q6k"][e], 512, 256, ff0, ffs) for e in range(32)]
        w["dn_planes"] = tuple(np.stack([p[i] for p in planes]) for i in range(4))
        r = {}
        r["xq"] = O.quantize_q8_1(x)
        logits_r, topi, topw, jgu, jdn, nj = O.router_route(w["router"], x, 4)
        assert np.array_equal(topi, ref_moe["topi"])   # the router is replicated: identical routing everywhere
        gu = O.moe_gate_up_q4k(w["gu_q4k"], w["gu_q4k"].shape[1], jgu, nj, r["xq"], 512, 2 * ffs, 16)
        part_dn = torch.from_numpy(O.moe_down_q6p(w["dn_planes"], jdn, nj, gu, 512, ffs, 16))
        dist.all_reduce(part_dn)
        assert np.allclose(part_dn.numpy(), ref_moe["part"], rtol=2e-2, atol=2e-3)   # each slice quantises its own h
        q.put((rank, "ok"))
    except Exception as e:   # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(res) == [(r, "ok") for r in range(world)], res
