"""GPU parity of the peer-memory sum across GPUs against the CPU oracle's ring order, on ONE GPU: the "peers" are other
buffers of the same device whose addends and flags are in place before the launch, so no launch waits for another.  A
second case leaves one peer's flag unset with a short poll limit and checks that the kernel gives up with error bit 1."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ring(L, G, torch, n, rank, slots, pads, state, limit, ll=None, ll_count=0):
    r = L.Ring()
    r.nrank, r.rank, r.state, r.spin_limit = n, rank, state.data_ptr(), limit
    for p in range(2):
        for k in range(n):
            r.slot[p][k] = slots[k][p].data_ptr()
            if ll is not None:
                r.ll[p][k] = ll[k][p].data_ptr()
    for k in range(n):
        r.pad[k] = pads[k].data_ptr()
    r.ll_count = ll_count
    return r


def _ll_areas(G, torch, n, rank, count, epoch, words_of):
    """The GPUs' receive areas [GPU][parity] of n runs of `count` 8-byte words, as they are when the emulated peers have sent
    exchange `epoch`: run s of this GPU's area of the epoch's parity holds words_of(s) (uint32 values) with the epoch in
    the upper halves; everything else is zero (the peers' areas receive this GPU's stores)."""
    areas = [[torch.zeros(n * count, dtype=torch.int64, device=G.DEV) for _ in range(2)] for _ in range(n)]
    mine = areas[rank][epoch % 2].view(n, count)
    for s_ in range(n):
        if s_ == rank:
            continue
        w = np.ascontiguousarray(words_of(s_)).reshape(-1).view(np.uint32).astype(np.int64) | (np.int64(epoch) << 32)
        mine[s_, :w.size] = G.dev(w)
    return areas


def _ll_sent(G, area, rank, count, nwords):
    """What this GPU stored into a peer's area: (values as uint32, exchange numbers)."""
    w = G.host(area.view(-1, count)[rank, :nwords])
    return (w & 0xffffffff).astype(np.uint32), (w >> 32).astype(np.uint32)


@pytest.mark.parametrize("n,T,row_len", [(2, 16, 3072), (4, 5, 1024), (8, 16, 3072), (3, 2, 20)])
def test_ring_sum_matches_ring_order(oracle, n, T, row_len):
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(n * 100 + T)
    xs = [(rng.standard_normal((T, row_len)) * 10 ** rng.uniform(-3, 3, (T, row_len))).astype(np.float32) for _ in range(n)]
    ref = oracle.ring_sum(xs)
    for epoch in (1, 2):   # both parities of the slots
        for rank in range(n):
            # every rank's addend already in its slot, every flag at the epoch: what the peers would have done
            slots = [[G.dev(xs[k]) if p == epoch % 2 else G.zeros((T, row_len)) for p in range(2)] for k in range(n)]
            pads = [torch.full((16,), epoch, dtype=torch.int32, device=G.DEV) for _ in range(n)]
            state = torch.tensor([epoch - 1, 0, 0, 0], dtype=torch.int32, device=G.DEV)
            err = G.zeros(1, torch.int32)
            x = G.dev(xs[rank])
            ring = _ring(L, G, torch, n, rank, slots, pads, state, 1 << 20)
            L.call("fnx_ring_sum", x.data_ptr(), T, row_len, C.byref(ring), err.data_ptr(), L.stream())
            G.sync()
            assert int(G.host(err)[0]) == 0
            assert np.array_equal(G.host(x).view(np.uint32), ref.view(np.uint32)), (n, rank, epoch)
            assert G.host(state).tolist()[:3] == [epoch, 0, 0]


def test_ring_sum_gives_up_when_a_peer_never_signals():
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    n, T, row_len = 2, 4, 256
    slots = [[G.zeros((T, row_len)) for _ in range(2)] for _ in range(n)]
    pads = [G.zeros(16, torch.int32) for _ in range(n)]   # nothing ever sets a flag
    state, err = G.zeros(4, torch.int32), G.zeros(1, torch.int32)
    x = G.dev(np.ones((T, row_len), np.float32))
    ring = _ring(L, G, torch, n, 0, slots, pads, state, 200)   # 200 polls: the wait runs out in well under a millisecond
    L.call("fnx_ring_sum", x.data_ptr(), T, row_len, C.byref(ring), err.data_ptr(), L.stream())
    G.sync()
    assert int(G.host(err)[0]) & 1 == 1
    y = G.zeros(8)   # the context is still usable
    y.fill_(3.0)
    G.sync()
    assert float(G.host(y)[0]) == 3.0


@pytest.mark.parametrize("n,T,width,moe", [(1, 16, 3072, True), (1, 5, 512, False), (2, 16, 3072, True), (8, 16, 3072, False), (4, 3, 1024, True)])
def test_boundary_rows_equals_the_separate_steps(n, T, width, moe):
    """The fused boundary (experts' rows weighted and added | the half's rows, summed across the GPUs, x += sum, RMS norm,
    q8_1) against fnx_moe_combine -> fnx_ring_sum -> fnx_rms_norm_rows on the same buffers, bit for bit; the peers of one
    GPU are emulated as in the ring test above (their addends and flags in place before the launch)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(7 * n + T)
    topk, nexp = 10, 32
    x0 = rng.standard_normal((T, width)).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    peers = [(rng.standard_normal((T, width)) * 10 ** rng.uniform(-2, 2, (T, width))).astype(np.float32) for _ in range(n)]
    part = rng.standard_normal((T * topk, width)).astype(np.float32)
    topw = rng.random((T, topk)).astype(np.float32)
    sh = rng.standard_normal((T, width)).astype(np.float32)
    logits = rng.standard_normal((T, nexp + 1)).astype(np.float32)
    st = L.stream()
    for rank in range(n):
        dpart, dtopw, dsh, dlog, dw = G.dev(part), G.dev(topw), G.dev(sh), G.dev(logits), G.dev(wn)
        # ---- the separate steps
        bo = G.zeros((T, width))
        if moe:
            L.call("fnx_moe_combine", dpart.data_ptr(), dtopw.data_ptr(), dsh.data_ptr(), dlog.data_ptr(), nexp, bo.data_ptr(), T, width, topk, st)
        else:
            bo.copy_(G.dev(peers[rank]))
        G.sync()
        mine = G.host(bo).copy()   # this GPU's addend; the emulated peers hold theirs
        adds = [mine if k == rank else peers[k] for k in range(n)]

        def ring_for(epoch):
            slots = [[G.dev(adds[k]) if p == epoch % 2 else G.zeros((T, width)) for p in range(2)] for k in range(n)]
            pads = [torch.full((16,), epoch, dtype=torch.int32, device=G.DEV) for _ in range(n)]
            state = torch.tensor([epoch - 1, 0, 0, 0], dtype=torch.int32, device=G.DEV)
            ll = _ll_areas(G, torch, n, rank, T * width, epoch, lambda k: adds[k])
            return _ring(L, G, torch, n, rank, slots, pads, state, 1 << 20, ll, T * width), (slots, pads, state, ll)

        err = G.zeros(1, torch.int32)
        ring, keep = ring_for(1)
        L.call("fnx_ring_sum", bo.data_ptr(), T, width, C.byref(ring), err.data_ptr(), st)
        x1, y1, q1 = G.dev(x0), G.zeros((T, width)), G.zeros(T * (width // 32) * 36, torch.uint8)
        L.call("fnx_rms_norm_rows", x1.data_ptr(), bo.data_ptr(), dw.data_ptr(), y1.data_ptr(), q1.data_ptr(), T, width, 1e-6, st)
        # ---- the one launch
        ring2, keep2 = ring_for(1)
        x2, y2, q2 = G.dev(x0), G.zeros((T, width)), G.zeros(T * (width // 32) * 36, torch.uint8)
        rows = L.MoeRows(dpart.data_ptr(), dtopw.data_ptr(), dsh.data_ptr(), dlog.data_ptr(), nexp, topk)
        bo2 = G.dev(peers[rank])
        L.call("fnx_boundary_rows", x2.data_ptr(), None if moe else bo2.data_ptr(), C.byref(rows) if moe else None, C.byref(ring2) if n > 1 else None,
               dw.data_ptr(), y2.data_ptr(), q2.data_ptr(), T, width, 1e-6, err.data_ptr(), st)
        G.sync()
        assert int(G.host(err)[0]) == 0
        assert np.array_equal(G.host(x2).view(np.uint32), G.host(x1).view(np.uint32)), (n, rank, "x")
        assert np.array_equal(G.host(y2).view(np.uint32), G.host(y1).view(np.uint32)), (n, rank, "y")
        assert np.array_equal(G.host(q2), G.host(q1)), (n, rank, "q8_1")
        if n > 1:
            assert G.host(keep2[2]).tolist()[:3] == [1, 0, 0]
            for k in range(n):   # every peer has this GPU's addend, marked with the exchange's number
                if k != rank:
                    vals, eps_ = _ll_sent(G, keep2[3][k][1], rank, T * width, T * width)
                    assert np.array_equal(vals, mine.reshape(-1).view(np.uint32)) and (eps_ == 1).all()
    # a window's first half: no addend, the norm alone
    x3, y3, q3 = G.dev(x0), G.zeros((T, width)), G.zeros(T * (width // 32) * 36, torch.uint8)
    x4, y4, q4 = G.dev(x0), G.zeros((T, width)), G.zeros(T * (width // 32) * 36, torch.uint8)
    dw = G.dev(wn)
    L.call("fnx_rms_norm_rows", x3.data_ptr(), None, dw.data_ptr(), y3.data_ptr(), q3.data_ptr(), T, width, 1e-6, st)
    L.call("fnx_boundary_rows", x4.data_ptr(), None, None, None, dw.data_ptr(), y4.data_ptr(), q4.data_ptr(), T, width, 1e-6, None, st)
    G.sync()
    assert np.array_equal(G.host(y4).view(np.uint32), G.host(y3).view(np.uint32)) and np.array_equal(G.host(q4), G.host(q3))
    assert np.array_equal(G.host(x4), x0)


@pytest.mark.parametrize("n,T,nq,hd", [(1, 16, 24, 256), (2, 16, 24, 256), (4, 5, 8, 128), (8, 16, 24, 256)])
def test_attn_finish_ring_equals_the_separate_steps(n, T, nq, hd):
    """The attention layer's exchange + merge + gate + q8_1 in one launch against fnx_attn_finish over gathered partials
    followed by fnx_quantize_q8_1, bit for bit; the peers of one GPU are emulated (their partials and flags in place
    before the launch).  One GPU's partial has no positions for some heads (m = -inf, z = 0)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(11 * n + T)
    parts = rng.standard_normal((n, T, nq, hd + 2)).astype(np.float32)
    parts[..., hd] = rng.standard_normal((n, T, nq)) * 5          # m
    parts[..., hd + 1] = rng.random((n, T, nq)) * 100 + 0.5       # z
    if n > 1:
        parts[n - 1, :, ::3, :hd] = 0
        parts[n - 1, :, ::3, hd] = -np.inf
        parts[n - 1, :, ::3, hd + 1] = 0
    qg = rng.standard_normal((T, nq, 2 * hd)).astype(np.float32)
    own, st = nq // n, L.stream()
    dparts, dqg = G.dev(parts), G.dev(qg)
    for rank in range(n):
        out1, q1 = G.zeros((T, own, hd)), G.zeros(T * (own * hd // 32) * 36, torch.uint8)
        L.call("fnx_attn_finish", dparts.data_ptr(), n, rank, dqg.data_ptr(), out1.data_ptr(), T, nq, rank * own, own, hd, st)
        L.call("fnx_quantize_q8_1", out1.data_ptr(), q1.data_ptr(), own * hd, T, st)
        for epoch in (1, 2):
            slots = [[G.zeros(4) for p in range(2)] for k in range(n)]
            pads = [G.zeros(16, torch.int32) for _ in range(n)]
            state = torch.tensor([epoch - 1, 0, 0, 0], dtype=torch.int32, device=G.DEV)
            err = G.zeros(1, torch.int32)
            cnt = T * own * (hd + 2)
            ll = _ll_areas(G, torch, n, rank, cnt, epoch, lambda k: parts[k][:, rank * own:(rank + 1) * own])
            ring = _ring(L, G, torch, n, rank, slots, pads, state, 1 << 20, ll, cnt)
            out2, q2 = G.zeros((T, own, hd)), G.zeros(T * (own * hd // 32) * 36, torch.uint8)
            mine = G.dev(parts[rank])
            L.call("fnx_attn_finish_ring", mine.data_ptr(), C.byref(ring) if n > 1 else None, dqg.data_ptr(), out2.data_ptr(), q2.data_ptr(), T, nq, hd,
                   err.data_ptr(), st)
            G.sync()
            assert int(G.host(err)[0]) == 0
            assert np.array_equal(G.host(out2).view(np.uint32), G.host(out1).view(np.uint32)), (n, rank, epoch)
            assert np.array_equal(G.host(q2), G.host(q1)), (n, rank, epoch, "q8_1")
            if n > 1:
                assert G.host(state).tolist()[:3] == [epoch, 0, 0]
                for k in range(n):   # every peer has this GPU's partials of the heads that peer owns
                    if k != rank:
                        vals, eps_ = _ll_sent(G, ll[k][epoch % 2], rank, cnt, cnt)
                        want = np.ascontiguousarray(parts[rank][:, k * own:(k + 1) * own]).reshape(-1).view(np.uint32)
                        assert np.array_equal(vals, want) and (eps_ == epoch).all(), "sent partials"


@pytest.mark.parametrize("n,na,nb", [(2, 16, 16), (8, 16, 16), (4, 1024, 1024), (3, 5, 0)])
def test_ring_gather(n, na, nb):
    """The small all-gather over the ring's slots (the per-GPU argmax pairs, the candidates): every rank's view, with the
    peers emulated (their words and flags in place before the launch)."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    rng = np.random.default_rng(5 * n + na)
    A = rng.standard_normal((n, na)).astype(np.float32)
    B = rng.integers(0, 1 << 30, (n, max(nb, 1)), dtype=np.int32)[:, :nb]
    st = L.stream()
    for rank in range(n):
        for epoch in (1, 2):
            slots = [[G.zeros(4) for p in range(2)] for k in range(n)]
            pads = [G.zeros(16, torch.int32) for _ in range(n)]
            state = torch.tensor([epoch - 1, 0, 0, 0], dtype=torch.int32, device=G.DEV)
            err = G.zeros(1, torch.int32)
            ll = _ll_areas(G, torch, n, rank, 4096, epoch, lambda k: np.concatenate([A[k].view(np.uint32), B[k].view(np.uint32)]))
            ring = _ring(L, G, torch, n, rank, slots, pads, state, 1 << 20, ll, 4096)
            a, b = G.dev(A[rank]), G.dev(np.ascontiguousarray(B[rank])) if nb else None
            all_a, all_b = G.zeros((n, na)), G.zeros((n, max(nb, 1)), torch.int32)
            L.call("fnx_ring_gather", a.data_ptr(), na, b.data_ptr() if nb else None, nb, C.byref(ring), all_a.data_ptr(),
                   all_b.data_ptr() if nb else None, err.data_ptr(), st)
            G.sync()
            assert int(G.host(err)[0]) == 0 and G.host(state).tolist()[0] == epoch
            assert np.array_equal(G.host(all_a).view(np.uint32), A.view(np.uint32)), (n, rank, epoch)
            if nb:
                assert np.array_equal(G.host(all_b)[:, :nb], B), (n, rank, epoch)


def test_window_exchange_gives_up_when_a_peer_never_sends():
    """The window's own exchanges poll this GPU's receive area for words that carry the exchange's number; with nothing
    arriving and a short poll limit the kernel gives up with error bit 1 and the context stays usable."""
    import torch

    from sfnx_b200 import lib as L
    from tests import gpu_util as G

    n, na = 2, 16
    slots = [[G.zeros(4) for _ in range(2)] for _ in range(n)]
    pads = [G.zeros(16, torch.int32) for _ in range(n)]
    ll = [[torch.zeros(n * 64, dtype=torch.int64, device=G.DEV) for _ in range(2)] for _ in range(n)]   # nothing ever arrives
    state, err = G.zeros(4, torch.int32), G.zeros(1, torch.int32)
    ring = _ring(L, G, torch, n, 0, slots, pads, state, 200, ll, 64)
    a, all_a = G.dev(np.arange(na, dtype=np.float32)), G.zeros((n, na))
    L.call("fnx_ring_gather", a.data_ptr(), na, None, 0, C.byref(ring), all_a.data_ptr(), None, err.data_ptr(), L.stream())
    G.sync()
    assert int(G.host(err)[0]) & 1 == 1
    assert np.array_equal(G.host(all_a)[0], np.arange(na, dtype=np.float32))   # its own words are in place all the same
    y = G.zeros(8)
    y.fill_(3.0)
    G.sync()
    assert float(G.host(y)[0]) == 3.0
