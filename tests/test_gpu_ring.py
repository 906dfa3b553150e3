"""GPU parity of the peer-memory sum across GPUs against the CPU oracle's ring order, on ONE GPU: the "peers" are other
buffers of the same device whose addends and flags are in place before the launch, so no launch waits for another.  A
second case leaves one peer's flag unset with a short poll limit and checks that the kernel gives up with error bit 1."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ring(L, G, torch, n, rank, slots, pads, state, limit):
    r = L.Ring()
    r.nrank, r.rank, r.state, r.spin_limit = n, rank, state.data_ptr(), limit
    for p in range(2):
        for k in range(n):
            r.slot[p][k] = slots[k][p].data_ptr()
    for k in range(n):
        r.pad[k] = pads[k].data_ptr()
    return r


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
