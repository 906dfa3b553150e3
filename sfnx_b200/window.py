"""Host-side plumbing of the verify window: a seeded synthetic stack in device memory, its slice for one GPU of several,
and a runner that captures the window's stages (and the collectives between them) into one CUDA graph.

torch is used for device memory, streams, CUDA graphs and torch.distributed (NCCL); every kernel is launched by
libsfnx_b200.so through the C ABI.  The split across GPUs follows the reference's rule (src/card_split.hpp:12-26,
docs/config.md:62-71): experts by FF width in 32-value blocks, DeltaNet by value heads, K/V by position in blocks of 4,
the vocabulary in contiguous ranges; the router, the norms and the embeddings are copied.
"""
import ctypes as C
import os
import sys
import torch

from . import lib as L
from .shapes import StackShape  # noqa: F401  (defined in a module without torch; re-exported here)


def _seed(base, layer, name):
    h = 1469598103934665603
    for ch in ("%d/%d/%s" % (base, layer, name)).encode():
        h = ((h ^ ch) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h & 0x7FFFFFFFFFFFFFFF


class SyntheticStack:
    """Random-init weights and states of one GPU's slice, generated on the device from seeds: every GPU generates the
    same full tensor and keeps its slice, so the slices of N GPUs are one model."""

    def __init__(self, shape, ncard=1, card=0, seed=0, device="cuda", gdn_log=True):
        """gdn_log: the DeltaNet layers keep a replay log instead of per-row checkpoints of the state (fnx_gdn_core_log);
        False: checkpoints, which windows of several sequences (LaneSet) need."""
        self.shape, self.ncard, self.card, self.seed, self.gdn_log = shape, ncard, card, seed, gdn_log
        self.dev = torch.device(device)
        self.keep = []
        self.named = {}   # (layer, name) -> tensors, for callers that need the values (tests, CPU baselines)
        s = shape
        lib = L.load()
        self.ff0 = lib.fnx_ff_lo(s.ff, ncard, card)
        self.ffs = lib.fnx_ff_lo(s.ff, ncard, card + 1) - self.ff0
        self.vheads = [v for v in range(s.nvh) if lib.fnx_vhead_card(s.nkh, s.nvh, ncard, v) == card]
        self.kh0 = lib.fnx_khead_first(s.nkh, s.nvh, ncard, card)
        self.nk = lib.fnx_khead_count(s.nkh, s.nvh, ncard, card)
        self.nv = len(self.vheads)
        self.v0, self.vrows = vocab_slice(s.vocab, ncard, card)
        self.kv_rows = lib.fnx_kv_rows_per_card(s.ctx + s.kv_slack, ncard)
        self.cfg = L.StackCfg(s.n, s.nexp, s.topk, self.ffs, self.nk, self.nv, s.nq, s.nkv, s.hd, s.nrot, self.v0, self.vrows,
                              len(s.kinds), ncard, card, s.eps, s.rope_base, s.hc if s.hc > 1 else 0, s.hc_lr, 1 if s.draft else 0,
                              s.qsa_top, 2048 if s.qsa_top else 0, (s.ctx + s.kv_slack) // 4 + 1 if s.qsa_top else 0)
        self.layers = (L.Layer * len(s.kinds))()
        self.gdn_state = []   # (S, hist) of the DeltaNet layers, for snapshots
        for l, kind in enumerate(s.kinds):
            self._build_layer(l, kind)
        self.head = L.Head(self._t(torch.ones(s.n, device=self.dev)).data_ptr(), self._q8s(len(s.kinds), "output", s.vocab, s.n,
                                                                                          row_slice=slice(self.v0, self.v0 + self.vrows)))
        if s.hc > 1:
            self.head.mix = self._hcw(len(s.kinds), "mix", inject=False)
        self.draft = None
        if s.draft:   # the draft layer's prologue (reference MtpCard: norm_emb, norm_hid, fc_emb, fc_hid; replicated)
            assert s.hc > 1, "a draft layer mixes residual streams"
            nl = len(s.kinds)
            ne = self._t(1 + 0.1 * self._normal(nl, "norm_emb", (s.n,), 1.0))
            nh = self._t(1 + 0.1 * self._normal(nl, "norm_hid", (s.hc * s.n,), 1.0))
            self.named[(nl, "norm_emb")], self.named[(nl, "norm_hid")] = ne, nh
            self.draft = L.Draft(ne.data_ptr(), nh.data_ptr(), self._q8s(nl, "fc_emb", s.n, s.n), self._q8s(nl, "fc_hid", s.n, s.n))
        emb = torch.empty(s.vocab * s.n, dtype=torch.float32, device=self.dev)
        L.call("fnx_synth_normal", emb.data_ptr(), emb.numel(), 1.0, _seed(seed, -1, "embed"), L.stream())
        self.embed = self._t(emb.half().view(s.vocab, s.n).view(torch.int16))
        del emb
        nbytes = lib.fnx_window_workspace_bytes(C.byref(self.cfg))
        assert nbytes > 0, lib.fnx_last_error()
        self.ws = torch.zeros(nbytes, dtype=torch.uint8, device=self.dev)
        L.call("fnx_window_init", C.byref(self.cfg), self.ws.data_ptr(), L.stream())
        torch.cuda.synchronize()

    # ---- tensors
    def _t(self, t):
        t = t.contiguous()
        self.keep.append(t)
        return t

    def _normal(self, layer, name, shape, sigma):
        t = torch.empty(shape, dtype=torch.float32, device=self.dev)
        L.call("fnx_synth_normal", t.data_ptr(), t.numel(), sigma, _seed(self.seed, layer, name), L.stream())
        return t

    def _blocks(self, layer, name, qtype, nvalues):
        bsz, per = {L.Q4_K: (144, 256), L.Q6_K: (210, 256), L.Q8_0: (34, 32)}[qtype]
        b = torch.empty(nvalues // per * bsz, dtype=torch.uint8, device=self.dev)
        L.call("fnx_synth_quant", qtype, b.data_ptr(), nvalues, self.shape.sigma, _seed(self.seed, layer, name), L.stream())
        return b

    def _q8s(self, layer, name, rows, cols, rows_idx=None, cols_idx=None, row_slice=None):
        """A Q8_0 matrix [rows][cols] of the full model in the split layout, cut to this GPU's rows / 32-aligned columns."""
        b = self._blocks(layer, name, L.Q8_0, rows * cols)
        q = torch.empty((rows, cols), dtype=torch.int8, device=self.dev)
        d = torch.empty((rows, cols // 32), dtype=torch.int16, device=self.dev)
        L.call("fnx_repack_q8_0_split", b.data_ptr(), q.data_ptr(), d.data_ptr(), rows, cols, L.stream())
        if row_slice is not None:
            q, d = q[row_slice], d[row_slice]
        if rows_idx is not None:
            q, d = q[rows_idx], d[rows_idx]
        if cols_idx is not None:
            q = q.view(q.shape[0], cols // 32, 32)[:, cols_idx].reshape(q.shape[0], -1)
            d = d[:, cols_idx]
        q, d = self._t(q), self._t(d)
        self.named[(layer, name)] = (q, d)
        return L.Q8S(q.data_ptr(), d.data_ptr())

    def _hcw(self, layer, name, inject=True):
        """One hyper-connection read's weights (replicated on every GPU): norm [hc n] near 1, down Q8_0 [lr][hc n], up Q8_0
        [hc n][lr], bf16 inject rows [hc][hc n]."""
        s = self.shape
        D = s.hc * s.n
        norm = self._t(1 + 0.1 * self._normal(layer, name + "_norm", (D,), 1.0))
        self.named[(layer, name + "_norm")] = norm
        hw = L.HcW(norm.data_ptr(), self._q8s(layer, name + "_down", s.hc_lr, D), self._q8s(layer, name + "_up", D, s.hc_lr), None)
        if inject:
            inj = self._t((self._normal(layer, name + "_inj", (s.hc, D), 0.05).view(torch.int32) >> 16).to(torch.int16))
            self.named[(layer, name + "_inj")] = inj
            hw.inj = inj.data_ptr()
        return hw

    def _kv_slice(self, layer, name):
        """This GPU's rows of a K or V cache N(0, 1) over every position: the whole cache is generated (the same on every
        GPU) and local row r = the row of position ((r / 4) ncard + card) 4 + r % 4.  With shape.kv_q8 the rows are int8
        in groups of 32 (d = max |x| / 127, f16 d), the rows' bytes first and their scales after them (one page)."""
        s = self.shape
        full = self._normal(layer, name, (self.kv_rows * self.ncard, s.nkv, s.hd), 1.0).half()
        if self.ncard > 1:
            r = torch.arange(self.kv_rows, device=self.dev)
            full = full[((r // 4) * self.ncard + self.card) * 4 + r % 4]
        if not s.kv_q8:
            return self._t(full.contiguous().view(torch.int16))
        g = full.float().reshape(self.kv_rows, -1, 32)
        d = g.abs().amax(-1) / 127.0
        y = g * torch.where(d != 0, 1.0 / d, torch.zeros_like(d)).unsqueeze(-1)
        q = (torch.sign(y) * torch.floor(y.abs() + 0.5)).to(torch.int8)
        words = torch.cat([q.reshape(-1).view(torch.int16), d.half().reshape(-1).view(torch.int16)])
        assert words.numel() == L.load().fnx_kvq_halves(self.kv_rows, s.nkv, s.hd)
        return self._t(words)

    def _idx(self, lst):
        return torch.tensor(lst, dtype=torch.long, device=self.dev)

    def _build_layer(self, l, kind):
        s, Lr = self.shape, self.layers[l]
        Lr.kind = kind
        Lr.norm1 = self._t(torch.ones(s.n, device=self.dev)).data_ptr()
        Lr.norm2 = self._t(torch.ones(s.n, device=self.dev)).data_ptr()
        if s.hc > 1:
            Lr.hcw[0], Lr.hcw[1] = self._hcw(l, "hc0"), self._hcw(l, "hc1")
        if kind == 0:
            HS = L.HS
            khs = list(range(self.kh0, self.kh0 + self.nk))
            rows = []
            for base, heads in ((0, khs), (s.nkh * HS, khs), (2 * s.nkh * HS, self.vheads), ((2 * s.nkh + s.nvh) * HS, self.vheads)):
                for h in heads:
                    rows += list(range(base + h * HS, base + (h + 1) * HS))
            Lr.qkvz = self._q8s(l, "qkvz", (2 * s.nkh + 2 * s.nvh) * HS, s.n, rows_idx=self._idx(rows))
            ab = self._normal(l, "ab", (2 * s.nvh, s.n), s.sigma)
            self.named[(l, "ab")] = self._t(ab[self._idx(self.vheads + [s.nvh + v for v in self.vheads])])
            Lr.ab = self.named[(l, "ab")].data_ptr()
            ch_full = (2 * s.nkh + s.nvh) * HS
            conv = self._normal(l, "conv", (ch_full, 4), 0.5)
            self.named[(l, "conv")] = self._t(conv[self._idx(rows[: (2 * self.nk + self.nv) * HS])])
            Lr.conv = self.named[(l, "conv")].data_ptr()
            Lr.dt = self._t(torch.zeros(self.nv, device=self.dev)).data_ptr()
            Lr.a = self._t(-torch.ones(self.nv, device=self.dev)).data_ptr()
            Lr.ssm_norm = self._t(torch.ones(HS, device=self.dev)).data_ptr()
            Lr.ssm_out = self._q8s(l, "ssm_out", s.n, s.nvh * HS, cols_idx=self._idx([v * 4 + b for v in self.vheads for b in range(4)]))
            seen, vmap = set(), []
            for v in self.vheads:   # value head v belongs to key head v % nkh; its first value head here writes q/k history
                kh = v % s.nkh
                vmap.append((kh - self.kh0) | ((0 if kh in seen else 1) << 8))
                seen.add(kh)
            self.named[(l, "vmap")] = self._t(torch.tensor(vmap, dtype=torch.int32, device=self.dev))
            Lr.vmap = self.named[(l, "vmap")].data_ptr()
            S = self._t(self._normal(l, "S", (s.nvh, HS, HS), 0.1)[self._idx(self.vheads)])
            hist = self._t(self._normal(l, "hist", (2, 3, ch_full), 1.0)[:, :, self._idx(rows[: (2 * self.nk + self.nv) * HS])])
            hsnap = self._t(torch.zeros((L.MAXT, 3, (2 * self.nk + self.nv) * HS), device=self.dev))
            Lr.S, Lr.hist, Lr.hsnap = S.data_ptr(), hist.data_ptr(), hsnap.data_ptr()
            if self.gdn_log:
                Lr.snap = None
                Lr.gdn_log = self._t(torch.zeros(L.load().fnx_gdn_log_floats(self.nk, self.nv), device=self.dev)).data_ptr()
            else:
                Lr.snap = self._t(torch.zeros((L.MAXT - 1, self.nv, HS, HS), device=self.dev)).data_ptr()
                Lr.gdn_log = None
            self.gdn_state.append((S, hist))
            self.named[(l, "S")], self.named[(l, "hist")] = S, hist
        else:
            own = s.nq // self.ncard
            Lr.wq = self._q8s(l, "wq", s.nq * s.hd * 2, s.n)
            Lr.wk = self._q8s(l, "wk", s.nkv * s.hd, s.n)
            Lr.wv = self._q8s(l, "wv", s.nkv * s.hd, s.n)
            nb = s.hd // 32
            Lr.wo = self._q8s(l, "wo", s.n, s.nq * s.hd, cols_idx=self._idx(list(range(self.card * own * nb, (self.card + 1) * own * nb))))
            Lr.q_norm = self._t(torch.ones(s.hd, device=self.dev)).data_ptr()
            Lr.k_norm = self._t(torch.ones(s.hd, device=self.dev)).data_ptr()
            kc, vc = self._kv_slice(l, "kc"), self._kv_slice(l, "vc")
            Lr.kc, Lr.vc = kc.data_ptr(), vc.data_ptr()
            self.named[(l, "kc")], self.named[(l, "vc")] = kc, vc
            Lr.pages = L.KvPages(None, 0, 0, self.kv_rows, 1 if s.kv_q8 else 0)
            if s.qsa_top:   # the indexer (replicated on every GPU), the raw keys of the last positions and the pooled keys of the context
                bf16 = lambda t: self._t(((t.view(torch.int32) + 0x7FFF + ((t.view(torch.int32) >> 16) & 1)) >> 16).to(torch.int16))
                iw = {"idx_wq": bf16(self._normal(l, "idx_wq", (512, s.n), 0.05)), "idx_wk": bf16(self._normal(l, "idx_wk", (128, s.n), 0.05)),
                      "idx_qn": self._t(1 + 0.1 * self._normal(l, "idx_qn", (128,), 1.0)), "idx_kn": self._t(1 + 0.1 * self._normal(l, "idx_kn", (128,), 1.0)),
                      "idx_ring": self._t(self._normal(l, "idx_ring", (self.cfg.qsa_ring_rows, 128), 1.0).half().view(torch.int16)),
                      "idx_pooled": self._t(self._normal(l, "idx_pooled", (self.cfg.qsa_max_pools, 128), 1.0).half().view(torch.int16))}
                for key, v in iw.items():
                    self.named[(l, key)] = v
                Lr.idx = L.QsaW(*(iw[k].data_ptr() for k in ("idx_wq", "idx_wk", "idx_qn", "idx_kn", "idx_ring", "idx_pooled")))
        # FFN
        self.named[(l, "router")] = self._t(self._normal(l, "router", (s.nexp + 1, s.n), s.sigma))
        Lr.router = self.named[(l, "router")].data_ptr()
        if s.experts == "q8_0":
            self._build_experts_q8(l)
            return
        row_b = s.n // 256 * 144
        gu = self._blocks(l, "gate_up", L.Q4_K, s.nexp * 2 * s.ff * s.n).view(s.nexp, 2, s.ff, row_b)
        gu = self._t(gu[:, :, self.ff0:self.ff0 + self.ffs].reshape(s.nexp, 2 * self.ffs * row_b))
        Lr.gate_up = L.Experts(L.Q4_K, 2 * self.ffs, s.n, gu.data_ptr(), None, None, None, 2 * self.ffs * row_b, 0)
        dn = self._blocks(l, "down", L.Q6_K, s.nexp * s.n * s.ff)
        nu, units = self.ffs // 32, s.nexp * s.n * (self.ffs // 32)
        QL = self._t(torch.empty(units * 16, dtype=torch.uint8, device=self.dev))
        QH = self._t(torch.empty(units * 8, dtype=torch.uint8, device=self.dev))
        SC = self._t(torch.empty(units * 2, dtype=torch.uint8, device=self.dev))
        D = self._t(torch.empty(units, dtype=torch.int16, device=self.dev))
        L.call("fnx_repack_q6k_units", dn.data_ptr(), s.nexp * s.n, s.ff, self.ff0, self.ffs, QL.data_ptr(), QH.data_ptr(), SC.data_ptr(),
               D.data_ptr(), L.stream())
        self.named[(l, "gate_up")] = gu
        self.named[(l, "down")] = (QL.view(s.nexp, s.n, nu, 16), QH.view(s.nexp, s.n, nu, 8), SC.view(s.nexp, s.n, nu, 2), D.view(s.nexp, s.n, nu))
        Lr.down = L.Experts(L.Q6_K, s.n, self.ffs, QL.data_ptr(), QH.data_ptr(), SC.data_ptr(), D.data_ptr(), s.n * nu, 0)
        self._build_shared(l)
        torch.cuda.synchronize()
        del dn

    def _build_shared(self, l):
        s, Lr = self.shape, self.layers[l]
        ffr = list(range(self.ff0, self.ff0 + self.ffs))
        Lr.sh_gate_up = self._q8s(l, "sh_gate_up", 2 * s.ff, s.n, rows_idx=self._idx(ffr + [s.ff + r for r in ffr]))
        Lr.sh_down = self._q8s(l, "sh_down", s.n, s.ff, cols_idx=self._idx(list(range(self.ff0 // 32, (self.ff0 + self.ffs) // 32))))

    def _build_experts_q8(self, l):
        """Routed experts in split Q8_0: gate|up [nexp][2 ffs][n], down [nexp][n][ffs], this GPU's FF range of each."""
        s, Lr = self.shape, self.layers[l]
        nb, fb0, fbs = s.n // 32, self.ff0 // 32, self.ffs // 32
        b = self._blocks(l, "gate_up", L.Q8_0, s.nexp * 2 * s.ff * s.n)
        q = torch.empty((s.nexp * 2 * s.ff, s.n), dtype=torch.int8, device=self.dev)
        d = torch.empty((s.nexp * 2 * s.ff, nb), dtype=torch.int16, device=self.dev)
        L.call("fnx_repack_q8_0_split", b.data_ptr(), q.data_ptr(), d.data_ptr(), s.nexp * 2 * s.ff, s.n, L.stream())
        gq = self._t(q.view(s.nexp, 2, s.ff, s.n)[:, :, self.ff0:self.ff0 + self.ffs].reshape(s.nexp, 2 * self.ffs, s.n))
        gd = self._t(d.view(s.nexp, 2, s.ff, nb)[:, :, self.ff0:self.ff0 + self.ffs].reshape(s.nexp, 2 * self.ffs, nb))
        del b, q, d
        Lr.gate_up = L.Experts(L.Q8_0, 2 * self.ffs, s.n, gq.data_ptr(), gd.data_ptr(), None, None, 2 * self.ffs * s.n, 2 * self.ffs * nb * 2)
        b = self._blocks(l, "down", L.Q8_0, s.nexp * s.n * s.ff)
        q = torch.empty((s.nexp * s.n, s.ff), dtype=torch.int8, device=self.dev)
        d = torch.empty((s.nexp * s.n, s.ff // 32), dtype=torch.int16, device=self.dev)
        L.call("fnx_repack_q8_0_split", b.data_ptr(), q.data_ptr(), d.data_ptr(), s.nexp * s.n, s.ff, L.stream())
        dq = self._t(q.view(s.nexp, s.n, s.ff)[:, :, self.ff0:self.ff0 + self.ffs].contiguous())
        dd = self._t(d.view(s.nexp, s.n, s.ff // 32)[:, :, fb0:fb0 + fbs].contiguous())
        del b, q, d
        Lr.down = L.Experts(L.Q8_0, s.n, self.ffs, dq.data_ptr(), dd.data_ptr(), None, None, s.n * self.ffs, s.n * fbs * 2)
        self.named[(l, "gate_up")] = (gq, gd)
        self.named[(l, "down")] = (dq, dd)
        self._build_shared(l)
        torch.cuda.synchronize()

    # ---- state
    def save_state(self):
        return [(S.clone(), h.clone()) for S, h in self.gdn_state]

    def load_state(self, saved):
        for (S, h), (S0, h0) in zip(self.gdn_state, saved):
            S.copy_(S0)
            h.copy_(h0)

    def buf(self, which, dtype, numel):
        """A tensor over one of the workspace's buffers."""
        p = L.load().fnx_window_buf(C.byref(self.cfg), self.ws.data_ptr(), which)
        off = p - self.ws.data_ptr()
        return self.ws[off: off + numel * torch.empty(0, dtype=dtype).element_size()].view(dtype)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.keep)

    def sequence_view(self, index):
        """Another sequence over the same weights: a copy of this stack's description whose DeltaNet states, conv
        histories and K/V caches are tensors of its own (seeded by `index`); the weights, the checkpoints' scratch and the
        workspace are shared, so windows of different sequences run one after the other on one stream."""
        import copy

        v = copy.copy(self)
        v.layers = type(self.layers).from_buffer_copy(self.layers)
        v.keep, v.named, v.gdn_state = [], dict(self.named), []
        s = self.shape
        for l, kind in enumerate(s.kinds):
            Lr = v.layers[l]
            if kind == 0:
                S0, h0 = self.named[(l, "S")], self.named[(l, "hist")]
                S = v._t(S0 * (1.0 + 0.05 * index))
                hist = v._t(h0 * (1.0 - 0.03 * index))
                Lr.S, Lr.hist = S.data_ptr(), hist.data_ptr()
                if self.gdn_log:
                    Lr.gdn_log = v._t(torch.zeros(L.load().fnx_gdn_log_floats(self.nk, self.nv), device=self.dev)).data_ptr()
                v.gdn_state.append((S, hist))
                v.named[(l, "S")], v.named[(l, "hist")] = S, hist
            else:
                kc, vc = v._t(self._kv_slice(l, "kc_seq%d" % index)), v._t(self._kv_slice(l, "vc_seq%d" % index))
                Lr.kc, Lr.vc = kc.data_ptr(), vc.data_ptr()
                v.named[(l, "kc")], v.named[(l, "vc")] = kc, vc
        return v


def merge_best(values, indices):
    """Per row, the token of the GPU whose slice holds the largest logit: strict > scanning GPU 0 upward, so the lower
    GPU wins a tie (reference src/engine_common.cu:781-787).  values, indices: [ngpu][T]."""
    out = []
    for t in range(values.shape[1]):
        b = 0
        for c in range(1, values.shape[0]):
            if values[c, t] > values[b, t]:
                b = c
        out.append(int(indices[b, t]))
    return out


def vocab_slice(vocab, ncard, card):
    """This GPU's contiguous vocabulary range, ceil(vocab / n) each, the last shorter (reference src/model.cpp:836)."""
    per = (vocab + ncard - 1) // ncard
    v0 = card * per
    return v0, max(0, min(vocab, v0 + per) - v0)


class LaneSet:
    """The per-sequence side of a window of several sequences ("lanes": reference src/engine.hpp LaneDev): every lane's
    DeltaNet states and conv histories (copies of the stack's, scaled a little apart), its run of pages of each attention
    layer's K/V pool (the stack's cache cut into nseg equal runs of pages of `rpp` local rows), its (position, tag) words,
    and the pointer tables the library's lanes entry points take (FnxWindowLanes)."""

    def __init__(self, stack, nseg, rows, rpp=64):
        assert nseg * rows <= L.MAXT
        assert not stack.gdn_log, "windows of several sequences keep checkpoints: build the stack with gdn_log=False"
        self.stack, self.nseg, self.rows, self.rpp = stack, nseg, rows, rpp
        dev, s, T = stack.dev, stack.shape, nseg * rows
        nl = len(s.kinds)
        self.region = stack.kv_rows // nseg // rpp * rpp   # local rows of a lane's run of pages
        assert self.region >= rpp, "the K/V pool is too small for %d lanes" % nseg
        self.keep = []
        ptr_dev = lambda ts: self._k(torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev))
        ptr_host = lambda ps: self._k((C.c_void_p * len(ps))(*ps))
        self.S, self.hist = {}, {}
        S_dev, h_dev, S_host, h_host = [None] * nl, [None] * nl, [None] * nl, [None] * nl
        gi = 0
        for l, kind in enumerate(s.kinds):
            if kind != 0:
                continue
            S0, h0 = stack.gdn_state[gi]
            gi += 1
            self.S[l] = [self._k((S0 * (1.0 + 0.05 * i)).contiguous()) for i in range(nseg)]
            self.hist[l] = [self._k((h0 * (1.0 - 0.03 * i)).contiguous()) for i in range(nseg)]
            S_dev[l], h_dev[l] = ptr_dev(self.S[l]).data_ptr(), ptr_dev(self.hist[l]).data_ptr()
            S_host[l] = C.addressof(ptr_host([t.data_ptr() for t in self.S[l]]))
            h_host[l] = C.addressof(ptr_host([t.data_ptr() for t in self.hist[l]]))
        # block selection: every lane's raw-key rings (one an attention layer); its pooled keys are its pages of the layer's pool
        self.rings, ring_host = {}, [None] * nl
        if s.qsa_top:
            for l, kind in enumerate(s.kinds):
                if kind != 1:
                    continue
                r0 = stack.named[(l, "idx_ring")]
                self.rings[l] = [self._k(torch.roll(r0, 7 * i, 0).contiguous()) for i in range(nseg)]   # the lanes' histories differ
                ring_host[l] = C.addressof(ptr_host([t.data_ptr() for t in self.rings[l]]))
        self.bpp = rpp // 4 * stack.ncard   # blocks of 4 positions a page holds (every GPU's)
        ppl = self.region // rpp   # pages per lane
        self.pt = [self._k(torch.arange(i * ppl, (i + 1) * ppl, dtype=torch.int32, device=dev)) for i in range(nseg)]
        self.ctl = self._k(torch.zeros((nseg, 2), dtype=torch.int32, device=dev))
        self.row_pos = self._k(torch.zeros(T, dtype=torch.int32, device=dev))
        self.row0 = self._k(torch.arange(nseg, dtype=torch.int32, device=dev) * rows)
        ctl_ptrs = [self.ctl[i].data_ptr() for i in range(nseg)]
        self.h_ctl = torch.zeros((nseg, 2), dtype=torch.int32).pin_memory()
        self.h_row_pos = torch.zeros(T, dtype=torch.int32).pin_memory()
        self.c = L.WindowLanes(
            nseg, rows,
            self._k(torch.tensor(ctl_ptrs, dtype=torch.int64, device=dev)).data_ptr(), self.row0.data_ptr(),
            self._k(torch.tensor([self.row_pos[t:t + 1].data_ptr() for t in range(T)], dtype=torch.int64, device=dev)).data_ptr(),
            self._k(torch.tensor([self.pt[t // rows].data_ptr() for t in range(T)], dtype=torch.int64, device=dev)).data_ptr(),
            C.addressof(ptr_host(ctl_ptrs)), C.addressof(ptr_host([t.data_ptr() for t in self.pt])),
            C.addressof(ptr_host(S_dev)), C.addressof(ptr_host(h_dev)), C.addressof(ptr_host(S_host)), C.addressof(ptr_host(h_host)),
            C.addressof(ptr_host(ring_host)) if s.qsa_top else None)
        assert not s.qsa_top or nseg * ppl * self.bpp <= stack.cfg.qsa_max_pools, "the pooled keys' pool is too small for the lanes' pages"
        # the attention layers' pools as pages of rpp local rows (a lane's table is filled in per call)
        self.paged = L.KvPages(None, rpp * s.nkv * s.hd, rpp, 0)

    def _k(self, x):
        self.keep.append(x)
        return x

    def set_paged(self, on):
        """Switches the stack's attention layers between the lanes' paged view of the K/V pool and the one-sequence view."""
        for l, kind in enumerate(self.stack.shape.kinds):
            if kind == 1:
                self.stack.layers[l].pages = self.paged if on else L.KvPages(None, 0, 0, self.stack.kv_rows)
                self.stack.layers[l].idx.page = self.bpp * 128 if on else 0   # the pooled keys' pool in pages of bpp keys

    def positions(self, pos, tags):
        """Lane i's window starts at position pos[i] with tag tags[i] (host lists)."""
        for i in range(self.nseg):
            self.h_ctl[i, 0], self.h_ctl[i, 1] = pos[i], tags[i]
            for r in range(self.rows):
                self.h_row_pos[i * self.rows + r] = pos[i] + r
        self.ctl.copy_(self.h_ctl, non_blocking=True)
        self.row_pos.copy_(self.h_row_pos, non_blocking=True)


class WindowRunner:
    """One window of T rows as a CUDA graph on its own stream: embedding rows from the token ids, every stage, and
    between stages the collectives of the process group (NCCL) when there is more than one GPU."""

    def __init__(self, stack, T, group=None, graph=True, overlap=True, sampled=False, lanes=None, stream=None):
        import torch.distributed as dist

        self.stack, self.T, self.group = stack, T, group
        self.lanes = lanes   # a LaneSet: the T rows are lanes.nseg sequences' rows (window_lanes, commit_lanes)
        if lanes is not None:
            assert T == lanes.nseg * lanes.rows
            lanes.set_paged(True)
        self.dist = dist if stack.ncard > 1 else None
        cfg, s = stack.cfg, stack.shape
        lib = L.load()
        # runners that share a workspace (several sequences over one stack) must share their stream too
        self.stream = stream if stream is not None else torch.cuda.Stream()
        # what a window takes from the host, one buffer and one copy: the token ids, then (position, tag); the window's
        # first node copies the pair into the workspace's control words
        self.d_in = torch.zeros(L.MAXT + 2, dtype=torch.int32, device=stack.dev)
        self.ids, self.ctl_in = self.d_in[:L.MAXT], self.d_in[L.MAXT:]
        self.x = stack.buf(0, torch.float32, T * s.n)
        if s.draft:   # a draft layer's inputs: rows of a window's residual streams, and the next tokens' embeddings
            self.src = torch.zeros((T, s.hc * s.n), dtype=torch.float32, device=stack.dev)
            self.demb = torch.zeros((T, s.n), dtype=torch.float32, device=stack.dev)
        self.bo = stack.buf(1, torch.float32, T * s.n)
        self.partials = stack.buf(2, torch.float32, stack.ncard * T * s.nq * (s.hd + 2))
        self.best_v = stack.buf(3, torch.float32, T)
        self.best_i = stack.buf(4, torch.int32, T)
        self.err = stack.buf(5, torch.int32, 1)
        self.ctl = stack.buf(6, torch.int32, 2)
        self.logits = stack.buf(7, torch.float32, T * stack.vrows).view(T, stack.vrows)
        # what the host reads back, one buffer and one copy: every GPU's (value, index) per row and the error word
        nb = stack.ncard * T
        self.d_out = torch.zeros(2 * nb + 1, dtype=torch.int32, device=stack.dev)
        self.all_v = self.d_out[:nb].view(torch.float32).view(stack.ncard, T)
        self.all_i = self.d_out[nb:2 * nb].view(stack.ncard, T)
        self.h_in = torch.zeros(L.MAXT + 2, dtype=torch.int32).pin_memory()
        self.h_ids, self.h_ctl = self.h_in[:L.MAXT], self.h_in[L.MAXT:]
        self.h_out = torch.zeros(2 * nb + 1, dtype=torch.int32).pin_memory()
        self.h_v = self.h_out[:nb].view(torch.float32).view(stack.ncard, T)
        self.h_i = self.h_out[nb:2 * nb].view(stack.ncard, T)
        self.h_err = self.h_out[2 * nb:]
        self.h_in_np, self.h_v_np, self.h_i_np = self.h_in.numpy(), self.h_v.numpy(), self.h_i.numpy()   # the same memory
        # sampled acceptance: every GPU's 64 best (value, token) of each row of its vocabulary range, merged on the host
        self.sampled = sampled
        if sampled:
            self.cand_v = torch.zeros((T, L.TOPK_N), dtype=torch.float32, device=stack.dev)
            self.cand_i = torch.zeros((T, L.TOPK_N), dtype=torch.int32, device=stack.dev)
            self.all_cv = torch.zeros((stack.ncard, T, L.TOPK_N), dtype=torch.float32, device=stack.dev)
            self.all_ci = torch.zeros((stack.ncard, T, L.TOPK_N), dtype=torch.int32, device=stack.dev)
            self.h_cv = torch.zeros((stack.ncard, T, L.TOPK_N), dtype=torch.float32).pin_memory()
            self.h_ci = torch.zeros((stack.ncard, T, L.TOPK_N), dtype=torch.int32).pin_memory()
        # the sum across GPUs after each half layer: the library's own peer-memory sum in the reference ring's order
        # (fnx_ring_sum) over torch's symmetric memory, or NCCL's all-reduce (FNX_RING=nccl, or when peer memory cannot
        # be set up)
        self.ring, self.ring_keep = None, None
        if self.dist is not None and os.environ.get("FNX_RING", "peer") != "nccl":
            self.ring = self._make_ring(max(L.MAXT * s.n, L.MAXT * s.nq * (s.hd + 2)))   # a slot holds a sum's rows or a GPU's attention partials
        # the plan depends on who sums across the GPUs: the library's boundary kernel over the ring, or the caller
        L.call("fnx_window_ring", C.byref(self.ring) if self.ring is not None else None)
        after = (C.c_int * 1024)()
        self.nstages = lib.fnx_window_plan(C.byref(cfg), stack.layers, after, 1024)
        assert 0 < self.nstages <= 1024, lib.fnx_last_error()
        self.after = list(after[: self.nstages])
        self.job_bytes = len(s.kinds) * (2 * C.sizeof(L.CopyJob) + C.sizeof(L.GdnReplay))
        self.h_jobs = torch.zeros(64 * self.job_bytes, dtype=torch.uint8).pin_memory()   # a ring of job tables
        self.commits = 0
        self.launches = 0
        self.graph = None
        # a side stream for the window's independent branches (the library forks and joins with these events)
        self.side = torch.cuda.Stream() if overlap else None
        self.ev_fork, self.ev_join = torch.cuda.Event(), torch.cuda.Event()
        self.ev_fork.record(self.stream)   # torch makes an event's handle at its first record
        self.ev_join.record(self.stream)
        with torch.cuda.stream(self.stream):
            for _ in range(2):   # warm-up: shared-memory opt-ins, NCCL channels
                self._enqueue()
            self.stream.synchronize()
            if graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self._enqueue()
                self.graph = g
        torch.cuda.synchronize()

    def _make_ring(self, count):
        """Two slots of `count` floats and 64 flag words that every GPU of the group can address, and this GPU's view of
        them (FnxRing).  Returns None (NCCL is used) when symmetric memory is not available."""
        ptrs, why = None, ""
        try:
            import torch.distributed._symmetric_memory as symm

            group = self.group if self.group is not None else self.dist.group.WORLD
            nr = self.stack.ncard
            buf = symm.empty(2 * count + 64 + 4 * nr * count, dtype=torch.float32, device=self.stack.dev)   # slots, flags, receive areas
            buf.zero_()
            torch.cuda.synchronize()
            hdl = symm.rendezvous(buf, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        except Exception as e:   # noqa: BLE001
            why = str(e)
        # the ranks must take the same path: the peer-memory sum only if every rank has its buffers (a rank that went to
        # NCCL alone would wait in a collective nobody else joins)
        ok = torch.tensor([1 if ptrs else 0], dtype=torch.int32, device=self.stack.dev)
        self.dist.all_reduce(ok, op=self.dist.ReduceOp.MIN, group=self.group)   # also: every slot and flag is zero before anyone signals
        torch.cuda.synchronize()
        if int(ok[0]) == 0:
            sys.stderr.write("peer-memory ring not available on every rank (%s): sums across GPUs go through NCCL\n" % (why or "a peer failed"))
            return None
        ring = L.Ring()
        ring.nrank, ring.rank = self.stack.ncard, self.stack.card
        for r in range(self.stack.ncard):
            ring.slot[0][r], ring.slot[1][r] = ptrs[r], ptrs[r] + count * 4
            ring.pad[r] = ptrs[r] + 2 * count * 4
            ll0 = ptrs[r] + (2 * count + 64) * 4   # 8-byte aligned: count is even
            ring.ll[0][r], ring.ll[1][r] = ll0, ll0 + self.stack.ncard * count * 8
        ring.ll_count = count
        self.ring_state = torch.zeros(4, dtype=torch.int32, device=self.stack.dev)
        ring.state = self.ring_state.data_ptr()
        ring.spin_limit = 1 << 20   # about a second of polling before a missing peer is reported
        self.ring_keep = (buf, hdl)
        return ring

    def _enqueue(self):
        st, stack, T = torch.cuda.current_stream().cuda_stream, self.stack, self.T
        if self.side is not None:
            L.call("fnx_window_side_stream", self.side.cuda_stream, self.ev_fork.cuda_event, self.ev_join.cuda_event)
        else:
            L.call("fnx_window_side_stream", None, None, None)
        L.call("fnx_window_ring", C.byref(self.ring) if self.ring is not None else None)
        self.ctl.copy_(self.ctl_in)
        if stack.shape.draft:
            L.call("fnx_embed_rows", stack.embed.data_ptr(), self.ids.data_ptr(), self.demb.data_ptr(), T, stack.shape.n, st)
            L.call("fnx_draft_begin", C.byref(stack.cfg), C.byref(stack.draft), stack.ws.data_ptr(), self.src.data_ptr(), self.demb.data_ptr(), T, st)
        else:
            L.call("fnx_embed_rows", stack.embed.data_ptr(), self.ids.data_ptr(), self.x.data_ptr(), T, stack.shape.n, st)
        for i in range(self.nstages):
            if self.lanes is not None:
                L.call("fnx_window_stage_lanes", C.byref(stack.cfg), stack.layers, C.byref(stack.head), stack.ws.data_ptr(), C.byref(self.lanes.c),
                       i, st)
            else:
                L.call("fnx_window_stage", C.byref(stack.cfg), stack.layers, C.byref(stack.head), stack.ws.data_ptr(), T, i, st)
            if self.dist is None:
                continue
            if self.after[i] == 1:
                if self.ring is not None:
                    L.call("fnx_ring_sum", self.bo.data_ptr(), T, stack.shape.n, C.byref(self.ring), self.err.data_ptr(), st)
                else:
                    self.dist.all_reduce(self.bo, group=self.group)
            elif self.after[i] == 2:
                per = self.partials.numel() // stack.ncard
                self.dist.all_gather_into_tensor(self.partials, self.partials[stack.card * per:(stack.card + 1) * per], group=self.group)
        if self.sampled:   # no penalties: the candidates of the plain logits (reference Engine::top_tokens)
            L.call("fnx_top_tokens", self.logits.data_ptr(), stack.vrows, T, stack.v0, None, None, None, 0, None, self.cand_v.data_ptr(),
                   self.cand_i.data_ptr(), self.err.data_ptr(), st)
        if self.dist is None:
            self.all_v[0].copy_(self.best_v)
            self.all_i[0].copy_(self.best_i)
            if self.sampled:
                self.all_cv[0].copy_(self.cand_v)
                self.all_ci[0].copy_(self.cand_i)
        elif self.ring is not None:   # the library's own small all-gather over the ring's slots: no NCCL call in a window
            L.call("fnx_ring_gather", self.best_v.data_ptr(), T, self.best_i.data_ptr(), T, C.byref(self.ring), self.all_v.data_ptr(),
                   self.all_i.data_ptr(), self.err.data_ptr(), st)
            if self.sampled:
                nc = T * L.TOPK_N
                L.call("fnx_ring_gather", self.cand_v.data_ptr(), nc, self.cand_i.data_ptr(), nc, C.byref(self.ring), self.all_cv.data_ptr(),
                       self.all_ci.data_ptr(), self.err.data_ptr(), st)
        else:
            self.dist.all_gather_into_tensor(self.all_v.view(-1), self.best_v, group=self.group)
            self.dist.all_gather_into_tensor(self.all_i.view(-1), self.best_i, group=self.group)
            if self.sampled:
                self.dist.all_gather_into_tensor(self.all_cv.view(-1), self.cand_v.view(-1), group=self.group)
                self.dist.all_gather_into_tensor(self.all_ci.view(-1), self.cand_i.view(-1), group=self.group)
        self.d_out[-1:].copy_(self.err)

    def launch(self):
        """Enqueues one window on the runner's stream (the caller has set ids and ctl)."""
        with torch.cuda.stream(self.stream):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._enqueue()

    def window(self, rows, pos0, tag):
        """One window from host token ids: uploads ids and (position, tag), runs, reads back every row's argmax (merged
        across GPUs: the lower GPU wins a tie) and the error word.  Returns the argmax tokens as a list."""
        T = self.T
        if pos0 + T > self.stack.shape.ctx + self.stack.shape.kv_slack:
            raise L.FnxError("window at position %d + %d rows is past the K/V cache (%d positions)" %
                             (pos0, T, self.stack.shape.ctx + self.stack.shape.kv_slack))
        self.h_in_np[:T] = rows
        self.h_in_np[L.MAXT], self.h_in_np[L.MAXT + 1] = pos0, tag
        return self._run()

    def _run(self):
        """Uploads the host's ids and control words, runs the window, reads the result back and merges it."""
        with torch.cuda.stream(self.stream):
            self.d_in.copy_(self.h_in, non_blocking=True)
            self.launch()
            self.h_out.copy_(self.d_out, non_blocking=True)
        self.stream.synchronize()
        err = int(self.h_err[0])
        if err != 0:
            with torch.cuda.stream(self.stream):
                self.err.zero_()   # reported: the next window starts clean
            self.stream.synchronize()
            raise L.FnxError("window error word %d (bit 1: a peer's addend never came; bit 8: a bounded on-chip wait ran out; bit 16: a "
                             "non-finite logit); the window's results are not to be used, the next window starts clean" % err)
        return self.merge_best()

    def draft_chain(self, src_row, token, pos0, k, tag):
        """A draft (MTP) layer's runner with T = 1: k tokens one after the other, as the reference's session drafts them
        (src/engine_common.cu:1197-1205 draft: the first step from a window's stream row, every later one from the draft
        layer's own streams as its last window left them; each step's token = the step before's argmax).  src_row:
        [hc n] floats on the device; returns the k drafted head rows (indices into the draft vocabulary)."""
        assert self.stack.shape.draft and self.T == 1, "a draft layer's runner of one row"
        streams = self.stack.buf(10, torch.float32, self.stack.shape.hc * self.stack.shape.n)
        out = []
        with torch.cuda.stream(self.stream):
            self.src[0].copy_(src_row.reshape(-1))
        for i in range(k):
            tok = self.window([token], pos0 + i, tag)[0]
            out.append(tok)
            token = tok
            with torch.cuda.stream(self.stream):
                self.src[0].copy_(streams)
        return out

    def window_lanes(self, rows, pos, tags):
        """One window of several sequences: rows = the T token ids (lane i's rows at i * lanes.rows ..), pos[i] / tags[i]
        lane i's first position and window tag.  Returns every row's argmax."""
        T, ln = self.T, self.lanes
        assert ln is not None, "build the runner with lanes=LaneSet(...)"
        for p in pos:
            if (p + ln.rows - 1) // 4 // self.stack.ncard * 4 + 4 > ln.region:
                raise L.FnxError("a lane at position %d + %d rows is past its run of K/V pages (%d local rows)" % (p, ln.rows, ln.region))
        self.h_in_np[:T] = rows
        with torch.cuda.stream(self.stream):
            ln.positions(pos, tags)
        return self._run()

    def commit_lanes(self, n, tags):
        """Keep the first n[i] rows of lane i of the last window."""
        ln = self.lanes
        nn, tt = (C.c_int * ln.nseg)(*n), (C.c_int * ln.nseg)(*tags)
        jobs = torch.zeros(len(self.stack.shape.kinds) * 2 * L.MAXT * C.sizeof(L.CopyJob), dtype=torch.uint8).pin_memory()
        with torch.cuda.stream(self.stream):
            L.call("fnx_window_commit_lanes", C.byref(self.stack.cfg), self.stack.layers, self.stack.ws.data_ptr(), C.byref(ln.c), nn, tt,
                   jobs.data_ptr(), torch.cuda.current_stream().cuda_stream)
        self.stream.synchronize()   # the job table is read by an asynchronous copy

    def merge_best(self):
        if self.stack.ncard == 1:
            return self.h_i_np[0].tolist()
        return merge_best(self.h_v_np, self.h_i_np)

    def window_sampled(self, rows, pos0, tag, rng, temperature=1.0, top_p=1.0, min_p=0.0, top_k=0):
        """One window with rejection-sampling acceptance against the fixed (one-hot) drafts rows[1:]: runs the window,
        reads back every GPU's 64 candidates per row, merges them and runs the reference's acceptance loop
        (src/session.cpp:469-510) with the caller's random stream (fnx_rng_new).  Returns (the emitted tokens, their
        number); the caller commits that many rows."""
        assert self.sampled, "build the runner with sampled=True"
        T, lib = self.T, L.load()
        self.window(rows, pos0, tag)
        with torch.cuda.stream(self.stream):
            self.h_cv.copy_(self.all_cv, non_blocking=True)
            self.h_ci.copy_(self.all_ci, non_blocking=True)
        self.stream.synchronize()
        mv = (C.c_float * (T * L.TOPK_N))()
        mi = (C.c_int * (T * L.TOPK_N))()
        if lib.fnx_top_merge(self.h_cv.data_ptr(), self.h_ci.data_ptr(), self.stack.ncard, T, mv, mi) != 0:
            raise L.FnxError(lib.fnx_last_error().decode())
        sp = L.Sampling(temperature, top_p, min_p, top_k)
        rc, out = (C.c_int * T)(*[int(r) for r in rows]), (C.c_int * T)()
        n = lib.fnx_accept_sampled(rc, T, mv, mi, C.byref(sp), rng, out)
        if n < 0:
            raise L.FnxError(lib.fnx_last_error().decode())
        return list(out[:n]), n

    def commit(self, n, tag):
        """Keep the first n rows of the last window: the DeltaNet layers' states and histories as after row n - 1 (with a
        replay log the states advance only here, also when every row is kept)."""
        if n >= self.T and not self.stack.gdn_log:
            return
        slot = self.commits % 64   # the table is read by an asynchronous copy: a slot is reused only 64 commits later
        self.commits += 1
        if slot == 0 and self.commits > 1:
            self.stream.synchronize()
        L.call("fnx_window_commit", C.byref(self.stack.cfg), self.stack.layers, self.stack.ws.data_ptr(), self.T, n, tag,
               self.h_jobs.data_ptr() + slot * self.job_bytes, self.stream.cuda_stream)

    def close(self):
        """Releases what must go before the process group does: the captured graph (its NCCL nodes hold the communicator)
        and the peer-mapped buffers of the sum across GPUs."""
        torch.cuda.synchronize()
        self.graph = None
        self.ring = None
        self.ring_keep = None
        torch.cuda.synchronize()

    def ring_self_check(self, rounds=8, seed=0):
        """The sum across GPUs on the real peers: every rank makes all ranks' seeded addends, runs `rounds` sums back to
        back on its own addend through this runner's ring - even rounds by fnx_ring_sum (slots and flags), odd rounds by the
        window's own exchange, fnx_boundary_rows on a zero x (value + exchange-number words into the peers' receive
        areas); both parities, the exchange numbers running on - and compares the bits with the same chunks added in the
        ring's order by plain elementwise float adds.  Returns {"rounds", "bits_equal", "err"}; None when the sums go
        through NCCL."""
        if self.ring is None:
            return None
        n, me, T, width = self.stack.ncard, self.stack.card, self.T, self.stack.shape.n
        NP = width // 2
        ok, err = True, 0
        x = torch.empty(T * width, dtype=torch.float32, device=self.stack.dev)
        errw = torch.zeros(1, dtype=torch.int32, device=self.stack.dev)
        ones = torch.ones(width, dtype=torch.float32, device=self.stack.dev)
        with torch.cuda.stream(self.stream):
            for r in range(rounds):
                g = torch.Generator(device=self.stack.dev)
                g.manual_seed(seed * 1000 + r)
                adds = torch.randn((n, T, width), generator=g, device=self.stack.dev) * (10.0 ** (r % 3))
                want = torch.empty((T, width), dtype=torch.float32, device=self.stack.dev)
                for c in range(n):   # chunk c: float pairs [c NP / n, (c + 1) NP / n) of every row, started by GPU c
                    lo, hi = 2 * (c * NP // n), 2 * ((c + 1) * NP // n)
                    acc = adds[c, :, lo:hi].clone()
                    for k in range(1, n):
                        acc = acc + adds[(c + k) % n, :, lo:hi]
                    want[:, lo:hi] = acc
                if r % 2 == 0:
                    x.copy_(adds[me].reshape(-1))
                    L.call("fnx_ring_sum", x.data_ptr(), T, width, C.byref(self.ring), errw.data_ptr(), self.stream.cuda_stream)
                else:   # x = 0 + sum: the sum's bits (no addend here is a zero)
                    x.zero_()
                    mine = adds[me].contiguous()
                    L.call("fnx_boundary_rows", x.data_ptr(), mine.data_ptr(), None, C.byref(self.ring), ones.data_ptr(), None, None, T, width,
                           1e-6, errw.data_ptr(), self.stream.cuda_stream)
                ok = ok and bool(torch.equal(x.view(torch.int32), want.reshape(-1).view(torch.int32)))
            self.stream.synchronize()
            err = int(errw[0])
        return {"rounds": rounds, "bits_equal": ok, "err": err}

    h2d_bytes = property(lambda self: (L.MAXT + 2) * 4)
    d2h_bytes = property(lambda self: self.stack.ncard * self.T * 8 + 4)
