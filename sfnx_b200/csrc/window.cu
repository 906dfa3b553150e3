// The window: one verify window of T rows over a stack of layers, enqueued stage by stage on a stream, and the
// rollback after acceptance.  Host code only (the counterpart of the reference's Engine::enqueue, ffn_half, attention
// and commit: src/engine.cu:900-1054, src/engine_common.cu:525-568); every kernel goes through the same C ABI entry
// points an external caller would use.  The stages end where the GPUs must exchange data, so that a caller driving
// several GPUs can put its collective between two stages.
#include <cstdlib>
#include <cstring>

#include <algorithm>

#include "common.cuh"
#include "moe_internal.cuh"

namespace fnxk {

static inline size_t al(size_t v) { return (v + 255) & ~(size_t) 255; }

// per-call timing of a window enqueued outside a graph: an event before and after every C ABI call of a stage (the
// engine's own per-window timers are the reference's counterpart, src/engine.hpp:182-187)
constexpr int TRACE_CAP = 4096;
struct Trace {
    bool on = false;
    int n = 0;
    cudaEvent_t ev[2 * TRACE_CAP];
    const char* name[TRACE_CAP];
    int layer[TRACE_CAP];
    bool made = false;
};
static Trace g_trace;

// a second stream beside the window's own, given by the caller (fnx_window_side_stream): the shared expert runs on it
// beside the router and the routed experts, the alpha/beta projection beside qkvz (the reference forks its st2 the same
// way, src/engine.cu:939-946, 1021-1026).  Fork and join are event records and waits: capture-safe.
struct Side {
    cudaStream_t st = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
static thread_local Side g_side;
static bool side_fork(void* st) {
    if (!g_side.st || g_trace.on) return false;   // a traced window stays on one stream: its events time single calls
    return cudaEventRecord(g_side.fork, (cudaStream_t) st) == cudaSuccess && cudaStreamWaitEvent(g_side.st, g_side.fork, 0) == cudaSuccess;
}
static int side_join(void* st) {
    if (cudaEventRecord(g_side.join, g_side.st) != cudaSuccess || cudaStreamWaitEvent((cudaStream_t) st, g_side.join, 0) != cudaSuccess)
        return fail("window: side stream join: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

// the peer-memory ring of the sum across GPUs, given by the caller (fnx_window_ring): with it a stage begins with the fused
// boundary kernel, which sums the ended half's addends itself, and the plan asks the caller for no sum between stages
static thread_local FnxRing g_ring;
static thread_local bool g_ring_set = false;
static bool fused_boundaries(const FnxStackCfg& c) { return c.ncard == 1 || g_ring_set; }

// FNX_EXACT=1: every kernel in the reference's order of sums (the window then equals the CPU statement of the reference bit
// for bit); default: the attention scan and the large dense projections run on the tcgen05 tensor cores in orders of their
// own (equal to fp32 rounding of the sums; the window is then held to the reference's KL bar).  FNX_ATTN_EXACT=1: the scan alone.
static bool env_on(const char* name) {
    const char* v = getenv(name);
    return v && v[0] == '1';
}
// a dense projection of the window: the tensor-core kernel where the shape is its and exactness is not asked for
static int dense(const FnxQ8S* ws, const int* rows, float* const* outs, int nseg, int cols, const void* xq, int T, void* st) {
    if (!env_on("FNX_EXACT")) {
        const int rc = q8s_umma_launch(ws, rows, outs, rows, nseg, cols, xq, T, strm(st), "window dense");
        if (rc >= 0) return rc;
    }
    return fnx_q8s_gemv_segs(ws, rows, outs, rows, nseg, cols, xq, T, st);
}

struct Traced {
    int slot = -1;
    cudaStream_t st;
    Traced(const char* name, int layer, void* stream) : st((cudaStream_t) stream) {
        if (!g_trace.on || g_trace.n >= TRACE_CAP) return;
        slot = g_trace.n++;
        g_trace.name[slot] = name;
        g_trace.layer[slot] = layer;
        cudaEventRecord(g_trace.ev[2 * slot], st);
    }
    ~Traced() {
        if (slot >= 0) cudaEventRecord(g_trace.ev[2 * slot + 1], st);
    }
};

// the workspace's buffers, as offsets from its base
struct Ws {
    size_t x, bo, xn, xq, qkvz, ab, yq, qg, k, v, att, partials, att_scratch, rlogits, topi, topw, jobs_gu, jobs_dn, njobs, rscratch, gu,
        hq, part, sh_gu, shq, sh, logits, keys, best_v, best_i, err, ctl, gdn_scratch, copy_jobs, replay_jobs, hc_R, hc_inj, hc_scratch, dr_en, dr_e2, dr_h2, dr_q, qsa_y, qsa_q, qsa_scores, qsa_cells, qsa_ncells, total;
};

static Ws carve(const FnxStackCfg& c) {
    Ws w;
    size_t o = 0;
    const size_t T = FNX_MAXT, n = c.n, P = T * c.topk;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o += al(bytes);
        return at;
    };
    const size_t gdn_rows = (size_t) (2 * c.nk + 2 * c.nv) * FNX_HS, vwidth = (size_t) c.nv * FNX_HS, qwidth = (size_t) c.nq * c.hd;
    const size_t widest = vwidth > qwidth ? vwidth : qwidth;
    w.x = take(T * n * 4);
    w.bo = take(T * n * 4);
    w.xn = take(T * n * 4);
    w.xq = take(T * ((n > widest ? n : widest) / 32) * 36);
    w.qkvz = take(T * gdn_rows * 4);
    w.ab = take(T * 2 * c.nv * 4);
    w.yq = take(T * (widest / 32) * 36);
    w.qg = take(T * qwidth * 2 * 4);
    w.k = take(T * (size_t) c.nkv * c.hd * 4);
    w.v = take(T * (size_t) c.nkv * c.hd * 4);
    w.att = take(T * qwidth * 4);
    w.partials = take((size_t) c.ncard * T * c.nq * (c.hd + 2) * 4);
    w.att_scratch = take(fnx_attn_scratch_floats(c.nq, c.hd, (int) T) * 4);
    w.rlogits = take(T * (c.nexp + 1) * 4);
    w.topi = take(P * 4);
    w.topw = take(P * 4);
    w.jobs_gu = take(P * sizeof(FnxJob));
    w.jobs_dn = take(P * sizeof(FnxJob));
    w.njobs = take(16);
    w.rscratch = take(fnx_router_scratch_bytes());
    w.gu = take(P * 2 * (size_t) c.ff * 4);
    w.hq = take(fnx_moe_h_bytes((int) P, c.ff));
    w.part = take(P * n * 4);
    w.sh_gu = take(T * 2 * (size_t) c.ff * 4);
    w.shq = take(fnx_moe_h_bytes((int) T, c.ff));
    w.sh = take(T * n * 4);
    w.logits = take(T * (size_t) c.vocab_rows * 4);
    w.keys = take(2 * T * 8);
    w.best_v = take(T * 4);
    w.best_i = take(T * 4);
    w.err = take(16);
    w.ctl = take(16);
    w.gdn_scratch = take(fnx_gdn_scratch_floats(c.nv) * 4);
    w.copy_jobs = take((size_t) c.nlayers * 2 * FNX_MAXT * sizeof(FnxCopyJob));   // up to a lane a row
    w.replay_jobs = take((size_t) c.nlayers * sizeof(FnxGdnReplay));
    const size_t hcn = c.hc > 1 ? (size_t) c.hc : 0;   // hyper-connections: the residual streams, the two halves' inject values, the read's scratch
    w.hc_R = take(T * hcn * n * 4);
    w.hc_inj = take(2 * T * (hcn ? hcn : 1) * 4);
    w.hc_scratch = take(hcn ? fnx_hc_scratch_floats((int) T, c.n, c.hc, c.hc_lr) * 4 : 0);
    const size_t dr = c.r_preset ? hcn : 0;   // the draft layer's prologue: normed embeddings, both projections, the streams' q8_1 rows
    w.dr_en = take(dr ? T * n * 4 : 0);
    w.dr_e2 = take(dr ? T * n * 4 : 0);
    w.dr_h2 = take(T * dr * n * 4);
    w.dr_q = take(T * dr * (n / 32) * 36);
    const size_t qs = c.qsa_top > 0 ? 1 : 0;   // the block selection: projection, query heads, scores, cells and their counts
    w.qsa_y = take(qs * T * fnx_qsa_rows() * 4);
    w.qsa_q = take(qs * T * FNX_QSA_HEADS * FNX_QSA_DIM * 4);
    w.qsa_scores = take(qs * T * (size_t) (c.qsa_max_pools > 0 ? c.qsa_max_pools : 0) * 4);
    w.qsa_cells = take(qs * T * (size_t) fnx_qsa_maxsel(c.qsa_top > 0 ? c.qsa_top : 0) * 4);
    w.qsa_ncells = take(qs * T * 4);
    w.total = o;
    return w;
}

static int check_cfg(const FnxStackCfg* c) {
    if (!c) return fail("window: no configuration");
    if (c->n <= 0 || c->n % 512 || c->ff <= 0 || c->ff % 32 || c->nlayers < 1 || c->ncard < 1 || c->card < 0 || c->card >= c->ncard)
        return fail("window: hidden %d, ff slice %d, %d layers, GPU %d of %d", c->n, c->ff, c->nlayers, c->card, c->ncard);
    if (c->topk < 1 || c->topk > 16 || c->nq % c->ncard) return fail("window: top-%d, %d query heads over %d GPUs", c->topk, c->nq, c->ncard);
    if (c->hc > 1 && (c->hc > 8 || c->hc_lr < 32 || c->hc_lr % 32 || c->hc_lr > 512))
        return fail("window: %d residual streams with low rank %d (up to 8 streams, rank a multiple of 32 up to 512)", c->hc, c->hc_lr);
    if (c->qsa_top > 0 && (c->qsa_ring_rows < FNX_MAXT + FNX_QSA_POOL || c->qsa_max_pools < 1))
        return fail("window: block selection with a ring of %d rows and %d pooled keys", c->qsa_ring_rows, c->qsa_max_pools);
    return 0;
}

// stage s of the plan: which layer, which part (0 mixer / first attention part, 1 attention finish, 2 FFN, 3 head)
struct Stage {
    int layer, part;
};
static int plan(const FnxStackCfg& c, const FnxLayer* L, Stage* out, int* after, int max) {
    int s = 0;
    auto put = [&](int layer, int part, int aft) {
        if (s < max) {
            if (out) out[s] = Stage{layer, part};
            if (after) after[s] = aft;
        }
        ++s;
    };
    const int sum = fused_boundaries(c) ? FNX_AFTER_NONE : FNX_AFTER_SUM_BO;   // fused: the next stage's first kernel sums
    for (int l = 0; l < c.nlayers; ++l) {
        if (L[l].kind == 1) {
            put(l, 0, fused_boundaries(c) ? FNX_AFTER_NONE : FNX_AFTER_GATHER_PARTIALS);   // fused: the finish kernel reads the peers' partials itself
            put(l, 1, sum);
        } else {
            put(l, 0, sum);
        }
        put(l, 2, sum);
    }
    put(c.nlayers, 3, FNX_AFTER_GATHER_BEST);
    return s;
}

}  // namespace fnxk

using namespace fnxk;

#define TRY(call)         \
    do {                  \
        if (call) return 1; \
    } while (0)
// a traced call
#define TRK(name, call)                      \
    do {                                     \
        Traced tr_(name, sg.layer, st);      \
        if (call) return 1;                  \
    } while (0)

extern "C" {

size_t fnx_window_workspace_bytes(const FnxStackCfg* cfg) {
    if (check_cfg(cfg)) return 0;
    return carve(*cfg).total;
}

void* fnx_window_buf(const FnxStackCfg* cfg, void* ws, int which) {
    if (check_cfg(cfg) || !ws) return nullptr;
    const Ws w = carve(*cfg);
    char* b = (char*) ws;
    switch (which) {
        case FNX_BUF_X: return b + w.x;
        case FNX_BUF_BO: return b + w.bo;
        case FNX_BUF_PARTIALS: return b + w.partials;
        case FNX_BUF_BEST_V: return b + w.best_v;
        case FNX_BUF_BEST_I: return b + w.best_i;
        case FNX_BUF_ERR: return b + w.err;
        case FNX_BUF_CTL: return b + w.ctl;
        case FNX_BUF_LOGITS: return b + w.logits;
        case FNX_BUF_COPY_JOBS: return b + w.copy_jobs;
        case FNX_BUF_NJOBS: return b + w.njobs;
        case FNX_BUF_STREAMS: return b + w.hc_R;
    }
    fail("window_buf: no buffer %d", which);
    return nullptr;
}

int fnx_window_init(const FnxStackCfg* cfg, void* ws, void* st) {
    TRY(check_cfg(cfg));
    const Ws w = carve(*cfg);
    char* b = (char*) ws;
    auto zero = [&](size_t at, size_t bytes) { return cudaMemsetAsync(b + at, 0, bytes, strm(st)) != cudaSuccess; };
    if (zero(w.rscratch, fnx_router_scratch_bytes()) || zero(w.keys, 2 * FNX_MAXT * 8) || zero(w.err, 16) || zero(w.njobs, 16) ||
        zero(w.gdn_scratch, fnx_gdn_scratch_floats(cfg->nv) * 4))
        return fail("window_init: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

int fnx_window_plan(const FnxStackCfg* cfg, const FnxLayer* layers, int* after, int max) {
    if (check_cfg(cfg) || !layers) return -1;
    return plan(*cfg, layers, nullptr, after, max);
}

// one stage; lanes null: the rows are one sequence's
static int window_stage(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, int T, int stage, const FnxWindowLanes* lanes,
                        void* st) {
    TRY(check_cfg(cfg));
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "window: T %d outside 1..%d", T, FNX_MAXT);
    const FnxStackCfg& c = *cfg;
    Stage stages[1024];
    const int ns = plan(c, layers, stages, nullptr, 1024);
    FNX_REQUIRE(ns <= 1024 && stage >= 0 && stage < ns, "window: stage %d of %d", stage, ns);
    const Stage sg = stages[stage];
    const Ws w = carve(c);
    char* b = (char*) ws;
    float* x = (float*) (b + w.x);
    float* bo = (float*) (b + w.bo);
    float* xn = (float*) (b + w.xn);
    void* xq = b + w.xq;
    const int* ctl = (const int*) (b + w.ctl);
    // the previous half's output is still pending: every stage that reads x first folds it into x (not stage 0, and not
    // the attention's second part, which continues its own layer's mixer).  Fused: one kernel takes the ended half's rows
    // (a mixer's bo, or the experts' rows with their weights), sums them across the GPUs, updates x and norms it; else the
    // ended FFN half has combined its rows into bo, the caller has summed bo, and the norm kernel adds it.
    const float* pending = stage == 0 ? nullptr : bo;
    const bool fused = fused_boundaries(c);
    const bool after_ffn = stage > 0 && stages[stage - 1].part == 2;
    const FnxMoeRows moe_rows{(const float*) (b + w.part), (const float*) (b + w.topw), (const float*) (b + w.sh), (const float*) (b + w.rlogits), c.nexp, c.topk};
    // Hyper-connections (cfg.hc > 1; reference src/engine.cu:935, 1013-1016, 1049): the residual is hc streams R, a half
    // begins with the read that folds the ended half's output into R (its sum across the GPUs first) and mixes the
    // streams into the half's input; the two halves' inject values alternate between two buffers.
    const bool hcm = c.hc > 1;
    float* hcR = (float*) (b + w.hc_R);
    float* inj_buf[2] = {(float*) (b + w.hc_inj), (float*) (b + w.hc_inj) + (size_t) FNX_MAXT * (hcm ? c.hc : 1)};
    auto hc_begin = [&](const FnxHcW& hw, bool ffn_half) -> int {
        // the ended half's rows into bo: the experts' rows weighted and added, or the mixer's output as it is
        if (after_ffn && fused)   // (not fused: the FFN stage combined them itself, for the caller's sum)
            TRY(fnx_moe_combine((const float*) (b + w.part), (const float*) (b + w.topw), (const float*) (b + w.sh), (const float*) (b + w.rlogits), c.nexp, bo,
                                T, c.n, c.topk, st));
        if (pending && c.ncard > 1 && g_ring_set) TRY(fnx_ring_sum(bo, T, c.n, &g_ring, (unsigned*) (b + w.err), st));
        if (stage == 0 && !c.r_preset) TRY(fnx_hc_expand(x, hcR, T, c.n, c.hc, st));
        // a read before a mixer half (or the head's) takes the FFN half's inject values (buffer 1) and leaves its own in
        // buffer 0; a read before an FFN half the other way round
        const float* inj_prev = ffn_half ? inj_buf[0] : inj_buf[1];
        float* inj_out = ffn_half ? inj_buf[1] : inj_buf[0];
        return fnx_hc_read(hcR, pending, pending ? inj_prev : nullptr, hw.norm, hw.down, hw.up, hw.inj, c.eps, xn, hw.inj ? inj_out : nullptr,
                           (float*) (b + w.hc_scratch), xq, T, c.n, c.hc, c.hc_lr, st);
    };
    auto begin_half = [&](const float* norm_w, float* y) -> int {
        if (hcm) {
            if (sg.part == 3) return hc_begin(head->mix, false);
            return hc_begin(sg.part == 2 ? layers[sg.layer].hcw[1] : layers[sg.layer].hcw[0], sg.part == 2);
        }
        if (!fused) return fnx_rms_norm_rows(x, pending, norm_w, y, xq, T, c.n, c.eps, st);
        return fnx_boundary_rows(x, after_ffn ? nullptr : pending, after_ffn ? &moe_rows : nullptr, c.ncard > 1 ? &g_ring : nullptr, norm_w, y, xq, T, c.n,
                                 c.eps, (unsigned*) (b + w.err), st);
    };
    const char* begin_name = hcm ? "hc_read" : fused ? "boundary" : "rms_norm";
    if (sg.part == 3) {
        FNX_REQUIRE(head, "window: no head");
        TRK(begin_name, begin_half(head->norm, nullptr));
        float* logits = (float*) (b + w.logits);
        {
            const FnxQ8S ws1[1] = {head->out};
            const int rows1[1] = {c.vocab_rows};
            float* const outs1[1] = {logits};
            TRK("head", dense(ws1, rows1, outs1, 1, c.n, xq, T, st));
        }
        TRK("argmax", fnx_argmax(logits, c.vocab_rows, T, c.vocab0, (float*) (b + w.best_v), (int*) (b + w.best_i),
                                    (unsigned long long*) (b + w.keys), (unsigned*) (b + w.err), st));
        return 0;
    }
    const FnxLayer& L = layers[sg.layer];
    if (sg.part == 0 && L.kind == 0) {   // Gated DeltaNet mixer
        const int rows = (2 * c.nk + 2 * c.nv) * FNX_HS;
        TRK(begin_name, begin_half(L.norm1, xn));
        const bool forked = side_fork(st);
        TRK("ab", fnx_gemv_f32(L.ab, xn, (float*) (b + w.ab), 2 * c.nv, c.n, T, forked ? (void*) g_side.st : st));
        {
            const FnxQ8S ws1[1] = {L.qkvz};
            const int rows1[1] = {rows};
            float* const outs1[1] = {(float*) (b + w.qkvz)};
            TRK("qkvz", dense(ws1, rows1, outs1, 1, c.n, xq, T, st));
        }
        if (forked) TRY(side_join(st));
        if (lanes) {   // every lane's rows chain through that lane's state, all lanes in one launch
            const FnxGdnLanes gl{lanes->S[sg.layer], lanes->hist[sg.layer], lanes->ctl, lanes->row0, L.snap, L.hsnap};
            TRK("gdn_core", fnx_gdn_core_segs((const float*) (b + w.qkvz), (const float*) (b + w.ab), L.conv, L.dt, L.a, L.ssm_norm, b + w.yq,
                                                 (float*) (b + w.gdn_scratch), c.nk, c.nv, L.vmap, &gl, lanes->nseg, lanes->rows, c.eps, st));
        } else if (L.gdn_log) {   // no checkpoints: the commit replays the kept rows from the log
            TRK("gdn_core", fnx_gdn_core_log((const float*) (b + w.qkvz), (const float*) (b + w.ab), L.hist, L.conv, L.dt, L.a, L.ssm_norm, L.S,
                                                b + w.yq, ctl, (float*) (b + w.gdn_scratch), L.gdn_log, L.hsnap, c.nk, c.nv, L.vmap, T, c.eps, st));
        } else
            TRK("gdn_core", fnx_gdn_core((const float*) (b + w.qkvz), (const float*) (b + w.ab), L.hist, L.conv, L.dt, L.a, L.ssm_norm, L.S,
                                            b + w.yq, ctl, (float*) (b + w.gdn_scratch), L.snap, L.hsnap, c.nk, c.nv, L.vmap, T, c.eps, st, nullptr));
        TRK("ssm_out", fnx_q8s_gemv(L.ssm_out, c.n, c.nv * FNX_HS, b + w.yq, bo, c.n, T, st));
        return 0;
    }
    if (sg.part == 0) {   // attention, up to this GPU's partials
        float* qg = (float*) (b + w.qg);
        float* k = (float*) (b + w.k);
        float* v = (float*) (b + w.v);
        const bool select = c.qsa_top > 0 && L.idx.wq;
        FNX_REQUIRE(!select || !lanes || (lanes->idx_ring_host && lanes->idx_ring_host[sg.layer]), "window: layer %d selects blocks but the lanes bring no raw-key rings",
                    sg.layer);
        TRK(begin_name, begin_half(L.norm1, select ? xn : nullptr));
        {   // q, k and v in one launch
            const FnxQ8S ws[3] = {L.wq, L.wk, L.wv};
            const int rows3[3] = {c.nq * c.hd * 2, c.nkv * c.hd, c.nkv * c.hd};
            float* const outs[3] = {qg, k, v};
            TRK("wqkv", dense(ws, rows3, outs, 3, c.n, xq, T, st));
        }
        const FnxRope rope{c.rope_base, c.nrot};
        float* mine = (float*) (b + w.partials) + (size_t) c.card * T * c.nq * (c.hd + 2);
        if (lanes) {
            // norm, rotary and append lane by lane (the lane's position and pages), then every row's partial at once, each
            // on its lane's position and pages, in the reference's order of sums (reference src/engine.cu:1186-1200)
            for (int sI = 0; sI < lanes->nseg; ++sI) {
                const size_t r0 = (size_t) sI * lanes->rows;
                FnxKvPages pg = L.pages;
                pg.pt = lanes->pt_host[sI];
                TRK("attn_prep_append", fnx_attn_prep_append(qg + r0 * c.nq * 2 * c.hd, k + r0 * c.nkv * c.hd, v + r0 * c.nkv * c.hd, L.q_norm, L.k_norm,
                                                                L.kc, L.vc, pg, c.card, c.ncard, lanes->rows, lanes->ctl_host[sI], c.eps, rope, c.nq,
                                                                c.nkv, c.hd, st));
            }
            const FnxLaneRows lr{lanes->row_pos, lanes->row_pt};
            if (select) {   // the projection over all rows, every lane's rows indexed on its ring and pages, then every row on its lane's
                float* y = (float*) (b + w.qsa_y);
                float* iq = (float*) (b + w.qsa_q);
                int* cells = (int*) (b + w.qsa_cells);
                int* n_cells = (int*) (b + w.qsa_ncells);
                FnxKvPages kp = L.pages;   // the pooled keys' pages: the lanes' page tables over the keys' own pool
                if (L.idx.page) kp.page = L.idx.page;
                TRK("qsa", fnx_qsa_proj(L.idx.wq, L.idx.wk, xn, y, T, c.n, st));
                for (int sI = 0; sI < lanes->nseg; ++sI) {
                    const size_t r0 = (size_t) sI * lanes->rows;
                    FnxKvPages pg = kp;
                    pg.pt = lanes->pt_host[sI];
                    TRK("qsa", fnx_qsa_index(y + r0 * fnx_qsa_rows(), L.idx.qn, L.idx.kn, lanes->idx_ring_host[sg.layer][sI], c.qsa_ring_rows, L.idx.pooled, pg,
                                             c.ncard, iq + r0 * FNX_QSA_HEADS * FNX_QSA_DIM, lanes->ctl_host[sI], lanes->rows, c.eps, FnxRope{c.rope_base, 64}, st));
                }
                TRK("qsa", fnx_qsa_select(iq, L.idx.pooled, kp, lr, (float*) (b + w.qsa_scores), cells, n_cells, c.qsa_max_pools, nullptr, T, c.card,
                                          c.ncard, c.qsa_top, st));
                TRK("attn_partial", fnx_attn_partial_cells(qg, L.kc, L.vc, L.pages, lr, mine, c.card, c.ncard, T, nullptr, c.nq, c.nkv, c.hd,
                                                              (float*) (b + w.att_scratch), cells, n_cells, fnx_qsa_maxsel(c.qsa_top), st));
                return 0;
            }
            TRK("attn_partial", fnx_attn_part_lanes(qg, L.kc, L.vc, L.pages, lr, mine, c.card, c.ncard, T, c.nq, c.nkv, c.hd,
                                                       (float*) (b + w.att_scratch), st));
            return 0;
        }
        TRK("attn_prep_append", fnx_attn_prep_append(qg, k, v, L.q_norm, L.k_norm, L.kc, L.vc, L.pages, c.card, c.ncard, T, ctl, c.eps,
                                                        rope, c.nq, c.nkv, c.hd, st));
        if (select) {   // the indexer on the half's input (reference src/engine.cu:911-912), then the scan over every row's cells
            int* cells = (int*) (b + w.qsa_cells);
            int* n_cells = (int*) (b + w.qsa_ncells);
            TRK("qsa", fnx_qsa(L.idx.wq, L.idx.wk, xn, c.n, (float*) (b + w.qsa_y), L.idx.qn, L.idx.kn, L.idx.ring, c.qsa_ring_rows, L.idx.pooled,
                               L.pages, (float*) (b + w.qsa_q), (float*) (b + w.qsa_scores), cells, n_cells, c.qsa_max_pools, ctl, T, c.eps,
                               FnxRope{c.rope_base, 64},
                               c.card, c.ncard, c.qsa_top, st));
            TRK("attn_partial", fnx_attn_partial_cells(qg, L.kc, L.vc, L.pages, FnxLaneRows{nullptr, nullptr}, mine, c.card, c.ncard, T, ctl, c.nq,
                                                          c.nkv, c.hd, (float*) (b + w.att_scratch), cells, n_cells, fnx_qsa_maxsel(c.qsa_top), st));
            return 0;
        }
        // FNX_ATTN_EXACT=1: the scan in the reference's order of sums (bit-reproducible against the CPU statement, several
        // times slower); default: the one-pass tensor-core scan
        if (env_on("FNX_EXACT") || env_on("FNX_ATTN_EXACT"))
            TRK("attn_partial", fnx_attn_partial_exact(qg, L.kc, L.vc, L.pages, mine, c.card, c.ncard, T, ctl, c.nq, c.nkv, c.hd,
                                                          (float*) (b + w.att_scratch), st));
        else
            TRK("attn_partial", fnx_attn_partial(qg, L.kc, L.vc, L.pages, mine, c.card, c.ncard, T, ctl, c.nq, c.nkv, c.hd,
                                                    (float*) (b + w.att_scratch), st));
        return 0;
    }
    if (sg.part == 1) {   // attention: merge the GPUs' partials for this GPU's heads, gate, output projection
        const int own = c.nq / c.ncard;
        float* att = (float*) (b + w.att);
        if (fused) {   // one launch: exchange of the partials over peer memory (more than one GPU), merge, gate, q8_1 rows
            const float* mine = (const float*) (b + w.partials) + (size_t) c.card * T * c.nq * (c.hd + 2);
            TRK("attn_finish", fnx_attn_finish_ring(mine, c.ncard > 1 ? &g_ring : nullptr, (const float*) (b + w.qg), att, b + w.yq, T, c.nq, c.hd,
                                                       (unsigned*) (b + w.err), st));
        } else {
            TRK("attn_finish", fnx_attn_finish((const float*) (b + w.partials), c.ncard, c.card, (const float*) (b + w.qg), att, T, c.nq,
                                                  c.card * own, own, c.hd, st));
            TRK("quantize", fnx_quantize_q8_1(att, b + w.yq, own * c.hd, T, st));
        }
        TRK("wo", fnx_q8s_gemv(L.wo, c.n, own * c.hd, b + w.yq, bo, c.n, T, st));
        return 0;
    }
    // FFN half
    const int P = T * c.topk;
    float* rl = (float*) (b + w.rlogits);
    TRK(begin_name, begin_half(L.norm2, xn));
    const bool forked = side_fork(st);   // the shared expert beside the router and the routed experts
    if (forked)
        TRY(fnx_shared_expert(L.sh_gate_up, L.sh_down, xq, T, c.n, c.ff, (float*) (b + w.sh_gu), b + w.shq, (float*) (b + w.sh), g_side.st));
    TRK("router_route", fnx_router_route(L.router, xn, rl, T, c.n, c.nexp, c.topk, (int*) (b + w.topi), (float*) (b + w.topw),
                                            (FnxJob*) (b + w.jobs_gu), (FnxJob*) (b + w.jobs_dn), (int*) (b + w.njobs), b + w.rscratch, st));
    TRK("moe_gate_up", fnx_moe_gate_up(&L.gate_up, (const FnxJob*) (b + w.jobs_gu), (const int*) (b + w.njobs), P, xq, (float*) (b + w.gu), st));
    TRK("moe_down", fnx_moe_down(&L.down, (const FnxJob*) (b + w.jobs_dn), (const int*) (b + w.njobs), P, (const float*) (b + w.gu), P,
                                    b + w.hq, (float*) (b + w.part), st));
    if (forked) {
        TRY(side_join(st));
    } else {
        TRK("shared_expert", fnx_shared_expert(L.sh_gate_up, L.sh_down, xq, T, c.n, c.ff, (float*) (b + w.sh_gu), b + w.shq, (float*) (b + w.sh), st));
    }
    if (!fused)   // fused: the next stage's first kernel weighs and adds the experts' rows itself
        TRK("moe_combine", fnx_moe_combine((const float*) (b + w.part), (const float*) (b + w.topw), (const float*) (b + w.sh), rl, c.nexp, bo,
                                              T, c.n, c.topk, st));
    return 0;
}

// a stage with the window's error word as the sink of its kernels' bounded waits (bit 8), so that a wait that ran out
// shows in the word the host reads after the window
static int window_stage_sunk(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, int T, int stage,
                             const FnxWindowLanes* lanes, void* st) {
    if (check_cfg(cfg) || !ws) return fail("window: no configuration or workspace");
    const Ws w = carve(*cfg);
    unsigned* err = (unsigned*) ((char*) ws + w.err);
    // the word is sticky across windows (a device-timed replay reads it once at the end); the host clears it after it has
    // reported a fault (the reference's engine throws on it after every window, src/engine_impl.hpp:154-167)
    fault_sink(err);
    const int rc = window_stage(cfg, layers, head, ws, T, stage, lanes, st);
    fault_sink(nullptr);
    return rc;
}

int fnx_draft_begin(const FnxStackCfg* cfg, const FnxDraft* d, void* ws, const float* src, const float* emb, int T, void* st) {
    TRY(check_cfg(cfg));
    FNX_REQUIRE(cfg->hc > 1 && cfg->r_preset && d && ws && src && emb, "draft_begin: a stack with residual streams made ahead (hc > 1, r_preset), weights and rows");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "draft_begin: T %d outside 1..%d", T, FNX_MAXT);
    const FnxStackCfg& c = *cfg;
    const Ws w = carve(c);
    char* b = (char*) ws;
    float *en = (float*) (b + w.dr_en), *e2 = (float*) (b + w.dr_e2), *h2 = (float*) (b + w.dr_h2);
    uint8_t* dq = (uint8_t*) (b + w.dr_q);
    const size_t rowq = (size_t) (c.n / 32) * 36;
    // the tokens' embeddings: RMS norm, q8_1, fc_embedding
    TRY(fnx_rms_norm_rows(const_cast<float*>(emb), nullptr, d->norm_emb, en, b + w.xq, T, c.n, c.eps, st));
    TRY(fnx_q8s_gemv(d->fc_emb, c.n, c.n, b + w.xq, e2, c.n, T, st));
    // the source rows: one RMS norm over all streams, then every stream of every row through fc_hidden (hc T rows of n)
    TRY(fnx_rms_norm_rows(const_cast<float*>(src), nullptr, d->norm_hid, nullptr, dq, T, c.n * c.hc, c.eps, st));
    for (int r0 = 0; r0 < c.hc * T; r0 += FNX_MAXT)
        TRY(fnx_q8s_gemv(d->fc_hid, c.n, c.n, dq + (size_t) r0 * rowq, h2 + (size_t) r0 * c.n, c.n, std::min((int) FNX_MAXT, c.hc * T - r0), st));
    return fnx_hc_add_streams(h2, e2, (float*) (b + w.hc_R), T, c.n, c.hc, st);
}

int fnx_window_stage(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, int T, int stage, void* st) {
    return window_stage_sunk(cfg, layers, head, ws, T, stage, nullptr, st);
}

int fnx_window_stage_lanes(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, const FnxWindowLanes* lanes, int stage,
                           void* st) {
    FNX_REQUIRE(lanes && lanes->nseg >= 1 && lanes->rows >= 1 && lanes->nseg * lanes->rows <= FNX_MAXT, "window: %d lanes of %d rows (at most %d rows)",
                lanes ? lanes->nseg : 0, lanes ? lanes->rows : 0, FNX_MAXT);
    FNX_REQUIRE(lanes->ctl && lanes->row0 && lanes->row_pos && lanes->row_pt && lanes->ctl_host && lanes->pt_host && lanes->S && lanes->hist,
                "window: lanes without their tables");
    return window_stage_sunk(cfg, layers, head, ws, lanes->nseg * lanes->rows, stage, lanes, st);
}

// keeps the first n[s] rows of lane s: its state and history from the checkpoints of window row s rows + n[s] - 1
int fnx_window_commit_lanes(const FnxStackCfg* cfg, const FnxLayer* layers, void* ws, const FnxWindowLanes* lanes, const int* n, const int* tags,
                            void* host_jobs, void* st) {
    TRY(check_cfg(cfg));
    FNX_REQUIRE(lanes && n && tags && lanes->S_host && lanes->hist_host, "commit: no lanes");
    const FnxStackCfg& c = *cfg;
    const Ws w = carve(c);
    FnxCopyJob* hj = (FnxCopyJob*) host_jobs;
    FNX_REQUIRE(hj, "commit: no host job table");
    const size_t ch = (size_t) (2 * c.nk + c.nv) * FNX_HS, state = (size_t) c.nv * FNX_HS * FNX_HS;
    int nj = 0;
    for (int sI = 0; sI < lanes->nseg; ++sI) {
        FNX_REQUIRE(n[sI] >= 1 && n[sI] <= lanes->rows, "commit: %d of lane %d's %d rows", n[sI], sI, lanes->rows);
        if (n[sI] == lanes->rows) continue;
        const size_t row = (size_t) sI * lanes->rows + n[sI] - 1;
        const unsigned written = ((unsigned) tags[sI] & 1u) ^ 1u;
        for (int l = 0; l < c.nlayers; ++l) {
            if (layers[l].kind != 0) continue;
            hj[nj++] = FnxCopyJob{lanes->S_host[l][sI], layers[l].snap + row * state, state * 4};
            hj[nj++] = FnxCopyJob{lanes->hist_host[l][sI] + (size_t) written * 3 * ch, layers[l].hsnap + row * 3 * ch, 3 * ch * 4};
        }
    }
    if (!nj) return 0;
    FnxCopyJob* dj = (FnxCopyJob*) ((char*) ws + w.copy_jobs);
    if (cudaMemcpyAsync(dj, hj, (size_t) nj * sizeof(FnxCopyJob), cudaMemcpyHostToDevice, strm(st)) != cudaSuccess)
        return fail("commit: job table upload: %s", cudaGetErrorString(cudaGetLastError()));
    return fnx_copy_many(dj, nj, st);
}

int fnx_window_commit(const FnxStackCfg* cfg, const FnxLayer* layers, void* ws, int T, int n, int tag, void* host_jobs, void* st) {
    TRY(check_cfg(cfg));
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && n >= 1 && n <= T, "commit: %d of %d rows", n, T);
    const FnxStackCfg& c = *cfg;
    const Ws w = carve(c);
    FNX_REQUIRE(host_jobs, "commit: no host job table");
    // the host table: nlayers * 2 copy jobs, then nlayers replay jobs
    FnxCopyJob* hj = (FnxCopyJob*) host_jobs;
    FnxGdnReplay* hr = (FnxGdnReplay*) ((char*) host_jobs + (size_t) c.nlayers * 2 * sizeof(FnxCopyJob));
    const size_t ch = (size_t) (2 * c.nk + c.nv) * FNX_HS, state = (size_t) c.nv * FNX_HS * FNX_HS;
    const unsigned written = ((unsigned) tag & 1u) ^ 1u;   // the window read half (tag & 1) and wrote the other
    int nj = 0, nr = 0;
    for (int l = 0; l < c.nlayers; ++l) {
        if (layers[l].kind != 0) continue;
        if (layers[l].gdn_log) hr[nr++] = FnxGdnReplay{layers[l].S, layers[l].gdn_log, layers[l].vmap, c.nk, c.nv, 0, n};   // also when every row is kept
        else if (n < T) hj[nj++] = FnxCopyJob{layers[l].S, layers[l].snap + (size_t) (n - 1) * state, state * 4};
        if (n < T) hj[nj++] = FnxCopyJob{layers[l].hist + (size_t) written * 3 * ch, layers[l].hsnap + (size_t) (n - 1) * 3 * ch, 3 * ch * 4};
    }
    if (nj) {
        FnxCopyJob* dj = (FnxCopyJob*) ((char*) ws + w.copy_jobs);
        if (cudaMemcpyAsync(dj, hj, (size_t) nj * sizeof(FnxCopyJob), cudaMemcpyHostToDevice, strm(st)) != cudaSuccess)
            return fail("commit: job table upload: %s", cudaGetErrorString(cudaGetLastError()));
        TRY(fnx_copy_many(dj, nj, st));
    }
    if (nr) {
        FnxGdnReplay* dr = (FnxGdnReplay*) ((char*) ws + w.replay_jobs);
        if (cudaMemcpyAsync(dr, hr, (size_t) nr * sizeof(FnxGdnReplay), cudaMemcpyHostToDevice, strm(st)) != cudaSuccess)
            return fail("commit: replay table upload: %s", cudaGetErrorString(cudaGetLastError()));
        TRY(fnx_gdn_replay(dr, nr, c.nv, st));
    }
    return 0;
}

// the side stream and the two events the forks use (null stream: everything on the window's stream)
int fnx_window_side_stream(void* st2, void* ev_fork, void* ev_join) {
    if (st2 && (!ev_fork || !ev_join)) return fail("window_side_stream: a side stream needs its fork and join events");
    g_side.st = (cudaStream_t) st2;
    g_side.fork = (cudaEvent_t) ev_fork;
    g_side.join = (cudaEvent_t) ev_join;
    return 0;
}

// the ring of the sum across GPUs for the calling thread's windows (null: none; the plan then asks the caller to sum)
int fnx_window_ring(const FnxRing* ring) {
    g_ring_set = ring != nullptr && ring->nrank > 1;
    if (g_ring_set) g_ring = *ring;
    return 0;
}

// ---- per-call trace of windows enqueued outside a graph
int fnx_trace_begin(void) {
    if (!g_trace.made) {
        for (int i = 0; i < 2 * TRACE_CAP; ++i)
            if (cudaEventCreate(&g_trace.ev[i]) != cudaSuccess) return fail("trace: event create failed");
        g_trace.made = true;
    }
    g_trace.n = 0;
    g_trace.on = true;
    pdl_hold(true);   // traced kernels run one after the other
    return 0;
}
// stops tracing; after the stream has drained, fills ms[i], layer[i] and name pointers for the traced calls (up to cap);
// returns how many there were
int fnx_trace_end(float* ms, int* layer, const char** names, int cap) {
    g_trace.on = false;
    pdl_hold(false);
    int n = g_trace.n < cap ? g_trace.n : cap;
    for (int i = 0; i < n; ++i) {
        if (cudaEventSynchronize(g_trace.ev[2 * i + 1]) != cudaSuccess) return -1;
        cudaEventElapsedTime(&ms[i], g_trace.ev[2 * i], g_trace.ev[2 * i + 1]);
        layer[i] = g_trace.layer[i];
        names[i] = g_trace.name[i];
    }
    return n;
}
// kernels this library has launched since the last reset (reset != 0: read and zero): counted where each launch is checked
long fnx_window_kernel_count(int reset) { return launch_count(reset != 0); }

// ---- the partition rule (reference src/card_split.hpp:12-26)
int fnx_ff_lo(int ff, int n, int c) {
    const int B = ff / 32;
    return 32 * (c * (B / n) + (c < B % n ? c : B % n));
}
int fnx_vhead_card(int nkh, int nvh, int n, int v) {
    const int vpk = nvh / nkh;
    return ((v % nkh) * vpk + v / nkh) / (nvh / n);
}
int fnx_khead_first(int nkh, int nvh, int n, int c) { return c * (nvh / n) / (nvh / nkh); }
int fnx_khead_count(int nkh, int nvh, int n, int c) {
    const int vpk = nvh / nkh;
    return ((c + 1) * (nvh / n) - 1) / vpk - fnx_khead_first(nkh, nvh, n, c) + 1;
}
}
