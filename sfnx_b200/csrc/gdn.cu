// Gated DeltaNet core of the verify window, with per-row state checkpoints for the rollback.  Covers what reference
// src/gdn_core.cuh (k_gdn_core) computes, with the same decomposition of every sum (so each value can be checked bit for
// bit), in two launches:
//
//  k_gdn_prep   everything that does not touch the state, once per channel instead of once per block that needs it:
//               causal conv (width 4) + SiLU of every local q, k and v channel, the L2 norms of q and k per key head,
//               the rows' gates, and the conv history left by keeping rows 0..t (hsnap) or the whole window (the other
//               half of hist).  A block per (head slot, row): 128 threads = the head's 128 channels.
//  k_gdn_rows   the delta rule.  A head's 128 x 128 fp32 state lives in the registers of a cluster of two blocks (64
//               value columns each, 256 threads) for the whole window.  A column's 128 key rows are cut as the
//               reference cuts them - 4 parts of 32 rows, 4 interleaved partial sums each - and one thread holds, for
//               4 neighbouring columns, the 8 rows of one (part, partial sum): a column's 16 partial sums sit in 16
//               lanes of one warp, so both levels of the reference's tree are warp shuffles (xor 1, 2: the four
//               interleaved sums; xor 4, 8: the four parts) and the row loop has no barrier.  After each row but the
//               last the thread streams its 8 x 4 state values to the checkpoint as eight 16-byte stores (the dominant
//               HBM traffic: a state-sized write per row).  The two blocks then exchange their outputs' square sums
//               through distributed shared memory and each norms, gates and quantises its own columns.
//
// The state's loads are issued before the kernel ahead in the stream has finished (they depend on nothing in the window).
//
// Checkpoints or a log.  fnx_gdn_core keeps the reference's contract: the state after every row but the last is written
// out (15 state-sized writes a window) and the rollback copies one back.  fnx_gdn_core_log writes no state at all: it
// leaves the state as it was and logs each row's decay, key and delta (a few hundred KB), from which k_gdn_replay rebuilds
// the state after the accepted rows with the window's own operations, bit for bit: 3 state-sized transfers a window
// instead of 17 (+2 for a rollback).
#include <cooperative_groups.h>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int HS = FNX_HS;
constexpr int GR_CL = 2, GR_COLS = HS / GR_CL, GR_THREADS = 256, GR_WARPS = GR_THREADS / 32;   // blocks a head; columns a block

struct GdnArgs {
    const float *qkvz, *ab;
    float* hist;
    const float *convw, *dt, *a, *nw;
    float* S;
    uint8_t* yq;
    const int* ctl;
    float *scratch, *snap, *hsnap;
    int nk, nv;
    const int* vmap;
    int T;
    float eps;
    float* y32;
    // several sequences in one launch (grid row = segment): segment s's state, conv history and ctl, its rows from window
    // row row0[s] (row s when row0 is null); null lS: one sequence, the fields above
    float* const* lS;
    float* const* lhist;
    const int* const* lctl;
    const int* row0;
    // the replay log (fnx_gdn_core_log): with it the rows kernel writes neither checkpoints nor the new state, only each
    // row's delta; the keys and gates go into the log instead of the scratch, and fnx_gdn_replay rebuilds the state after
    // the first n rows from the untouched state
    float* log;
};

// the replay log of one layer and sequence: k [MAXT][nk][128] (permuted as the scratch's), gates [MAXT][nv][2], delta
// [MAXT][nv][128]: what S_t = g_t S_(t-1) + k_t (x) delta_t needs, row by row
struct GdnLog {
    float *k, *g, *delta;
};
__host__ __device__ inline GdnLog gdn_log(float* p, int nk, int nv) {
    GdnLog r;
    r.k = p;
    r.g = r.k + (size_t) FNX_MAXT * nk * HS;
    r.delta = r.g + (size_t) FNX_MAXT * nv * 2;
    return r;
}

// scratch (by window row): q [MAXT][nk][128] and k likewise, each head's 128 values permuted so that the 8 rows a thread of
// k_gdn_rows needs are neighbours (element r = 32 part + 4 i + j at part * 32 + j * 8 + i); v [MAXT][nv][128]; gates
// [MAXT][nv][2] (decay, beta)
struct GdnScratch {
    float *q, *k, *v, *g;
};
__host__ __device__ inline GdnScratch gdn_scratch(float* s, int nk, int nv) {
    GdnScratch r;
    r.q = s;
    r.k = r.q + (size_t) FNX_MAXT * nk * HS;
    r.v = r.k + (size_t) FNX_MAXT * nk * HS;
    r.g = r.v + (size_t) FNX_MAXT * nv * HS;
    return r;
}

// block (head slot, row t, segment): slots [0, nk) the q heads, [nk, 2 nk) the k heads, then the nv v heads
__global__ void __launch_bounds__(HS) k_gdn_prep(const GdnArgs g) {
    const int slot = blockIdx.x, t = blockIdx.y, i = threadIdx.x, lane = i & 31, warp = i >> 5, nk = g.nk, nv = g.nv, T = g.T;
    const int ch = (2 * nk + nv) * HS, row_stride = ch + nv * HS, c = slot * HS + i;
    float* hist = g.hist;
    const int* ctl = g.ctl;
    int r0 = 0;
    if (g.lS) {
        const int seg = blockIdx.z;
        hist = g.lhist[seg], ctl = g.lctl[seg], r0 = g.row0 ? g.row0[seg] : seg;
    }
    const float4 cw = *reinterpret_cast<const float4*>(g.convw + (size_t) c * 4);   // older than the window
    pdl_wait();
    pdl_go();
    const unsigned parity = ((const unsigned*) ctl)[1] & 1u;
    const float* hin = hist + (size_t) parity * 3 * ch;
    const float* rows = g.qkvz + (size_t) r0 * row_stride;
    float in[4];   // the four taps: the window's rows t - 3 .. t, from the history before row 0
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int tt = t - 3 + k;
        in[k] = tt >= 0 ? rows[(size_t) tt * row_stride + c] : hin[(size_t) (tt + 3) * ch + c];
    }
    float x = fmul(cw.x, in[0]);
    x = ffma(cw.y, in[1], x);
    x = ffma(cw.z, in[2], x);
    x = ffma(cw.w, in[3], x);
    const float y = ex_silu(x);
    {   // the history if only rows 0..t are kept; after the last row, the new one
        float* h = t + 1 < T ? g.hsnap + (size_t) (r0 + t) * 3 * ch : hist + (size_t) (parity ^ 1u) * 3 * ch;
        h[c] = in[1], h[(size_t) ch + c] = in[2], h[(size_t) 2 * ch + c] = in[3];
    }
    GdnScratch sc = gdn_scratch(g.scratch, nk, nv);
    if (g.log) {
        const GdnLog lg = gdn_log(g.log, nk, nv);
        sc.k = lg.k, sc.g = lg.g;
    }
    if (slot < 2 * nk) {   // L2 norm over the head: 32-element groups by warp trees, the four groups added in order
        __shared__ float gs[4];
        const float w = wsum(fmul(y, y));
        if (lane == 0) gs[warp] = w;
        __syncthreads();
        const float sq = fadd(fadd(fadd(fadd(0.f, gs[0]), gs[1]), gs[2]), gs[3]);
        const float v = fmul(y, ex_rsqrt(fadd(sq, 1e-6f)));
        const int kh = slot < nk ? slot : slot - nk, part = i >> 5, ii = (i >> 2) & 7, j = i & 3;
        (slot < nk ? sc.q : sc.k)[((size_t) (r0 + t) * nk + kh) * HS + part * 32 + j * 8 + ii] = v;
    } else {
        const int lv = slot - 2 * nk;
        sc.v[((size_t) (r0 + t) * nv + lv) * HS + i] = y;
        if (i == 0) {
            const float* abt = g.ab + (size_t) (r0 + t) * 2 * nv;
            const float xg = fadd(abt[lv], g.dt[lv]);
            const float sp = xg > 20.0f ? xg : ex_log1pf_pos(ex_expf(xg));
            sc.g[((size_t) (r0 + t) * nv + lv) * 2] = ex_expf(fmul(sp, g.a[lv]));
            sc.g[((size_t) (r0 + t) * nv + lv) * 2 + 1] = fdiv(1.0f, fadd(1.0f, ex_expf(-abt[nv + lv])));
        }
    }
}

__device__ __forceinline__ void stcs4(float* p, float a, float b, float c, float d) { __stcs(reinterpret_cast<float4*>(p), make_float4(a, b, c, d)); }

__global__ void __cluster_dims__(GR_CL, 1, 1) __launch_bounds__(GR_THREADS, 1) k_gdn_rows(const GdnArgs g) {
    namespace cg = cooperative_groups;
    const int lv = blockIdx.x / GR_CL, half = blockIdx.x % GR_CL, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vm = g.vmap[lv], kh = vm & 255, nk = g.nk, nv = g.nv, T = g.T;
    const int ch = (2 * nk + nv) * HS, row_stride = ch + nv * HS;
    float* S = g.S;
    int r0 = 0;
    if (g.lS) {
        const int seg = blockIdx.y;
        S = g.lS[seg], r0 = g.row0 ? g.row0[seg] : seg;
    }
    // lane = j + 4 part + 16 (column quad & 1); warp w holds column quads 2 w, 2 w + 1 of the block's 16
    const int j = lane & 3, part = (lane >> 2) & 3, cq = 2 * warp + (lane >> 4), col = half * GR_COLS + 4 * cq;
    float* st = S + (size_t) lv * HS * HS + (size_t) (part * 32 + j) * HS + col;   // row 32 part + 4 i + j at st + 4 i HS
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(st + (size_t) 4 * i * HS));
        s[i][0] = v.x, s[i][1] = v.y, s[i][2] = v.z, s[i][3] = v.w;
    }
    __shared__ __align__(16) float qs[FNX_MAXT][HS], ks[FNX_MAXT][HS];   // permuted as the prep kernel wrote them
    __shared__ __align__(16) float vs[FNX_MAXT][GR_COLS], osm[FNX_MAXT][GR_COLS];
    __shared__ float gates[FNX_MAXT][2];
    __shared__ float sqs[FNX_MAXT][2];   // per row: the square sums of this block's two 32-column quarters
    pdl_wait();
    pdl_go();
    GdnScratch sc = gdn_scratch(g.scratch, nk, nv);
    float* dlog = nullptr;
    if (g.log) {
        const GdnLog lg = gdn_log(g.log, nk, nv);
        sc.k = lg.k, sc.g = lg.g;
        dlog = lg.delta + ((size_t) r0 * nv + lv) * HS + col;
    }
    for (int e = tid; e < T * (HS / 4); e += GR_THREADS) {
        const int t = e / (HS / 4), c4 = e % (HS / 4);
        const size_t at = ((size_t) (r0 + t) * nk + kh) * HS + 4 * c4;
        *reinterpret_cast<float4*>(&qs[t][4 * c4]) = *reinterpret_cast<const float4*>(sc.q + at);
        *reinterpret_cast<float4*>(&ks[t][4 * c4]) = *reinterpret_cast<const float4*>(sc.k + at);
    }
    for (int e = tid; e < T * (GR_COLS / 4); e += GR_THREADS) {
        const int t = e / (GR_COLS / 4), c4 = e % (GR_COLS / 4);
        *reinterpret_cast<float4*>(&vs[t][4 * c4]) = *reinterpret_cast<const float4*>(sc.v + ((size_t) (r0 + t) * nv + lv) * HS + half * GR_COLS + 4 * c4);
    }
    if (tid < 2 * T) gates[tid >> 1][tid & 1] = sc.g[((size_t) (r0 + (tid >> 1)) * nv + lv) * 2 + (tid & 1)];
    // what the epilogue's (row, 32-column block) tasks of this warp need from global memory, asked for now: the gate
    // inputs z and the norm weights would otherwise be a dependent load at the head of every task
    const float* qkvz = g.qkvz + (size_t) r0 * row_stride;
    constexpr int NTASK = 2 * FNX_MAXT / GR_WARPS;
    float zpre[NTASK], nwpre[2];
#pragma unroll
    for (int k = 0; k < NTASK; ++k) {
        const int task = warp + k * GR_WARPS, t = task >> 1, b = task & 1;
        zpre[k] = t < T ? qkvz[(size_t) t * row_stride + ch + lv * HS + half * GR_COLS + 32 * b + lane] : 0.f;
    }
    nwpre[0] = g.nw[half * GR_COLS + lane], nwpre[1] = g.nw[half * GR_COLS + 32 + lane];
    __syncthreads();
    const float scale = ex_rsqrt((float) HS);
    float* snap = g.snap ? g.snap + ((size_t) r0 * nv + lv) * HS * HS + (st - (S + (size_t) lv * HS * HS)) : nullptr;
    auto tree = [](float v) {   // (p0 + p1) + (p2 + p3) over the interleaved sums, then the same over the parts
        v = fadd(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fadd(v, __shfl_xor_sync(0xffffffffu, v, 2));
        v = fadd(v, __shfl_xor_sync(0xffffffffu, v, 4));
        return fadd(v, __shfl_xor_sync(0xffffffffu, v, 8));
    };
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float gv = gates[t][0], bv = gates[t][1];
        float kx[8], qx[8];
        {
            const float4 k0 = *reinterpret_cast<const float4*>(&ks[t][part * 32 + j * 8]), k1 = *reinterpret_cast<const float4*>(&ks[t][part * 32 + j * 8 + 4]);
            const float4 q0 = *reinterpret_cast<const float4*>(&qs[t][part * 32 + j * 8]), q1 = *reinterpret_cast<const float4*>(&qs[t][part * 32 + j * 8 + 4]);
            kx[0] = k0.x, kx[1] = k0.y, kx[2] = k0.z, kx[3] = k0.w, kx[4] = k1.x, kx[5] = k1.y, kx[6] = k1.z, kx[7] = k1.w;
            qx[0] = q0.x, qx[1] = q0.y, qx[2] = q0.z, qx[3] = q0.w, qx[4] = q1.x, qx[5] = q1.y, qx[6] = q1.z, qx[7] = q1.w;
        }
        const float4 vv = *reinterpret_cast<const float4*>(&vs[t][4 * cq]);
        const float vc[4] = {vv.x, vv.y, vv.z, vv.w};
        float delta[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float kj = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) kj = ffma(s[i][c], kx[i], kj);
            delta[c] = fmul(ffma(-gv, tree(kj), vc[c]), bv);
        }
        float o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float aj = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s[i][c] = ffma(kx[i], delta[c], fmul(gv, s[i][c]));
                aj = ffma(s[i][c], qx[i], aj);
            }
            o[c] = fmul(tree(aj), scale);
        }
        if ((lane & 15) == 0) {
            *reinterpret_cast<float4*>(&osm[t][4 * cq]) = make_float4(o[0], o[1], o[2], o[3]);
            if (dlog) *reinterpret_cast<float4*>(dlog + (size_t) t * nv * HS) = make_float4(delta[0], delta[1], delta[2], delta[3]);
        }
        if (!dlog && t < T - 1) {
            float* sp = snap + (size_t) t * nv * HS * HS;
#pragma unroll
            for (int i = 0; i < 8; ++i) stcs4(sp + (size_t) 4 * i * HS, s[i][0], s[i][1], s[i][2], s[i][3]);
        }
    }
    if (!dlog) {
#pragma unroll
        for (int i = 0; i < 8; ++i) *reinterpret_cast<float4*>(st + (size_t) 4 * i * HS) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
    }
    __syncthreads();
    if (tid < 2 * T) {   // a 32-column quarter's square sum: eight columns by a tree (a warp's butterfly over them), the four eights in order
        const int t = tid >> 1, qq = tid & 1;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float c[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) c[k] = fmul(osm[t][32 * qq + 8 * w + k], osm[t][32 * qq + 8 * w + k]);
            v = fadd(v, fadd(fadd(fadd(c[0], c[4]), fadd(c[2], c[6])), fadd(fadd(c[1], c[5]), fadd(c[3], c[7]))));
        }
        sqs[t][qq] = v;
    }
    // ---- gated RMS norm over the head's 128 outputs: the head's two blocks read each other's square sums through
    // distributed shared memory; each block then norms, gates and quantises its own columns (two q8_1 blocks per row)
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const float* sq0 = &cluster.map_shared_rank(&sqs[0][0], 0)[0];
    const float* sq1 = &cluster.map_shared_rank(&sqs[0][0], 1)[0];
#pragma unroll
    for (int k = 0; k < NTASK; ++k) {
        const int task = warp + k * GR_WARPS, t = task >> 1, b = task & 1;   // row, which of this block's two 32-column blocks
        if (t >= T) break;
        const float ms = fdiv(fadd(fadd(fadd(sq0[2 * t], sq0[2 * t + 1]), sq1[2 * t]), sq1[2 * t + 1]), (float) HS);
        const int c = half * GR_COLS + 32 * b + lane;
        const float v = osm[t][32 * b + lane];
        const float z = zpre[k];
        const float xi = fdiv(fmul(fmul(v, ex_rsqrt(fadd(ms, g.eps))), b ? nwpre[1] : nwpre[0]), fadd(1.0f, ex_expf(-z)));
        if (g.y32) g.y32[(size_t) (r0 + t) * nv * HS + lv * HS + c] = xi;
        const float amax = wmax(fabsf(xi)), sm = wsum(xi);
        const float d = fdiv(amax, 127.0f);
        uint8_t* blk = g.yq + ((size_t) (r0 + t) * (nv * HS / 32) + lv * 4 + 2 * half + b) * 36;
        reinterpret_cast<int8_t*>(blk + 4)[lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
        if (lane == 0) {
            reinterpret_cast<uint16_t*>(blk)[0] = f2h(d);
            reinterpret_cast<uint16_t*>(blk)[1] = f2h(sm);
        }
    }
    cluster.sync();   // no block leaves while its square sums may still be read
}

// ---- the state after the first n rows of a logged window: S <- g_t S + k_t (x) delta_t for t < n, every element with the
// very operations the rows kernel applied to it (fmul then ffma), so the bits are those of the window's own states.  Block
// (value head, job): 256 threads, thread = a quad of columns and 16 rows of it.
__global__ void __launch_bounds__(256) k_gdn_replay(const FnxGdnReplay* __restrict__ jobs) {
    const FnxGdnReplay jb = jobs[blockIdx.y];
    const int lv = blockIdx.x, tid = threadIdx.x, cq = tid & 31, rb = tid >> 5;
    if (lv >= jb.nv || jb.n <= 0) return;
    const int kh = jb.vmap[lv] & 255;
    const GdnLog lg = gdn_log(const_cast<float*>(jb.log), jb.nk, jb.nv);
    float* Sh = jb.S + (size_t) lv * HS * HS + 4 * cq;
    float s[16][4];
    int kidx[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = rb + 8 * i;
        const float4 v = *reinterpret_cast<const float4*>(Sh + (size_t) r * HS);
        s[i][0] = v.x, s[i][1] = v.y, s[i][2] = v.z, s[i][3] = v.w;
        kidx[i] = (r >> 5) * 32 + (r & 3) * 8 + ((r >> 2) & 7);   // where the log keeps key row r
    }
    for (int t = 0; t < jb.n; ++t) {
        const size_t row = (size_t) jb.row0 + t;
        const float gv = lg.g[(row * jb.nv + lv) * 2];
        const float4 d = *reinterpret_cast<const float4*>(lg.delta + (row * jb.nv + lv) * HS + 4 * cq);
        const float* k = lg.k + (row * jb.nk + kh) * HS;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float kx = k[kidx[i]];
            s[i][0] = ffma(kx, d.x, fmul(gv, s[i][0]));
            s[i][1] = ffma(kx, d.y, fmul(gv, s[i][1]));
            s[i][2] = ffma(kx, d.z, fmul(gv, s[i][2]));
            s[i][3] = ffma(kx, d.w, fmul(gv, s[i][3]));
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) *reinterpret_cast<float4*>(Sh + (size_t) (rb + 8 * i) * HS) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
}

static int gdn_launch(const GdnArgs& g, int nseg, cudaStream_t st, const char* what) {
    launch(5, k_gdn_prep, dim3(2 * g.nk + g.nv, g.T, nseg), HS, 0, st, g);
    if (launch_ok(what)) return 1;
    launch(8, k_gdn_rows, dim3(g.nv * GR_CL, nseg), GR_THREADS, 0, st, g);
    return launch_ok(what);
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

// q, k, v after conv / SiLU / norm and the gates, by window row (no zeroing needed; nk <= nv)
size_t fnx_gdn_scratch_floats(int nv) { return (size_t) FNX_MAXT * 3 * nv * HS + (size_t) FNX_MAXT * nv * 2; }

int fnx_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a,
                 const float* nw, float* S, void* yq, const int* ctl, float* scratch, float* snap, float* hsnap, int nk, int nv,
                 const int* vmap, int T, float eps, void* st, float* y32) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "gdn_core: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(nk >= 1 && nk <= 255 && nv >= 1 && nk <= nv, "gdn_core: %d key heads, %d value heads", nk, nv);
    FNX_REQUIRE(T == 1 || (snap && hsnap), "gdn_core: a window of %d rows needs snap and hsnap", T);
    FNX_REQUIRE(scratch && ((uintptr_t) scratch % 16) == 0 && ((uintptr_t) S % 16) == 0 && (!snap || ((uintptr_t) snap % 16) == 0),
                "gdn_core: scratch, state and checkpoints must be 16-byte aligned");
    GdnArgs g{qkvz, ab, hist, convw, dt, a, nw, S, (uint8_t*) yq, ctl, scratch, snap, hsnap, nk, nv, vmap, T, eps, y32, nullptr, nullptr, nullptr, nullptr, nullptr};
    return gdn_launch(g, 1, strm(st), "gdn_core");
}

size_t fnx_gdn_log_floats(int nk, int nv) { return (size_t) FNX_MAXT * ((size_t) nk * HS + (size_t) nv * 2 + (size_t) nv * HS); }

int fnx_gdn_core_log(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a, const float* nw,
                     const float* S, void* yq, const int* ctl, float* scratch, float* log, float* hsnap, int nk, int nv, const int* vmap, int T, float eps,
                     void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "gdn_core_log: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(nk >= 1 && nk <= 255 && nv >= 1 && nk <= nv, "gdn_core_log: %d key heads, %d value heads", nk, nv);
    FNX_REQUIRE(T == 1 || hsnap, "gdn_core_log: a window of %d rows needs hsnap", T);
    FNX_REQUIRE(scratch && log && ((uintptr_t) scratch % 16) == 0 && ((uintptr_t) log % 16) == 0 && ((uintptr_t) S % 16) == 0,
                "gdn_core_log: scratch, log and state must be 16-byte aligned");
    GdnArgs g{qkvz, ab, hist, convw, dt, a, nw, const_cast<float*>(S), (uint8_t*) yq, ctl, scratch, nullptr, hsnap, nk, nv, vmap, T, eps, nullptr,
              nullptr, nullptr, nullptr, nullptr, log};
    return gdn_launch(g, 1, strm(st), "gdn_core_log");
}

int fnx_gdn_replay(const FnxGdnReplay* jobs, int njobs, int nv_max, void* st) {
    if (njobs <= 0) return 0;
    FNX_REQUIRE(jobs && nv_max >= 1, "gdn_replay: no jobs");
    launch(0, k_gdn_replay, dim3(nv_max, njobs), 256, 0, strm(st), jobs);
    return launch_ok("gdn_replay");
}

int fnx_gdn_core_segs(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                      float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int nseg, int T, float eps, void* st) {
    FNX_REQUIRE(T >= 1 && nseg >= 1 && nseg * T <= FNX_MAXT, "gdn_core_segs: %d segments of %d rows (at most %d rows in all)", nseg, T, FNX_MAXT);
    FNX_REQUIRE(nk >= 1 && nk <= 255 && nv >= 1 && nk <= nv, "gdn_core_segs: %d key heads, %d value heads", nk, nv);
    FNX_REQUIRE(gl && gl->S && gl->hist && gl->ctl, "gdn_core_segs: no lanes");
    FNX_REQUIRE(T == 1 || (gl->snap && gl->hsnap && gl->row0), "gdn_core_segs: segments of %d rows need row0, snap and hsnap", T);
    FNX_REQUIRE(scratch && ((uintptr_t) scratch % 16) == 0, "gdn_core_segs: scratch must be 16-byte aligned");
    GdnArgs g{qkvz, ab, nullptr, convw, dt, a, nw, nullptr, (uint8_t*) yq, nullptr, scratch, gl->snap, gl->hsnap, nk, nv, vmap, T, eps, nullptr,
              gl->S, gl->hist, gl->ctl, gl->row0, nullptr};
    return gdn_launch(g, nseg, strm(st), "gdn_core_segs");
}

int fnx_gdn_core_lanes(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                       float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int T, float eps, void* st) {
    FNX_REQUIRE(T >= 1 && gl && !gl->row0, "gdn_core_lanes: %d rows, one lane each (no row0)", T);
    return fnx_gdn_core_segs(qkvz, ab, convw, dt, a, nw, yq, scratch, nk, nv, vmap, gl, T, 1, eps, st);
}
}
