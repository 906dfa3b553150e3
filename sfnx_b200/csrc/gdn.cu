// Gated DeltaNet core of the verify window in one launch, with per-row state checkpoints for the rollback.
// Replaces reference src/gdn_core.cuh (k_gdn_core) with the same decomposition of the sums (so each value can be
// checked bit for bit): 4 blocks per local value head, each owning 32 value columns of the head's 128 x 128 fp32
// state.  A column's 128 key rows are cut as the reference cuts them, into 4 parts of 32 rows with 4 interleaved
// partial sums each, but every partial sum has a thread of its own here: thread (part, column, j) keeps rows
// 32 part + 4 i + j (i = 0..7) in registers over the whole window, the four j of a part meet by warp shuffles and the
// four parts through shared memory, in the reference's order.  The state after every row but the last is streamed to
// snap (the dominant HBM traffic: T state-sized writes per head), the conv history variants to hsnap.  The head's four
// blocks form a thread-block cluster: they exchange their outputs' square sums through distributed shared memory and
// each norms, gates and quantises its own columns.
#include <cooperative_groups.h>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int HS = FNX_HS, GDN_Q = 4, GDN_QC = HS / GDN_Q, GDN_THREADS = 512, GDN_WARPS = GDN_THREADS / 32;

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
};

__global__ void __cluster_dims__(GDN_Q, 1, 1) __launch_bounds__(GDN_THREADS, 2) k_gdn_core(const GdnArgs g) {
    namespace cg = cooperative_groups;
    const int lv = blockIdx.x / GDN_Q, qq = blockIdx.x % GDN_Q, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vm = g.vmap[lv], kh = vm & 255, writes_hist = vm >> 8, nk = g.nk, nv = g.nv, T = g.T;
    const int ch = (2 * nk + nv) * HS, row_stride = ch + nv * HS;
    // a segment's own state, history and rows (the pointer arrays are older than the window)
    float *S = g.S, *hist = g.hist;
    const int* ctl = g.ctl;
    int r0 = 0;
    if (g.lS) {
        const int seg = blockIdx.y;
        S = g.lS[seg], hist = g.lhist[seg], ctl = g.lctl[seg], r0 = g.row0 ? g.row0[seg] : seg;
    }
    const float* qkvz = g.qkvz + (size_t) r0 * row_stride;
    const float* ab = g.ab + (size_t) r0 * 2 * nv;
    float* snap = g.snap ? g.snap + (size_t) r0 * nv * HS * HS : nullptr;
    float* hsnap = g.hsnap ? g.hsnap + (size_t) r0 * 3 * ch : nullptr;
    // the state's loads go out first: they depend on no kernel of this window and have the whole prologue to land
    const int part = tid >> 7, cl = (tid >> 2) & 31, j = tid & 3, col = qq * GDN_QC + cl;
    float* st = S + (size_t) lv * HS * HS + (size_t) (part * 32 + j) * HS + col;
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = __ldcs(st + (size_t) 4 * i * HS);
    pdl_wait();
    pdl_go();
    const unsigned parity = ((const unsigned*) ctl)[1] & 1u;
    const float* hin = hist + (size_t) parity * 3 * ch;
    float* hout = hist + (size_t) (parity ^ 1u) * 3 * ch;
    __shared__ float xs[2][FNX_MAXT][32][4];   // q, k after conv, silu, L2 norm: element i at [i % 32][i / 32]
    __shared__ float vs[FNX_MAXT][GDN_QC];
    __shared__ float gates[FNX_MAXT][2];
    __shared__ float pk[4][GDN_QC], pa[4][GDN_QC];   // the four parts' sums of a column: k . S and q . S
    __shared__ float osm[FNX_MAXT][GDN_QC];          // this block's outputs and, per row, their square sum
    __shared__ float sqs[FNX_MAXT];
    if (tid < T) {
        const float* abt = ab + (size_t) tid * 2 * nv;
        const float x = fadd(abt[lv], g.dt[lv]);
        const float sp = x > 20.0f ? x : ex_log1pf_pos(ex_expf(x));
        gates[tid][0] = ex_expf(fmul(sp, g.a[lv]));
        gates[tid][1] = fdiv(1.0f, fadd(1.0f, ex_expf(-abt[nv + lv])));
    }
    // ---- causal conv (width 4) + silu: the key head's q and k channels, this block's 32 v channels; one item per
    // (row, channel), its four taps read from the window's rows or, before row 0, from the history
    constexpr int NCH = 2 * HS + GDN_QC, CI = 3;   // items in flight per thread
#pragma unroll 1
    for (int it0 = tid; it0 < T * NCH; it0 += CI * GDN_THREADS) {
        float in[CI][4];   // a batch's loads go out before its first sum
        float4 cw[CI];
        auto channel = [&](int e, int& pt, int& i) {
            pt = e < HS ? 0 : e < 2 * HS ? 1 : 2, i = pt < 2 ? e - pt * HS : e - 2 * HS;
            return pt == 0 ? kh * HS + i : pt == 1 ? nk * HS + kh * HS + i : 2 * nk * HS + lv * HS + qq * GDN_QC + i;
        };
#pragma unroll
        for (int m = 0; m < CI; ++m) {
            const int it = it0 + m * GDN_THREADS;
            if (it < T * NCH) {
                int pt, i;
                const int t = it / NCH, c = channel(it % NCH, pt, i);
                cw[m] = *reinterpret_cast<const float4*>(g.convw + (size_t) c * 4);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int tt = t - 3 + k;
                    in[m][k] = tt >= 0 ? qkvz[(size_t) tt * row_stride + c] : hin[(size_t) (tt + 3) * ch + c];
                }
            }
        }
#pragma unroll
        for (int m = 0; m < CI; ++m) {
            const int it = it0 + m * GDN_THREADS;
            if (it < T * NCH) {
                int pt, i;
                const int t = it / NCH, c = channel(it % NCH, pt, i);
                float x = fmul(cw[m].x, in[m][0]);
                x = ffma(cw[m].y, in[m][1], x);
                x = ffma(cw[m].z, in[m][2], x);
                x = ffma(cw[m].w, in[m][3], x);
                const float y = ex_silu(x);
                if (pt < 2) xs[pt][t][i % 32][i / 32] = y;
                else vs[t][i] = y;
                if (pt == 2 || (writes_hist && qq == 0)) {   // the history if only rows 0..t are kept; after the last row, the new one
                    float* h = t + 1 < T ? hsnap + (size_t) t * 3 * ch : hout;
                    h[c] = in[m][1], h[(size_t) ch + c] = in[m][2], h[(size_t) 2 * ch + c] = in[m][3];
                }
            }
        }
    }
    __syncthreads();
    // ---- L2 norms of q and k, a warp per row: 32-element groups by warp trees, the four groups in order
    for (int t = warp; t < T; t += GDN_WARPS) {
        float qv[4], kv[4], sq = 0.f, sk = 0.f;
#pragma unroll
        for (int gI = 0; gI < 4; ++gI) {
            qv[gI] = xs[0][t][lane][gI], kv[gI] = xs[1][t][lane][gI];
            sq = fadd(sq, wsum(fmul(qv[gI], qv[gI])));
            sk = fadd(sk, wsum(fmul(kv[gI], kv[gI])));
        }
        const float rq = ex_rsqrt(fadd(sq, 1e-6f)), rk = ex_rsqrt(fadd(sk, 1e-6f));
#pragma unroll
        for (int gI = 0; gI < 4; ++gI) xs[0][t][lane][gI] = fmul(qv[gI], rq), xs[1][t][lane][gI] = fmul(kv[gI], rk);
    }
    __syncthreads();
    // ---- the delta rule over the rows.  A column's four parts sit in warps w, w + 4, w + 8, w + 12 (w = the column's
    // eighth of the block's 32), so the exchange of their sums needs only those four warps to meet: a named barrier per
    // group of four warps instead of the whole block's
    const float scale = ex_rsqrt((float) HS);
    auto group_sync = [&] { asm volatile("bar.sync %0, 128;" ::"r"(1 + (warp & 3)) : "memory"); };
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float gv = gates[t][0], bv = gates[t][1];
        float kx[8], kj = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            kx[i] = xs[1][t][4 * i + j][part];
            kj = ffma(s[i], kx[i], kj);
        }
        kj = fadd(kj, __shfl_xor_sync(0xffffffffu, kj, 1));   // (k0 + k1), (k2 + k3)
        kj = fadd(kj, __shfl_xor_sync(0xffffffffu, kj, 2));
        if (j == 0) pk[part][cl] = kj;
        group_sync();
        const float kvd = fadd(fadd(pk[0][cl], pk[1][cl]), fadd(pk[2][cl], pk[3][cl]));
        const float delta = fmul(ffma(-gv, kvd, vs[t][cl]), bv);
        float aj = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s[i] = ffma(kx[i], delta, fmul(gv, s[i]));
            aj = ffma(s[i], xs[0][t][4 * i + j][part], aj);
        }
        aj = fadd(aj, __shfl_xor_sync(0xffffffffu, aj, 1));
        aj = fadd(aj, __shfl_xor_sync(0xffffffffu, aj, 2));
        if (j == 0) pa[part][cl] = aj;
        if (t < T - 1) {
            float* sp = snap + (size_t) t * nv * HS * HS + (st - S);
#pragma unroll
            for (int i = 0; i < 8; ++i) __stcs(sp + (size_t) 4 * i * HS, s[i]);
        }
        group_sync();
        if (part == 0 && j == 0) osm[t][cl] = fmul(fadd(fadd(pa[0][cl], pa[1][cl]), fadd(pa[2][cl], pa[3][cl])), scale);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) st[(size_t) 4 * i * HS] = s[i];
    __syncthreads();
    if (tid < T) {   // the row's square sum: eight columns by a tree (a warp's butterfly over them), the four eights in order
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float c[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) c[k] = fmul(osm[tid][8 * w + k], osm[tid][8 * w + k]);
            v = fadd(v, fadd(fadd(fadd(c[0], c[4]), fadd(c[2], c[6])), fadd(fadd(c[1], c[5]), fadd(c[3], c[7]))));
        }
        sqs[tid] = v;
    }
    // ---- gated RMS norm over the head's 128 outputs: the head's four blocks are one thread-block cluster and read each
    // other's square sums through distributed shared memory; each block then norms, gates and quantises its own 32
    // columns (one q8_1 block per row)
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const float* rsq[GDN_Q];
#pragma unroll
    for (int r = 0; r < GDN_Q; ++r) rsq[r] = cluster.map_shared_rank(sqs, r);
    for (int t = warp; t < T; t += GDN_WARPS) {
        const float ms = fdiv(fadd(fadd(fadd(rsq[0][t], rsq[1][t]), rsq[2][t]), rsq[3][t]), (float) HS);
        const int c = qq * GDN_QC + lane;
        const float v = osm[t][lane];
        const float z = qkvz[(size_t) t * row_stride + ch + lv * HS + c];
        const float xi = fdiv(fmul(fmul(v, ex_rsqrt(fadd(ms, g.eps))), g.nw[c]), fadd(1.0f, ex_expf(-z)));
        if (g.y32) g.y32[(size_t) (r0 + t) * nv * HS + lv * HS + c] = xi;
        const float amax = wmax(fabsf(xi)), sm = wsum(xi);
        const float d = fdiv(amax, 127.0f);
        uint8_t* blk = g.yq + ((size_t) (r0 + t) * (nv * HS / 32) + lv * 4 + qq) * 36;
        reinterpret_cast<int8_t*>(blk + 4)[lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
        if (lane == 0) {
            reinterpret_cast<uint16_t*>(blk)[0] = f2h(d);
            reinterpret_cast<uint16_t*>(blk)[1] = f2h(sm);
        }
    }
    cluster.sync();   // no block leaves while its square sums may still be read
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

size_t fnx_gdn_scratch_floats(int nv) { return (size_t) FNX_MAXT * nv * HS + (size_t) nv * FNX_MAXT * GDN_Q + (size_t) nv; }

int fnx_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a,
                 const float* nw, float* S, void* yq, const int* ctl, float* scratch, float* snap, float* hsnap, int nk, int nv,
                 const int* vmap, int T, float eps, void* st, float* y32) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "gdn_core: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(nk >= 1 && nk <= 255 && nv >= 1, "gdn_core: %d key heads, %d value heads", nk, nv);
    FNX_REQUIRE(T == 1 || (snap && hsnap), "gdn_core: a window of %d rows needs snap and hsnap", T);
    GdnArgs g{qkvz, ab, hist, convw, dt, a, nw, S, (uint8_t*) yq, ctl, scratch, snap, hsnap, nk, nv, vmap, T, eps, y32, nullptr, nullptr, nullptr, nullptr};
    launch(5, k_gdn_core, nv * GDN_Q, GDN_THREADS, 0, strm(st), g);
    return launch_ok("gdn_core");
}

int fnx_gdn_core_segs(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                      float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int nseg, int T, float eps, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && nseg >= 1 && nseg <= 65535, "gdn_core_segs: %d segments of %d rows", nseg, T);
    FNX_REQUIRE(nk >= 1 && nk <= 255 && nv >= 1, "gdn_core_segs: %d key heads, %d value heads", nk, nv);
    FNX_REQUIRE(gl && gl->S && gl->hist && gl->ctl, "gdn_core_segs: no lanes");
    FNX_REQUIRE(T == 1 || (gl->snap && gl->hsnap && gl->row0), "gdn_core_segs: segments of %d rows need row0, snap and hsnap", T);
    GdnArgs g{qkvz, ab, nullptr, convw, dt, a, nw, nullptr, (uint8_t*) yq, nullptr, scratch, gl->snap, gl->hsnap, nk, nv, vmap, T, eps, nullptr,
              gl->S, gl->hist, gl->ctl, gl->row0};
    launch(5, k_gdn_core, dim3(nv * GDN_Q, nseg), GDN_THREADS, 0, strm(st), g);
    return launch_ok("gdn_core_segs");
}

int fnx_gdn_core_lanes(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                       float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int T, float eps, void* st) {
    FNX_REQUIRE(T >= 1 && gl && !gl->row0, "gdn_core_lanes: %d rows, one lane each (no row0)", T);
    return fnx_gdn_core_segs(qkvz, ab, convw, dt, a, nw, yq, scratch, nk, nv, vmap, gl, T, 1, eps, st);
}
}
