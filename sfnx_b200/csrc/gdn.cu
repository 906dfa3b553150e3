// Gated DeltaNet core of the verify window in one launch, with per-row state checkpoints for the rollback.
// Replaces reference src/gdn_core.cuh (k_gdn_core) with the same decomposition of the sums (so each value can be
// checked bit for bit): 4 blocks per local value head, each owning 32 value columns of the head's 128 x 128 fp32
// state; thread (column, part) keeps key rows [32 part, 32 part + 32) of its column in registers over the whole
// window; the state after every row but the last is streamed to snap (the dominant HBM traffic: T state-sized writes
// per head), the conv history variants to hsnap.  The head's four blocks form a thread-block cluster: they exchange
// their outputs' square sums through distributed shared memory and each norms, gates and quantises its own columns.
#include <cooperative_groups.h>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int HS = FNX_HS, GDN_Q = 4, GDN_QC = HS / GDN_Q, GDN_THREADS = 128;

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
};

__global__ void __cluster_dims__(GDN_Q, 1, 1) __launch_bounds__(GDN_THREADS) k_gdn_core(const GdnArgs g) {
    namespace cg = cooperative_groups;
    const int lv = blockIdx.x / GDN_Q, qq = blockIdx.x % GDN_Q, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vm = g.vmap[lv], kh = vm & 255, writes_hist = vm >> 8, nk = g.nk, nv = g.nv, T = g.T;
    const int ch = (2 * nk + nv) * HS, row_stride = ch + nv * HS;
    const unsigned parity = ((const unsigned*) g.ctl)[1] & 1u;
    const float* hin = g.hist + (size_t) parity * 3 * ch;
    float* hout = g.hist + (size_t) (parity ^ 1u) * 3 * ch;
    __shared__ float xs[2][FNX_MAXT][32][4];   // q, k after conv, silu, L2 norm: element i at [i % 32][i / 32]
    __shared__ float vs[FNX_MAXT][GDN_QC];
    __shared__ float red[GDN_THREADS / 32][2 * FNX_MAXT];
    __shared__ float gates[FNX_MAXT][2];
    __shared__ float osm[FNX_MAXT][GDN_QC];   // this block's outputs and, per row, their square sum
    __shared__ float sqs[FNX_MAXT];
    if (tid < T) {
        const float* abt = g.ab + (size_t) tid * 2 * nv;
        const float x = fadd(abt[lv], g.dt[lv]);
        const float sp = x > 20.0f ? x : ex_log1pf_pos(ex_expf(x));
        gates[tid][0] = ex_expf(fmul(sp, g.a[lv]));
        gates[tid][1] = fdiv(1.0f, fadd(1.0f, ex_expf(-abt[nv + lv])));
    }
    // ---- causal conv (width 4) + silu: the key head's q and k channels, this block's 32 v channels
    for (int e = tid; e < 2 * HS + GDN_QC; e += GDN_THREADS) {
        const int part = e < HS ? 0 : e < 2 * HS ? 1 : 2, i = part < 2 ? e - part * HS : e - 2 * HS;
        const int c = part == 0 ? kh * HS + i : part == 1 ? nk * HS + kh * HS + i : 2 * nk * HS + lv * HS + qq * GDN_QC + i;
        const bool wh = part == 2 || (writes_hist && qq == 0);
        float h0 = hin[c], h1 = hin[(size_t) ch + c], h2 = hin[(size_t) 2 * ch + c];
        const float4 w = *reinterpret_cast<const float4*>(g.convw + (size_t) c * 4);
        float xr[FNX_MAXT];   // the window's rows of this channel, all loads in flight before any store
#pragma unroll
        for (int t = 0; t < FNX_MAXT; ++t) xr[t] = t < T ? g.qkvz[(size_t) t * row_stride + c] : 0.f;
#pragma unroll
        for (int t = 0; t < FNX_MAXT; ++t) {
            if (t >= T) break;
            const float xt = xr[t];
            float x = fmul(w.x, h0);
            x = ffma(w.y, h1, x);
            x = ffma(w.z, h2, x);
            x = ffma(w.w, xt, x);
            const float y = ex_silu(x);
            if (part < 2) xs[part][t][i % 32][i / 32] = y;
            else vs[t][i] = y;
            h0 = h1, h1 = h2, h2 = xt;
            if (wh && t + 1 < T) {   // the history if only rows 0..t are kept
                g.hsnap[((size_t) t * 3 + 0) * ch + c] = h0;
                g.hsnap[((size_t) t * 3 + 1) * ch + c] = h1;
                g.hsnap[((size_t) t * 3 + 2) * ch + c] = h2;
            }
        }
        if (wh) hout[c] = h0, hout[(size_t) ch + c] = h1, hout[(size_t) 2 * ch + c] = h2;
    }
    __syncthreads();
    // ---- L2 norms of q and k per row: thread i holds element i of each; warp trees, the four warps in order
    {
        for (int t = 0; t < T; ++t) {
            const float qv = xs[0][t][tid % 32][tid / 32], kv = xs[1][t][tid % 32][tid / 32];
            const float sq = wsum(fmul(qv, qv)), sk = wsum(fmul(kv, kv));
            if (lane == 0) red[warp][t] = sq, red[warp][FNX_MAXT + t] = sk;
        }
        __syncthreads();
        for (int t = 0; t < T; ++t) {
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int w = 0; w < GDN_THREADS / 32; ++w) sq = fadd(sq, red[w][t]), sk = fadd(sk, red[w][FNX_MAXT + t]);
            xs[0][t][tid % 32][tid / 32] = fmul(xs[0][t][tid % 32][tid / 32], ex_rsqrt(fadd(sq, 1e-6f)));
            xs[1][t][tid % 32][tid / 32] = fmul(xs[1][t][tid % 32][tid / 32], ex_rsqrt(fadd(sk, 1e-6f)));
        }
    }
    __syncthreads();
    // ---- the delta rule over the rows
    const int cl = tid >> 2, part = tid & 3, col = qq * GDN_QC + cl;
    float* st = g.S + (size_t) lv * HS * HS + (size_t) part * 32 * HS + col;
    float s[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) s[r] = st[(size_t) r * HS];
    const float scale = ex_rsqrt((float) HS);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float gv = gates[t][0], bv = gates[t][1];
        float k0 = 0.f, k1 = 0.f, k2 = 0.f, k3 = 0.f;
#pragma unroll
        for (int r = 0; r < 32; r += 4) {
            k0 = ffma(s[r], xs[1][t][r][part], k0);
            k1 = ffma(s[r + 1], xs[1][t][r + 1][part], k1);
            k2 = ffma(s[r + 2], xs[1][t][r + 2][part], k2);
            k3 = ffma(s[r + 3], xs[1][t][r + 3][part], k3);
        }
        float kvd = fadd(fadd(k0, k1), fadd(k2, k3));
        kvd = fadd(kvd, __shfl_xor_sync(0xffffffffu, kvd, 1));
        kvd = fadd(kvd, __shfl_xor_sync(0xffffffffu, kvd, 2));
        const float delta = fmul(ffma(-gv, kvd, vs[t][cl]), bv);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int r = 0; r < 32; r += 4) {
            s[r] = ffma(xs[1][t][r][part], delta, fmul(gv, s[r]));
            s[r + 1] = ffma(xs[1][t][r + 1][part], delta, fmul(gv, s[r + 1]));
            s[r + 2] = ffma(xs[1][t][r + 2][part], delta, fmul(gv, s[r + 2]));
            s[r + 3] = ffma(xs[1][t][r + 3][part], delta, fmul(gv, s[r + 3]));
            a0 = ffma(s[r], xs[0][t][r][part], a0);
            a1 = ffma(s[r + 1], xs[0][t][r + 1][part], a1);
            a2 = ffma(s[r + 2], xs[0][t][r + 2][part], a2);
            a3 = ffma(s[r + 3], xs[0][t][r + 3][part], a3);
        }
        float at = fadd(fadd(a0, a1), fadd(a2, a3));
        at = fadd(at, __shfl_xor_sync(0xffffffffu, at, 1));
        at = fadd(at, __shfl_xor_sync(0xffffffffu, at, 2));
        const float ov = part == 0 ? fmul(at, scale) : 0.f;
        if (part == 0) osm[t][cl] = ov;
        const float ss = wsum(fmul(ov, ov));
        if (lane == 0) red[warp][t] = ss;
        if (t < T - 1) {
            float* sp = g.snap + (size_t) t * nv * HS * HS + (st - g.S);
#pragma unroll
            for (int r = 0; r < 32; ++r) __stcs(sp + (size_t) r * HS, s[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < 32; ++r) st[(size_t) r * HS] = s[r];
    __syncthreads();
    if (tid < T) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GDN_THREADS / 32; ++w) v = fadd(v, red[w][tid]);
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
    for (int t = warp; t < T; t += GDN_THREADS / 32) {
        const float ms = fdiv(fadd(fadd(fadd(rsq[0][t], rsq[1][t]), rsq[2][t]), rsq[3][t]), (float) HS);
        const int c = qq * GDN_QC + lane;
        const float v = osm[t][lane];
        const float z = g.qkvz[(size_t) t * row_stride + ch + lv * HS + c];
        const float xi = fdiv(fmul(fmul(v, ex_rsqrt(fadd(ms, g.eps))), g.nw[c]), fadd(1.0f, ex_expf(-z)));
        if (g.y32) g.y32[(size_t) t * nv * HS + lv * HS + c] = xi;
        const float amax = wmax(fabsf(xi)), sm = wsum(xi);
        const float d = fdiv(amax, 127.0f);
        uint8_t* blk = g.yq + ((size_t) t * (nv * HS / 32) + lv * 4 + qq) * 36;
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
    GdnArgs g{qkvz, ab, hist, convw, dt, a, nw, S, (uint8_t*) yq, ctl, scratch, snap, hsnap, nk, nv, vmap, T, eps, y32};
    k_gdn_core<<<nv * GDN_Q, GDN_THREADS, 0, strm(st)>>>(g);
    return launch_ok("gdn_core");
}
}
