// The attention layers' block selection (the indexer): what reference src/qsa.cuh computes, launched as
// src/kernels.cu:1152-1239 does (qsa_proj, qsa_index, qsa_select, qsa).
//
// Positions go in blocks of 4.  Every row leaves its raw indexer key (f16) in a ring of the last positions; the row that
// completes a block pools it (mean of the four raw keys, RMS norm, rotary at the block's first position, f16) into
// `pooled`, which every GPU holds whole.  A row at position p sees the blocks [0, (p + 1) / 4); if that is more than
// `top`, each block gets the score sum_h relu(q_h . key) / sqrt(128) over the row's 4 normed and rotated query heads, the
// `top` highest are kept (the lower block among equal scores), and the row attends this GPU's part of them plus its own
// tail positions: cells[t] holds those local K/V rows in ascending order, n_cells[t] their count (-1: every block kept).
//
// How the work is laid out here:
//   projection  a warp per weight row (bf16), 4 rows a block (160 blocks for the 640 rows), lanes over column pairs;
//   index       block (row, part): 4 query heads, the raw key, the pooling - 128 threads, one per dimension;
//   scores      a thread per block of positions holds its pooled key in registers and walks the window's rows, whose
//               queries sit in shared memory: the pooled keys are read once per window instead of once per row;
//   selection   a block per row: four 8-bit radix passes find the top-th highest score (warp-aggregated histogram
//               updates), then tiles of 1024 scores are compacted in index order with ballot prefix counts.
// Arithmetic (the oracle's oracle/oqsa.c states the same): a lane's column pairs 2 lane, 2 lane + 64, ..., the odd
// column's product first; a score's chain over the key's dimensions in pairs, odd first; heads added in order.
#include <cmath>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int QD = FNX_QSA_DIM, QH = FNX_QSA_HEADS, QPOOL = FNX_QSA_POOL, QROT = 64, QROWS = QH * QD + QD;
constexpr int QP_WARPS = 4, QS_THREADS = 256, QSEL_THREADS = 1024;

struct QsaFreqs {
    float f[QROT / 2];   // unit frequency of pair i, base^(-2 i / 64), by the host's powf
};

__device__ __forceinline__ float bf16f(uint16_t h) { return __uint_as_float((unsigned) h << 16); }

// block b's pooled key (halves from `pooled`): a page holds every GPU's blocks of its positions
__device__ __forceinline__ size_t pooled_at(const FnxKvPages& g, int b, int ncard) {
    if (!g.pt) return (size_t) b * QD;
    const int bpp = g.rows / 4 * ncard;
    return (size_t) g.pt[b / bpp] * g.page + (size_t) (b % bpp) * QD;
}

__global__ void __launch_bounds__(QP_WARPS * 32) k_qsa_proj(const uint16_t* __restrict__ wq, const uint16_t* __restrict__ wk,
                                                           const float* __restrict__ x, float* __restrict__ y, int T, int n) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = blockIdx.x * QP_WARPS + warp;
    if (r >= QROWS) return;
    const uint16_t* w = r < QH * QD ? wq + (size_t) r * n : wk + (size_t) (r - QH * QD) * n;
    float acc[FNX_MAXT];
#pragma unroll
    for (int t = 0; t < FNX_MAXT; ++t) acc[t] = 0.f;
    pdl_wait();
    pdl_go();
#pragma unroll 2
    for (int c = lane * 2; c < n; c += 64) {
        const unsigned wv = *reinterpret_cast<const unsigned*>(w + c);
        const float w0 = bf16f((uint16_t) (wv & 0xffffu)), w1 = bf16f((uint16_t) (wv >> 16));
#pragma unroll
        for (int t = 0; t < FNX_MAXT; ++t)
            if (t < T) {
                const float2 xv = *reinterpret_cast<const float2*>(x + (size_t) t * n + c);
                acc[t] = ffma(w0, xv.x, ffma(w1, xv.y, acc[t]));
            }
    }
#pragma unroll
    for (int t = 0; t < FNX_MAXT; ++t)
        if (t < T) {
            const float v = wsum(acc[t]);
            if (lane == 0) y[(size_t) t * QROWS + r] = v;
        }
}

// this thread's dimension of a 128-wide vector: RMS norm with weight (warp trees, the 4 warps added in ascending order),
// then the rotation of the pairs (i, i + 32), i < 32, at position pos
__device__ __forceinline__ float qsa_norm_rope(float v, const float* w, int pos, float eps, const QsaFreqs& rf, float* sh, float* buf) {
    const int i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const float ws = wsum(fmul(v, v));
    if (lane == 0) sh[warp] = ws;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < QD / 32; ++k) tot = fadd(tot, sh[k]);
    const float y = fmul(fmul(v, ex_rsqrt(fadd(fdiv(tot, (float) QD), eps))), w[i]);
    buf[i] = y;
    __syncthreads();
    float out = y;
    if (i < QROT) {
        const int k = i % (QROT / 2);
        const float theta = fmul((float) pos, rf.f[k]);
        float sn, cs;
        ex_sincos((double) theta, &sn, &cs);
        const float x0 = buf[k], x1 = buf[k + QROT / 2];
        out = i < QROT / 2 ? ffma(-x1, sn, fmul(x0, cs)) : ffma(x1, cs, fmul(x0, sn));
    }
    __syncthreads();
    return out;
}

// block (row t, part): part < 4 a query head; 4 the raw key into the ring; 5 the pooling of the block the row completes
// (the window's own raw keys from y, rounded to f16 as the ring holds them; earlier ones from the ring)
__global__ void __launch_bounds__(QD) k_qsa_index(const float* __restrict__ y, const float* __restrict__ qn, const float* __restrict__ kn,
                                                 uint16_t* ring, int ring_rows, float* __restrict__ q, uint16_t* pooled, FnxKvPages g,
                                                 int ncard, const int* pos0p, float eps, QsaFreqs rf) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.x, part = blockIdx.y, i = threadIdx.x, pos0 = *pos0p, p = pos0 + t;
    __shared__ float sh[QD / 32];
    __shared__ float buf[QD];
    const float* yt = y + (size_t) t * QROWS;
    if (part < QH) {
        q[((size_t) t * QH + part) * QD + i] = qsa_norm_rope(yt[part * QD + i], qn, p, eps, rf, sh, buf);
    } else if (part == QH) {
        ring[(size_t) (p % ring_rows) * QD + i] = f2h(yt[QH * QD + i]);
    } else {
        if ((p + 1) % QPOOL != 0) return;
        float v = 0.f;
#pragma unroll
        for (int m = 0; m < QPOOL; ++m) {
            const int pm = p - (QPOOL - 1) + m;
            v = fadd(v, h2f(pm >= pos0 ? f2h(y[(size_t) (pm - pos0) * QROWS + QH * QD + i]) : ring[(size_t) (pm % ring_rows) * QD + i]));
        }
        v = fmul(v, 1.0f / (float) QPOOL);
        const float o = qsa_norm_rope(v, kn, p - (QPOOL - 1), eps, rf, sh, buf);
        pooled[pooled_at(g, (p + 1) / QPOOL - 1, ncard) + i] = f2h(o);
    }
}

// scores[t][j] of the visible blocks j of the rows that see more than `top`.  LANES: every row on a page table of its own
template <bool LANES>
__global__ void __launch_bounds__(QS_THREADS) k_qsa_score(const float* __restrict__ q, const uint16_t* __restrict__ pooled, FnxKvPages g,
                                                         float* __restrict__ scores, int max_pools, const int* pos0p, FnxLaneRows lr, int T,
                                                         int ncard, int top) {
    pdl_wait();
    pdl_go();
    __shared__ float4 qs[FNX_MAXT * QH * QD / 4];
    __shared__ int nv_s[FNX_MAXT];
    const int tid = threadIdx.x, j = blockIdx.x * QS_THREADS + tid;
    if (tid < T) nv_s[tid] = ((lr.pos ? *lr.pos[tid] : *pos0p + tid) + 1) / QPOOL;
    __syncthreads();
    int nv_max = 0;
    for (int t = 0; t < T; ++t)
        if (nv_s[t] > top) nv_max = max(nv_max, nv_s[t]);
    if ((int) (blockIdx.x * QS_THREADS) >= nv_max) return;
    for (int e = tid; e < T * QH * QD / 4; e += QS_THREADS) qs[e] = reinterpret_cast<const float4*>(q)[e];
    __syncthreads();
    uint4 key[QD / 8];
    if (!LANES && j < nv_max) {
        const uint4* kr = reinterpret_cast<const uint4*>(pooled + pooled_at(g, j, ncard));
#pragma unroll
        for (int c = 0; c < QD / 8; ++c) key[c] = kr[c];
    }
    const float w = ex_rsqrt((float) QD);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const int nv = nv_s[t];
        if (nv <= top || j >= nv) continue;
        if (LANES) {
            FnxKvPages gt = g;
            if (lr.pt) gt.pt = lr.pt[t];
            const uint4* kr = reinterpret_cast<const uint4*>(pooled + pooled_at(gt, j, ncard));
#pragma unroll
            for (int c = 0; c < QD / 8; ++c) key[c] = kr[c];
        }
        const float4* qt = qs + (size_t) t * QH * QD / 4;
        float d[QH];
#pragma unroll
        for (int h = 0; h < QH; ++h) d[h] = 0.f;
#pragma unroll
        for (int c = 0; c < QD / 8; ++c) {
            const unsigned kw[4] = {key[c].x, key[c].y, key[c].z, key[c].w};
#pragma unroll
            for (int h = 0; h < QH; ++h) {
                const float4 qa = qt[h * (QD / 4) + 2 * c], qb = qt[h * (QD / 4) + 2 * c + 1];
                float a = d[h];
                a = ffma(qa.x, h2f((uint16_t) (kw[0] & 0xffff)), ffma(qa.y, h2f((uint16_t) (kw[0] >> 16)), a));
                a = ffma(qa.z, h2f((uint16_t) (kw[1] & 0xffff)), ffma(qa.w, h2f((uint16_t) (kw[1] >> 16)), a));
                a = ffma(qb.x, h2f((uint16_t) (kw[2] & 0xffff)), ffma(qb.y, h2f((uint16_t) (kw[2] >> 16)), a));
                a = ffma(qb.z, h2f((uint16_t) (kw[3] & 0xffff)), ffma(qb.w, h2f((uint16_t) (kw[3] >> 16)), a));
                d[h] = a;
            }
        }
        float s = 0.f;
#pragma unroll
        for (int h = 0; h < QH; ++h) s = fadd(s, fmul(fmaxf(d[h], 0.f), w));
        scores[(size_t) t * max_pools + j] = s;
    }
}

// a block per row.  Scores are >= +0, so their bit patterns order as unsigned integers.
__global__ void __launch_bounds__(QSEL_THREADS) k_qsa_select(const float* __restrict__ scores, int* __restrict__ cells, int* __restrict__ n_cells,
                                                            int max_pools, const int* pos0p, FnxLaneRows lr, int card, int ncard, int top) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = lr.pos ? *lr.pos[t] : *pos0p + t, nv = (p + 1) / QPOOL, n_tail = (p + 1) % QPOOL;
    if (nv <= top) {
        if (tid == 0) n_cells[t] = -1;
        return;
    }
    const unsigned* key = reinterpret_cast<const unsigned*>(scores + (size_t) t * max_pools);
    __shared__ unsigned hist[256], above[257];
    __shared__ unsigned prefix_s, want_s;
    __shared__ int wcount[2][QSEL_THREADS / 32];
    // ---- the top-th highest key: a byte at a time from the top, among the keys that match the bytes found so far
    unsigned prefix = 0, mask = 0, want = (unsigned) top;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int j0 = 0; j0 < nv; j0 += QSEL_THREADS) {   // neighbouring scores share their high bytes: one atomic a warp and bin
            const int j = j0 + tid;
            const unsigned k = j < nv ? key[j] : 0u;
            const bool in = j < nv && (k & mask) == prefix;
            const unsigned bin = in ? (k >> shift) & 255u : 256u;
            const unsigned same = __match_any_sync(0xffffffffu, bin);
            if (in && lane == __ffs(same) - 1) atomicAdd(&hist[bin], (unsigned) __popc(same));
        }
        __syncthreads();
        // above[b]: keys in bins >= b (a suffix scan over the 256 bins)
        if (tid < 256) above[tid] = hist[tid];
        if (tid == 256) above[256] = 0;
        __syncthreads();
        for (int o = 1; o < 256; o <<= 1) {
            unsigned v = 0;
            if (tid < 256 && tid + o < 256) v = above[tid + o];
            __syncthreads();
            if (tid < 256) above[tid] += v;
            __syncthreads();
        }
        if (tid < 256 && above[tid] >= want && above[tid + 1] < want) {   // exactly one bin
            prefix_s = prefix | ((unsigned) tid << shift);
            want_s = want - above[tid + 1];
        }
        __syncthreads();
        prefix = prefix_s, want = want_s;
        mask |= 255u << shift;
    }
    // ---- every key above the threshold and the first `want` equal to it, in index order; this GPU's blocks of them
    const unsigned thr = prefix;
    int* row = cells + (size_t) t * (top * QPOOL + QPOOL - 1);
    int eq_seen = 0, out = 0;
    for (int j0 = 0; j0 < nv; j0 += QSEL_THREADS) {
        const int j = j0 + tid;
        const unsigned k = j < nv ? key[j] : 0u;
        const bool gt = j < nv && k > thr, eq = j < nv && k == thr;
        const unsigned be = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) wcount[0][warp] = __popc(be);
        __syncthreads();
        int eq_before = eq_seen, eq_tile = 0;
        for (int w2 = 0; w2 < QSEL_THREADS / 32; ++w2) {
            const int c = wcount[0][w2];
            if (w2 < warp) eq_before += c;
            eq_tile += c;
        }
        eq_before += __popc(be & ((1u << lane) - 1));
        const bool own = (gt || (eq && eq_before < (int) want)) && j % ncard == card;
        const unsigned bo = __ballot_sync(0xffffffffu, own);
        if (lane == 0) wcount[1][warp] = __popc(bo);
        __syncthreads();
        int at = out, own_tile = 0;
        for (int w2 = 0; w2 < QSEL_THREADS / 32; ++w2) {
            const int c = wcount[1][w2];
            if (w2 < warp) at += c;
            own_tile += c;
        }
        at += __popc(bo & ((1u << lane) - 1));
        if (own) {
#pragma unroll
            for (int m = 0; m < QPOOL; ++m) row[at * QPOOL + m] = (j / ncard) * QPOOL + m;
        }
        eq_seen += eq_tile, out += own_tile;
    }
    if (tid == 0) {
        int n = out * QPOOL;
        const int jt = p / QPOOL;   // the row's own, incomplete block
        if (jt % ncard == card)
            for (int m = 0; m < n_tail; ++m) row[n++] = (jt / ncard) * QPOOL + (p - n_tail + 1 + m) % QPOOL;
        n_cells[t] = n;
    }
}

static QsaFreqs qsa_freqs(FnxRope rope) {
    QsaFreqs rf;
    for (int i = 0; i < QROT / 2; ++i) rf.f[i] = powf(rope.base, -2.0f * (float) i / (float) QROT);
    return rf;
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_qsa_rows(void) { return QROWS; }
int fnx_qsa_maxsel(int top) { return top * QPOOL + QPOOL - 1; }

int fnx_qsa_proj(const uint16_t* wq, const uint16_t* wk, const float* x, float* y, int T, int n, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "qsa_proj: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(n >= 64 && n % 64 == 0, "qsa_proj: width %d (whole steps of 64 columns)", n);
    launch(0, k_qsa_proj, dim3((QROWS + QP_WARPS - 1) / QP_WARPS), QP_WARPS * 32, 0, strm(st), wq, wk, x, y, T, n);
    return launch_ok("qsa_proj");
}

int fnx_qsa_index(const float* y, const float* qn, const float* kn, uint16_t* ring, int ring_rows, uint16_t* pooled, FnxKvPages g, int ncard,
                  float* q, const int* pos0, int T, float eps, FnxRope rope, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "qsa_index: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(ring_rows >= T + QPOOL, "qsa_index: a ring of %d rows is shorter than a window and a block", ring_rows);
    FNX_REQUIRE(rope.nrot == QROT, "qsa_index: rotary width %d (the indexer rotates %d dimensions)", rope.nrot, QROT);
    FNX_REQUIRE(ncard >= 1 && (!g.pt || (g.rows > 0 && g.rows % 4 == 0)), "qsa_index: %d GPUs, %d rows a page", ncard, g.rows);
    launch(0, k_qsa_index, dim3(T, QH + 2), QD, 0, strm(st), y, qn, kn, ring, ring_rows, q, pooled, g, ncard, pos0, eps, qsa_freqs(rope));
    return launch_ok("qsa_index");
}

int fnx_qsa_select(const float* q, const uint16_t* pooled, FnxKvPages g, FnxLaneRows lr, float* scores, int* cells, int* n_cells, int max_pools,
                   const int* pos0, int T, int card, int ncard, int top, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "qsa_select: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(top >= 1 && max_pools >= 1, "qsa_select: top %d of at most %d blocks", top, max_pools);
    FNX_REQUIRE(ncard >= 1 && card >= 0 && card < ncard, "qsa_select: GPU %d of %d", card, ncard);
    FNX_REQUIRE(lr.pos || pos0, "qsa_select: no positions");
    const dim3 grid((max_pools + QS_THREADS - 1) / QS_THREADS);
    if (lr.pt) launch(0, k_qsa_score<true>, grid, QS_THREADS, 0, strm(st), q, pooled, g, scores, max_pools, pos0, lr, T, ncard, top);
    else launch(0, k_qsa_score<false>, grid, QS_THREADS, 0, strm(st), q, pooled, g, scores, max_pools, pos0, lr, T, ncard, top);
    if (launch_ok("qsa scores")) return 1;
    launch(0, k_qsa_select, dim3(T), QSEL_THREADS, 0, strm(st), scores, cells, n_cells, max_pools, pos0, lr, card, ncard, top);
    return launch_ok("qsa select");
}

int fnx_qsa(const uint16_t* wq, const uint16_t* wk, const float* x, int n, float* y, const float* qn, const float* kn, uint16_t* ring,
            int ring_rows, uint16_t* pooled, FnxKvPages g, float* q, float* scores, int* cells, int* n_cells, int max_pools, const int* pos0,
            int T, float eps, FnxRope rope, int card, int ncard, int top, void* st) {
    if (wq && fnx_qsa_proj(wq, wk, x, y, T, n, st)) return 1;
    if (fnx_qsa_index(y, qn, kn, ring, ring_rows, pooled, g, ncard, q, pos0, T, eps, rope, st)) return 1;
    return fnx_qsa_select(q, pooled, g, FnxLaneRows{nullptr, nullptr}, scores, cells, n_cells, max_pools, pos0, T, card, ncard, top, st);
}

}  // extern "C"
