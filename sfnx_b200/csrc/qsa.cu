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
//   projection  a warp per weight row (bf16) and 4 of the window's rows, lanes over column pairs;
//   index       block (row, part): 4 query heads, the raw key, the pooling - 128 threads, one per dimension;
//   scores      a lane per block of positions holds its pooled key as f32 in registers; a thread block takes 32 keys and
//               its 4 warps split the window's rows, whose queries sit in shared memory: the pooled keys come from DRAM
//               once per window instead of once per row;
//   selection   a cluster of 8 blocks per row, each keeping an eighth of the scores in shared memory: four 8-bit radix
//               passes find the top-th highest score (the blocks' histograms added through distributed shared memory),
//               then the kept blocks are compacted in index order with ballot prefix counts.
// Arithmetic (the oracle's oracle/oqsa.c states the same): a lane's column pairs 2 lane, 2 lane + 64, ..., the odd
// column's product first; a score's chain over the key's dimensions in pairs, odd first; heads added in order.
#include <cooperative_groups.h>

#include <cmath>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"

namespace fnxk {

constexpr int QD = FNX_QSA_DIM, QH = FNX_QSA_HEADS, QPOOL = FNX_QSA_POOL, QROT = 64, QROWS = QH * QD + QD;
constexpr int QP_WARPS = 8, QP_TG = FNX_MAXT / 4, QS_THREADS = 128, QS_KEYS = 32, QSEL_THREADS = 1024;

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

// a warp takes one weight row and 4 of the window's rows: 8 warps a block = 2 weight rows x 4 groups of window rows, so
// that 640 rows make 320 blocks of 8 warps (the weights' second to fourth readers hit L1)
__global__ void __launch_bounds__(QP_WARPS * 32) k_qsa_proj(const uint16_t* __restrict__ wq, const uint16_t* __restrict__ wk,
                                                           const float* __restrict__ x, float* __restrict__ y, int T, int n) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = blockIdx.x * (QP_WARPS / 4) + warp / 4, t0 = (warp % 4) * QP_TG;
    if (r >= QROWS || t0 >= T) return;
    const uint16_t* w = r < QH * QD ? wq + (size_t) r * n : wk + (size_t) (r - QH * QD) * n;
    float acc[QP_TG];
#pragma unroll
    for (int i = 0; i < QP_TG; ++i) acc[i] = 0.f;
    const int nt = min(QP_TG, T - t0);
    pdl_wait();
    pdl_go();
    const float* xr = x + (size_t) t0 * n;
#pragma unroll 4
    for (int c = lane * 2; c < n; c += 64) {
        const unsigned wv = __ldg(reinterpret_cast<const unsigned*>(w + c));
        const float w0 = bf16f((uint16_t) (wv & 0xffffu)), w1 = bf16f((uint16_t) (wv >> 16));
#pragma unroll
        for (int i = 0; i < QP_TG; ++i)
            if (i < nt) {
                const float2 xv = *reinterpret_cast<const float2*>(xr + (size_t) i * n + c);
                acc[i] = ffma(w0, xv.x, ffma(w1, xv.y, acc[i]));
            }
    }
#pragma unroll
    for (int i = 0; i < QP_TG; ++i)
        if (i < nt) {
            const float v = wsum(acc[i]);
            if (lane == 0) y[(size_t) (t0 + i) * QROWS + r] = v;
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
    const int tid = threadIdx.x, j = blockIdx.x * QS_KEYS + (tid & 31);   // lane = key; the block's warps split the window's rows
    if (tid < T) nv_s[tid] = min(((lr.pos ? *lr.pos[tid] : *pos0p + tid) + 1) / QPOOL, max_pools);   // (never past the scores' row)
    __syncthreads();
    int nv_max = 0;
    for (int t = 0; t < T; ++t)
        if (nv_s[t] > top) nv_max = max(nv_max, nv_s[t]);
    if ((int) (blockIdx.x * QS_KEYS) >= nv_max) return;
    for (int e = tid; e < T * QH * QD / 4; e += QS_THREADS) qs[e] = reinterpret_cast<const float4*>(q)[e];
    __syncthreads();
    float key[QD];   // the block's key as f32, converted once for all the window's rows
    auto fetch = [&](const FnxKvPages& gk) {
        const uint4* kr = reinterpret_cast<const uint4*>(pooled + pooled_at(gk, j, ncard));
#pragma unroll
        for (int c = 0; c < QD / 8; ++c) {
            const uint4 u = __ldg(kr + c);
            const unsigned kw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) key[8 * c + 2 * k] = h2f((uint16_t) (kw[k] & 0xffff)), key[8 * c + 2 * k + 1] = h2f((uint16_t) (kw[k] >> 16));
        }
    };
    if (!LANES && j < nv_max) fetch(g);
    const float w = ex_rsqrt((float) QD);
#pragma unroll 1
    for (int t = tid >> 5; t < T; t += QS_THREADS / 32) {
        const int nv = nv_s[t];
        if (nv <= top || j >= nv) continue;
        if (LANES) {
            FnxKvPages gt = g;
            if (lr.pt) gt.pt = lr.pt[t];
            fetch(gt);
        }
        const float4* qt = qs + (size_t) t * QH * QD / 4;
        float d[QH];
#pragma unroll
        for (int h = 0; h < QH; ++h) d[h] = 0.f;
#pragma unroll
        for (int c = 0; c < QD / 4; ++c) {
#pragma unroll
            for (int h = 0; h < QH; ++h) {
                const float4 qa = qt[h * (QD / 4) + c];
                d[h] = ffma(qa.x, key[4 * c], ffma(qa.y, key[4 * c + 1], d[h]));
                d[h] = ffma(qa.z, key[4 * c + 2], ffma(qa.w, key[4 * c + 3], d[h]));
            }
        }
        float s = 0.f;
#pragma unroll
        for (int h = 0; h < QH; ++h) s = fadd(s, fmul(fmaxf(d[h], 0.f), w));
        scores[(size_t) t * max_pools + j] = s;
    }
}

// A cluster of 8 blocks per row, block r of it the r-th eighth of the row's visible blocks (whole tiles of 1024), whose
// scores it keeps in shared memory.  Scores are >= +0, so their bit patterns order as unsigned integers.
//   threshold   four 8-bit radix passes from the top byte: every block counts its keys that match the bytes found so far
//               (one shared-memory atomic per warp and bin), every block then adds the 8 histograms through distributed
//               shared memory and finds the same bin;
//   selection   keys above the threshold and the first `want` equal to it, in index order: the blocks exchange how many
//               equal keys, then how many of their own kept blocks, lie before each of them, and every block writes its
//               cells at its place with ballot prefix counts tile by tile.
constexpr int QSEL_CL = 8;
static_assert(QSEL_THREADS == 1024, "the selection's prefix counts take the block's 32 warps one a lane");
__global__ void __cluster_dims__(QSEL_CL, 1, 1) __launch_bounds__(QSEL_THREADS)
    k_qsa_select(const float* __restrict__ scores, int* __restrict__ cells, int* __restrict__ n_cells, int max_pools, const int* pos0p,
                 FnxLaneRows lr, int card, int ncard, int top) {
    namespace cg = cooperative_groups;
    cg::cluster_group cl = cg::this_cluster();
    pdl_wait();
    pdl_go();
    const int t = blockIdx.x / QSEL_CL, rank = (int) cl.block_rank(), tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int p = lr.pos ? *lr.pos[t] : *pos0p + t, nv = min((p + 1) / QPOOL, max_pools), n_tail = (p + 1) % QPOOL;
    if (nv <= top) {   // the whole cluster leaves
        if (rank == 0 && tid == 0) n_cells[t] = -1;
        return;
    }
    extern __shared__ unsigned qsel_keys[];   // this block's scores
    __shared__ unsigned hist[256], total[256];   // this block's histogram; the row's (the 8 blocks' added)
    __shared__ unsigned prefix_s, want_s;
    __shared__ int wcount[2][QSEL_THREADS / 32];
    __shared__ int eq_tot, own_tot, base_s;
    const int chunk = (nv + QSEL_CL * QSEL_THREADS - 1) / (QSEL_CL * QSEL_THREADS) * QSEL_THREADS;
    const int j_lo = min(nv, rank * chunk), cnt = min(nv, j_lo + chunk) - j_lo;
    const unsigned* key_g = reinterpret_cast<const unsigned*>(scores + (size_t) t * max_pools) + j_lo;
    for (int i = tid; i < cnt; i += QSEL_THREADS) qsel_keys[i] = key_g[i];
    __syncthreads();
    // ---- the top-th highest key of the row
    unsigned prefix = 0, mask = 0, want = (unsigned) top;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i0 = 0; i0 < cnt; i0 += QSEL_THREADS) {
            const int i = i0 + tid;
            const unsigned k = i < cnt ? qsel_keys[i] : 0u;
            const bool in = i < cnt && (k & mask) == prefix;
            const unsigned bin = in ? (k >> shift) & 255u : 256u;
            const unsigned same = __match_any_sync(0xffffffffu, bin);
            if (in && lane == __ffs(same) - 1) atomicAdd(&hist[bin], (unsigned) __popc(same));
        }
        cl.sync();   // every block's histogram is complete
        if (tid < 256) {
            unsigned v = 0;
#pragma unroll
            for (int r = 0; r < QSEL_CL; ++r) v += *cl.map_shared_rank(&hist[tid], r);
            total[tid] = v;
        }
        __syncthreads();
        if (warp == 0) {   // lane l holds the bins 255 - 8 l down to 248 - 8 l: counts from the top bin down, across the lanes
            unsigned mine = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) mine += total[255 - 8 * lane - i];
            unsigned upto = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned v = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += v;
            }
            const unsigned reached = __ballot_sync(0xffffffffu, upto >= want);   // never empty: the matching keys are at least `want`
            if (lane == __ffs(reached) - 1) {
                unsigned higher = upto - mine;   // keys in bins above the one looked at
                int bin = 255 - 8 * lane;
                while (higher + total[bin] < want) higher += total[bin--];
                prefix_s = prefix | ((unsigned) bin << shift);
                want_s = want - higher;
            }
        }
        cl.sync();   // the histograms have been read: the next pass may clear them
        prefix = prefix_s, want = want_s;
        mask |= 255u << shift;
    }
    const unsigned thr = prefix;
    // ---- keys equal to the threshold in the blocks before this one
    {
        int c = 0;
        for (int i = tid; i < cnt; i += QSEL_THREADS) c += qsel_keys[i] == thr;
#pragma unroll
        for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) wcount[0][warp] = c;
        __syncthreads();
        if (warp == 0) {
            const int s = __reduce_add_sync(0xffffffffu, wcount[0][lane]);
            if (lane == 0) eq_tot = s;
        }
    }
    cl.sync();
    // a value of the blocks before this one in the cluster, added up by the first warp for all
    auto before_me = [&](int* mine) {
        if (warp == 0) {
            const int s = __reduce_add_sync(0xffffffffu, lane < rank ? *cl.map_shared_rank(mine, lane) : 0);
            if (lane == 0) base_s = s;
        }
        __syncthreads();
        const int v = base_s;
        __syncthreads();
        return v;
    };
    const int eq_base = before_me(&eq_tot);
    // ---- two sweeps in index order: count this GPU's kept blocks, exchange, then write the cells at their places
    int* row = cells + (size_t) t * (top * QPOOL + QPOOL - 1);
    int out_base = 0;
    for (int sweep = 0; sweep < 2; ++sweep) {
        int eq_seen = eq_base, out = out_base;
        for (int i0 = 0; i0 < cnt; i0 += QSEL_THREADS) {
            const int i = i0 + tid, j = j_lo + i;
            const unsigned k = i < cnt ? qsel_keys[i] : 0u;
            const bool gt = i < cnt && k > thr, eq = i < cnt && k == thr;
            const unsigned be = __ballot_sync(0xffffffffu, eq);
            if (lane == 0) wcount[0][warp] = __popc(be);
            __syncthreads();
            // the 32 warps' counts, one a lane: those of the warps before this one, and the tile's
            const int ce = wcount[0][lane];
            const int eq_tile = __reduce_add_sync(0xffffffffu, ce);
            const int eq_before = eq_seen + __reduce_add_sync(0xffffffffu, lane < warp ? ce : 0) + __popc(be & ((1u << lane) - 1));
            const bool own = (gt || (eq && eq_before < (int) want)) && j % ncard == card;
            const unsigned bo = __ballot_sync(0xffffffffu, own);
            if (lane == 0) wcount[1][warp] = __popc(bo);
            __syncthreads();
            const int co = wcount[1][lane];
            const int own_tile = __reduce_add_sync(0xffffffffu, co);
            const int at = out + __reduce_add_sync(0xffffffffu, lane < warp ? co : 0) + __popc(bo & ((1u << lane) - 1));
            if (sweep == 1 && own) {
#pragma unroll
                for (int m = 0; m < QPOOL; ++m) row[at * QPOOL + m] = (j / ncard) * QPOOL + m;
            }
            eq_seen += eq_tile, out += own_tile;
        }
        if (sweep == 0) {
            if (tid == 0) own_tot = out;
            cl.sync();
            out_base = before_me(&own_tot);
            if (rank == 0 && tid == 0) {   // the row's count: every block's kept blocks of this GPU, then the tail positions
                int n = 0;
                for (int r = 0; r < QSEL_CL; ++r) n += *cl.map_shared_rank(&own_tot, r);
                n *= QPOOL;
                const int jt = p / QPOOL;   // the row's own, incomplete block
                if (jt % ncard == card)
                    for (int m = 0; m < n_tail; ++m) row[n++] = (jt / ncard) * QPOOL + (p - n_tail + 1 + m) % QPOOL;
                n_cells[t] = n;
            }
        }
    }
    cl.sync();   // no block leaves while another may still read its shared memory
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
    launch(0, k_qsa_proj, dim3((QROWS + QP_WARPS / 4 - 1) / (QP_WARPS / 4)), QP_WARPS * 32, 0, strm(st), wq, wk, x, y, T, n);
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
    const dim3 grid((max_pools + QS_KEYS - 1) / QS_KEYS);
    if (lr.pt) launch(0, k_qsa_score<true>, grid, QS_THREADS, 0, strm(st), q, pooled, g, scores, max_pools, pos0, lr, T, ncard, top);
    else launch(0, k_qsa_score<false>, grid, QS_THREADS, 0, strm(st), q, pooled, g, scores, max_pools, pos0, lr, T, ncard, top);
    if (launch_ok("qsa scores")) return 1;
    // a block of the selection keeps its eighth of a row's scores (whole tiles of 1024) in shared memory
    const size_t keys = (size_t) ((max_pools + QSEL_CL * QSEL_THREADS - 1) / (QSEL_CL * QSEL_THREADS)) * QSEL_THREADS * sizeof(unsigned);
    FNX_REQUIRE(keys <= 200 * 1024, "qsa_select: %d blocks a row are more than the selection's shared memory holds", max_pools);
    if (smem_optin(k_qsa_select, keys, "qsa select")) return 1;
    launch(0, k_qsa_select, dim3(T * QSEL_CL), QSEL_THREADS, keys, strm(st), scores, cells, n_cells, max_pools, pos0, lr, card, ncard, top);
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
