/* CPU ORACLE - test infrastructure, not product code.
 *
 * The attention layers' block selection (the indexer), restated with IEEE arithmetic from the reference's src/qsa.cuh:
 *   projection y = [wq; wk] x, bf16 weights, f32 activations            src/qsa.cuh:23-45 (k_idx_proj)
 *   query heads: RMS norm + NEOX rotary at the row's position; the raw key rounded to f16 into a ring of the last
 *     positions; a completed block of 4 positions pooled: the mean of its members' f16 raw keys, normed, rotated to
 *     its first member, kept as f16                                       src/qsa.cuh:48-124
 *   a visible block's score: sum over the heads of relu(q_h . k) / sqrt(128)   src/qsa.cuh:127-156 (k_idx_score)
 *   the selection: the `top` highest scores (the lower block among equal scores), this card's part of them as local
 *     rows in ascending order, then the row's tail positions              src/qsa.cuh:224-343 (k_idx_select)
 * Orders kept from the reference: a lane's column pairs (2 lane, 2 lane + 64, ...), the odd column first inside a pair,
 * lanes joined by the descending xor-tree; a score's chain over the key's dimensions in pairs, odd first; the heads
 * added in order.  A row at position p sees the blocks [0, (p + 1) / 4); with `top` or fewer of them every block is kept
 * and the row is marked dense (n_cells = -1).
 *
 * Parity unpinned: the reference's tests hold no vectors for the indexer (it is exercised only through whole-model
 * logits) and its kernels were not run against this file; what pins it is the float64 restatement and the selection's
 * definition (tests/test_oracle_path.py).
 */
#include "oracle.h"

#define QD 128 /* key width */
#define QH 4   /* query heads */
#define QPOOL 4
#define QROT 64

void orc_norm_rope(float* x, const float* w, int pos, float eps, const float* freq, float mscale, int hd, int nrot);

static float bf2f(uint16_t h) { return o_bitsf((uint32_t) h << 16); }

/* y [T][QH QD + QD] */
void orc_qsa_proj(const uint16_t* wq, const uint16_t* wk, const float* x, float* y, int T, int n) {
    const int rows = QH * QD + QD;
#pragma omp parallel for
    for (int r = 0; r < rows; ++r) {
        const uint16_t* w = r < QH * QD ? wq + (size_t) r * n : wk + (size_t) (r - QH * QD) * n;
        for (int t = 0; t < T; ++t) {
            float lanes[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.f;
                for (int c = 2 * l; c < n; c += 64)
                    acc = fmaf(bf2f(w[c]), x[(size_t) t * n + c], fmaf(bf2f(w[c + 1]), x[(size_t) t * n + c + 1], acc));
                lanes[l] = acc;
            }
            y[(size_t) t * rows + r] = o_butterfly(lanes, 32);
        }
    }
}

static size_t pooled_at(const OrcKvPages* g, int b, int ncard) {
    if (!g->pt) return (size_t) b * QD;
    const int bpp = g->rows / 4 * ncard; /* blocks a page holds: every card's */
    return (size_t) g->pt[b / bpp] * g->page + (size_t) (b % bpp) * QD;
}

/* q [T][QH][QD]; ring [ring_rows][QD] f16; pooled: f16 rows of QD, block b at pooled_at */
void orc_qsa_index(const float* y, const float* qn, const float* kn, o_half* ring, int ring_rows, o_half* pooled, const OrcKvPages* g,
                   int ncard, float* q, int pos0, int T, float eps, float rope_base) {
    const int rows = QH * QD + QD;
    float freq[QROT / 2];
    orc_rope_freqs(rope_base, QROT, freq);
    for (int t = 0; t < T; ++t) {
        const int p = pos0 + t;
        for (int h = 0; h < QH; ++h) {
            float* o = q + ((size_t) t * QH + h) * QD;
            memcpy(o, y + (size_t) t * rows + h * QD, QD * sizeof(float));
            orc_norm_rope(o, qn, p, eps, freq, 1.0f, QD, QROT);
        }
        for (int i = 0; i < QD; ++i) ring[(size_t) (p % ring_rows) * QD + i] = o_f2h(y[(size_t) t * rows + QH * QD + i]);
    }
    for (int t = 0; t < T; ++t) {
        const int p = pos0 + t;
        if ((p + 1) % QPOOL != 0) continue;
        float v[QD];
        for (int i = 0; i < QD; ++i) {
            float s = 0.f;
            for (int m = 0; m < QPOOL; ++m) s = s + o_h2f(ring[(size_t) ((p - (QPOOL - 1) + m) % ring_rows) * QD + i]);
            v[i] = s * (1.0f / (float) QPOOL);
        }
        orc_norm_rope(v, kn, p - (QPOOL - 1), eps, freq, 1.0f, QD, QROT);
        o_half* dst = pooled + pooled_at(g, (p + 1) / QPOOL - 1, ncard);
        for (int i = 0; i < QD; ++i) dst[i] = o_f2h(v[i]);
    }
}

static int cmp_desc(const void* a, const void* b) {
    const uint32_t x = *(const uint32_t*) a, y = *(const uint32_t*) b;
    return x < y ? 1 : x > y ? -1 : 0;
}

/* row t at position pos[t] on the page table pts[t] (pts NULL: g's own).  scores [T][max_pools], cells [T][top 4 + 3] */
void orc_qsa_select(const float* q, const o_half* pooled, const OrcKvPages* g, float* scores, int* cells, int* n_cells, int max_pools,
                    const int* pos, const int* const* pts, int T, int card, int ncard, int top) {
    const int maxsel = top * QPOOL + QPOOL - 1;
    const float w = o_rsqrt((float) QD);
#pragma omp parallel for
    for (int t = 0; t < T; ++t) {
        const int p = pos[t], nv = (p + 1) / QPOOL, n_tail = (p + 1) % QPOOL;
        if (nv <= top) {
            n_cells[t] = -1;
            continue;
        }
        OrcKvPages gt = *g;
        if (pts) gt.pt = pts[t];
        float* sc = scores + (size_t) t * max_pools;
        for (int j = 0; j < nv; ++j) {
            const o_half* k = pooled + pooled_at(&gt, j, ncard);
            float s = 0.f;
            float d[QH] = {0};
            for (int dim = 0; dim < QD; dim += 2) {
                const float kx = o_h2f(k[dim]), ky = o_h2f(k[dim + 1]);
                for (int h = 0; h < QH; ++h) {
                    const float* qh = q + ((size_t) t * QH + h) * QD;
                    d[h] = fmaf(qh[dim], kx, fmaf(qh[dim + 1], ky, d[h]));
                }
            }
            for (int h = 0; h < QH; ++h) s = s + fmaxf(d[h], 0.f) * w;
            sc[j] = s;
        }
        uint32_t* key = (uint32_t*) malloc((size_t) nv * sizeof(uint32_t));
        for (int j = 0; j < nv; ++j) key[j] = o_fbits(sc[j]);
        qsort(key, (size_t) nv, sizeof(uint32_t), cmp_desc);
        const uint32_t thr = key[top - 1];
        int above = 0;
        for (int j = 0; j < nv; ++j) above += o_fbits(sc[j]) > thr;
        free(key);
        int ties = top - above, n = 0;
        int* row = cells + (size_t) t * maxsel;
        for (int j = 0; j < nv; ++j) {
            const uint32_t kj = o_fbits(sc[j]);
            int take = kj > thr;
            if (kj == thr && ties > 0) take = 1, --ties;
            if (take && j % ncard == card)
                for (int m = 0; m < QPOOL; ++m) row[n++] = (j / ncard) * QPOOL + m;
        }
        const int jt = p / QPOOL;
        if (jt % ncard == card)
            for (int m = 0; m < n_tail; ++m) row[n++] = (jt / ncard) * QPOOL + (p - n_tail + 1 + m) % QPOOL;
        n_cells[t] = n;
    }
}
