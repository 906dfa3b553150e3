/* CPU ORACLE - test infrastructure, not product code.
 *
 * Position-split attention of the verify window, restated with IEEE arithmetic from the reference:
 *   per-head RMS norm + NEOX rotary + K/V append     src/kernels.cu:451-469, 1539-1569; src/rope.hpp:29-39
 *   K/V placement (blocks of 4 positions dealt round-robin)  src/kernels.hpp:126-130, src/kernels.cu:491-495
 *   split-K online softmax over owned positions      src/kernels.cu:497-582
 *   merge of the 16 splits                           src/kernels.cu:585-606
 *   merge of the cards' partials in ring order, gate src/kernels.cu:609-672
 *   int8 K/V rows (groups of 32, f16 scale)          src/kernels.hpp:149-181; append src/kernels.cu:1561-1566; scan :531-537
 *     stated with IEEE division where the reference's fast-math build divides: d = amax / 127, id = 1 / d,
 *     q = roundf(x id), value read back as (float) q * f16(d)
 */
#include "oracle.h"

#define ATT_SPLITS 16
#define ATT_CH 32

int orc_kv_owned(int p, int card, int ncard) { /* positions <= p that `card` owns */
    const int b = p / 4;
    const int blocks = (b + ncard - 1 - card) / ncard;
    return blocks * 4 + (b % ncard == card ? p % 4 + 1 : 0);
}

static size_t kv_row_at(const OrcKvPages* g, int r, int nkv, int hd) {
    if (!g->pt) return (size_t) r * nkv * hd;
    return (size_t) g->pt[r / g->rows] * g->page + (size_t) (r % g->rows) * nkv * hd;
}

/* int8 rows: row r's first byte and its first scale (in halves), both from the layer's pointer; a page's scales follow
 * its rows (kvq_row, kvq_scale); without a page table the cache is one page of g->cap rows */
static size_t kvq_row_at(const OrcKvPages* g, int r, int nkv, int hd) {
    if (!g->pt) return (size_t) r * nkv * hd;
    return (size_t) g->pt[r / g->rows] * g->page * 2 + (size_t) (r % g->rows) * nkv * hd;
}
static size_t kvq_scale_at(const OrcKvPages* g, int r, int nkv, int hd) {
    if (!g->pt) return (size_t) g->cap * nkv * hd / 2 + (size_t) r * nkv * hd / 32;
    return (size_t) g->pt[r / g->rows] * g->page + (size_t) g->rows * nkv * hd / 2 + (size_t) (r % g->rows) * nkv * hd / 32;
}
/* element e of head kvh of local row r as the scan reads it */
static float kv_value(const o_half* cache, const OrcKvPages* g, int r, int nkv, int hd, int kvh, int d) {
    if (!g->q8) return o_h2f(cache[kv_row_at(g, r, nkv, hd) + (size_t) kvh * hd + d]);
    const int e = kvh * hd + d;
    const int8_t q = ((const int8_t*) cache)[kvq_row_at(g, r, nkv, hd) + e];
    return (float) q * o_h2f(cache[kvq_scale_at(g, r, nkv, hd) + e / 32]);
}
static void kv_append_row(o_half* cache, const OrcKvPages* g, int r, int nkv, int hd, const float* x) {
    if (!g->q8) {
        const size_t at = kv_row_at(g, r, nkv, hd);
        for (int e = 0; e < nkv * hd; ++e) cache[at + e] = o_f2h(x[e]);
        return;
    }
    for (int b = 0; b < nkv * hd / 32; ++b) {
        float amax = 0.f;
        for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(x[b * 32 + l]));
        const float d = amax / 127.f, id = d != 0.f ? 1.f / d : 0.f;
        for (int l = 0; l < 32; ++l) ((int8_t*) cache)[kvq_row_at(g, r, nkv, hd) + b * 32 + l] = (int8_t) roundf(x[b * 32 + l] * id);
        cache[kvq_scale_at(g, r, nkv, hd) + b] = o_f2h(d);
    }
}

/* RMS norm with weight, then rotation of the pairs (i, i + nrot/2), i < nrot/2, at position pos */
void orc_norm_rope(float* x, const float* w, int pos, float eps, const float* freq, float mscale, int hd, int nrot) {
    float tot = 0.f;
    for (int wp = 0; wp < hd / 32; ++wp) {
        float v[32];
        for (int l = 0; l < 32; ++l) v[l] = x[wp * 32 + l] * x[wp * 32 + l];
        tot = tot + o_butterfly(v, 32);
    }
    const float rr = o_rsqrt(tot / (float) hd + eps);
    for (int i = 0; i < hd; ++i) x[i] = x[i] * rr * w[i];
    for (int i = 0; i < nrot / 2; ++i) {
        const float theta = (float) pos * freq[i];
        float sn, cs;
        o_sincos((double) theta, &sn, &cs);
        sn = sn * mscale;
        cs = cs * mscale;
        const float x0 = x[i], x1 = x[i + nrot / 2];
        x[i] = fmaf(-x1, sn, x0 * cs);
        x[i + nrot / 2] = fmaf(x1, cs, x0 * sn);
    }
}

/* the rotary's unit frequencies, base^(-2 i / nrot) with the host libm's powf (unscaled rope, src/rope.hpp:33-35) */
void orc_rope_freqs(float base, int nrot, float* freq) {
    for (int i = 0; i < nrot / 2; ++i) freq[i] = powf(base, -2.0f * (float) i / (float) nrot);
}

/* qg [T][nq][2 hd] (q | gate) and k [T][nkv][hd] normed and rotated in place; K and V rows of the positions this
 * card owns rounded to f16 into the cache at local row (j / ncard) * 4 + p % 4, j = p / 4 */
void orc_attn_prep_append(float* qg, float* k, const float* v, const float* q_norm, const float* k_norm, o_half* kc, o_half* vc,
                          const OrcKvPages* g, int card, int ncard, int T, int pos0, float eps, float rope_base, int nq,
                          int nkv, int hd, int nrot) {
    float freq[128];
    orc_rope_freqs(rope_base, nrot, freq);
    for (int t = 0; t < T; ++t) {
        const int p = pos0 + t, j = p / 4;
        for (int h = 0; h < nq; ++h) orc_norm_rope(qg + ((size_t) t * nq + h) * 2 * hd, q_norm, p, eps, freq, 1.0f, hd, nrot);
        for (int h = 0; h < nkv; ++h) orc_norm_rope(k + ((size_t) t * nkv + h) * hd, k_norm, p, eps, freq, 1.0f, hd, nrot);
        if (j % ncard != card) continue;
        const int r = (j / ncard) * 4 + p % 4;
        kv_append_row(kc, g, r, nkv, hd, k + (size_t) t * nkv * hd);
        kv_append_row(vc, g, r, nkv, hd, v + (size_t) t * nkv * hd);
    }
}

/* this card's partial for every (row, head): part[(t nq + h) (hd + 2)] = acc[hd], m, z.  cells / n_cells (NULL: none): a
 * row with n_cells[t] >= 0 attends the n_cells[t] local rows cells[t maxsel ...] in that order instead of every owned
 * position up to its own (the block selection's list, src/kernels.cu:504-505, 525) */
void orc_attn_partial_cells(const float* qg, const o_half* kc, const o_half* vc, const OrcKvPages* g, float* part, int card,
                            int ncard, int T, int pos0, int nq, int nkv, int hd, const int* cells, const int* n_cells, int maxsel) {
    const int qpk = nq / nkv;
    const float rs = o_rsqrt((float) hd);
#pragma omp parallel for collapse(2)
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < nq; ++h) {
            const int kvh = h / qpk;
            const float* q = qg + ((size_t) t * nq + h) * 2 * hd;
            const int* list = cells && n_cells[t] >= 0 ? cells + (size_t) t * maxsel : NULL;
            const int ctx = list ? n_cells[t] : orc_kv_owned(pos0 + t, card, ncard);
            const int len = ((ctx + ATT_SPLITS - 1) / ATT_SPLITS + ATT_CH - 1) / ATT_CH * ATT_CH;
            float sm[ATT_SPLITS], sz[ATT_SPLITS];
            float* sacc = (float*) calloc((size_t) ATT_SPLITS * hd, sizeof(float));
            for (int s = 0; s < ATT_SPLITS; ++s) {
                const int p0 = s * len, p1 = ctx < p0 + len ? ctx : p0 + len;
                float m = -INFINITY, z = 0.f;
                float* acc = sacc + (size_t) s * hd;
                for (int c0 = p0; c0 < p1; c0 += ATT_CH) {
                    const int np = p1 - c0 < ATT_CH ? p1 - c0 : ATT_CH;
                    float sv[ATT_CH], w[ATT_CH], wl[ATT_CH];
                    float cmax = -INFINITY;
                    for (int pp = 0; pp < ATT_CH; ++pp) {
                        if (pp >= np) {
                            sv[pp] = -INFINITY;
                            continue;
                        }
                        float a = 0.f;
                        for (int d = 0; d < hd; ++d) a = fmaf(q[d], kv_value(kc, g, list ? list[c0 + pp] : c0 + pp, nkv, hd, kvh, d), a);
                        sv[pp] = a * rs;
                        cmax = fmaxf(cmax, sv[pp]);
                    }
                    const float mn = fmaxf(m, cmax);
                    for (int pp = 0; pp < ATT_CH; ++pp) wl[pp] = w[pp] = sv[pp] == -INFINITY ? 0.f : o_expf(sv[pp] - mn);
                    const float sc = m == -INFINITY ? 0.f : o_expf(m - mn);
                    z = fmaf(z, sc, o_butterfly(wl, ATT_CH));
                    m = mn;
                    for (int d = 0; d < hd; ++d) acc[d] = acc[d] * sc;
                    for (int pp = 0; pp < np; ++pp) {
                        for (int d = 0; d < hd; ++d) acc[d] = fmaf(w[pp], kv_value(vc, g, list ? list[c0 + pp] : c0 + pp, nkv, hd, kvh, d), acc[d]);
                    }
                }
                sm[s] = m;
                sz[s] = z;
            }
            float mx = -INFINITY;
            for (int s = 0; s < ATT_SPLITS; ++s) mx = fmaxf(mx, sm[s]);
            float* o = part + ((size_t) t * nq + h) * (hd + 2);
            float z = 0.f;
            for (int d = 0; d < hd; ++d) o[d] = 0.f;
            for (int s = 0; s < ATT_SPLITS; ++s) {
                if (sm[s] == -INFINITY) continue;
                const float w = o_expf(sm[s] - mx);
                z = fmaf(w, sz[s], z);
                for (int d = 0; d < hd; ++d) o[d] = fmaf(w, sacc[(size_t) s * hd + d], o[d]);
            }
            o[hd] = mx;
            o[hd + 1] = z;
            free(sacc);
        }
}

void orc_attn_partial(const float* qg, const o_half* kc, const o_half* vc, const OrcKvPages* g, float* part, int card,
                      int ncard, int T, int pos0, int nq, int nkv, int hd) {
    orc_attn_partial_cells(qg, kc, vc, g, part, card, ncard, T, pos0, nq, nkv, hd, NULL, NULL, 0);
}

/* the cards' partials merged per head in ring order for the head's owner card c (heads [c nq/ncard, (c+1) nq/ncard)):
 * ((P[c+1] + P[c+2]) + ... + P[c-1]) + P[c]; out[t][nq][hd] = a / z * sigmoid(gate).  parts[card] as orc_attn_partial
 * wrote them.  ncard == 1: the partial itself. */
void orc_attn_merge(const float* const* parts, const float* qg, float* out, int ncard, int T, int nq, int hd) {
    const int own = nq / ncard;
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < nq; ++h) {
            const int c = h / own;
            const size_t at = ((size_t) t * nq + h) * (hd + 2);
            const float* first = parts[(c + 1) % ncard] + at;
            float m = first[hd], z = first[hd + 1];
            float* a = (float*) malloc(sizeof(float) * hd);
            memcpy(a, first, sizeof(float) * hd);
            for (int s = 2; s <= ncard; ++s) {
                const float* p2 = parts[(c + s) % ncard] + at;
                const float m2 = p2[hd], z2 = p2[hd + 1];
                const float mn = fmaxf(m, m2);
                const float w1 = m == -INFINITY ? 0.f : o_expf(m - mn), w2 = m2 == -INFINITY ? 0.f : o_expf(m2 - mn);
                z = fmaf(w2, z2, w1 * z);
                for (int d = 0; d < hd; ++d) a[d] = fmaf(w2, p2[d], w1 * a[d]);
                m = mn;
            }
            const float* gate = qg + ((size_t) t * nq + h) * 2 * hd + hd;
            for (int d = 0; d < hd; ++d) out[((size_t) t * nq + h) * hd + d] = a[d] / z * o_sigmoid(gate[d]);
            free(a);
        }
}
