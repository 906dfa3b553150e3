/* CPU ORACLE - test infrastructure, not product code.
 *
 * Output-head reductions and acceptance of the verify window, restated from the reference:
 *   argmax per vocabulary slice and merge across slices   src/kernels.cu:870-908, src/engine_common.cu:781-787
 *   sampler penalties + exact top-64                       src/topk.cuh:17-138 (host statement tools/topk_test.cu:33-49),
 *                                                          merge of the slices' lists src/engine_common.cu:640-653
 *   candidate distribution and draw                        src/session.cpp:39-82
 *   greedy prefix acceptance / rejection sampling          src/session.cpp:469-510
 *   all-reduce addition order of the ring                  src/kernels.cu:808-868
 */
#include "oracle.h"

/* best[t] = (largest value, lowest index on ties) of logits[t][0..rows), index + v0; returns 16 if a logit is not finite */
unsigned orc_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i) {
    unsigned err = 0;
    for (int t = 0; t < T; ++t) {
        uint64_t best = 0;
        for (int i = 0; i < rows; ++i) {
            const float v = logits[(size_t) t * rows + i];
            if (!isfinite(v)) err |= 16u;
            const uint64_t k = ((uint64_t) o_fkey(v) << 32) | (uint32_t) ~(uint32_t) i;
            if (k > best) best = k;
        }
        const uint32_t kv = (uint32_t) (best >> 32);
        best_v[t] = o_bitsf((kv & 0x80000000u) ? (kv & 0x7fffffffu) : ~kv);
        best_i[t] = (int) ~(uint32_t) best + v0;
    }
    return err;
}

/* across slices: strict > scanning slice 0 upward, so the lower slice wins ties */
void orc_argmax_merge(const float* best_v, const int* best_i, int nslice, int T, int* out) {
    for (int t = 0; t < T; ++t) {
        int b = 0;
        for (int c = 1; c < nslice; ++c)
            if (best_v[c * T + t] > best_v[b * T + t]) b = c;
        out[t] = best_i[b * T + t];
    }
}

typedef struct {
    float v;
    int i;
} Cand;
static int cand_cmp(const void* pa, const void* pb) { /* logit descending, id ascending */
    const Cand* a = (const Cand*) pa;
    const Cand* b = (const Cand*) pb;
    if (a->v > b->v) return -1;
    if (a->v < b->v) return 1;
    return a->i < b->i ? -1 : a->i > b->i ? 1 : 0;
}

/* per row: penalties in place on this slice (tokens v0 .. v0 + n), then its 64 highest as (logit desc, id asc) */
unsigned orc_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n,
                        int pen_stride, const float* pen_par, float* out_v, int* out_i) {
    unsigned err = 0;
    Cand* c = (Cand*) malloc(sizeof(Cand) * (size_t) n);
    for (int row = 0; row < T; ++row) {
        float* L = logits + (size_t) row * n;
        for (int j = 0; j < n; ++j)
            if (!isfinite(L[j])) err |= 16u;
        const float repeat = pen_par[row * 3], freq = pen_par[row * 3 + 1], present = pen_par[row * 3 + 2];
        for (int i = 0; i < pen_n[row]; ++i) {
            const int tok = pen_tok[row * pen_stride + i] - v0, cnt = pen_cnt[row * pen_stride + i];
            if (tok < 0 || tok >= n || cnt <= 0) continue;
            float l = L[tok];
            l = l <= 0.f ? l * repeat : l / repeat;
            L[tok] = l - (float) cnt * freq - present;
        }
        for (int j = 0; j < n; ++j) {
            c[j].v = L[j];
            c[j].i = j;
        }
        qsort(c, (size_t) n, sizeof(Cand), cand_cmp);
        for (int k = 0; k < ORC_TOPK_N; ++k) {
            out_v[row * ORC_TOPK_N + k] = c[k].v;
            out_i[row * ORC_TOPK_N + k] = v0 + c[k].i;
        }
    }
    free(c);
    return err;
}

/* the slices' lists (each sorted) merged into the row's 64 best by the same order */
void orc_top_merge(const float* vs, const int* is, int nslice, int T, float* out_v, int* out_i) {
    Cand* c = (Cand*) malloc(sizeof(Cand) * (size_t) nslice * ORC_TOPK_N);
    for (int t = 0; t < T; ++t) {
        for (int s = 0; s < nslice; ++s)
            for (int k = 0; k < ORC_TOPK_N; ++k) {
                c[s * ORC_TOPK_N + k].v = vs[((size_t) s * T + t) * ORC_TOPK_N + k];
                c[s * ORC_TOPK_N + k].i = is[((size_t) s * T + t) * ORC_TOPK_N + k];
            }
        qsort(c, (size_t) nslice * ORC_TOPK_N, sizeof(Cand), cand_cmp);
        for (int k = 0; k < ORC_TOPK_N; ++k) {
            out_v[t * ORC_TOPK_N + k] = c[k].v;
            out_i[t * ORC_TOPK_N + k] = c[k].i;
        }
    }
    free(c);
}

/* ---- sampling (host policy; double arithmetic with the host libm, as the reference's own host code) */
typedef struct {
    int n;
    int ids[ORC_TOPK_N];
    double p[ORC_TOPK_N];
} Dist;

static void make_dist(const float* cv, const int* ci, int ncand, const OrcSampling* s, Dist* d) {
    const int k = (s->top_k <= 0 || s->top_k > ncand) ? ncand : s->top_k;
    int keep = k;
    const double mx = cv[0];
    if (s->top_p < 1.f) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += exp((double) cv[i] - mx);
        double cum = 0.0;
        for (int i = 0; i < k; ++i) {
            cum += exp((double) cv[i] - mx) / sum;
            if (cum >= (double) s->top_p) {
                keep = i + 1;
                break;
            }
        }
    }
    if (s->min_p > 0.f) {
        const float thresh = cv[0] + logf(s->min_p);
        for (int i = 1; i < keep; ++i)
            if (cv[i] < thresh) {
                keep = i;
                break;
            }
    }
    const double inv_t = 1.0 / s->temperature, smx = cv[0] * inv_t;
    double sum = 0.0;
    d->n = keep;
    for (int i = 0; i < keep; ++i) {
        d->ids[i] = ci[i];
        d->p[i] = exp(cv[i] * inv_t - smx);
        sum += d->p[i];
    }
    for (int i = 0; i < keep; ++i) d->p[i] /= sum;
}
static double dist_prob(const Dist* d, int id) {
    for (int i = 0; i < d->n; ++i)
        if (d->ids[i] == id) return d->p[i];
    return 0.0;
}
static int dist_draw(const Dist* d, double u) {
    double cum = 0.0;
    for (int i = 0; i < d->n; ++i) {
        cum += d->p[i];
        if (u < cum) return d->ids[i];
    }
    return d->ids[d->n - 1];
}

void orc_make_dist(const float* cv, const int* ci, int ncand, const OrcSampling* s, int* n_out, int* ids, double* p) {
    Dist d;
    make_dist(cv, ci, ncand, s, &d);
    *n_out = d.n;
    memcpy(ids, d.ids, sizeof(int) * d.n);
    memcpy(p, d.p, sizeof(double) * d.n);
}

/* the 64-bit Mersenne twister (Matsumoto & Nishimura 2004, as std::mt19937_64) and the unit uniform the C++ library
 * builds on it for double: one draw x, u = (double) x / 2^64, the value below 1 when that rounds to 1 */
void orc_mt_seed(OrcMt* g, uint64_t seed) {
    g->mt[0] = seed;
    for (int i = 1; i < 312; ++i) g->mt[i] = 6364136223846793005ULL * (g->mt[i - 1] ^ (g->mt[i - 1] >> 62)) + (uint64_t) i;
    g->idx = 312;
}
uint64_t orc_mt_next(OrcMt* g) {
    if (g->idx >= 312) {
        for (int i = 0; i < 312; ++i) {
            const uint64_t x = (g->mt[i] & 0xFFFFFFFF80000000ULL) | (g->mt[(i + 1) % 312] & 0x7FFFFFFFULL);
            g->mt[i] = g->mt[(i + 156) % 312] ^ (x >> 1) ^ ((x & 1ULL) ? 0xB5026F5AA96619E9ULL : 0ULL);
        }
        g->idx = 0;
    }
    uint64_t y = g->mt[g->idx++];
    y ^= (y >> 29) & 0x5555555555555555ULL;
    y ^= (y << 17) & 0x71D67FFFEDA60000ULL;
    y ^= (y << 37) & 0xFFF7EEE000000000ULL;
    y ^= y >> 43;
    return y;
}
double orc_mt_unif(OrcMt* g) {
    const double u = (double) orc_mt_next(g) / 18446744073709551616.0;
    return u >= 1.0 ? nextafter(1.0, 0.0) : u;
}

/* greedy: rows[0] is the last committed token, rows[1..] the drafts, out[t] row t's argmax; n = 1 + the longest
 * prefix with rows[n] == out[n - 1] */
/* n-gram lookup drafts (reference src/session.cpp:377-394).  Written as the definition reads: among the starts s < n - 3 of a
 * trigram equal to the last one take the largest; it yields drafts only if position s + 3 exists before the end and holds d1
 * (when d1 >= 0); the count is min(lk, max(3, m)) where m - 3 is how many tokens before both trigrams agree (capped so that
 * m <= lk and the earlier run does not leave the context); image cells end the list. */
int orc_lookup_drafts(const int* ctx, int n, int lk, int d1, int image_tok, int* out) {
    if (lk == 0 || n <= 3) return 0;
    const int n0 = n - 3;
    int s = -1;
    for (int c = 0; c < n0; ++c)
        if (ctx[c] == ctx[n0] && ctx[c + 1] == ctx[n0 + 1] && ctx[c + 2] == ctx[n0 + 2]) s = c; /* the last one found is the latest */
    if (s < 0) return 0;
    if (!(s + 3 < n)) return 0;
    if (d1 >= 0 && ctx[s + 3] != d1) return 0;
    int back = 0;
    while (3 + back < lk && back < s && ctx[s - 1 - back] == ctx[n0 - 1 - back]) ++back;
    int k = 3 + back;
    if (k < 3) k = 3;
    if (k > lk) k = lk;
    int cnt = 0;
    for (int i = s + 3; i < n && i < s + 3 + k; ++i) {
        if (ctx[i] >= image_tok) break;
        out[cnt++] = ctx[i];
    }
    return cnt;
}

int orc_accept_greedy(const int* rows, const int* out, int T) {
    int n = 1;
    while (n < T && rows[n] == out[n - 1]) ++n;
    return n;
}

/* sampled, fixed (one-hot) drafts: row n's candidates cand_v/cand_i [T][64]; o[] receives the emitted tokens;
 * returns how many.  One uniform per accept test, one per draw. */
int orc_accept_sampled(const int* rows, int T, const float* cand_v, const int* cand_i, const OrcSampling* s, OrcMt* rng,
                       int* o) {
    int n;
    for (n = 0; n < T; ++n) {
        Dist d;
        make_dist(cand_v + (size_t) n * ORC_TOPK_N, cand_i + (size_t) n * ORC_TOPK_N, ORC_TOPK_N, s, &d);
        if (n + 1 < T) {
            const int dr = rows[n + 1];
            if (orc_mt_unif(rng) * 1.0 < dist_prob(&d, dr)) {
                o[n] = dr;
                continue;
            }
            const Dist p0 = d;
            double rest = 0.0;
            for (int i = 0; i < d.n; ++i) {
                const double qi = d.ids[i] == dr ? 1.0 : 0.0;
                d.p[i] = d.p[i] - qi > 0.0 ? d.p[i] - qi : 0.0;
                rest += d.p[i];
            }
            if (rest > 1e-12)
                for (int i = 0; i < d.n; ++i) d.p[i] /= rest;
            else d = p0;
        }
        o[n] = dist_draw(&d, orc_mt_unif(rng));
        ++n;
        break;
    }
    return n;
}

/* all-reduce(sum) of n ranks' addends x[r][len] in the ring's order: the elements are cut into n chunks of pairs
 * (pairs [c NP / n, (c+1) NP / n), NP = row_len / 2, per row); chunk c is started by rank c and each next rank adds its
 * own: ((x_c + x_{c+1}) + ...) + x_{c+n-1} */
void orc_ring_sum(const float* const* x, float* out, int nrank, int T, int row_len) {
    const int NP = row_len / 2;
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < nrank; ++c) {
            const int lo = c * NP / nrank, hi = (c + 1) * NP / nrank;
            for (int e = 2 * lo; e < 2 * hi; ++e) {
                float v = x[c][(size_t) t * row_len + e];
                for (int s = 1; s < nrank; ++s) v = v + x[(c + s) % nrank][(size_t) t * row_len + e];
                out[(size_t) t * row_len + e] = v;
            }
        }
}
