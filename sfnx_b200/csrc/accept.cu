// Acceptance of a verify window on the host: greedy prefix match and rejection sampling against fixed drafts over the
// rows' 64 candidates, and the merge of the GPUs' candidate lists.  Restated from the reference's Session, statement for
// statement where the arithmetic demands it (src/session.cpp:39-82 make_dist / draw, 469-510 the acceptance loop;
// src/engine_common.cu:640-653 the merge), as free functions over plain arrays: this is host policy the drop-in keeps,
// and the reference's own object code is its checker (oracle/ref_accept.cpp).
#include <algorithm>
#include <cmath>
#include <random>
#include <vector>

#include "common.cuh"

namespace {

struct Dist {
    int n = 0;
    int ids[FNX_TOPK_N];
    double p[FNX_TOPK_N];
    double prob(int id) const {
        for (int i = 0; i < n; ++i)
            if (ids[i] == id) return p[i];
        return 0.0;
    }
};

// top_k, then top_p over the untempered softmax (double), then min_p as a logit threshold, then the temperature's
// softmax over the survivors; cand sorted by (logit desc, id asc)
Dist make_dist(const float* cv, const int* ci, int ncand, const FnxSampling& s) {
    const int k = (s.top_k <= 0 || s.top_k > ncand) ? ncand : s.top_k;
    int keep = k;
    const double mx = cv[0];
    if (s.top_p < 1.f) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += std::exp((double) cv[i] - mx);
        double cum = 0.0;
        for (int i = 0; i < k; ++i) {
            cum += std::exp((double) cv[i] - mx) / sum;
            if (cum >= (double) s.top_p) {
                keep = i + 1;
                break;
            }
        }
    }
    if (s.min_p > 0.f) {
        const float thresh = cv[0] + std::log(s.min_p);
        for (int i = 1; i < keep; ++i)
            if (cv[i] < thresh) {
                keep = i;
                break;
            }
    }
    Dist d;
    const double inv_t = 1.0 / s.temperature, smx = cv[0] * inv_t;
    double sum = 0.0;
    d.n = keep;
    for (int i = 0; i < keep; ++i) {
        d.ids[i] = ci[i];
        d.p[i] = std::exp(cv[i] * inv_t - smx);
        sum += d.p[i];
    }
    for (int i = 0; i < keep; ++i) d.p[i] /= sum;
    return d;
}

int draw(const Dist& d, double u) {
    double cum = 0.0;
    for (int i = 0; i < d.n; ++i) {
        cum += d.p[i];
        if (u < cum) return d.ids[i];
    }
    return d.ids[d.n - 1];
}

struct Rng {
    std::mt19937_64 gen;
    std::uniform_real_distribution<double> unif{0.0, 1.0};
};

}  // namespace

extern "C" {

int fnx_accept_greedy(const int* rows, const int* out, int T) {
    int n = 1;
    while (n < T && rows[n] == out[n - 1]) ++n;
    return n;
}

void* fnx_rng_new(unsigned long long seed) {
    Rng* r = new Rng;
    r->gen.seed(seed);
    return r;
}
void fnx_rng_free(void* rng) { delete (Rng*) rng; }

// draft rows[n + 1] stands with probability min(1, p_n(draft)) (a fixed draft's q is all on it); else row n's token is
// drawn from max(0, p_n - q_n) normalised and the window ends; all standing: one more from the last row.  One uniform
// per test and per draw.
int fnx_accept_sampled(const int* rows, int T, const float* cand_v, const int* cand_i, const FnxSampling* s, void* rng, int* o) {
    Rng& r = *(Rng*) rng;
    int n;
    for (n = 0; n < T; ++n) {
        Dist d = make_dist(cand_v + (size_t) n * FNX_TOPK_N, cand_i + (size_t) n * FNX_TOPK_N, FNX_TOPK_N, *s);
        if (n + 1 < T) {
            const int dr = rows[n + 1];
            if (r.unif(r.gen) * 1.0 < d.prob(dr)) {
                o[n] = dr;
                continue;
            }
            const Dist p0 = d;
            double rest = 0.0;
            for (int i = 0; i < d.n; ++i) {
                const double qi = d.ids[i] == dr ? 1.0 : 0.0;
                d.p[i] = std::max(0.0, d.p[i] - qi);
                rest += d.p[i];
            }
            if (rest > 1e-12)
                for (int i = 0; i < d.n; ++i) d.p[i] /= rest;
            else d = p0;
        }
        o[n] = draw(d, r.unif(r.gen));
        ++n;
        break;
    }
    return n;
}

// n-gram lookup drafts (reference src/session.cpp:377-394, lookup_drafts; LOOKUP_N = LOOKUP_MIN = 3): the tokens that followed
// the latest earlier occurrence of the context's last three tokens.  Only that latest occurrence is looked at; it offers
// drafts if a token follows it and (d1 >= 0) that token is d1.  How many: the match is grown backwards from the trigram, up
// to lk tokens, and k = min(lk, max(3, match length)) tokens are taken (fewer at the context's end); tokens from the first
// image cell (>= image_tok) on are dropped.  Returns the number of drafts written to out (room for lk).
int fnx_lookup_drafts(const int* ctx, int n, int lk, int d1, int image_tok, int* out) {
    constexpr int NG = 3, KMIN = 3;
    if (!ctx || !out || n < 0 || lk < 0) return -fnxk::fail("lookup_drafts: bad arguments (%d tokens, %d drafts)", n, lk);
    if (lk == 0 || n <= NG) return 0;
    const int tail = n - NG;   // where the context's last trigram starts
    int found = -1;
    for (int s = tail - 1; s >= 0 && found < 0; --s)
        if (ctx[s] == ctx[tail] && ctx[s + 1] == ctx[tail + 1] && ctx[s + 2] == ctx[tail + 2]) found = s;
    if (found < 0 || found + NG >= n || (d1 >= 0 && ctx[found + NG] != d1)) return 0;
    int m = NG;   // tokens before the two trigrams that agree as well
    while (m < lk && m - NG < found && ctx[found - 1 - (m - NG)] == ctx[tail - 1 - (m - NG)]) ++m;
    const int k = std::min(lk, std::max(KMIN, m)), end = std::min(n, found + NG + k);
    int cnt = 0;
    for (int i = found + NG; i < end && ctx[i] < image_tok; ++i) out[cnt++] = ctx[i];
    return cnt;
}

int fnx_top_merge(const float* vs, const int* is, int nslice, int T, float* out_v, int* out_i) {
    if (nslice < 1 || T < 1) return fnxk::fail("top_merge: %d slices, %d rows", nslice, T);
    std::vector<std::pair<float, int>> c((size_t) nslice * FNX_TOPK_N);
    for (int t = 0; t < T; ++t) {
        for (int s = 0; s < nslice; ++s)
            for (int k = 0; k < FNX_TOPK_N; ++k)
                c[(size_t) s * FNX_TOPK_N + k] = {vs[((size_t) s * T + t) * FNX_TOPK_N + k], is[((size_t) s * T + t) * FNX_TOPK_N + k]};
        std::sort(c.begin(), c.end(), [](const std::pair<float, int>& a, const std::pair<float, int>& b) {
            return a.first > b.first || (a.first == b.first && a.second < b.second);
        });
        for (int k = 0; k < FNX_TOPK_N; ++k) out_v[t * FNX_TOPK_N + k] = c[k].first, out_i[t * FNX_TOPK_N + k] = c[k].second;
    }
    return 0;
}
}
