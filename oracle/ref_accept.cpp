// CPU ORACLE - test infrastructure, not product code.
//
// The reference's own host policy code (johnfink8/sfnx src/session.cpp, compiled unmodified from where it lies)
// behind a C interface: make_dist and draw (src/session.cpp:39-82) are the reference's object code; the acceptance
// loop around them restates src/session.cpp:469-510 with the same std::mt19937_64 / uniform_real_distribution.
// The Engine methods session.cpp references are never reached from here and are stubbed to abort.
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "session.hpp"

namespace fnx {
void Engine::load_state(const Engine::SeqState&) { std::abort(); }
std::shared_ptr<Engine::SeqState> Engine::save_state(bool) { std::abort(); }
void Engine::set_images(const std::vector<Engine::Image>&) { std::abort(); }
std::vector<std::vector<std::pair<float, int>>> Engine::top_tokens(int, const Engine::Penalties&) { std::abort(); }
int Engine::draft(int, bool, int, const std::vector<int>&, int, const Engine::Penalties::Row*, bool) { std::abort(); }
void Engine::reset() { std::abort(); }
void Engine::commit(int) { std::abort(); }
std::vector<int> Engine::verify(const std::vector<int>&) { std::abort(); }
void Engine::prefill(const std::vector<int>&, int) { std::abort(); }
void Engine::use_lane(int) { std::abort(); }
void Engine::ngram_prefetch(const std::vector<int>&) const { std::abort(); }
bool Engine::ngram_reads_ahead() const { std::abort(); }
size_t Engine::SeqState::total() const { std::abort(); }
}  // namespace fnx

extern "C" {

struct RefSampling {
    float temperature, top_p, min_p;
    int top_k;
};

static fnx::Sampling to_s(const RefSampling* s) {
    fnx::Sampling r;
    r.temperature = s->temperature;
    r.top_p = s->top_p;
    r.min_p = s->min_p;
    r.top_k = s->top_k;
    return r;
}

void ref_make_dist(const float* cv, const int* ci, int ncand, const RefSampling* s, int* n_out, int* ids, double* p) {
    std::vector<std::pair<float, int>> cand;
    for (int i = 0; i < ncand; ++i) cand.emplace_back(cv[i], ci[i]);
    const fnx::Dist d = fnx::make_dist(cand, to_s(s));
    *n_out = (int) d.ids.size();
    for (size_t i = 0; i < d.ids.size(); ++i) ids[i] = d.ids[i], p[i] = d.p[i];
}

// rows[0] the last committed token, rows[1..] fixed (one-hot) drafts; cand [T][64]; returns the tokens emitted
int ref_accept_sampled(const int* rows, int T, const float* cand_v, const int* cand_i, const RefSampling* s, unsigned long long seed,
                       int skip_draws, int* o, double* u_used) {
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<double> unif(0.0, 1.0);
    for (int i = 0; i < skip_draws; ++i) (void) unif(rng);
    const fnx::Sampling sm = to_s(s);
    int n, nu = 0;
    for (n = 0; n < T; ++n) {
        std::vector<std::pair<float, int>> cand;
        for (int i = 0; i < 64; ++i) cand.emplace_back(cand_v[n * 64 + i], cand_i[n * 64 + i]);
        fnx::Dist d = fnx::make_dist(cand, sm);
        if (n + 1 < T) {
            const int dr = rows[n + 1];
            const double u = unif(rng);
            if (u_used) u_used[nu] = u;
            ++nu;
            if (u * 1.0 < d.prob(dr)) {
                o[n] = dr;
                continue;
            }
            const fnx::Dist p0 = d;
            double rest = 0.0;
            for (size_t i = 0; i < d.ids.size(); ++i) {
                const double qi = d.ids[i] == dr ? 1.0 : 0.0;
                d.p[i] = std::max(0.0, d.p[i] - qi);
                rest += d.p[i];
            }
            if (rest > 1e-12) for (double& v : d.p) v /= rest;
            else d = p0;
        }
        const double u = unif(rng);
        if (u_used) u_used[nu] = u;
        ++nu;
        o[n] = fnx::draw(d, u);
        ++n;
        break;
    }
    return n;
}

// the reference's own lookup_drafts (src/session.cpp:377-394): returns the number of drafts written to out
int ref_lookup_drafts(const int* ctx, int n, int lk, int d1, int* out) {
    const std::vector<int> r = fnx::lookup_drafts(std::vector<int>(ctx, ctx + n), lk, d1);
    for (size_t i = 0; i < r.size(); ++i) out[i] = r[i];
    return (int) r.size();
}

// the unit uniforms std::mt19937_64(seed) gives through uniform_real_distribution<double>(0, 1)
void ref_uniforms(unsigned long long seed, int n, double* u) {
    std::mt19937_64 rng(seed);
    std::uniform_real_distribution<double> unif(0.0, 1.0);
    for (int i = 0; i < n; ++i) u[i] = unif(rng);
}
}
