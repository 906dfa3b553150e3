// TEST INFRASTRUCTURE: a C ABI over the reference's own kernel launchers (namespace fnx, src/kernels.hpp), so that the
// GPU tests can run the reference's kernels - compiled unmodified from its tree for sm_100a by oracle/Makefile
// (`make refgpu`) into oracle/_ref/libref_kernels.so - beside this library's on the same inputs.  Only launchers whose
// kernels neither wait on another GPU nor on a grid-wide barrier are exposed (not ring_sum, attn / attn_finish's merge,
// hc_read).  The reference's shapes are compile-time constants (src/model.hpp:40-45): ref_shapes() reports them.
#include <cuda_runtime.h>

#include <cstdio>
#include <stdexcept>

#include "kernels.hpp"

namespace {
thread_local char g_err[512];
template <typename F> int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        snprintf(g_err, sizeof g_err, "%s", e.what());
        return 1;
    }
}
}  // namespace

extern "C" {

const char* ref_last_error(void) { return g_err; }

// N, NEXP, TOPK, FF, NKH, NVH, HS, NQH, NKVH, HD, NROT, MAXT, NCARD, attn_rows()
int ref_shapes(int* out) {
    const int v[14] = {fnx::N, fnx::NEXP, fnx::TOPK, fnx::FF, fnx::NKH, fnx::NVH, fnx::HS, fnx::NQH, fnx::NKVH, fnx::HD, fnx::NROT, fnx::MAXT, fnx::NCARD,
                       fnx::attn_rows()};
    for (int i = 0; i < 14; ++i) out[i] = v[i];
    return 14;
}

int ref_quantize_q8_1(const float* x, void* q, int n, int rows, void* st) {
    return guarded([&] { fnx::quantize_q8_1(x, q, n, rows, st); });
}

int ref_router_route(const float* W, const float* x, float* logits, int T, int* topi, float* topw, void* jobs_gu, void* jobs_dn, int* njobs, void* st) {
    return guarded([&] { fnx::router_route(W, x, logits, T, topi, topw, (fnx::Job*) jobs_gu, (fnx::Job*) jobs_dn, njobs, st); });
}

// Q4_K experts: expert e's stacked [gate | up] rows (nrows of ncols values, GGUF blocks) at a + e * stride
int ref_moe_gate_up_q4k(const void* a, size_t stride, int nrows, int ncols, const void* jobs, const int* njobs, int njobs_max, const void* xq, float* gu,
                        void* st) {
    return guarded([&] {
        fnx::DW A;
        A.p = const_cast<void*>(a);
        A.type = fnx::T_Q4_K;
        A.n_in = ncols, A.n_out = nrows;
        A.row_bytes = (size_t) ncols / 256 * 144;
        fnx::moe_gate_up(A, stride, (const fnx::Job*) jobs, njobs, njobs_max, xq, gu, st);
    });
}

int ref_q8s_gemv(const int8_t* q, const uint16_t* d, int rows, int cols, const void* y, float* out, int out_stride, int T, void* st) {
    return guarded([&] {
        fnx::Q8S w;
        w.q = const_cast<int8_t*>(q), w.d = const_cast<uint16_t*>(d);
        fnx::q8s_gemv(w, rows, cols, y, out, out_stride, T, st);
    });
}

size_t ref_gdn_scratch_floats(int nv) { return fnx::gdn_scratch_floats(nv); }
int ref_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a, const float* nw, float* S, void* yq,
                 const int* ctl, float* scratch, float* snap, float* hsnap, int nk, int nv, const int* vmap, int T, float eps, void* st, float* y32) {
    return guarded([&] { fnx::gdn_core(qkvz, ab, hist, convw, dt, a, nw, S, yq, ctl, scratch, snap, hsnap, nk, nv, vmap, T, eps, st, y32); });
}

// the scan's per-run partials of T rows, each row at *pos[t] on the page table pt[t] (f16 K/V, every owned position):
// scratch gets acc [T][NQH][16][HD] and, ref_attn_mz_offset() floats in, (m, z) [T][NQH][16]
size_t ref_attn_scratch_floats(void) { return fnx::attn_scratch_floats(fnx::NQH); }
size_t ref_attn_mz_offset(void) { return (size_t) fnx::attn_rows() * fnx::NQH * 16 * fnx::HD; }
int ref_attn_part_lanes(const float* qg, const uint16_t* kc, const uint16_t* vc, size_t page, int rows, const int* const* pos, const int* const* pt, int T,
                        float* scratch, int card, void* st) {
    return guarded([&] {
        fnx::KvPages g;
        g.pt = nullptr, g.page = page, g.rows = rows, g.q8 = 0;
        fnx::LaneRows lr;
        lr.pos = pos, lr.pt = pt;
        fnx::attn_part_lanes(qg, kc, vc, g, lr, T, scratch, st, nullptr, nullptr, card);
    });
}

int ref_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i, unsigned long long* keys, unsigned* err, void* st) {
    return guarded([&] { fnx::argmax(logits, rows, T, v0, best_v, best_i, keys, err, st); });
}

int ref_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n, int pen_stride, const float* pen_par,
                   float* out_v, int* out_i, unsigned* err, void* st) {
    // the reference's kernel reads the penalty arrays whatever their counts: null arrays are refused here
    if (!pen_tok || !pen_cnt || !pen_n || !pen_par) {
        snprintf(g_err, sizeof g_err, "ref_top_tokens: the reference's kernel needs its penalty arrays (counts may be zero)");
        return 1;
    }
    return guarded([&] { fnx::top_tokens(logits, n, T, v0, pen_tok, pen_cnt, pen_n, pen_stride, pen_par, out_v, out_i, err, st); });
}
}
