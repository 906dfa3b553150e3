/* CPU ORACLE - test infrastructure, not product code.
 *
 * Gated DeltaNet core of the verify window with per-row state checkpoints, restated from the reference's fused
 * kernel src/gdn_core.cuh:17-229 (simpler unfused statement: src/kernels.cu:361-445) with IEEE arithmetic, and the
 * rollback of src/engine_common.cu:525-568.  Products that the reference's compiler may fuse are written as explicit
 * fused steps: acc += a b is fma(a, b, acc); g s + k delta is fma(k, delta, g s); v - g kv is fma(-g, kv, v).
 */
#include "oracle.h"

#define HS 128

/* qkvz rows [q (nk HS) | k (nk HS) | v (nv HS) | z (nv HS)], ab rows [alpha (nv) | beta (nv)], hist [2][3][ch],
 * convw [ch][4], S [nv][HS key][HS value]; vmap[lv] = local key head | writes_hist << 8; ctl[1] & 1 = history parity.
 * Outputs: yq q8_1 rows of nv HS, y32 (optional), snap [T-1][nv][HS][HS], hsnap [T][3][ch] (variant n-1, n < T),
 * the other parity half of hist, S. */
void orc_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a,
                  const float* nw, float* S, uint8_t* yq, const int* ctl, float* snap, float* hsnap, int nk, int nv,
                  const int* vmap, int T, float eps, float* y32) {
    const int ch = (2 * nk + nv) * HS, row_stride = ch + nv * HS;
    const unsigned parity = ((const unsigned*) ctl)[1] & 1u;
    const float* hin = hist + (size_t) parity * 3 * ch;
    float* hout = hist + (size_t) (parity ^ 1u) * 3 * ch;
    float* conv = (float*) malloc((size_t) T * ch * sizeof(float));
    /* causal conv (width 4) + silu on every local channel; history out and the cut-back variants */
    for (int c = 0; c < ch; ++c) {
        float win[3 + 16];
        for (int k = 0; k < 3; ++k) win[k] = hin[(size_t) k * ch + c];
        for (int t = 0; t < T; ++t) win[3 + t] = qkvz[(size_t) t * row_stride + c];
        const float w0 = convw[c * 4], w1 = convw[c * 4 + 1], w2 = convw[c * 4 + 2], w3 = convw[c * 4 + 3];
        for (int t = 0; t < T; ++t) {
            float x = w0 * win[t];
            x = fmaf(w1, win[t + 1], x);
            x = fmaf(w2, win[t + 2], x);
            x = fmaf(w3, win[t + 3], x);
            conv[(size_t) t * ch + c] = o_silu(x);
        }
        for (int k = 0; k < 3; ++k) hout[(size_t) k * ch + c] = win[T + k];
        for (int n = 1; n < T; ++n)
            for (int k = 0; k < 3; ++k) hsnap[((size_t) (n - 1) * 3 + k) * ch + c] = win[n + k];
    }
    /* L2 norms of q and k per key head and row: warp (32 consecutive elements) xor-trees, the four added in order */
    for (int t = 0; t < T; ++t)
        for (int part = 0; part < 2; ++part)
            for (int kh = 0; kh < nk; ++kh) {
                float* x = conv + (size_t) t * ch + (size_t) part * nk * HS + (size_t) kh * HS;
                float sq = 0.f;
                for (int w = 0; w < 4; ++w) {
                    float v[32];
                    for (int l = 0; l < 32; ++l) v[l] = x[w * 32 + l] * x[w * 32 + l];
                    sq = sq + o_butterfly(v, 32);
                }
                const float r = o_rsqrt(sq + 1e-6f);
                for (int i = 0; i < HS; ++i) x[i] = x[i] * r;
            }
    const float scale = o_rsqrt((float) HS);
    float* o_all = (float*) malloc((size_t) T * nv * HS * sizeof(float));
#pragma omp parallel for
    for (int lv = 0; lv < nv; ++lv) {
        const int kh = vmap[lv] & 255;
        float* Sh = S + (size_t) lv * HS * HS;
        for (int t = 0; t < T; ++t) {
            const float* abt = ab + (size_t) t * 2 * nv;
            const float x = abt[lv] + dt[lv];
            const float sp = x > 20.0f ? x : o_log1pf_pos(o_expf(x));
            const float gv = o_expf(sp * a[lv]);
            const float bv = 1.0f / (1.0f + o_expf(-abt[nv + lv]));
            const float* q = conv + (size_t) t * ch + (size_t) kh * HS;
            const float* k = conv + (size_t) t * ch + (size_t) nk * HS + (size_t) kh * HS;
            const float* v = conv + (size_t) t * ch + (size_t) 2 * nk * HS + (size_t) lv * HS;
            for (int c = 0; c < HS; ++c) {
                float pk[4];
                for (int p = 0; p < 4; ++p) {
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int r = 0; r < 32; ++r) s4[r & 3] = fmaf(Sh[(size_t) (p * 32 + r) * HS + c], k[p * 32 + r], s4[r & 3]);
                    pk[p] = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                }
                const float kvd = (pk[0] + pk[1]) + (pk[2] + pk[3]);
                const float delta = fmaf(-gv, kvd, v[c]) * bv;
                float pa[4];
                for (int p = 0; p < 4; ++p) {
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int r = 0; r < 32; ++r) {
                        float* s = &Sh[(size_t) (p * 32 + r) * HS + c];
                        *s = fmaf(k[p * 32 + r], delta, gv * *s);
                        s4[r & 3] = fmaf(*s, q[p * 32 + r], s4[r & 3]);
                    }
                    pa[p] = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                }
                o_all[((size_t) t * nv + lv) * HS + c] = ((pa[0] + pa[1]) + (pa[2] + pa[3])) * scale;
            }
            if (t < T - 1) memcpy(snap + ((size_t) t * nv + lv) * HS * HS, Sh, sizeof(float) * HS * HS);
        }
        /* gated RMS norm over the head's HS outputs: per quarter of 32 columns, warps of 8 columns (xor-tree over the
         * warp with the other lanes zero), the four warps added in order; the four quarters added in order */
        for (int t = 0; t < T; ++t) {
            const float* o = o_all + ((size_t) t * nv + lv) * HS;
            float sq[4];
            for (int qq = 0; qq < 4; ++qq) {
                float tot = 0.f;
                for (int w = 0; w < 4; ++w) {
                    float lane[32];
                    for (int l = 0; l < 32; ++l) lane[l] = 0.f;
                    for (int j = 0; j < 8; ++j) {
                        const float ov = o[qq * 32 + w * 8 + j];
                        lane[4 * j] = ov * ov;
                    }
                    tot = tot + o_butterfly(lane, 32);
                }
                sq[qq] = tot;
            }
            const float ms = (((sq[0] + sq[1]) + sq[2]) + sq[3]) / (float) HS;
            const float rr = o_rsqrt(ms + eps);
            for (int b = 0; b < 4; ++b) {
                float xi[32], sv[32], amax = 0.f;
                for (int l = 0; l < 32; ++l) {
                    const int c = b * 32 + l;
                    const float z = qkvz[(size_t) t * row_stride + ch + (size_t) lv * HS + c];
                    xi[l] = o[c] * rr * nw[c] / (1.0f + o_expf(-z));
                    if (y32) y32[((size_t) t * nv + lv) * HS + c] = xi[l];
                    amax = fmaxf(amax, fabsf(xi[l]));
                    sv[l] = xi[l];
                }
                const float sm = o_butterfly(sv, 32), d = amax / 127.0f;
                uint8_t* p = yq + ((size_t) t * (nv * HS / 32) + (size_t) lv * 4 + b) * 36;
                const o_half hd = o_f2h(d), hs = o_f2h(sm);
                memcpy(p, &hd, 2);
                memcpy(p + 2, &hs, 2);
                for (int l = 0; l < 32; ++l) ((int8_t*) (p + 4))[l] = amax == 0.0f ? 0 : (int8_t) roundf(xi[l] / d);
            }
        }
    }
    free(conv);
    free(o_all);
}

/* keep the first n of a window's T rows: S <- snap[n-1], the history half the window wrote <- hsnap[n-1]
 * (reference src/engine_common.cu:525-568); n == T: nothing to do.  ctl[1] is the parity the window READ. */
void orc_gdn_rollback(float* S, float* hist, const float* snap, const float* hsnap, const int* ctl, int nk, int nv, int T,
                      int n) {
    if (n >= T) return;
    const int ch = (2 * nk + nv) * HS;
    const unsigned parity = ((const unsigned*) ctl)[1] & 1u;
    memcpy(S, snap + (size_t) (n - 1) * nv * HS * HS, sizeof(float) * (size_t) nv * HS * HS);
    memcpy(hist + (size_t) (parity ^ 1u) * 3 * ch, hsnap + (size_t) (n - 1) * 3 * ch, sizeof(float) * 3 * (size_t) ch);
}
