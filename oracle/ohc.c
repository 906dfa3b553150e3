/* CPU ORACLE - test infrastructure, not product code.
 *
 * Hyper-connections of the residual streams, restated with IEEE arithmetic from the reference:
 *   the write  R += bo * 2 sigmoid(inj / HC)                       src/kernels.cu:1493-1503 (k_hc_write)
 *   the read   (build_hc_mix) with the write folded in              src/hc.cuh:54-57 (rprime), :130-380 (k_hc)
 * The reference runs the read as one launch with two grid barriers; what is restated here is its arithmetic: which
 * values are rounded where, and the order of every sum.
 *   slices of 512 columns of the HC * n wide row (a slice lies inside one stream);
 *   xs = R' * w_norm, quantised per 32 as int8 with a float scale amax / 127 (not rounded to f16), src/hc.cuh:62-67;
 *   a slice's square sum of R': warp xor-trees over 32 columns, the 16 warps added in ascending order;
 *   down (Q8_0 rows x int8 xs): 8 lanes a row, lane j the 8-column chunks j, j + 8, ..., each
 *     acc = fma(f16 scale * xd, (float) integer dot, acc), lanes joined by an xor-tree with rising offsets (1, 2, 4);
 *   inject rows (bf16 weights on xs itself): per chunk t = b0 x0, t = fma(b_i, x_i, t), acc = acc + t (the reference's
 *     eight-term sum may be contracted by its compiler; this is the form both sides of this build use);
 *   rs = 1 / sqrt(sum of the stream's slice sums / n + eps), slices added in ascending order;
 *   lo = silu(sum_c fma(rs_c, p_c, .) / HC), p_c the stream's slices' partials added in ascending order, as int8 per 32;
 *   up (Q8_0 rows [HC n][lr] x int8 lo): 16 lanes a column, lane b < lr / 32 the block b, (scale * d_lo) * (float) dot,
 *     xor-tree (1, 2, 4, 8) with the idle lanes' zeros;
 *   mixed = (g_0 + g_1 + g_2 + g_3) / HC with g_c = sigmoid(up_c) * ((R' * w_norm) * rs_c); mixed also as q8_1.
 *
 * Parity unpinned: the reference's tests hold no vectors for the read (it is exercised only through whole-model logits) and
 * its kernel was not run against this file; what pins it is the float64 restatement (tests/test_oracle_path.py).
 */
#include "oracle.h"

#define HSL 512

static float bf2f(uint16_t h) { return o_bitsf((uint32_t) h << 16); }

/* the xor-tree with rising offsets (1, 2, 4, ...) as every lane ends up holding it: neighbours first */
static float tree_up(float* v, int n) {
    for (int o = 1; o < n; o <<= 1)
        for (int l = 0; l < n; l += 2 * o) v[l] = v[l] + v[l + o];
    return v[0];
}

void orc_hc_write(float* R, const float* bo, const float* inj, int T, int n, int hc) {
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < hc; ++c) {
            const float g = (1.0f + o_expf(-inj[t * hc + c] / (float) hc));
            for (int i = 0; i < n; ++i) {
                float* r = R + ((size_t) t * hc + c) * n + i;
                *r = *r + bo[(size_t) t * n + i] * 2.0f / g;
            }
        }
}

static float rprime(const float* R, const float* bo, const float* inj_prev, int t, int c, int i, int n, int hc) {
    float r = R[((size_t) t * hc + c) * n + i];
    if (bo) r = fmaf(bo[(size_t) t * n + i], 2.0f * o_sigmoid(inj_prev[t * hc + c] / (float) hc), r);
    return r;
}

/* q8: NULL or [T][n / 32][36] */
void orc_hc_read(float* R, const float* bo_prev, const float* inj_prev, const float* w_norm, const int8_t* down_q, const o_half* down_d,
                 const int8_t* up_q, const o_half* up_d, const uint16_t* w_inj, float eps, float* mixed, float* inject, uint8_t* q8, int T,
                 int n, int hc, int lr) {
    const int D = n * hc, ns = D / HSL, sps = n / HSL, rows = lr + hc;
    float* part = (float*) calloc((size_t) ns * T * rows, sizeof(float));
    float* ssp = (float*) calloc((size_t) T * ns, sizeof(float));
    float* rp = (float*) calloc((size_t) T * D, sizeof(float));
    int8_t* loq = (int8_t*) calloc((size_t) T * lr, 1);
    float* lod = (float*) calloc((size_t) T * (lr / 32), sizeof(float));
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < hc; ++c)
            for (int i = 0; i < n; ++i) rp[(size_t) t * D + c * n + i] = rprime(R, bo_prev, inj_prev, t, c, i, n, hc);
    /* ---- down, a slice at a time */
#pragma omp parallel for
    for (int s = 0; s < ns; ++s) {
        const int col0 = s * HSL;
        float xs[HSL], xd[HSL / 32];
        int8_t xq[HSL];
        for (int k = 0; k < T; ++k) {
            float v = 0.f;
            for (int w = 0; w < HSL / 32; ++w) {
                float sq[32];
                for (int l = 0; l < 32; ++l) {
                    const float r = rp[(size_t) k * D + col0 + w * 32 + l];
                    sq[l] = r * r;
                    xs[w * 32 + l] = r * w_norm[col0 + w * 32 + l];
                }
                v = v + o_butterfly(sq, 32);
            }
            ssp[(size_t) k * ns + s] = v;
            for (int b = 0; b < HSL / 32; ++b) {
                float amax = 0.f;
                for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(xs[b * 32 + l]));
                const float sc = amax / 127.0f;
                for (int l = 0; l < 32; ++l) xq[b * 32 + l] = amax == 0.0f ? 0 : (int8_t) roundf(xs[b * 32 + l] / sc);
                xd[b] = sc;
            }
            for (int row = 0; row < (w_inj ? rows : lr); ++row) {
                float lanes[8];
                for (int j = 0; j < 8; ++j) {
                    float acc = 0.f;
                    for (int q = 0; q < HSL / 64; ++q) {
                        const int ch = q * 8 + j;   /* 8-column chunk of the slice */
                        if (row < lr) {
                            const int8_t* w = down_q + (size_t) row * D + col0 + ch * 8;
                            const float sc = o_h2f(down_d[((size_t) row * D + col0) / 32 + ch / 4]);
                            int dot = 0;
                            for (int e = 0; e < 8; ++e) dot += (int) w[e] * (int) xq[ch * 8 + e];
                            acc = fmaf(sc * xd[ch / 4], (float) dot, acc);
                        } else {
                            const uint16_t* w = w_inj + (size_t) (row - lr) * D + col0 + ch * 8;
                            float t8 = bf2f(w[0]) * xs[ch * 8];
                            for (int e = 1; e < 8; ++e) t8 = fmaf(bf2f(w[e]), xs[ch * 8 + e], t8);
                            acc = acc + t8;
                        }
                    }
                    lanes[j] = acc;
                }
                part[((size_t) s * T + k) * rows + row] = tree_up(lanes, 8);
            }
        }
    }
    /* ---- reduce */
    float* rs = (float*) calloc((size_t) T * hc, sizeof(float));
    for (int k = 0; k < T; ++k)
        for (int c = 0; c < hc; ++c) {
            float v = 0.f;
            for (int ss = 0; ss < sps; ++ss) v = v + ssp[(size_t) k * ns + c * sps + ss];
            rs[k * hc + c] = o_rsqrt(v / (float) n + eps);
        }
    for (int k = 0; k < T; ++k) {
        float pre[1024];   /* the row's lo before the activation (lr <= 1024) */
        for (int r = 0; r < (w_inj ? rows : lr); ++r) {
            float sum = 0.f;
            for (int c = 0; c < hc; ++c) {
                float p = 0.f;
                for (int ss = 0; ss < sps; ++ss) p = p + part[((size_t) (c * sps + ss) * T + k) * rows + r];
                sum = fmaf(rs[k * hc + c], p, sum);
            }
            if (r >= lr) inject[k * hc + (r - lr)] = sum;
            else pre[r] = sum;
        }
        for (int b = 0; b < lr / 32; ++b) {
            float v[32], amax = 0.f;
            for (int l = 0; l < 32; ++l) {
                v[l] = o_silu(pre[b * 32 + l] / (float) hc);
                amax = fmaxf(amax, fabsf(v[l]));
            }
            const float sc = amax / 127.0f;
            for (int l = 0; l < 32; ++l) loq[(size_t) k * lr + b * 32 + l] = amax == 0.0f ? 0 : (int8_t) roundf(v[l] / sc);
            lod[k * (lr / 32) + b] = sc;
        }
    }
    /* ---- up */
#pragma omp parallel for
    for (int dc = 0; dc < n; ++dc)
        for (int k = 0; k < T; ++k) {
            float gs[16] = {0};
            for (int c = 0; c < hc; ++c) {
                const size_t urow = (size_t) c * n + dc;
                float lanes[16];
                for (int uj = 0; uj < 16; ++uj) {
                    if (uj >= lr / 32) {
                        lanes[uj] = 0.f;
                        continue;
                    }
                    int dot = 0;
                    for (int e = 0; e < 32; ++e) dot += (int) up_q[urow * lr + uj * 32 + e] * (int) loq[(size_t) k * lr + uj * 32 + e];
                    lanes[uj] = o_h2f(up_d[urow * (lr / 32) + uj]) * lod[k * (lr / 32) + uj] * (float) dot;
                }
                const float g = tree_up(lanes, 16);
                const float rv = rp[(size_t) k * D + c * n + dc];
                gs[c] = o_sigmoid(g) * (rv * w_norm[c * n + dc] * rs[k * hc + c]);
            }
            float sum = gs[0];
            for (int c = 1; c < hc; ++c) sum = sum + gs[c];
            mixed[(size_t) k * n + dc] = sum / (float) hc;
        }
    if (bo_prev) memcpy(R, rp, (size_t) T * D * sizeof(float));
    if (q8) orc_quantize_q8_1(mixed, q8, n, T);
    free(part), free(ssp), free(rp), free(loq), free(lod), free(rs);
}
