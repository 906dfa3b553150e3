/* CPU ORACLE - test infrastructure, not product code.
 *
 * Routed-expert FFN of the verify window, restated from the reference's kernels with IEEE arithmetic:
 *   router + top-k + jobs      reference src/moe.cuh:73-202 (host statement: tools/kbench.cu:59-96)
 *   Q4_K gate|up               reference src/moe_q4k.cuh:30-109, lane sum src/moe.cuh:224-235
 *   Q8_0 split GEMV            reference src/dense.cuh:55-153
 *   SwiGLU -> q8_1, down       reference src/moe.cuh:284-345 (32-column units, summed in ascending order)
 *   combine                    reference src/kernels.cu:797-803
 * The per-unit product of the down projection lives in an un-vendored dependency of the reference (ggml-cuda of
 * llama.cpp at a37cc46; call site src/moe.cuh:247), so its fp32 grouping is stated here by analogy with the Q4_K
 * gate|up arithmetic: PARITY UNPINNED for that grouping (exact integer sub-block dots, fp32 combine per unit).
 */
#include "oracle.h"

/* the four-term chunk product of the fp32 GEMVs: ((wx bx + wy by) + wz bz) + ww bw with each + a fused step */
static inline float dot4(const float* w, const float* b) {
    float t = w[0] * b[0];
    t = fmaf(w[1], b[1], t);
    t = fmaf(w[2], b[2], t);
    t = fmaf(w[3], b[3], t);
    return t;
}

/* y[t][row] = W[row] . x[t], `parts` warps per row each taking a contiguous share of the float4 chunks; lane l of a
 * warp takes chunks i*32 + l in ascending i; xor-tree over the lanes; the warps' sums added in ascending order.
 * parts = 2 with first = 1 is the router (half0 + half1, src/moe.cuh:119); parts = 4 with first = 0 is the block
 * GEMV (0 + p0 + p1 + p2 + p3, src/kernels.cu:222-226). n % (128 parts) == 0. */
void orc_gemv_f32(const float* W, const float* x, float* y, int rows, int n, int T, int parts, int y_stride) {
    const int nc = n / 4 / 32 / parts;
    for (int row = 0; row < rows; ++row)
        for (int t = 0; t < T; ++t) {
            float ps[8];
            for (int p = 0; p < parts; ++p) {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    float a = 0.f;
                    for (int i = 0; i < nc; ++i) {
                        const size_t c = ((size_t) p * nc * 32 + (size_t) i * 32 + l) * 4;
                        a = a + dot4(W + (size_t) row * n + c, x + (size_t) t * n + c);
                    }
                    lane[l] = a;
                }
                ps[p] = o_butterfly(lane, 32);
            }
            float v;
            if (parts == 2) v = ps[0] + ps[1];
            else {
                v = 0.f;
                for (int p = 0; p < parts; ++p) v = v + ps[p];
            }
            y[(size_t) t * y_stride + row] = v;
        }
}

/* logits [T][nexp + 1] (row nexp: the shared expert's gate), top-k by logit (ties: lower index), weights
 * exp(l - l_top) / sum in pick order, jobs per distinct expert numbered by first pick in pair order p = t k + k'. */
void orc_router_route(const float* W, const float* x, float* logits, int T, int n, int nexp, int topk, int* topi,
                      float* topw, OrcJob* gu, OrcJob* dn, int* njobs) {
    const int L = nexp + 1;
#pragma omp parallel for
    for (int row = 0; row < L; ++row) orc_gemv_f32(W + (size_t) row * n, x, logits + row, 1, n, T, 2, L);
    for (int t = 0; t < T; ++t) {
        const float* r = logits + (size_t) t * L;
        char* taken = (char*) calloc((size_t) nexp, 1);
        float top0 = 0.f, z = 0.f, ek[64];
        for (int k = 0; k < topk; ++k) {
            float bv = -INFINITY;
            int bi = nexp;
            for (int i = 0; i < nexp; ++i)
                if (!taken[i] && (r[i] > bv)) {
                    bv = r[i];
                    bi = i;
                }
            if (bi < nexp) taken[bi] = 1;
            if (k == 0) top0 = bv;
            ek[k] = o_expf(bv - top0);
            z = z + ek[k];
            topi[t * topk + k] = bi;
        }
        for (int k = 0; k < topk; ++k) topw[t * topk + k] = ek[k] / z;
        free(taken);
    }
    int nj = 0;
    for (int p = 0; p < T * topk; ++p) {
        int j = 0;
        while (j < nj && gu[j].w != topi[p]) ++j;
        if (j == nj) {
            memset(&gu[j], 0, sizeof(OrcJob));
            memset(&dn[j], 0, sizeof(OrcJob));
            gu[j].w = dn[j].w = topi[p];
            ++nj;
        }
        gu[j].y[gu[j].n] = p / topk;
        gu[j].out[gu[j].n] = dn[j].y[dn[j].n] = dn[j].out[dn[j].n] = p;
        ++gu[j].n;
        ++dn[j].n;
    }
    njobs[0] = nj;
    njobs[1] = 0;
}

static inline int dp4(const uint8_t* q, const int8_t* a, int n) { /* unsigned codes x signed activations */
    int s = 0;
    for (int i = 0; i < n; ++i) s += (int) q[i] * (int) a[i];
    return s;
}
static inline int dp4s(const int8_t* q, const int8_t* a, int n) {
    int s = 0;
    for (int i = 0; i < n; ++i) s += (int) q[i] * (int) a[i];
    return s;
}
static inline int isum(const int8_t* a, int n) {
    int s = 0;
    for (int i = 0; i < n; ++i) s += a[i];
    return s;
}

/* one Q4_K row (n columns) . one q8_1 row: 8 lanes, lane l owns the 64-value groups l, l + 8, ... in ascending
 * order; lanes combined by xor 4, 2, 1 */
static float q4k_row_dot(const uint8_t* wrow, const uint8_t* yrow, int n) {
    float lane[8];
    const int ngroups = n / 64;
    for (int l = 0; l < 8; ++l) {
        float tmp = 0.f;
        for (int g = l; g < ngroups; g += 8) {
            const int b = g >> 2, jg = g & 3;
            const uint8_t* blk = wrow + (size_t) b * 144;
            o_half hd, hm;
            memcpy(&hd, blk, 2);
            memcpy(&hm, blk + 2, 2);
            const float d = o_h2f(hd), dmin = o_h2f(hm);
            int sc0, m0, sc1, m1;
            orc_q4k_scale_min(blk + 4, 2 * jg, &sc0, &m0);
            orc_q4k_scale_min(blk + 4, 2 * jg + 1, &sc1, &m1);
            const uint8_t* qs = blk + 16 + 32 * jg;
            const uint8_t* y0 = yrow + (size_t) (b * 8 + jg * 2) * 36;
            const uint8_t* y1 = y0 + 36;
            const int8_t* a0 = (const int8_t*) (y0 + 4);
            const int8_t* a1 = (const int8_t*) (y1 + 4);
            int dl = 0, dh = 0;
            for (int i = 0; i < 32; ++i) {
                dl += (int) (qs[i] & 0xF) * (int) a0[i];
                dh += (int) (qs[i] >> 4) * (int) a1[i];
            }
            const int sl = isum(a0, 32), sh = isum(a1, 32);
            o_half h0, h1;
            memcpy(&h0, y0, 2);
            memcpy(&h1, y1, 2);
            const float d8l = o_h2f(h0), d8h = o_h2f(h1);
            const float pos = d * (d8l * ((float) sc0 * (float) dl) + d8h * ((float) sc1 * (float) dh));
            const float neg = dmin * (d8l * ((float) m0 * (float) sl) + d8h * ((float) m1 * (float) sh));
            tmp = tmp + (pos - neg);
        }
        lane[l] = tmp;
    }
    return o_butterfly(lane, 8);
}

/* gate|up over Q4_K experts: A = experts of [2 ffs][n] Q4_K rows, expert stride sa bytes; gu[out][2 ffs] */
void orc_moe_gate_up_q4k(const uint8_t* A, size_t sa, const OrcJob* jobs, int njobs, const uint8_t* xq, float* gu, int n,
                         int nrows) {
    const size_t row_b = (size_t) n / 256 * 144, yb = (size_t) n / 32 * 36;
#pragma omp parallel for schedule(dynamic)
    for (int j = 0; j < njobs; ++j)
        for (int r = 0; r < nrows; ++r)
            for (int s = 0; s < jobs[j].n; ++s)
                gu[(size_t) jobs[j].out[s] * nrows + r] =
                    q4k_row_dot(A + (size_t) jobs[j].w * sa + (size_t) r * row_b, xq + (size_t) jobs[j].y[s] * yb, n);
}

/* one split-Q8_0 row . one activation row given as an int8 plane a[cols] and per-block scales da[cols/32]:
 * lane l takes 16 columns at c = 16 l + 512 k (k ascending), acc = fma(dw da, (float) isum16, acc); xor tree 16..1 */
float orc_q8s_row_dot(const int8_t* wq, const o_half* wd, const int8_t* a, const float* da, int cols) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        for (int c = l * 16; c < cols; c += 512) {
            const int b = c >> 5;
            const int s = dp4s(wq + c, a + c, 16);
            acc = fmaf(o_h2f(wd[b]) * da[b], (float) s, acc);
        }
        lane[l] = acc;
    }
    return o_butterfly(lane, 32);
}

/* q8_1 rows -> int8 plane + float scales of the f16-rounded d (the reference's "twin", src/kernels.cu:109-112) */
void orc_q8_1_unpack(const uint8_t* yq, int cols, int rows, int8_t* a, float* da) {
    const int nb = cols / 32;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const uint8_t* p = yq + ((size_t) r * nb + b) * 36;
            o_half hd;
            memcpy(&hd, p, 2);
            da[(size_t) r * nb + b] = o_h2f(hd);
            memcpy(a + (size_t) r * cols + b * 32, p + 4, 32);
        }
}

/* out[t][r] = W[r] . y[t]: split Q8_0 [rows][cols] x q8_1 rows */
void orc_q8s_gemv(const int8_t* wq, const o_half* wd, int rows, int cols, const uint8_t* yq, float* out, int out_stride,
                  int T) {
    int8_t* a = (int8_t*) malloc((size_t) T * cols);
    float* da = (float*) malloc((size_t) T * (cols / 32) * 4);
    orc_q8_1_unpack(yq, cols, T, a, da);
#pragma omp parallel for
    for (int r = 0; r < rows; ++r)
        for (int t = 0; t < T; ++t)
            out[(size_t) t * out_stride + r] = orc_q8s_row_dot(wq + (size_t) r * cols, wd + (size_t) r * (cols / 32),
                                                              a + (size_t) t * cols, da + (size_t) t * (cols / 32), cols);
    free(a);
    free(da);
}

/* The same product with its sums in block order: acc = fma(fl(dw_b da_b), (float) isum_b, acc) for the 32-column blocks b in
 * ascending order, isum_b the block's exact integer dot.  This is NOT the reference's order of sums (its kernel adds
 * half-block terms on 32 interleaved lanes and a tree, orc_q8s_row_dot above); it is the order of this library's tensor-core
 * dense kernel (fnx_q8s_gemv_blocks), stated here so that the kernel can be checked bit for bit; against the reference's
 * order the two agree to fp32 rounding of the sum. */
void orc_q8s_gemv_blocks(const int8_t* wq, const o_half* wd, int rows, int cols, const uint8_t* yq, float* out, int out_stride, int T) {
    int8_t* a = (int8_t*) malloc((size_t) T * cols);
    float* da = (float*) malloc((size_t) T * (cols / 32) * 4);
    orc_q8_1_unpack(yq, cols, T, a, da);
    const int nb = cols / 32;
#pragma omp parallel for
    for (int r = 0; r < rows; ++r)
        for (int t = 0; t < T; ++t) {
            float acc = 0.f;
            for (int b = 0; b < nb; ++b) {
                int isum = 0;
                for (int l = 0; l < 32; ++l) isum += (int) wq[(size_t) r * cols + b * 32 + l] * (int) a[(size_t) t * cols + b * 32 + l];
                acc = fmaf(o_h2f(wd[(size_t) r * nb + b]) * da[(size_t) t * nb + b], (float) isum, acc);
            }
            out[(size_t) t * out_stride + r] = acc;
        }
    free(a);
    free(da);
}

/* gate|up over split-Q8_0 experts (expert e: planes at wq + e sq, wd + e sd): the dense row dot per (job row, pair) */
void orc_moe_gate_up_q8(const int8_t* wq, size_t sq, const o_half* wd, size_t sd, const OrcJob* jobs, int njobs,
                        const uint8_t* xq, int T, float* gu, int n, int nrows) {
    int8_t* a = (int8_t*) malloc((size_t) T * n);
    float* da = (float*) malloc((size_t) T * (n / 32) * 4);
    orc_q8_1_unpack(xq, n, T, a, da);
#pragma omp parallel for schedule(dynamic)
    for (int j = 0; j < njobs; ++j)
        for (int r = 0; r < nrows; ++r)
            for (int s = 0; s < jobs[j].n; ++s) {
                const int t = jobs[j].y[s];
                gu[(size_t) jobs[j].out[s] * nrows + r] =
                    orc_q8s_row_dot(wq + (size_t) jobs[j].w * sq + (size_t) r * n, wd + (size_t) jobs[j].w * sd + (size_t) r * (n / 32),
                                    a + (size_t) t * n, da + (size_t) t * (n / 32), n);
            }
    free(a);
    free(da);
}

/* h = silu(gate) * up of a gu row [gate (ffs) | up (ffs)] as an int8 plane + f16-rounded scales (q8_1 rounding) */
void orc_swiglu_q8(const float* gu_row, int ffs, int8_t* hq, float* hd) {
    for (int b = 0; b < ffs / 32; ++b) {
        float xi[32], amax = 0.f;
        for (int l = 0; l < 32; ++l) {
            xi[l] = o_silu(gu_row[b * 32 + l]) * gu_row[ffs + b * 32 + l];
            amax = fmaxf(amax, fabsf(xi[l]));
        }
        const float d = amax / 127.0f;
        for (int l = 0; l < 32; ++l) hq[b * 32 + l] = amax == 0.0f ? 0 : (int8_t) roundf(xi[l] / d);
        hd[b] = o_h2f(o_f2h(d));
    }
}

/* down over Q6_K planes (orc_q6k_to_planes of expert e at QL + e sQL, ...): part[out][row] = sum over the 32-column
 * units u ascending of d_u * (d8_u * (float) (sc0 isum0 + sc1 isum1)), isum over (code - 32) * h */
void orc_moe_down_q6p(const uint8_t* QL, const uint8_t* QH, const int8_t* SC, const o_half* D, size_t expert_units,
                      const OrcJob* jobs, int njobs, const float* gu, float* part, int nrows, int ffs) {
    const int nu = ffs / 32;
#pragma omp parallel for schedule(dynamic)
    for (int j = 0; j < njobs; ++j) {
        int8_t* hq = (int8_t*) malloc((size_t) ffs);
        float* hd = (float*) malloc((size_t) nu * 4);
        for (int s = 0; s < jobs[j].n; ++s) {
            orc_swiglu_q8(gu + (size_t) jobs[j].y[s] * 2 * ffs, ffs, hq, hd);
            for (int r = 0; r < nrows; ++r) {
                float acc = 0.f;
                for (int u = 0; u < nu; ++u) {
                    const size_t at = (size_t) jobs[j].w * expert_units + (size_t) r * nu + u;
                    int is0 = 0, is1 = 0;
                    for (int i = 0; i < 32; ++i) {
                        const int q = orc_q6p_q(QL + at * 16, QH + at * 8, i) - 32;
                        if (i < 16) is0 += q * hq[u * 32 + i];
                        else is1 += q * hq[u * 32 + i];
                    }
                    const int I = (int) SC[at * 2] * is0 + (int) SC[at * 2 + 1] * is1;
                    acc = acc + o_h2f(D[at]) * (hd[u] * (float) I);
                }
                part[(size_t) jobs[j].out[s] * nrows + r] = acc;
            }
        }
        free(hq);
        free(hd);
    }
}

/* down over split-Q8_0 experts: units of 32 columns, (dw d8) * (float) isum, summed in ascending order */
void orc_moe_down_q8(const int8_t* wq, size_t sq, const o_half* wd, size_t sd, const OrcJob* jobs, int njobs,
                     const float* gu, float* part, int nrows, int ffs) {
    const int nu = ffs / 32;
#pragma omp parallel for schedule(dynamic)
    for (int j = 0; j < njobs; ++j) {
        int8_t* hq = (int8_t*) malloc((size_t) ffs);
        float* hd = (float*) malloc((size_t) nu * 4);
        for (int s = 0; s < jobs[j].n; ++s) {
            orc_swiglu_q8(gu + (size_t) jobs[j].y[s] * 2 * ffs, ffs, hq, hd);
            for (int r = 0; r < nrows; ++r) {
                const int8_t* w = wq + (size_t) jobs[j].w * sq + (size_t) r * ffs;
                const o_half* d = wd + (size_t) jobs[j].w * sd + (size_t) r * nu;
                float acc = 0.f;
                for (int u = 0; u < nu; ++u) acc = acc + (o_h2f(d[u]) * hd[u]) * (float) dp4s(w + u * 32, hq + u * 32, 32);
                part[(size_t) jobs[j].out[s] * nrows + r] = acc;
            }
        }
        free(hq);
        free(hd);
    }
}

/* shared expert: Q8_0 gate|up over the q8_1 rows, SwiGLU -> int8, Q8_0 down, all in the dense row-dot order
 * (reference src/dense.cuh:162-198); out[t][n] */
void orc_shared_expert(const int8_t* guq, const o_half* gud, const int8_t* dnq, const o_half* dnd, const uint8_t* xq, int T,
                       int n, int ffs, float* sh_gu, float* out) {
    orc_q8s_gemv(guq, gud, 2 * ffs, n, xq, sh_gu, 2 * ffs, T);
    int8_t* hq = (int8_t*) malloc((size_t) T * ffs);
    float* hd = (float*) malloc((size_t) T * (ffs / 32) * 4);
    for (int t = 0; t < T; ++t) orc_swiglu_q8(sh_gu + (size_t) t * 2 * ffs, ffs, hq + (size_t) t * ffs, hd + (size_t) t * (ffs / 32));
#pragma omp parallel for
    for (int r = 0; r < n; ++r)
        for (int t = 0; t < T; ++t)
            out[(size_t) t * n + r] = orc_q8s_row_dot(dnq + (size_t) r * ffs, dnd + (size_t) r * (ffs / 32), hq + (size_t) t * ffs,
                                                      hd + (size_t) t * (ffs / 32), ffs);
    free(hq);
    free(hd);
}

/* out[t][i] = sum_k fma(topw[t][k], part[t topk + k][i], .) then fma(sigmoid(sh_logit[t]), sh[t][i], .) */
void orc_moe_combine(const float* part, const float* topw, const float* sh, const float* logits, int logit_stride,
                     int sh_col, float* out, int T, int n, int topk) {
    for (int t = 0; t < T; ++t) {
        const float g = o_sigmoid(logits[(size_t) t * logit_stride + sh_col]);
        for (int i = 0; i < n; ++i) {
            float s = 0.f;
            for (int k = 0; k < topk; ++k) s = fmaf(topw[t * topk + k], part[((size_t) t * topk + k) * n + i], s);
            out[(size_t) t * n + i] = fmaf(g, sh[(size_t) t * n + i], s);
        }
    }
}

/* y[r] = x[r] * (1 / sqrt(mean(x[r]^2) + eps)) * w (reference src/kernels.cu:2199-2206): 1024 threads, thread i sums
 * x[i], x[i + 1024], ... squares in order; warp xor-trees; the 32 warp sums added in ascending order */
void orc_rms_norm_rows(const float* x, const float* w, float* y, int rows, int n, float eps) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t) r * n;
        float tsum[1024];
        for (int i = 0; i < 1024; ++i) {
            float s = 0.f;
            for (int c = i; c < n; c += 1024) s = fmaf(xr[c], xr[c], s);
            tsum[i] = s;
        }
        float tot = 0.f;
        for (int wp = 0; wp < 32; ++wp) tot = tot + o_butterfly(tsum + wp * 32, 32);
        const float rr = o_rsqrt(tot / (float) n + eps);
        for (int c = 0; c < n; ++c) y[(size_t) r * n + c] = xr[c] * rr * w[c];
    }
}
