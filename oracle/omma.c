/* CPU ORACLE - test infrastructure, not product code.
 *
 * The routed experts over many rows as the reference's prompt path computes them (reference src/moe_mma.cuh): every
 * weight dequantised to f16 with ONE rounding, activations f16, products summed in fp32 on the tensor cores.  The order
 * of a sum's terms inside the tensor cores is not stated anywhere, so this file states the f16 weights bit for bit
 * (orc_mma_weights_*) and the sums in double (every product of two f16 values is exact in double); a GPU result is
 * compared with them to a bound on fp32 summation error that the tests state.
 *
 *  Q4_K (reference src/moe_mma.cuh:56-60, 79-113): ds = f16(d * sc), nm = f16(-(dmin * m)), w = f16(q * ds + nm) as one
 *        fused step (__hfma2: a single rounding);
 *  Q8_0 (reference src/moe_mma.cuh:184-216): w = f16(q * d) (__hmul2);
 *  Q6_K in 32-column units: not a type of the reference's prompt path; by the same rule ds = f16(d * sc),
 *        w = f16((q - 32) * ds).
 *  h16 (reference src/moe_mma.cuh:381-388): f16(silu(g) * u).
 */
#include <stdlib.h>

#include "omath.h"
#include "oracle.h"

/* double -> f16 with one rounding to nearest even: through a float made odd when inexact, so that the second rounding
 * cannot land on a tie it did not start from (a float has more than 2 * 11 + 2 bits) */
static o_half d2h(double x) {
    float f = (float) x;
    if ((double) f != x) {
        uint32_t b = o_fbits(f);
        if (fabs((double) f) > fabs(x)) b -= 1; /* one step towards zero: the truncated value */
        b |= 1u;
        f = o_bitsf(b);
    }
    return o_f2h(f);
}

o_half orc_d2h(double x) { return d2h(x); }

/* the f16 weights of `rows` Q4_K rows of n columns */
void orc_mma_weights_q4k(const uint8_t* A, int rows, int n, o_half* w) {
    const int nb = n / 256;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const uint8_t* blk = A + ((size_t) r * nb + b) * 144;
            o_half hd, hm;
            memcpy(&hd, blk, 2);
            memcpy(&hm, blk + 2, 2);
            const float d = o_h2f(hd), dmin = o_h2f(hm);
            for (int s = 0; s < 8; ++s) {
                int sc, m;
                orc_q4k_scale_min(blk + 4, s, &sc, &m);
                const o_half ds = o_f2h(d * (float) sc), nm = o_f2h(-(dmin * (float) m));
                for (int l = 0; l < 32; ++l) {
                    const uint8_t byte = blk[16 + 32 * (s / 2) + l];
                    const int q = s & 1 ? byte >> 4 : byte & 15;
                    w[(size_t) r * n + b * 256 + s * 32 + l] = d2h((double) q * (double) o_h2f(ds) + (double) o_h2f(nm));
                }
            }
        }
}

void orc_mma_weights_q8(const int8_t* wq, const o_half* wd, int rows, int n, o_half* w) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < n; ++c) w[(size_t) r * n + c] = o_f2h((float) wq[(size_t) r * n + c] * o_h2f(wd[(size_t) r * (n / 32) + c / 32]));
}

void orc_mma_weights_q6p(const uint8_t* QL, const uint8_t* QH, const int8_t* SC, const o_half* D, int rows, int n, o_half* w) {
    const int nu = n / 32;
    for (int r = 0; r < rows; ++r)
        for (int u = 0; u < nu; ++u) {
            const size_t at = (size_t) r * nu + u;
            const float d = o_h2f(D[at]);
            const o_half ds[2] = {o_f2h(d * (float) SC[at * 2]), o_f2h(d * (float) SC[at * 2 + 1])};
            for (int i = 0; i < 32; ++i) {
                const int q = orc_q6p_q(QL + at * 16, QH + at * 8, i) - 32;
                w[(size_t) r * n + u * 32 + i] = o_f2h((float) q * o_h2f(ds[i / 16]));
            }
        }
}

/* out[jobs[j].out[s]][r] = sum_k w[jobs[j].w][r][k] x[jobs[j].y[s]][k] in double; mag the same sum over |products| (what
 * the error bound of an fp32 summation in another order scales with).  w: [experts][nrows][n] f16 */
void orc_moe_mma(const o_half* w, const OrcBigJob* jobs, int njobs, const o_half* x, int nrows, int n, double* out, double* mag) {
#pragma omp parallel for schedule(dynamic)
    for (int j = 0; j < njobs; ++j) {
        float* xf = (float*) malloc((size_t) n * 4);
        for (int s = 0; s < jobs[j].n; ++s) {
            for (int k = 0; k < n; ++k) xf[k] = o_h2f(x[(size_t) jobs[j].y[s] * n + k]);
            for (int r = 0; r < nrows; ++r) {
                const o_half* wr = w + ((size_t) jobs[j].w * nrows + r) * n;
                double acc = 0.0, m = 0.0;
                for (int k = 0; k < n; ++k) {
                    const double p = (double) o_h2f(wr[k]) * (double) xf[k];
                    acc += p;
                    m += fabs(p);
                }
                out[(size_t) jobs[j].out[s] * nrows + r] = acc;
                mag[(size_t) jobs[j].out[s] * nrows + r] = m;
            }
        }
        free(xf);
    }
}

void orc_swiglu_h16(const float* gu, int ffs, int P, o_half* h) {
    for (int p = 0; p < P; ++p)
        for (int i = 0; i < ffs; ++i) h[(size_t) p * ffs + i] = o_f2h(o_silu(gu[(size_t) p * 2 * ffs + i]) * gu[(size_t) p * 2 * ffs + ffs + i]);
}
