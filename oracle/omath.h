/* CPU ORACLE - test infrastructure, not product code.
 *
 * Exact scalar math of the verify-window oracle.  Every function here is built only from IEEE-754 single (or
 * double) +, *, /, sqrt and fused multiply-add in a fixed order, so that the CUDA kernels, which restate the same
 * sequences with the round-to-nearest intrinsics, can be compared with this file bit for bit.  The reference's
 * kernels use __expf / rsqrtf / sincosf under --use_fast_math (reference Makefile:67), whose bits no CPU can
 * reproduce; the functions below are the IEEE statements of the same quantities.
 *
 * Build with -ffp-contract=off (the only fused operations are the explicit fmaf / fma calls) and -mfma -mf16c.
 */
#ifndef ORACLE_OMATH_H
#define ORACLE_OMATH_H

#include <math.h>
#include <stdint.h>
#include <string.h>

typedef uint16_t o_half; /* IEEE binary16 bit pattern */

static inline float o_h2f(o_half h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float) v;
}
static inline o_half o_f2h(float f) { /* round to nearest even, as __float2half_rn */
    _Float16 v = (_Float16) f;
    o_half h;
    memcpy(&h, &v, 2);
    return h;
}
static inline uint32_t o_fbits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
static inline float o_bitsf(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* e^x.  k = rint(x log2 e), r = x - k ln2 in two fused steps, degree-5 polynomial in r on r^2, scaled by 2^k through
 * the exponent field.  Outside [-86, 88] the result is 0 or +inf (no subnormal results). */
static inline float o_expf(float x) {
    if (x > 88.0f) return INFINITY;
    if (x < -86.0f) return 0.0f;
    const float k = rintf(x * 1.44269504f);
    float r = fmaf(k, -0.693145752f, x);
    r = fmaf(k, -1.42860677e-06f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = r * r;
    float e = fmaf(p, r2, r);
    e = e + 1.0f;
    return o_bitsf(o_fbits(e) + ((uint32_t) (int32_t) k << 23));
}

/* ln(u) for finite u >= 1: u = m 2^e with m in [sqrt(1/2), sqrt 2), ln m = 2 atanh(s), s = (m-1)/(m+1). */
static inline float o_logf_ge1(float u) {
    uint32_t b = o_fbits(u);
    int e = (int) (b >> 23) - 127;
    b = (b & 0x007fffffu) | 0x3f800000u;
    float m = o_bitsf(b);
    if (m > 1.41421354f) {
        m = m * 0.5f;
        e += 1;
    }
    const float f = m - 1.0f;
    const float s = f / (2.0f + f);
    const float z = s * s;
    float R = 0.24279078841f;
    R = fmaf(R, z, 0.28498786688f);
    R = fmaf(R, z, 0.40000972152f);
    R = fmaf(R, z, 0.66666662693f);
    const float lm = fmaf(s * z, R, 2.0f * s);
    const float fe = (float) e;
    return fmaf(fe, 0.693145752f, fmaf(fe, 1.42860677e-06f, lm));
}

/* ln(1 + y) for y >= 0 (the softplus of the DeltaNet decay gate): ln(u) y / (u - 1), u = fl(1 + y). */
static inline float o_log1pf_pos(float y) {
    const float u = 1.0f + y;
    if (u == 1.0f) return y;
    if (isinf(u)) return u;
    return o_logf_ge1(u) * (y / (u - 1.0f));
}

static inline float o_sigmoid(float x) { return 1.0f / (1.0f + o_expf(-x)); }
static inline float o_silu(float x) { return x / (1.0f + o_expf(-x)); }
static inline float o_rsqrt(float x) { return 1.0f / sqrtf(x); }

/* sin and cos of a double angle theta >= 0 (rotary position x frequency, up to ~1e6), rounded to float.
 * Cody-Waite reduction by pi/2 in two fused steps, then the standard minimax kernels on [-pi/4, pi/4]. */
static inline void o_sincos(double theta, float* sn, float* cs) {
    const double k = rint(theta * 0.63661977236758134308);
    double r = fma(-k, 1.57079632673412561417e+00, theta);
    r = fma(-k, 6.07710050650619224932e-11, r);
    const double z = r * r;
    double ps = 1.58969099521155010221e-10;
    ps = fma(ps, z, -2.50507602534068634195e-08);
    ps = fma(ps, z, 2.75573137070700676789e-06);
    ps = fma(ps, z, -1.98412698298579493134e-04);
    ps = fma(ps, z, 8.33333333332248946124e-03);
    ps = fma(ps, z, -1.66666666666666324348e-01);
    const double s = fma(r * z, ps, r);
    double pc = -1.13596475577881948265e-11;
    pc = fma(pc, z, 2.08757232129817482790e-09);
    pc = fma(pc, z, -2.75573143513906633035e-07);
    pc = fma(pc, z, 2.48015872894767294178e-05);
    pc = fma(pc, z, -1.38888888888741095749e-03);
    pc = fma(pc, z, 4.16666666666666019037e-02);
    const double c = fma(z * z, pc, fma(z, -0.5, 1.0));
    const int q = (int) ((long long) k & 3);
    const double so = q == 0 ? s : q == 1 ? c : q == 2 ? -s : -c;
    const double co = q == 0 ? c : q == 1 ? -s : q == 2 ? -c : s;
    *sn = (float) so;
    *cs = (float) co;
}

/* monotone key of a float: a larger float has a larger key (reference src/kernels.cu:872-875) */
static inline uint32_t o_fkey(float v) {
    const uint32_t u = o_fbits(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/* xor-butterfly sum of 2^k lane values as lane 0 ends up holding it (reference wsum, src/kernels.cu:36-40):
 * offsets n/2, n/4, ..., 1.  v is overwritten. */
static inline float o_butterfly(float* v, int n) {
    for (int o = n / 2; o; o >>= 1)
        for (int l = 0; l < o; ++l) v[l] = v[l] + v[l + o];
    return v[0];
}

#endif
