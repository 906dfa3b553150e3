// Exact scalar math for the verify-window kernels.  Every function is a fixed sequence of IEEE-754 round-to-nearest
// operations (the _rn intrinsics are never contracted or reordered by the compiler), so results do not depend on
// compiler flags and can be reproduced bit for bit on a CPU.  The reference's kernels use __expf / rsqrtf / sincosf
// under --use_fast_math (reference Makefile:67); these are the IEEE statements of the same quantities.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace fnxk {

__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float ffma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }

// e^x: k = rint(x log2 e), r = x - k ln2 in two fused steps, degree-5 polynomial on r^2, 2^k through the exponent
// field; 0 below -86, +inf above 88
__device__ __forceinline__ float ex_expf(float x) {
    if (x > 88.0f) return __int_as_float(0x7f800000);
    if (x < -86.0f) return 0.0f;
    const float k = rintf(fmul(x, 1.44269504f));
    float r = ffma(k, -0.693145752f, x);
    r = ffma(k, -1.42860677e-06f, r);
    float p = 1.9875691500e-4f;
    p = ffma(p, r, 1.3981999507e-3f);
    p = ffma(p, r, 8.3334519073e-3f);
    p = ffma(p, r, 4.1665795894e-2f);
    p = ffma(p, r, 1.6666665459e-1f);
    p = ffma(p, r, 5.0000001201e-1f);
    const float r2 = fmul(r, r);
    float e = ffma(p, r2, r);
    e = fadd(e, 1.0f);
    return __uint_as_float(__float_as_uint(e) + ((unsigned) (int) k << 23));
}

// ln(u), finite u >= 1
__device__ __forceinline__ float ex_logf_ge1(float u) {
    unsigned b = __float_as_uint(u);
    int e = (int) (b >> 23) - 127;
    b = (b & 0x007fffffu) | 0x3f800000u;
    float m = __uint_as_float(b);
    if (m > 1.41421354f) {
        m = fmul(m, 0.5f);
        e += 1;
    }
    const float f = fsub(m, 1.0f);
    const float s = fdiv(f, fadd(2.0f, f));
    const float z = fmul(s, s);
    float R = 0.24279078841f;
    R = ffma(R, z, 0.28498786688f);
    R = ffma(R, z, 0.40000972152f);
    R = ffma(R, z, 0.66666662693f);
    const float lm = ffma(fmul(s, z), R, fmul(2.0f, s));
    const float fe = (float) e;
    return ffma(fe, 0.693145752f, ffma(fe, 1.42860677e-06f, lm));
}

// ln(1 + y), y >= 0
__device__ __forceinline__ float ex_log1pf_pos(float y) {
    const float u = fadd(1.0f, y);
    if (u == 1.0f) return y;
    if (isinf(u)) return u;
    return fmul(ex_logf_ge1(u), fdiv(y, fsub(u, 1.0f)));
}

__device__ __forceinline__ float ex_sigmoid(float x) { return fdiv(1.0f, fadd(1.0f, ex_expf(-x))); }
__device__ __forceinline__ float ex_silu(float x) { return fdiv(x, fadd(1.0f, ex_expf(-x))); }
__device__ __forceinline__ float ex_rsqrt(float x) { return fdiv(1.0f, __fsqrt_rn(x)); }

// sin and cos of a double angle >= 0, rounded to float: Cody-Waite reduction by pi/2 in two fused steps, minimax
// kernels on [-pi/4, pi/4]
__device__ __forceinline__ void ex_sincos(double theta, float* sn, float* cs) {
    const double k = rint(__dmul_rn(theta, 0.63661977236758134308));
    double r = __fma_rn(-k, 1.57079632673412561417e+00, theta);
    r = __fma_rn(-k, 6.07710050650619224932e-11, r);
    const double z = __dmul_rn(r, r);
    double ps = 1.58969099521155010221e-10;
    ps = __fma_rn(ps, z, -2.50507602534068634195e-08);
    ps = __fma_rn(ps, z, 2.75573137070700676789e-06);
    ps = __fma_rn(ps, z, -1.98412698298579493134e-04);
    ps = __fma_rn(ps, z, 8.33333333332248946124e-03);
    ps = __fma_rn(ps, z, -1.66666666666666324348e-01);
    const double s = __fma_rn(__dmul_rn(r, z), ps, r);
    double pc = -1.13596475577881948265e-11;
    pc = __fma_rn(pc, z, 2.08757232129817482790e-09);
    pc = __fma_rn(pc, z, -2.75573143513906633035e-07);
    pc = __fma_rn(pc, z, 2.48015872894767294178e-05);
    pc = __fma_rn(pc, z, -1.38888888888741095749e-03);
    pc = __fma_rn(pc, z, 4.16666666666666019037e-02);
    const double c = __fma_rn(__dmul_rn(z, z), pc, __fma_rn(z, -0.5, 1.0));
    const int q = (int) ((long long) k & 3);
    const double so = q == 0 ? s : q == 1 ? c : q == 2 ? -s : -c;
    const double co = q == 0 ? c : q == 1 ? -s : q == 2 ? -c : s;
    *sn = (float) so;
    *cs = (float) co;
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

// monotone key of a float (a larger float, a larger key)
__device__ __forceinline__ unsigned fkey(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

// xor-butterfly sums and maxima over a warp (offsets 16..1) or over groups of 8 lanes (4, 2, 1)
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fadd(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sum8(float v) {
#pragma unroll
    for (int o = 4; o; o >>= 1) v = fadd(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace fnxk
