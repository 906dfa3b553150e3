/* CPU ORACLE - test infrastructure, not product code.
 * Element-wise probes of the exact math (omath.h) so the tests can compare it with libm and with the device. */
#include "oracle.h"

/* op 0 exp, 1 log1p (x >= 0), 2 sigmoid, 3 silu, 4 rsqrt, 5 sin, 6 cos, 7 f16 round trip */
void orc_math_probe(int op, const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float s, c;
        switch (op) {
            case 0: y[i] = o_expf(x[i]); break;
            case 1: y[i] = o_log1pf_pos(x[i]); break;
            case 2: y[i] = o_sigmoid(x[i]); break;
            case 3: y[i] = o_silu(x[i]); break;
            case 4: y[i] = o_rsqrt(x[i]); break;
            case 5: o_sincos((double) x[i], &s, &c); y[i] = s; break;
            case 6: o_sincos((double) x[i], &s, &c); y[i] = c; break;
            default: y[i] = o_h2f(o_f2h(x[i])); break;
        }
    }
}
