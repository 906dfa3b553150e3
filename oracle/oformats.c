/* CPU ORACLE - test infrastructure, not product code.
 *
 * Quantised block formats of the verify window: dequantisers, a plain quantiser for synthetic weights, and the
 * repacks into the device layouts.  Block layouts are the published GGUF ones (sizes: reference src/gguf.cpp:19-37);
 * the Q4_K scale unpacking follows reference src/moe_q4k.cuh:9-23 and tools/moe_mma_bench.cu:43-69, Q8_0 follows
 * src/engine.cu:860-864.  Dequantisers are cross-checked against the `gguf` Python package in the tests.
 */
#include "oracle.h"

/* ---- Q4_K: 144 B = half d, half dmin, u8 scales[12], u8 qs[128]; 256 values */
void orc_q4k_scale_min(const uint8_t* sc12, int j, int* sc, int* m) {
    if (j < 4) {
        *sc = sc12[j] & 63;
        *m = sc12[j + 4] & 63;
    } else {
        *sc = (sc12[j + 4] & 0xF) | ((sc12[j - 4] >> 6) << 4);
        *m = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4);
    }
}

void orc_dequant_q4k(const uint8_t* blocks, float* out, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* p = blocks + b * 144;
        o_half hd, hm;
        memcpy(&hd, p, 2);
        memcpy(&hm, p + 2, 2);
        const float d = o_h2f(hd), dmin = o_h2f(hm);
        for (int s = 0; s < 8; ++s) {
            int sc, m;
            orc_q4k_scale_min(p + 4, s, &sc, &m);
            const float ds = d * (float) sc, dm = dmin * (float) m;
            for (int l = 0; l < 32; ++l) {
                const uint8_t byte = p[16 + 32 * (s / 2) + l];
                const int q = (s & 1) ? (byte >> 4) : (byte & 0xF);
                out[b * 256 + s * 32 + l] = ds * (float) q - dm;
            }
        }
    }
}

/* ---- Q6_K: 210 B = u8 ql[128], u8 qh[64], i8 scales[16], half d; 256 values; value = d * sc[i/16] * (q - 32) */
int orc_q6k_q(const uint8_t* blk, int i) { /* the 6-bit code of value i */
    const int half = i / 128, r = i % 128, l = r % 32, quad = r / 32;
    const uint8_t* ql = blk + 64 * half;
    const uint8_t* qh = blk + 128 + 32 * half;
    const int lo = (quad & 1) ? ql[l + 32] : ql[l];
    const int nib = (quad >= 2) ? (lo >> 4) : (lo & 0xF);
    const int hi = (qh[l] >> (2 * quad)) & 3;
    return nib | (hi << 4);
}

void orc_dequant_q6k(const uint8_t* blocks, float* out, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* p = blocks + b * 210;
        o_half hd;
        memcpy(&hd, p + 208, 2);
        const float d = o_h2f(hd);
        const int8_t* sc = (const int8_t*) (p + 192);
        for (int i = 0; i < 256; ++i) out[b * 256 + i] = (d * (float) sc[i / 16]) * (float) (orc_q6k_q(p, i) - 32);
    }
}

/* ---- Q8_0: 34 B = half d, i8 qs[32] */
void orc_dequant_q8_0(const uint8_t* blocks, float* out, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* p = blocks + b * 34;
        o_half hd;
        memcpy(&hd, p, 2);
        const float d = o_h2f(hd);
        for (int l = 0; l < 32; ++l) out[b * 32 + l] = d * (float) ((const int8_t*) (p + 2))[l];
    }
}

/* ---- a plain quantiser for synthetic weights (ours; parity is on the dequantisation of the same bytes, not on
 * matching any other quantiser).  Q8_0: d = amax / 127. */
void orc_quantize_q8_0(const float* x, uint8_t* blocks, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        float amax = 0.f;
        for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(x[b * 32 + l]));
        const float d = amax / 127.0f;
        const o_half hd = o_f2h(d);
        const float df = o_h2f(hd);
        uint8_t* p = blocks + b * 34;
        memcpy(p, &hd, 2);
        for (int l = 0; l < 32; ++l) {
            int q = df == 0.f ? 0 : (int) roundf(x[b * 32 + l] / df);
            q = q > 127 ? 127 : q < -127 ? -127 : q;
            ((int8_t*) (p + 2))[l] = (int8_t) q;
        }
    }
}

/* Q4_K: per 32-value sub-block scale = (max - min) / 15 and offset = -min (min clamped to <= 0); the super-block
 * holds d = max scale / 63, dmin = max offset / 63 as f16 and the 6-bit codes of both. */
void orc_quantize_q4k(const float* x, uint8_t* blocks, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        const float* xb = x + b * 256;
        float scale[8], off[8], smax = 0.f, omax = 0.f;
        for (int s = 0; s < 8; ++s) {
            float mn = 0.f, mx = 0.f;
            for (int l = 0; l < 32; ++l) {
                mn = fminf(mn, xb[s * 32 + l]);
                mx = fmaxf(mx, xb[s * 32 + l]);
            }
            scale[s] = (mx - mn) / 15.0f;
            off[s] = -mn;
            smax = fmaxf(smax, scale[s]);
            omax = fmaxf(omax, off[s]);
        }
        const o_half hd = o_f2h(smax / 63.0f), hm = o_f2h(omax / 63.0f);
        const float d = o_h2f(hd), dmin = o_h2f(hm);
        uint8_t* p = blocks + b * 144;
        memset(p, 0, 144);
        memcpy(p, &hd, 2);
        memcpy(p + 2, &hm, 2);
        int sc[8], m[8];
        for (int s = 0; s < 8; ++s) {
            sc[s] = d == 0.f ? 0 : (int) roundf(scale[s] / d);
            m[s] = dmin == 0.f ? 0 : (int) roundf(off[s] / dmin);
            sc[s] = sc[s] > 63 ? 63 : sc[s];
            m[s] = m[s] > 63 ? 63 : m[s];
        }
        uint8_t* s12 = p + 4;
        for (int j = 0; j < 4; ++j) {
            s12[j] = (uint8_t) ((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
            s12[j + 4] = (uint8_t) ((m[j] & 63) | ((m[j + 4] >> 4) << 6));
            s12[j + 8] = (uint8_t) ((sc[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
        }
        for (int s = 0; s < 8; ++s) {
            const float ds = d * (float) sc[s], dm = dmin * (float) m[s];
            for (int l = 0; l < 32; ++l) {
                int q = ds == 0.f ? 0 : (int) roundf((xb[s * 32 + l] + dm) / ds);
                q = q < 0 ? 0 : q > 15 ? 15 : q;
                uint8_t* byte = p + 16 + 32 * (s / 2) + l;
                *byte = (uint8_t) ((s & 1) ? (*byte | (q << 4)) : (*byte | q));
            }
        }
    }
}

/* Q6_K: per 16-value sub-block scale = amax / 31; d = max scale / 127 (f16); 8-bit signed codes of the scales. */
void orc_quantize_q6k(const float* x, uint8_t* blocks, size_t nblocks) {
    for (size_t b = 0; b < nblocks; ++b) {
        const float* xb = x + b * 256;
        float scale[16], smax = 0.f;
        for (int s = 0; s < 16; ++s) {
            float amax = 0.f;
            for (int l = 0; l < 16; ++l) amax = fmaxf(amax, fabsf(xb[s * 16 + l]));
            scale[s] = amax / 31.0f;
            smax = fmaxf(smax, scale[s]);
        }
        const o_half hd = o_f2h(smax / 127.0f);
        const float d = o_h2f(hd);
        uint8_t* p = blocks + b * 210;
        memset(p, 0, 210);
        memcpy(p + 208, &hd, 2);
        int8_t* sc = (int8_t*) (p + 192);
        for (int s = 0; s < 16; ++s) {
            int v = d == 0.f ? 0 : (int) roundf(scale[s] / d);
            sc[s] = (int8_t) (v > 127 ? 127 : v);
        }
        for (int i = 0; i < 256; ++i) {
            const float ds = d * (float) sc[i / 16];
            int q = ds == 0.f ? 32 : (int) roundf(xb[i] / ds) + 32;
            q = q < 0 ? 0 : q > 63 ? 63 : q;
            const int half = i / 128, r = i % 128, l = r % 32, quad = r / 32;
            uint8_t* ql = p + 64 * half + ((quad & 1) ? l + 32 : l);
            *ql = (uint8_t) ((quad >= 2) ? (*ql | ((q & 0xF) << 4)) : (*ql | (q & 0xF)));
            p[128 + 32 * half + l] |= (uint8_t) ((q >> 4) << (2 * quad));
        }
    }
}

/* ---- device layouts
 * Q8_0 split layout (the reference's Q8S, src/model.hpp:71-87): int8 plane [rows][cols], f16 scales [rows][cols/32]. */
void orc_q8_0_to_split(const uint8_t* blocks, int8_t* q, o_half* d, size_t rows, size_t cols) {
    const size_t nb = cols / 32;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* p = blocks + (r * nb + b) * 34;
            memcpy(&d[r * nb + b], p, 2);
            memcpy(q + r * cols + b * 32, p + 2, 32);
        }
}

/* Q6_K planes in 32-column units (our layout; the same 210 bytes per 256 values, regrouped so that a matrix can be
 * cut by columns at any multiple of 32, which the FF split across GPUs needs: reference src/model.cpp:206-210
 * refuses 256-wide blocks for the down matrices for that reason).  For a matrix of rows x cols (cols % 32 == 0,
 * the source rows being whole Q6_K super-blocks of a wider matrix src_cols, columns [c0, c0 + cols)):
 *   QL [rows][cols/32][16]  byte j: low nibble = code(j) & 15, high nibble = code(j + 16) & 15
 *   QH [rows][cols/32][8]   byte j: 2-bit fields k = 0..3 hold code(4 k' ...) >> 4, see orc_q6p_q
 *   SC [rows][cols/32][2]   int8 scales of the unit's two 16-value sub-blocks
 *   D  [rows][cols/32]      f16 super-block scale, repeated per unit
 * code(i) of unit u is the 6-bit code of column c0 + 32 u + i.  In QH, value i = 4 w + b of (word w = 0..7 of
 * four values, byte b): words 0..3 are values 0..15 (the low nibbles' order), words 4..7 values 16..31; the two
 * high bits of value 4 w + b sit in QH byte (w / 4) * 4 + b at bit 2 (w % 4). */
void orc_q6k_to_planes(const uint8_t* blocks, size_t rows, size_t src_cols, size_t c0, size_t cols, uint8_t* QL,
                       uint8_t* QH, int8_t* SC, o_half* D) {
    const size_t nu = cols / 32, nsb = src_cols / 256;
    memset(QL, 0, rows * nu * 16);
    memset(QH, 0, rows * nu * 8);
    for (size_t r = 0; r < rows; ++r)
        for (size_t u = 0; u < nu; ++u) {
            const size_t col = c0 + u * 32;
            const uint8_t* blk = blocks + (r * nsb + col / 256) * 210;
            const int i0 = (int) (col % 256);
            uint8_t* ql = QL + (r * nu + u) * 16;
            uint8_t* qh = QH + (r * nu + u) * 8;
            for (int i = 0; i < 32; ++i) {
                const int q = orc_q6k_q(blk, i0 + i);
                if (i < 16) ql[i] |= (uint8_t) (q & 15);
                else ql[i - 16] |= (uint8_t) ((q & 15) << 4);
                const int w = i / 4, b = i % 4;
                qh[(w / 4) * 4 + b] |= (uint8_t) ((q >> 4) << (2 * (w % 4)));
            }
            SC[(r * nu + u) * 2] = ((const int8_t*) (blk + 192))[i0 / 16];
            SC[(r * nu + u) * 2 + 1] = ((const int8_t*) (blk + 192))[i0 / 16 + 1];
            memcpy(&D[r * nu + u], blk + 208, 2);
        }
}

int orc_q6p_q(const uint8_t* ql16, const uint8_t* qh8, int i) {
    const int lo = i < 16 ? (ql16[i] & 15) : (ql16[i - 16] >> 4);
    const int w = i / 4, b = i % 4;
    const int hi = (qh8[(w / 4) * 4 + b] >> (2 * (w % 4))) & 3;
    return lo | (hi << 4);
}

/* ---- q8_1 activations (reference src/kernels.cu:99-113): 36 B = half d, half sum, i8 qs[32] */
void orc_quantize_q8_1(const float* x, uint8_t* q, int n, int rows) {
    const int nb = n / 32;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const float* xb = x + (size_t) r * n + b * 32;
            float v[32], a[32];
            for (int l = 0; l < 32; ++l) {
                v[l] = xb[l];
                a[l] = fabsf(xb[l]);
            }
            float amax = 0.f;
            for (int l = 0; l < 32; ++l) amax = fmaxf(amax, a[l]);
            const float sum = o_butterfly(v, 32);
            const float d = amax / 127.0f;
            uint8_t* p = q + ((size_t) r * nb + b) * 36;
            const o_half hd = o_f2h(d), hs = o_f2h(sum);
            memcpy(p, &hd, 2);
            memcpy(p + 2, &hs, 2);
            for (int l = 0; l < 32; ++l) ((int8_t*) (p + 4))[l] = amax == 0.0f ? 0 : (int8_t) roundf(xb[l] / d);
        }
}
