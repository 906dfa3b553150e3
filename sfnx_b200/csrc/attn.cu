// Position-split attention of the verify window: per-head RMS norm + NEOX rotary + K/V append, the scan over the
// positions this GPU owns in the reference's order of sums (bit-reproducible; also the scan of windows of several
// sequences), the joining of its runs, and the merge of the GPUs' partials with the output gate.  Covers what reference
// src/kernels.cu:451-469, 480-691, 1539-1569 compute.
//
// K/V placement (reference src/kernels.hpp:126-130): blocks of 4 positions are dealt round-robin, block j on GPU
// j % ncard at local block j / ncard; local row = local block * 4 + p % 4.
#include <cmath>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "umma.cuh"

namespace fnxk {

constexpr int ATT_SPLITS = 16, ATT_CH = 32, ATT_MAXQPK = 16;

__host__ __device__ inline int kv_owned(int p, int card, int ncard) {   // positions <= p this GPU owns
    const int b = p / 4;
    const int blocks = (b + ncard - 1 - card) / ncard;
    return blocks * 4 + (b % ncard == card ? p % 4 + 1 : 0);
}
__device__ __forceinline__ size_t kv_row_at(const FnxKvPages& g, int r, int nkv, int hd) {
    if (!g.pt) return (size_t) r * nkv * hd;
    return (size_t) g.pt[r / g.rows] * g.page + (size_t) (r % g.rows) * nkv * hd;
}

// int8 rows (reference src/kernels.hpp:172-177 kvq_row, kvq_scale): row r's first byte, and its first scale in halves,
// both from the layer's K (or V) pointer; a page's scales follow its rows, and a cache without a page table is one page
// of g.cap rows
__device__ __forceinline__ size_t kvq_row_at(const FnxKvPages& g, int r, int nkv, int hd) {
    if (!g.pt) return (size_t) r * nkv * hd;
    return (size_t) g.pt[r / g.rows] * g.page * 2 + (size_t) (r % g.rows) * nkv * hd;
}
__device__ __forceinline__ size_t kvq_scale_at(const FnxKvPages& g, int r, int nkv, int hd) {
    if (!g.pt) return (size_t) g.cap * nkv * hd / 2 + (size_t) r * nkv * hd / 32;
    return (size_t) g.pt[r / g.rows] * g.page + (size_t) g.rows * nkv * hd / 2 + (size_t) (r % g.rows) * nkv * hd / 32;
}

struct RopeFreqs {
    float f[64];   // unit frequency of pair i, base^(-2 i / nrot), computed by the host's powf
    int nrot;
};

// one head's row: RMS norm with weight (warp trees, the warps added in ascending order), then the rotation of the
// pairs (i, i + nrot / 2) by theta = (float) pos * f[i]
__device__ void norm_rope(float* x, const float* w, int pos, float eps, const RopeFreqs& rf, int hd, float* sh) {
    const int i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const float v = x[i];
    const float ws = wsum(fmul(v, v));
    if (lane == 0) sh[warp] = ws;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < hd / 32; ++k) tot = fadd(tot, sh[k]);
    const float y = fmul(fmul(v, ex_rsqrt(fadd(fdiv(tot, (float) hd), eps))), w[i]);
    __syncthreads();
    x[i] = y;
    __syncthreads();
    if (i < rf.nrot / 2) {
        const float theta = fmul((float) pos, rf.f[i]);
        float sn, cs;
        ex_sincos((double) theta, &sn, &cs);
        const float x0 = x[i], x1 = x[i + rf.nrot / 2];
        x[i] = ffma(-x1, sn, fmul(x0, cs));
        x[i + rf.nrot / 2] = ffma(x1, cs, fmul(x0, sn));
    }
}

// block (h, row t), hd threads: h < nq the q heads; then the nkv k heads (normed, rotated, appended); then the v heads
__global__ void k_attn_prep_append(float* qg, float* k, const float* v, const float* qn, const float* kn, uint16_t* kc, uint16_t* vc,
                                   FnxKvPages g, int card, int ncard, const int* pos0p, float eps, RopeFreqs rf, int nq, int nkv,
                                   int hd) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.y, h = blockIdx.x, i = threadIdx.x, p = *pos0p + t, j = p / 4;
    __shared__ float sh[32];
    if (h < nq) {
        norm_rope(qg + ((size_t) t * nq + h) * 2 * hd, qn, p, eps, rf, hd, sh);
        return;
    }
    const bool is_k = h < nq + nkv;
    const int kh = h - nq - (is_k ? 0 : nkv), e = kh * hd + i;
    float x;
    if (is_k) {
        float* kr = k + ((size_t) t * nkv + kh) * hd;
        norm_rope(kr, kn, p, eps, rf, hd, sh);
        __syncthreads();
        x = kr[i];
    } else {
        x = v[(size_t) t * nkv * hd + e];
    }
    if (j % ncard != card) return;
    const int r = (j / ncard) * 4 + p % 4;
    if (!g.pt && g.cap > 0 && r >= g.cap) return;   // past the cache: the caller refuses such windows; never write outside
    uint16_t* cache = is_k ? kc : vc;
    if (g.q8) {   // a warp's 32 elements are one group (reference src/kernels.cu:1561-1566)
        const float d = fdiv(wmax(fabsf(x)), 127.f), id = d != 0.f ? fdiv(1.f, d) : 0.f;
        reinterpret_cast<int8_t*>(cache)[kvq_row_at(g, r, nkv, hd) + e] = (int8_t) roundf(fmul(x, id));
        if ((e & 31) == 0) cache[kvq_scale_at(g, r, nkv, hd) + e / 32] = f2h(d);
        return;
    }
    cache[kv_row_at(g, r, nkv, hd) + e] = f2h(x);
}

// ---------------------------------------------------------------- the scan in the reference's order of sums
// The reference's statement (src/kernels.cu:497-606) fixes, for every (row, head), a split of the row's owned positions
// into 16 runs of `len` rows, chunks of 32 positions inside a run, a score as one fused chain over the head dimension,
// an online-softmax step per chunk (warp xor-trees over the chunk's 32 weights) and value rows added in ascending
// position; this kernel keeps all of that and changes who does it.  One block takes (run s, KV head, group of rows):
// the rows of a window that read the same K/V (the same sequence) and have the same `len` walk the same chunks, so the
// block stages each chunk of K and V once, as f32, and applies it to every (row, head) pair of the group - up to 96
// pairs at a time - instead of once per row.  Rows group themselves on the device: block z = t works only if row t is
// the first of its group, and then takes every later row of the group with it.
//   scores : warp w holds pairs w, w + 8, ...; lane = position of the chunk; 12 independent chains a thread, the
//            pair's query row read as float4 broadcasts
//   softmax: the pair's 32 weights sit across the lanes of one warp, as the reference's trees want them
//   values : thread = head dimension, one accumulator per pair in registers, the chunk's 32 V values of that
//            dimension in registers too
// PT is how many (row, head) pairs a block applies a chunk to at a time: 96 for the groups of rows that attend every owned
// position, 8 or 16 (a pair or two a warp, more blocks an SM) for a row with a list of its own, which shares its chunks
// with no other row.
// scratch: acc [T][nq][16][hd], then (m, z) [T][nq][16].
struct AttPart {
    float m, z;
};
constexpr int AX_THREADS = 256, AX_WARPS = AX_THREADS / 32, AX_PT = 96, AX_PPW = AX_PT / AX_WARPS;

template <int HD, int PT>
__global__ void __launch_bounds__(AX_THREADS, PT <= 16 ? 2 : 1) k_attn_rows(const float* __restrict__ qg, const uint16_t* __restrict__ kc,
                                                           const uint16_t* __restrict__ vc, FnxKvPages g, float* __restrict__ acc_out,
                                                           AttPart* __restrict__ mz_out, int T, int nq, int nkv,
                                                           const int* __restrict__ pos0p, int card, int ncard, FnxLaneRows lr,
                                                           const int* __restrict__ cells, const int* __restrict__ n_cells, int maxsel, int which) {
    constexpr int G = AX_THREADS / HD, APT = PT / G, PPW = PT / AX_WARPS, KLD = HD + 4;   // thread groups over the pairs; accumulators a thread
    const int s = blockIdx.x, kvl = blockIdx.y, lead = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int qpk = nq / nkv;
    if (which && (cells && n_cells[lead] >= 0) != (which == 2)) return;   // this launch takes the other kind of rows
    __shared__ int ctx_s[FNX_MAXT], len_s[FNX_MAXT], rows_s[FNX_MAXT], list_s[FNX_MAXT], nr_s;
    __shared__ const int* pt_s[FNX_MAXT];
    if (tid < T) {
        const bool listed = cells && n_cells[tid] >= 0;   // the row attends a list of its own (the block selection's)
        const int c = listed ? n_cells[tid] : kv_owned(lr.pos ? *lr.pos[tid] : *pos0p + tid, card, ncard);
        list_s[tid] = listed;
        ctx_s[tid] = c;
        len_s[tid] = ((c + ATT_SPLITS - 1) / ATT_SPLITS + ATT_CH - 1) / ATT_CH * ATT_CH;
        pt_s[tid] = lr.pt ? lr.pt[tid] : g.pt;
    }
    __syncthreads();
    if (tid == 0) {
        int nr = 0;
        bool first = true;
        for (int t = 0; t < T; ++t) {
            if (pt_s[t] != pt_s[lead] || len_s[t] != len_s[lead]) continue;
            if (t != lead && (list_s[t] || list_s[lead])) continue;   // a listed row is a group of its own
            if (t < lead) first = false;
            else rows_s[nr++] = t;
        }
        // which: 0 every group; 1 only rows that attend every owned position; 2 only rows with a list of their own
        nr_s = first && !(which == 1 && list_s[lead]) && !(which == 2 && !list_s[lead]) ? nr : 0;
    }
    __syncthreads();
    const int nr = nr_s;
    if (nr == 0) return;   // an earlier row leads this row's group
    g.pt = pt_s[lead];
    const int len = len_s[lead], p0 = s * len;
    const int* list = list_s[lead] ? cells + (size_t) lead * maxsel : nullptr;
    int pend = 0;          // where the group's longest row ends inside this run
    for (int r = 0; r < nr; ++r) pend = max(pend, min(ctx_s[rows_s[r]], p0 + len));
    extern __shared__ __align__(16) float ax_sm[];
    float* q_s = ax_sm;                          // [PT][HD]
    float* k_s = q_s + (size_t) PT * HD;      // [32][HD + 4]
    float* v_s = k_s + (size_t) ATT_CH * KLD;    // [32][HD]
    float* w_s = v_s + (size_t) ATT_CH * HD;     // [PT][32]
    float* sc_s = w_s + (size_t) PT * ATT_CH; // [PT]
    int* np_s = reinterpret_cast<int*>(sc_s + PT);   // [PT]: positions of the chunk the pair takes (0: none)
    const float rs = ex_rsqrt((float) HD);
    const int grp = tid / HD, d = tid % HD;
    const int npairs = nr * qpk;
#pragma unroll 1
    for (int pb = 0; pb < npairs; pb += PT) {
        const int npt = min(PT, npairs - pb);
        __syncthreads();
        for (int e = tid; e < npt * (HD / 4); e += AX_THREADS) {
            const int pi = e / (HD / 4), c4 = e % (HD / 4), t = rows_s[(pb + pi) / qpk], h = kvl * qpk + (pb + pi) % qpk;
            reinterpret_cast<float4*>(q_s + (size_t) pi * HD)[c4] = reinterpret_cast<const float4*>(qg + ((size_t) t * nq + h) * 2 * HD)[c4];
        }
        float m[PPW], z[PPW];
#pragma unroll
        for (int i = 0; i < PPW; ++i) m[i] = -INFINITY, z[i] = 0.f;
        float acc[APT];
#pragma unroll
        for (int i = 0; i < APT; ++i) acc[i] = 0.f;
#pragma unroll 1
        for (int c0 = p0; c0 < pend; c0 += ATT_CH) {
            const int npmax = min(ATT_CH, pend - c0);
            __syncthreads();   // the chunk before has been used up
            // ---- the chunk's K and V rows as f32: 16-byte pieces of 8 halves
            for (int e = tid; e < ATT_CH * (HD / 8); e += AX_THREADS) {
                const int pp = e / (HD / 8), c8 = e % (HD / 8);
                float kf[8], vf[8];
                if (g.q8) {   // int8 values times their group's scale (reference src/kernels.cu:531-537): 8 values of one group
                    uint2 kr = make_uint2(0, 0), vr = kr;
                    float kd8 = 0.f, vd8 = 0.f;
                    if (pp < npmax) {
                        const int r = list ? list[c0 + pp] : c0 + pp;
                        const size_t at = kvq_row_at(g, r, nkv, HD) + (size_t) kvl * HD + 8 * c8;
                        const size_t sc = kvq_scale_at(g, r, nkv, HD) + ((size_t) kvl * HD + 8 * c8) / 32;
                        kr = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(kc) + at);
                        vr = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(vc) + at);
                        kd8 = h2f(kc[sc]), vd8 = h2f(vc[sc]);
                    }
                    const unsigned kw[2] = {kr.x, kr.y}, vw[2] = {vr.x, vr.y};
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        kf[k] = fmul((float) (int8_t) (kw[k >> 2] >> (8 * (k & 3))), kd8);
                        vf[k] = fmul((float) (int8_t) (vw[k >> 2] >> (8 * (k & 3))), vd8);
                    }
                } else {
                    uint4 kr = make_uint4(0, 0, 0, 0), vr = kr;
                    if (pp < npmax) {
                        const size_t at = kv_row_at(g, list ? list[c0 + pp] : c0 + pp, nkv, HD) + (size_t) kvl * HD + 8 * c8;
                        kr = *reinterpret_cast<const uint4*>(kc + at);
                        vr = *reinterpret_cast<const uint4*>(vc + at);
                    }
                    const unsigned kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        kf[2 * k] = h2f((uint16_t) (kw[k] & 0xffff)), kf[2 * k + 1] = h2f((uint16_t) (kw[k] >> 16));
                        vf[2 * k] = h2f((uint16_t) (vw[k] & 0xffff)), vf[2 * k + 1] = h2f((uint16_t) (vw[k] >> 16));
                    }
                }
                float4* kd = reinterpret_cast<float4*>(k_s + (size_t) pp * KLD + 8 * c8);
                float4* vd = reinterpret_cast<float4*>(v_s + (size_t) pp * HD + 8 * c8);
                kd[0] = make_float4(kf[0], kf[1], kf[2], kf[3]), kd[1] = make_float4(kf[4], kf[5], kf[6], kf[7]);
                vd[0] = make_float4(vf[0], vf[1], vf[2], vf[3]), vd[1] = make_float4(vf[4], vf[5], vf[6], vf[7]);
            }
            __syncthreads();
            // ---- scores: this lane's position against the warp's pairs, each a fused chain over the head dimension
            float sa[PPW];
#pragma unroll
            for (int i = 0; i < PPW; ++i) sa[i] = 0.f;
            const float4* k4 = reinterpret_cast<const float4*>(k_s + (size_t) lane * KLD);
#pragma unroll 2
            for (int c4 = 0; c4 < HD / 4; ++c4) {
                const float4 kk = k4[c4];
#pragma unroll
                for (int i = 0; i < PPW; ++i) {
                    const float4 qq = reinterpret_cast<const float4*>(q_s + (size_t) (warp + AX_WARPS * i) * HD)[c4];
                    sa[i] = ffma(qq.x, kk.x, sa[i]);
                    sa[i] = ffma(qq.y, kk.y, sa[i]);
                    sa[i] = ffma(qq.z, kk.z, sa[i]);
                    sa[i] = ffma(qq.w, kk.w, sa[i]);
                }
            }
            // ---- the online-softmax step of every pair of the warp (all lanes hold the pair's m and z)
#pragma unroll
            for (int i = 0; i < PPW; ++i) {
                const int pi = warp + AX_WARPS * i;
                if (pi < npt) {
                    const int t = rows_s[(pb + pi) / qpk];
                    const int np = min(ATT_CH, min(ctx_s[t], p0 + len) - c0);   // <= 0: this row's run ended before the chunk
                    if (np > 0) {
                        const float sv = lane < np ? fmul(sa[i], rs) : -INFINITY;
                        const float mn = fmaxf(m[i], wmax(sv));
                        const float w = sv == -INFINITY ? 0.f : ex_expf(fsub(sv, mn));
                        const float sc = m[i] == -INFINITY ? 0.f : ex_expf(fsub(m[i], mn));
                        z[i] = ffma(z[i], sc, wsum(w));
                        m[i] = mn;
                        w_s[pi * ATT_CH + lane] = w;
                        if (lane == 0) sc_s[pi] = sc;
                    }
                    if (lane == 0) np_s[pi] = max(np, 0);
                }
            }
            __syncthreads();
            // ---- values: acc = acc sc, then + w v in ascending position, for this thread's dimension
            float vv[ATT_CH];
#pragma unroll
            for (int pp = 0; pp < ATT_CH; ++pp) vv[pp] = v_s[(size_t) pp * HD + d];
#pragma unroll
            for (int i = 0; i < APT; ++i) {
                const int pi = grp * APT + i;
                if (pi < npt) {
                    const int np = np_s[pi];
                    if (np == ATT_CH) {
                        float a = fmul(acc[i], sc_s[pi]);
                        const float4* w4 = reinterpret_cast<const float4*>(w_s + (size_t) pi * ATT_CH);
#pragma unroll
                        for (int p4 = 0; p4 < ATT_CH / 4; ++p4) {
                            const float4 ww = w4[p4];
                            a = ffma(ww.x, vv[4 * p4], a);
                            a = ffma(ww.y, vv[4 * p4 + 1], a);
                            a = ffma(ww.z, vv[4 * p4 + 2], a);
                            a = ffma(ww.w, vv[4 * p4 + 3], a);
                        }
                        acc[i] = a;
                    } else if (np > 0) {   // a row's last, partial chunk
                        float a = fmul(acc[i], sc_s[pi]);
                        for (int pp = 0; pp < np; ++pp) a = ffma(w_s[pi * ATT_CH + pp], v_s[(size_t) pp * HD + d], a);
                        acc[i] = a;
                    }
                }
            }
        }
        // ---- this run's partial of every pair of the tile
#pragma unroll
        for (int i = 0; i < APT; ++i) {
            const int pi = grp * APT + i;
            if (pi < npt) {
                const int t = rows_s[(pb + pi) / qpk], h = kvl * qpk + (pb + pi) % qpk;
                acc_out[(((size_t) t * nq + h) * ATT_SPLITS + s) * HD + d] = acc[i];
            }
        }
#pragma unroll
        for (int i = 0; i < PPW; ++i) {
            const int pi = warp + AX_WARPS * i;
            if (pi < npt && lane == 0) {
                const int t = rows_s[(pb + pi) / qpk], h = kvl * qpk + (pb + pi) % qpk;
                mz_out[((size_t) t * nq + h) * ATT_SPLITS + s] = AttPart{m[i], z[i]};
            }
        }
    }
}

// ---------------------------------------------------------------- a row with a list of its own (the block selection's cells)
// The same sums in the same order as k_attn_rows, laid out for a row that shares its positions with no other row: a block
// takes (run s, KV head, row t) and up to `nch` chunks of 32 positions at a time.
//   K rows   gathered into shared memory as f16 by one bulk (TMA) copy a position, rows padded by 16 bytes so that every
//            lane reads its own row without bank conflicts;
//   scores   warp c takes chunk c, lane = position: one fused chain over the head dimension per (position, head), the KV
//            head's query heads side by side in registers (QM slots), so a lane runs up to QM independent chains;
//   softmax  the chunks' maxima are exchanged through shared memory; warp c then knows the running maximum before its
//            chunk (maxima are exact in any order) and makes its chunk's weights, their warp-tree sum and the rescale
//            factor; z is chained over the chunks in order by one thread per head;
//   values   thread = head dimension: per chunk in order, acc = acc * rescale, then + w v in ascending position, the 32
//            V values of the dimension read straight from the cache (f16) into registers.
// f16 caches only (an int8 cache's listed rows go through k_attn_rows).
template <int HD, int QM>
__global__ void __launch_bounds__(AX_THREADS) k_attn_cells(const float* __restrict__ qg, const uint16_t* __restrict__ kc, const uint16_t* __restrict__ vc,
                                                          FnxKvPages g, float* __restrict__ acc_out, AttPart* __restrict__ mz_out, int nq, int nkv,
                                                          FnxLaneRows lr, const int* __restrict__ cells, const int* __restrict__ n_cells, int maxsel,
                                                          int nch, unsigned* fault) {
    constexpr int KLD = HD + 8;   // halves a staged K row takes
    const int s = blockIdx.x, kvl = blockIdx.y, t = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ctx = n_cells[t];
    if (ctx < 0) return;   // the row attends every owned position: k_attn_rows' launch takes it
    const int qpk = nq / nkv;
    if (lr.pt) g.pt = lr.pt[t];
    const int* list = cells + (size_t) t * maxsel;
    const int len = ((ctx + ATT_SPLITS - 1) / ATT_SPLITS + ATT_CH - 1) / ATT_CH * ATT_CH, p0 = s * len, p1 = min(ctx, p0 + len);
    extern __shared__ __align__(16) unsigned char ac_sm[];
    float* q_s = reinterpret_cast<float*>(ac_sm);                                  // [qpk][HD]
    uint16_t* k_s = reinterpret_cast<uint16_t*>(q_s + (size_t) qpk * HD);          // [nch 32][KLD]
    size_t* row_s = reinterpret_cast<size_t*>(k_s + (size_t) nch * ATT_CH * KLD);  // [nch 32] the positions' rows in the cache (halves)
    float* w_s = reinterpret_cast<float*>(row_s + nch * ATT_CH);                   // [nch][qpk][32]
    float* cm_s = w_s + (size_t) nch * qpk * ATT_CH;                               // [nch][qpk] chunk maxima
    float* sc_s = cm_s + nch * qpk;                                                // [nch][qpk] rescale factors
    float* sum_s = sc_s + nch * qpk;                                               // [nch][qpk] sums of weights
    float* m_s = sum_s + nch * qpk;                                                // [qpk] running maximum before the group
    float* z_s = m_s + qpk;                                                        // [qpk]
    for (int e = tid; e < qpk * (HD / 4); e += AX_THREADS) {
        const int pi = e / (HD / 4), c4 = e % (HD / 4);
        reinterpret_cast<float4*>(q_s + (size_t) pi * HD)[c4] = reinterpret_cast<const float4*>(qg + ((size_t) t * nq + kvl * qpk + pi) * 2 * HD)[c4];
    }
    if (tid < qpk) m_s[tid] = -INFINITY, z_s[tid] = 0.f;
    __shared__ __align__(8) unsigned long long kbar;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&kbar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    unsigned kphase = 0;
    float acc[QM];
#pragma unroll
    for (int i = 0; i < QM; ++i) acc[i] = 0.f;
    const float rs = ex_rsqrt((float) HD);
#pragma unroll 1
    for (int g0 = p0; g0 < p1; g0 += nch * ATT_CH) {
        const int ng = min(nch * ATT_CH, p1 - g0), nck = (ng + ATT_CH - 1) / ATT_CH;
        __syncthreads();   // the group before has been used up (and q_s, m_s, z_s are written)
        // one bulk copy a position: its K row (HD halves) into the padded row of k_s, all of the group's in flight at once,
        // counted as bytes on the block's mbarrier (a bounded wait: on a timeout the fault word is set and the block goes on)
        if (tid == 0) um_expect_tx(&kbar, (unsigned) ng * HD * 2);
        __syncthreads();
        for (int i = tid; i < ng; i += AX_THREADS) {
            const size_t r = kv_row_at(g, list[g0 + i], nkv, HD) + (size_t) kvl * HD;
            row_s[i] = r;
            um_bulk(um_s32(k_s + (size_t) i * KLD), kc + r, HD * 2, &kbar);
        }
        um_wait(&kbar, kphase, fault);
        kphase ^= 1u;
        __syncthreads();   // (row_s is complete for the values)
        // ---- scores of chunk `warp`
        float sv[QM];
        const int at = warp * ATT_CH + lane;
        const bool have = warp < nck, valid = have && at < ng;
        if (have) {
            float sa[QM];
#pragma unroll
            for (int i = 0; i < QM; ++i) sa[i] = 0.f;
            if (valid) {
                const uint4* kr = reinterpret_cast<const uint4*>(k_s + (size_t) at * KLD);
#pragma unroll 2
                for (int c8 = 0; c8 < HD / 8; ++c8) {
                    const uint4 u = kr[c8];
                    const unsigned kw[4] = {u.x, u.y, u.z, u.w};
                    float kf[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) kf[2 * k] = h2f((uint16_t) (kw[k] & 0xffff)), kf[2 * k + 1] = h2f((uint16_t) (kw[k] >> 16));
#pragma unroll
                    for (int i = 0; i < QM; ++i)
                        if (i < qpk) {
                            const float4 qa = reinterpret_cast<const float4*>(q_s + (size_t) i * HD)[2 * c8];
                            const float4 qb = reinterpret_cast<const float4*>(q_s + (size_t) i * HD)[2 * c8 + 1];
                            float a = sa[i];
                            a = ffma(qa.x, kf[0], a), a = ffma(qa.y, kf[1], a), a = ffma(qa.z, kf[2], a), a = ffma(qa.w, kf[3], a);
                            a = ffma(qb.x, kf[4], a), a = ffma(qb.y, kf[5], a), a = ffma(qb.z, kf[6], a), a = ffma(qb.w, kf[7], a);
                            sa[i] = a;
                        }
                }
            }
#pragma unroll
            for (int i = 0; i < QM; ++i)
                if (i < qpk) {
                    sv[i] = valid ? fmul(sa[i], rs) : -INFINITY;
                    const float cm = wmax(sv[i]);
                    if (lane == 0) cm_s[warp * qpk + i] = cm;
                }
        }
        __syncthreads();
        // ---- the chunk's weights against the running maximum before it
        if (have) {
#pragma unroll
            for (int i = 0; i < QM; ++i)
                if (i < qpk) {
                    float mb = m_s[i];
                    for (int c = 0; c < warp; ++c) mb = fmaxf(mb, cm_s[c * qpk + i]);
                    const float mn = fmaxf(mb, cm_s[warp * qpk + i]);
                    const float w = sv[i] == -INFINITY ? 0.f : ex_expf(fsub(sv[i], mn));
                    const float sc = mb == -INFINITY ? 0.f : ex_expf(fsub(mb, mn));
                    const float ws = wsum(w);
                    w_s[((size_t) warp * qpk + i) * ATT_CH + lane] = w;
                    if (lane == 0) sc_s[warp * qpk + i] = sc, sum_s[warp * qpk + i] = ws;
                }
        }
        __syncthreads();
        if (tid < qpk) {   // z and the maximum, chained over the group's chunks in order
            float z = z_s[tid], m = m_s[tid];
            for (int c = 0; c < nck; ++c) z = ffma(z, sc_s[c * qpk + tid], sum_s[c * qpk + tid]), m = fmaxf(m, cm_s[c * qpk + tid]);
            z_s[tid] = z, m_s[tid] = m;   // read again only after the next group's first barriers
        }
        // ---- values
        if (tid < HD) {
            auto use = [&](const float* vv, int c) {
                const int np = min(ATT_CH, ng - c * ATT_CH);
#pragma unroll
                for (int i = 0; i < QM; ++i)
                    if (i < qpk) {
                        float a = fmul(acc[i], sc_s[c * qpk + i]);
                        const float4* w4 = reinterpret_cast<const float4*>(w_s + ((size_t) c * qpk + i) * ATT_CH);
#pragma unroll
                        for (int p4 = 0; p4 < ATT_CH / 4; ++p4) {
                            const float4 ww = w4[p4];
                            if (4 * p4 < np) a = ffma(ww.x, vv[4 * p4], a);
                            if (4 * p4 + 1 < np) a = ffma(ww.y, vv[4 * p4 + 1], a);
                            if (4 * p4 + 2 < np) a = ffma(ww.z, vv[4 * p4 + 2], a);
                            if (4 * p4 + 3 < np) a = ffma(ww.w, vv[4 * p4 + 3], a);
                        }
                        acc[i] = a;
                    }
            };
#pragma unroll 1
            for (int c = 0; c < nck; ++c) {
                // the chunk's 32 V values of this dimension, asked for together: every load is unconditional (a chunk's missing
                // positions read its last one again; their weights are never used)
                const int np = min(ATT_CH, ng - c * ATT_CH);
                float vv[ATT_CH];
#pragma unroll
                for (int pp = 0; pp < ATT_CH; ++pp) vv[pp] = h2f(__ldg(vc + row_s[c * ATT_CH + min(pp, np - 1)] + tid));
                use(vv, c);
            }
        }
    }
    __syncthreads();
    if (tid < HD) {
#pragma unroll
        for (int i = 0; i < QM; ++i)
            if (i < qpk) acc_out[(((size_t) t * nq + kvl * qpk + i) * ATT_SPLITS + s) * HD + tid] = acc[i];
    }
    if (tid < qpk) mz_out[((size_t) t * nq + kvl * qpk + tid) * ATT_SPLITS + s] = AttPart{m_s[tid], z_s[tid]};
}

// the 16 runs of every (row t, head) as one partial: part[(t nq + h) (hd + 2)] = acc[hd], m, z.  Block = (row t, head); its
// first warp turns the runs' maxima into weights exp(m_s - max) (a run without positions is left out), z added in
// run order by one lane; then every thread adds its elements' 16 weighted accumulators in run order.
__global__ void __launch_bounds__(256) k_attn_join_runs(const float* __restrict__ acc_in, const AttPart* __restrict__ mz_in,
                                                        float* __restrict__ part, int nq, int hd) {
    __shared__ float jw[ATT_SPLITS];   // the runs' weights, negative where the run is left out
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const size_t base = ((size_t) t * nq + h) * ATT_SPLITS;
    if (tid < 32) {
        const AttPart p = lane < ATT_SPLITS ? mz_in[base + lane] : AttPart{-INFINITY, 0.f};
        const float mx = wmax(p.m);
        const float w = p.m == -INFINITY ? -1.f : ex_expf(fsub(p.m, mx));
        if (lane < ATT_SPLITS) jw[lane] = w;
        float zs = 0.f;
        for (int r = 0; r < ATT_SPLITS; ++r) {
            const float wr = __shfl_sync(0xffffffffu, w, r), zr = __shfl_sync(0xffffffffu, p.z, r);
            if (wr >= 0.f) zs = ffma(wr, zr, zs);
        }
        if (lane == 0) {
            float* o = part + ((size_t) t * nq + h) * (hd + 2);
            o[hd] = mx, o[hd + 1] = zs;
        }
    }
    __syncthreads();
    for (int i = tid; i < hd; i += 256) {
        const float* a = acc_in + base * hd + i;
        float v[ATT_SPLITS], acc = 0.f;
#pragma unroll
        for (int r = 0; r < ATT_SPLITS; ++r) v[r] = a[(size_t) r * hd];
#pragma unroll
        for (int r = 0; r < ATT_SPLITS; ++r) {
            const float w = jw[r];
            if (w >= 0.f) acc = ffma(w, v[r], acc);
        }
        part[((size_t) t * nq + h) * (hd + 2) + i] = acc;
    }
}

// the GPUs' partials of head h0 + blockIdx.x merged in ring order starting at partial `first` + 1 and ending with
// `first` (the head's owner): ((P[f+1] + P[f+2]) + ...) + P[f]; out[t][head - h0] = a / z * sigmoid(gate)
__global__ void k_attn_finish(const float* __restrict__ parts, int nparts, int first, const float* __restrict__ qg,
                              float* __restrict__ out, int nq, int h0, int hd) {
    pdl_wait();
    pdl_go();
    const int h = h0 + blockIdx.x, t = blockIdx.y, i = threadIdx.x, T = gridDim.y;
    const size_t psz = (size_t) T * nq * (hd + 2), at = ((size_t) t * nq + h) * (hd + 2);
    const float* p1 = parts + (size_t) ((first + 1) % nparts) * psz + at;
    float m = p1[hd], z = p1[hd + 1], a = p1[i];
    for (int s = 2; s <= nparts; ++s) {
        const float* p2 = parts + (size_t) ((first + s) % nparts) * psz + at;
        const float m2 = p2[hd], z2 = p2[hd + 1];
        const float mn = fmaxf(m, m2);
        const float w1 = m == -INFINITY ? 0.f : ex_expf(fsub(m, mn)), w2 = m2 == -INFINITY ? 0.f : ex_expf(fsub(m2, mn));
        z = ffma(w2, z2, fmul(w1, z));
        a = ffma(w2, p2[i], fmul(w1, a));
        m = mn;
    }
    out[((size_t) t * gridDim.x + blockIdx.x) * hd + i] = fmul(fdiv(a, z), ex_sigmoid(qg[((size_t) t * nq + h) * 2 * hd + hd + i]));
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_kv_rows_per_card(int n_ctx, int ncard) { return ((n_ctx + 3) / 4 + ncard - 1) / ncard * 4; }

int fnx_attn_prep_append(float* qg, float* k, const float* v, const float* q_norm, const float* k_norm, uint16_t* kc, uint16_t* vc,
                         FnxKvPages g, int card, int ncard, int T, const int* pos0, float eps, FnxRope rope, int nq, int nkv,
                         int hd, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "attn_prep_append: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(hd % 32 == 0 && hd >= 32 && hd <= 1024, "attn_prep_append: head dim %d", hd);
    FNX_REQUIRE(rope.nrot % 2 == 0 && rope.nrot >= 2 && rope.nrot <= 128 && rope.nrot <= hd, "attn_prep_append: rotary width %d", rope.nrot);
    FNX_REQUIRE(ncard >= 1 && card >= 0 && card < ncard, "attn_prep_append: GPU %d of %d", card, ncard);
    FNX_REQUIRE(!g.q8 || g.pt || g.cap > 0, "attn_prep_append: an int8 cache without a page table needs its row count (cap)");
    RopeFreqs rf;
    rf.nrot = rope.nrot;
    for (int i = 0; i < rope.nrot / 2; ++i) rf.f[i] = powf(rope.base, -2.0f * (float) i / (float) rope.nrot);
    launch(0, k_attn_prep_append, dim3(nq + 2 * nkv, T), hd, 0, strm(st), qg, k, v, q_norm, k_norm, kc, vc, g, card, ncard, pos0, eps, rf,
           nq, nkv, hd);
    return launch_ok("attn_prep_append");
}

size_t fnx_kvq_halves(int rows, int nkv, int hd) { return (size_t) rows * nkv * hd / 2 + (size_t) rows * nkv * hd / 32; }

size_t fnx_attn_scratch_floats(int nq, int hd, int T) {   // the larger of the exact scan's 16 splits and the fast scan's (at most 148)
    const size_t exact = (size_t) T * nq * ATT_SPLITS * (hd + 2), fast = (size_t) T * nq * 148 * (hd + 2) + (size_t) 8 * 32768;
    return exact > fast ? exact : fast;   // fast: at most 148 splits' partials, then the queries' tensor-core image (8 KV heads)
}

static int attn_partial_rows(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard, int T,
                             const int* pos0, FnxLaneRows lr, int nq, int nkv, int hd, float* scratch, void* st,
                             const int* cells = nullptr, const int* n_cells = nullptr, int maxsel = 0) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "attn: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(hd == 256 || hd == 128, "attn: head dim %d (128 or 256)", hd);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQPK, "attn: %d query heads over %d KV heads", nq, nkv);
    FNX_REQUIRE(ncard >= 1 && card >= 0 && card < ncard, "attn: GPU %d of %d", card, ncard);
    FNX_REQUIRE(!g.q8 || lr.pt || g.pt || g.cap > 0, "attn: an int8 cache without a page table needs its row count (cap)");
    float* acc = scratch;
    AttPart* mz = (AttPart*) (scratch + (size_t) T * nq * ATT_SPLITS * hd);
    const dim3 grid(ATT_SPLITS, nkv, T);   // block z = t works only when row t leads a group of rows
    auto run = [&](auto kern, int pt, int which) -> int {
        const size_t sm = ((size_t) pt * hd + (size_t) ATT_CH * (hd + 4) + (size_t) ATT_CH * hd + (size_t) pt * ATT_CH + 2 * pt) * sizeof(float);
        if (smem_optin(kern, sm, "attn partial")) return 1;
        kern<<<grid, AX_THREADS, sm, strm(st)>>>(qg, kc, vc, g, acc, mz, T, nq, nkv, pos0, card, ncard, lr, cells, n_cells, maxsel, which);
        return 0;
    };
    auto listed = [&](auto kern) -> int {   // rows with a list over an f16 cache: as many chunks a group as the longest run has, 8 at most
        const int qpk = nq / nkv, len_max = ((maxsel + ATT_SPLITS - 1) / ATT_SPLITS + ATT_CH - 1) / ATT_CH * ATT_CH;
        const int nch = len_max / ATT_CH < AX_WARPS ? len_max / ATT_CH : AX_WARPS;
        const size_t sm = (size_t) qpk * hd * 4 + (size_t) nch * ATT_CH * (hd + 8) * 2 + (size_t) nch * qpk * ATT_CH * 4 + (size_t) 3 * nch * qpk * 4 +
                          (size_t) (2 * qpk + 2) * 4 + (size_t) nch * ATT_CH * sizeof(size_t) + 16;
        if (smem_optin(kern, sm, "attn cells")) return 1;
        unsigned* fault = device_fault_word();
        if (!fault) return fail("attn cells: no fault word");
        kern<<<grid, AX_THREADS, sm, strm(st)>>>(qg, kc, vc, g, acc, mz, nq, nkv, lr, cells, n_cells, maxsel, nch, fault);
        return 0;
    };
    // rows with a list of their own go in a launch of their own; the others in groups of up to 96 pairs
    const bool small = nq / nkv <= 8;
    if (hd == 256) {
        if (run(k_attn_rows<256, AX_PT>, AX_PT, cells ? 1 : 0)) return 1;
        if (cells && g.q8 && (small ? run(k_attn_rows<256, 8>, 8, 2) : run(k_attn_rows<256, 16>, 16, 2))) return 1;
        if (cells && !g.q8 && (small ? listed(k_attn_cells<256, 8>) : listed(k_attn_cells<256, 16>))) return 1;
    } else {
        if (run(k_attn_rows<128, AX_PT>, AX_PT, cells ? 1 : 0)) return 1;
        if (cells && g.q8 && (small ? run(k_attn_rows<128, 8>, 8, 2) : run(k_attn_rows<128, 16>, 16, 2))) return 1;
        if (cells && !g.q8 && (small ? listed(k_attn_cells<128, 8>) : listed(k_attn_cells<128, 16>))) return 1;
    }
    if (launch_ok("attn partial")) return 1;
    k_attn_join_runs<<<dim3(T, nq), 256, 0, strm(st)>>>(acc, mz, part, nq, hd);
    return launch_ok("attn join");
}

int fnx_attn_partial_exact(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard, int T,
                           const int* pos0, int nq, int nkv, int hd, float* scratch, void* st) {
    return attn_partial_rows(qg, kc, vc, g, part, card, ncard, T, pos0, FnxLaneRows{nullptr, nullptr}, nq, nkv, hd, scratch, st);
}

int fnx_attn_part_lanes(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, FnxLaneRows lr, float* part, int card, int ncard,
                        int T, int nq, int nkv, int hd, float* scratch, void* st) {
    FNX_REQUIRE(lr.pos, "attn_part_lanes: no position words");
    return attn_partial_rows(qg, kc, vc, g, part, card, ncard, T, nullptr, lr, nq, nkv, hd, scratch, st);
}

int fnx_attn_partial_cells(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, FnxLaneRows lr, float* part, int card,
                           int ncard, int T, const int* pos0, int nq, int nkv, int hd, float* scratch, const int* cells, const int* n_cells,
                           int maxsel, void* st) {
    FNX_REQUIRE(lr.pos || pos0, "attn_partial_cells: no positions");
    FNX_REQUIRE(!cells || (n_cells && maxsel > 0), "attn_partial_cells: a cell list without its counts or width");
    return attn_partial_rows(qg, kc, vc, g, part, card, ncard, T, pos0, lr, nq, nkv, hd, scratch, st, cells, n_cells, maxsel);
}

int fnx_attn_finish(const float* parts, int nparts, int first_part, const float* qg, float* out, int T, int nq, int h0, int nh,
                    int hd, void* st) {
    FNX_REQUIRE(nparts >= 1 && first_part >= 0 && first_part < nparts, "attn_finish: partial %d of %d", first_part, nparts);
    FNX_REQUIRE(nh >= 1 && h0 >= 0 && h0 + nh <= nq, "attn_finish: heads [%d, %d) of %d", h0, h0 + nh, nq);
    launch(0, k_attn_finish, dim3(nh, T), hd, 0, strm(st), parts, nparts, first_part, qg, out, nq, h0, hd);
    return launch_ok("attn_finish");
}
}
