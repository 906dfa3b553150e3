// Position-split attention of the verify window: per-head RMS norm + NEOX rotary + K/V append, the split-K
// online-softmax scan over the positions this GPU owns, the merge of the splits, and the merge of the GPUs' partials
// with the output gate.  Replaces reference src/kernels.cu:451-469, 480-691, 1539-1569.
//
// K/V placement (reference src/kernels.hpp:126-130): blocks of 4 positions are dealt round-robin, block j on GPU
// j % ncard at local block j / ncard; local row = local block * 4 + p % 4.
#include <cmath>

#include "common.cuh"
#include "exact_math.cuh"

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
    (is_k ? kc : vc)[kv_row_at(g, r, nkv, hd) + e] = f2h(x);
}

// ---------------------------------------------------------------- exact split-K scan (the reference's order of sums)
// block (split s, row t, KV head kvl), hd threads: positions [s len, (s + 1) len) of the row's owned positions in
// chunks of 32; thread i holds dimension i of the chunk's V rows and of every local head's accumulator; warp w scores
// head w (lane = position) and takes its online-softmax step.  scratch: acc [T][nq][16][hd], then (m, z) [T][nq][16].
struct AttPart {
    float m, z;
};

template <int HD>
__global__ void __launch_bounds__(HD) k_attn_part(const float* __restrict__ qg, const uint16_t* __restrict__ kc,
                                                  const uint16_t* __restrict__ vc, FnxKvPages g, float* __restrict__ acc_out,
                                                  AttPart* __restrict__ mz_out, int nq, int nkv, const int* __restrict__ pos0p, int card,
                                                  int ncard, FnxLaneRows lr) {
    const int s = blockIdx.x, t = blockIdx.y, kvl = blockIdx.z, i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const int qpk = nq / nkv, h0 = kvl * qpk;
    // a row of a lane of its own: the lane's position word and page table (reference src/kernels.hpp:189-193)
    if (lr.pt) g.pt = lr.pt[t];
    const int ctx = kv_owned(lr.pos ? *lr.pos[t] : *pos0p + t, card, ncard);
    const int len = ((ctx + ATT_SPLITS - 1) / ATT_SPLITS + ATT_CH - 1) / ATT_CH * ATT_CH;
    const int p0 = s * len, p1 = min(ctx, p0 + len);
    extern __shared__ __align__(16) float att_sm[];
    float* q = att_sm;                                  // [qpk][HD]
    float* kk = q + (size_t) qpk * HD;                  // [32][HD + 1]
    float* e = kk + (size_t) ATT_CH * (HD + 1);         // [qpk][32]
    float* scale = e + (size_t) qpk * ATT_CH;           // [qpk]
    for (int k = i; k < qpk * HD; k += HD) q[k] = qg[((size_t) t * nq + h0 + k / HD) * 2 * HD + k % HD];
    constexpr int NW = HD / 32, HPW = (ATT_MAXQPK + NW - 1) / NW;
    float m[HPW], z[HPW];
#pragma unroll
    for (int k = 0; k < HPW; ++k) m[k] = -INFINITY, z[k] = 0.f;
    float acc[ATT_MAXQPK];
#pragma unroll
    for (int hh = 0; hh < ATT_MAXQPK; ++hh) acc[hh] = 0.f;
    const float rs = ex_rsqrt((float) HD);
    __syncthreads();
#pragma unroll 1
    for (int c0 = p0; c0 < p1; c0 += ATT_CH) {
        const int np = min(ATT_CH, p1 - c0);
        float vr[ATT_CH];
#pragma unroll
        for (int pp = 0; pp < ATT_CH; ++pp) {
            const size_t r = kv_row_at(g, pp < np ? c0 + pp : 0, nkv, HD) + (size_t) kvl * HD + i;
            kk[pp * (HD + 1) + i] = pp < np ? h2f(kc[r]) : 0.f;
            vr[pp] = pp < np ? h2f(vc[r]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HPW; ++k) {
            const int hh = warp + k * NW;
            if (hh >= qpk) break;
            float sacc = 0.f;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) sacc = ffma(q[hh * HD + d], kk[lane * (HD + 1) + d], sacc);
            const float sv = lane < np ? fmul(sacc, rs) : -INFINITY;
            const float mn = fmaxf(m[k], wmax(sv));
            const float w = sv == -INFINITY ? 0.f : ex_expf(fsub(sv, mn));
            const float sc = m[k] == -INFINITY ? 0.f : ex_expf(fsub(m[k], mn));
            z[k] = ffma(z[k], sc, wsum(w));
            m[k] = mn;
            e[hh * ATT_CH + lane] = w;
            if (lane == 0) scale[hh] = sc;
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < ATT_MAXQPK; ++hh)
            if (hh < qpk) acc[hh] = fmul(acc[hh], scale[hh]);
#pragma unroll
        for (int pp = 0; pp < ATT_CH; ++pp)
#pragma unroll
            for (int hh = 0; hh < ATT_MAXQPK; ++hh)
                if (hh < qpk) acc[hh] = ffma(e[hh * ATT_CH + pp], vr[pp], acc[hh]);
        __syncthreads();
    }
#pragma unroll
    for (int hh = 0; hh < ATT_MAXQPK; ++hh) {
        if (hh >= qpk) break;
        acc_out[(((size_t) t * nq + h0 + hh) * ATT_SPLITS + s) * HD + i] = acc[hh];
    }
#pragma unroll
    for (int k = 0; k < HPW; ++k) {
        const int hh = warp + k * NW;
        if (hh < qpk && lane == 0) mz_out[((size_t) t * nq + h0 + hh) * ATT_SPLITS + s] = AttPart{m[k], z[k]};
    }
}

// the 16 splits of (row t, head h) as one partial: part[(t nq + h) (hd + 2)] = acc[hd], m, z
__global__ void k_attn_local(const float* __restrict__ acc_in, const AttPart* __restrict__ mz_in, float* __restrict__ part, int nq,
                             int hd) {
    const int h = blockIdx.x, t = blockIdx.y, i = threadIdx.x;
    const size_t base = ((size_t) t * nq + h) * ATT_SPLITS;
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < ATT_SPLITS; ++s) mx = fmaxf(mx, mz_in[base + s].m);
    float z = 0.f, acc = 0.f;
#pragma unroll
    for (int s = 0; s < ATT_SPLITS; ++s) {
        const AttPart p = mz_in[base + s];
        if (p.m == -INFINITY) continue;
        const float w = ex_expf(fsub(p.m, mx));
        z = ffma(w, p.z, z);
        acc = ffma(w, acc_in[(base + s) * hd + i], acc);
    }
    float* o = part + ((size_t) t * nq + h) * (hd + 2);
    o[i] = acc;
    if (i == 0) o[hd] = mx, o[hd + 1] = z;
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
    RopeFreqs rf;
    rf.nrot = rope.nrot;
    for (int i = 0; i < rope.nrot / 2; ++i) rf.f[i] = powf(rope.base, -2.0f * (float) i / (float) rope.nrot);
    launch(0, k_attn_prep_append, dim3(nq + 2 * nkv, T), hd, 0, strm(st), qg, k, v, q_norm, k_norm, kc, vc, g, card, ncard, pos0, eps, rf,
           nq, nkv, hd);
    return launch_ok("attn_prep_append");
}

size_t fnx_attn_scratch_floats(int nq, int hd, int T) {   // the larger of the exact scan's 16 splits and the fast scan's (at most 148)
    const size_t exact = (size_t) T * nq * ATT_SPLITS * (hd + 2), fast = (size_t) T * nq * 148 * (hd + 2) + (size_t) 8 * 32768;
    return exact > fast ? exact : fast;   // fast: at most 148 splits' partials, then the queries' tensor-core image (8 KV heads)
}

static int attn_partial_rows(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard, int T,
                             const int* pos0, FnxLaneRows lr, int nq, int nkv, int hd, float* scratch, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "attn: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(hd == 256 || hd == 128, "attn: head dim %d (128 or 256)", hd);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQPK, "attn: %d query heads over %d KV heads", nq, nkv);
    FNX_REQUIRE(ncard >= 1 && card >= 0 && card < ncard, "attn: GPU %d of %d", card, ncard);
    const int qpk = nq / nkv;
    float* acc = scratch;
    AttPart* mz = (AttPart*) (scratch + (size_t) T * nq * ATT_SPLITS * hd);
    const size_t sm = ((size_t) qpk * hd + (size_t) ATT_CH * (hd + 1) + (size_t) qpk * ATT_CH + qpk) * sizeof(float);
    const dim3 grid(ATT_SPLITS, T, nkv);
    if (hd == 256) {
        if (sm > 48 * 1024) cudaFuncSetAttribute(k_attn_part<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm);
        k_attn_part<256><<<grid, 256, sm, strm(st)>>>(qg, kc, vc, g, acc, mz, nq, nkv, pos0, card, ncard, lr);
    } else {
        if (sm > 48 * 1024) cudaFuncSetAttribute(k_attn_part<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm);
        k_attn_part<128><<<grid, 128, sm, strm(st)>>>(qg, kc, vc, g, acc, mz, nq, nkv, pos0, card, ncard, lr);
    }
    if (launch_ok("attn partial")) return 1;
    k_attn_local<<<dim3(nq, T), hd, 0, strm(st)>>>(acc, mz, part, nq, hd);
    return launch_ok("attn local");
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

int fnx_attn_finish(const float* parts, int nparts, int first_part, const float* qg, float* out, int T, int nq, int h0, int nh,
                    int hd, void* st) {
    FNX_REQUIRE(nparts >= 1 && first_part >= 0 && first_part < nparts, "attn_finish: partial %d of %d", first_part, nparts);
    FNX_REQUIRE(nh >= 1 && h0 >= 0 && h0 + nh <= nq, "attn_finish: heads [%d, %d) of %d", h0, h0 + nh, nq);
    launch(0, k_attn_finish, dim3(nh, T), hd, 0, strm(st), parts, nparts, first_part, qg, out, nq, h0, hd);
    return launch_ok("attn_finish");
}
}
