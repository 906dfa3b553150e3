// Hyper-connections of the residual streams: the write R += bo * 2 sigmoid(inj / HC) and the read (the streams mixed
// through a low-rank pair of Q8_0 matrices into one row, with the previous half's write folded in).  Replaces reference
// src/kernels.cu:1493-1503 (k_hc_write) and src/hc.cuh (k_hc); every value is rounded where the reference rounds it and
// every sum runs in its order, stated with IEEE operations, so results can be checked bit for bit.
//
// The reference's read is one launch of a block per SM with two grid-wide barriers (spins on a counter, every block
// resident, nothing else on the GPU meanwhile).  Here the three parts are three launches in stream order, each started
// while the one before still runs (programmatic dependent launch) with its weights already on their way: no kernel
// waits on another kernel's blocks, and the read can sit in a captured graph beside other streams' work.
//   down   : block (slice of 512 columns, group of 96 rows): R' for the slice, xs = R' w_norm, the slice's square sums,
//            xs as int8 per 32, the group's rows' partial dots over the slice
//   reduce : a warp per (row k, 32 rows of lo): rs per stream, lo = silu(sum of rs-weighted partials / HC) as int8 per
//            32; the inject rows
//   up     : block = 32 columns: every stream's up row . lo, the sigmoid mix, R <- R', mixed (also as q8_1)
#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"

namespace fnxk {

constexpr int HC_SL = 512, HC_RPG = 96, HC_TPR = 8, HC_DT = HC_RPG * HC_TPR, HC_MAXS = 8;   // slice; rows a group; lanes a row; streams
constexpr int HC_UPC = 32, HC_TPU = 16, HC_UT = HC_UPC * HC_TPU;                           // up: columns a block, lanes a column

struct HcArgs {
    float* R;
    const float* bo;
    const float* inj_prev;
    const float* w_norm;
    FnxQ8S down, up;
    const uint16_t* w_inj;
    float eps;
    float* mixed;
    float* inject;
    float* part;   // [ns][T][lr + hc]
    float* ssp;    // [T][ns]: the slices' square sums
    int8_t* loq;   // [T][lr]
    float* lod;    // [T][lr / 32]
    uint8_t* q8;   // mixed as q8_1 rows, or null
    int T, n, hc, lr;
};

__global__ void k_hc_write(float* __restrict__ R, const float* __restrict__ bo, const float* __restrict__ inj, int n, int hc) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n * hc) return;
    const int c = e / n, i = e % n;
    const float g = fadd(1.0f, ex_expf(fdiv(-inj[t * hc + c], (float) hc)));
    float* r = R + (size_t) t * n * hc + e;
    *r = fadd(*r, fdiv(fmul(bo[(size_t) t * n + i], 2.0f), g));
}

// a window's first residual: every stream starts as the token's embedding row
__global__ void k_hc_expand(const float* __restrict__ x, float* __restrict__ R, int n, int hc) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n * hc) R[(size_t) t * n * hc + e] = x[(size_t) t * n + e % n];
}

// R[t][c][i] = h[t][c][i] + e[t][i] (reference src/kernels.cu:2207-2212)
__global__ void k_hc_add_streams(const float* __restrict__ h, const float* __restrict__ e, float* __restrict__ R, int n, int hc) {
    pdl_wait();
    pdl_go();
    const int t = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n * hc) R[(size_t) t * n * hc + j] = fadd(h[(size_t) t * n * hc + j], e[(size_t) t * n + j % n]);
}

__device__ __forceinline__ float hc_rprime(const HcArgs& a, int t, int c, int i) {
    float r = a.R[((size_t) t * a.hc + c) * a.n + i];
    if (a.bo) r = ffma(a.bo[(size_t) t * a.n + i], fmul(2.0f, ex_sigmoid(fdiv(a.inj_prev[t * a.hc + c], (float) a.hc))), r);
    return r;
}
__device__ __forceinline__ int hc_dot8(const uint2 w, const int2 x) { return __dp4a((int) w.y, x.y, __dp4a((int) w.x, x.x, 0)); }
// rs of row k, stream c from the slices' square sums, the slices in ascending order
__device__ __forceinline__ float hc_rs(const HcArgs& a, int k, int c) {
    const int ns = a.n * a.hc / HC_SL, sps = a.n / HC_SL;
    float v = 0.f;
    for (int ss = 0; ss < sps; ++ss) v = fadd(v, a.ssp[(size_t) k * ns + c * sps + ss]);
    return ex_rsqrt(fadd(fdiv(v, (float) a.n), a.eps));
}

// dynamic shared memory: xs [T][512] f32, xq [T][512] int8, xd [T][16] f32, red [T][16] f32
__global__ void __launch_bounds__(HC_DT) k_hc_down(const HcArgs a) {
    extern __shared__ __align__(16) unsigned char hc_sm[];
    const int T = a.T, D = a.n * a.hc, rows_all = a.lr + a.hc;
    float* xs = reinterpret_cast<float*>(hc_sm);
    int8_t* xq = reinterpret_cast<int8_t*>(xs + (size_t) T * HC_SL);
    float* xd = reinterpret_cast<float*>(xq + (size_t) T * HC_SL);
    float* red = xd + (size_t) T * (HC_SL / 32);
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int s = blockIdx.x, grp = blockIdx.y, col0 = s * HC_SL, c = col0 / a.n, i0 = col0 - c * a.n;
    // this thread's weights do not depend on the kernel before: 8 lanes a row, lane j the 8-column chunks j, j + 8, ...
    constexpr int NQ = HC_SL / 8 / HC_TPR;
    const int j = t % HC_TPR, row = grp * HC_RPG + t / HC_TPR;
    const int nrows = a.w_inj ? rows_all : a.lr;
    const bool live = row < nrows;
    const int rr = live ? row : 0;
    // one register set for either kind of row: a down row's 8 chunks (two words each) and their 8 block scales, or an
    // inject row's 8 chunks of 8 bf16 (four words each)
    unsigned wr[4 * NQ];
    if (rr < a.lr) {
        const uint2* w2 = reinterpret_cast<const uint2*>(a.down.q + (size_t) rr * D + col0);
        const uint16_t* wd = a.down.d + ((size_t) rr * D + col0) / 32;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const uint2 v = __ldg(w2 + q * HC_TPR + j);
            wr[2 * q] = v.x, wr[2 * q + 1] = v.y;
            wr[2 * NQ + q] = __float_as_uint(h2f(__ldg(wd + (q * HC_TPR + j) / 4)));
        }
    } else {
        const uint4* w4 = reinterpret_cast<const uint4*>(a.w_inj + (size_t) (rr - a.lr) * D + col0);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const uint4 v = __ldg(w4 + q * HC_TPR + j);
            wr[4 * q] = v.x, wr[4 * q + 1] = v.y, wr[4 * q + 2] = v.z, wr[4 * q + 3] = v.w;
        }
    }
    pdl_wait();
    pdl_go();
    if (t < HC_SL) {
        const float wn = a.w_norm[col0 + t];
        for (int k = 0; k < T; ++k) {
            const float r = hc_rprime(a, k, c, i0 + t);
            xs[(size_t) k * HC_SL + t] = fmul(r, wn);
            if (grp == 0) {   // block-uniform; warps 0..15 hold the slice
                const float v = wsum(fmul(r, r));
                if (lane == 0) red[k * (HC_SL / 32) + warp] = v;
            }
        }
    }
    __syncthreads();
    if (grp == 0 && t < T) {
        float v = 0.f;
        for (int w = 0; w < HC_SL / 32; ++w) v = fadd(v, red[t * (HC_SL / 32) + w]);
        a.ssp[(size_t) t * (D / HC_SL) + s] = v;
    }
    for (int q = warp; q < T * (HC_SL / 32); q += HC_DT / 32) {   // a warp quantises a 32-value block: float scale amax / 127
        const int k = q / (HC_SL / 32), blk = q % (HC_SL / 32);
        const float v = xs[(size_t) k * HC_SL + blk * 32 + lane];
        const float amax = wmax(fabsf(v)), d = fdiv(amax, 127.0f);
        xq[(size_t) k * HC_SL + blk * 32 + lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(v, d));
        if (lane == 0) xd[k * (HC_SL / 32) + blk] = d;
    }
    __syncthreads();
    const int ns = D / HC_SL;
    (void) ns;
#pragma unroll 1
    for (int k = 0; k < T; ++k) {
        float acc = 0.f;
        if (rr < a.lr) {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const int ch = q * HC_TPR + j;
                acc = ffma(fmul(__uint_as_float(wr[2 * NQ + q]), xd[k * (HC_SL / 32) + ch / 4]),
                           (float) hc_dot8(make_uint2(wr[2 * q], wr[2 * q + 1]), *reinterpret_cast<const int2*>(xq + (size_t) k * HC_SL + ch * 8)), acc);
            }
        } else {
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const int ch = q * HC_TPR + j;
                const unsigned w[4] = {wr[4 * q], wr[4 * q + 1], wr[4 * q + 2], wr[4 * q + 3]};
                const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t) k * HC_SL + ch * 8);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t) k * HC_SL + ch * 8 + 4);
                const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                float t8 = fmul(__uint_as_float(w[0] << 16), xv[0]);
#pragma unroll
                for (int e = 1; e < 8; ++e) t8 = ffma(__uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16)), xv[e], t8);
                acc = fadd(acc, t8);
            }
        }
        for (int o = 1; o < HC_TPR; o <<= 1) acc = fadd(acc, __shfl_xor_sync(0xffffffffu, acc, o));
        if (live && j == 0) a.part[((size_t) s * T + k) * rows_all + row] = acc;
    }
}

// a warp per item: (row k, block b of lo) for the first T * lr / 32 items, then row k's inject rows
__global__ void __launch_bounds__(256) k_hc_reduce(const HcArgs a) {
    pdl_wait();
    pdl_go();
    const int T = a.T, nb = a.lr / 32, rows_all = a.lr + a.hc, sps = a.n / HC_SL;
    const int it = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (it >= T * nb + T) return;
    const bool inj_item = it >= T * nb;
    const int k = inj_item ? it - T * nb : it / nb;
    const bool active = !inj_item || (a.w_inj && lane < a.hc);
    const int r = !active ? 0 : inj_item ? a.lr + lane : (it % nb) * 32 + lane;
    float sum = 0.f;
    for (int cc = 0; cc < a.hc; ++cc) {
        float p = 0.f;
        for (int ss = 0; ss < sps; ++ss) p = fadd(p, a.part[((size_t) (cc * sps + ss) * T + k) * rows_all + r]);
        sum = ffma(hc_rs(a, k, cc), p, sum);
    }
    if (inj_item) {
        if (active) a.inject[k * a.hc + lane] = sum;
        return;
    }
    const float v = ex_silu(fdiv(sum, (float) a.hc));
    const float amax = wmax(fabsf(v)), d = fdiv(amax, 127.0f);
    a.loq[(size_t) k * a.lr + r] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(v, d));
    if (lane == 0) a.lod[k * nb + r / 32] = d;
}

// dynamic shared memory: lq [T][lr] int8, ld [T][lr / 32], rs [T][hc], ms [T][32], gs [T][hc][32]
__global__ void __launch_bounds__(HC_UT) k_hc_up(const HcArgs a) {
    extern __shared__ __align__(16) unsigned char hc_sm[];
    const int T = a.T, nb = a.lr / 32, hc = a.hc;
    int8_t* lq = reinterpret_cast<int8_t*>(hc_sm);
    float* ld = reinterpret_cast<float*>(lq + (size_t) T * a.lr);
    float* rs = ld + (size_t) T * nb;
    float* ms = rs + (size_t) T * hc;
    float* gs = ms + (size_t) T * HC_UPC;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, b = blockIdx.x;
    const int uj = t % HC_TPU, udd = t / HC_TPU;
    const bool ulive = uj < nb;
    // this lane's block of each stream's up row: asked for while the reduction still runs
    uint4 wq[HC_MAXS][2];
    float wsc[HC_MAXS];
#pragma unroll
    for (int cc = 0; cc < HC_MAXS; ++cc) {
        wq[cc][0] = wq[cc][1] = make_uint4(0, 0, 0, 0);
        wsc[cc] = 0.f;
        if (cc < hc && ulive) {
            const size_t urow = (size_t) cc * a.n + (size_t) b * HC_UPC + udd;
            const uint4* wp = reinterpret_cast<const uint4*>(a.up.q + urow * a.lr + uj * 32);
            wq[cc][0] = __ldg(wp);
            wq[cc][1] = __ldg(wp + 1);
            wsc[cc] = h2f(__ldg(a.up.d + urow * nb + uj));
        }
    }
    pdl_wait();
    pdl_go();
    if (t < T * hc) rs[t] = hc_rs(a, t / hc, t % hc);
    for (int e = t; e < T * a.lr / 4; e += HC_UT) reinterpret_cast<int*>(lq)[e] = reinterpret_cast<const int*>(a.loq)[e];
    for (int e = t; e < T * nb; e += HC_UT) ld[e] = a.lod[e];
    __syncthreads();
#pragma unroll 1
    for (int k = 0; k < T; ++k) {
        const int4* xp = reinterpret_cast<const int4*>(lq + (size_t) k * a.lr + (ulive ? uj : 0) * 32);
        const int4 x0 = xp[0], x1 = xp[1];
        const float dl = ld[k * nb + (ulive ? uj : 0)];
#pragma unroll
        for (int cc = 0; cc < HC_MAXS; ++cc) {
            if (cc >= hc) break;
            const uint4 w0 = wq[cc][0], w1 = wq[cc][1];
            int sacc = __dp4a((int) w0.x, x0.x, 0);
            sacc = __dp4a((int) w0.y, x0.y, sacc);
            sacc = __dp4a((int) w0.z, x0.z, sacc);
            sacc = __dp4a((int) w0.w, x0.w, sacc);
            sacc = __dp4a((int) w1.x, x1.x, sacc);
            sacc = __dp4a((int) w1.y, x1.y, sacc);
            sacc = __dp4a((int) w1.z, x1.z, sacc);
            sacc = __dp4a((int) w1.w, x1.w, sacc);
            float acc = fmul(fmul(wsc[cc], dl), (float) sacc);   // an idle lane: 0 * dl * 0
            for (int o = 1; o < HC_TPU; o <<= 1) acc = fadd(acc, __shfl_xor_sync(0xffffffffu, acc, o));
            if (uj == 0) gs[((size_t) k * hc + cc) * HC_UPC + udd] = acc;
        }
    }
    __syncthreads();
    for (int e = t; e < T * hc * HC_UPC; e += HC_UT) {
        const int col = e % HC_UPC, cc = (e / HC_UPC) % hc, k = e / (HC_UPC * hc), dc = b * HC_UPC + col;
        const float rv = hc_rprime(a, k, cc, dc);
        if (a.bo) a.R[((size_t) k * hc + cc) * a.n + dc] = rv;
        gs[e] = fmul(ex_sigmoid(gs[e]), fmul(fmul(rv, a.w_norm[cc * a.n + dc]), rs[k * hc + cc]));
    }
    __syncthreads();
    for (int e = t; e < T * HC_UPC; e += HC_UT) {
        const int col = e % HC_UPC, k = e / HC_UPC;
        float sum = gs[((size_t) k * hc) * HC_UPC + col];
        for (int cc = 1; cc < hc; ++cc) sum = fadd(sum, gs[((size_t) k * hc + cc) * HC_UPC + col]);
        sum = fdiv(sum, (float) hc);
        a.mixed[(size_t) k * a.n + b * HC_UPC + col] = sum;
        ms[e] = sum;
    }
    if (!a.q8) return;
    __syncthreads();
    if (warp < T) {   // the block's 32 columns are one q8_1 block of every row
        const float xi = ms[warp * HC_UPC + lane];
        const float amax = wmax(fabsf(xi)), sm = wsum(xi);
        const float dq = fdiv(amax, 127.0f);
        uint8_t* blk = a.q8 + ((size_t) warp * (a.n / 32) + b) * 36;
        reinterpret_cast<int8_t*>(blk + 4)[lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, dq));
        if (lane == 0) {
            reinterpret_cast<uint16_t*>(blk)[0] = f2h(dq);
            reinterpret_cast<uint16_t*>(blk)[1] = f2h(sm);
        }
    }
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_hc_write(float* R, const float* bo, const float* inj, int T, int n, int hc, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && n >= 1 && hc >= 1, "hc_write: %d rows, %d streams of %d", T, hc, n);
    launch(0, k_hc_write, dim3((n * hc + 255) / 256, T), 256, 0, strm(st), R, bo, inj, n, hc);
    return launch_ok("hc_write");
}

int fnx_hc_expand(const float* x, float* R, int T, int n, int hc, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && n >= 1 && hc >= 1, "hc_expand: %d rows, %d streams of %d", T, hc, n);
    launch(0, k_hc_expand, dim3((n * hc + 255) / 256, T), 256, 0, strm(st), x, R, n, hc);
    return launch_ok("hc_expand");
}

int fnx_hc_add_streams(const float* h, const float* e, float* R, int T, int n, int hc, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && n >= 1 && hc >= 1, "hc_add_streams: %d rows, %d streams of %d", T, hc, n);
    launch(0, k_hc_add_streams, dim3((n * hc + 255) / 256, T), 256, 0, strm(st), h, e, R, n, hc);
    return launch_ok("hc_add_streams");
}

size_t fnx_hc_scratch_floats(int T, int n, int hc, int lr) {
    const size_t ns = (size_t) n * hc / HC_SL;
    return ns * T * (lr + hc) + (size_t) T * ns + (size_t) T * lr / 4 + (size_t) T * (lr / 32) + 16;
}

int fnx_hc_read(float* R, const float* bo_prev, const float* inj_prev, const float* w_norm, FnxQ8S w_down, FnxQ8S w_up, const uint16_t* w_inj,
                float eps, float* mixed, float* inject, float* scratch, void* q8, int T, int n, int hc, int lr, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "hc_read: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(n >= HC_SL && n % HC_SL == 0 && hc >= 1 && hc <= HC_MAXS, "hc_read: %d streams of %d (a multiple of %d, at most %d streams)", hc, n,
                HC_SL, HC_MAXS);
    FNX_REQUIRE(lr >= 32 && lr % 32 == 0 && lr / 32 <= HC_TPU, "hc_read: low rank %d (a multiple of 32 up to %d)", lr, 32 * HC_TPU);
    FNX_REQUIRE(hc <= 32 && (!bo_prev || inj_prev) && (!w_inj || inject), "hc_read: a folded write needs inj_prev, inject rows their output");
    FNX_REQUIRE(((uintptr_t) w_down.q % 16) == 0 && ((uintptr_t) w_up.q % 16) == 0 && (!w_inj || ((uintptr_t) w_inj % 16) == 0) &&
                    ((uintptr_t) scratch % 16) == 0,
                "hc_read: weights and scratch must be 16-byte aligned");
    const size_t ns = (size_t) n * hc / HC_SL;
    HcArgs a{R, bo_prev, inj_prev, w_norm, w_down, w_up, w_inj, eps, mixed, inject, nullptr, nullptr, nullptr, nullptr, (uint8_t*) q8, T, n, hc, lr};
    a.part = scratch;
    a.ssp = a.part + ns * T * (lr + hc);
    a.loq = (int8_t*) (a.ssp + (size_t) T * ns);
    a.lod = a.ssp + (size_t) T * ns + (size_t) T * lr / 4;
    const int rg = (lr + hc + HC_RPG - 1) / HC_RPG;
    const size_t sm1 = (size_t) T * HC_SL * 4 + (size_t) T * HC_SL + (size_t) 2 * T * (HC_SL / 32) * 4;
    if (smem_optin(k_hc_down, sm1, "hc_read down")) return 1;
    launch(0, k_hc_down, dim3((unsigned) ns, rg), HC_DT, sm1, strm(st), a);
    if (launch_ok("hc_read down")) return 1;
    launch(0, k_hc_reduce, (T * (lr / 32) + T + 7) / 8, 256, 0, strm(st), a);
    if (launch_ok("hc_read reduce")) return 1;
    const size_t sm3 = (size_t) T * lr + ((size_t) T * (lr / 32) + (size_t) T * hc + (size_t) T * HC_UPC + (size_t) T * hc * HC_UPC) * 4;
    if (smem_optin(k_hc_up, sm3, "hc_read up")) return 1;
    launch(0, k_hc_up, n / HC_UPC, HC_UT, sm3, strm(st), a);
    return launch_ok("hc_read up");
}
}
