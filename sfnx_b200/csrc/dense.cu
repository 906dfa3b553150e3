// Dense projections of the verify window: split-layout Q8_0 matrix x up to 16 quantised activation rows (output head,
// qkvz, wq/wk/wv/wo, ssm_out, the shared expert), and the small f32 GEMV (alpha/beta).  Replaces reference
// src/dense.cuh and src/kernels.cu:184-227 with the same order of every sum: a lane takes 16 columns at
// c = 16 lane + 512 k, acc = fma(dw da, (float) isum16, acc) in ascending k, lanes combined by xor 16..1.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int Q8S_THREADS = 256, Q8S_R = 4;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// activations into shared memory as an int8 plane [T][cols] and float scales [T][cols / 32]: from q8_1 rows (yq), or
// from planes already in that form (pq, pd)
__device__ __forceinline__ void stage_act(int8_t* sq, float* sd, const uint8_t* __restrict__ yq, const int8_t* __restrict__ pq,
                                          const float* __restrict__ pd, int T, int cols) {
    const int nb = cols / 32;
    if (yq) {
        for (int it = threadIdx.x; it < T * nb; it += blockDim.x) {
            const unsigned* src = reinterpret_cast<const unsigned*>(yq + (size_t) it * 36);
            unsigned w[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) w[k] = src[k];
            uint4* dst = reinterpret_cast<uint4*>(sq + (size_t) it * 32);
            dst[0] = make_uint4(w[1], w[2], w[3], w[4]);
            dst[1] = make_uint4(w[5], w[6], w[7], w[8]);
            sd[it] = h2f((uint16_t) (w[0] & 0xffff));
        }
    } else {
        for (int it = threadIdx.x; it < T * cols / 16; it += blockDim.x)
            reinterpret_cast<uint4*>(sq)[it] = reinterpret_cast<const uint4*>(pq)[it];
        for (int it = threadIdx.x; it < T * nb; it += blockDim.x) sd[it] = pd[it];
    }
}

// rows [row0, row0 + Q8S_R) of one warp against the staged activations; out[t * out_stride + row]
template <int TT>
__device__ __forceinline__ void q8s_rows(const int8_t* __restrict__ wq, const uint16_t* __restrict__ wd, int rows, int cols, int row0,
                                         const int8_t* sq, const float* sd, int T, float* __restrict__ out, int out_stride) {
    const int lane = threadIdx.x & 31, nb = cols / 32;
    float acc[Q8S_R][TT];
#pragma unroll
    for (int r = 0; r < Q8S_R; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) acc[r][t] = 0.f;
#pragma unroll 2
    for (int c = lane * 16; c < cols; c += 512) {
        const int b = c >> 5;
        uint4 w[Q8S_R];
        float dw[Q8S_R];
#pragma unroll
        for (int r = 0; r < Q8S_R; ++r) {
            const size_t row = (size_t) min(row0 + r, rows - 1);
            w[r] = ldg_stream16(wq + row * cols + c);
            dw[r] = h2f(__ldg(wd + row * nb + b));
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (t >= T) break;
            const uint4 a = *reinterpret_cast<const uint4*>(sq + (size_t) t * cols + c);
            const float da = sd[t * nb + b];
#pragma unroll
            for (int r = 0; r < Q8S_R; ++r) {
                int s = __dp4a((int) w[r].x, (int) a.x, 0);
                s = __dp4a((int) w[r].y, (int) a.y, s);
                s = __dp4a((int) w[r].z, (int) a.z, s);
                s = __dp4a((int) w[r].w, (int) a.w, s);
                acc[r][t] = ffma(fmul(dw[r], da), (float) s, acc[r][t]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < Q8S_R; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (t >= T) break;
            const float v = wsum(acc[r][t]);
            if (lane == 0 && row0 + r < rows) out[(size_t) t * out_stride + row0 + r] = v;
        }
}

template <int TT>
__global__ void __launch_bounds__(Q8S_THREADS, 2) k_q8s(const int8_t* __restrict__ wq, const uint16_t* __restrict__ wd, int rows, int cols,
                                                    const uint8_t* __restrict__ yq, const int8_t* __restrict__ pq,
                                                    const float* __restrict__ pd, int T, float* __restrict__ out, int out_stride,
                                                    int rows_per_block) {
    extern __shared__ __align__(16) unsigned char smem[];
    int8_t* sq = reinterpret_cast<int8_t*>(smem);
    float* sd = reinterpret_cast<float*>(smem + (size_t) T * cols);
    stage_act(sq, sd, yq, pq, pd, T, cols);
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    const int base = blockIdx.x * rows_per_block;
    for (int r0 = warp * Q8S_R; r0 < rows_per_block; r0 += (Q8S_THREADS / 32) * Q8S_R) {
        if (base + r0 >= rows) break;
        q8s_rows<TT>(wq, wd, rows, cols, base + r0, sq, sd, T, out, out_stride);
    }
}

// ---------------------------------------------------------------- the same sums on the tensor cores
// A row's result is the xor-tree over 32 "lanes" of per-lane sums, lane l adding the scaled integer dots of the 16-column
// pieces at c = 16 l + 512 k in ascending k.  Here a 16-column piece of 16 weight rows against up to 16 activation rows
// is one (or two) mma.sync m16n8k16 s8 x s8 -> s32, exact; the scaling by fl(dw da) and the per-lane f32 sums are done on
// the accumulator fragments in the same order, so the result has the same bits as the dp4a kernel's.  Warp w owns lanes
// 4 w .. 4 w + 3 (64 contiguous columns of every 512), for two 16-row tiles; the 32 lane sums of every output meet in
// shared memory for the tree.  The integer accumulator starts at the bits of 1.5 * 2^23, so reinterpreting it as f32
// and subtracting that constant converts it without a convert instruction (|dot| < 2^22).
constexpr int QM_THREADS = 256, QM_MT = 2, QM_ROWS = 16 * QM_MT, QM_APAD = 16;
constexpr int QM_MAGIC = 0x4B400000, QM_RING_LD = 80;

__device__ __forceinline__ void mma_s8_16816(int (&d)[4], unsigned a0, unsigned a1, unsigned b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(QM_MAGIC));
}
// two f32 in a 64-bit register, each half rounded as its scalar operation would be (Blackwell's packed f32 pipe): the
// scaling and adding of the accumulator fragments takes half the instructions and keeps every bit
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 pack2i(int lo, int hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned ldg_u32(const void* p) {
    unsigned v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// up to three matrices of the same width over the same activations in one launch (reference src/dense.cuh:8-19): the
// blocks of segment s follow those of segment s - 1
struct QSegs {
    const int8_t* q[3];
    const uint16_t* d[3];
    float* out[3];
    int stride[3], rows[3], blk_end[3];
};

// ---------------------------------------------------------------- the same sums, weights streamed by persistent blocks
// One block of 16 warps per multiprocessor stages the activations once and walks row tiles (16 MT rows) until the
// matrix is done.  With WPT = 8 the block is two groups of 8 warps on tiles of their own (their only shared state is
// the activations); with WPT = 16 (wide matrices, whose activations leave less room) one group.  Warp w of a group owns
// the 32-column pieces at 32 w and (WPT = 8) 256 + 32 w of every 512 columns, i.e. lanes 2 w, 2 w + 1 and their
// partners 16 up in the row's xor tree, so the tree's first level is an add inside the warp and 16 lane sums per
// output meet in shared memory instead of 32.  A warp's pieces of the tile (full 32-byte sectors, with the f16 block
// scales as 4-byte words beside them) flow through a cp.async ring of QS_S stages that runs on across tiles, so a
// multiprocessor always has about two steps of every warp in flight.
constexpr int QS_THREADS = 512, QS_S = 3;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned) __cvta_generic_to_shared(dst)), "l"(src));
}

struct QTile {   // what a tile index means: its matrix, first row and output
    const int8_t* wq;
    const uint16_t* wd;
    int rows, row0;
};
__device__ __forceinline__ QTile q_tile(const QSegs& sg, int tile, int tile_rows) {
    const int seg = tile < sg.blk_end[0] ? 0 : tile < sg.blk_end[1] ? 1 : 2;
    QTile t;
    t.wq = seg == 0 ? sg.q[0] : seg == 1 ? sg.q[1] : sg.q[2];
    t.wd = seg == 0 ? sg.d[0] : seg == 1 ? sg.d[1] : sg.d[2];
    t.rows = seg == 0 ? sg.rows[0] : seg == 1 ? sg.rows[1] : sg.rows[2];
    t.row0 = (tile - (seg == 0 ? 0 : seg == 1 ? sg.blk_end[0] : sg.blk_end[1])) * tile_rows;
    return t;
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

template <int NT, int MT, int WPT>
__global__ void __launch_bounds__(QS_THREADS, 1) k_q8s_stream(const QSegs sg, int cols, const uint8_t* __restrict__ yq,
                                                             const int8_t* __restrict__ pq, const float* __restrict__ pd, int T, int ntiles,
                                                             unsigned ring_off, unsigned red_off) {
    constexpr int G = 16 / WPT, NP = 16 / WPT, CW = 32 * NP, RL = CW + 16, ROWS = 16 * MT, TO = 8 * NT, NL = WPT == 8 ? 16 : 32;
    constexpr int NPC = MT * NP, NSC = (ROWS * NP + 31) / 32;   // 16-byte pieces and scale words a lane copies per step
    extern __shared__ __align__(16) unsigned char smem[];
    const int nb = cols / 32, lda = cols + QM_APAD, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane & 3, r8 = lane >> 2;
    const int g = warp / WPT, wg = warp % WPT, gtid = tid - g * WPT * 32, par = wg & 1, nsteps = (cols + 511) / 512;
    int8_t* sq = reinterpret_cast<int8_t*>(smem);                          // [8 NT][cols + pad], rows >= T zero
    float* sd = reinterpret_cast<float*>(smem + (size_t) 8 * NT * lda);    // [nb][4][NT][2]: block, lane % 4, 8-row tile, row pair
    unsigned char* ringw = smem + ring_off + (size_t) warp * QS_S * ROWS * RL;
    float* red = reinterpret_cast<float*>(smem + red_off) + (size_t) g * NL * 16 * TO;   // [NL][16 rows][TO], a 16-row pass at a time
    const int gstride = gridDim.x * G;
    // ---- the copies run ahead of the sums by QS_S - 1 steps, across tile boundaries; a lane's pieces of a step sit at
    // fixed offsets from the tile's first row, computed when the tile changes, and at fixed places of a ring stage
    constexpr unsigned STAGE = ROWS * RL;
    const unsigned ring_s0 = (unsigned) __cvta_generic_to_shared(ringw);
    const bool whole = cols % 512 == 0;   // every piece of every step exists
    int pf_tile = blockIdx.x * G + g, pf_k = 0;
    unsigned pf_stage = ring_s0;
    const int8_t* pf_q = nullptr;      // the tile's matrix, advanced by the step
    const uint16_t* pf_d = nullptr;
    unsigned poff[NPC], soff[NSC], pdst[NPC], sdst[NSC];
#pragma unroll
    for (int i = 0; i < NPC; ++i) {
        const int j = lane + 32 * i, row = j / (2 * NP), p16 = j % (2 * NP);
        pdst[i] = row * RL + 16 * p16;
    }
#pragma unroll
    for (int i = 0; i < NSC; ++i) {
        const int j = min(lane + 32 * i, ROWS * NP - 1), row = j / NP, pi = j % NP;
        sdst[i] = row * RL + CW + 4 * pi;
    }
    auto pf_set = [&]() {
        const QTile t = q_tile(sg, pf_tile, ROWS);
        pf_q = t.wq, pf_d = t.wd;
#pragma unroll
        for (int i = 0; i < NPC; ++i) {
            const int j = lane + 32 * i, row = j / (2 * NP), p16 = j % (2 * NP);
            poff[i] = (unsigned) min(t.row0 + row, t.rows - 1) * (unsigned) cols + 32 * wg + 256 * (p16 >> 1) + 16 * (p16 & 1);
        }
#pragma unroll
        for (int i = 0; i < NSC; ++i) {
            const int j = min(lane + 32 * i, ROWS * NP - 1), row = j / NP, pi = j % NP;
            soff[i] = (unsigned) min(t.row0 + row, t.rows - 1) * (unsigned) nb + ((wg + 8 * pi) & ~1);
        }
    };
    if (pf_tile < ntiles) pf_set();
    auto issue = [&]() {
        if (pf_tile < ntiles) {
#pragma unroll
            for (int i = 0; i < NPC; ++i)   // 16-byte pieces: 2 NP a row
                if (whole || 512 * pf_k + 32 * wg + 256 * (((lane + 32 * i) % (2 * NP)) >> 1) < cols)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pf_stage + pdst[i]), "l"(pf_q + poff[i]));
#pragma unroll
            for (int i = 0; i < NSC; ++i)   // the pieces' block scales: the aligned f16 pair that holds each
                if (lane + 32 * i < ROWS * NP && (whole || 512 * pf_k + 32 * wg + 256 * ((lane + 32 * i) % NP) < cols))
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(pf_stage + sdst[i]), "l"(pf_d + soff[i]));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        pf_stage = pf_stage + STAGE == ring_s0 + QS_S * STAGE ? ring_s0 : pf_stage + STAGE;
        pf_q += 512, pf_d += 16;
        if (++pf_k == nsteps) {
            pf_k = 0, pf_tile += gstride;
            if (pf_tile < ntiles) pf_set();
        }
    };
#pragma unroll
    for (int i = 0; i < QS_S - 1; ++i) issue();   // the weights wait neither for the activations nor for the kernel that makes them
    pdl_wait();
    pdl_go();
    for (int it = tid; it < 8 * NT * nb; it += QS_THREADS) {
        const int t = it / nb, b = it % nb;
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        float d = 0.f;
        if (t < T) {
            if (yq) {
                const unsigned* src = reinterpret_cast<const unsigned*>(yq + (size_t) it * 36);
                d = h2f((uint16_t) (src[0] & 0xffff));
                v0 = make_uint4(src[1], src[2], src[3], src[4]);
                v1 = make_uint4(src[5], src[6], src[7], src[8]);
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(pq + (size_t) t * cols + b * 32);
                v0 = src[0], v1 = src[1];
                d = pd[it];
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(sq + (size_t) t * lda + b * 32);
        dst[0] = v0, dst[1] = v1;
        sd[((b * 4 + ((t & 7) >> 1)) * NT + (t >> 3)) * 2 + (t & 1)] = d;
    }
    __syncthreads();
    const f32x2 unmagic = pack2(-12582912.0f, -12582912.0f);
    // ldmatrix row addresses of this lane: 8 x 16-byte matrices; lanes 8 m .. 8 m + 7 give matrix m's rows
    const unsigned a_lane = (unsigned) ((8 * ((lane >> 3) & 1) + (lane & 7)) * RL + 16 * (lane >> 4));   // rows 0-7 | 8-15, then 16 columns on
    const unsigned b_lane = NT == 2 ? (unsigned) ((8 * ((lane >> 3) & 1) + (lane & 7)) * lda + 16 * (lane >> 4))
                                    : (unsigned) ((lane & 7) * lda + 16 * ((lane >> 3) & 1));
    const unsigned sq_s = (unsigned) __cvta_generic_to_shared(sq) + b_lane;
    const unsigned dw_lane = (unsigned) (r8 * RL + CW + 2 * par);   // this lane's row's scales in a stage
    unsigned stage = ring_s0;
#pragma unroll 1
    for (int tile = blockIdx.x * G + g; tile < ntiles; tile += gstride) {
        f32x2 acc[MT][2 * NP][NT][2];   // [..][h]: row 8 h + lane / 4 of the 16-row tile, activation rows 2 (lane % 4), + 1
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int v = 0; v < 2 * NP; ++v)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) acc[mt][v][nt][0] = acc[mt][v][nt][1] = 0ull;
#pragma unroll 1
        for (int k = 0; k < nsteps; ++k) {
            issue();   // into the stage read one step ago
            asm volatile("cp.async.wait_group %0;" ::"n"(QS_S - 1) : "memory");
            __syncwarp();
            const unsigned rs_s = stage + a_lane, rs_d = stage + dw_lane;
#pragma unroll
            for (int pi = 0; pi < NP; ++pi) {
                const int cbp = 512 * k + 32 * wg + 256 * pi, b = cbp >> 5;
                if (cbp < cols) {   // the same for the whole warp
                    unsigned bf[2][NT];   // [16-column half][8-row tile]
                    f32x2 da[NT];
                    if (NT == 2) {
                        unsigned r[4];
                        ldmatrix_x4(r, sq_s + cbp);
                        bf[0][0] = r[0], bf[0][NT - 1] = r[1], bf[1][0] = r[2], bf[1][NT - 1] = r[3];
                        const ulonglong2 dd = *reinterpret_cast<const ulonglong2*>(sd + (size_t) (b * 4 + q) * 4);
                        da[0] = dd.x, da[NT - 1] = dd.y;
                    } else {
                        unsigned r[2];
                        ldmatrix_x2(r, sq_s + cbp);
                        bf[0][0] = r[0], bf[1][0] = r[1];
                        da[0] = *reinterpret_cast<const f32x2*>(sd + (size_t) (b * 4 + q) * 2);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        unsigned a[4];   // a0, a1 of the first half, then of the second
                        ldmatrix_x4(a, rs_s + (16 * mt) * RL + 32 * pi);
                        f32x2 w[2][NT];   // fl(dw da) of (row, activation row pair) for this block
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            unsigned short dwh;
                            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(dwh) : "r"(rs_d + (16 * mt + 8 * h) * RL + 4 * pi));
                            const float dw = h2f(dwh);
                            const f32x2 dw2 = pack2(dw, dw);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) w[h][nt] = mul2(dw2, da[nt]);
                        }
#pragma unroll
                        for (int half = 0; half < 2; ++half)
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const int v = 2 * pi + half;
                                int d[4];
                                mma_s8_16816(d, a[2 * half], a[2 * half + 1], bf[half][nt]);
                                acc[mt][v][nt][0] = fma2(w[0][nt], add2(pack2i(d[0], d[1]), unmagic), acc[mt][v][nt][0]);
                                acc[mt][v][nt][1] = fma2(w[1][nt], add2(pack2i(d[2], d[3]), unmagic), acc[mt][v][nt][1]);
                            }
                    }
                }
            }
            __syncwarp();   // every lane has read this stage before the next step's copies land in it
            stage = stage + STAGE == ring_s0 + QS_S * STAGE ? ring_s0 : stage + STAGE;
        }
        // ---- the lane sums meet in shared memory, 16 rows at a time, and a thread adds two neighbouring outputs' trees
        const int seg = tile < sg.blk_end[0] ? 0 : tile < sg.blk_end[1] ? 1 : 2;
        float* __restrict__ out = seg == 0 ? sg.out[0] : seg == 1 ? sg.out[1] : sg.out[2];
        const int out_stride = seg == 0 ? sg.stride[0] : seg == 1 ? sg.stride[1] : sg.stride[2];
        const int rows = seg == 0 ? sg.rows[0] : seg == 1 ? sg.rows[1] : sg.rows[2];
        const int row0 = (tile - (seg == 0 ? 0 : seg == 1 ? sg.blk_end[0] : sg.blk_end[1])) * ROWS;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(WPT * 32) : "memory");   // the pass before has been read
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const f32x2 val = NP == 2 ? add2(acc[mt][half][nt][h], acc[mt][NP == 2 ? 2 + half : half][nt][h]) : acc[mt][half][nt][h];
                        const int row = 8 * h + r8, t = (8 * nt + 2 * q) ^ (NT == 2 ? ((row >> 1) & 1) << 3 : 0);   // swizzled against bank conflicts
                        *reinterpret_cast<f32x2*>(red + ((size_t) (2 * wg + half) * 16 + row) * TO + t) = val;
                    }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "r"(WPT * 32) : "memory");
            for (int o = 2 * gtid; o < 16 * TO; o += 2 * WPT * 32) {
                const int row = o / TO, t = o % TO, ts = t ^ (NT == 2 ? ((row >> 1) & 1) << 3 : 0);
                f32x2 p[NL];
#pragma unroll
                for (int l = 0; l < NL; ++l) p[l] = *reinterpret_cast<const f32x2*>(red + ((size_t) l * 16 + row) * TO + ts);
#pragma unroll
                for (int w2 = NL / 2; w2; w2 >>= 1)
#pragma unroll
                    for (int l = 0; l < NL / 2; ++l)
                        if (l < w2) p[l] = add2(p[l], p[l + w2]);
                float v0, v1;
                unpack2(p[0], v0, v1);
                const int orow = row0 + 16 * mt + row;
                if (orow < rows && t < T) out[(size_t) t * out_stride + orow] = v0;
                if (orow < rows && t + 1 < T) out[(size_t) (t + 1) * out_stride + orow] = v1;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// f32 GEMV, a block of 4 warps per row, warp p the p-th quarter of the float4 chunks (reference
// src/kernels.cu:184-227 with WPR = 4): lane sums its chunks in ascending order, xor-tree, 0 + p0 + p1 + p2 + p3
__global__ void __launch_bounds__(128) k_gemv_f32(const float* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                                                  int rows, int n, int T) {
    // block (row, group of 4 activation rows): the four rows' loads and sums overlap, and the groups run side by side
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.x, nc = n / 512, t0 = blockIdx.y * 4;
    __shared__ float red[4][4];
    const float4* w4 = reinterpret_cast<const float4*>(W + (size_t) row * n) + warp * nc * 32;
    float4 wv[8];   // the warp's quarter of the row (n <= 4096)
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < nc) wv[i] = __ldg(w4 + i * 32 + lane);
    pdl_wait();   // the weights above are asked for while the kernel before still runs
    pdl_go();
    float a[4];
    const float4* x4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        a[k] = 0.f;
        x4[k] = reinterpret_cast<const float4*>(x + (size_t) min(t0 + k, T - 1) * n) + warp * nc * 32;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < nc) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 w = wv[i], b = x4[k][i * 32 + lane];
                float p = fmul(w.x, b.x);
                p = ffma(w.y, b.y, p);
                p = ffma(w.z, b.z, p);
                p = ffma(w.w, b.w, p);
                a[k] = fadd(a[k], p);
            }
        }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float v = wsum(a[k]);
        if (lane == 0) red[k][warp] = v;
    }
    __syncthreads();
    if (threadIdx.x < 4 && t0 + threadIdx.x < T) {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) v = fadd(v, red[threadIdx.x][k]);
        y[(size_t) (t0 + threadIdx.x) * rows + row] = v;
    }
}

// h = silu(gate) * up of T rows [gate | up] as an int8 plane + float(f16(d)) scales (see moe.cu k_swiglu_q8)
__global__ void __launch_bounds__(256) k_swiglu_rows(const float* __restrict__ gu, int ffs, int nrows, int8_t* __restrict__ hq,
                                                     float* __restrict__ hd) {
    const int nb = ffs / 32, q = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_go();
    if (q >= nrows * nb) return;
    const int e = q / nb, b = q % nb;
    const float* g = gu + (size_t) e * 2 * ffs;
    const float xi = fmul(ex_silu(g[b * 32 + lane]), g[ffs + b * 32 + lane]);
    const float amax = wmax(fabsf(xi));
    const float d = fdiv(amax, 127.0f);
    hq[(size_t) e * ffs + b * 32 + lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
    if (lane == 0) hd[(size_t) e * nb + b] = h2f(f2h(d));
}

static int sm_count() {
    static int n[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!n[dev] && cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n[dev] = 148;
    return n[dev];
}

// the persistent streaming kernel; -1 when the shape does not fit it
int q8s_stream_launch(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int nseg, int cols, const void* yq,
                      const int8_t* pq, const float* pd, int T, cudaStream_t st, const char* what) {
    if (cols % 64) return -1;
    for (int s = 0; s < nseg; ++s)
        if ((uintptr_t) w[s].q % 16 || (uintptr_t) w[s].d % 4) return -1;   // 16-byte pieces, 4-byte scale pairs
    const int NT = T <= 8 ? 1 : 2, TO = 8 * NT, nsm = sm_count();
    const size_t act = ((size_t) 8 * NT * (cols + QM_APAD) + (size_t) 8 * NT * (cols / 32) * 4 + 15) & ~(size_t) 15, cap = 226 * 1024;
    long rows_all = 0, tiles32 = 0;
    for (int s = 0; s < nseg; ++s) rows_all += rows[s], tiles32 += (rows[s] + 31) / 32;
    // two groups of 8 warps when their rings fit beside the activations, else one group of 16; 32-row tiles when there
    // are enough of them to keep every group busy for a few rounds
    auto bytes = [&](int wpt, int mt) {
        const int np = 16 / wpt, nl = wpt == 8 ? 16 : 32, g = 16 / wpt;
        return act + (size_t) 16 * QS_S * 16 * mt * (32 * np + 16) + (size_t) g * nl * 16 * TO * 4;
    };
    // how well a choice fills the machine: tiles over (groups x rounds)
    auto fill = [&](int wpt, int mt) {
        if ((wpt == 16 && mt == 2) || bytes(wpt, mt) > cap) return -1.0;
        long tiles = 0;
        for (int s = 0; s < nseg; ++s) tiles += (rows[s] + 16 * mt - 1) / (16 * mt);
        const long groups = (long) nsm * (16 / wpt), rounds = (tiles + groups - 1) / groups;
        return (double) tiles / (double) (groups * rounds);
    };
    // relative instructions a byte of the shapes (measured): smaller tiles repeat the activation-side work more often
    const double f82 = fill(8, 2), f81 = fill(8, 1) / 1.3, f161 = fill(16, 1) / 1.5;
    int WPT = 8, MT = 2;
    double best = f82;
    if (f81 > best) best = f81, MT = 1;
    if (f161 > best) best = f161, WPT = 16, MT = 1;
    if (best <= 0) return -1;
    if ((size_t) rows_all * cols >= ((size_t) 1 << 32)) return -1;   // 32-bit piece offsets
    const int tile_rows = 16 * MT, G = 16 / WPT;
    QSegs sg{};
    int ntiles = 0;
    for (int s = 0; s < 3; ++s) {
        const int k = s < nseg ? s : nseg - 1;
        sg.q[s] = w[k].q, sg.d[s] = w[k].d, sg.out[s] = out[k], sg.stride[s] = out_stride[k], sg.rows[s] = rows[k];
        if (s < nseg) ntiles += (rows[s] + tile_rows - 1) / tile_rows;
        sg.blk_end[s] = ntiles;
    }
    const int grid = std::min(nsm, (ntiles + G - 1) / G);
    const size_t smm = bytes(WPT, MT);
    const unsigned ring_off = (unsigned) act, red_off = (unsigned) (act + (size_t) 16 * QS_S * tile_rows * (32 * (16 / WPT) + 16));
#define QS_CASE(NTv, MTv, WPTv)                                                                                                   \
    if (NT == NTv && MT == MTv && WPT == WPTv) {                                                                                  \
        if (cudaFuncSetAttribute(k_q8s_stream<NTv, MTv, WPTv>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smm) != cudaSuccess) \
            return fail("%s: shared memory opt-in failed", what);                                                                 \
        launch(1, k_q8s_stream<NTv, MTv, WPTv>, grid, QS_THREADS, smm, st, sg, cols, (const uint8_t*) yq, pq, pd, T, ntiles, ring_off, red_off); \
        return launch_ok(what);                                                                                                   \
    }
    QS_CASE(1, 1, 8) QS_CASE(1, 2, 8) QS_CASE(2, 1, 8) QS_CASE(2, 2, 8) QS_CASE(1, 1, 16) QS_CASE(2, 1, 16)
#undef QS_CASE
    return -1;
}

int q8s_launch(FnxQ8S w, int rows, int cols, const void* yq, const int8_t* pq, const float* pd, float* out, int out_stride, int T,
               cudaStream_t st, const char* what) {
    if (!(T >= 1 && T <= FNX_MAXT)) return fail("%s: T %d outside 1..%d", what, T, FNX_MAXT);
    if (!(cols > 0 && cols % 32 == 0 && rows > 0)) return fail("%s: %d x %d (columns a multiple of 32)", what, rows, cols);
    if (cols % 64 == 0) {   // the persistent tensor-core kernel
        const FnxQ8S ws[1] = {w};
        const int rs[1] = {rows}, strides[1] = {out_stride};
        float* outs[1] = {out};
        const int rc = q8s_stream_launch(ws, rs, outs, strides, 1, cols, yq, pq, pd, T, st, what);
        if (rc >= 0) return rc;
    }
    // enough blocks to fill the GPU twice over, at most 128 rows each so the staged activations are amortised
    int rpb = (rows / 296 + 31) / 32 * 32;
    rpb = rpb < 32 ? 32 : rpb > 128 ? 128 : rpb;
    const int grid = (rows + rpb - 1) / rpb;
    const size_t sm = (size_t) T * cols + (size_t) T * (cols / 32) * 4;
    if (sm > 227 * 1024) return fail("%s: %d columns x %d rows of activations do not fit shared memory", what, cols, T);
#define Q8S_CASE(TT)                                                                                                          \
    {                                                                                                                         \
        if (sm > 48 * 1024 && cudaFuncSetAttribute(k_q8s<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm) != cudaSuccess) \
            return fail("%s: shared memory opt-in failed", what);                                                             \
        k_q8s<TT><<<grid, Q8S_THREADS, sm, st>>>(w.q, w.d, rows, cols, (const uint8_t*) yq, pq, pd, T, out, out_stride, rpb);  \
    }
    if (T <= 1) Q8S_CASE(1)
    else if (T <= 2) Q8S_CASE(2)
    else if (T <= 4) Q8S_CASE(4)
    else if (T <= 8) Q8S_CASE(8)
    else Q8S_CASE(16)
#undef Q8S_CASE
    return launch_ok(what);
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_q8s_gemv(FnxQ8S w, int rows, int cols, const void* y, float* out, int out_stride, int T, void* st) {
    return q8s_launch(w, rows, cols, y, nullptr, nullptr, out, out_stride, T, strm(st), "q8s_gemv");
}

int fnx_q8s_gemv_segs(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int n, int cols, const void* y, int T,
                      void* st) {
    FNX_REQUIRE(n >= 1 && n <= 3, "q8s_gemv_segs: %d matrices (1..3)", n);
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "q8s_gemv_segs: T %d outside 1..%d", T, FNX_MAXT);
    if (cols % 64 == 0) {
        const int rc = q8s_stream_launch(w, rows, out, out_stride, n, cols, y, nullptr, nullptr, T, strm(st), "q8s_gemv_segs");
        if (rc >= 0) return rc;
    }
    for (int s = 0; s < n; ++s)
        if (q8s_launch(w[s], rows[s], cols, y, nullptr, nullptr, out[s], out_stride[s], T, strm(st), "q8s_gemv_segs")) return 1;
    return 0;
}

int fnx_gemv_f32(const float* W, const float* x, float* y, int rows, int n, int T, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "gemv_f32: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(n > 0 && n % 512 == 0 && n <= 4096 && rows > 0, "gemv_f32: %d x %d (columns a multiple of 512 up to 4096)", rows, n);
    launch(7, k_gemv_f32, dim3(rows, (T + 3) / 4), 128, 0, strm(st), W, x, y, rows, n, T);
    return launch_ok("gemv_f32");
}

int fnx_q8s_gemv_f32(FnxQ8S w, int rows, int cols, const void* y, float* out, const float* W, const float* x, float* yf, int rf, int T,
                     void* st) {
    // the reference fuses the two into one launch to save a launch's latency on a V100; here they are two launches in
    // stream order (the window itself runs the f32 one on a side stream beside the quantised one), the same values
    if (fnx_q8s_gemv(w, rows, cols, y, out, rows, T, st)) return 1;
    return fnx_gemv_f32(W, x, yf, rf, cols, T, st);
}

int fnx_shared_expert(FnxQ8S gate_up, FnxQ8S down, const void* xq, int T, int n, int ffs, float* sh_gu, void* hq, float* out,
                      void* st) {
    FNX_REQUIRE(ffs > 0 && ffs % 32 == 0 && ((size_t) T * ffs) % 16 == 0, "shared_expert: ff width %d", ffs);
    if (q8s_launch(gate_up, 2 * ffs, n, xq, nullptr, nullptr, sh_gu, 2 * ffs, T, strm(st), "shared expert gate|up")) return 1;
    int8_t* h8 = (int8_t*) hq;
    float* hd = (float*) ((char*) hq + (size_t) T * ffs);
    launch(0, k_swiglu_rows, (T * (ffs / 32) + 7) / 8, 256, 0, strm(st), sh_gu, ffs, T, h8, hd);
    if (launch_ok("shared expert swiglu")) return 1;
    return q8s_launch(down, n, ffs, nullptr, h8, hd, out, n, T, strm(st), "shared expert down");
}
}
