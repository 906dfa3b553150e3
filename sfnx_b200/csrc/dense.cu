// Dense projections of the verify window: split-layout Q8_0 matrix x up to 16 quantised activation rows (output head,
// qkvz, wq/wk/wv/wo, ssm_out, the shared expert), and the small f32 GEMV (alpha/beta).  Replaces reference
// src/dense.cuh and src/kernels.cu:184-227 with the same order of every sum: a lane takes 16 columns at
// c = 16 lane + 512 k, acc = fma(dw da, (float) isum16, acc) in ascending k, lanes combined by xor 16..1.
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

template <int NT>   // activation rows in tiles of 8: 1 (T <= 8) or 2
__global__ void __launch_bounds__(QM_THREADS, 2) k_q8s_mma(const QSegs sg, int cols,
                                                          const uint8_t* __restrict__ yq, const int8_t* __restrict__ pq,
                                                          const float* __restrict__ pd, int T, unsigned sw_off, unsigned ring_off) {
    extern __shared__ __align__(16) unsigned char smem[];
    // this block's segment, by selects (indexing the parameter arrays at run time would put them in local memory)
    const int seg = (int) blockIdx.x < sg.blk_end[0] ? 0 : (int) blockIdx.x < sg.blk_end[1] ? 1 : 2;
    const int8_t* __restrict__ wq = seg == 0 ? sg.q[0] : seg == 1 ? sg.q[1] : sg.q[2];
    const uint16_t* __restrict__ wd = seg == 0 ? sg.d[0] : seg == 1 ? sg.d[1] : sg.d[2];
    float* __restrict__ out = seg == 0 ? sg.out[0] : seg == 1 ? sg.out[1] : sg.out[2];
    const int out_stride = seg == 0 ? sg.stride[0] : seg == 1 ? sg.stride[1] : sg.stride[2];
    const int rows = seg == 0 ? sg.rows[0] : seg == 1 ? sg.rows[1] : sg.rows[2];
    const int blk0 = seg == 0 ? 0 : seg == 1 ? sg.blk_end[0] : sg.blk_end[1];
    const int nb = cols / 32, lda = cols + QM_APAD, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, q = lane & 3, r8 = lane >> 2;
    int8_t* sq = reinterpret_cast<int8_t*>(smem);                          // [8 NT][cols + pad], rows >= T zero
    float* sd = reinterpret_cast<float*>(smem + (size_t) 8 * NT * lda);    // [8 NT][nb]
    float* red = reinterpret_cast<float*>(smem);                           // after the main loop: [32 lanes][QM_ROWS][8 NT]
    float* sw = reinterpret_cast<float*>(smem + sw_off);                   // the block's weight scales [QM_ROWS][nb + 1]
    const int row0 = ((int) blockIdx.x - blk0) * QM_ROWS;
    for (int it = tid; it < QM_ROWS * nb; it += QM_THREADS) {
        const int r = it / nb, b = it % nb;
        sw[r * (nb + 1) + b] = h2f(__ldg(wd + (size_t) min(row0 + r, rows - 1) * nb + b));
    }
    for (int it = tid; it < 8 * NT * nb; it += QM_THREADS) {
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
        sd[it] = d;
    }
    __syncthreads();
    float acc[QM_MT][4][NT][4];
#pragma unroll
    for (int mt = 0; mt < QM_MT; ++mt)
#pragma unroll
        for (int v = 0; v < 4; ++v)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[mt][v][nt][0] = acc[mt][v][nt][1] = acc[mt][v][nt][2] = acc[mt][v][nt][3] = 0.f;
    // the warp's weights: its 64 columns of the block's 32 rows per step (2 KB) come through a two-stage ring of its own,
    // filled with 16-byte cp.async (4 lanes cover a row's 64 contiguous bytes) one step ahead of the MMAs; rows are padded
    // to 80 bytes so that the fragment reads (row lane / 4, 4 bytes at 4 (lane % 4)) hit 32 different banks
    unsigned char* ring = smem + ring_off + (size_t) warp * 2 * QM_ROWS * QM_RING_LD;
    const int8_t* src[4];
    unsigned dst[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = lane + 32 * i, row = j >> 2, seg = j & 3;
        src[i] = wq + (size_t) min(row0 + row, rows - 1) * cols + 16 * seg;
        dst[i] = (unsigned) __cvta_generic_to_shared(ring + row * QM_RING_LD + 16 * seg);
    }
    auto issue = [&](int cb, int stage) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst[i] + stage * QM_ROWS * QM_RING_LD), "l"(src[i] + cb));
        asm volatile("cp.async.commit_group;");
    };
    if (64 * warp < cols) issue(64 * warp, 0);
    int it = 0;
#pragma unroll 1
    for (int cb = 64 * warp; cb < cols; cb += 512, ++it) {
        if (cb + 512 < cols) {
            issue(cb + 512, (it + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const unsigned char* rs = ring + (size_t) (it & 1) * QM_ROWS * QM_RING_LD + r8 * QM_RING_LD + 4 * q;
        unsigned a[QM_MT][4][2];
#pragma unroll
        for (int mt = 0; mt < QM_MT; ++mt)
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                a[mt][v][0] = *reinterpret_cast<const unsigned*>(rs + (16 * mt) * QM_RING_LD + 16 * v);
                a[mt][v][1] = *reinterpret_cast<const unsigned*>(rs + (16 * mt + 8) * QM_RING_LD + 16 * v);
            }
#pragma unroll
        for (int bb = 0; bb < 2; ++bb) {   // the two 32-column blocks of the warp's 64 columns
            const int b = (cb >> 5) + bb;
            float w[QM_MT][2][NT][2];   // fl(dw da) of (row, activation row) for this block
            float da[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) da[nt][0] = sd[(8 * nt + 2 * q) * nb + b], da[nt][1] = sd[(8 * nt + 2 * q + 1) * nb + b];
#pragma unroll
            for (int mt = 0; mt < QM_MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float dw = sw[(16 * mt + 8 * h + r8) * (nb + 1) + b];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) w[mt][h][nt][0] = fmul(dw, da[nt][0]), w[mt][h][nt][1] = fmul(dw, da[nt][1]);
                }
#pragma unroll
            for (int vv = 0; vv < 2; ++vv) {
                const int v = 2 * bb + vv, c = cb + 16 * v;
                unsigned bf[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) bf[nt] = *reinterpret_cast<const unsigned*>(sq + (size_t) (8 * nt + r8) * lda + c + 4 * q);
#pragma unroll
                for (int mt = 0; mt < QM_MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        int d[4];
                        mma_s8_16816(d, a[mt][v][0], a[mt][v][1], bf[nt]);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            acc[mt][v][nt][i] = ffma(w[mt][i >> 1][nt][i & 1], fsub(__int_as_float(d[i]), 12582912.0f), acc[mt][v][nt][i]);
                    }
            }
        }
        __syncwarp();   // every lane has read this stage before the next step's copies land in it
    }
    __syncthreads();   // the activations are no longer read: their memory takes the lane sums
    constexpr int TO = 8 * NT, OUTS = QM_ROWS * TO;
#pragma unroll
    for (int mt = 0; mt < QM_MT; ++mt)
#pragma unroll
        for (int v = 0; v < 4; ++v)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    red[(size_t) (4 * warp + v) * OUTS + (16 * mt + 8 * (i >> 1) + r8) * TO + 8 * nt + 2 * q + (i & 1)] = acc[mt][v][nt][i];
    __syncthreads();
    for (int o = tid; o < OUTS; o += QM_THREADS) {
        float p[32];
#pragma unroll
        for (int l = 0; l < 32; ++l) p[l] = red[(size_t) l * OUTS + o];
#pragma unroll
        for (int w2 = 16; w2; w2 >>= 1)
#pragma unroll
            for (int l = 0; l < 16; ++l)
                if (l < w2) p[l] = fadd(p[l], p[l + w2]);
        const int row = row0 + o / TO, t = o % TO;
        if (row < rows && t < T) out[(size_t) t * out_stride + row] = p[0];
    }
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
    if (q >= nrows * nb) return;
    const int e = q / nb, b = q % nb;
    const float* g = gu + (size_t) e * 2 * ffs;
    const float xi = fmul(ex_silu(g[b * 32 + lane]), g[ffs + b * 32 + lane]);
    const float amax = wmax(fabsf(xi));
    const float d = fdiv(amax, 127.0f);
    hq[(size_t) e * ffs + b * 32 + lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
    if (lane == 0) hd[(size_t) e * nb + b] = h2f(f2h(d));
}

// the tensor-core kernel over 1..3 matrices; -1 when its shared memory does not fit (the caller falls back)
int q8s_mma_launch(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int nseg, int cols, const void* yq,
                   const int8_t* pq, const float* pd, int T, cudaStream_t st, const char* what) {
    const int NT = T <= 8 ? 1 : 2;
    const size_t act = (size_t) 8 * NT * (cols + QM_APAD) + (size_t) 8 * NT * (cols / 32) * 4, redb = (size_t) 32 * QM_ROWS * 8 * NT * 4;
    // activations | weight scales | the warps' rings; the lane sums reuse the whole region after the main loop
    const size_t sw_off = (act + 15) & ~(size_t) 15;
    const size_t ring_off = (sw_off + (size_t) QM_ROWS * (cols / 32 + 1) * 4 + 15) & ~(size_t) 15;
    const size_t used = ring_off + (size_t) (QM_THREADS / 32) * 2 * QM_ROWS * QM_RING_LD;
    const size_t smm = used > redb ? used : redb;
    if (smm > 227 * 1024) return -1;
    for (int s = 0; s < nseg; ++s)
        if ((uintptr_t) w[s].q % 16) return -1;   // the 16-byte copies need aligned rows
    QSegs sg{};
    int g = 0;
    for (int s = 0; s < 3; ++s) {
        const int k = s < nseg ? s : nseg - 1;
        sg.q[s] = w[k].q, sg.d[s] = w[k].d, sg.out[s] = out[k], sg.stride[s] = out_stride[k], sg.rows[s] = rows[k];
        if (s < nseg) g += (rows[s] + QM_ROWS - 1) / QM_ROWS;
        sg.blk_end[s] = g;
    }
    if (NT == 1) {
        if (smm > 48 * 1024 && cudaFuncSetAttribute(k_q8s_mma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smm) != cudaSuccess)
            return fail("%s: shared memory opt-in failed", what);
        k_q8s_mma<1><<<g, QM_THREADS, smm, st>>>(sg, cols, (const uint8_t*) yq, pq, pd, T, (unsigned) sw_off, (unsigned) ring_off);
    } else {
        if (smm > 48 * 1024 && cudaFuncSetAttribute(k_q8s_mma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smm) != cudaSuccess)
            return fail("%s: shared memory opt-in failed", what);
        k_q8s_mma<2><<<g, QM_THREADS, smm, st>>>(sg, cols, (const uint8_t*) yq, pq, pd, T, (unsigned) sw_off, (unsigned) ring_off);
    }
    return launch_ok(what);
}

int q8s_launch(FnxQ8S w, int rows, int cols, const void* yq, const int8_t* pq, const float* pd, float* out, int out_stride, int T,
               cudaStream_t st, const char* what) {
    if (!(T >= 1 && T <= FNX_MAXT)) return fail("%s: T %d outside 1..%d", what, T, FNX_MAXT);
    if (!(cols > 0 && cols % 32 == 0 && rows > 0)) return fail("%s: %d x %d (columns a multiple of 32)", what, rows, cols);
    if (cols % 64 == 0) {   // the tensor-core kernel: 32 rows a block
        const FnxQ8S ws[1] = {w};
        const int rs[1] = {rows}, strides[1] = {out_stride};
        float* outs[1] = {out};
        const int rc = q8s_mma_launch(ws, rs, outs, strides, 1, cols, yq, pq, pd, T, st, what);
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
        const int rc = q8s_mma_launch(w, rows, out, out_stride, n, cols, y, nullptr, nullptr, T, strm(st), "q8s_gemv_segs");
        if (rc >= 0) return rc;
    }
    for (int s = 0; s < n; ++s)
        if (q8s_launch(w[s], rows[s], cols, y, nullptr, nullptr, out[s], out_stride[s], T, strm(st), "q8s_gemv_segs")) return 1;
    return 0;
}

int fnx_gemv_f32(const float* W, const float* x, float* y, int rows, int n, int T, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "gemv_f32: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(n > 0 && n % 512 == 0 && n <= 4096 && rows > 0, "gemv_f32: %d x %d (columns a multiple of 512 up to 4096)", rows, n);
    k_gemv_f32<<<dim3(rows, (T + 3) / 4), 128, 0, strm(st)>>>(W, x, y, rows, n, T);
    return launch_ok("gemv_f32");
}

int fnx_shared_expert(FnxQ8S gate_up, FnxQ8S down, const void* xq, int T, int n, int ffs, float* sh_gu, void* hq, float* out,
                      void* st) {
    FNX_REQUIRE(ffs > 0 && ffs % 32 == 0 && ((size_t) T * ffs) % 16 == 0, "shared_expert: ff width %d", ffs);
    if (q8s_launch(gate_up, 2 * ffs, n, xq, nullptr, nullptr, sh_gu, 2 * ffs, T, strm(st), "shared expert gate|up")) return 1;
    int8_t* h8 = (int8_t*) hq;
    float* hd = (float*) ((char*) hq + (size_t) T * ffs);
    k_swiglu_rows<<<(T * (ffs / 32) + 7) / 8, 256, 0, strm(st)>>>(sh_gu, ffs, T, h8, hd);
    if (launch_ok("shared expert swiglu")) return 1;
    return q8s_launch(down, n, ffs, nullptr, h8, hd, out, n, T, strm(st), "shared expert down");
}
}
