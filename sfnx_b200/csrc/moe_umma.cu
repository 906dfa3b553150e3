// The routed experts over many rows (the prompt path's jobs of up to 64 rows of one expert) on Blackwell's fifth-generation
// tensor cores.  Replaces reference src/moe_mma.cu:28-59 / src/moe_mma.cuh:63-379 (moe_gate_up_mma, swiglu_h16,
// moe_down_mma; HMMA.884 there).
//
// The values are the reference's: each weight dequantised to f16 with one rounding (Q4_K: the sub-block scale d sc and
// min dmin m rounded to f16, then one half fma q * f16(d sc) - f16(dmin m), src/moe_mma.cuh:56-60, 79-113; Q8_0: one
// half product q * d, :184-216; Q6_K in 32-column units, which the reference's prompt path does not take, by the same
// rule: one half product (q - 32) * f16(d sc)), activations f16, products summed in fp32.
//
// A CTA takes 128 of an expert's rows and one or two of the expert's jobs (consecutive jobs of one expert are paired, so
// that their weights are dequantised once).  The rows are the M side of tcgen05.mma (kind::f16, cta_group::1, M 128),
// the jobs' activation rows the N side (16 to 128), and the 128 x N fp32 result sits in tensor memory.  Eight producer
// warps turn 64 columns at a time into the A operand (128 rows x 128 bytes, K-major, 128-byte swizzle) in one of three
// shared-memory stages, next to the jobs' activation rows for those columns (the B operand, same form, by cp.async);
// raw weight bytes are fetched a step ahead into registers (a Q4_K super-block, four stages' worth, at a time).  A
// ninth warp waits for a stage to be full, issues its four MMAs (K 16 each) and lets tcgen05.commit hand the stage
// back.  Two CTAs share an SM (97 KB of shared memory and 128 columns of tensor memory each), so one streams while the
// other starts or drains.  Every wait is bounded and feeds the device fault word.
#include <algorithm>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "umma.cuh"

namespace fnxk {

constexpr int MU_BM = 128, MU_KC = 64, MU_NS = 3, MU_PROD = 256, MU_THREADS = MU_PROD + 32, MU_PAIR = 2, MU_NMAX = MU_PAIR * FNX_PF_JOB;
constexpr int MU_ABYTES = MU_BM * 128, MU_BBYTES = MU_NMAX * 128, MU_STAGE = MU_ABYTES + MU_BBYTES;
constexpr size_t MU_SMEM = (size_t) MU_NS * MU_STAGE + 1024;

__device__ __forceinline__ void mu_arrive(unsigned long long* bar) {
    asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(um_s32(bar)) : "memory");
}

// four bytes (each 0..255) as f16 pairs {b0, b1}, {b2, b3} less `bias`: 0x6400 | b is the f16 1024 + b exactly
__device__ __forceinline__ void mu_bytes(unsigned w, __half2 bias, __half2& lo, __half2& hi) {
    const unsigned p = __byte_perm(w, 0x64646464u, 0x4140), q = __byte_perm(w, 0x64646464u, 0x4342);
    lo = __hsub2(*reinterpret_cast<const __half2*>(&p), bias);
    hi = __hsub2(*reinterpret_cast<const __half2*>(&q), bias);
}
__device__ __forceinline__ __half2 mu_h2(unsigned short bits) { return __half2half2(__ushort_as_half(bits)); }
__device__ __forceinline__ unsigned mu_u(__half2 h) { return *reinterpret_cast<const unsigned*>(&h); }

struct MuArgs {
    int type, nrows, ncols;
    const unsigned char *a, *b, *c, *d;
    size_t stride, stride_b;
    const FnxBigJob* jobs;
    const int* njobs;
    const uint16_t* x;
    float* out;
    unsigned* fault;
};

// The raw bytes of one thread's share, (row, half) of the 128 x 64 weight tile, for STEPS consecutive tiles: a Q4_K
// super-block (256 columns) is one 16-byte header and four 32-byte runs of quants, so a thread takes its half of all four
// runs and the header in five loads; the other types are fetched tile by tile.
template <int TYPE> struct MuRaw {
    static constexpr int STEPS = 1;
    uint4 q0, q1;   // Q8_0: the 32 quants; Q6_K: q0 = low nibbles, q1.xy = high bits
    unsigned s, d;  // Q8_0: s = scale; Q6_K: s = the two scales, d = d
    __device__ __forceinline__ void fetch(const MuArgs& a, int expert, int row, int half, int step) {
        const int k0 = step * MU_KC;
        if (32 * half >= a.ncols - k0) return;   // a last tile of 32 columns
        if (TYPE == FNX_Q8_0) {
            const int blkc = k0 / 32 + half;
            const uint4* q = reinterpret_cast<const uint4*>(a.a + (size_t) expert * a.stride + (size_t) row * a.ncols + (size_t) blkc * 32);
            q0 = __ldg(q);
            q1 = __ldg(q + 1);
            s = __ldg(reinterpret_cast<const uint16_t*>(a.b + (size_t) expert * a.stride_b) + (size_t) row * (a.ncols / 32) + blkc);
        } else {
            const size_t g = (size_t) expert * a.stride + (size_t) row * (a.ncols / 32) + k0 / 32 + half;
            q0 = __ldg(reinterpret_cast<const uint4*>(a.a) + g);
            const uint2 h = __ldg(reinterpret_cast<const uint2*>(a.b) + g);
            q1.x = h.x, q1.y = h.y;
            s = __ldg(reinterpret_cast<const uint16_t*>(a.c) + g);
            d = __ldg(reinterpret_cast<const uint16_t*>(a.d) + g);
        }
    }
};
template <> struct MuRaw<FNX_Q4_K> {
    static constexpr int STEPS = 4;
    uint4 hd, q[4];
    __device__ __forceinline__ void fetch(const MuArgs& a, int expert, int row, int half, int step) {
        const unsigned char* blk = a.a + (size_t) expert * a.stride + ((size_t) row * (a.ncols / 256) + step) * 144;
        hd = __ldg(reinterpret_cast<const uint4*>(blk));
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * j + 16 * half));
    }
};

// 8 consecutive f16 values of row `row` at 16-byte piece `chunk` of the 128-byte row
__device__ __forceinline__ void mu_put(unsigned tile, int row, int chunk, __half2 v0, __half2 v1, __half2 v2, __half2 v3) {
    const unsigned at = tile + row * 128 + ((chunk ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(mu_u(v0)), "r"(mu_u(v1)), "r"(mu_u(v2)), "r"(mu_u(v3)) : "memory");
}

// tile j of the raw set (j < STEPS) into the A operand's stage
__device__ __forceinline__ void mu_dequant(const MuRaw<FNX_Q4_K>& r, int j, unsigned tile, int row, int half) {
    // byte l of the 16: value 16 half + l of sub-block 2 j (low nibble) and of sub-block 2 j + 1 (high nibble)
    const float d = h2f((uint16_t) (r.hd.x & 0xffff)), dmin = h2f((uint16_t) (r.hd.x >> 16));
    float sc0, m0, sc1, m1;
    q4k_scale_min_pair(r.hd, j, sc0, m0, sc1, m1);
    const __half2 d0 = __float2half2_rn(fmul(d, sc0)), n0 = __float2half2_rn(-fmul(dmin, m0));
    const __half2 d1 = __float2half2_rn(fmul(d, sc1)), n1 = __float2half2_rn(-fmul(dmin, m1));
    const __half2 k = mu_h2(0x6400);
    const unsigned q[4] = {r.q[j].x, r.q[j].y, r.q[j].z, r.q[j].w};
    __half2 lo[8], hi[8];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        __half2 u, v;
        mu_bytes(q[w] & 0x0F0F0F0Fu, k, u, v);
        lo[2 * w] = __hfma2(u, d0, n0), lo[2 * w + 1] = __hfma2(v, d0, n0);
        mu_bytes((q[w] >> 4) & 0x0F0F0F0Fu, k, u, v);
        hi[2 * w] = __hfma2(u, d1, n1), hi[2 * w + 1] = __hfma2(v, d1, n1);
    }
    mu_put(tile, row, 2 * half, lo[0], lo[1], lo[2], lo[3]);
    mu_put(tile, row, 2 * half + 1, lo[4], lo[5], lo[6], lo[7]);
    mu_put(tile, row, 4 + 2 * half, hi[0], hi[1], hi[2], hi[3]);
    mu_put(tile, row, 5 + 2 * half, hi[4], hi[5], hi[6], hi[7]);
}
__device__ __forceinline__ void mu_dequant(const MuRaw<FNX_Q8_0>& r, int, unsigned tile, int row, int half) {
    // the signed quants offset by 128 become bytes 0..255: 1024 + 128 + q, less 1152
    const __half2 d = mu_h2((unsigned short) r.s), k = mu_h2(0x6480);
    const unsigned q[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    __half2 y[16];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        __half2 u, v;
        mu_bytes(q[w] ^ 0x80808080u, k, u, v);
        y[2 * w] = __hmul2(u, d), y[2 * w + 1] = __hmul2(v, d);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) mu_put(tile, row, 4 * half + c, y[4 * c], y[4 * c + 1], y[4 * c + 2], y[4 * c + 3]);
}
__device__ __forceinline__ void mu_dequant(const MuRaw<FNX_Q6_K>& r, int, unsigned tile, int row, int half) {
    // a unit: byte i of the 16 holds value i (low nibble) and value 16 + i (high nibble); the two high bits of value
    // 4 w + b sit in byte (w / 4) 4 + b of the 8 at bit 2 (w % 4); codes 0..63 less 32; scale 0 for values < 16
    const float d = h2f((uint16_t) r.d);
    const int s0 = (int) (signed char) (r.s & 0xff), s1 = (int) (signed char) ((r.s >> 8) & 0xff);
    const __half2 d0 = __float2half2_rn(fmul(d, (float) s0)), d1 = __float2half2_rn(fmul(d, (float) s1));
    const __half2 k = mu_h2(0x6420);   // 1024 + 32
    const unsigned q[4] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w};
    __half2 lo[8], hi[8];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        __half2 u, v;
        mu_bytes((q[w] & 0x0F0F0F0Fu) | (((r.q1.x >> (2 * w)) & 0x03030303u) << 4), k, u, v);
        lo[2 * w] = __hmul2(u, d0), lo[2 * w + 1] = __hmul2(v, d0);
        mu_bytes(((q[w] >> 4) & 0x0F0F0F0Fu) | (((r.q1.y >> (2 * w)) & 0x03030303u) << 4), k, u, v);
        hi[2 * w] = __hmul2(u, d1), hi[2 * w + 1] = __hmul2(v, d1);
    }
    mu_put(tile, row, 4 * half, lo[0], lo[1], lo[2], lo[3]);
    mu_put(tile, row, 4 * half + 1, lo[4], lo[5], lo[6], lo[7]);
    mu_put(tile, row, 4 * half + 2, hi[0], hi[1], hi[2], hi[3]);
    mu_put(tile, row, 4 * half + 3, hi[4], hi[5], hi[6], hi[7]);
}

// out[jb.out[j] * nrows + row] = sum_k W_e[row][k] x[jb.y[j] * ncols + k]
template <int TYPE>
__global__ void __launch_bounds__(MU_THREADS, 2) k_moe_umma(const MuArgs a) {
    const int ji = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int njobs = *a.njobs;
    if (ji >= njobs) return;
    // Consecutive jobs of one expert share the dequantised weights: the jobs of an expert are taken two at a time, the
    // first of a pair does both (its rows in columns 0..63 of the result, the partner's from column 64), the second
    // leaves at once.  A pair is counted from the expert's first job.
    const int expert = a.jobs[ji].w;
    int first = ji;
    while (first > 0 && a.jobs[first - 1].w == expert) --first;
    if ((ji - first) & 1) return;
    const bool paired = ji + 1 < njobs && a.jobs[ji + 1].w == expert;
    extern __shared__ __align__(1024) unsigned char mu_smem[];
    // the swizzle is a function of the shared-memory address: operand tiles start on 1024-byte boundaries
    unsigned char* stages = mu_smem + ((1024u - (um_s32(mu_smem) & 1023u)) & 1023u);
    __shared__ FnxBigJob jb, jb2;
    __shared__ __align__(8) unsigned long long full[MU_NS], empty[MU_NS], done;
    __shared__ unsigned tmem_base;
    for (int i = tid; i < (int) (sizeof(FnxBigJob) / 4); i += MU_THREADS) {
        reinterpret_cast<int*>(&jb)[i] = reinterpret_cast<const int*>(a.jobs + ji)[i];
        reinterpret_cast<int*>(&jb2)[i] = paired ? reinterpret_cast<const int*>(a.jobs + ji + 1)[i] : 0;
    }
    if (tid == 0) {
        for (int s = 0; s < MU_NS; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(um_s32(&full[s])), "r"(MU_PROD));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&empty[s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&done)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MU_PROD / 32) {   // 128 columns of tensor memory: the 128 x (64 + 64) fp32 result
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(um_s32(&tmem_base)), "r"(MU_NMAX));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // a last step of 32 columns (an FF slice of 96) fills half a stage: two MMAs instead of four
    const int n = min(max(jb.n, 0), FNX_PF_JOB), n2 = paired ? min(max(jb2.n, 0), FNX_PF_JOB) : 0;
    const int ncol = paired ? FNX_PF_JOB + 16 * ((n2 + 15) / 16) : 16 * ((n + 15) / 16);   // N of the MMAs
    const int nk = (a.ncols + MU_KC - 1) / MU_KC, row0 = blockIdx.x * MU_BM;
    const unsigned st_s = um_s32(stages);
    bool alive = true;   // false after a wait ran out
    if (warp < MU_PROD / 32) {
        // ---- producers.  Weights: warp w owns rows 16 w .. + 15 of the tile, lanes 0..15 the first 32 columns of a step
        // and lanes 16..31 the last 32 (the two lanes of a row read neighbouring bytes: a warp's load touches 16 lines, and
        // a quarter-warp's stores 8 different rows of one 16-byte column: no bank conflicts).  Activations: 16-byte pieces
        // tid and tid + 256 of 64 rows x 8, copied asynchronously one step ahead straight into the stage.
        using Raw = MuRaw<TYPE>;
        const int row = 16 * warp + (lane & 15), half = lane >> 4;
        const int wrow = min(row0 + row, a.nrows - 1);   // rows past the matrix repeat the last one; never written out
        const int xc = tid & 7;
        const uint16_t* xp[MU_NMAX / 32];   // B rows tid / 8 + 32 i: rows 0..63 the job's, 64..127 its partner's
        unsigned xd[MU_NMAX / 32];
#pragma unroll
        for (int i = 0; i < MU_NMAX / 32; ++i) {
            const int j = (tid >> 3) + 32 * i, jj = j & (FNX_PF_JOB - 1);
            const bool has = j < FNX_PF_JOB ? jj < n : jj < n2;
            xp[i] = has ? a.x + (size_t) (j < FNX_PF_JOB ? jb.y[jj] : jb2.y[jj]) * a.ncols + xc * 8 : nullptr;
            xd[i] = MU_ABYTES + j * 128 + ((xc ^ (j & 7)) << 4);
        }
        auto xcopy = [&](int k) {   // the job's rows for step k, once its stage is free
            if (k < nk) {
                const int s = k % MU_NS;
                if (k >= MU_NS && alive) alive = um_wait(&empty[s], (unsigned) ((k / MU_NS - 1) & 1), a.fault);
                const unsigned tile = st_s + s * MU_STAGE;
                const bool in = 8 * xc < a.ncols - k * MU_KC;
#pragma unroll
                for (int i = 0; i < MU_NMAX / 32; ++i)
                    if (xp[i] && in) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tile + xd[i]), "l"(xp[i] + k * MU_KC));
            }
            asm volatile("cp.async.commit_group;");
        };
        auto produce = [&](const Raw& r, int j, int k) {
            xcopy(k + 1);   // also makes sure that the stage the next step writes is free
            const unsigned tile = st_s + (k % MU_NS) * MU_STAGE;
            if (32 * half < a.ncols - k * MU_KC) mu_dequant(r, j, tile, row, half);
            asm volatile("cp.async.wait_group 1;" ::: "memory");          // this step's activation pieces have landed
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes before the tensor core's reads
            mu_arrive(&full[k % MU_NS]);
        };
        const int nsteps = (nk + Raw::STEPS - 1) / Raw::STEPS;
        Raw r0, r1;
        r0.fetch(a, expert, wrow, half, 0);
        xcopy(0);
#pragma unroll 1
        for (int sidx = 0; sidx < nsteps; sidx += 2) {
            if (sidx + 1 < nsteps) r1.fetch(a, expert, wrow, half, sidx + 1);
#pragma unroll
            for (int j = 0; j < Raw::STEPS; ++j)
                if (sidx * Raw::STEPS + j < nk) produce(r0, j, sidx * Raw::STEPS + j);
            if (sidx + 1 < nsteps) {
                if (sidx + 2 < nsteps) r0.fetch(a, expert, wrow, half, sidx + 2);
#pragma unroll
                for (int j = 0; j < Raw::STEPS; ++j)
                    if ((sidx + 1) * Raw::STEPS + j < nk) produce(r1, j, (sidx + 1) * Raw::STEPS + j);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ---- the issuing warp: stage k's four MMAs once it is full; the commit frees the stage
        const unsigned idesc = (1u << 4) | ((unsigned) (ncol >> 3) << 17) | ((128u >> 4) << 24);   // D f32, A and B f16 K-major
#pragma unroll 1
        for (int k = 0; k < nk; ++k) {
            const int s = k % MU_NS;
            if (alive) alive = um_wait(&full[s], (unsigned) ((k / MU_NS) & 1), a.fault);
            alive = __all_sync(0xffffffffu, alive);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const unsigned long long da = um_desc(st_s + s * MU_STAGE), db = um_desc(st_s + s * MU_STAGE + MU_ABYTES);
#pragma unroll
                for (int ks = 0; ks < MU_KC / 16; ++ks)
                    if (16 * ks < a.ncols - k * MU_KC) um_mma(tmem_base, da + 2 * ks, db + 2 * ks, idesc, (unsigned) (k | ks));
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(um_s32(&empty[s])) : "memory");
            }
            __syncwarp();
        }
        if (lane == 0) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(um_s32(&done)) : "memory");
    }
    // ---- the result out of tensor memory: warp w reads lanes 32 (w % 4) .. + 31 (its quarter), rows of the tile; warps
    // 0..3 take the first half of the job's rows, warps 4..7 the second; a warp's 32 lanes write 32 consecutive floats
    if (warp < MU_PROD / 32) {
        bool ok = alive && um_wait(&done, 0u, a.fault);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = row0 + 32 * (warp & 3) + lane, cols = ncol / 2, c0 = (warp >> 2) * cols;
        if (ok)
            for (int c = c0; c < c0 + cols; c += 8) {
                unsigned v[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                             : "r"(tmem_base + ((unsigned) (32 * (warp & 3)) << 16) + (unsigned) c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int col = c + i, jj = col & (FNX_PF_JOB - 1);
                    const bool second = paired && col >= FNX_PF_JOB;
                    if (jj < (second ? n2 : n) && row < a.nrows) a.out[(size_t) (second ? jb2.out[jj] : jb.out[jj]) * a.nrows + row] = __uint_as_float(v[i]);
                }
            }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MU_PROD / 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(MU_NMAX));
}

// h = silu(gate) * up of the stacked rows, rounded to f16 (reference src/moe_mma.cuh:381-388)
__global__ void __launch_bounds__(256) k_swiglu_h16(const float* __restrict__ gu, int ffs, size_t total, uint16_t* __restrict__ h) {
    for (size_t e = (size_t) blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t) gridDim.x * 256) {
        const size_t r = e / ffs, i = e % ffs;
        const float g = gu[r * 2 * ffs + i];
        h[e] = f2h(fmul(ex_silu(g), gu[r * 2 * ffs + ffs + i]));
    }
}

static int moe_umma(const char* what, const FnxExperts* A, const FnxBigJob* jobs, const int* njobs, int njobs_cap, const uint16_t* x, float* out,
                    cudaStream_t st) {
    FNX_REQUIRE(A && jobs && njobs && njobs_cap >= 1 && x && out, "%s: no experts, jobs, rows or output", what);
    FNX_REQUIRE(A->nrows >= 1 && A->ncols >= 32 && A->ncols % 32 == 0, "%s: %d x %d (columns in units of 32)", what, A->nrows, A->ncols);
    FNX_REQUIRE(((uintptr_t) x % 16) == 0, "%s: activation rows not 16-byte aligned", what);
    unsigned* fault = device_fault_word();
    FNX_REQUIRE(fault, "%s: no device fault word (no current device?)", what);
    MuArgs a{A->type, A->nrows, A->ncols, (const unsigned char*) A->a, (const unsigned char*) A->b, (const unsigned char*) A->c,
             (const unsigned char*) A->d, A->stride, A->stride_b, jobs, njobs, x, out, fault};
    const dim3 grid((A->nrows + MU_BM - 1) / MU_BM, njobs_cap);
#define MU_LAUNCH(T)                                                            \
    if (smem_optin(k_moe_umma<T>, MU_SMEM, what)) return 1;                     \
    k_moe_umma<T><<<grid, MU_THREADS, MU_SMEM, st>>>(a);                        \
    return launch_ok(what);
    if (A->type == FNX_Q4_K) {
        FNX_REQUIRE(A->ncols % 256 == 0 && ((uintptr_t) A->a % 16) == 0 && A->stride % 16 == 0, "%s q4_K: %d columns, rows 16-byte aligned", what, A->ncols);
        MU_LAUNCH(FNX_Q4_K)
    }
    if (A->type == FNX_Q8_0) {
        FNX_REQUIRE(((uintptr_t) A->a % 16) == 0 && A->stride % 16 == 0 && A->stride_b % 2 == 0, "%s q8_0: planes 16-byte aligned", what);
        MU_LAUNCH(FNX_Q8_0)
    }
    if (A->type == FNX_Q6_K) {
        FNX_REQUIRE(((uintptr_t) A->a % 16) == 0 && ((uintptr_t) A->b % 8) == 0, "%s q6_K: unit planes not aligned", what);
        MU_LAUNCH(FNX_Q6_K)
    }
#undef MU_LAUNCH
    return fail("%s: expert type %d not supported (Q4_K, Q8_0, Q6_K units)", what, A->type);
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_moe_gate_up_mma(const FnxExperts* A, const FnxBigJob* jobs, const int* njobs, int njobs_cap, const uint16_t* xh, float* gu, void* st) {
    return moe_umma("moe_gate_up_mma", A, jobs, njobs, njobs_cap, xh, gu, strm(st));
}

int fnx_swiglu_h16(const float* gu, int ffs, int P, uint16_t* h16, void* st) {
    FNX_REQUIRE(gu && h16 && ffs >= 1 && P >= 0, "swiglu_h16: %d rows of %d", P, ffs);
    if (!P) return 0;
    const size_t total = (size_t) P * ffs;
    k_swiglu_h16<<<(unsigned) std::min<size_t>(4096, (total + 255) / 256), 256, 0, strm(st)>>>(gu, ffs, total, h16);
    return launch_ok("swiglu_h16");
}

int fnx_moe_down_mma(const FnxExperts* A, const FnxBigJob* jobs, const int* njobs, int njobs_cap, const uint16_t* h16, float* part, void* st) {
    return moe_umma("moe_down_mma", A, jobs, njobs, njobs_cap, h16, part, strm(st));
}
}
