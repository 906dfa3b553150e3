// Routed-expert FFN of the verify window: router + top-k + job list, dequant-fused gate|up, SwiGLU + down, combine.
// Replaces reference src/moe.cuh, src/moe_q4k.cuh and the combine of src/kernels.cu:797-803; the arithmetic order of
// every sum is the reference's, stated with IEEE operations (exact_math.cuh), so results can be checked bit for bit.
#include <cstdlib>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "umma.cuh"

namespace fnxk {

// ================================================================ router (reference src/moe.cuh:73-202)
// logits: a row's columns in two halves, a warp each; lane l accumulates the float4 chunks i * 32 + l in ascending i, each
// chunk ((wx bx + wy by) + wz bz) + ww bw with fused steps; xor-tree; half0 + half1.  The grid's last block then picks the
// top-k per row and builds the jobs.
//
// A block takes four rows of W.  A warp holds one column half of two of them in registers and walks rows of x in shared
// memory once for both; the block's two sets of four warps share the window's rows between them in groups of four
// (a logit's sum is over one row of x: which warp takes which group changes no value).  x arrives by bulk copies (the
// TMA unit's untiled copy: one instruction per group, any number of bytes in flight), a group an mbarrier, so the sums
// over the first group run while the later ones are in flight; every block asks for the groups in an order of its own
// (starting with group blockIdx mod groups) so that the blocks do not all pull on the same lines of the L2 at once.
constexpr int RR_THREADS = 256, RR_ROWS = 4, RR_TG = 4;   // rows of W a block; rows of x taken together

struct RouterArgs {
    const float* W;
    const float* x;
    float* logits;
    int T, n, nexp, topk;
    int* topi;
    float* topw;
    FnxJob *gu, *dn;
    int* njobs;
    unsigned* counter;
    unsigned* fault;
};

__device__ __forceinline__ float dot4(const float4& w, const float4& b) {
    float t = fmul(w.x, b.x);
    t = ffma(w.y, b.y, t);
    t = ffma(w.z, b.z, t);
    return ffma(w.w, b.w, t);
}

__device__ void route_tail(const RouterArgs& a);

template <bool SMEM>
__global__ void __launch_bounds__(RR_THREADS) k_router_route(const RouterArgs a) {
    const int e = threadIdx.x, warp = e >> 5, lane = e & 31, set = warp >> 2, pair = (warp >> 1) & 1, half = warp & 1;
    const int L = a.nexp + 1, nc = a.n / 256;   // float4 chunks per lane
    extern __shared__ __align__(128) float xs_sm[];   // the window's rows of x, read once per block (when they fit)
    __shared__ float rsum[FNX_MAXT][RR_ROWS][2];
    __shared__ __align__(8) unsigned long long xbar[(FNX_MAXT + RR_TG - 1) / RR_TG];
    const int ngroups = (a.T + RR_TG - 1) / RR_TG, g_first = blockIdx.x % ngroups;
    if (SMEM && e == 0) {
        for (int g = 0; g < ngroups; ++g) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&xbar[g])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the first rows' weights are asked for before the kernel ahead in the stream has finished (they do not depend on it)
    const int first0 = blockIdx.x * RR_ROWS;
    float4 wv[2][16];   // the column half of two rows held in registers (up to 16 float4 a lane and row: n <= 4096)
    auto fetch = [&](int row0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = min(row0 + 2 * pair + r, L - 1);   // past the last row: the last row again, never written
            const float4* w4 = reinterpret_cast<const float4*>(a.W + (size_t) row * a.n) + half * nc * 32;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < nc) wv[r][i] = __ldg(w4 + i * 32 + lane);
        }
    };
    if (first0 < L) fetch(first0);
    if (SMEM) __syncthreads();   // the mbarriers are set up
    pdl_wait();
    pdl_go();
    if (SMEM && e == 0 && first0 < L) {
        for (int gg = 0; gg < ngroups; ++gg) {
            const int g = (gg + g_first) % ngroups, t0 = g * RR_TG;
            const unsigned bytes = (unsigned) (min(a.T, t0 + RR_TG) - t0) * a.n * 4u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(um_s32(&xbar[g])), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             um_s32(xs_sm + (size_t) t0 * a.n)),
                         "l"(a.x + (size_t) t0 * a.n), "r"(bytes), "r"(um_s32(&xbar[g]))
                         : "memory");
        }
    }
    for (int row0 = first0; row0 < L; row0 += gridDim.x * RR_ROWS) {
        if (row0 != first0) fetch(row0);
        for (int gg = set; gg < ngroups; gg += 2) {
            const int t = ((gg + g_first) % ngroups) * RR_TG;
            if (SMEM) um_wait(&xbar[t / RR_TG], 0, a.fault);   // this group's rows of x have landed (bounded)
            float s[2][RR_TG];
            const float4* x4[RR_TG];
#pragma unroll
            for (int k = 0; k < RR_TG; ++k) {
                s[0][k] = s[1][k] = 0.f;
                const size_t at = (size_t) min(t + k, a.T - 1) * a.n;
                x4[k] = reinterpret_cast<const float4*>(SMEM ? xs_sm + at : a.x + at) + half * nc * 32;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < nc) {
#pragma unroll
                    for (int k = 0; k < RR_TG; ++k) {
                        const float4 xv = x4[k][i * 32 + lane];
                        s[0][k] = fadd(s[0][k], dot4(wv[0][i], xv));
                        s[1][k] = fadd(s[1][k], dot4(wv[1][i], xv));
                    }
                }
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int k = 0; k < RR_TG; ++k) {
                    const float v = wsum(s[r][k]);
                    if (lane == 0 && t + k < a.T) rsum[t + k][2 * pair + r][half] = v;
                }
        }
        __syncthreads();
        for (int q = e; q < a.T * RR_ROWS; q += RR_THREADS) {
            const int t = q / RR_ROWS, r = q % RR_ROWS, lrow = row0 + r;
            if (lrow < L) a.logits[(size_t) t * L + lrow] = fadd(rsum[t][r][0], rsum[t][r][1]);
        }
        __syncthreads();
    }
    // every group was waited for by one of the warp sets before the barrier above: no copy is in flight at exit
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (e == 0) last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    route_tail(a);
}

// top-k per row by logit (ties: the lower index), weights exp(l - l_top) / sum in pick order; jobs: one per distinct
// expert numbered by its first pick in pair order p = t topk + k, a job's rows in pair order.
//
// A pick is two warp-wide integer reductions: the logits become order-preserving 32-bit keys (-0 folded into +0, which
// compares equal), the largest key is a redux max and, among the lanes that hold it, the lowest expert index a redux
// min; a taken expert's key drops to 0, below every number's key.  The picks of one row are distinct experts, so a
// 16-bit mask of rows per expert gives a pair its place inside the job (rows below it) and the job's row count, and an
// atomic minimum gives the expert's first pair.
__device__ __forceinline__ unsigned logit_key(float v) {
    const unsigned b = __float_as_uint(fadd(v, 0.f));
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_logit(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k); }

__device__ void route_tail(const RouterArgs& a) {
    const int e = threadIdx.x, warp = e >> 5, lane = e & 31, L = a.nexp + 1, P = a.T * a.topk, per = a.nexp / 32;
    constexpr int NW = RR_THREADS / 32, PW = FNX_MAXT * 16 / 32, MAXE = 512;   // warps; 32-pair words; experts (16 a lane)
    __shared__ int ex[FNX_MAXT * 16];
    __shared__ unsigned rowmask[MAXE];
    __shared__ int firstpair[MAXE];
    __shared__ unsigned firstmask[PW];
    __shared__ unsigned candk[NW][2][32];   // a warp's candidates for its two rows: keys, experts; then its picks in order
    __shared__ int candi[NW][2][32];
    __shared__ unsigned selk[NW][2][16];
    __shared__ int seli[NW][2][16];
    if (e < PW) firstmask[e] = 0u;
    for (int i = e; i < a.nexp; i += RR_THREADS) rowmask[i] = 0u, firstpair[i] = P;
    // a warp takes its rows two at a time (rows t and t + NW), the two picks' instructions interleaved: each is a chain
    // of dependent warp-wide steps, and two warps a scheduler do not hide their latency
    for (int tb = warp; tb < a.T; tb += 2 * NW) {
        const int nu = tb + NW < a.T ? 2 : 1;
        unsigned key[2][16];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < 16; ++i)
                key[u][i] = (i < per && u < nu) ? logit_key(__ldcg(a.logits + (size_t) (tb + u * NW) * L + lane + 32 * i)) : 0u;
        float mine[2] = {0.f, 0.f}, top0[2] = {0.f, 0.f};   // lane k keeps pick k's logit
        // The k-th largest of the 32 lanes' maxima is a lower bound of the k-th largest key (k keys reach it), so the
        // picks are among the keys that reach it: a handful, ranked by counting (a greater key, or an equal key of a
        // lower expert, comes first).  Many equal keys can make the candidates more than a warp holds: then pick by pick.
        unsigned lm[2], hitm[2] = {0u, 0u};
        int rk[2] = {0, 0}, cnt[2], pre[2], total[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            lm[u] = key[u][0];
#pragma unroll
            for (int i = 1; i < 16; ++i) lm[u] = max(lm[u], key[u][i]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const unsigned o = __shfl_sync(0xffffffffu, lm[u], j);
                rk[u] += (o > lm[u]) | ((o == lm[u]) & (j < lane));
            }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const unsigned bound = __reduce_max_sync(0xffffffffu, rk[u] == a.topk - 1 ? lm[u] : 0u);
#pragma unroll
            for (int i = 0; i < 16; ++i) hitm[u] |= (unsigned) (i < per && u < nu && key[u][i] >= bound) << i;
            cnt[u] = pre[u] = __popc(hitm[u]);   // pre: inclusive scan over the lanes
        }
#pragma unroll
        for (int d = 1; d < 32; d <<= 1)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int o = __shfl_up_sync(0xffffffffu, pre[u], d);
                if (lane >= d) pre[u] += o;
            }
#pragma unroll
        for (int u = 0; u < 2; ++u) total[u] = __shfl_sync(0xffffffffu, pre[u], 31);
        const bool fast = a.topk <= 32 && total[0] <= 32 && total[1] <= 32;   // warp-uniform
        if (fast) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                int o = pre[u] - cnt[u];
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if ((hitm[u] >> i) & 1u) {
                        candk[warp][u][o] = key[u][i];
                        candi[warp][u][o] = lane + 32 * i;
                        ++o;
                    }
            }
            __syncwarp();
            unsigned myk[2];
            int myi[2], r[2] = {0, 0};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                myk[u] = lane < total[u] ? candk[warp][u][lane] : 0u;
                myi[u] = lane < total[u] ? candi[warp][u][lane] : 0x7fffffff;
            }
            const int tmax = max(total[0], total[1]);
            for (int j = 0; j < tmax; ++j)
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const unsigned ok = j < total[u] ? candk[warp][u][j] : 0u;
                    const int oi = j < total[u] ? candi[warp][u][j] : 0x7fffffff;
                    r[u] += (ok > myk[u]) | ((ok == myk[u]) & (oi < myi[u]));
                }
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (lane < total[u] && r[u] < a.topk) selk[warp][u][r[u]] = myk[u], seli[warp][u][r[u]] = myi[u];
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u >= nu) break;
                const int t = tb + u * NW;
                top0[u] = key_logit(selk[warp][u][0]);
                if (lane < a.topk) {
                    const int bi = seli[warp][u][lane];
                    mine[u] = key_logit(selk[warp][u][lane]);
                    a.topi[t * a.topk + lane] = bi;
                    ex[t * a.topk + lane] = bi;
                }
            }
            __syncwarp();
        } else {
            for (int u = 0; u < nu; ++u) {
                const int t = tb + u * NW;
                unsigned kk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) kk[i] = u ? key[1][i] : key[0][i];
                float mn = 0.f, tp = 0.f;
                for (int k = 0; k < a.topk; ++k) {
                    unsigned m = kk[0];
#pragma unroll
                    for (int i = 1; i < 16; ++i) m = max(m, kk[i]);
                    const unsigned M = __reduce_max_sync(0xffffffffu, m);
                    unsigned hit = 0u;
#pragma unroll
                    for (int i = 0; i < 16; ++i) hit |= (unsigned) (kk[i] == M) << i;
                    const unsigned cand = hit ? (unsigned) (lane + 32 * (__ffs(hit) - 1)) : 0xffffffffu;
                    const int bi = (int) __reduce_min_sync(0xffffffffu, cand);
                    if ((bi & 31) == lane) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i == (bi >> 5)) kk[i] = 0u;
                    }
                    const float bv = key_logit(M);
                    if (k == 0) tp = bv;
                    if (lane == k) {
                        mn = bv;
                        a.topi[t * a.topk + k] = bi;
                        ex[t * a.topk + k] = bi;
                    }
                }
                if (u) mine[1] = mn, top0[1] = tp;
                else mine[0] = mn, top0[0] = tp;
            }
        }
        float ek[2], z[2] = {0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 2; ++u) ek[u] = ex_expf(fsub(mine[u], top0[u]));
        for (int k = 0; k < a.topk; ++k)
#pragma unroll
            for (int u = 0; u < 2; ++u) z[u] = fadd(z[u], __shfl_sync(0xffffffffu, ek[u], k));
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (u < nu && lane < a.topk) a.topw[(tb + u * NW) * a.topk + lane] = fdiv(ek[u], z[u]);
    }
    __syncthreads();
    for (int p = e; p < P; p += RR_THREADS) {
        atomicOr(&rowmask[ex[p]], 1u << (p / a.topk));
        atomicMin(&firstpair[ex[p]], p);
    }
    __syncthreads();
    for (int p = e; p < P; p += RR_THREADS)
        if (firstpair[ex[p]] == p) atomicOr(&firstmask[p >> 5], 1u << (p & 31));
    __syncthreads();
    const int words = (P + 31) / 32;
    for (int p = e; p < P; p += RR_THREADS) {
        const int x = ex[p], fp = firstpair[x], t = p / a.topk;
        int j = 0;   // jobs that start before this pair's expert's first pair
        for (int k = 0; k < words; ++k) {
            if (32 * k + 31 < fp) j += __popc(firstmask[k]);
            else if (32 * k <= fp) j += __popc(firstmask[k] & ((1u << (fp - 32 * k)) - 1u));
        }
        const unsigned rows = rowmask[x];
        const int s = __popc(rows & ((1u << t) - 1u));
        a.gu[j].y[s] = t;
        a.gu[j].out[s] = a.dn[j].y[s] = a.dn[j].out[s] = p;
        if (fp == p) {
            a.gu[j].w = a.dn[j].w = x;
            a.gu[j].n = a.dn[j].n = __popc(rows);
        }
    }
    if (e == 0) {
        int n = 0;
        for (int k = 0; k < words; ++k) n += __popc(firstmask[k]);
        a.njobs[0] = n;
        a.njobs[1] = 0;
        *a.counter = 0u;
    }
}

// ================================================================ job activations in shared memory
// the job's q8_1 rows as an int8 plane [nj][n] (16-byte loads), the f16-rounded block scales and the blocks' integer
// sums [nj][n / 32]
struct JobAct {
    int8_t* q;
    float* d;
    int* s;
};
__device__ __forceinline__ JobAct job_act_carve(unsigned char* smem, int maxrows, int n) {
    JobAct a;
    a.q = reinterpret_cast<int8_t*>(smem);
    a.d = reinterpret_cast<float*>(smem + (size_t) maxrows * n);
    a.s = reinterpret_cast<int*>(smem + (size_t) maxrows * n + (size_t) maxrows * (n / 32) * 4);
    return a;
}
__host__ __device__ inline size_t job_act_bytes(int maxrows, int n) { return (size_t) maxrows * (n + (n / 32) * 8); }

__device__ __forceinline__ void job_act_stage(const JobAct& a, const uint8_t* __restrict__ xq, const FnxJob& jb, int n) {
    const int nb = n / 32;
    for (int it = threadIdx.x; it < jb.n * nb; it += blockDim.x) {
        const int j = it / nb, b = it % nb;
        const unsigned* src = reinterpret_cast<const unsigned*>(xq + ((size_t) jb.y[j] * nb + b) * 36);
        unsigned w[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) w[k] = src[k];
        int sum = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) sum = __dp4a(0x01010101, (int) w[1 + k], sum);
        uint4* dst = reinterpret_cast<uint4*>(a.q + (size_t) j * n + b * 32);
        dst[0] = make_uint4(w[1], w[2], w[3], w[4]);
        dst[1] = make_uint4(w[5], w[6], w[7], w[8]);
        a.d[j * nb + b] = h2f((uint16_t) (w[0] & 0xffff));
        a.s[j * nb + b] = sum;
    }
}

// ================================================================ gate|up, Q4_K (reference src/moe_q4k.cuh:30-109)
// 8 lanes a weight row; lane l owns the 64-value groups l + 8 i (32 bytes of nibbles + the super-block's 16-byte
// header: three 16-byte loads), all of a row's groups in flight at once; per group and activation row the integer
// sub-block dots, then d (d8l (sc0 dl) + d8h (sc1 dh)) - dmin (d8l (m0 sl) + d8h (m1 sh)) added in group order; the 8
// lanes combined by xor 4, 2, 1.
constexpr int GU_THREADS = 256;

// bytes of a taken as unsigned, of b as signed
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Read-once weights.  A lane's 16-byte pieces are halves of 32-byte sectors whose other halves the next load of the same
// lanes takes (a Q4_K superblock is 4.5 sectors long), so the lines do go through L1, first to leave: with L1 bypassed
// every sector crossed the L2 -> SM path twice.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Expert gate|up rows against the rows of x routed to the expert.  Each weight byte is used once and the work per byte
// is small, so what bounds the kernel is how many loads a multiprocessor keeps in flight: a lane group (8 lanes) owns
// GU_R consecutive rows and takes them two at a time, the 16-byte pieces of the step after the one being summed
// already on their way in a second set of registers (through a cp.async ring in shared memory instead, the ring's
// writes and reads saturated the shared-memory pipe).  A lane reads the activations of its column group from shared
// memory once per step and applies them to both rows; the rows of a job are taken GU_TC at a time (three jobs in four
// have one row, one in a hundred more than three) and the pipeline runs on across those passes.
// GU_R rows a lane group: four where an expert has many rows (a block then covers 128), two where the FF slice of a GPU
// leaves it a few hundred (twice the blocks, each half as long: the launch is over sooner)
constexpr int GU_TC = 2, GU_RS = 2, GU_MAGIC = 0x4B400000;

struct GuStep {   // one step's weights of a lane: two rows' header and 32 bytes of nibbles
    uint4 hdr[GU_RS], q0[GU_RS], q1[GU_RS];
};

template <int GPL, int GU_R>
__global__ void __launch_bounds__(GU_THREADS, 2) k_moe_gu_q4k(const uint8_t* __restrict__ A, size_t sa, int nrows, int n,
                                                          const FnxJob* __restrict__ jobs, const int* __restrict__ njobs,
                                                          const uint8_t* __restrict__ xq, float* __restrict__ out) {
    const int ji = blockIdx.y;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ FnxJob jb;
    pdl_wait();              // the jobs come from the kernel before
    pdl_go();
    const int nj = *njobs;   // read beside the job, not before it (the job array has a slot for every block row)
    if (threadIdx.x < sizeof(FnxJob) / 4) reinterpret_cast<int*>(&jb)[threadIdx.x] = reinterpret_cast<const int*>(jobs + ji)[threadIdx.x];
    if (ji >= nj) return;
    __syncthreads();
    const int lane8 = threadIdx.x & 7, nb = n / 32, jg = lane8 & 3;
    int8_t* aq = reinterpret_cast<int8_t*>(smem);                              // [GU_TC][n]
    float4* ag = reinterpret_cast<float4*>(smem + (size_t) GU_TC * n);         // [GU_TC][n / 64]: d8 low, d8 high, sum low, sum high
    const size_t row_b = (size_t) n / 256 * 144;
    constexpr int GU_RPB = GU_THREADS / 8 * GU_R;
    const int row0 = blockIdx.x * GU_RPB + (threadIdx.x >> 3) * GU_R;          // this lane group's GU_R consecutive rows
    const uint8_t* wrow = A + (size_t) jb.w * sa + (size_t) min(row0, nrows - 1) * row_b;
    unsigned roff[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int rr = 0; rr < GU_R; ++rr) roff[rr] = (unsigned) ((min(row0 + rr, nrows - 1) - min(row0, nrows - 1)) * row_b);
    // step s of a pass: rows 2 (s / GPL), +1 of the lane group, column group lane8 + 8 (s % GPL)
    constexpr int NS = GU_R / GU_RS * GPL;
    auto load = [&](GuStep& w, int s) {
        const int h = s / GPL, g = lane8 + (s % GPL) * 8;
#pragma unroll
        for (int rr = 0; rr < GU_RS; ++rr) {
            const uint8_t* blk = wrow + (h ? roff[GU_RS + rr] : roff[rr]) + (size_t) (g >> 2) * 144;
            w.hdr[rr] = ldg_stream(blk);
            w.q0[rr] = ldg_stream(blk + 16 + 32 * jg);
            w.q1[rr] = ldg_stream(blk + 32 + 32 * jg);
        }
    };
    float tmp[GU_RS][GU_TC];
    int cn = 0, c0 = 0;
    auto sums = [&](const GuStep& w, int s) {
        const int h = s / GPL, i = s % GPL, g = lane8 + i * 8, yb = (g >> 2) * 8 + jg * 2, sw = (g >> 1) & 3;   // sw: the staging's swizzle
        if (i == 0) {
#pragma unroll
            for (int rr = 0; rr < GU_RS; ++rr)
#pragma unroll
                for (int r = 0; r < GU_TC; ++r) tmp[rr][r] = 0.f;
        }
        float d[GU_RS], dmin[GU_RS], sc0[GU_RS], m0[GU_RS], sc1[GU_RS], m1[GU_RS];
#pragma unroll
        for (int rr = 0; rr < GU_RS; ++rr) {
            d[rr] = h2f((uint16_t) (w.hdr[rr].x & 0xffff)), dmin[rr] = h2f((uint16_t) (w.hdr[rr].x >> 16));
            q4k_scale_min_pair(w.hdr[rr], jg, sc0[rr], m0[rr], sc1[rr], m1[rr]);
        }
#pragma unroll
        for (int r = 0; r < GU_TC; ++r) {
            if (r >= cn) break;
            const uint4* ap = reinterpret_cast<const uint4*>(aq + (size_t) r * n + yb * 32);
            const uint4 a0 = ap[sw], a1 = ap[1 ^ sw], a2 = ap[2 ^ sw], a3 = ap[3 ^ sw];
            const float4 sg = ag[(size_t) r * (nb / 2) + (yb >> 1)];   // d8l, d8h, (float) sl, (float) sh
            const unsigned al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const unsigned ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
#pragma unroll
            for (int rr = 0; rr < GU_RS; ++rr) {
                const unsigned qw[8] = {w.q0[rr].x, w.q0[rr].y, w.q0[rr].z, w.q0[rr].w, w.q1[rr].x, w.q1[rr].y, w.q1[rr].z, w.q1[rr].w};
                int dl = GU_MAGIC, dh = GU_MAGIC;   // started at the bits of 1.5 * 2^23: as floats minus that, (float) dot
#pragma unroll
                for (int k = 0; k < 8; ++k) {   // the high nibbles stay where they are: their dot is 16 x the sub-block's, exactly
                    dl = dp4a_us(qw[k] & 0x0F0F0F0Fu, al[k], dl);
                    dh = dp4a_us(qw[k] & 0xF0F0F0F0u, ah[k], dh);
                }
                const float fl = fsub(__int_as_float(dl), 12582912.0f);
                const float fh = fmul(fsub(__int_as_float(dh), 12582912.0f), 0.0625f);
                const float pos = fmul(d[rr], fadd(fmul(sg.x, fmul(sc0[rr], fl)), fmul(sg.y, fmul(sc1[rr], fh))));
                const float neg = fmul(dmin[rr], fadd(fmul(sg.x, fmul(m0[rr], sg.z)), fmul(sg.y, fmul(m1[rr], sg.w))));
                tmp[rr][r] = fadd(tmp[rr][r], fsub(pos, neg));
            }
        }
        if (i == GPL - 1) {
#pragma unroll
            for (int rr = 0; rr < GU_RS; ++rr)
#pragma unroll
                for (int r = 0; r < GU_TC; ++r) {
                    if (r >= cn) break;
                    const float v = sum8(tmp[rr][r]);
                    const int row = row0 + h * GU_RS + rr;
                    if (lane8 == 0 && row < nrows) out[(size_t) jb.out[c0 + r] * nrows + row] = v;
                }
        }
    };
    GuStep w0, w1;
    load(w0, 0);   // the weights do not wait for the activations
#pragma unroll 1
    for (c0 = 0; c0 < jb.n; c0 += GU_TC) {
        cn = min(GU_TC, jb.n - c0);
        const bool more = c0 + GU_TC < jb.n;
        if (c0) __syncthreads();
        for (int it = threadIdx.x; it < cn * nb; it += GU_THREADS) {
            const int j = it / nb, b = it % nb;
            const unsigned* src = reinterpret_cast<const unsigned*>(xq + ((size_t) jb.y[c0 + j] * nb + b) * 36);
            unsigned w[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) w[k] = src[k];
            int sum = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) sum = __dp4a(0x01010101, (int) w[1 + k], sum);
            // 16-byte pieces swizzled inside each 64 bytes by the 64-byte group's index / 2: the eight lanes of a row
            // group read pieces 64 bytes apart, which would otherwise share two bank groups four ways
            uint4* dst = reinterpret_cast<uint4*>(aq + (size_t) j * n);
            const int u0 = 2 * b, sw = (u0 >> 3) & 3;
            dst[(u0 & ~3) | ((u0 & 3) ^ sw)] = make_uint4(w[1], w[2], w[3], w[4]);
            dst[(u0 & ~3) | (((u0 & 3) + 1) ^ sw)] = make_uint4(w[5], w[6], w[7], w[8]);
            float* gq = reinterpret_cast<float*>(ag + (size_t) j * (nb / 2) + (b >> 1));
            gq[b & 1] = h2f((uint16_t) (w[0] & 0xffff));
            gq[2 + (b & 1)] = (float) sum;
        }
        __syncthreads();
#pragma unroll 1
        for (int s = 0; s < NS; s += 2) {   // NS is even
            load(w1, s + 1);
            sums(w0, s);
            if (s + 2 < NS || more) load(w0, s + 2 < NS ? s + 2 : 0);
            sums(w1, s + 1);
        }
    }
}

// ================================================================ gate|up, split Q8_0 experts (reference src/moe.cuh:258-272
// with the in-tree Q8_0 order of src/dense.cuh:86-138)
// A row's result is the dense row dot: lane l adds fl(dw da) (float) isum16 over the 16-column pieces at
// c = 16 l + 512 k in ascending k, the 32 lanes meet by xor 16..1.  A warp takes G8_R rows at a time (their 16-byte
// loads of one step in flight together, the next step's behind them) against the job's rows, GU_TC at a time, staged in
// shared memory as an int8 plane and float scales.  With 1-2 rows per job the integer dots are a few dp4a: no tensor
// cores here.
// G8_WR rows a warp (G8_R at a time): sixteen where an expert has many rows, four where a GPU's FF slice leaves it a few
// hundred (four times the blocks, each a single pass: the launch is over sooner)
constexpr int G8_R = 4;

template <int G8_WR>
__global__ void __launch_bounds__(GU_THREADS, 3) k_moe_gu_q8(const int8_t* __restrict__ WQ, size_t sq, const uint16_t* __restrict__ WD,
                                                            size_t sd, int nrows, int n, const FnxJob* __restrict__ jobs,
                                                            const int* __restrict__ njobs, const uint8_t* __restrict__ xq,
                                                            float* __restrict__ out) {
    const int ji = blockIdx.y;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ FnxJob jb;
    pdl_wait();
    pdl_go();
    const int nj = *njobs;
    if (threadIdx.x < sizeof(FnxJob) / 4) reinterpret_cast<int*>(&jb)[threadIdx.x] = reinterpret_cast<const int*>(jobs + ji)[threadIdx.x];
    if (ji >= nj) return;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nb = n / 32;
    int8_t* aq = reinterpret_cast<int8_t*>(smem);                       // [GU_TC][n]
    float* ad = reinterpret_cast<float*>(smem + (size_t) GU_TC * n);    // [GU_TC][nb]
    const int8_t* wq = WQ + (size_t) jb.w * sq;
    const uint16_t* wd = WD + (size_t) jb.w * sd;
#pragma unroll 1
    for (int c0 = 0; c0 < jb.n; c0 += GU_TC) {
        const int cn = min(GU_TC, jb.n - c0);
        if (c0) __syncthreads();
        for (int it = threadIdx.x; it < cn * nb; it += GU_THREADS) {
            const int j = it / nb, b = it % nb;
            const unsigned* src = reinterpret_cast<const unsigned*>(xq + ((size_t) jb.y[c0 + j] * nb + b) * 36);
            uint4* dst = reinterpret_cast<uint4*>(aq + (size_t) j * n + b * 32);
            dst[0] = make_uint4(src[1], src[2], src[3], src[4]);
            dst[1] = make_uint4(src[5], src[6], src[7], src[8]);
            ad[it] = h2f((uint16_t) (src[0] & 0xffff));
        }
        __syncthreads();
#pragma unroll 1
        constexpr int G8_RPB = GU_THREADS / 32 * G8_WR;
        for (int r0 = blockIdx.x * G8_RPB + warp * G8_WR; r0 < blockIdx.x * G8_RPB + warp * G8_WR + G8_WR; r0 += G8_R) {
            if (r0 >= nrows) break;
            float acc[G8_R][GU_TC];
#pragma unroll
            for (int r = 0; r < G8_R; ++r)
#pragma unroll
                for (int t = 0; t < GU_TC; ++t) acc[r][t] = 0.f;
#pragma unroll 2
            for (int c = lane * 16; c < n; c += 512) {
                const int b = c >> 5;
                uint4 w[G8_R];
                float dw[G8_R];
#pragma unroll
                for (int r = 0; r < G8_R; ++r) {
                    const size_t row = (size_t) min(r0 + r, nrows - 1);
                    w[r] = ldg_stream(wq + row * n + c);
                    dw[r] = h2f(__ldg(wd + row * nb + b));
                }
#pragma unroll
                for (int t = 0; t < GU_TC; ++t) {
                    if (t >= cn) break;
                    const uint4 a = *reinterpret_cast<const uint4*>(aq + (size_t) t * n + c);
                    const float da = ad[t * nb + b];
#pragma unroll
                    for (int r = 0; r < G8_R; ++r) {
                        int sI = __dp4a((int) w[r].x, (int) a.x, GU_MAGIC);   // see GU_MAGIC: no convert instruction
                        sI = __dp4a((int) w[r].y, (int) a.y, sI);
                        sI = __dp4a((int) w[r].z, (int) a.z, sI);
                        sI = __dp4a((int) w[r].w, (int) a.w, sI);
                        acc[r][t] = ffma(fmul(dw[r], da), fsub(__int_as_float(sI), 12582912.0f), acc[r][t]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < G8_R; ++r)
#pragma unroll
                for (int t = 0; t < GU_TC; ++t) {
                    if (t >= cn) break;
                    const float v = wsum(acc[r][t]);
                    if (lane == 0 && r0 + r < nrows) out[(size_t) jb.out[c0 + t] * nrows + r0 + r] = v;
                }
        }
    }
}

// ================================================================ h = silu(gate) * up as int8 + scales
// a warp per (row, 32 columns) of gu rows [gate (ffs) | up (ffs)]: the q8_1 rounding with the scale kept as the float
// of its f16 value (reference src/moe.cuh:284-295, src/dense.cuh:187-194).  hq: int8 [rows][ffs], then float
// [rows][ffs / 32] from hq + rows_cap * ffs
__global__ void __launch_bounds__(256) k_swiglu_q8(const float* __restrict__ gu, int ffs, int nrows, int8_t* __restrict__ hq,
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

// ================================================================ down, Q6_K in 32-column units
// thread per unit (16 B low nibbles, 8 B high bits, 2 int8 scales, f16 d: all coalesced across a warp's consecutive
// units); unit value d (d8 (float) (sc0 isum0 + sc1 isum1)) per activation row into shared memory; then a row's units
// added in ascending order (reference src/moe.cuh:330-344).
constexpr int DN_THREADS = 256;

constexpr int DN_TC = 2, DN_UPT = 3;   // activation rows a pass; weight rows a thread
// row groups a block (dnk): four when rows are wide, fewer for a GPU's narrow FF slice (a pass then covers many rows and
// the blocks would be few and long)
static int dn_groups(int nu) { return nu <= 6 ? 1 : nu <= 12 ? 2 : 4; }

// Thread (u, r) takes 32-column unit u of rows r, r + RP, r + 2 RP of a row group (RP = 256 / units-per-row rows a pass),
// so the activations of its unit are read from shared memory once per activation row and used for three weight rows:
// the kernel is bound by the shared-memory data pipe otherwise.  Lanes run over consecutive units of consecutive rows,
// so every plane is read in contiguous 16-, 8- and 2-byte pieces.  A block stages the job's activation rows once and
// walks dnk row groups, the next group's weights on their way while this group's are summed: a block's life is a
// chain of dependent global reads (job, weights, activations) and short sums, so the reads are issued as early as
// their addresses are known.
struct DnRaw {
    uint4 ql[DN_UPT], qx[DN_UPT];   // qx: the second 16 bytes of a Q8_0 unit
    uint2 qh[DN_UPT];
    unsigned scw[DN_UPT], dh[DN_UPT];
};

// Q8: the same walk over split Q8_0 experts (reference src/moe.cuh:299-345 with the Q8_0 unit value of src/dense.cuh):
// a unit is 32 int8 values (QL: two 16-byte pieces) and an f16 scale (D); unit value (dw d8) (float) isum.
template <bool Q8>
__global__ void __launch_bounds__(DN_THREADS, 3) k_moe_down_q6p(const uint4* __restrict__ QL, const uint2* __restrict__ QH,
                                                               const uint16_t* __restrict__ SC, const uint16_t* __restrict__ D,
                                                               size_t expert_units, int nrows, int ffs, const FnxJob* __restrict__ jobs,
                                                               const int* __restrict__ njobs, const int8_t* __restrict__ hq,
                                                               const float* __restrict__ hd, float* __restrict__ out, int dnk) {
    const int ji = blockIdx.y;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ FnxJob jb;
    // the jobs are older than the kernel before this one (the SwiGLU of the pairs), so the job and this block's first
    // weights are read while that kernel still runs
    const int nj = *njobs;   // read beside the job, not before it (the job array has a slot for every block row)
    if (threadIdx.x < sizeof(FnxJob) / 4) reinterpret_cast<int*>(&jb)[threadIdx.x] = reinterpret_cast<const int*>(jobs + ji)[threadIdx.x];
    if (ji >= nj) return;
    __syncthreads();
    const int nu = ffs / 32, RP = DN_THREADS / nu, rpb = RP * DN_UPT, pu = nu + 1;   // pu: padded units a row in `part`
    const int jn = min(jb.n, FNX_MAXT);
    uint4* sq = reinterpret_cast<uint4*>(smem);                                   // [jn][2 halves][nu] 16 bytes each
    float* sd = reinterpret_cast<float*>(sq + (size_t) FNX_MAXT * 2 * nu);        // [jn][nu]
    int2* ss = reinterpret_cast<int2*>(sd + (size_t) FNX_MAXT * nu);              // [jn][nu]: 32 x the sums of each half
    float* part = reinterpret_cast<float*>(ss + (size_t) FNX_MAXT * nu);          // [2][DN_TC][rpb][pu]
    const int rowB = blockIdx.x * rpb * dnk, u = threadIdx.x % nu, r = threadIdx.x / nu;
    const bool active = r < RP;
    auto load = [&](DnRaw& w, int row0) {
#pragma unroll
        for (int k = 0; k < DN_UPT; ++k) {
            const int row = min(row0 + k * RP + min(r, RP - 1), nrows - 1);
            const size_t g = (size_t) jb.w * expert_units + (size_t) row * nu + u;
            if (Q8) {
                w.ql[k] = ldg_stream(QL + 2 * g);
                w.qx[k] = ldg_stream(QL + 2 * g + 1);
            } else {
                w.ql[k] = ldg_stream(QL + g);
                w.qh[k] = __ldg(QH + g);
                w.scw[k] = SC[g];
            }
            w.dh[k] = D[g];
        }
    };
    DnRaw raw;
    load(raw, rowB);
    pdl_wait();   // the pairs' h
    pdl_go();
    for (int it = threadIdx.x; it < jn * nu; it += DN_THREADS) {
        const int j = it / nu, uu = it % nu;
        sd[it] = hd[(size_t) jb.y[j] * nu + uu];
        const uint4* hp = reinterpret_cast<const uint4*>(hq + (size_t) jb.y[j] * ffs + uu * 32);
        const uint4 h0 = hp[0], h1 = hp[1];
        sq[(size_t) (j * 2) * nu + uu] = h0;        // the two halves in planes of their own: a warp's 16-byte reads
        sq[(size_t) (j * 2 + 1) * nu + uu] = h1;    // are contiguous
        int s0 = __dp4a(0x01010101, (int) h0.x, 0), s1 = __dp4a(0x01010101, (int) h1.x, 0);
        s0 = __dp4a(0x01010101, (int) h0.y, s0), s1 = __dp4a(0x01010101, (int) h1.y, s1);
        s0 = __dp4a(0x01010101, (int) h0.z, s0), s1 = __dp4a(0x01010101, (int) h1.z, s1);
        s0 = __dp4a(0x01010101, (int) h0.w, s0), s1 = __dp4a(0x01010101, (int) h1.w, s1);
        ss[it] = make_int2(32 * s0, 32 * s1);
    }
    __syncthreads();
    int buf = 0;
#pragma unroll 1
    for (int kk = 0; kk < dnk; ++kk) {
        const int row0 = rowB + kk * rpb;
        if (row0 >= nrows) break;
        // this group's weights: codes 0..63 (the -32 goes through ss), kept for every pass over the job's rows
        unsigned v[DN_UPT][8];
        float d[DN_UPT];
        int sc0[DN_UPT], sc1[DN_UPT];
#pragma unroll
        for (int k = 0; k < DN_UPT; ++k) {
            d[k] = h2f((uint16_t) raw.dh[k]);
            const unsigned lw[4] = {raw.ql[k].x, raw.ql[k].y, raw.ql[k].z, raw.ql[k].w};
            if (Q8) {
                const unsigned xw[4] = {raw.qx[k].x, raw.qx[k].y, raw.qx[k].z, raw.qx[k].w};
                sc0[k] = sc1[k] = 1;
#pragma unroll
                for (int w = 0; w < 4; ++w) v[k][w] = lw[w], v[k][4 + w] = xw[w];
            } else {
                sc0[k] = (int) (int8_t) (raw.scw[k] & 0xff), sc1[k] = (int) (int8_t) (raw.scw[k] >> 8);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    v[k][w] = (lw[w] & 0x0F0F0F0Fu) | (((raw.qh[k].x >> (2 * w)) & 0x03030303u) << 4);
                    v[k][4 + w] = ((lw[w] >> 4) & 0x0F0F0F0Fu) | (((raw.qh[k].y >> (2 * w)) & 0x03030303u) << 4);
                }
            }
        }
        if (kk + 1 < dnk && row0 + rpb < nrows) load(raw, row0 + rpb);
        const int live_rows = min(rpb, nrows - row0);
#pragma unroll 1
        for (int c0 = 0; c0 < jn; c0 += DN_TC) {
            const int cn = min(DN_TC, jn - c0);
            float* pt = part + (size_t) buf * DN_TC * rpb * pu;
            if (active) {
#pragma unroll
                for (int j = 0; j < DN_TC; ++j) {
                    if (j >= cn) break;
                    const int jj = c0 + j;
                    const uint4 a0 = sq[(size_t) (jj * 2) * nu + u], a1 = sq[(size_t) (jj * 2 + 1) * nu + u];
                    int2 bias = ss[jj * nu + u];   // sum (code - 32) a = sum code a - 32 sum a, exactly
                    if (Q8) bias = make_int2(0, 0);
                    const float dj = sd[jj * nu + u];
#pragma unroll
                    for (int k = 0; k < DN_UPT; ++k) {
                        int is0 = __dp4a((int) v[k][0], (int) a0.x, -bias.x);
                        is0 = __dp4a((int) v[k][1], (int) a0.y, is0);
                        is0 = __dp4a((int) v[k][2], (int) a0.z, is0);
                        is0 = __dp4a((int) v[k][3], (int) a0.w, is0);
                        int is1 = __dp4a((int) v[k][4], (int) a1.x, -bias.y);
                        is1 = __dp4a((int) v[k][5], (int) a1.y, is1);
                        is1 = __dp4a((int) v[k][6], (int) a1.z, is1);
                        is1 = __dp4a((int) v[k][7], (int) a1.w, is1);
                        const int I = Q8 ? is0 + is1 : sc0[k] * is0 + sc1[k] * is1;
                        pt[((size_t) j * rpb + k * RP + r) * pu + u] = Q8 ? fmul(fmul(d[k], dj), (float) I) : fmul(d[k], fmul(dj, (float) I));
                    }
                }
            }
            __syncthreads();   // the one barrier of a pass: the next pass writes the other half of `part`
            for (int e = threadIdx.x; e < cn * live_rows; e += DN_THREADS) {
                const int j = e / live_rows, rr = e % live_rows;
                const float* pr = pt + ((size_t) j * rpb + rr) * pu;
                float s = 0.f;
                for (int k0 = 0; k0 < nu; k0 += 8) {   // the loads of eight units ahead of their ordered sums
                    float t[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) t[k] = pr[min(k0 + k, nu - 1)];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (k0 + k < nu) s = fadd(s, t[k]);
                }
                out[(size_t) jb.out[c0 + j] * nrows + row0 + rr] = s;
            }
            buf ^= 1;
        }
    }
}

// ================================================================ combine (reference src/kernels.cu:797-803)
__global__ void __launch_bounds__(256) k_moe_combine(const float* __restrict__ part, const float* __restrict__ topw,
                                                     const float* __restrict__ sh, const float* __restrict__ logits, int nexp,
                                                     float* __restrict__ out, int n, int topk) {
    const int t = blockIdx.y, i = blockIdx.x * 256 + threadIdx.x;
    pdl_wait();
    pdl_go();
    if (i >= n) return;
    float s = 0.f;
    for (int k = 0; k < topk; ++k) s = ffma(topw[t * topk + k], part[((size_t) t * topk + k) * n + i], s);
    out[(size_t) t * n + i] = ffma(ex_sigmoid(logits[(size_t) t * (nexp + 1) + nexp]), sh[(size_t) t * n + i], s);
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

size_t fnx_router_scratch_bytes(void) { return 16; }

int fnx_router_route(const float* W, const float* x, float* logits, int T, int n, int nexp, int topk, int* topi, float* topw,
                     FnxJob* jobs_gu, FnxJob* jobs_dn, int* njobs, void* scratch, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "router_route: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(n > 0 && n % 256 == 0 && n <= 4096, "router_route: n %d must be a multiple of 256 up to 4096", n);
    FNX_REQUIRE(nexp % 32 == 0 && nexp >= 32 && nexp <= 512, "router_route: %d experts (a multiple of 32 up to 512)", nexp);
    FNX_REQUIRE(topk >= 1 && topk <= 16 && topk <= nexp, "router_route: top-%d", topk);
    unsigned* fault = device_fault_word();
    FNX_REQUIRE(fault, "router_route: no device fault word (no current device?)");
    RouterArgs a{W, x, logits, T, n, nexp, topk, topi, topw, jobs_gu, jobs_dn, njobs, (unsigned*) scratch, fault};
    // a block per four rows of W, every block with all of x in its shared memory when it fits (bulk copies: 16-byte
    // aligned rows); else straight from the L2
    const size_t xbytes = (size_t) T * n * 4;
    const bool fits = xbytes <= 200 * 1024 && ((uintptr_t) x % 16) == 0;
    int grid = (nexp + 1 + RR_ROWS - 1) / RR_ROWS;
    if (grid > 148) grid = 148;
    if (fits) {
        if (smem_optin(k_router_route<true>, xbytes, "router_route")) return 1;
        launch(2, k_router_route<true>, grid, RR_THREADS, xbytes, strm(st), a);
    } else {
        launch(2, k_router_route<false>, grid, RR_THREADS, 0, strm(st), a);
    }
    return launch_ok("router_route");
}

size_t fnx_moe_h_bytes(int pairs, int ffs) { return (size_t) pairs * ffs + (size_t) pairs * (ffs / 32) * 4; }

int fnx_moe_gate_up(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const void* xq, float* gu, void* st) {
    FNX_REQUIRE(A && njobs_max >= 1, "moe_gate_up: no experts or jobs");
    const int n = A->ncols, nrows = A->nrows, maxrows = FNX_MAXT;
    if (A->type == FNX_Q4_K) {
        FNX_REQUIRE(n % 512 == 0 && n / 512 >= 1 && n / 512 <= 8, "moe gate|up q4_K: %d columns (multiples of 512 up to 4096)", n);
        // blocks of 128 rows with direct 16-byte loads one step ahead (measured faster than staging the weights through
        // shared memory, by cp.async rings or bulk copies: there every operand crosses the shared-memory pipe)
        const int R = nrows <= 512 && (n / 512) % 2 == 0 ? 2 : 4, rpb = GU_THREADS / 8 * R;   // the step count must stay even
        const dim3 grid((nrows + rpb - 1) / rpb, njobs_max);
        const size_t sm = (size_t) GU_TC * (n + (n / 64) * 16);
        const uint8_t* a = (const uint8_t*) A->a;
#define GU_LAUNCH(G, RR)                                                                                                          \
    {                                                                                                                             \
        if (smem_optin(k_moe_gu_q4k<G, RR>, sm, "moe gate|up q4_K")) return 1;                                                    \
        launch(3, k_moe_gu_q4k<G, RR>, grid, GU_THREADS, sm, strm(st), a, A->stride, nrows, n, jobs, njobs, (const uint8_t*) xq, gu); \
    }
#define GU_CASE(G)                      \
    case G:                             \
        if (R == 2) GU_LAUNCH(G, 2)     \
        else GU_LAUNCH(G, 4)            \
        break;
        switch (n / 512) {
            GU_CASE(1) GU_CASE(2) GU_CASE(3) GU_CASE(4) GU_CASE(5) GU_CASE(6) GU_CASE(7) GU_CASE(8)
        }
#undef GU_CASE
#undef GU_LAUNCH
        return launch_ok("moe gate|up q4_K");
    }
    if (A->type == FNX_Q8_0) {
        FNX_REQUIRE(n % 32 == 0 && ((uintptr_t) A->a % 16) == 0 && A->stride % 16 == 0 && n % 16 == 0,
                    "moe gate|up q8_0: %d columns, planes 16-byte aligned", n);
        const int wr = nrows <= 512 ? 4 : 16, rpb = GU_THREADS / 32 * wr;
        const dim3 grid((nrows + rpb - 1) / rpb, njobs_max);
        const size_t sm = (size_t) GU_TC * (n + (n / 32) * 4);
        if (wr == 4) {
            if (smem_optin(k_moe_gu_q8<4>, sm, "moe gate|up q8_0")) return 1;
            launch(3, k_moe_gu_q8<4>, grid, GU_THREADS, sm, strm(st), (const int8_t*) A->a, A->stride, (const uint16_t*) A->b, A->stride_b / 2, nrows, n,
                   jobs, njobs, (const uint8_t*) xq, gu);
        } else {
            if (smem_optin(k_moe_gu_q8<16>, sm, "moe gate|up q8_0")) return 1;
            launch(3, k_moe_gu_q8<16>, grid, GU_THREADS, sm, strm(st), (const int8_t*) A->a, A->stride, (const uint16_t*) A->b, A->stride_b / 2, nrows, n,
                   jobs, njobs, (const uint8_t*) xq, gu);
        }
        return launch_ok("moe gate|up q8_0");
    }
    return fail("moe_gate_up: expert type %d not supported (Q4_K, Q8_0)", A->type);
}

int fnx_mmvq(const FnxExperts* W, const FnxJob* jobs, const int* njobs, int njobs_max, const void* y, float* out, int out_stride, void* st) {
    FNX_REQUIRE(W && out_stride == W->nrows, "mmvq: output rows of %d values only (the matrix's rows)", W ? W->nrows : 0);
    FNX_REQUIRE(W->type == FNX_Q4_K || W->type == FNX_Q8_0, "mmvq: weight type %d not handled (Q4_K, Q8_0)", W->type);
    return fnx_moe_gate_up(W, jobs, njobs, njobs_max, y, out, st);
}

int fnx_moe_down(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const float* gu, int npairs, void* hq,
                 float* part, void* st) {
    FNX_REQUIRE(A && njobs_max >= 1 && npairs >= 1, "moe_down: no experts, jobs or pairs");
    const int ffs = A->ncols, nrows = A->nrows, maxrows = FNX_MAXT;
    FNX_REQUIRE(ffs % 32 == 0 && ffs > 0, "moe_down: ff width %d not a multiple of 32", ffs);
    int8_t* h8 = (int8_t*) hq;
    float* hd = (float*) ((char*) hq + (size_t) npairs * ffs);
    FNX_REQUIRE(((size_t) npairs * ffs) % 16 == 0 && ffs % 16 == 0, "moe_down: h rows must be 16-byte multiples");
    launch(0, k_swiglu_q8, (npairs * (ffs / 32) + 7) / 8, 256, 0, strm(st), gu, ffs, npairs, h8, hd);
    if (launch_ok("moe_down swiglu")) return 1;
    if (A->type == FNX_Q6_K) {
        const int nu = ffs / 32;
        FNX_REQUIRE(nu <= DN_THREADS, "moe_down: ff width %d too wide for a block", ffs);
        const int rpb = DN_THREADS / nu * DN_UPT;
        const size_t sm = (size_t) FNX_MAXT * nu * (32 + 4 + 8) + (size_t) 2 * DN_TC * rpb * (nu + 1) * 4;
        if (smem_optin(k_moe_down_q6p<false>, sm, "moe_down q6_K")) return 1;
        const int dnk = dn_groups(nu);
        const dim3 grid((nrows + rpb * dnk - 1) / (rpb * dnk), njobs_max);
        launch(4, k_moe_down_q6p<false>, grid, DN_THREADS, sm, strm(st), (const uint4*) A->a, (const uint2*) A->b, (const uint16_t*) A->c,
               (const uint16_t*) A->d, A->stride, nrows, ffs, jobs, njobs, (const int8_t*) h8, (const float*) hd, part, dnk);
        return launch_ok("moe_down q6_K");
    }
    if (A->type == FNX_Q8_0) {   // expert e: values at a + e stride (nrows x ffs int8), scales at b + e stride_b
        const int nu = ffs / 32;
        FNX_REQUIRE(nu <= DN_THREADS, "moe_down: ff width %d too wide for a block", ffs);
        FNX_REQUIRE(((uintptr_t) A->a % 16) == 0 && A->stride == (size_t) nrows * ffs && A->stride_b == (size_t) nrows * nu * 2,
                    "moe_down q8_0: experts must be dense planes of %d x %d", nrows, ffs);
        const int rpb = DN_THREADS / nu * DN_UPT;
        const size_t sm = (size_t) FNX_MAXT * nu * (32 + 4 + 8) + (size_t) 2 * DN_TC * rpb * (nu + 1) * 4;
        if (smem_optin(k_moe_down_q6p<true>, sm, "moe_down q8_0")) return 1;
        const int dnk = dn_groups(nu);
        const dim3 grid((nrows + rpb * dnk - 1) / (rpb * dnk), njobs_max);
        launch(4, k_moe_down_q6p<true>, grid, DN_THREADS, sm, strm(st), (const uint4*) A->a, (const uint2*) nullptr, (const uint16_t*) nullptr,
               (const uint16_t*) A->b, (size_t) nrows * nu, nrows, ffs, jobs, njobs, (const int8_t*) h8, (const float*) hd, part, dnk);
        return launch_ok("moe_down q8_0");
    }
    return fail("moe_down: expert type %d not supported (Q6_K units, Q8_0)", A->type);
}

// ---- the down projection for callers that cannot allocate device memory
// Some hosts of these kernels have no allocator to give: a plug-in running inside another engine's captured stream, a
// callback with a fixed memory budget, a process whose allocations are all made at start-up by someone else.  For them the
// scratch of fnx_moe_down (the pairs' quantised h) lives in the library itself: a file-scope device array of
// FNX_DOWN_NOALLOC_BYTES, resident on every GPU that loads the library until the process exits.
static __device__ __align__(256) unsigned char g_down_scratch[FNX_DOWN_NOALLOC_BYTES];

// In host code the array's name is only a handle for the runtime, not a device address; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.  The per-device cache below is read and written
// without synchronisation: two host threads that meet here for the same device both ask the runtime and both store the
// same address (the write is idempotent and pointer-sized), so the race is benign and costs at most one extra lookup.
static void* down_scratch_ptr(void) {
    static void* ptr[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fail("moe_down_noalloc: no current device");
        return nullptr;
    }
    if (!ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_down_scratch);
        if (e != cudaSuccess) {
            fail("moe_down_noalloc: scratch address: %s", cudaGetErrorString(e));
            return nullptr;
        }
        ptr[dev] = p;
    }
    return ptr[dev];
}

int fnx_moe_down_noalloc(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const float* gu, int npairs,
                         float* part, void* st) {
    FNX_REQUIRE(A && npairs >= 1, "moe_down_noalloc: no experts or pairs");
    const size_t need = fnx_moe_h_bytes(npairs, A->ncols);
    FNX_REQUIRE(need <= FNX_DOWN_NOALLOC_BYTES, "moe_down_noalloc: %d pairs x ff %d need %zu bytes of scratch, the built-in array holds %d",
                npairs, A->ncols, need, FNX_DOWN_NOALLOC_BYTES);
    void* hq = down_scratch_ptr();
    if (!hq) return 1;
    // every byte of the scratch that is read is written first by this call (the pairs' h), so nothing needs clearing
    return fnx_moe_down(A, jobs, njobs, njobs_max, gu, npairs, hq, part, st);
}

int fnx_moe_combine(const float* part, const float* topw, const float* sh, const float* logits, int nexp, float* out, int T,
                    int n, int topk, void* st) {
    FNX_REQUIRE(T >= 1 && n >= 1, "moe_combine: empty");
    launch(0, k_moe_combine, dim3((n + 255) / 256, T), 256, 0, strm(st), part, topw, sh, logits, nexp, out, n, topk);
    return launch_ok("moe_combine");
}
}
