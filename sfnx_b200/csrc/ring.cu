// All-reduce(sum) of the window's rows across the GPUs of one box, in the reference ring's order, over peer memory.
// Replaces reference src/kernels.cu:755-868 (k_ring) / src/kernels.hpp:321-353 (ring_sum, Ring) for the fp32 payload.
//
// The reference passes chunk c (pairs [c NP / n, (c + 1) NP / n) of the NP float pairs) around a ring that starts at
// GPU c (chunks are cut within each row), every GPU adding its addend in turn: ((x_c + x_{c+1}) + ...) + x_{c+n-1}.  Behind an NVSwitch every GPU reaches
// every peer at full bandwidth, so here nothing is passed on: each GPU publishes its addend in a slot its peers can
// read, tells them so, waits until all of them have published, and then adds the n addends of every chunk itself in the
// ring's order with plain peer loads.  One launch, one exchange of flags, the same bits as the ring on every GPU.
//
// Slots come in two parities so that a slot is rewritten only two sums later: a GPU can be that far only after every
// peer has signalled the sum in between, which a peer does after it has finished reading the older slot.
// Every wait is bounded: when a peer's flag does not arrive within `spin_limit` polls the kernel sets bit 1 of the
// error word (the reference's "peer value never came", src/kernels.hpp:335) and goes on; the context stays usable.
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"
#include "exact_math.cuh"

namespace cg = cooperative_groups;

namespace fnxk {

constexpr int RS_THREADS = 256;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ float ld_cg(const float* p) {   // peer memory: not through L1
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_peer(const float* p) {   // peer memory: not through L1
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// ---- the window's own exchanges: a value and the exchange's number in one 8-byte store into the reader's memory
// ("LL" words, as the reference's ring stores them, src/kernels.cu:755-868).  The store is one transaction, so a reader
// that sees the number sees the value: no flag, no fence, one one-way trip.  An area is rewritten two exchanges later,
// which a GPU can reach only after every peer has sent the exchange in between, i.e. after it has read this one.
__device__ __forceinline__ void ll_store(unsigned long long* p, unsigned bits, unsigned epoch) {
    asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(epoch) : "memory");
}
// polls this GPU's own memory (not through L1) until the word carries `epoch`; gives up after `limit` polls (bit 1 of *err)
__device__ __forceinline__ unsigned ll_load(const unsigned long long* p, unsigned epoch, unsigned limit, unsigned* err) {
    unsigned x, y, spins = 0;
    for (;;) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "l"(p) : "memory");
        if (y == epoch) return x;
        if (++spins >= limit) {
            atomicOr(err, 1u);
            return 0u;
        }
        if (spins > 8) __nanosleep(32);
    }
}

__global__ void __launch_bounds__(RS_THREADS) k_ring_sum(float* __restrict__ x, int count, int row_len, const FnxRing ring, unsigned* err) {
    const int n = ring.nrank, me = ring.rank, tid = threadIdx.x;
    unsigned* state = ring.state;              // [0] sums done so far, [1] blocks that have published, [2] blocks that are done
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(state) + 1u;
    const int parity = (int) (epoch & 1u);
    float* mine = ring.slot[parity][me];
    // ---- publish this GPU's addend
    const int n4 = count / 4;
    for (int i = blockIdx.x * RS_THREADS + tid; i < n4; i += gridDim.x * RS_THREADS)
        reinterpret_cast<float4*>(mine)[i] = reinterpret_cast<const float4*>(x)[i];
    __threadfence_system();
    __syncthreads();
    __shared__ bool last;
    if (tid == 0) last = atomicAdd(&state[1], 1u) == gridDim.x - 1;
    __syncthreads();
    if (last) {   // the whole addend is in the slot: tell every peer (its flag word for this GPU)
        __threadfence_system();
        if (tid < n && tid != me) st_release_sys(ring.pad[tid] + me, epoch);
        if (tid == 0) state[1] = 0u;
    }
    // ---- wait until every peer has published this sum's addend
    if (tid < n && tid != me) {
        const unsigned* flag = ring.pad[me] + tid;
        unsigned spins = 0;
        while ((int) (ld_acquire_sys(flag) - epoch) < 0) {
            if (++spins >= ring.spin_limit) {
                atomicOr(err, 1u);
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    // ---- every chunk's addends in the ring's order: chunk c of a row (its pairs [c NP / n, (c + 1) NP / n)) starts at GPU c
    const int NP = row_len / 2;
    auto chunk_of = [&](int p) {   // the chunk that holds pair p of a row
        int c = (int) ((long long) p * n / NP);
        while (c + 1 < n && (long long) (c + 1) * NP / n <= p) ++c;
        while (c > 0 && (long long) c * NP / n > p) --c;
        return c;
    };
    for (int i = blockIdx.x * RS_THREADS + tid; i < n4; i += gridDim.x * RS_THREADS) {
        const int p0 = (4 * i % row_len) / 2;   // a float4 is two pairs of one row (row_len % 4 == 0)
        const int ca = chunk_of(p0), cb = chunk_of(p0 + 1);
        float4 v[FNX_RING_MAX];
#pragma unroll
        for (int r = 0; r < FNX_RING_MAX; ++r)
            if (r < n) v[r] = r == me ? reinterpret_cast<const float4*>(mine)[i] : ld_peer(ring.slot[parity][r] + 4 * (size_t) i);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < FNX_RING_MAX; ++k)
            if (k < n) {
                const int ra = ca + k < n ? ca + k : ca + k - n, rb = cb + k < n ? cb + k : cb + k - n;
                float ax = 0.f, ay = 0.f, bz = 0.f, bw = 0.f;
#pragma unroll
                for (int r = 0; r < FNX_RING_MAX; ++r) {   // selects, not indexing: the addends stay in registers
                    if (r == ra) ax = v[r].x, ay = v[r].y;
                    if (r == rb) bz = v[r].z, bw = v[r].w;
                }
                if (k == 0) acc = make_float4(ax, ay, bz, bw);
                else acc.x = fadd(acc.x, ax), acc.y = fadd(acc.y, ay), acc.z = fadd(acc.z, bz), acc.w = fadd(acc.w, bw);
            }
        reinterpret_cast<float4*>(x)[i] = acc;
    }
    // ---- the last block out counts the sum
    __syncthreads();
    if (tid == 0 && atomicAdd(&state[2], 1u) == gridDim.x - 1) {
        state[2] = 0u;
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(state) = epoch;
    }
}

// ---------------------------------------------------------------- a half layer's boundary in one launch
// What sits between two halves of a layer, in one kernel instead of three: the addend of the half that ended (its
// output rows, or the routed experts' rows weighted and added with the gated shared expert: reference src/kernels.cu:
// 797-806, ring_x), the sum of the GPUs' addends in the ring's order (k_ring_sum's, over the ring's receive areas: every
// value goes to every peer as a value + exchange number word), the residual update x += sum, and the RMS norm of the new x with its q8_1 copy for the half that begins
// (k_rms_norm_rows' order of sums).  A cluster of eight blocks per row (see the kernel).
struct BoundaryArgs {
    float* x;
    const float* bo;
    FnxMoeRows moe;
    FnxRing ring;
    const float* w;
    float* y;
    uint8_t* q;
    int n;
    float eps;
    unsigned* err;
};
constexpr int BD_THREADS = 1024, BD_MAXN = 4096, BD_CL = 8, BD_CT = BD_THREADS / BD_CL, BD_MAXC = BD_MAXN / BD_THREADS;

__device__ __forceinline__ void bd_q8_1_store(float xi, uint8_t* blk, int lane) {
    const float amax = wmax(fabsf(xi)), sum = wsum(xi);
    const float d = fdiv(amax, 127.0f);
    reinterpret_cast<int8_t*>(blk + 4)[lane] = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
    if (lane == 0) {
        reinterpret_cast<uint16_t*>(blk)[0] = f2h(d);
        reinterpret_cast<uint16_t*>(blk)[1] = f2h(sum);
    }
}

// A row is the work of 1024 "virtual" threads - thread i owns columns i, i + 1024, ... and the 32 warps' square sums are
// added in warp order, which is k_rms_norm_rows' order of sums - spread over a cluster of eight blocks of 128 threads:
// a row's loads (ten expert rows a column) come from eight SMs instead of one, and the norm's 32 partial sums meet
// through distributed shared memory.  The values stay in registers between the steps.
__global__ void __cluster_dims__(BD_CL, 1, 1) __launch_bounds__(BD_CT) k_boundary_rows(const BoundaryArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float sh[32];   // every block of the cluster gets all 32 warp sums
    const int t = blockIdx.x / BD_CL, cr = blockIdx.x % BD_CL, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int vt = cr * BD_CT + tid, n = a.n, nr = a.ring.nrank, me = a.ring.rank;
    float* xr = a.x + (size_t) t * n;
    pdl_wait();
    pdl_go();
    const bool has_add = a.bo || a.moe.part;
    // ---- this GPU's addend of the row, this thread's columns
    float add[BD_MAXC];
#pragma unroll
    for (int k = 0; k < BD_MAXC; ++k) add[k] = 0.f;
    if (a.moe.part) {
        const int topk = a.moe.topk;
        const float gate = ex_sigmoid(a.moe.logits[(size_t) t * (a.moe.nexp + 1) + a.moe.nexp]);
#pragma unroll
        for (int k = 0; k < BD_MAXC; ++k) {
            const int i = vt + BD_THREADS * k;
            if (i < n) {
                float s = 0.f;
                for (int kk = 0; kk < topk; ++kk) s = ffma(a.moe.topw[t * topk + kk], a.moe.part[((size_t) t * topk + kk) * n + i], s);
                add[k] = ffma(gate, a.moe.sh[(size_t) t * n + i], s);
            }
        }
    } else if (a.bo) {
#pragma unroll
        for (int k = 0; k < BD_MAXC; ++k) {
            const int i = vt + BD_THREADS * k;
            if (i < n) add[k] = a.bo[(size_t) t * n + i];
        }
    }
    if (nr > 1 && has_add) {
        unsigned* state = a.ring.state;
        const unsigned epoch = *reinterpret_cast<volatile unsigned*>(state) + 1u;
        const int parity = (int) (epoch & 1u);
        const size_t cnt = a.ring.ll_count;
        // ---- this thread's values to every peer's receive area, then the peers' values out of this GPU's own
#pragma unroll
        for (int k = 0; k < BD_MAXC; ++k) {
            const int i = vt + BD_THREADS * k;
            if (i < n) {
#pragma unroll
                for (int r = 0; r < FNX_RING_MAX; ++r)
                    if (r < nr && r != me) ll_store(a.ring.ll[parity][r] + (size_t) me * cnt + (size_t) t * n + i, __float_as_uint(add[k]), epoch);
            }
        }
        float pv[BD_MAXC][FNX_RING_MAX];
#pragma unroll
        for (int k = 0; k < BD_MAXC; ++k) {
            const int i = vt + BD_THREADS * k;
#pragma unroll
            for (int r = 0; r < FNX_RING_MAX; ++r) {
                pv[k][r] = 0.f;
                if (i < n && r < nr)
                    pv[k][r] = r == me ? add[k]
                                       : __uint_as_float(ll_load(a.ring.ll[parity][me] + (size_t) r * cnt + (size_t) t * n + i, epoch, a.ring.spin_limit, a.err));
            }
        }
        const int NP = n / 2;
#pragma unroll
        for (int k = 0; k < BD_MAXC; ++k) {
            const int i = vt + BD_THREADS * k;
            if (i < n) {   // the chunk that holds the column's pair starts the ring's order (NP * nr fits 32 bits)
                const int p = i / 2;
                int c = p * nr / NP;
                while (c + 1 < nr && (c + 1) * NP / nr <= p) ++c;
                while (c > 0 && c * NP / nr > p) --c;
                float acc = 0.f;
#pragma unroll
                for (int kk = 0; kk < FNX_RING_MAX; ++kk)
                    if (kk < nr) {
                        const int r = c + kk < nr ? c + kk : c + kk - nr;
                        float v = 0.f;
#pragma unroll
                        for (int q = 0; q < FNX_RING_MAX; ++q)   // selects, not indexing: the values stay in registers
                            if (q == r) v = pv[k][q];
                        acc = kk ? fadd(acc, v) : v;
                    }
                add[k] = acc;
            }
        }
        __syncthreads();   // the last block out counts the exchange
        if (tid == 0 && atomicAdd(&state[2], 1u) == gridDim.x - 1) {
            state[2] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(state) = epoch;
        }
    }
    // ---- x += sum; RMS norm: thread i the squares of columns i, i + 1024, ... in order, warp trees, the warps in order
    float v[BD_MAXC], s = 0.f;
#pragma unroll
    for (int k = 0; k < BD_MAXC; ++k) {
        const int i = vt + BD_THREADS * k;
        v[k] = 0.f;
        if (i < n) {
            float val = xr[i];
            if (has_add) {
                val = fadd(val, add[k]);
                xr[i] = val;
            }
            v[k] = val;
            s = ffma(val, val, s);
        }
    }
    s = wsum(s);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < BD_CL; ++r) cluster.map_shared_rank(sh, r)[cr * (BD_CT / 32) + warp] = s;
    }
    cluster.sync();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) tot = fadd(tot, sh[i]);
    const float r = ex_rsqrt(fadd(fdiv(tot, (float) n), a.eps));
#pragma unroll
    for (int k = 0; k < BD_MAXC; ++k) {
        const int i = vt + BD_THREADS * k;
        if (i - lane < n) {   // warp-uniform: a warp's 32 columns are one q8_1 block (n is a multiple of 32)
            const float val = fmul(fmul(v[k], r), a.w[i]);
            if (a.y) a.y[(size_t) t * n + i] = val;
            if (a.q) bd_q8_1_store(val, a.q + ((size_t) t * (n / 32) + (i >> 5)) * 36, lane);
        }
    }
}


// ---------------------------------------------------------------- the attention layer's merge across GPUs in one launch
// Every GPU has scanned the positions it owns for every head; a head's output is the merge of the GPUs' partials in
// ring order ending with the head's owner (reference src/kernels.cu:609-672, k_att_merge over the ring).  Here a GPU
// stores, into every peer's receive area, its partials of the heads that peer owns (value + exchange number words), and
// takes the partials of its own heads out of its own area as they arrive (bounded polls); the gate and the q8_1 rows for
// the output projection follow in the same kernel.  ring null: one GPU, the partial is the result.
// Block (owned head, row), hd threads; part: this GPU's partials [T][nq][hd + 2] (acc, m, z).
struct FinishArgs {
    const float* part;
    FnxRing ring;
    const float* qg;
    float* out;
    uint8_t* q8;
    int nq, hd, nrank;
    unsigned* err;
};

__global__ void k_attn_finish_ring(const FinishArgs a) {
    pdl_wait();
    pdl_go();
    const int n = a.nrank, me = n > 1 ? a.ring.rank : 0, hd = a.hd, nq = a.nq, own = gridDim.x, T = gridDim.y;
    const int hx = blockIdx.x, t = blockIdx.y, i = threadIdx.x, h = me * own + hx;
    const size_t at = ((size_t) t * nq + h) * (hd + 2);
    unsigned epoch = 0;
    int parity = 0;
    const size_t cnt = a.ring.ll_count;
    if (n > 1) {
        epoch = *reinterpret_cast<volatile unsigned*>(a.ring.state) + 1u;
        parity = (int) (epoch & 1u);
        // ---- every peer gets this GPU's partials of the heads it owns: run `me` of its receive area, [T][own][hd + 2];
        // block (hx, t) sends head hx of each peer's heads, row t
        for (int r = 0; r < n; ++r) {
            if (r == me) continue;
            const float* srcp = a.part + ((size_t) t * nq + r * own + hx) * (hd + 2);
            unsigned long long* dst = a.ring.ll[parity][r] + (size_t) me * cnt + ((size_t) t * own + hx) * (hd + 2);
            for (int e = i; e < hd + 2; e += blockDim.x) ll_store(dst + e, __float_as_uint(srcp[e]), epoch);
        }
    }
    // a peer's partial of (row t, owned head hx): element e, out of this GPU's receive area
    auto peer = [&](int r, int e) {
        return __uint_as_float(ll_load(a.ring.ll[parity][me] + (size_t) r * cnt + ((size_t) t * own + hx) * (hd + 2) + e, epoch, a.ring.spin_limit, a.err));
    };
    auto val = [&](int r, int e) { return r == me || n == 1 ? a.part[at + e] : peer(r, e); };
    const int r1 = (me + 1) % n;
    float m = val(r1, hd), z = val(r1, hd + 1), acc = val(r1, i);
    for (int s = 2; s <= n; ++s) {
        const int r2 = (me + s) % n;
        const float m2 = val(r2, hd), z2 = val(r2, hd + 1);
        const float mn = fmaxf(m, m2);
        const float w1 = m == -INFINITY ? 0.f : ex_expf(fsub(m, mn)), w2 = m2 == -INFINITY ? 0.f : ex_expf(fsub(m2, mn));
        z = ffma(w2, z2, fmul(w1, z));
        acc = ffma(w2, val(r2, i), fmul(w1, acc));
        m = mn;
    }
    const float v = fmul(fdiv(acc, z), ex_sigmoid(a.qg[((size_t) t * nq + h) * 2 * hd + hd + i]));
    if (a.out) a.out[((size_t) t * own + hx) * hd + i] = v;
    if (a.q8) bd_q8_1_store(v, a.q8 + (((size_t) t * own + hx) * (hd / 32) + (i >> 5)) * 36, i & 31);
    if (n > 1) {   // the last block out counts the exchange
        __syncthreads();
        if (i == 0 && atomicAdd(&a.ring.state[2], 1u) == gridDim.x * gridDim.y - 1) {
            a.ring.state[2] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(a.ring.state) = epoch;
        }
    }
}


// ---------------------------------------------------------------- a small all-gather over the ring's receive areas
// Every GPU's few words (the argmax (value, index) of its vocabulary range, its 64 candidates a row) to every GPU: the
// same exchange once more - the words stored into every peer's area, the peers' polled out of the own - as one block.
// Two arrays of 4-byte words a call; all_a [nrank][na], all_b [nrank][nb].
__global__ void __launch_bounds__(1024) k_ring_gather(const unsigned* __restrict__ a, int na, const unsigned* __restrict__ b, int nb, const FnxRing ring,
                                                      unsigned* __restrict__ all_a, unsigned* __restrict__ all_b, unsigned* err) {
    pdl_wait();
    pdl_go();
    const int n = ring.nrank, me = ring.rank, tid = threadIdx.x;
    unsigned* state = ring.state;
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(state) + 1u;
    const int parity = (int) (epoch & 1u);
    const size_t cnt = ring.ll_count;
    for (int i = tid; i < (n - 1) * (na + nb); i += blockDim.x) {   // this GPU's words to every peer's receive area
        const int q = i / (na + nb), k = i % (na + nb), r = q < me ? q : q + 1;
        ll_store(ring.ll[parity][r] + (size_t) me * cnt + k, k < na ? a[k] : b[k - na], epoch);
    }
    for (int i = tid; i < n * (na + nb); i += blockDim.x) {
        const int r = i / (na + nb), k = i % (na + nb);
        const unsigned v = r == me ? (k < na ? a[k] : b[k - na]) : ll_load(ring.ll[parity][me] + (size_t) r * cnt + k, epoch, ring.spin_limit, err);
        if (k < na) all_a[(size_t) r * na + k] = v;
        else all_b[(size_t) r * nb + (k - na)] = v;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(state) = epoch;
    }
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_ring_sum(float* x, int rows, int row_len, const FnxRing* ring, unsigned* err, void* st) {
    FNX_REQUIRE(ring && ring->nrank >= 1 && ring->nrank <= FNX_RING_MAX && ring->rank >= 0 && ring->rank < ring->nrank,
                "ring_sum: GPU %d of %d", ring ? ring->rank : -1, ring ? ring->nrank : 0);
    if (ring->nrank == 1) return 0;   // the identity
    FNX_REQUIRE(rows > 0 && row_len > 0 && row_len % 4 == 0, "ring_sum: %d rows of %d values (a multiple of 4)", rows, row_len);
    const int count = rows * row_len;
    FNX_REQUIRE(ring->state && ring->spin_limit > 0, "ring_sum: no state words or spin limit");
    for (int r = 0; r < ring->nrank; ++r)
        FNX_REQUIRE(ring->slot[0][r] && ring->slot[1][r] && ring->pad[r], "ring_sum: GPU %d's slots or flags are missing", r);
    // few enough blocks to be resident together on any part of the GPU: every block waits for the flags itself
    const int blocks = std::min(64, (count / 4 + RS_THREADS - 1) / RS_THREADS);
    k_ring_sum<<<blocks, RS_THREADS, 0, strm(st)>>>(x, count, row_len, *ring, err);
    return launch_ok("ring_sum");
}

int fnx_boundary_rows(float* x, const float* bo, const FnxMoeRows* moe, const FnxRing* ring, const float* w, float* y, void* q, int T, int n,
                      float eps, unsigned* err, void* st) {
    FNX_REQUIRE(x && w && T >= 1 && T <= FNX_MAXT, "boundary_rows: %d rows (1..%d)", T, FNX_MAXT);
    FNX_REQUIRE(n > 0 && n % 32 == 0 && n <= BD_MAXN, "boundary_rows: %d columns (a multiple of 32 up to %d)", n, BD_MAXN);
    FNX_REQUIRE(!(bo && moe), "boundary_rows: the ended half's rows or the experts' rows, not both");
    BoundaryArgs a{};
    a.x = x, a.bo = bo, a.w = w, a.y = y, a.q = (uint8_t*) q, a.n = n, a.eps = eps, a.err = err;
    if (moe) {
        FNX_REQUIRE(moe->part && moe->topw && moe->sh && moe->logits && moe->topk >= 1 && moe->nexp >= 1, "boundary_rows: the experts' rows are incomplete");
        a.moe = *moe;
    }
    a.ring.nrank = 1;
    if (ring && ring->nrank > 1 && (bo || moe)) {
        FNX_REQUIRE(ring->nrank <= FNX_RING_MAX && ring->rank >= 0 && ring->rank < ring->nrank, "boundary_rows: GPU %d of %d", ring->rank, ring->nrank);
        FNX_REQUIRE(ring->state && ring->spin_limit > 0 && err && n % 4 == 0, "boundary_rows: no state words, spin limit or error word");
        FNX_REQUIRE(ring->ll_count >= (size_t) T * n, "boundary_rows: receive areas of %zu words for %d x %d values", ring->ll_count, T, n);
        for (int r = 0; r < ring->nrank; ++r)
            FNX_REQUIRE(ring->ll[0][r] && ring->ll[1][r], "boundary_rows: GPU %d's receive areas are missing", r);
        a.ring = *ring;
    }
    launch(0, k_boundary_rows, T * BD_CL, BD_CT, 0, strm(st), a);
    return launch_ok("boundary_rows");
}

int fnx_attn_finish_ring(const float* part, const FnxRing* ring, const float* qg, float* out, void* q8, int T, int nq, int hd, unsigned* err,
                         void* st) {
    const int n = ring ? ring->nrank : 1;
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && hd % 32 == 0 && hd >= 32 && hd <= 1024, "attn_finish_ring: %d rows, head dim %d", T, hd);
    FNX_REQUIRE(n >= 1 && n <= FNX_RING_MAX && nq % n == 0, "attn_finish_ring: %d query heads over %d GPUs", nq, n);
    FNX_REQUIRE(!ring || (ring->rank >= 0 && ring->rank < n && ring->state && err && ring->spin_limit > 0), "attn_finish_ring: rank, state or error word missing");
    if (n > 1) {
        FNX_REQUIRE(ring->ll_count >= (size_t) T * (nq / n) * (hd + 2), "attn_finish_ring: receive areas of %zu words for %d x %d x %d", ring->ll_count, T,
                    nq / n, hd + 2);
        for (int r = 0; r < n; ++r) FNX_REQUIRE(ring->ll[0][r] && ring->ll[1][r], "attn_finish_ring: GPU %d's receive areas are missing", r);
    }
    FinishArgs a{part, ring ? *ring : FnxRing{}, qg, out, (uint8_t*) q8, nq, hd, n, err};
    launch(0, k_attn_finish_ring, dim3(nq / n, T), hd, 0, strm(st), a);
    return launch_ok("attn_finish_ring");
}

int fnx_ring_gather(const void* a, int na, const void* b, int nb, const FnxRing* ring, void* all_a, void* all_b, unsigned* err, void* st) {
    FNX_REQUIRE(ring && ring->nrank >= 2 && ring->nrank <= FNX_RING_MAX && ring->rank >= 0 && ring->rank < ring->nrank && ring->state && err,
                "ring_gather: no ring of at least two GPUs, state or error word");
    FNX_REQUIRE(a && all_a && na >= 1 && nb >= 0 && (nb == 0 || (b && all_b)), "ring_gather: %d + %d words without their arrays", na, nb);
    FNX_REQUIRE(ring->ll_count >= (size_t) (na + nb) && ring->spin_limit > 0, "ring_gather: receive areas of %zu words for %d", ring->ll_count, na + nb);
    for (int r = 0; r < ring->nrank; ++r) FNX_REQUIRE(ring->ll[0][r] && ring->ll[1][r], "ring_gather: GPU %d's receive areas are missing", r);
    launch(0, k_ring_gather, 1, 1024, 0, strm(st), (const unsigned*) a, na, (const unsigned*) b, nb, *ring, (unsigned*) all_a, (unsigned*) all_b, err);
    return launch_ok("ring_gather");
}
}
