// Position-split attention, the fast scan on Blackwell's fifth-generation tensor cores (head dimension 256).
//
// Same plan as attn_fast.cu (one CTA per KV head and range of owned positions, all T x (query heads per KV head) query
// rows at once, K/V chunks through cp.async, partial (acc, m, z) per split), with both products as tcgen05.mma and
// chunks of 64 positions.  S = Q K^T: the queries (split into high and low f16 halves, x = hi + lo) sit in shared memory
// as the A operand, rows x 256 dims in four K-blocks of 64 dims with the 128-byte swizzle, the chunk's K rows as the B
// operand in the same form, and the 128 x 64 fp32 scores accumulate in tensor memory (32 MMAs of M 128, N 64, K 16: hi
// then lo).  One thread issues them; tcgen05.commit signals an mbarrier.  Six warps then read the scores out of tensor
// memory with tcgen05.ld.16x256b, whose register layout is the accumulator fragment of mma.sync m16n8 (a warp reads the
// 16 rows it owns: warp w may touch lanes 32 (w % 4) .. + 31 of tensor memory, so the 16-row tiles go to warps 0, 4, 1,
// 5, 2, 6; warp 3 issues the MMAs and warp 7 makes the copies).  O += P V is described further down.
// The mma.sync scan measured 2.2 us of 4.1 us per 32 positions in S = Q K^T alone; here a chunk of 64 takes about 2.4 us
// in all, most of it the row warps' softmax step (six warps cannot hide their own latencies).
// Every wait on an mbarrier is bounded; on a timeout the fault word is set and the CTA finishes with what it has.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "umma.cuh"

namespace fnxk {

constexpr int AU_HD = 256, AU_ROWS = 128;   // AU_ROWS: rows of the queries' image in global memory (and M of the MMAs)
constexpr int AU_QBYTES = 4 * AU_ROWS * 128, AU_THREADS = 256;

__host__ __device__ inline int au_kv_owned(int p, int card, int ncard) {
    const int b = p / 4;
    const int blocks = (b + ncard - 1 - card) / ncard;
    return blocks * 4 + (b % ncard == card ? p % 4 + 1 : 0);
}
__device__ __forceinline__ size_t au_row_at(const FnxKvPages& g, int r, int nkv) {
    if (!g.pt) return (size_t) r * nkv * AU_HD;
    return (size_t) g.pt[r / g.rows] * g.page + (size_t) (r % g.rows) * nkv * AU_HD;
}
__device__ __forceinline__ void au_split(float x, __half& hi, __half& lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

// x = hi + lo with hi = f16(x), lo = f16(x - hi): two values packed as f16x2 (first value in the low half)
__device__ __forceinline__ void au_split2(float x, float y, unsigned& hi, unsigned& lo) {
    __half hx, lx, hy, ly;
    au_split(x, hx, lx);
    au_split(y, hy, ly);
    hi = (unsigned) __half_as_ushort(hx) | ((unsigned) __half_as_ushort(hy) << 16);
    lo = (unsigned) __half_as_ushort(lx) | ((unsigned) __half_as_ushort(ly) << 16);
}

// K and V of this GPU's own cache as 2-D tensors [local row][KV heads x 256] for the TMA unit (plain loads, no multicast)
struct AuMaps {
    CUtensorMap k, v;
};

struct AuArgs {
    const float* qg;
    const uint16_t *kc, *vc;
    FnxKvPages g;
    float* scratch;          // [nkv][nsplit][M][HD + 2]
    unsigned char* qsplit;   // [nkv][hi, lo][4 K-blocks][128 rows][128 B]: the A operand's shared-memory image
    int nq, nkv, T, card, ncard, nsplit;
    const int* pos0;
    unsigned* fault;
};

// The queries of every KV head as the tensor core wants them: high and low f16 halves, 128 rows (row m = hh T + t is row
// t of head kvl qpk + hh; rows >= M zero) x 256 dims in four K-blocks of 64 dims, 16-byte pieces swizzled by the row.
// Made once per launch so that the scan's CTAs (37 a KV head) copy the image instead of each splitting the rows again.
__global__ void __launch_bounds__(256) k_attn_qsplit(const AuArgs a) {
    pdl_wait();
    pdl_go();
    const int qpk = a.nq / a.nkv, M = a.T * qpk;
    const int idx = blockIdx.x * 256 + threadIdx.x;   // (kvl, m, pair of dims)
    if (idx >= a.nkv * AU_ROWS * (AU_HD / 2)) return;
    const int kvl = idx / (AU_ROWS * (AU_HD / 2)), m = idx / (AU_HD / 2) % AU_ROWS, d = idx % (AU_HD / 2) * 2;
    float2 x = make_float2(0.f, 0.f);
    if (m < M) x = *reinterpret_cast<const float2*>(a.qg + ((size_t) (m % a.T) * a.nq + kvl * qpk + m / a.T) * 2 * AU_HD + d);
    __half h0, l0, h1, l1;
    au_split(x.x, h0, l0);
    au_split(x.y, h1, l1);
    const size_t off = (size_t) (d >> 6) * (AU_ROWS * 128) + m * 128 + ((((d & 63) >> 3) ^ (m & 7)) << 4) + (d & 7) * 2;
    unsigned char* img = a.qsplit + (size_t) kvl * 2 * AU_QBYTES;
    *reinterpret_cast<unsigned*>(img + off) = (unsigned) __half_as_ushort(h0) | ((unsigned) __half_as_ushort(h1) << 16);
    *reinterpret_cast<unsigned*>(img + AU_QBYTES + off) = (unsigned) __half_as_ushort(l0) | ((unsigned) __half_as_ushort(l1) << 16);
}

// ---------------------------------------------------------------- both products on the tensor cores
// O += P V as tcgen05.mma too: the weights P of a chunk go to shared memory as the A operand (96 rows x 64 positions,
// high and low f16 halves, 128-byte swizzle), the chunk's V rows are the B operand as they lie in memory (dims
// contiguous: "MN-major", 128-byte swizzle, the same shared-memory form as K), and the 128 x 256 fp32 output accumulates
// in tensor memory over the whole range (8 MMAs of M 128, N 256, K 16 per chunk: hi and lo halves of P, four 16-position
// steps).  The row warps therefore hold no accumulators; they read each chunk's scores, take the softmax step and write
// P.  Rescaling the accumulator every chunk would mean a round trip through tensor memory, so the exponentials use a
// reference maximum that is only raised (and the accumulator only rescaled, tcgen05.ld / scale / tcgen05.st) when a row's
// maximum has grown by more than 8: the weights stay below e^8, well inside f16, and (acc, m_ref, z) is an exact
// partial for any reference.
//
// Why chunks of 64: the row warps are few (six warps for 96 rows: a warp may read only its quarter of tensor memory), so
// what a chunk costs them is largely latency that does not grow with the chunk (waits, barriers, the round trip of
// tcgen05.ld, shuffles), and an MMA of N 64 costs the issuing thread little more than one of N 32 (the A operand's 4 KB
// from shared memory bounds both): 80 -> 66 us per launch at 32,768 positions against chunks of 32.  Shared memory is
// what a chunk of 64 needs more of: the queries' image keeps only its 96 real rows per K-block (the MMAs of M 128 read
// the 32 rows past a block from whatever follows, into accumulator rows nobody reads), K and V share three buffers (see
// the kernel), and the P tile is 96 rows x 128 bytes per half.
constexpr unsigned AU2_COL_S = 256;   // tensor memory: O in columns 0..255, the two score tiles after it
constexpr int A3_CH = 64, A3_QROWS = 96, A3_QBLK = A3_QROWS * 128, A3_QBYTES = 4 * A3_QBLK, A3_KBLK = A3_CH * 128, A3_KBYTES = 4 * A3_KBLK;
constexpr int A3_NBUF = 3, A3_PBYTES = A3_QROWS * 128, A3_PAD = 4096;   // the pad: what an MMA reads past the last P row

// TMA: the cache is one contiguous run of rows whose count the caller gave (no page table), so K and V chunks come as
// tensor loads (four boxes of 64 rows x 64 dims, the 128-byte swizzle applied by the copy unit, completion on an
// mbarrier a buffer) and the queries' image as bulk copies; one lane asks, nobody moves bytes.  Otherwise (pages, or
// an unknown row count) a warp copies with cp.async as described above.
template <bool TMA>
__global__ void __launch_bounds__(AU_THREADS) k_attn_umma(const __grid_constant__ AuMaps maps, const AuArgs a) {
    constexpr int HD = AU_HD;
    const int split = blockIdx.x, kvl = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthreads = blockDim.x;
    const int qpk = a.nq / a.nkv, M = a.T * qpk;
    extern __shared__ __align__(1024) unsigned char au_smem[];
    unsigned char* Qhi = au_smem + ((1024u - (um_s32(au_smem) & 1023u)) & 1023u);
    unsigned char* Qlo = Qhi + A3_QBYTES;                       // each: 4 K-blocks x [96 rows x 128 B], swizzled
    unsigned char* KVst = Qlo + A3_QBYTES;                      // [3] 4 blocks of 64 dims x [64 rows x 128 B], swizzled: K(c), then V(c)
    unsigned char* Pst = KVst + A3_NBUF * A3_KBYTES;            // hi, lo: [96 rows x 128 B], 128-byte swizzle; then the pad
    __shared__ __align__(8) unsigned long long mbar_s[2], mbar_o, kvbar[A3_NBUF], qbar;
    __shared__ unsigned tmem_base;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&mbar_s[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&mbar_s[1])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&mbar_o)));
        for (int b = 0; b < A3_NBUF; ++b) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&kvbar[b])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&qbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();   // the rows appended by the kernel before are among the positions read
    pdl_go();
    const int pos0 = *a.pos0;
    const int ctx_max = au_kv_owned(pos0 + a.T - 1, a.card, a.ncard);
    const int nchunks = (ctx_max + A3_CH - 1) / A3_CH, cps = (nchunks + a.nsplit - 1) / a.nsplit;
    const int c_begin = split * cps, nc = max(0, min(nchunks, c_begin + cps) - c_begin);
    float* out = a.scratch + ((size_t) (kvl * a.nsplit + split) * M) * (HD + 2);
    const int tile = (warp & 3) * 2 + (warp >> 2);   // the 16 rows this warp owns: inside the quarter of tensor memory it may read
    const bool worker = (warp & 3) != 3;
    const int r0 = tile * 16 + (lane >> 2), r1 = r0 + 8, q4 = lane & 3;
    if (nc == 0) {
        for (int i = tid; i < M * (HD + 2); i += nthreads) out[i] = (i % (HD + 2)) == HD ? -INFINITY : 0.f;
        return;
    }
    // ---- the copies (K and V rows take the same shared-memory form) are the work of warp 7, which owns no rows: a lane
    // moves the 16-byte column piece `lane` of all 64 rows of a chunk, so the row warps spend nothing on them
    const bool copier = warp == 7;
    const int seg = lane;
    const size_t row_elems = (size_t) a.nkv * HD;
    // a buffer's mbarrier completes a phase per load: K(c) the even ones, V(c) the odd ones (waited for with parity 0, 1)
    auto tma_rows = [&](const CUtensorMap* map, int c, int b) {
        if (!copier || lane) return;
        um_expect_tx(&kvbar[b], A3_KBYTES);
#pragma unroll
        for (int blk = 0; blk < 4; ++blk)
            um_tma2d(um_s32(KVst) + b * A3_KBYTES + blk * A3_KBLK, map, kvl * HD + blk * 64, c * A3_CH, &kvbar[b]);
    };
    auto load_rows = [&](const uint16_t* cache, int c, unsigned dst_base) {
        if (!copier) return;
        const unsigned dcol = dst_base + (seg >> 3) * A3_KBLK;
        if (!a.g.pt && (c + 1) * A3_CH <= ctx_max) {   // a whole chunk of contiguous rows
            const uint16_t* src = cache + (size_t) c * A3_CH * row_elems + (size_t) kvl * HD + seg * 8;
#pragma unroll 8
            for (int row = 0; row < A3_CH; ++row)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dcol + row * 128 + (((seg & 7) ^ (row & 7)) << 4)), "l"(src + (size_t) row * row_elems));
            return;
        }
#pragma unroll 4
        for (int row = 0; row < A3_CH; ++row) {
            const int pos = c * A3_CH + row;
            const bool valid = pos < ctx_max;
            const uint16_t* src = cache + au_row_at(a.g, valid ? pos : 0, a.nkv) + (size_t) kvl * HD + seg * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dcol + row * 128 + (((seg & 7) ^ (row & 7)) << 4)), "l"(src),
                         "r"(valid ? 16 : 0));   // invalid rows: zeros
        }
    };
    // Three buffers in rotation, chunk c in buffer c % 3: first its K rows, for S(c); once those MMAs are done its V rows
    // over them, for O += P(c) V(c); once those are done the K rows of chunk c + 3.  V(c) so has more than a chunk's time to
    // arrive and K(c + 3) most of one, with the memory two stages of each would take less one.
    const unsigned kv_s = um_s32(KVst);
    auto load_k = [&](int c) {
        if (TMA) tma_rows(&maps.k, c_begin + c, c % A3_NBUF);
        else load_rows(a.kc, c_begin + c, kv_s + (c % A3_NBUF) * A3_KBYTES);
    };
    auto load_v = [&](int c) {
        if (TMA) tma_rows(&maps.v, c_begin + c, c % A3_NBUF);
        else load_rows(a.vc, c_begin + c, kv_s + (c % A3_NBUF) * A3_KBYTES);
    };
    load_k(0);
    if (nc > 1) load_k(1);
    if (nc > 2) load_k(2);
    if (TMA) {   // the queries' image, made by k_attn_qsplit: rows 0..95 of each of its K-blocks of 128 rows, a bulk copy each
        if (copier && lane == 0) {
            const unsigned char* img = a.qsplit + (size_t) kvl * 2 * AU_QBYTES;
            um_expect_tx(&qbar, 2 * A3_QBYTES);
            for (int blk = 0; blk < 8; ++blk)   // 0..3 hi, 4..7 lo
                um_bulk(um_s32(Qhi + (size_t) blk * A3_QBLK), img + (size_t) blk * (AU_ROWS * 128), A3_QBLK, &qbar);
        }
    } else {
        const unsigned char* img = a.qsplit + (size_t) kvl * 2 * AU_QBYTES;
        for (int i = tid; i < 2 * 4 * A3_QROWS * 8; i += nthreads) {
            const int piece = i & 7, row = (i >> 3) % A3_QROWS, blk = (i >> 3) / A3_QROWS;   // blk: 0..3 hi, 4..7 lo
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(um_s32(Qhi + (size_t) blk * A3_QBLK + row * 128 + piece * 16)),
                         "l"(img + (size_t) blk * (AU_ROWS * 128) + row * 128 + piece * 16));
        }
    }
    asm volatile("cp.async.commit_group;");
    if (warp == 0) {   // all 512 columns: O (256), two score tiles (128)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(um_s32(&tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    const int lim0 = worker && r0 < M ? au_kv_owned(pos0 + r0 % a.T, a.card, a.ncard) : 0;
    const int lim1 = worker && r1 < M ? au_kv_owned(pos0 + r1 % a.T, a.card, a.ncard) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, z0 = 0.f, z1 = 0.f;   // reference maxima and sums of this thread's two rows
    const float rs = 1.0f / sqrtf((float) HD);
    const unsigned idesc_s = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);               // S: N 64, both operands K-major
    const unsigned idesc_o = (1u << 4) | (1u << 16) | ((256u >> 3) << 17) | ((128u >> 4) << 24);   // O: N 256, B MN-major
    auto issue_scores = [&](int c) {
        const unsigned tb = tmem_base + AU2_COL_S + (c & 1) * A3_CH;
        const unsigned long long dk = um_desc(um_s32(KVst + (size_t) (c % A3_NBUF) * A3_KBYTES));
        const unsigned long long dh = um_desc(um_s32(Qhi)), dl = um_desc(um_s32(Qlo));
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const unsigned long long ob = (unsigned long long) ((kb * A3_KBLK + ks * 32) >> 4), oa = (unsigned long long) ((kb * A3_QBLK + ks * 32) >> 4);
                um_mma(tb, dh + oa, dk + ob, idesc_s, kb | ks);
                um_mma(tb, dl + oa, dk + ob, idesc_s, 1u);
            }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(um_s32(&mbar_s[c & 1])) : "memory");
    };
    auto issue_output = [&](int c) {   // O (+)= (Phi + Plo) V(c)
        const unsigned long long dv = um_desc_x(um_s32(KVst + (size_t) (c % A3_NBUF) * A3_KBYTES), A3_KBLK, 1024, 2);
        const unsigned long long dph = um_desc(um_s32(Pst)), dpl = um_desc(um_s32(Pst + A3_PBYTES));
#pragma unroll
        for (int ks = 0; ks < A3_CH / 16; ++ks) {
            um_mma(tmem_base, dph + (unsigned long long) (ks * 32 >> 4), dv + (unsigned long long) (ks * 16 * 128 >> 4), idesc_o, c | ks);
            um_mma(tmem_base, dpl + (unsigned long long) (ks * 32 >> 4), dv + (unsigned long long) (ks * 16 * 128 >> 4), idesc_o, 1u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(um_s32(&mbar_o)) : "memory");
    };
    auto sync_all = [&] {   // stores and landed copies of every thread visible to the tensor core, tensor-memory accesses ordered
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    };
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    sync_all();
    const bool issuer = tid == 3 * 32;   // warp 3, lane 0
    if (issuer) {
        if (TMA) um_wait(&qbar, 0u, a.fault), um_wait(&kvbar[0], 0u, a.fault);   // the queries and K(0) have landed
        issue_scores(0);
    }
    bool alive = true;   // false after a wait ran out
    auto copier_wait = [&](unsigned long long* bar, unsigned parity) {   // the copying warp alone waits for a set of MMAs
        bool ok = alive && um_wait(bar, parity, a.fault);
        ok = __all_sync(0xffffffffu, ok);
        alive = alive && ok;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    };
    if (copier) {
        copier_wait(&mbar_s[0], 0u);   // S(0) is complete: V(0) over K(0)
        load_v(0);
    }
    asm volatile("cp.async.commit_group;");
#pragma unroll 1
    for (int i = 0; i < nc; ++i) {
        const int buf = i & 1;
        if (issuer && i + 1 < nc) {   // the next chunk's scores while this chunk's are used
            if (TMA) um_wait(&kvbar[(i + 1) % A3_NBUF], 0u, a.fault);   // K(i + 1) has landed
            issue_scores(i + 1);
        }
        float sacc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = -INFINITY;
        if (worker) {
            bool ok = alive && um_wait(&mbar_s[buf], (i >> 1) & 1, a.fault);
            ok = __all_sync(0xffffffffu, ok);
            alive = alive && ok;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    unsigned r[16];
                    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(tmem_base + AU2_COL_S + buf * A3_CH + hf * 32 + ((unsigned) (tile * 16) << 16)));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sacc[4 * hf + j][e] = __uint_as_float(r[4 * j + e]);
                }
            }
        }
        // ---- the chunk's maxima; a row's reference is raised when its maximum has grown by more than 8
        const int pc = (c_begin + i) * A3_CH + 2 * q4;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int pcol = pc + 8 * j + e;
                sacc[j][e] = pcol < lim0 ? sacc[j][e] * rs : -INFINITY;
                sacc[j][2 + e] = pcol < lim1 ? sacc[j][2 + e] * rs : -INFINITY;
                mx0 = fmaxf(mx0, sacc[j][e]);
                mx1 = fmaxf(mx1, sacc[j][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const bool up0 = mx0 > m0 + 8.0f || (m0 == -INFINITY && mx0 != -INFINITY), up1 = mx1 > m1 + 8.0f || (m1 == -INFINITY && mx1 != -INFINITY);
        const float f0 = !up0 ? 1.0f : m0 == -INFINITY ? 0.f : __expf(m0 - mx0), f1 = !up1 ? 1.0f : m1 == -INFINITY ? 0.f : __expf(m1 - mx1);
        if (up0) m0 = mx0;
        if (up1) m1 = mx1;
        // ---- the accumulator and the P tile are free once the MMAs of the chunk before are done
        if (i > 0) {
            bool ok = alive && um_wait(&mbar_o, (i - 1) & 1, a.fault);
            ok = __all_sync(0xffffffffu, ok);
            alive = alive && ok;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        if (i > 0 && i + 2 < nc) load_k(i + 2);   // over V(i - 1), whose MMAs are done
        asm volatile("cp.async.commit_group;");
        if (copier && i + 1 < nc) {
            copier_wait(&mbar_s[buf ^ 1], (unsigned) (((i + 1) >> 1) & 1));   // S(i + 1) is complete: V(i + 1) over K(i + 1)
            load_v(i + 1);
        }
        asm volatile("cp.async.commit_group;");
        if (worker) {
            // rows of this warp whose reference went up (and had something accumulated): O row *= f, 32 columns at a time
            if (i > 0 && __any_sync(0xffffffffu, f0 != 1.0f || f1 != 1.0f)) {
#pragma unroll 1
                for (int cb = 0; cb < HD / 32; ++cb) {
                    unsigned r[16];
                    const unsigned ta = tmem_base + cb * 32 + ((unsigned) (tile * 16) << 16);
                    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(ta));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) * f0), r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) * f0);
                        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) * f1), r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) * f1);
                    }
                    asm volatile("tcgen05.st.sync.aligned.16x256b.x4.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(r[0]), "r"(r[1]),
                                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
                                 "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(ta)
                                 : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // ---- the weights against the references, their sums, and the P tile (hi and lo halves, 64-byte swizzle)
            float ps0 = 0.f, ps1 = 0.f;
            unsigned char* prow0 = Pst + r0 * 128 + 4 * q4;
            unsigned char* prow1 = Pst + r1 * 128 + 4 * q4;
            const int sw0 = r0 & 7, sw1 = r1 & 7;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    p[e] = sacc[j][e] == -INFINITY ? 0.f : __expf(sacc[j][e] - m0);
                    p[2 + e] = sacc[j][2 + e] == -INFINITY ? 0.f : __expf(sacc[j][2 + e] - m1);
                }
                ps0 += p[0] + p[1];
                ps1 += p[2] + p[3];
                unsigned h0, l0, h1, l1;
                au_split2(p[0], p[1], h0, l0);
                au_split2(p[2], p[3], h1, l1);
                *reinterpret_cast<unsigned*>(prow0 + ((j ^ sw0) << 4)) = h0;
                *reinterpret_cast<unsigned*>(prow0 + A3_PBYTES + ((j ^ sw0) << 4)) = l0;
                *reinterpret_cast<unsigned*>(prow1 + ((j ^ sw1) << 4)) = h1;
                *reinterpret_cast<unsigned*>(prow1 + A3_PBYTES + ((j ^ sw1) << 4)) = l1;
            }
            ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
            ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
            ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
            ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
            z0 = z0 * f0 + ps0;
            z1 = z1 * f1 + ps1;
        }
        // ---- P is written; V(i), asked for a chunk ago, and K(i + 2) have landed: the output MMAs of this chunk
        asm volatile("cp.async.wait_group 1;" ::: "memory");   // all but V(i + 1), just asked for
        if (TMA && copier) {
            // V(i) has landed.  Rows of the range's last chunk past the newest position hold whatever the cache holds
            // there: their weights are zero, but zero times a stray NaN is not, so they are cleared
            copier_wait(&kvbar[i % A3_NBUF], 1u);
            const int have = ctx_max - (c_begin + i) * A3_CH;
            for (int row = max(have, 0); row < A3_CH; ++row)
                *reinterpret_cast<uint4*>(KVst + (size_t) (i % A3_NBUF) * A3_KBYTES + (lane >> 3) * A3_KBLK + row * 128 + (lane & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        sync_all();
        if (issuer) issue_output(i);
    }
    // ---- this split's partial: the accumulator out of tensor memory, m_ref, z per row
    {
        bool ok = alive && um_wait(&mbar_o, (nc - 1) & 1, a.fault);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (worker) {
#pragma unroll 1
            for (int cb = 0; cb < HD / 32; ++cb) {
                unsigned r[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) r[e] = 0u;
                if (ok) {
                    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                                 : "r"(tmem_base + cb * 32 + ((unsigned) (tile * 16) << 16)));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int col = cb * 32 + j * 8 + 2 * q4;
                    if (r0 < M) *reinterpret_cast<float2*>(out + (size_t) r0 * (HD + 2) + col) = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
                    if (r1 < M) *reinterpret_cast<float2*>(out + (size_t) r1 * (HD + 2) + col) = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
            }
            if (q4 == 0) {
                if (r0 < M) out[(size_t) r0 * (HD + 2) + HD] = m0, out[(size_t) r0 * (HD + 2) + HD + 1] = z0;
                if (r1 < M) out[(size_t) r1 * (HD + 2) + HD] = m1, out[(size_t) r1 * (HD + 2) + HD + 1] = z1;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
}

size_t attn_umma_smem() { return (size_t) 2 * A3_QBYTES + A3_NBUF * A3_KBYTES + 2 * A3_PBYTES + A3_PAD + 1024; }


// the scan part of fnx_attn_partial for head dimension 256 and at most 96 query rows a KV head; -1 when it does not apply
int attn_umma_launch(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* scratch, int card, int ncard, int T,
                     const int* pos0, int nq, int nkv, int nsplit, cudaStream_t st) {
    const int M = T * (nq / nkv);
    unsigned* fault = device_fault_word();
    if (M > 96 || nkv > 8 || !fault) return -1;
    // the queries' image sits in the scratch after the splits' partials (fnx_attn_scratch_floats leaves room for it)
    unsigned char* qsplit = reinterpret_cast<unsigned char*>(scratch + (size_t) nkv * nsplit * M * (AU_HD + 2));
    if ((uintptr_t) qsplit % 16) return -1;
    AuArgs a{qg, kc, vc, g, scratch, qsplit, nq, nkv, T, card, ncard, nsplit, pos0, fault};
    launch(0, k_attn_qsplit, (nkv * AU_ROWS * (AU_HD / 2) + 255) / 256, 256, 0, st, a);
    if (launch_ok("attn query split")) return 1;
    const size_t sm3 = attn_umma_smem();
    AuMaps maps;
    memset(&maps, 0, sizeof(maps));
    // tensor loads when the cache is a contiguous run of a known number of rows; its rows past the newest position are
    // inside the maps (read and cleared in shared memory), rows past the cache read as zeros
    UmEncode enc = um_encoder();
    bool tma = enc && !g.pt && g.cap >= 1 && (uintptr_t) kc % 16 == 0 && (uintptr_t) vc % 16 == 0 && !getenv("FNX_ATTN_NO_TMA");
    if (tma) {
        const cuuint64_t gd[2] = {(cuuint64_t) nkv * AU_HD, (cuuint64_t) g.cap}, gs[1] = {(cuuint64_t) nkv * AU_HD * 2};
        const cuuint32_t bx[2] = {64, A3_CH}, es[2] = {1, 1};
        tma = enc(&maps.k, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*) kc, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
              enc(&maps.v, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*) vc, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (tma) {
        if (cudaFuncSetAttribute(k_attn_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm3) != cudaSuccess) return -1;
        launch(6, k_attn_umma<true>, dim3(nsplit, nkv), AU_THREADS, sm3, st, maps, a);
    } else {
        if (cudaFuncSetAttribute(k_attn_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm3) != cudaSuccess) return -1;
        launch(6, k_attn_umma<false>, dim3(nsplit, nkv), AU_THREADS, sm3, st, maps, a);
    }
    return launch_ok("attn scan (tcgen05)");
}

// floats the tcgen05 scan needs in the scratch beyond the splits' partials
size_t attn_umma_scratch_floats(int nkv) { return (size_t) nkv * 2 * AU_QBYTES / 4; }

}  // namespace fnxk
