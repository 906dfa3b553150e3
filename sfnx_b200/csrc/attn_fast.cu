// Position-split attention, the fast scan: one pass over this GPU's K/V rows for all rows of the window at once.
// A CTA takes one KV head and a contiguous range of the owned positions; its M = T x (query heads per KV head) query
// rows (96 at T = 16) are 16-row tiles, one warp each, so the window is a dense contraction on the tensor cores:
// S = Q K^T and O += P V with mma.sync m16n8k16 (f16 inputs, f32 accumulate).  To keep f32 accuracy with f16 operands
// the f32 queries and the softmax weights are split into a high and a low f16 part (x = hi + lo, two MMAs): K and V
// are f16 already.  K/V chunks of 32 positions are staged through shared memory with cp.async (3 stages); each K/V
// byte is read from HBM once per window instead of once per row.  The partial (acc, m, z) of every split goes to
// scratch and a second kernel merges the splits into the per-GPU partial the cross-GPU merge takes.
// The sums are not in the reference's order (src/kernels.cu:497-606): results agree with the exact-order scan to f32
// rounding, not bit for bit.
#include <cstdlib>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"

namespace fnxk {

constexpr int AF_CH = 32, AF_STAGES = 3, AF_PAD = 8;   // positions a chunk; row pad in halves (16 B): conflict-free ldmatrix

__host__ __device__ inline int af_kv_owned(int p, int card, int ncard) {
    const int b = p / 4;
    const int blocks = (b + ncard - 1 - card) / ncard;
    return blocks * 4 + (b % ncard == card ? p % 4 + 1 : 0);
}
__device__ __forceinline__ size_t af_row_at(const FnxKvPages& g, int r, int nkv, int hd) {
    if (!g.pt) return (size_t) r * nkv * hd;
    return (size_t) g.pt[r / g.rows] * g.page + (size_t) (r % g.rows) * nkv * hd;
}
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(unsigned& a, unsigned& b, unsigned& c, unsigned& d, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm4t(unsigned& a, unsigned& b, unsigned& c, unsigned& d, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// x = hi + lo with hi = f16(x), lo = f16(x - hi): two values packed as f16x2 (first value in the low half)
__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
    const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
    const __half lx = __float2half_rn(x - __half2float(hx)), ly = __float2half_rn(y - __half2float(hy));
    hi = (unsigned) __half_as_ushort(hx) | ((unsigned) __half_as_ushort(hy) << 16);
    lo = (unsigned) __half_as_ushort(lx) | ((unsigned) __half_as_ushort(ly) << 16);
}

struct AfArgs {
    const float* qg;
    const uint16_t *kc, *vc;
    FnxKvPages g;
    float* scratch;   // [nkv][nsplit][M][HD + 2]
    int nq, nkv, T, card, ncard, nsplit;
    const int* pos0;
};

template <int HD, int STAGES>
__global__ void __launch_bounds__(256) k_attn_fast(const AfArgs a) {
    constexpr int LD = HD + AF_PAD, KS = HD / 16, NT = HD / 8;
    const int split = blockIdx.x, kvl = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthreads = blockDim.x;
    const int qpk = a.nq / a.nkv, M = a.T * qpk, Mpad = (M + 15) / 16 * 16;
    extern __shared__ __align__(16) unsigned char af_smem[];
    __half* Qhi = reinterpret_cast<__half*>(af_smem);
    __half* Qlo = Qhi + (size_t) Mpad * LD;
    __half* KV = Qlo + (size_t) Mpad * LD;   // [STAGES][K, V][32][LD]
    pdl_wait();   // the rows appended by the kernel before are among the positions read
    pdl_go();
    const int pos0 = *a.pos0;
    const int ctx_max = af_kv_owned(pos0 + a.T - 1, a.card, a.ncard);
    const int nchunks = (ctx_max + AF_CH - 1) / AF_CH, cps = (nchunks + a.nsplit - 1) / a.nsplit;
    const int c_begin = split * cps, nc = max(0, min(nchunks, c_begin + cps) - c_begin);
    auto load_chunk = [&](int c, int stage) {
        __half* Ks = KV + (size_t) stage * 2 * AF_CH * LD;
        __half* Vs = Ks + (size_t) AF_CH * LD;
        constexpr int SEG = HD / 8;
        for (int idx = tid; idx < 2 * AF_CH * SEG; idx += nthreads) {
            const int which = idx / (AF_CH * SEG), rem = idx % (AF_CH * SEG), row = rem / SEG, seg = rem % SEG;
            const int pos = c * AF_CH + row;
            const bool valid = pos < ctx_max;
            const uint16_t* src = (which ? a.vc : a.kc) + af_row_at(a.g, valid ? pos : 0, a.nkv, HD) + (size_t) kvl * HD + seg * 8;
            cp_async16((which ? Vs : Ks) + (size_t) row * LD + seg * 8, src, valid ? 16 : 0);   // invalid rows: zero fill
        }
    };
    // this thread's two rows of its warp's tile and the positions they may see
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int lim0 = r0 < M ? af_kv_owned(pos0 + r0 % a.T, a.card, a.ncard) : 0;
    const int lim1 = r1 < M ? af_kv_owned(pos0 + r1 % a.T, a.card, a.ncard) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, z0 = 0.f, z1 = 0.f;
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    const float rs = 1.0f / sqrtf((float) HD);
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nc) load_chunk(c_begin + s, s);
        cp_async_commit();
    }
    // (the first K/V chunks are on their way while the queries are staged)
    // the query rows, split into high and low halves: row m = hh T + t is row t of head kvl qpk + hh
    for (int idx0 = tid; idx0 < Mpad * (HD / 2); idx0 += 8 * nthreads) {   // eight loads in flight a thread
        float2 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = idx0 + u * nthreads, m = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
            x[u] = make_float2(0.f, 0.f);
            if (idx < Mpad * (HD / 2) && m < M)
                x[u] = *reinterpret_cast<const float2*>(a.qg + ((size_t) (m % a.T) * a.nq + kvl * qpk + m / a.T) * 2 * HD + d);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int idx = idx0 + u * nthreads, m = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
            if (idx >= Mpad * (HD / 2)) break;
            unsigned hi, lo;
            split2(x[u].x, x[u].y, hi, lo);
            *reinterpret_cast<unsigned*>(Qhi + (size_t) m * LD + d) = hi;
            *reinterpret_cast<unsigned*>(Qlo + (size_t) m * LD + d) = lo;
        }
    }
#pragma unroll 1
    for (int i = 0; i < nc; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (i + STAGES - 1 < nc) load_chunk(c_begin + i + STAGES - 1, (i + STAGES - 1) % STAGES);
        cp_async_commit();
        const __half* Ks = KV + (size_t) (i % STAGES) * 2 * AF_CH * LD;
        const __half* Vs = Ks + (size_t) AF_CH * LD;
        // ---- S = Q K^T for the warp's 16 rows x 32 positions
        float sacc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll 4
        for (int ks = 0; ks < KS; ++ks) {
            unsigned ah[4], al[4];
            const size_t qoff = (size_t) (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4);
            ldsm4(ah[0], ah[1], ah[2], ah[3], Qhi + qoff);
            ldsm4(al[0], al[1], al[2], al[3], Qlo + qoff);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                unsigned b[4];
                ldsm4(b[0], b[1], b[2], b[3], Ks + (size_t) (16 * jj + 8 * (lane >> 4) + (lane & 7)) * LD + ks * 16 + 8 * ((lane >> 3) & 1));
                mma16816(sacc[2 * jj], ah[0], ah[1], ah[2], ah[3], b[0], b[1]);
                mma16816(sacc[2 * jj], al[0], al[1], al[2], al[3], b[0], b[1]);
                mma16816(sacc[2 * jj + 1], ah[0], ah[1], ah[2], ah[3], b[2], b[3]);
                mma16816(sacc[2 * jj + 1], al[0], al[1], al[2], al[3], b[2], b[3]);
            }
        }
        // ---- online softmax step per row (a row's 32 scores sit in the 4 lanes of a quad)
        const int pc = (c_begin + i) * AF_CH + 2 * (lane & 3);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
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
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float sc0 = m0 == -INFINITY ? 0.f : __expf(m0 - mn0), sc1 = m1 == -INFINITY ? 0.f : __expf(m1 - mn1);
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                sacc[j][e] = sacc[j][e] == -INFINITY ? 0.f : __expf(sacc[j][e] - mn0);
                sacc[j][2 + e] = sacc[j][2 + e] == -INFINITY ? 0.f : __expf(sacc[j][2 + e] - mn1);
                ps0 += sacc[j][e];
                ps1 += sacc[j][2 + e];
            }
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
        z0 = z0 * sc0 + ps0;
        z1 = z1 * sc1 + ps1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            o[nt][0] *= sc0;
            o[nt][1] *= sc0;
            o[nt][2] *= sc1;
            o[nt][3] *= sc1;
        }
        // ---- O += P V, the weights as high + low f16 halves
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            unsigned ph[4], pl[4];
            split2(sacc[2 * kk][0], sacc[2 * kk][1], ph[0], pl[0]);
            split2(sacc[2 * kk][2], sacc[2 * kk][3], ph[1], pl[1]);
            split2(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], ph[2], pl[2]);
            split2(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], ph[3], pl[3]);
            const __half* vrow = Vs + (size_t) (16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + 8 * (lane >> 4);
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                unsigned b[4];
                ldsm4t(b[0], b[1], b[2], b[3], vrow + n2 * 16);
                mma16816(o[2 * n2], ph[0], ph[1], ph[2], ph[3], b[0], b[1]);
                mma16816(o[2 * n2], pl[0], pl[1], pl[2], pl[3], b[0], b[1]);
                mma16816(o[2 * n2 + 1], ph[0], ph[1], ph[2], ph[3], b[2], b[3]);
                mma16816(o[2 * n2 + 1], pl[0], pl[1], pl[2], pl[3], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    // ---- this split's partial: acc[HD], m, z per row
    float* out = a.scratch + ((size_t) (kvl * a.nsplit + split) * M) * (HD + 2);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + 2 * (lane & 3);
        if (r0 < M) *reinterpret_cast<float2*>(out + (size_t) r0 * (HD + 2) + col) = make_float2(o[nt][0], o[nt][1]);
        if (r1 < M) *reinterpret_cast<float2*>(out + (size_t) r1 * (HD + 2) + col) = make_float2(o[nt][2], o[nt][3]);
    }
    if ((lane & 3) == 0) {
        if (r0 < M) out[(size_t) r0 * (HD + 2) + HD] = m0, out[(size_t) r0 * (HD + 2) + HD + 1] = z0;
        if (r1 < M) out[(size_t) r1 * (HD + 2) + HD] = m1, out[(size_t) r1 * (HD + 2) + HD + 1] = z1;
    }
}

// the splits of (row t, head h) merged into this GPU's partial: part[(t nq + h) (hd + 2)] = acc[hd], m, z
__global__ void k_attn_fast_merge(const float* __restrict__ scratch, float* __restrict__ part, int nq, int nkv, int T, int nsplit, int hd) {
    pdl_wait();
    pdl_go();
    const int h = blockIdx.x, t = blockIdx.y, i = threadIdx.x, qpk = nq / nkv, kvl = h / qpk, m = (h % qpk) * T + t, M = T * qpk;
    const float* base = scratch + ((size_t) kvl * nsplit * M + m) * (hd + 2);
    const size_t step = (size_t) M * (hd + 2);
    __shared__ float sm_m[160], sm_w[160], sm_z[160];   // nsplit <= 148
    for (int s = i; s < nsplit; s += blockDim.x) sm_m[s] = base[s * step + hd], sm_z[s] = base[s * step + hd + 1];
    __syncthreads();
    float mx = -INFINITY;
    for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, sm_m[s]);
    for (int s = i; s < nsplit; s += blockDim.x) sm_w[s] = sm_m[s] == -INFINITY ? 0.f : ex_expf(fsub(sm_m[s], mx));
    __syncthreads();
    float z = 0.f, acc = 0.f;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {   // eight splits' loads in flight
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = s0 + k < nsplit ? base[(s0 + k) * step + i] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (s0 + k < nsplit && sm_m[s0 + k] != -INFINITY) {
                z = ffma(sm_w[s0 + k], sm_z[s0 + k], z);
                acc = ffma(sm_w[s0 + k], v[k], acc);
            }
    }
    float* o = part + ((size_t) t * nq + h) * (hd + 2);
    o[i] = acc;
    if (i == 0) o[hd] = mx, o[hd + 1] = z;
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

// the fast scan's split count: one CTA per SM over the KV heads (148 SMs)
int fnx_attn_splits(int nkv) { return nkv >= 148 ? 1 : 148 / nkv; }

int fnx_attn_partial(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard, int T,
                     const int* pos0, int nq, int nkv, int hd, float* scratch, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "attn: T %d outside 1..%d", T, FNX_MAXT);
    FNX_REQUIRE(hd == 256 || hd == 128, "attn: head dim %d (128 or 256)", hd);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && T * (nq / nkv) <= 128, "attn: %d query heads over %d KV heads, %d rows", nq, nkv, T);
    FNX_REQUIRE(ncard >= 1 && card >= 0 && card < ncard, "attn: GPU %d of %d", card, ncard);
    // int8 rows are read by the exact-order scan only (it turns them into f32 as it stages them)
    if (g.q8) return fnx_attn_partial_exact(qg, kc, vc, g, part, card, ncard, T, pos0, nq, nkv, hd, scratch, st);
    const int M = T * (nq / nkv), Mpad = (M + 15) / 16 * 16, nsplit = fnx_attn_splits(nkv);
    // head dimension 256: S = Q K^T on tcgen05 with the scores in tensor memory (attn_umma.cu); FNX_ATTN_MMA=1 keeps the
    // mma.sync scan below, which also serves the other shapes
    static const bool legacy = getenv("FNX_ATTN_MMA") != nullptr;
    if (hd == 256 && !legacy) {
        const int rc = attn_umma_launch(qg, kc, vc, g, scratch, card, ncard, T, pos0, nq, nkv, nsplit, strm(st));
        if (rc > 0) return 1;
        if (rc == 0) {
            launch(0, k_attn_fast_merge, dim3(nq, T), hd, 0, strm(st), scratch, part, nq, nkv, T, nsplit, hd);
            return launch_ok("attn merge");
        }
    }
    AfArgs a{qg, kc, vc, g, scratch, nq, nkv, T, card, ncard, nsplit, pos0};
    const int LD = hd + AF_PAD;
    const int stages = ((size_t) (2 * Mpad + 3 * 2 * AF_CH) * LD * 2 <= 227 * 1024) ? 3 : 2;
    const size_t sm = (size_t) (2 * Mpad + stages * 2 * AF_CH) * LD * 2;
    const dim3 grid(nsplit, nkv);
#define AF_LAUNCH(HD, ST)                                                                                         \
    {                                                                                                             \
        if (cudaFuncSetAttribute(k_attn_fast<HD, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm) != cudaSuccess) \
            return fail("attn: shared memory opt-in (%zu bytes) failed", sm);                                     \
        launch(6, k_attn_fast<HD, ST>, grid, 2 * Mpad, sm, strm(st), a);                                            \
    }
    if (hd == 256 && stages == 3) AF_LAUNCH(256, 3)
    else if (hd == 256) AF_LAUNCH(256, 2)
    else if (stages == 3) AF_LAUNCH(128, 3)
    else AF_LAUNCH(128, 2)
#undef AF_LAUNCH
    if (launch_ok("attn scan")) return 1;
    launch(0, k_attn_fast_merge, dim3(nq, T), hd, 0, strm(st), scratch, part, nq, nkv, T, nsplit, hd);
    return launch_ok("attn merge");
}
}
