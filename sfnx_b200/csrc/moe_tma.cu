// Expert gate|up for Q4_K weights, TMA-staged: a persistent kernel with one CTA per SM.  The window's work is the list
// of (job, 32-row panel) tiles; a CTA takes a contiguous run of them, so it stages the activations of one or two jobs
// only.  A panel (32 rows of one expert, contiguous in memory: 55 KB at 3072 columns) is brought into shared memory by
// one bulk copy through a 3-stage ring, so two panels are in flight per SM while a third is consumed; the consumer
// threads read the super-blocks from shared memory with 16-byte loads.  The arithmetic and the order of every sum are
// those of the direct-load kernel in moe.cu (reference src/moe_q4k.cuh:30-109).
#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "tma.cuh"

namespace fnxk {

constexpr int GT_THREADS = 256, GT_ROWS = 32, GT_STAGES = 3;

__device__ __forceinline__ unsigned gt_sbyte(const uint4& h, int k) {
    const unsigned word = k < 4 ? h.y : k < 8 ? h.z : h.w;
    return (word >> (8 * (k & 3))) & 0xFFu;
}
__device__ __forceinline__ void gt_scale_min(const uint4& h, int j, float& sc, float& m) {
    if (j < 4) {
        sc = (float) (gt_sbyte(h, j) & 63);
        m = (float) (gt_sbyte(h, j + 4) & 63);
    } else {
        sc = (float) ((gt_sbyte(h, j + 4) & 0xF) | ((gt_sbyte(h, j - 4) >> 6) << 4));
        m = (float) ((gt_sbyte(h, j + 4) >> 4) | ((gt_sbyte(h, j) >> 6) << 4));
    }
}

// shared memory: [stages][32 rows][row_b] panels, then the job's activations: int8 [16][n], f16 scales [16][n / 32],
// int16 block sums [16][n / 32], then the barriers
template <int GPL>
__global__ void __launch_bounds__(GT_THREADS, 1) k_moe_gu_q4k_tma(const uint8_t* __restrict__ A, size_t sa, int nrows, int n,
                                                                 const FnxJob* __restrict__ jobs, const int* __restrict__ njobs,
                                                                 const uint8_t* __restrict__ xq, float* __restrict__ out) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane8 = tid & 7, nb = n / 32;
    const unsigned row_b = (unsigned) (n / 256 * 144), panel_b = GT_ROWS * row_b;
    unsigned char* panels = smem;
    int8_t* aq = reinterpret_cast<int8_t*>(smem + (size_t) GT_STAGES * panel_b);
    __half* ad = reinterpret_cast<__half*>(aq + (size_t) FNX_MAXT * n);
    short* as = reinterpret_cast<short*>(ad + (size_t) FNX_MAXT * nb);
    uint64_t* full = reinterpret_cast<uint64_t*>(as + (size_t) FNX_MAXT * nb);
    __shared__ FnxJob jb;
    const int npanels = (nrows + GT_ROWS - 1) / GT_ROWS, total = *njobs * npanels;
    const int tpb = (total + gridDim.x - 1) / gridDim.x;
    const int t0 = blockIdx.x * tpb, t1 = min(total, t0 + tpb), nt = t1 - t0;
    if (nt <= 0) return;
    if (tid == 0) {
        for (int s = 0; s < GT_STAGES; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    auto issue = [&](int i) {   // tile t0 + i into stage i % stages (thread 0)
        const int tile = t0 + i, j = tile / npanels, p = tile % npanels;
        const int rows = min(GT_ROWS, nrows - p * GT_ROWS);
        const uint8_t* src = A + (size_t) jobs[j].w * sa + (size_t) p * GT_ROWS * row_b;
        uint64_t* bar = &full[i % GT_STAGES];
        mbar_expect_tx(bar, rows * row_b);
        bulk_g2s(panels + (size_t) (i % GT_STAGES) * panel_b, src, rows * row_b, bar);
    };
    if (tid == 0)
        for (int i = 0; i < GT_STAGES - 1 && i < nt; ++i) issue(i);
    int cur_job = -1;
#pragma unroll 1
    for (int i = 0; i < nt; ++i) {
        const int tile = t0 + i, j = tile / npanels, p = tile % npanels;
        if (tid == 0 && i + GT_STAGES - 1 < nt) issue(i + GT_STAGES - 1);   // its stage was consumed in iteration i - 1
        if (j != cur_job) {   // block-uniform
            cur_job = j;
            if (tid < (int) (sizeof(FnxJob) / 4)) reinterpret_cast<int*>(&jb)[tid] = reinterpret_cast<const int*>(jobs + j)[tid];
            __syncthreads();
            for (int it = tid; it < jb.n * nb; it += GT_THREADS) {
                const int r = it / nb, b = it % nb;
                const unsigned* src = reinterpret_cast<const unsigned*>(xq + ((size_t) jb.y[r] * nb + b) * 36);
                unsigned w[9];
#pragma unroll
                for (int k = 0; k < 9; ++k) w[k] = src[k];
                int sum = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) sum = __dp4a(0x01010101, (int) w[1 + k], sum);
                uint4* dst = reinterpret_cast<uint4*>(aq + (size_t) r * n + b * 32);
                dst[0] = make_uint4(w[1], w[2], w[3], w[4]);
                dst[1] = make_uint4(w[5], w[6], w[7], w[8]);
                ad[r * nb + b] = __ushort_as_half((unsigned short) (w[0] & 0xffff));
                as[r * nb + b] = (short) sum;
            }
            __syncthreads();
        }
        mbar_wait(&full[i % GT_STAGES], (unsigned) (i / GT_STAGES) & 1u);
        const int row = p * GT_ROWS + (tid >> 3);
        const bool live = row < nrows;
        const unsigned char* wrow = panels + (size_t) (i % GT_STAGES) * panel_b + (size_t) (live ? (tid >> 3) : 0) * row_b;
        uint4 hdr[GPL], q0[GPL], q1[GPL];
#pragma unroll
        for (int ii = 0; ii < GPL; ++ii) {
            const int g = lane8 + ii * 8, b = g >> 2, jg = g & 3;
            const unsigned char* blk = wrow + (size_t) b * 144;
            hdr[ii] = *reinterpret_cast<const uint4*>(blk);
            q0[ii] = *reinterpret_cast<const uint4*>(blk + 16 + 32 * jg);
            q1[ii] = *reinterpret_cast<const uint4*>(blk + 32 + 32 * jg);
        }
#pragma unroll 1
        for (int r = 0; r < jb.n; ++r) {
            float tmp = 0.f;
#pragma unroll
            for (int ii = 0; ii < GPL; ++ii) {
                const int g = lane8 + ii * 8, b = g >> 2, jg = g & 3, yb = b * 8 + jg * 2;
                const float d = h2f((uint16_t) (hdr[ii].x & 0xffff)), dmin = h2f((uint16_t) (hdr[ii].x >> 16));
                float sc0, m0, sc1, m1;
                gt_scale_min(hdr[ii], 2 * jg, sc0, m0);
                gt_scale_min(hdr[ii], 2 * jg + 1, sc1, m1);
                const uint4* ap = reinterpret_cast<const uint4*>(aq + (size_t) r * n + yb * 32);
                const uint4 a0 = ap[0], a1 = ap[1], a2 = ap[2], a3 = ap[3];
                const unsigned qw[8] = {q0[ii].x, q0[ii].y, q0[ii].z, q0[ii].w, q1[ii].x, q1[ii].y, q1[ii].z, q1[ii].w};
                const unsigned al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const unsigned ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
                int dl = 0, dh = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    dl = __dp4a((int) (qw[w] & 0x0F0F0F0Fu), (int) al[w], dl);
                    dh = __dp4a((int) ((qw[w] >> 4) & 0x0F0F0F0Fu), (int) ah[w], dh);
                }
                const float sl = (float) as[r * nb + yb], sh = (float) as[r * nb + yb + 1];
                const float d8l = __half2float(ad[r * nb + yb]), d8h = __half2float(ad[r * nb + yb + 1]);
                const float pos = fmul(d, fadd(fmul(d8l, fmul(sc0, (float) dl)), fmul(d8h, fmul(sc1, (float) dh))));
                const float neg = fmul(dmin, fadd(fmul(d8l, fmul(m0, sl)), fmul(d8h, fmul(m1, sh))));
                tmp = fadd(tmp, fsub(pos, neg));
            }
            tmp = sum8(tmp);
            if (live && lane8 == 0) out[(size_t) jb.out[r] * nrows + row] = tmp;
        }
        __syncthreads();   // the stage may be refilled, the job's activations replaced
    }
}

size_t gu_q4k_tma_smem(int n) { return (size_t) GT_STAGES * GT_ROWS * (n / 256 * 144) + (size_t) FNX_MAXT * (n + (n / 32) * 4) + 64; }

int gu_q4k_tma_launch(const uint8_t* A, size_t sa, int nrows, int n, const FnxJob* jobs, const int* njobs, const uint8_t* xq, float* gu,
                      cudaStream_t st) {
    const size_t sm = gu_q4k_tma_smem(n);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
#define GT_CASE(G)                                                                                                         \
    case G:                                                                                                                \
        if (cudaFuncSetAttribute(k_moe_gu_q4k_tma<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sm) != cudaSuccess) \
            return fail("moe gate|up q4_K: shared memory opt-in (%zu bytes) failed", sm);                                  \
        k_moe_gu_q4k_tma<G><<<sms, GT_THREADS, sm, st>>>(A, sa, nrows, n, jobs, njobs, xq, gu);                            \
        break;
    switch (n / 512) {
        GT_CASE(1) GT_CASE(2) GT_CASE(3) GT_CASE(4) GT_CASE(5) GT_CASE(6) GT_CASE(7) GT_CASE(8)
        default: return fail("moe gate|up q4_K: %d columns", n);
    }
#undef GT_CASE
    return launch_ok("moe gate|up q4_K (staged)");
}

unsigned* device_fault_word() {
    static unsigned* ptr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev] && cudaGetSymbolAddress((void**) &ptr[dev], g_fault) != cudaSuccess) ptr[dev] = nullptr;
    return ptr[dev];
}

}  // namespace fnxk

extern "C" unsigned fnx_device_fault(void) {
    unsigned v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, fnxk::g_fault, sizeof v) != cudaSuccess) return ~0u;
    if (v) cudaMemcpyToSymbol(fnxk::g_fault, &zero, sizeof zero);
    return v;
}
