// Dense split-Q8_0 projections of the verify window (the output head, qkvz, wq|wk|wv) on Blackwell's fifth-generation
// tensor cores: the same product as dense.cu's kernels - out[t][r] = sum over 32-column blocks of fl(dw da) (float) isum -
// with the sums in block order (oracle: orc_q8s_gemv_blocks), not the reference's lane-and-tree order, so results agree with
// the reference's to fp32 rounding of the sum (dense.cu keeps the reference's order, bit for bit).
//
// A block's integer dot of 128 weight rows against the window's 16 rows is ONE tcgen05.mma (kind::i8, M 128, N 16, K 32)
// into 16 columns of tensor memory; nothing is accumulated on the tensor cores, because every block has scales of its own.
// A persistent CTA (one per SM) walks 128-row tiles:
//   warp 16   the TMA unit's driver: for every 128 bytes of K (four blocks) one cp.async.bulk.tensor load of the 128 x 128
//             byte weight tile into a 128-byte-swizzled stage (six stages), and per tile one load of its f16 block scales;
//             it starts before the kernel ahead in the stream has finished (weights depend on nothing in the window)
//   warp 17   issues the four MMAs of a stage, each into its own 16 columns of one of eight 64-column groups of tensor
//             memory; tcgen05.commit hands the stage back to the TMA warp and the group to the epilogue
//   warps 0-15  the epilogue: warp w reads rows 32 (w % 4) .. + 31 (its quarter of tensor memory) and window rows
//             4 (w / 4) .. + 3: tcgen05.ld, the integer dots to float by the 1.5 * 2^23 offset (no convert instruction),
//             scale by fl(dw da) and add - sixteen warps so that the CUDA-core work of a 4 KB block step (128 rows x 16
//             values) stays well under the time HBM needs to deliver the step.
// The window's activations (int8 plane as the MMAs' B operand, 16 rows x K, and their float scales) are staged once per
// CTA.  Every wait is bounded; a wait that runs out sets bit 8 of the fault word and the CTA finishes without waiting again.
#include <cuda.h>

#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "exact_math.cuh"
#include "moe_internal.cuh"
#include "umma.cuh"

namespace fnxk {

constexpr int DU_M = 128, DU_KC = 128, DU_STAGES = 6, DU_SLOTS = 8, DU_EPI = 16, DU_THREADS = (DU_EPI + 2) * 32, DU_MAXCOLS = 3072;
constexpr int DU_ABYTES = DU_M * DU_KC, DU_BCHUNK = 16 * DU_KC, DU_MAGIC = 0x4B400000;

struct DuMaps {
    CUtensorMap w[3], d[3];
};
struct DuArgs {
    int nseg, rows[3], tile_end[3], stride[3];
    float* out[3];
    int cols, T, ntiles;
    const uint8_t* yq;
    unsigned* fault;
};

__device__ __forceinline__ void du_arrive(unsigned long long* bar) {
    asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(um_s32(bar)) : "memory");
}
// D[tmem] = A B, 128 x 16 x 32, int8 operands through descriptors, int32 result; issued by one thread
__device__ __forceinline__ void du_mma_i8(unsigned tmem, unsigned long long da, unsigned long long db, unsigned idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem), "l"(da), "l"(db),
                 "r"(idesc), "r"(0)   // p false: D = A B, nothing is accumulated across blocks
                 : "memory");
}
__device__ __forceinline__ void du_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(um_s32(bar)) : "memory");
}

// two f32 in a 64-bit register, each half rounded as its scalar operation would be (Blackwell's packed f32 pipe)
typedef unsigned long long du_f32x2;
__device__ __forceinline__ du_f32x2 du_pack(float lo, float hi) {
    du_f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ du_f32x2 du_packi(int lo, int hi) {
    du_f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ du_f32x2 du_fma2(du_f32x2 a, du_f32x2 b, du_f32x2 c) {
    du_f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ du_f32x2 du_add2(du_f32x2 a, du_f32x2 b) {
    du_f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ du_f32x2 du_mul2(du_f32x2 a, du_f32x2 b) {
    du_f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

struct DuTile {
    int seg, row0;
};
__device__ __forceinline__ DuTile du_tile(const DuArgs& a, int tile) {
    const int seg = tile < a.tile_end[0] ? 0 : tile < a.tile_end[1] ? 1 : 2;
    return DuTile{seg, (tile - (seg == 0 ? 0 : seg == 1 ? a.tile_end[0] : a.tile_end[1])) * DU_M};
}

__global__ void __launch_bounds__(DU_THREADS, 1) k_q8s_umma(const __grid_constant__ DuMaps maps, const DuArgs a) {
    extern __shared__ unsigned char du_smem[];
    unsigned char* base = du_smem + ((1024u - (um_s32(du_smem) & 1023u)) & 1023u);   // swizzled tiles start on 1024-byte boundaries
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nb = a.cols / 32, nkc = a.cols / DU_KC;
    unsigned char* a_st = base;                                                // [DU_STAGES][128 rows][128 bytes], swizzled
    unsigned char* b_op = a_st + (size_t) DU_STAGES * DU_ABYTES;               // [nkc][16 rows][128 bytes], swizzled
    uint16_t* dw_s = reinterpret_cast<uint16_t*>(b_op + (size_t) nkc * DU_BCHUNK);   // [2][128][nb] f16 block scales of a tile
    float* da_s = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(dw_s) + (size_t) 2 * DU_M * nb * 2);   // [nb][16]
    __shared__ __align__(8) unsigned long long full_a[DU_STAGES], empty_a[DU_STAGES], tm_full[DU_SLOTS], tm_empty[DU_SLOTS], dw_full[2], dw_empty[2];
    __shared__ unsigned tmem_base;
    if (tid == 0) {
        for (int s = 0; s < DU_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&full_a[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&empty_a[s])));
        }
        for (int s = 0; s < DU_SLOTS; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&tm_full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(um_s32(&tm_empty[s])), "r"(DU_EPI));
        }
        for (int s = 0; s < 2; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(um_s32(&dw_full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(um_s32(&dw_empty[s])), "r"(DU_EPI));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DU_EPI + 1) {   // all 512 columns of tensor memory: eight groups of 4 x 16
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(um_s32(&tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned a_s32 = um_s32(a_st), b_s32 = um_s32(b_op);
    bool alive = true;   // false after a wait ran out: no further wait, the results are not to be used (fault bit 8)
    if (warp == DU_EPI) {
        // ---- the TMA warp: weights do not wait for the kernel ahead
        if (lane == 0) {
            int c = 0, tp = 0, nt = 0;
            for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x, ++nt, tp ^= 1) {
                const DuTile t = du_tile(a, tile);
                const CUtensorMap* mw = &maps.w[t.seg];
                const CUtensorMap* md = &maps.d[t.seg];
                if (nt >= 2 && alive) alive = um_wait(&dw_empty[tp], (unsigned) ((nt / 2 - 1) & 1), a.fault);
                um_expect_tx(&dw_full[tp], (unsigned) (DU_M * nb * 2));
                um_tma2d(um_s32(dw_s + (size_t) tp * DU_M * nb), md, 0, t.row0, &dw_full[tp]);
                for (int kc = 0; kc < nkc; ++kc, ++c) {
                    const int s = c % DU_STAGES;
                    if (c >= DU_STAGES && alive) alive = um_wait(&empty_a[s], (unsigned) ((c / DU_STAGES - 1) & 1), a.fault);
                    um_expect_tx(&full_a[s], DU_ABYTES);
                    um_tma2d(a_s32 + s * DU_ABYTES, mw, kc * DU_KC, t.row0, &full_a[s]);
                }
            }
        }
    } else {
        // ---- everyone else: the window's activations, once the kernel that makes them has finished
        pdl_wait();
        pdl_go();
        const int et = tid < DU_EPI * 32 ? tid : tid - 32;   // 544 threads without the TMA warp
        for (int it = et; it < 16 * nb; it += DU_THREADS - 32) {
            const int t = it / nb, b = it % nb, kc = b >> 2, ch = (b & 3) * 2;
            uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
            float d = 0.f;
            if (t < a.T) {
                const unsigned* src = reinterpret_cast<const unsigned*>(a.yq + ((size_t) t * nb + b) * 36);
                d = h2f((uint16_t) (src[0] & 0xffff));
                v0 = make_uint4(src[1], src[2], src[3], src[4]);
                v1 = make_uint4(src[5], src[6], src[7], src[8]);
            }
            unsigned char* rowp = b_op + (size_t) kc * DU_BCHUNK + (t >> 3) * 1024 + (t & 7) * 128;
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (t & 7)) << 4)) = v0;
            *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ (t & 7)) << 4)) = v1;
            da_s[b * 16 + t] = d;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes before the tensor core's reads
        asm volatile("bar.sync 1, %0;" ::"n"(DU_THREADS - 32) : "memory");
        if (warp == DU_EPI + 1) {
            // ---- the issuing warp
            const unsigned idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);   // D s32, A and B s8 K-major, N 16, M 128
            int c = 0;
            for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x)
                for (int kc = 0; kc < nkc; ++kc, ++c) {
                    const int s = c % DU_STAGES, slot = c % DU_SLOTS;
                    if (alive) alive = um_wait(&full_a[s], (unsigned) ((c / DU_STAGES) & 1), a.fault);
                    if (c >= DU_SLOTS && alive) alive = um_wait(&tm_empty[slot], (unsigned) ((c / DU_SLOTS - 1) & 1), a.fault);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (lane == 0) {
                        const unsigned long long da = um_desc(a_s32 + s * DU_ABYTES), db = um_desc(b_s32 + kc * DU_BCHUNK);
#pragma unroll
                        for (int j = 0; j < 4; ++j) du_mma_i8(tmem_base + (unsigned) (slot * 64 + 16 * j), da + 2 * j, db + 2 * j, idesc);
                        du_commit(&empty_a[s]);
                        du_commit(&tm_full[slot]);
                    }
                    __syncwarp();
                }
        } else {
            // ---- the epilogue warps
            const int q = warp & 3, g = warp >> 2, r_in = 32 * q + lane;
            int c = 0, tp = 0, nt = 0;
            for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x, ++nt, tp ^= 1) {
                const DuTile t = du_tile(a, tile);
                if (alive) alive = um_wait(&dw_full[tp], (unsigned) ((nt / 2) & 1), a.fault);
                alive = __all_sync(0xffffffffu, alive);
                const uint16_t* dwr = dw_s + ((size_t) tp * DU_M + r_in) * nb;
                du_f32x2 acc01 = 0ull, acc23 = 0ull;   // window rows 4 g, + 1 and + 2, + 3 of this thread's weight row
                const du_f32x2 unmagic = du_pack(-12582912.0f, -12582912.0f);
                const float* dap = da_s + 4 * g;
#pragma unroll 2
                for (int kc = 0; kc < nkc; ++kc, ++c) {
                    const int slot = c % DU_SLOTS;
                    const uint2 dwh = *reinterpret_cast<const uint2*>(dwr + 4 * kc);   // this stage's four block scales
                    if (alive) alive = um_wait(&tm_full[slot], (unsigned) ((c / DU_SLOTS) & 1), a.fault);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned v[16];
                    const unsigned ta = tmem_base + ((unsigned) (32 * q) << 16) + (unsigned) (slot * 64 + 4 * g);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(v[4 * j]), "=r"(v[4 * j + 1]), "=r"(v[4 * j + 2]), "=r"(v[4 * j + 3])
                                     : "r"(ta + 16 * j));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) du_arrive(&tm_empty[slot]);   // the group may be overwritten: its values are in registers
                    const unsigned dww[2] = {dwh.x, dwh.y};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float dw = h2f((uint16_t) (j & 1 ? dww[j >> 1] >> 16 : dww[j >> 1] & 0xffff));
                        const du_f32x2 dw2 = du_pack(dw, dw);
                        const ulonglong2 da4 = *reinterpret_cast<const ulonglong2*>(dap + (size_t) (4 * kc + j) * 16);
                        // (float) isum exactly: the bits of 1.5 * 2^23 + isum, less 1.5 * 2^23; then acc = fma(fl(dw da), ., acc)
                        const du_f32x2 f01 = du_add2(du_packi((int) v[4 * j] + DU_MAGIC, (int) v[4 * j + 1] + DU_MAGIC), unmagic);
                        const du_f32x2 f23 = du_add2(du_packi((int) v[4 * j + 2] + DU_MAGIC, (int) v[4 * j + 3] + DU_MAGIC), unmagic);
                        acc01 = du_fma2(du_mul2(dw2, da4.x), f01, acc01);
                        acc23 = du_fma2(du_mul2(dw2, da4.y), f23, acc23);
                    }
                }
                float acc[4];
                asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[0]), "=f"(acc[1]) : "l"(acc01));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[2]), "=f"(acc[3]) : "l"(acc23));
                __syncwarp();
                if (lane == 0) du_arrive(&dw_empty[tp]);
                const int seg = t.seg, row = t.row0 + r_in;
                float* out = seg == 0 ? a.out[0] : seg == 1 ? a.out[1] : a.out[2];
                const int stride = seg == 0 ? a.stride[0] : seg == 1 ? a.stride[1] : a.stride[2];
                const int rows = seg == 0 ? a.rows[0] : seg == 1 ? a.rows[1] : a.rows[2];
                if (row < rows) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (4 * g + i < a.T) out[(size_t) (4 * g + i) * stride + row] = acc[i];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == DU_EPI + 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
}

// ---- host side: tensor maps over this GPU's own memory (plain loads, no multicast)
size_t q8s_umma_smem(int cols) {
    const int nb = cols / 32, nkc = cols / DU_KC;
    return (size_t) DU_STAGES * DU_ABYTES + (size_t) nkc * DU_BCHUNK + (size_t) 2 * DU_M * nb * 2 + (size_t) nb * 16 * 4 + 1024;
}

// the tensor-core dense kernel over 1..3 matrices of `cols` columns; -1 when the shape is not its (the caller uses the
// kernels of dense.cu), 1 on an error
int q8s_umma_launch(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int nseg, int cols, const void* yq, int T, cudaStream_t st,
                    const char* what) {
    if (cols % 256 || cols < 256 || cols > DU_MAXCOLS || nseg < 1 || nseg > 3 || T < 1 || T > FNX_MAXT) return -1;
    long tiles = 0;
    for (int s = 0; s < nseg; ++s) {
        if ((uintptr_t) w[s].q % 16 || (uintptr_t) w[s].d % 16 || rows[s] < 1) return -1;
        tiles += (rows[s] + DU_M - 1) / DU_M;
    }
    if (tiles < 64) return -1;   // too few 128-row tiles to fill the GPU: the streaming kernel does better
    UmEncode enc = um_encoder();
    unsigned* fault = device_fault_word();
    if (!enc || !fault) return fail("%s: no tensor-map encoder or fault word", what);
    DuMaps maps;
    DuArgs a{};
    a.nseg = nseg, a.cols = cols, a.T = T, a.yq = (const uint8_t*) yq, a.fault = fault;
    int nt = 0;
    for (int s = 0; s < 3; ++s) {
        const int k = s < nseg ? s : nseg - 1;
        const cuuint64_t gd_w[2] = {(cuuint64_t) cols, (cuuint64_t) rows[k]}, gs_w[1] = {(cuuint64_t) cols};
        const cuuint32_t bx_w[2] = {DU_KC, DU_M}, es[2] = {1, 1};
        const cuuint64_t gd_d[2] = {(cuuint64_t) (cols / 32), (cuuint64_t) rows[k]}, gs_d[1] = {(cuuint64_t) (cols / 32) * 2};
        const cuuint32_t bx_d[2] = {(cuuint32_t) (cols / 32), DU_M};
        if (enc(&maps.w[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*) w[k].q, gd_w, gs_w, bx_w, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            enc(&maps.d[s], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, (void*) w[k].d, gd_d, gs_d, bx_d, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return fail("%s: tensor map of a %d x %d matrix refused", what, rows[k], cols);
        a.rows[s] = rows[k], a.stride[s] = out_stride[k], a.out[s] = out[k];
        if (s < nseg) nt += (rows[s] + DU_M - 1) / DU_M;
        a.tile_end[s] = nt;
    }
    a.ntiles = nt;
    static int nsm = 0;
    if (!nsm) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || nsm < 1) nsm = 148;
    }
    const size_t sm = q8s_umma_smem(cols);
    if (smem_optin(k_q8s_umma, sm, what)) return 1;
    launch(1, k_q8s_umma, std::min(nsm, nt), DU_THREADS, sm, st, maps, a);
    return launch_ok(what);
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_q8s_gemv_blocks(FnxQ8S w, int rows, int cols, const void* y, float* out, int out_stride, int T, void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT, "q8s_gemv_blocks: T %d outside 1..%d", T, FNX_MAXT);
    const FnxQ8S ws[1] = {w};
    const int rs[1] = {rows}, strides[1] = {out_stride};
    float* outs[1] = {out};
    const int rc = q8s_umma_launch(ws, rs, outs, strides, 1, cols, y, T, strm(st), "q8s_gemv_blocks");
    if (rc < 0) return fail("q8s_gemv_blocks: %d x %d is not a shape of the tensor-core kernel (columns a multiple of 256 up to %d, at least 64 tiles of 128 rows, 16-byte aligned planes)", rows, cols, DU_MAXCOLS);
    return rc;
}
}
