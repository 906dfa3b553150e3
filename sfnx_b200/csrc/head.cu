// Output-head reductions of the verify window: per-slice argmax and the sampler's exact 64 candidates with penalties.
// Covers what reference src/kernels.cu:870-908 (argmax), :1454-1470 (penalize_row) and src/topk.cuh (top_tokens)
// compute; the kernels are this library's own.
//
// Both selections order logits by a 64-bit composite: (order-preserving key of the value, with -0 folded into +0)
// in the high word and the complement of the index in the low word, so "larger composite" means "larger logit, then lower
// index" and no two elements compare equal.
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

__device__ __forceinline__ unsigned long long composite(float v, unsigned idx) {
    return ((unsigned long long) fkey(fadd(v, 0.f)) << 32) | (0xffffffffu - idx);
}
__device__ __forceinline__ unsigned comp_index(unsigned long long c) { return 0xffffffffu - (unsigned) (c & 0xffffffffu); }

// ---------------------------------------------------------------- argmax
// One launch: grid (AM_SPLIT, T).  A block scans its stripe of row t with every thread keeping the largest composite it
// has seen, the block's largest goes into keys[t] by one 64-bit atomic, and the block that arrives last at the row's
// counter (keys[FNX_MAXT + t]) decodes the row's result and puts both words back to zero for the next call.
constexpr int AM_THREADS = 512, AM_SPLIT = 64;

__global__ void __launch_bounds__(AM_THREADS) k_argmax_rows(const float* __restrict__ logits, int rows, int v0, float* __restrict__ bv,
                                                           int* __restrict__ bi, unsigned long long* keys, unsigned* err) {
    const int t = blockIdx.y, tid = threadIdx.x;
    const float* row = logits + (size_t) t * rows;
    pdl_wait();
    pdl_go();
    const int per = (rows + gridDim.x - 1) / gridDim.x, lo = blockIdx.x * per, hi = min(rows, lo + per);
    unsigned long long best = 0ull;
    unsigned finite = 1u;
    for (int i0 = lo; i0 < hi; i0 += 4 * AM_THREADS) {   // four independent loads a thread before the compares
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * AM_THREADS + tid;
            v[k] = i < hi ? row[i] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * AM_THREADS + tid;
            if (i < hi) {
                finite &= (unsigned) isfinite(v[k]);
                // the plain key here (not the folded one): the result is a value, and -0 must come back as -0
                const unsigned long long c = ((unsigned long long) fkey(v[k]) << 32) | (0xffffffffu - (unsigned) i);
                best = c > best ? c : best;
            }
        }
    }
    __shared__ unsigned long long wbest[AM_THREADS / 32];
    __shared__ unsigned any_bad;
    if (tid == 0) any_bad = 0u;
    __syncthreads();
    if (!finite) any_bad = 1u;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const unsigned long long other = __shfl_down_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((tid & 31) == 0) wbest[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < AM_THREADS / 32; ++w) best = wbest[w] > best ? wbest[w] : best;
        if (any_bad) atomicOr(err, 16u);
        atomicMax(&keys[t], best);
        __threadfence();
        unsigned* count = reinterpret_cast<unsigned*>(&keys[FNX_MAXT + t]);
        if (atomicAdd(count, 1u) == gridDim.x - 1) {   // the row's last block: every stripe's maximum is in keys[t]
            __threadfence();
            const unsigned long long k = atomicExch(&keys[t], 0ull);
            bv[t] = fkey_inv((unsigned) (k >> 32));
            bi[t] = (int) comp_index(k) + v0;
            *count = 0u;
        }
    }
}

// ---------------------------------------------------------------- penalties
__device__ __forceinline__ float penalized(float l, int cnt, float repeat, float freq, float present) {
    l = l <= 0.f ? fmul(l, repeat) : fdiv(l, repeat);
    return fsub(fsub(l, fmul((float) cnt, freq)), present);
}
// pen = [k, k token ids, k counts]; par = (repeat, frequency, presence)
__global__ void k_penalize_list(float* row, int n, const int* __restrict__ pen, const float* __restrict__ par) {
    const int k = pen[0];
    const float repeat = par[0], freq = par[1], present = par[2];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < k; i += gridDim.x * blockDim.x) {
        const int tok = pen[1 + i], cnt = pen[1 + k + i];
        if (tok >= 0 && tok < n && cnt > 0) row[tok] = penalized(row[tok], cnt, repeat, freq, present);
    }
}

// ---------------------------------------------------------------- the 64 best of every row
// A cluster of TK_CL blocks per row, each on an eighth of the row (the logits are a few MB and sit in L2).
//  1. A bound that costs one pass: the row is cut into 64 groups (four warps' stripes each); every group's maximum is
//     an element of the row, so the smallest of the 64 maxima has at least 64 elements at or above it.  For logits that
//     are spread out, a few hundred elements pass it.
//  2. One more pass gathers every element at or above the bound as a composite into the block's list; the lists meet in
//     the cluster's first block through distributed shared memory.
//  3. There an element's place in the output is the number of gathered composites larger than its own: places 0..63 are
//     written, already in (logit descending, id ascending) order.
// If more than TK_CAP elements pass the bound (wide ties, a flat row) the bound is first raised by a most-significant-
// digit radix selection over the composites, 11 bits a pass with the blocks' histograms added through distributed
// shared memory, until what is at or above it fits the lists; composites are distinct, so that always ends (six passes
// at most) and ties of any width are cut in index order.
constexpr int TK_CL = 8, TK_THREADS = 1024, TK_WARPS = TK_THREADS / 32, TK_BINS = 2048, TK_CAP = 2048, TK_GROUPS_PER_BLOCK = 64 / TK_CL;

struct TopkArgs {
    float* logits;
    int n, v0;
    const int *pen_tok, *pen_cnt, *pen_n;
    int pen_stride;
    const float* pen_par;
    float* out_v;
    int* out_i;
    unsigned* err;
};

__global__ void __cluster_dims__(TK_CL, 1, 1) __launch_bounds__(TK_THREADS) k_top64_rows(const TopkArgs a) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int row = blockIdx.y, rank = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* L = a.logits + (size_t) row * a.n;
    const int per = (a.n + TK_CL - 1) / TK_CL, lo = rank * per, hi = min(a.n, lo + per);
    __shared__ unsigned hist[TK_BINS];
    __shared__ unsigned long long mine[TK_CAP], all[TK_CAP];
    __shared__ unsigned long long gmax[TK_WARPS];
    __shared__ unsigned long long block_min, low_s;   // this block's smallest group maximum; the bound everyone agreed on
    __shared__ unsigned n_mine, n_pass, n_all, wtot[TK_WARPS];
    __shared__ unsigned sel_bin, sel_above, sel_count;
    // ---- penalties on this block's part of the row (the listed tokens are few)
    if (a.pen_n) {
        const float repeat = a.pen_par[row * 3], freq = a.pen_par[row * 3 + 1], present = a.pen_par[row * 3 + 2];
        for (int i = tid; i < a.pen_n[row]; i += TK_THREADS) {
            const int tok = a.pen_tok[row * a.pen_stride + i] - a.v0, cnt = a.pen_cnt[row * a.pen_stride + i];
            if (tok < lo || tok >= hi || cnt <= 0) continue;
            const float l = L[tok];
            if (!isfinite(l)) atomicOr(a.err, 16u);
            L[tok] = penalized(l, cnt, repeat, freq, present);
        }
        __syncthreads();
    }
    // ---- 1. group maxima -> bound
    {
        unsigned long long best = 0ull;
        unsigned finite = 1u;
        for (int j = lo + tid; j < hi; j += TK_THREADS) {
            const float v = L[j];
            finite &= (unsigned) isfinite(v);
            const unsigned long long c = composite(v, (unsigned) j);
            best = c > best ? c : best;
        }
        if (!finite) atomicOr(a.err, 16u);
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) gmax[warp] = best;
        if (tid == 0) n_mine = 0u, n_pass = 0u;
        __syncthreads();
        if (tid == 0) {
            unsigned long long bm = ~0ull;
            for (int g = 0; g < TK_GROUPS_PER_BLOCK; ++g) {   // a group = TK_WARPS / TK_GROUPS_PER_BLOCK neighbouring warps
                unsigned long long m = 0ull;
                for (int w = 0; w < TK_WARPS / TK_GROUPS_PER_BLOCK; ++w) {
                    const unsigned long long x = gmax[g * (TK_WARPS / TK_GROUPS_PER_BLOCK) + w];
                    m = x > m ? x : m;
                }
                bm = m < bm ? m : bm;
            }
            block_min = bm;   // 0 when a group is empty: then nothing is excluded
        }
    }
    cluster.sync();
    if (tid == 0) {
        unsigned long long b = ~0ull;
        for (int r = 0; r < TK_CL; ++r) {
            const unsigned long long x = *cluster.map_shared_rank(&block_min, r);
            b = x < b ? x : b;
        }
        low_s = b & 0xffffffff00000000ull;   // every index of that value
    }
    __syncthreads();
    unsigned long long low = low_s;
    // ---- 2. gather what is at or above `low` (optimistically: past the list's end only the count goes on)
    auto gather = [&]() {
        for (int j0 = lo; j0 < hi; j0 += TK_THREADS) {
            const int j = j0 + tid;
            const unsigned long long c = j < hi ? composite(L[j], (unsigned) j) : 0ull;
            const bool in = j < hi && c >= low;
            const unsigned bal = __ballot_sync(0xffffffffu, in);
            if (bal) {
                unsigned base = 0;
                if (lane == 0) base = atomicAdd(&n_pass, (unsigned) __popc(bal));
                base = __shfl_sync(0xffffffffu, base, 0);
                const unsigned at = base + (unsigned) __popc(bal & ((1u << lane) - 1u));
                if (in && at < TK_CAP) mine[at] = c;
            }
        }
    };
    gather();
    cluster.sync();
    unsigned total = 0;
    for (int r = 0; r < TK_CL; ++r) total += *cluster.map_shared_rank(&n_pass, r);
    if (total > TK_CAP) {
        // ---- the bound is too low: radix selection over the composites at or above it
        unsigned want = FNX_TOPK_N;
        unsigned long long prefix = 0ull, hi_mask = 0ull;
        int shift = 64;
#pragma unroll 1
        while (true) {
            const int width = shift >= 11 ? 11 : shift;
            shift -= width;
            cluster.sync();   // the histograms of the pass before have been read by every block
            for (int b = tid; b < TK_BINS; b += TK_THREADS) hist[b] = 0u;
            __syncthreads();
            for (int j = lo + tid; j < hi; j += TK_THREADS) {
                const unsigned long long c = composite(L[j], (unsigned) j);
                if (c >= low && (c & hi_mask) == prefix) atomicAdd(&hist[(unsigned) (c >> shift) & ((1u << width) - 1u)], 1u);
            }
            cluster.sync();
            // thread i owns bins 2 i, 2 i + 1 of the cluster-wide histogram; an inclusive suffix sum over the threads
            unsigned c0 = 0, c1 = 0;
            for (int r = 0; r < TK_CL; ++r) {
                const unsigned* h = cluster.map_shared_rank(hist, r);
                c0 += h[2 * tid], c1 += h[2 * tid + 1];
            }
            unsigned suf = c0 + c1;   // of this thread and every thread above it
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned x = __shfl_down_sync(0xffffffffu, suf, o);
                if (lane + o < 32) suf += x;
            }
            if (lane == 0) wtot[warp] = suf;
            __syncthreads();
            unsigned above_warps = 0;
            for (int w = warp + 1; w < TK_WARPS; ++w) above_warps += wtot[w];
            suf += above_warps;
            const unsigned above_me = suf - c0 - c1;                // in bins above 2 i + 1
            if (above_me < want && above_me + c1 >= want) sel_bin = 2 * tid + 1, sel_above = above_me, sel_count = c1;
            else if (above_me + c1 < want && suf >= want) sel_bin = 2 * tid, sel_above = above_me + c1, sel_count = c0;
            __syncthreads();
            want -= sel_above;
            prefix |= (unsigned long long) sel_bin << shift;
            hi_mask |= (unsigned long long) ((1u << width) - 1u) << shift;
            // what lies above the chosen digit is at most 63 elements; with the digit's own it must fit the list
            if (FNX_TOPK_N - want + sel_count <= TK_CAP || shift == 0) break;
        }
        low = prefix > low ? prefix : low;
        cluster.sync();   // nobody still reads n_pass or the histograms
        if (tid == 0) n_pass = 0u;
        __syncthreads();
        gather();
        cluster.sync();
    }
    // ---- 3. the cluster's first block places the candidates
    if (rank == 0) {
        if (tid == 0) n_all = 0u;
        __syncthreads();
        for (int r = 0; r < TK_CL; ++r) {
            const unsigned cnt = min(*cluster.map_shared_rank(&n_pass, r), (unsigned) TK_CAP);
            const unsigned long long* src = cluster.map_shared_rank(mine, r);
            __shared__ unsigned base_s;
            if (tid == 0) base_s = n_all, n_all = min(n_all + cnt, (unsigned) TK_CAP);
            __syncthreads();
            for (unsigned i = tid; i < cnt && base_s + i < TK_CAP; i += TK_THREADS) all[base_s + i] = src[i];
            __syncthreads();
        }
        const unsigned n = n_all;
        for (unsigned i = tid; i < n; i += TK_THREADS) {
            const unsigned long long c = all[i];
            unsigned place = 0;
            for (unsigned k = 0; k < n; ++k) place += (unsigned) (all[k] > c);
            if (place < FNX_TOPK_N) {
                const unsigned j = comp_index(c);
                a.out_i[row * FNX_TOPK_N + place] = a.v0 + (int) j;
                a.out_v[row * FNX_TOPK_N + place] = L[j];
            }
        }
    }
    cluster.sync();   // no block leaves while its list may still be read
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i, unsigned long long* keys, unsigned* err,
               void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && rows >= 1, "argmax: T %d, %d logits a row", T, rows);
    FNX_REQUIRE(logits && best_v && best_i && keys && err, "argmax: a null buffer");
    // stripes of about 2048 logits (one round of four loads a thread), at most AM_SPLIT a row
    const int split = std::max(1, std::min(AM_SPLIT, rows / (4 * AM_THREADS)));
    launch(0, k_argmax_rows, dim3(split, T), AM_THREADS, 0, strm(st), logits, rows, v0, best_v, best_i, keys, err);
    return launch_ok("argmax");
}

int fnx_penalize_row(float* row, int n, const int* pen, const float* par, void* st) {
    FNX_REQUIRE(row && pen && par && n >= 1, "penalize_row: a null buffer");
    k_penalize_list<<<4, 256, 0, strm(st)>>>(row, n, pen, par);
    return launch_ok("penalize_row");
}

int fnx_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n, int pen_stride,
                   const float* pen_par, float* out_v, int* out_i, unsigned* err, void* st) {
    FNX_REQUIRE(n >= FNX_TOPK_N, "top_tokens: %d logits a row, fewer than the %d candidates", n, FNX_TOPK_N);
    FNX_REQUIRE(T >= 1 && T <= 65535, "top_tokens: %d rows", T);
    FNX_REQUIRE(!pen_n || (pen_tok && pen_cnt && pen_par), "top_tokens: penalty counts without their lists");
    const TopkArgs a{logits, n, v0, pen_tok, pen_cnt, pen_n, pen_stride, pen_par, out_v, out_i, err};
    k_top64_rows<<<dim3(TK_CL, T), TK_THREADS, 0, strm(st)>>>(a);
    return launch_ok("top_tokens");
}
}
