// Output-head reductions of the verify window: per-slice argmax and the sampler's exact top-64 with penalties.
// Replaces reference src/kernels.cu:870-908 (k_argmax, k_argmax_fin), :1454-1470 (k_penalize_row) and src/topk.cuh.
#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

// ---------------------------------------------------------------- argmax
// keys[t] = max over the row of (fkey(value) << 32 | ~index): the largest value, the lowest index on a tie
constexpr int AM_THREADS = 256;

__global__ void __launch_bounds__(AM_THREADS) k_argmax(const float* __restrict__ logits, int rows, unsigned long long* keys,
                                                      unsigned* err) {
    const int t = blockIdx.y;
    const float* r = logits + (size_t) t * rows;
    pdl_wait();
    pdl_go();
    unsigned long long best = 0;
    bool bad = false;
    for (int i = blockIdx.x * AM_THREADS + threadIdx.x; i < rows; i += gridDim.x * AM_THREADS) {
        const float v = r[i];
        bad = bad || !isfinite(v);
        const unsigned long long k = (unsigned long long) fkey(v) << 32 | (unsigned) ~i;
        best = k > best ? k : best;
    }
    if (bad) atomicOr(err, 16u);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
        best = ok > best ? ok : best;
    }
    __shared__ unsigned long long wbest[AM_THREADS / 32];   // one atomic per block
    if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < AM_THREADS / 32; ++w) best = wbest[w] > best ? wbest[w] : best;
        atomicMax(&keys[t], best);
    }
}
// decodes the keys into (value, index + v0) and leaves them at zero for the next call
__global__ void k_argmax_fin(unsigned long long* keys, int T, int v0, float* bv, int* bi) {
    const int t = threadIdx.x;
    pdl_wait();
    pdl_go();
    if (t >= T) return;
    const unsigned long long k = keys[t];
    bv[t] = fkey_inv((unsigned) (k >> 32));
    bi[t] = (int) ~(unsigned) k + v0;
    keys[t] = 0ull;
}

// ---------------------------------------------------------------- penalties
__device__ __forceinline__ float penalized(float l, int cnt, float repeat, float freq, float present) {
    l = l <= 0.f ? fmul(l, repeat) : fdiv(l, repeat);
    return fsub(fsub(l, fmul((float) cnt, freq)), present);
}
__global__ void k_penalize_row(float* L, int n, const int* pen, const float* par) {
    const int k = pen[0];
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const int j = pen[1 + i], cnt = pen[1 + k + i];
        if (j < 0 || j >= n || cnt <= 0) continue;
        L[j] = penalized(L[j], cnt, par[0], par[1], par[2]);
    }
}

// ---------------------------------------------------------------- top-64 per row
// A block per row.  Four 8-bit radix passes find the key K of the 64th highest logit and how many of the logits equal
// to K are needed (`want`); every logit above K is a candidate, and the ties at K are taken in ascending index order
// by a block-wide ordered count, so the set is exact however wide the tie; the 64 are then sorted by (logit desc, id
// asc).
constexpr int TK_THREADS = 1024;

__global__ void __launch_bounds__(TK_THREADS) k_topk_rows(float* __restrict__ logits, int n, int v0, const int* __restrict__ pen_tok,
                                                         const int* __restrict__ pen_cnt, const int* __restrict__ pen_n, int pen_stride,
                                                         const float* __restrict__ pen_par, float* __restrict__ out_v,
                                                         int* __restrict__ out_i, unsigned* err) {
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* L = logits + (size_t) row * n;
    bool bad = false;
    for (int j = tid; j < n; j += TK_THREADS) bad = bad || !isfinite(L[j]);
    if (bad) atomicOr(err, 16u);
    __syncthreads();
    if (pen_n) {
        const float repeat = pen_par[row * 3], freq = pen_par[row * 3 + 1], present = pen_par[row * 3 + 2];
        for (int i = tid; i < pen_n[row]; i += TK_THREADS) {
            const int tok = pen_tok[row * pen_stride + i] - v0, cnt = pen_cnt[row * pen_stride + i];
            if (tok < 0 || tok >= n || cnt <= 0) continue;
            L[tok] = penalized(L[tok], cnt, repeat, freq, present);
        }
    }
    __syncthreads();
    __shared__ unsigned hist[256];
    __shared__ unsigned prefix_s, want_s;
    unsigned prefix = 0, mask = 0, want = FNX_TOPK_N;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = tid; b < 256; b += TK_THREADS) hist[b] = 0;
        __syncthreads();
        for (int jb = 0; jb < n; jb += TK_THREADS) {
            const int j = jb + tid;
            const unsigned k = j < n ? fkey(L[j]) : 0u;
            const bool in = j < n && (k & mask) == prefix;
            const unsigned bin = in ? (k >> shift) & 255u : 256u;
            const unsigned peers = __match_any_sync(0xffffffffu, bin);
            if (in && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned) __popc(peers));
        }
        __syncthreads();
        if (tid == 0) {
            unsigned acc = 0;
            int b = 255;
            for (; b > 0; --b) {
                if (acc + hist[b] >= want) break;
                acc += hist[b];
            }
            prefix_s = prefix | ((unsigned) b << shift);
            want_s = want - acc;
        }
        __syncthreads();
        prefix = prefix_s;
        want = want_s;
        mask |= 255u << shift;
        __syncthreads();
    }
    __shared__ unsigned long long cand[FNX_TOPK_N];
    __shared__ unsigned n_above;
    __shared__ unsigned warp_n[TK_THREADS / 32];
    if (tid == 0) n_above = 0;
    if (tid < FNX_TOPK_N) cand[tid] = 0ull;
    __syncthreads();
    for (int j = tid; j < n; j += TK_THREADS) {
        const unsigned k = fkey(L[j]);
        if (k > prefix) {
            const unsigned s = atomicAdd(&n_above, 1u);
            if (s < FNX_TOPK_N) cand[s] = ((unsigned long long) k << 32) | (0xffffffffu - (unsigned) j);
        }
    }
    const unsigned base = FNX_TOPK_N - want;   // how many lie above K
    unsigned taken = 0;
    for (int jb = 0; jb < n && taken < want; jb += TK_THREADS) {
        const int j = jb + tid;
        const bool eq = j < n && fkey(L[j]) == prefix;
        const unsigned bal = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) warp_n[warp] = (unsigned) __popc(bal);
        __syncthreads();
        unsigned before = (unsigned) __popc(bal & ((1u << lane) - 1u)), total = 0;
        for (int w = 0; w < TK_THREADS / 32; ++w) {
            before += w < warp ? warp_n[w] : 0u;
            total += warp_n[w];
        }
        if (eq && taken + before < want) cand[base + taken + before] = ((unsigned long long) prefix << 32) | (0xffffffffu - (unsigned) j);
        taken += total;
        __syncthreads();
    }
    __syncthreads();
    for (int size = 2; size <= FNX_TOPK_N; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < FNX_TOPK_N) {
                const int o = tid ^ stride;
                if (o > tid) {
                    const bool desc = (tid & size) == 0;
                    const unsigned long long a = cand[tid], b = cand[o];
                    if (desc ? a < b : a > b) {
                        cand[tid] = b;
                        cand[o] = a;
                    }
                }
            }
            __syncthreads();
        }
    if (tid < FNX_TOPK_N) {
        const unsigned long long c = cand[tid];
        const int j = (int) (0xffffffffu - (unsigned) (c & 0xffffffffu));
        out_i[row * FNX_TOPK_N + tid] = v0 + j;
        out_v[row * FNX_TOPK_N + tid] = L[j];
    }
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

int fnx_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i, unsigned long long* keys, unsigned* err,
               void* st) {
    FNX_REQUIRE(T >= 1 && T <= FNX_MAXT && rows >= 1, "argmax: T %d, %d logits a row", T, rows);
    int gx = (rows + AM_THREADS * 8 - 1) / (AM_THREADS * 8);
    gx = gx < 1 ? 1 : gx > 64 ? 64 : gx;
    launch(0, k_argmax, dim3(gx, T), AM_THREADS, 0, strm(st), logits, rows, keys, err);
    if (launch_ok("argmax")) return 1;
    launch(0, k_argmax_fin, 1, 32, 0, strm(st), keys, T, v0, best_v, best_i);
    return launch_ok("argmax fin");
}

int fnx_penalize_row(float* row, int n, const int* pen, const float* par, void* st) {
    k_penalize_row<<<1, 256, 0, strm(st)>>>(row, n, pen, par);
    return launch_ok("penalize_row");
}

int fnx_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n, int pen_stride,
                   const float* pen_par, float* out_v, int* out_i, unsigned* err, void* st) {
    FNX_REQUIRE(n >= FNX_TOPK_N, "top_tokens: %d logits a row, fewer than the %d candidates", n, FNX_TOPK_N);
    FNX_REQUIRE(T >= 1, "top_tokens: no rows");
    k_topk_rows<<<T, TK_THREADS, 0, strm(st)>>>(logits, n, v0, pen_tok, pen_cnt, pen_n, pen_stride, pen_par, out_v, out_i, err);
    return launch_ok("top_tokens");
}
}
