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
#include <algorithm>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

constexpr int RS_THREADS = 256;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ float4 ld_peer(const float* p) {   // peer memory: not through L1
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
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
}
