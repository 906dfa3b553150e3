// Error reporting, activation quantisation, RMS norm, batched copies, load-time repacks, synthetic weights.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "exact_math.cuh"

namespace fnxk {

char* err_buf() {
    static thread_local char buf[512];
    return buf;
}
int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), 512, fmt, ap);
    va_end(ap);
    return 1;
}
bool g_pdl_hold = false;
bool pdl_on(int kind) {
    static const bool off = getenv("FNX_NO_PDL") != nullptr;
    // classes: 0 small row kernels, 1 dense streaming, 2 router, 3 expert gate|up, 4 expert down, 5 DeltaNet, 6 attention
    // scan, 7 f32 GEMV.  Measured on the 8-layer benchmark window (ms per window; none 2.52): dense alone 2.39, router
    // alone 2.43, gate|up alone 2.74 (its blocks take the registers of every multiprocessor while the router still runs
    // and push the shared expert off its overlap), classes 0, 1, 2, 4, 5 together 2.32.
    static const unsigned mask = getenv("FNX_PDL_MASK") ? (unsigned) strtoul(getenv("FNX_PDL_MASK"), nullptr, 0) : 0x17u;
    return !off && !g_pdl_hold && (mask >> kind & 1u);
}
void pdl_hold(bool hold) { g_pdl_hold = hold; }

// ---- the device-side fault word: bit 8 = a bounded on-chip wait (an mbarrier of the tcgen05 kernels) ran out.  Kernels
// launched inside a window report into the window's own error word instead (fault_sink), so that the host sees the
// timeout with the window's other faults.
static __device__ unsigned g_fault = 0;
static thread_local unsigned* g_fault_sink = nullptr;
void fault_sink(unsigned* err) { g_fault_sink = err; }
unsigned* device_fault_word() {
    if (g_fault_sink) return g_fault_sink;
    static unsigned* ptr[64] = {};   // per device; written without a lock: every writer stores the same address
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev] && cudaGetSymbolAddress((void**) &ptr[dev], g_fault) != cudaSuccess) ptr[dev] = nullptr;
    return ptr[dev];
}
// every kernel launch of the library is followed by one launch_ok(): the launches are counted here
static std::atomic<long> g_launches{0};
long launch_count(bool reset) { return reset ? g_launches.exchange(0) : g_launches.load(); }
int launch_ok(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
}

// ---------------------------------------------------------------- q8_1 (reference src/kernels.cu:99-113)
// a warp per 32-value block: d = amax / 127, q = round-half-away(x / d), the block's f16 d and f16 sum
__device__ __forceinline__ void q8_1_store(float xi, uint8_t* blk, int lane) {
    const float amax = wmax(fabsf(xi)), sum = wsum(xi);
    const float d = fdiv(amax, 127.0f);
    const int8_t qv = amax == 0.0f ? 0 : (int8_t) roundf(fdiv(xi, d));
    reinterpret_cast<int8_t*>(blk + 4)[lane] = qv;
    if (lane == 0) {
        reinterpret_cast<uint16_t*>(blk)[0] = f2h(d);
        reinterpret_cast<uint16_t*>(blk)[1] = f2h(sum);
    }
}

__global__ void __launch_bounds__(256) k_quantize_q8_1(const float* __restrict__ x, uint8_t* __restrict__ q, int n) {
    const int row = blockIdx.y, b = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_go();
    if (b >= n / 32) return;
    q8_1_store(x[(size_t) row * n + b * 32 + lane], q + ((size_t) row * (n / 32) + b) * 36, lane);
}

// ---------------------------------------------------------------- RMS norm (reference src/kernels.cu:2199-2206)
// 1024 threads a row: thread i sums the squares of columns i, i + 1024, ... in order, warp xor-trees, the 32 warps
// added in ascending order; y = (x r) w.  Optional residual add first and q8_1 copy of y after.
__global__ void __launch_bounds__(1024) k_rms_norm_rows(float* __restrict__ x, const float* __restrict__ add,
                                                        const float* __restrict__ w, float* __restrict__ y,
                                                        uint8_t* __restrict__ q, int n, float eps) {
    __shared__ float sh[32];
    float* xr = x + (size_t) blockIdx.x * n;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    pdl_go();
    float s = 0.f;
    for (int i = tid; i < n; i += 1024) {
        float v = xr[i];
        if (add) {
            v = fadd(v, add[(size_t) blockIdx.x * n + i]);
            xr[i] = v;
        }
        s = ffma(v, v, s);
    }
    s = wsum(s);
    if (lane == 0) sh[warp] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) tot = fadd(tot, sh[i]);
    const float r = ex_rsqrt(fadd(fdiv(tot, (float) n), eps));
    for (int i0 = 0; i0 < n; i0 += 1024) {   // n % 32 == 0: a warp's columns are one q8_1 block
        const int i = i0 + tid;
        const bool live = i < n;
        const float v = live ? fmul(fmul(xr[i], r), w[i]) : 0.f;
        if (live && y) y[(size_t) blockIdx.x * n + i] = v;
        if (q && (i0 + warp * 32) < n) q8_1_store(v, q + ((size_t) blockIdx.x * (n / 32) + (i >> 5)) * 36, lane);
    }
}

// ---------------------------------------------------------------- batched copies (reference src/kernels.cu:1473-1485)
__global__ void __launch_bounds__(256) k_copy_many(const FnxCopyJob* __restrict__ jobs) {
    pdl_wait();
    pdl_go();
    const FnxCopyJob j = jobs[blockIdx.y];
    float4* d = reinterpret_cast<float4*>(j.dst);
    const float4* s = reinterpret_cast<const float4*>(j.src);
    const size_t n = j.bytes / 16, step = (size_t) gridDim.x * blockDim.x;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) d[i] = s[i];
}

// ---------------------------------------------------------------- L2 prefetch (reference src/kernels.cu:2173-2193)
// The reference touches every 32-byte sector with a load; here the TMA unit's bulk prefetch brings 32 KB a thread into L2
// (cp.async.bulk.prefetch.L2: no registers, no shared memory, nothing to wait for), so a launch of a few hundred threads
// covers tens of MB and leaves the multiprocessors to the kernels it runs beside.
constexpr unsigned PF_CHUNK = 32 * 1024;
__global__ void k_l2_prefetch(const char* p, size_t bytes) {
    const size_t at = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * PF_CHUNK;
    if (at >= bytes) return;
    const unsigned n = (unsigned) (bytes - at < PF_CHUNK ? bytes - at : PF_CHUNK) & ~15u;
    if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + at), "r"(n) : "memory");
}

// ---------------------------------------------------------------- repacks
__global__ void k_repack_q8_0(const uint8_t* __restrict__ blocks, int8_t* __restrict__ q, uint16_t* __restrict__ d, size_t nblocks) {
    const size_t b = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint8_t* p = blocks + b * 34;
    d[b] = (uint16_t) (p[0] | (p[1] << 8));
    for (int l = 0; l < 32; ++l) q[b * 32 + l] = (int8_t) p[2 + l];
}

__device__ __forceinline__ int q6k_code(const uint8_t* blk, int i) {
    const int half = i / 128, r = i % 128, l = r % 32, quad = r / 32;
    const uint8_t* ql = blk + 64 * half;
    const uint8_t* qh = blk + 128 + 32 * half;
    const int lo = (quad & 1) ? ql[l + 32] : ql[l];
    const int nib = (quad >= 2) ? (lo >> 4) : (lo & 0xF);
    return nib | (((qh[l] >> (2 * quad)) & 3) << 4);
}
// a thread per 32-column unit
__global__ void k_repack_q6k(const uint8_t* __restrict__ blocks, size_t rows, size_t src_cols, size_t c0, size_t cols,
                             uint8_t* __restrict__ QL, uint8_t* __restrict__ QH, int8_t* __restrict__ SC, uint16_t* __restrict__ D) {
    const size_t nu = cols / 32, g = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= rows * nu) return;
    const size_t r = g / nu, u = g % nu, col = c0 + u * 32;
    const uint8_t* blk = blocks + (r * (src_cols / 256) + col / 256) * 210;
    const int i0 = (int) (col % 256);
    uint8_t ql[16] = {}, qh[8] = {};
    for (int i = 0; i < 32; ++i) {
        const int c = q6k_code(blk, i0 + i);
        if (i < 16) ql[i] |= (uint8_t) (c & 15);
        else ql[i - 16] |= (uint8_t) ((c & 15) << 4);
        const int w = i / 4, b = i % 4;
        qh[(w / 4) * 4 + b] |= (uint8_t) ((c >> 4) << (2 * (w % 4)));
    }
    for (int i = 0; i < 16; ++i) QL[g * 16 + i] = ql[i];
    for (int i = 0; i < 8; ++i) QH[g * 8 + i] = qh[i];
    SC[g * 2] = (int8_t) blk[192 + i0 / 16];
    SC[g * 2 + 1] = (int8_t) blk[192 + i0 / 16 + 1];
    D[g] = (uint16_t) (blk[208] | (blk[209] << 8));
}

// ---------------------------------------------------------------- synthetic weights
// value i of stream `seed`: a 64-bit mix of (seed, i) -> two uniforms -> Box-Muller (deterministic on a given GPU;
// the tests that compare with the CPU oracle read the generated bytes back rather than regenerate them)
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float synth_val(unsigned long long seed, unsigned long long i, float sigma) {
    const unsigned long long h = mix64(seed * 0x9E3779B97F4A7C15ULL + i + 1);
    const float u1 = ((float) (unsigned) (h >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (float) (unsigned) ((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    return sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}
__global__ void k_synth_normal(float* out, size_t n, float sigma, unsigned long long seed) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = synth_val(seed, i, sigma);
}
// a thread per Q8_0 block
__global__ void k_synth_q8_0(uint8_t* blocks, size_t nblocks, float sigma, unsigned long long seed) {
    const size_t b = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    float amax = 0.f;
    for (int l = 0; l < 32; ++l) amax = fmaxf(amax, fabsf(synth_val(seed, b * 32 + l, sigma)));
    const uint16_t hd = f2h(amax / 127.0f);
    const float d = h2f(hd);
    uint8_t* p = blocks + b * 34;
    p[0] = (uint8_t) hd;
    p[1] = (uint8_t) (hd >> 8);
    for (int l = 0; l < 32; ++l) {
        int q = d == 0.f ? 0 : (int) roundf(synth_val(seed, b * 32 + l, sigma) / d);
        p[2 + l] = (uint8_t) (int8_t) max(-127, min(127, q));
    }
}
// a thread per Q4_K super-block: sub-block scale (max - min) / 15 and offset -min, 6-bit codes against f16 d, dmin
__global__ void k_synth_q4k(uint8_t* blocks, size_t nblocks, float sigma, unsigned long long seed) {
    const size_t b = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    float scale[8], off[8], smax = 0.f, omax = 0.f;
    for (int s = 0; s < 8; ++s) {
        float mn = 0.f, mx = 0.f;
        for (int l = 0; l < 32; ++l) {
            const float v = synth_val(seed, b * 256 + s * 32 + l, sigma);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        scale[s] = (mx - mn) / 15.0f;
        off[s] = -mn;
        smax = fmaxf(smax, scale[s]);
        omax = fmaxf(omax, off[s]);
    }
    const uint16_t hd = f2h(smax / 63.0f), hm = f2h(omax / 63.0f);
    const float d = h2f(hd), dmin = h2f(hm);
    uint8_t* p = blocks + b * 144;
    p[0] = (uint8_t) hd, p[1] = (uint8_t) (hd >> 8), p[2] = (uint8_t) hm, p[3] = (uint8_t) (hm >> 8);
    int sc[8], m[8];
    for (int s = 0; s < 8; ++s) {
        sc[s] = d == 0.f ? 0 : min(63, (int) roundf(scale[s] / d));
        m[s] = dmin == 0.f ? 0 : min(63, (int) roundf(off[s] / dmin));
    }
    for (int j = 0; j < 4; ++j) {
        p[4 + j] = (uint8_t) ((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        p[8 + j] = (uint8_t) ((m[j] & 63) | ((m[j + 4] >> 4) << 6));
        p[12 + j] = (uint8_t) ((sc[j + 4] & 0xF) | ((m[j + 4] & 0xF) << 4));
    }
    for (int g = 0; g < 4; ++g) {
        const float ds0 = d * (float) sc[2 * g], dm0 = dmin * (float) m[2 * g];
        const float ds1 = d * (float) sc[2 * g + 1], dm1 = dmin * (float) m[2 * g + 1];
        for (int l = 0; l < 32; ++l) {
            const float v0 = synth_val(seed, b * 256 + (2 * g) * 32 + l, sigma);
            const float v1 = synth_val(seed, b * 256 + (2 * g + 1) * 32 + l, sigma);
            const int q0 = ds0 == 0.f ? 0 : max(0, min(15, (int) roundf((v0 + dm0) / ds0)));
            const int q1 = ds1 == 0.f ? 0 : max(0, min(15, (int) roundf((v1 + dm1) / ds1)));
            p[16 + 32 * g + l] = (uint8_t) (q0 | (q1 << 4));
        }
    }
}
// a thread per Q6_K super-block: 16-value sub-block scale amax / 31 against f16 d = max scale / 127
__global__ void k_synth_q6k(uint8_t* blocks, size_t nblocks, float sigma, unsigned long long seed) {
    const size_t b = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    float scale[16], smax = 0.f;
    for (int s = 0; s < 16; ++s) {
        float amax = 0.f;
        for (int l = 0; l < 16; ++l) amax = fmaxf(amax, fabsf(synth_val(seed, b * 256 + s * 16 + l, sigma)));
        scale[s] = amax / 31.0f;
        smax = fmaxf(smax, scale[s]);
    }
    const uint16_t hd = f2h(smax / 127.0f);
    const float d = h2f(hd);
    uint8_t* p = blocks + b * 210;
    for (int i = 0; i < 192; ++i) p[i] = 0;
    p[208] = (uint8_t) hd, p[209] = (uint8_t) (hd >> 8);
    int sc[16];
    for (int s = 0; s < 16; ++s) {
        sc[s] = d == 0.f ? 0 : min(127, (int) roundf(scale[s] / d));
        p[192 + s] = (uint8_t) (int8_t) sc[s];
    }
    for (int i = 0; i < 256; ++i) {
        const float ds = d * (float) sc[i / 16];
        const int q = ds == 0.f ? 32 : max(0, min(63, (int) roundf(synth_val(seed, b * 256 + i, sigma) / ds) + 32));
        const int half = i / 128, r = i % 128, l = r % 32, quad = r / 32;
        uint8_t* ql = p + 64 * half + ((quad & 1) ? l + 32 : l);
        *ql = (uint8_t) ((quad >= 2) ? (*ql | ((q & 0xF) << 4)) : (*ql | (q & 0xF)));
        p[128 + 32 * half + l] |= (uint8_t) ((q >> 4) << (2 * quad));
    }
}

// x[t][:] = table[ids[t]][:] (f16 rows -> f32): the window's input rows from a device-resident embedding table
__global__ void k_embed_rows(const uint16_t* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x, int n) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[(size_t) t * n + i] = h2f(table[(size_t) ids[t] * n + i]);
}

__global__ void k_math_probe(int op, const float* x, float* y, size_t n) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s, c;
    switch (op) {
        case 0: y[i] = ex_expf(x[i]); break;
        case 1: y[i] = ex_log1pf_pos(x[i]); break;
        case 2: y[i] = ex_sigmoid(x[i]); break;
        case 3: y[i] = ex_silu(x[i]); break;
        case 4: y[i] = ex_rsqrt(x[i]); break;
        case 5: ex_sincos((double) x[i], &s, &c); y[i] = s; break;
        case 6: ex_sincos((double) x[i], &s, &c); y[i] = c; break;
        default: y[i] = h2f(f2h(x[i])); break;
    }
}

}  // namespace fnxk

using namespace fnxk;

extern "C" {

const char* fnx_last_error(void) { return err_buf(); }
int fnx_built_arch(void) { return 100; }
unsigned fnx_device_fault(void) {
    unsigned v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, fnxk::g_fault, sizeof v) != cudaSuccess) return ~0u;
    if (v) cudaMemcpyToSymbol(fnxk::g_fault, &zero, sizeof zero);
    return v;
}

int fnx_quantize_q8_1(const float* x, void* q, int n, int rows, void* st) {
    FNX_REQUIRE(n > 0 && n % 32 == 0 && rows >= 0, "quantize_q8_1: n %d must be a positive multiple of 32", n);
    if (!rows) return 0;
    launch(0, k_quantize_q8_1, dim3((n / 32 + 7) / 8, rows), 256, 0, strm(st), x, (uint8_t*) q, n);
    return launch_ok("quantize_q8_1");
}

int fnx_rms_norm_rows(float* x, const float* add, const float* w, float* y, void* q, int rows, int n, float eps, void* st) {
    FNX_REQUIRE(n > 0 && n % 32 == 0, "rms_norm_rows: n %d must be a positive multiple of 32", n);
    if (rows <= 0) return 0;
    launch(0, k_rms_norm_rows, rows, 1024, 0, strm(st), x, add, w, y, (uint8_t*) q, n, eps);
    return launch_ok("rms_norm_rows");
}

int fnx_l2_prefetch(const void* p, size_t bytes, void* st) {
    if (!p || !bytes) return 0;
    const char* a = (const char*) (((uintptr_t) p + 15) & ~(uintptr_t) 15);   // the bulk prefetch wants 16-byte alignment
    const size_t skip = (size_t) (a - (const char*) p);
    if (bytes <= skip + 16) return 0;
    const size_t n = bytes - skip, chunks = (n + PF_CHUNK - 1) / PF_CHUNK;
    k_l2_prefetch<<<(unsigned) ((chunks + 63) / 64), 64, 0, strm(st)>>>(a, n);
    return launch_ok("l2_prefetch");
}

int fnx_copy_many(const FnxCopyJob* jobs, int n, void* st) {
    if (n <= 0) return 0;
    launch(0, k_copy_many, dim3(74, n), 256, 0, strm(st), jobs);
    return launch_ok("copy_many");
}

int fnx_repack_q8_0_split(const void* blocks, int8_t* q, uint16_t* d, size_t rows, size_t cols, void* st) {
    FNX_REQUIRE(cols % 32 == 0, "repack_q8_0_split: cols %zu not a multiple of 32", cols);
    const size_t nb = rows * (cols / 32);
    if (!nb) return 0;
    k_repack_q8_0<<<(unsigned) ((nb + 255) / 256), 256, 0, strm(st)>>>((const uint8_t*) blocks, q, d, nb);
    return launch_ok("repack_q8_0_split");
}

int fnx_repack_q6k_units(const void* blocks, size_t rows, size_t src_cols, size_t c0, size_t cols, void* QL, void* QH, void* SC,
                         void* D, void* st) {
    FNX_REQUIRE(src_cols % 256 == 0 && c0 % 32 == 0 && cols % 32 == 0 && c0 + cols <= src_cols,
                "repack_q6k_units: columns [%zu, %zu) of %zu", c0, c0 + cols, src_cols);
    const size_t n = rows * (cols / 32);
    if (!n) return 0;
    k_repack_q6k<<<(unsigned) ((n + 127) / 128), 128, 0, strm(st)>>>((const uint8_t*) blocks, rows, src_cols, c0, cols, (uint8_t*) QL,
                                                                  (uint8_t*) QH, (int8_t*) SC, (uint16_t*) D);
    return launch_ok("repack_q6k_units");
}

int fnx_synth_normal(float* out, size_t n, float sigma, unsigned long long seed, void* st) {
    if (!n) return 0;
    k_synth_normal<<<(unsigned) ((n + 255) / 256), 256, 0, strm(st)>>>(out, n, sigma, seed);
    return launch_ok("synth_normal");
}

int fnx_synth_quant(int type, void* blocks, size_t nvalues, float sigma, unsigned long long seed, void* st) {
    if (type == FNX_Q8_0) {
        FNX_REQUIRE(nvalues % 32 == 0, "synth_quant: %zu values not whole Q8_0 blocks", nvalues);
        const size_t nb = nvalues / 32;
        k_synth_q8_0<<<(unsigned) ((nb + 127) / 128), 128, 0, strm(st)>>>((uint8_t*) blocks, nb, sigma, seed);
    } else if (type == FNX_Q4_K || type == FNX_Q6_K) {
        FNX_REQUIRE(nvalues % 256 == 0, "synth_quant: %zu values not whole super-blocks", nvalues);
        const size_t nb = nvalues / 256;
        if (type == FNX_Q4_K) k_synth_q4k<<<(unsigned) ((nb + 63) / 64), 64, 0, strm(st)>>>((uint8_t*) blocks, nb, sigma, seed);
        else k_synth_q6k<<<(unsigned) ((nb + 63) / 64), 64, 0, strm(st)>>>((uint8_t*) blocks, nb, sigma, seed);
    } else {
        return fail("synth_quant: type %d is not Q4_K, Q6_K or Q8_0", type);
    }
    return launch_ok("synth_quant");
}

int fnx_embed_rows(const uint16_t* table, const int* ids, float* x, int T, int n, void* st) {
    if (T <= 0 || n <= 0) return 0;
    k_embed_rows<<<dim3((n + 255) / 256, T), 256, 0, strm(st)>>>(table, ids, x, n);
    return launch_ok("embed_rows");
}

int fnx_math_probe(int op, const float* x, float* y, size_t n, void* st) {
    if (!n) return 0;
    k_math_probe<<<(unsigned) ((n + 255) / 256), 256, 0, strm(st)>>>(op, x, y, n);
    return launch_ok("math_probe");
}
}
