/* sfnx_b200 - C ABI of the B200 (sm_100a) verify-window kernels.
 *
 * A drop-in for the host<->kernel boundary of johnfink8/sfnx (src/kernels.hpp, namespace fnx): the same launch
 * wrappers, with the model's shapes as run-time arguments instead of compile-time constants, plain pointers and
 * sizes, an int status instead of exceptions, and no C++ types in the signatures.
 *
 * Conventions (as the reference's, src/kernels.hpp:1-2 and 36-49):
 *  - every pointer is device memory unless its comment says "host"; `st` is a cudaStream_t; all launches are
 *    asynchronous on `st`, allocate nothing, read no device data on the host and may be captured into a CUDA graph
 *    (per-window values such as the position, the job count and the history parity live in device memory);
 *  - activations are f32 rows, one row per window row (or per routed pair); quantised activations are q8_1 rows
 *    (36-byte blocks of 32: f16 d, f16 sum, 32 int8);
 *  - the return value is 0, or non-zero after a refused argument or a failed launch, with the text in
 *    fnx_last_error() (the reference throws std::runtime_error with the same kind of text);
 *  - device-side faults never trap: kernels OR bits into a caller-supplied `unsigned* err` word
 *    (bit 1: a peer's addend never came; bit 8: a bounded on-chip wait ran out; bit 16: a non-finite logit; reference
 *    src/kernels.hpp:329-332) and run to completion.
 */
#ifndef SFNX_B200_H
#define SFNX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNX_MAXT 16   /* rows per window (reference src/model.hpp:45) */
#define FNX_TOPK_N 64 /* sampler candidates per row (reference src/kernels.hpp:392) */
#define FNX_HS 128    /* DeltaNet head size (reference src/model.hpp:42) */

/* one matrix (an expert's) applied to up to FNX_MAXT activation rows: reference src/kernels.hpp:18-23 (Job) */
typedef struct FnxJob {
    int w;             /* expert */
    int n;             /* rows of the job */
    int y[FNX_MAXT];   /* activation rows */
    int out[FNX_MAXT]; /* output rows */
} FnxJob;

/* the prompt path's expert jobs, up to FNX_PF_JOB rows of one expert: reference src/kernels.hpp:25-32 (PF_JOB, BigJob) */
#define FNX_PF_JOB 64
typedef struct FnxBigJob {
    int w;               /* expert */
    int n;               /* rows of the job */
    int y[FNX_PF_JOB];   /* activation rows */
    int out[FNX_PF_JOB]; /* output rows */
} FnxBigJob;

/* a Q8_0 matrix in the split layout: int8 values [rows][cols], f16 scales [rows][cols / 32]
 * (reference src/model.hpp:71-87, Q8S) */
typedef struct FnxQ8S {
    const int8_t* q;
    const uint16_t* d;
} FnxQ8S;

/* the routed experts' matrices of one projection (reference src/moe_w.cuh:2-9 MoeW, src/model.hpp DW):
 *  type FNX_Q4_K: GGUF Q4_K rows (144-byte super-blocks), expert e at a + e * stride bytes;
 *  type FNX_Q8_0: split layout, expert e's values at a + e * stride, its scales at b + e * stride_b;
 *  type FNX_Q6_K: Q6_K regrouped in 32-column units (fnx_repack_q6k_units): planes QL a (16 B a unit), QH b (8 B),
 *                 SC c (2 B), D d (f16), expert e at unit index e * stride */
enum { FNX_Q4_K = 12, FNX_Q6_K = 14, FNX_Q8_0 = 8 }; /* GGUF type numbers */
typedef struct FnxExperts {
    int type;
    int nrows, ncols;
    const void *a, *b, *c, *d;
    size_t stride, stride_b;
} FnxExperts;

/* the paged K/V pool of one layer on this GPU: reference src/kernels.hpp:160-165 (KvPages); pt null: local rows
 * are contiguous.
 * q8 (reference kv_q8, src/kernels.hpp:149-181): the rows are int8 in groups of 32 with an f16 scale a group
 * (d = max |x| / 127, q = round(x / d): src/kernels.cu:1561-1566).  kc / vc then point at bytes: local row r's int8
 * values start at byte pt[r / rows] * page * 2 + (r % rows) * nkv * hd and its scales at half pt[r / rows] * page +
 * rows * nkv * hd / 2 + (r % rows) * nkv * hd / 32 (a page's scales follow its rows: kvq_row, kvq_scale); without a
 * page table the cache is one such page of `cap` rows (cap must be given).  The scan in the reference's order of sums
 * and the append read and write them; the tensor-core scans take f16 rows only (fnx_attn_partial then runs the
 * exact-order scan). */
typedef struct FnxKvPages {
    const int* pt; /* device: logical page -> physical page */
    size_t page;   /* halves per page */
    int rows;      /* local rows per page */
    int cap;       /* local rows the cache holds when pt is null (0: unchecked); a row past it is not appended */
    int q8;        /* the rows are int8 with f16 group scales */
} FnxKvPages;

/* unscaled rotary: reference src/rope.hpp:22-27 (Rope, base only) */
typedef struct FnxRope {
    float base;
    int nrot;
} FnxRope;

/* device-to-device copy job: reference src/kernels.hpp:375-379 (CopyJob) */
typedef struct FnxCopyJob {
    void* dst;
    const void* src;
    size_t bytes;
} FnxCopyJob;

const char* fnx_last_error(void);
/* the compute capability the library was built for (100) and whether the current device matches it */
int fnx_built_arch(void);
/* reads and clears the library's own device-side fault word: 0, or bit 8 when a bounded on-chip wait of a tcgen05 kernel
 * (fnx_attn_partial, fnx_moe_gate_up_mma, fnx_moe_down_mma) ran out: the kernel then finished with what it had instead
 * of spinning (reference kernels report through err words the same way, src/kernels.hpp:329-332).  Inside
 * fnx_window_stage the same bit goes into the window's error word (FNX_BUF_ERR) instead. */
unsigned fnx_device_fault(void);

/* ---- activations */
/* reference src/kernels.hpp:36 quantize_q8_1 (src/kernels.cu:99-113): f32 rows of n -> q8_1 rows */
int fnx_quantize_q8_1(const float* x, void* q, int n, int rows, void* st);
/* reference src/kernels.hpp:359 rms_norm_rows (src/kernels.cu:2199-2206): y = x / sqrt(mean(x^2) + eps) * w.
 * With add: x += add first (the residual update of the previous half), written back to x.  With q: y also as
 * q8_1 rows (the reference's hc_read hands both forms to the layer, src/kernels.hpp:64-66) */
int fnx_rms_norm_rows(float* x, const float* add, const float* w, float* y, void* q, int rows, int n, float eps, void* st);

/* the window's input rows from an f16 embedding table in device memory: x[t] = table[ids[t]] (the reference embeds
 * on the host and uploads the rows, src/engine.cu:783-789; a B200 holds the table) */
int fnx_embed_rows(const uint16_t* table, const int* ids, float* x, int T, int n, void* st);

/* reference src/kernels.hpp:364 l2_prefetch (src/kernels.cu:2173-2193): asks for [p, p + bytes) to be brought into L2; returns
 * at once (nothing waits for the data), capture-safe.  The window uses it on its side stream to bring a projection's weights
 * in while a latency-bound kernel leaves HBM idle. */
int fnx_l2_prefetch(const void* p, size_t bytes, void* st);

/* ---- dense projections */
/* reference src/kernels.hpp:47 q8s_gemv (src/dense.cuh:24-160): out[t][r] = W[r] . y[t], T <= FNX_MAXT */
int fnx_q8s_gemv(FnxQ8S w, int rows, int cols, const void* y, float* out, int out_stride, int T, void* st);
/* The same product on the tcgen05 tensor cores (no counterpart in the reference): a 32-column block's integer dot of 128 weight
 * rows against the window's rows is one tcgen05.mma kind::i8 into tensor memory, the blocks' terms fl(dw da) (float) isum are
 * added in ascending block order - not the reference's order (16-column pieces on 32 interleaved lanes and a tree), so the
 * result equals fnx_q8s_gemv's to fp32 rounding of the sum, not bit for bit.  Shapes: cols a multiple of 256 up to 3072, at
 * least 64 tiles of 128 rows, planes 16-byte aligned; refused otherwise.  Capture-safe (the tensor maps are built on the host
 * at enqueue time and passed by value).  The window uses it for the head, qkvz and wq|wk|wv unless FNX_EXACT=1. */
int fnx_q8s_gemv_blocks(FnxQ8S w, int rows, int cols, const void* y, float* out, int out_stride, int T, void* st);
/* reference src/kernels.hpp:365-368 q8s_gemv_segs: n (1..3) Q8_0 matrices of `cols` columns over the same q8_1 rows in one
 * launch; each output as fnx_q8s_gemv of that matrix alone gives it */
int fnx_q8s_gemv_segs(const FnxQ8S* w, const int* rows, float* const* out, const int* out_stride, int n, int cols, const void* y, int T,
                      void* st);
/* reference src/kernels.hpp:369-372 q8s_gemv_f32: fnx_q8s_gemv(w, rows, cols, y, out, rows) and fnx_gemv_f32(W, x, yf, rf, cols)
 * behind one call, the same values (two launches in stream order here) */
int fnx_q8s_gemv_f32(FnxQ8S w, int rows, int cols, const void* y, float* out, const float* W, const float* x, float* yf, int rf, int T,
                     void* st);
/* reference src/kernels.hpp:49 gemv_f32 (src/kernels.cu:184-227, the block-per-row form): y[t][r] = W[r] . x[t] */
int fnx_gemv_f32(const float* W, const float* x, float* y, int rows, int n, int T, void* st);

/* ---- routed experts */
/* reference src/kernels.hpp:276-278 router_route (src/moe.cuh:73-202): logits [T][nexp + 1] = W . x, top-k per row
 * by logit (ties: lower index), weights = softmax over the picks, one job per distinct expert numbered by first
 * pick; njobs[0] = the count.  scratch: fnx_router_scratch_bytes() bytes, zeroed once */
size_t fnx_router_scratch_bytes(void);
int fnx_router_route(const float* W, const float* x, float* logits, int T, int n, int nexp, int topk, int* topi, float* topw,
                     FnxJob* jobs_gu, FnxJob* jobs_dn, int* njobs, void* scratch, void* st);
/* reference src/kernels.hpp:281-282 moe_gate_up (src/moe_q4k.cuh:91-154; src/moe.cuh:258-272): gu[out][2 ffs] =
 * [gate | up] rows of each job's expert over its q8_1 rows of xq (rows of A.ncols) */
int fnx_moe_gate_up(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const void* xq, float* gu, void* st);
/* reference src/kernels.hpp:43-45 mmvq (src/kernels.cu:935-968): out[jobs[j].out[s]][r] = W[jobs[j].w][r] . y[jobs[j].y[s]] over
 * q8_1 rows y; Q4_K and split-Q8_0 matrices, with fnx_moe_gate_up's arithmetic (the reference's other types run through
 * ggml's dot products); out_stride = W->nrows */
int fnx_mmvq(const FnxExperts* W, const FnxJob* jobs, const int* njobs, int njobs_max, const void* y, float* out, int out_stride, void* st);
/* reference src/kernels.hpp:305 moe_down (src/moe.cuh:284-345): part[out][n] from h = silu(gate) * up of the gu rows.
 * hq: fnx_moe_h_bytes(pairs, ffs) bytes of scratch for the pairs' quantised h (the reference keeps it in a
 * __device__ global, src/moe.cuh:281) */
size_t fnx_moe_h_bytes(int pairs, int ffs);
int fnx_moe_down(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const float* gu, int npairs, void* hq,
                 float* part, void* st);
/* No counterpart in the reference.  fnx_moe_down for callers that cannot allocate device memory (a plug-in inside another
 * engine's stream, a host whose memory was all handed out at start-up): the scratch for the pairs' quantised h is an
 * array inside the library, FNX_DOWN_NOALLOC_BYTES on every GPU that loads it, so the caller passes only inputs and
 * outputs and the call allocates nothing.  Refused (non-zero, text in fnx_last_error) when fnx_moe_h_bytes(npairs,
 * A->ncols) exceeds the array.  The first call on a device looks the array's address up (once per device, with that
 * device current): make that first call before any stream capture.  All calls share the one array and it keeps the last
 * call's contents; each call writes what it reads, so nothing is cleared, but two calls that overlap on the GPU (two
 * streams, two threads) race on it: keep them in stream order. */
#define FNX_DOWN_NOALLOC_BYTES (288 * 1024) /* 256 pairs x ff 1024: 256 KiB of int8 h + 32 KiB of scales */
int fnx_moe_down_noalloc(const FnxExperts* A, const FnxJob* jobs, const int* njobs, int njobs_max, const float* gu, int npairs,
                         float* part, void* st);
/* ---- routed experts over many rows, on the tensor cores (the reference's prompt path)
 * reference src/kernels.hpp:289-292 moe_gate_up_mma, swiglu_h16, moe_down_mma (src/moe_mma.cu:28-59, src/moe_mma.cuh:63-388):
 * out[jobs[j].out[s]][r] = sum_k f16(W_e[r][k]) * x[jobs[j].y[s]][k] for every job j < *njobs (device) and row s of it; every
 * weight dequantised to f16 with one rounding (Q4_K: q * f16(d sc) - f16(dmin m) as one half fma; Q8_0: q * d; Q6_K in
 * 32-column units: (q - 32) * f16(d sc)), x rows of A->ncols f16 values, fp32 sums on tcgen05 tensor cores (the order
 * of a sum's terms is the hardware's).  A->ncols in units of 32.  njobs_cap: the most jobs there can be (grid rows). */
int fnx_moe_gate_up_mma(const FnxExperts* A, const FnxBigJob* jobs, const int* njobs, int njobs_cap, const uint16_t* xh, float* gu,
                        void* st);
/* h16[p][i] = f16(silu(gu[p][i]) * gu[p][ffs + i]) for P rows of [gate | up] */
int fnx_swiglu_h16(const float* gu, int ffs, int P, uint16_t* h16, void* st);
int fnx_moe_down_mma(const FnxExperts* A, const FnxBigJob* jobs, const int* njobs, int njobs_cap, const uint16_t* h16, float* part,
                     void* st);
/* reference src/kernels.hpp:307 swiglu_stacked_q8_1 + src/dense.cuh:162-198 (the shared expert): T rows of
 * [gate | up] -> h as int8 + f16-rounded scales, then the Q8_0 down into out[t][n] */
int fnx_shared_expert(FnxQ8S gate_up, FnxQ8S down, const void* xq, int T, int n, int ffs, float* sh_gu, void* hq, float* out,
                      void* st);
/* reference src/kernels.hpp:77 moe_combine / 308-313 RingMoe (src/kernels.cu:797-803): out[t] = sum_k topw[t][k]
 * part[t topk + k] + sigmoid(logits[t][nexp]) sh[t] */
int fnx_moe_combine(const float* part, const float* topw, const float* sh, const float* logits, int nexp, float* out, int T,
                    int n, int topk, void* st);

/* ---- Gated DeltaNet */
/* reference src/kernels.hpp:90-93 gdn_scratch_floats, gdn_core (src/gdn_core.cuh:17-229).  scratch zeroed once. */
size_t fnx_gdn_scratch_floats(int nv);
int fnx_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a,
                 const float* nw, float* S, void* yq, const int* ctl, float* scratch, float* snap, float* hsnap, int nk, int nv,
                 const int* vmap, int T, float eps, void* st, float* y32);
/* The same window without checkpoints (no counterpart in the reference, whose rollback copies a checkpoint back,
 * src/engine_common.cu:525-568): S is read and left as it is; each row's decay, key and delta go into `log`
 * (fnx_gdn_log_floats(nk, nv) floats, this layer's and sequence's own), and fnx_gdn_replay then sets S to the state after the
 * first n rows - S <- g_t S + k_t (x) delta_t for t < n, the window's own operations, so the bits are those the
 * checkpoints would hold - for n = T as well: a logged window's state advances only through the replay.  yq, hist and hsnap
 * as fnx_gdn_core's.  A window moves 3 state-sized transfers instead of 17. */
size_t fnx_gdn_log_floats(int nk, int nv);
int fnx_gdn_core_log(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a, const float* nw,
                     const float* S, void* yq, const int* ctl, float* scratch, float* log, float* hsnap, int nk, int nv, const int* vmap, int T, float eps,
                     void* st);
typedef struct FnxGdnReplay {
    float* S;        /* [nv][128][128], advanced in place */
    const float* log;
    const int* vmap; /* as fnx_gdn_core's */
    int nk, nv;
    int row0, n;     /* the log's rows row0 .. row0 + n - 1 */
} FnxGdnReplay;
/* jobs: device array; a block per (value head < nv_max, job) */
int fnx_gdn_replay(const FnxGdnReplay* jobs, int njobs, int nv_max, void* st);
/* reference src/kernels.hpp:94-111 GdnLanes, gdn_core_lanes, gdn_core_segs: several sequences ("lanes") in one launch.
 * Device arrays give segment s's state, conv history (this layer's) and ctl; its rows are window rows row0[s] ..
 * row0[s] + T - 1 of qkvz, ab and yq, and its snapshots (snap, hsnap as fnx_gdn_core's) are written from window row
 * row0[s] on.  Each segment's rows chain through its lane's state exactly as a window of T rows on that lane alone.
 * fnx_gdn_core_lanes: T rows, one lane each (row0 null, no snapshots). */
typedef struct FnxGdnLanes {
    float* const* S;
    float* const* hist;
    const int* const* ctl;
    const int* row0;
    float* snap;
    float* hsnap;
} FnxGdnLanes;
int fnx_gdn_core_segs(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                      float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int nseg, int T, float eps, void* st);
int fnx_gdn_core_lanes(const float* qkvz, const float* ab, const float* convw, const float* dt, const float* a, const float* nw, void* yq,
                       float* scratch, int nk, int nv, const int* vmap, const FnxGdnLanes* gl, int T, float eps, void* st);
/* reference src/kernels.hpp:380 copy_many (src/kernels.cu:1473-1485): the rollback's batched copies */
int fnx_copy_many(const FnxCopyJob* jobs, int n, void* st);

/* ---- attention */
/* reference src/kernels.hpp:262 kv_rows_per_card */
int fnx_kv_rows_per_card(int n_ctx, int ncard);
/* reference src/kernels.hpp:251-252 attn_prep_append (src/kernels.cu:1539-1569) */
int fnx_attn_prep_append(float* qg, float* k, const float* v, const float* q_norm, const float* k_norm, uint16_t* kc, uint16_t* vc,
                         FnxKvPages g, int card, int ncard, int T, const int* pos0, float eps, FnxRope rope, int nq, int nkv,
                         int hd, void* st);
/* reference src/kernels.hpp:125 attn_scratch_floats, 230-236 attn / attn_part_lanes / attn_finish
 * (src/kernels.cu:497-691).  fnx_attn_partial leaves this GPU's partial per (row, head) in part
 * [T][nq][hd + 2] (acc, m, z); fnx_attn_finish merges nparts partials (this GPU's and the peers', gathered by the
 * caller, parts[p] at parts + p * T * nq * (hd + 2)) in ring order for heads [h0, h0 + nh) and applies the gate:
 * out [T][nh][hd] */
size_t fnx_attn_scratch_floats(int nq, int hd, int T);
/* halves of one layer's K (or V) rows when they are int8: reference src/kernels.hpp:152-155 kvp_rows_halves */
size_t fnx_kvq_halves(int rows, int nkv, int hd);
/* the fast scan (all rows of the window in one pass over the K/V rows, tensor cores, sums in its own order: equal to
 * the exact-order scan to f32 rounding) and the scan in the reference's order of sums (bit-reproducible, slower) */
int fnx_attn_partial(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard, int T,
                     const int* pos0, int nq, int nkv, int hd, float* scratch, void* st);
int fnx_attn_partial_exact(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, float* part, int card, int ncard,
                           int T, const int* pos0, int nq, int nkv, int hd, float* scratch, void* st);
/* reference src/kernels.hpp:182-193 LaneRows, :232-235 attn_part_lanes (src/kernels.cu:1262-1281): the partials of a
 * batched window's T rows, each of a lane (sequence) of its own: row t at position *pos[t] on the page table pt[t] (device
 * arrays of device pointers; pt null: g's table for every row).  The reference's order of sums, as
 * fnx_attn_partial_exact; merged by fnx_attn_finish as any other partials. */
typedef struct FnxLaneRows {
    const int* const* pos;
    const int* const* pt;
} FnxLaneRows;
int fnx_attn_part_lanes(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, FnxLaneRows lr, float* part, int card, int ncard,
                        int T, int nq, int nkv, int hd, float* scratch, void* st);
/* the same scan for rows with a selection of positions (reference src/kernels.cu:504-505, 525: attn / attn_part_lanes with
 * cells, n_cells): row t with n_cells[t] >= 0 attends the n_cells[t] local rows cells[t * maxsel ...] in that order, a row
 * with n_cells[t] = -1 every owned position up to its own.  lr empty (both null): one sequence at *pos0 + t */
int fnx_attn_partial_cells(const float* qg, const uint16_t* kc, const uint16_t* vc, FnxKvPages g, FnxLaneRows lr, float* part, int card,
                           int ncard, int T, const int* pos0, int nq, int nkv, int hd, float* scratch, const int* cells, const int* n_cells,
                           int maxsel, void* st);
int fnx_attn_splits(int nkv);
int fnx_attn_finish(const float* parts, int nparts, int first_part, const float* qg, float* out, int T, int nq, int h0, int nh,
                    int hd, void* st);

/* ---- the attention layers' block selection (reference src/qsa.cuh; src/kernels.hpp:195-217 qsa_maxsel, qsa_rows, qsa_index,
 * qsa_select, qsa_select_lanes, qsa).  Keys of FNX_QSA_DIM, FNX_QSA_HEADS query heads, blocks of FNX_QSA_POOL positions,
 * the first 64 dimensions rotated; `top` (the reference's 2048 / 4 = 512) is how many blocks a row keeps.
 *   y       [T][fnx_qsa_rows()]  the projection: 4 query heads, then the raw key (fnx_qsa_proj: bf16 weights wq [512][n],
 *                                wk [128][n] as bit patterns, x [T][n] f32)
 *   ring    [ring_rows][128] f16 the raw keys of the last positions (position p at row p % ring_rows; ring_rows >= T + 4)
 *   pooled  f16 rows of 128      block b's key at b * 128, or with a page table at pt[b / bpp] * page + (b % bpp) * 128,
 *                                bpp = g.rows / 4 * ncard (a page holds every GPU's blocks; every GPU holds all keys)
 *   q       [T][4][128]          the normed, rotated query heads (fnx_qsa_index writes q, ring and pooled)
 *   scores  [T][max_pools], cells [T][fnx_qsa_maxsel(top)], n_cells [T] (-1: the row keeps every block)
 * fnx_qsa runs the three in order (wq null: y already holds the projection), as the reference's qsa(). */
#define FNX_QSA_DIM 128
#define FNX_QSA_HEADS 4
#define FNX_QSA_POOL 4
int fnx_qsa_rows(void);
int fnx_qsa_maxsel(int top);
int fnx_qsa_proj(const uint16_t* wq, const uint16_t* wk, const float* x, float* y, int T, int n, void* st);
int fnx_qsa_index(const float* y, const float* qn, const float* kn, uint16_t* ring, int ring_rows, uint16_t* pooled, FnxKvPages g, int ncard,
                  float* q, const int* pos0, int T, float eps, FnxRope rope, void* st);
int fnx_qsa_select(const float* q, const uint16_t* pooled, FnxKvPages g, FnxLaneRows lr, float* scores, int* cells, int* n_cells, int max_pools,
                   const int* pos0, int T, int card, int ncard, int top, void* st);
int fnx_qsa(const uint16_t* wq, const uint16_t* wk, const float* x, int n, float* y, const float* qn, const float* kn, uint16_t* ring,
            int ring_rows, uint16_t* pooled, FnxKvPages g, float* q, float* scores, int* cells, int* n_cells, int max_pools, const int* pos0,
            int T, float eps, FnxRope rope, int card, int ncard, int top, void* st);

/* ---- hyper-connections of the residual streams (R: [T][hc][n], hc streams of width n)
 * reference src/kernels.hpp:356 hc_write (src/kernels.cu:1493-1503): R[t][c] += bo[t] * 2 sigmoid(inj[t][c] / hc) */
int fnx_hc_write(float* R, const float* bo, const float* inj, int T, int n, int hc, void* st);
/* reference src/kernels.hpp:51-66 hc_read / hc_scratch_floats (src/hc.cuh k_hc): the read with the previous half's write
 * folded in when bo_prev is not null (R' = R + bo_prev * 2 sigmoid(inj_prev / hc), R <- R'):
 *   mixed[t] = mean over the streams of xn_c * sigmoid(w_up_c . lo),  lo = silu(w_down . xn / hc) as int8 per 32,
 *   xn = R' w_norm rs (rs the stream's RMS factor), inject[t][c] = w_inj[c] . xn when w_inj (bf16 [hc][hc n]) is given;
 *   mixed also as q8_1 rows into q8 when not null.  w_down: split Q8_0 [lr][hc n]; w_up: split Q8_0 [hc n][lr].
 * The reference's single launch holds two grid-wide spin barriers (every block resident, nothing else on the GPU,
 * err bit 4 on a timeout); here the read is three launches in stream order, so it has no barrier, takes no err word
 * and may run beside other streams' work.  scratch: fnx_hc_scratch_floats floats, never read before written. */
size_t fnx_hc_scratch_floats(int T, int n, int hc, int lr);
/* R[t][c] = x[t] for every stream c: a window's first residual (the reference's host fills the streams with the embedding
 * row before it uploads them, src/engine.cu:782-789 embed_into) */
int fnx_hc_expand(const float* x, float* R, int T, int n, int hc, void* st);
/* reference src/kernels.hpp add_streams (src/kernels.cu:2207-2222): R[t][c] = h[t][c] + e[t] */
int fnx_hc_add_streams(const float* h, const float* e, float* R, int T, int n, int hc, void* st);
int fnx_hc_read(float* R, const float* bo_prev, const float* inj_prev, const float* w_norm, FnxQ8S w_down, FnxQ8S w_up, const uint16_t* w_inj,
                float eps, float* mixed, float* inject, float* scratch, void* q8, int T, int n, int hc, int lr, void* st);

/* ---- sum across GPUs */
/* all-reduce(sum) of x[rows][row_len] in the reference ring's order, chunk c = float pairs [c NP / n, (c + 1) NP / n) of
 * every row (NP = row_len / 2) summed as ((x_c + x_{c+1}) + ...) + x_{c+n-1} (reference src/kernels.hpp:321-353 ring_sum / Ring, src/kernels.cu:755-868
 * k_ring, fp32 payload), over memory the GPUs of one box can read and write directly:
 *   slot[p][r]  GPU r's slot of parity p (rows * row_len floats), as addressed from this GPU
 *   pad[r]      GPU r's flag words (nrank of them, zeroed once), as addressed from this GPU
 *   state       three words of this GPU's own memory, zeroed once
 *   spin_limit  polls a wait may take before it gives up and sets bit 1 of *err
 *   ll[p][r]    GPU r's receive area of parity p, as addressed from this GPU: nrank runs of ll_count 8-byte words, run s
 *               written by GPU s (zeroed once).  The window's own exchanges (fnx_boundary_rows, fnx_attn_finish_ring,
 *               fnx_ring_gather) push every value to the peers as one 8-byte store {value bits, exchange number}, as the
 *               reference's ring stores its LL words (src/kernels.cu:755-868): a reader polls its own memory until the
 *               number is the current one, so an exchange costs one one-way trip and needs no flags or fences.
 * x is summed in place; every GPU gets the same bits.  Capture-safe; nrank == 1 does nothing. */
enum { FNX_RING_MAX = 8 };
typedef struct FnxRing {
    int nrank, rank;
    float* slot[2][FNX_RING_MAX];
    unsigned* pad[FNX_RING_MAX];
    unsigned* state;
    unsigned spin_limit;
    unsigned long long* ll[2][FNX_RING_MAX];
    size_t ll_count;
} FnxRing;
int fnx_ring_sum(float* x, int rows, int row_len, const FnxRing* ring, unsigned* err, void* st);
/* A small all-gather over the ring's receive areas (one more exchange in the GPUs' common order): every GPU's
 * na + nb 4-byte words (na + nb <= ll_count) to all_a [nrank][na] and all_b [nrank][nb] on every GPU.  The window's
 * caller uses it where the plan says FNX_AFTER_GATHER_BEST: the per-GPU argmax (value, index), the 64 candidates a row.
 * No counterpart in the reference, whose host reads every card's values itself (src/engine_common.cu:781-787). */
int fnx_ring_gather(const void* a, int na, const void* b, int nb, const FnxRing* ring, void* all_a, void* all_b, unsigned* err, void* st);
/* The attention layer's merge across GPUs, the gate and the q8_1 rows for the output projection in one launch (reference
 * src/kernels.cu:609-672 k_att_merge over its ring, :621-672 the gate; src/kernels.hpp:230-236 attn): this GPU's partials
 * part [T][nq][hd + 2] go to the peers' receive areas, each peer the heads it owns (ll_count >= T * nq / nrank * (hd + 2)),
 * the peers' arrive in this GPU's (bounded wait: bit 1 of *err), and the heads this GPU owns
 * ([rank * nq / nrank, + nq / nrank)) are merged in ring order ending with this GPU.  out [T][nq / nrank][hd] and / or q8
 * (q8_1 rows of nq / nrank * hd values) may be null.  ring null: one GPU.  One more exchange in the GPUs' common order
 * (the ring's state counts them). */
int fnx_attn_finish_ring(const float* part, const FnxRing* ring, const float* qg, float* out, void* q8, int T, int nq, int hd, unsigned* err,
                         void* st);


/* What lies between two halves of a layer, in one launch (the reference folds the same steps into its ring: src/kernels.hpp:
 * 308-313 RingMoe, src/kernels.cu:797-806 ring_x; the norm is its hc_read's): the ended half's addend - bo[T][n], or the
 * routed experts' rows weighted and added with the gated shared expert as fnx_moe_combine does (moe), or none (both null:
 * a window's first half) - summed across the GPUs in fnx_ring_sum's order (ring with nrank > 1, over its receive areas:
 * ll_count >= T * n), x += sum, then y = RMS norm of the new x with weight w (y may be null) and its q8_1 rows q (may be
 * null), all as the separate entry points give them, bit for bit. */
typedef struct FnxMoeRows {
    const float *part, *topw, *sh, *logits; /* [T topk][n], [T][topk], [T][n], router logits [T][nexp + 1] */
    int nexp, topk;
} FnxMoeRows;
int fnx_boundary_rows(float* x, const float* bo, const FnxMoeRows* moe, const FnxRing* ring, const float* w, float* y, void* q, int T, int n,
                      float eps, unsigned* err, void* st);

/* ---- head */
/* reference src/kernels.hpp:384 argmax (src/kernels.cu:870-908): per row the largest logit and its index + v0, the lowest
 * index on a tie; a non-finite logit sets bit 16 of *err.  keys: 2 * FNX_MAXT 64-bit words, zeroed once (left at zero) */
int fnx_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i, unsigned long long* keys, unsigned* err,
               void* st);
/* reference src/kernels.hpp:387 penalize_row (src/kernels.cu:1454-1470) */
int fnx_penalize_row(float* row, int n, const int* pen, const float* par, void* st);
/* reference src/kernels.hpp:393-394 top_tokens (src/topk.cuh:17-138) */
int fnx_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n, int pen_stride,
                   const float* pen_par, float* out_v, int* out_i, unsigned* err, void* st);

/* ---- the window: every GPU's work for one verify window of T rows over a stack of layers, in stream order.
 * The counterpart of the reference's Engine::enqueue / ffn_half / attention (src/engine.cu:900-1054), without the
 * hyper-connection, QSA and n-gram blocks: each layer is (RMS norm -> DeltaNet or attention mixer -> sum across GPUs ->
 * residual) then (RMS norm -> routed + shared experts -> sum across GPUs -> residual); then the head.  The caller owns
 * all memory: weights and states through FnxLayer, everything a window writes through one workspace. */
typedef struct FnxStackCfg {
    int n, nexp, topk, ff; /* hidden width, experts, picks per row, this GPU's FF slice */
    int nk, nv;            /* this GPU's DeltaNet key and value heads */
    int nq, nkv, hd, nrot; /* attention: query heads, KV heads, head dim, rotary width */
    int vocab0, vocab_rows; /* this GPU's vocabulary slice [vocab0, vocab0 + vocab_rows) */
    int nlayers, ncard, card;
    float eps, rope_base;
    int hc, hc_lr; /* residual streams (0 or 1: one stream, plain residual + RMS norm) and the hyper-connections' low rank */
    int r_preset;  /* hc > 1: the streams are in place before stage 0 (fnx_draft_begin made them), not expanded from x */
    /* the attention layers' block selection (0: none): blocks a row keeps, rows of a layer's raw-key ring, blocks a layer's
     * pooled keys hold.  With a selection the attention runs the exact-order scan over each row's cells */
    int qsa_top, qsa_ring_rows, qsa_max_pools;
} FnxStackCfg;

/* one hyper-connection read's weights (reference LayerW hc_norm / hc_down / hc_up / hc_inj, src/model.hpp:120-124):
 * norm [hc n], down split Q8_0 [lr][hc n], up split Q8_0 [hc n][lr], inj bf16 [hc][hc n] or null (the head's mixer) */
typedef struct FnxHcW {
    const float* norm;
    FnxQ8S down, up;
    const uint16_t* inj;
} FnxHcW;

/* an attention layer's indexer (reference LayerW idx_wq / idx_wk / idx_qn / idx_kn, src/engine.cu:911-912) with the
 * sequence's raw-key ring and pooled keys of that layer; wq null: the layer selects nothing */
typedef struct FnxQsaW {
    const uint16_t *wq, *wk; /* bf16 [512][n], [128][n] */
    const float *qn, *kn;    /* [128] each */
    uint16_t *ring, *pooled; /* f16 [qsa_ring_rows][128], [qsa_max_pools][128] (or paged by the layer's page tables) */
    size_t page;             /* paged: halves a page of the pooled keys' pool takes (0: the K/V pages' own pitch, the keys
                              * lying inside the K/V pages as in the reference's pool) */
} FnxQsaW;

typedef struct FnxLayer {
    int kind; /* 0: Gated DeltaNet, 1: attention */
    const float *norm1, *norm2;
    /* DeltaNet (reference LayerW: attn_qkv + attn_gate as qkvz, ssm_alpha/beta as ab, ssm_conv1d, ssm_dt.bias, ssm_a,
     * ssm_norm, ssm_out; src/model.cpp:759-836) and its per-sequence state */
    FnxQ8S qkvz;
    const float* ab;
    const float *conv, *dt, *a, *ssm_norm;
    FnxQ8S ssm_out;
    const int* vmap;
    float *S, *hist, *snap, *hsnap;
    /* attention (attn_q, attn_k, attn_v, attn_output, attn_q_norm, attn_k_norm) and its K/V cache */
    FnxQ8S wq, wk, wv, wo;
    const float *q_norm, *k_norm;
    uint16_t *kc, *vc;
    FnxKvPages pages;
    /* FFN (ffn_gate_inp + ffn_gate_inp_shexp as router rows, ffn_gate_exps | ffn_up_exps stacked, ffn_down_exps,
     * ffn_{gate,up,down}_shexp) */
    const float* router;
    FnxExperts gate_up, down;
    FnxQ8S sh_gate_up, sh_down;
    /* DeltaNet: this sequence's replay log (fnx_gdn_log_floats), or null.  With a log the window runs fnx_gdn_core_log (snap
     * is not used) and fnx_window_commit replays the kept rows into S, also when every row is kept; without one it runs
     * fnx_gdn_core and the commit copies a checkpoint back. */
    float* gdn_log;
    /* with cfg.hc > 1: the reads before the mixer half [0] and before the FFN half [1] (norm1 / norm2 are then unused) */
    FnxHcW hcw[2];
    FnxQsaW idx;
} FnxLayer;

typedef struct FnxHead {
    const float* norm;
    FnxQ8S out;
    FnxHcW mix; /* with cfg.hc > 1: the final mixer (no inject rows) instead of norm */
} FnxHead;

/* The draft (MTP) layer: one attention layer with hyper-connections, its FFN, a final mixer and a head over a draft
 * vocabulary, fed by a window's residual streams and the next tokens' embeddings (reference MtpCard, src/model.hpp:207-218;
 * Engine::mtp_enqueue, src/engine.cu:1275-1313).  It runs as a one-layer stack (cfg with kinds = {attention}, hc > 1,
 * r_preset = 1, vocab rows = this GPU's draft-vocabulary rows) whose streams fnx_draft_begin makes first:
 *   R[t][c] = fc_hid . rms(src[t] over all streams, norm_hid)[c] + fc_emb . rms(emb[t], norm_emb)
 * src [T][hc n] (rows of a window's streams), emb [T][n]; then fnx_window_stage for stages 0 .. as for any stack. */
typedef struct FnxDraft {
    const float *norm_emb, *norm_hid; /* [n], [hc n] */
    FnxQ8S fc_emb, fc_hid;            /* [n][n] each */
} FnxDraft;
int fnx_draft_begin(const FnxStackCfg* cfg, const FnxDraft* d, void* ws, const float* src, const float* emb, int T, void* st);

/* what the caller must do across GPUs after a stage (nothing when ncard is 1) */
enum { FNX_AFTER_NONE = 0, FNX_AFTER_SUM_BO = 1, FNX_AFTER_GATHER_PARTIALS = 2, FNX_AFTER_GATHER_BEST = 3 };
/* workspace buffers a caller reads or writes */
enum { FNX_BUF_X = 0, FNX_BUF_BO = 1, FNX_BUF_PARTIALS = 2, FNX_BUF_BEST_V = 3, FNX_BUF_BEST_I = 4, FNX_BUF_ERR = 5, FNX_BUF_CTL = 6,
       FNX_BUF_LOGITS = 7, FNX_BUF_COPY_JOBS = 8, FNX_BUF_NJOBS = 9,
       FNX_BUF_STREAMS = 10 /* hc > 1: the residual streams [T][hc n] as the window left them (a draft layer's source rows) */ };

size_t fnx_window_workspace_bytes(const FnxStackCfg* cfg);
/* zeroes the counters the kernels expect at zero (once, before the first window) */
int fnx_window_init(const FnxStackCfg* cfg, void* ws, void* st);
/* the stages of a window over these layers: returns their number and fills after[i] (up to max) */
int fnx_window_plan(const FnxStackCfg* cfg, const FnxLayer* layers, int* after, int max);
/* enqueues stage `stage` of a window of T rows: the input rows are in FNX_BUF_X (f32 [T][n]), the position and the
 * window tag in FNX_BUF_CTL (int [2]); capture-safe */
int fnx_window_stage(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, int T, int stage, void* st);
void* fnx_window_buf(const FnxStackCfg* cfg, void* ws, int which);
/* keep the first n of the last window's T rows (reference Engine::commit, src/engine_common.cu:525-568): per DeltaNet
 * layer S <- snap[n-1] and the written history half <- hsnap[n-1]; tag is the window's tag (its parity names the
 * half).  host_jobs: pinned host memory for nlayers * (2 FnxCopyJob + 1 FnxGdnReplay), copied into the workspace */
int fnx_window_commit(const FnxStackCfg* cfg, const FnxLayer* layers, void* ws, int T, int n, int tag, void* host_jobs, void* st);

/* a second stream for work that does not depend on its neighbours (the shared expert beside the routed experts, the
 * alpha/beta projection beside qkvz; the reference's st2, src/engine.cu:939-946), with the two events (cudaEvent_t) the
 * forks and joins record; set per host thread, null to stay on one stream.  Capture-safe. */
int fnx_window_side_stream(void* st2, void* ev_fork, void* ev_join);
/* the peer-memory ring (FnxRing, slots of FNX_MAXT * n floats) of the calling thread's windows, null for none.  With a
 * ring - and always on one GPU - a stage begins with fnx_boundary_rows, which sums the ended half's addends across the GPUs
 * itself, and fnx_window_plan asks for no FNX_AFTER_SUM_BO; without one the caller sums FNX_BUF_BO between the stages (any
 * all-reduce).  Set it before fnx_window_plan and before the stages are enqueued. */
int fnx_window_ring(const FnxRing* ring);

/* A window of several sequences ("lanes"; reference src/engine.cu:1137-1216 enqueue_rows / src/engine_common.cu:1136-1195
 * commit_rows): nseg lanes x `rows` window rows each, at most FNX_MAXT rows in all; lane s's rows are window rows
 * s rows .. s rows + rows - 1.  Everything shared (norms, projections, router, experts, head) runs over all rows as in a
 * window of one sequence; the DeltaNet core chains each lane's rows through that lane's state (fnx_gdn_core_segs), the K/V
 * rows are appended lane by lane and every row's attention partial is taken on its lane's position and pages
 * (fnx_attn_part_lanes, the reference's order of sums).  With block selection (cfg.qsa_top > 0) the projection runs over
 * all rows, every lane's rows are indexed on that lane's ring and pages, and the scores, the selection and the scan over
 * the cells take every row on its lane's position and pages (reference src/engine.cu:1186-1200).  Each lane's results are
 * those of a window of its rows alone.
 * The layers' S / hist fields are not used; kc / vc are the layer's paged pool. */
typedef struct FnxWindowLanes {
    int nseg, rows;
    const int* const* ctl;      /* device [nseg]: lane s's (position of its first row, tag) words */
    const int* row0;            /* device [nseg]: s * rows */
    const int* const* row_pos;  /* device [nseg * rows]: row t's position word */
    const int* const* row_pt;   /* device [nseg * rows]: row t's lane's page table */
    const int* const* ctl_host; /* host [nseg]: the same device pointers as ctl */
    const int* const* pt_host;  /* host [nseg]: the lanes' page tables (device pointers) */
    float* const* const* S;     /* host [nlayers]: device array [nseg] of the lanes' states (DeltaNet layers) */
    float* const* const* hist;  /* host [nlayers]: device array [nseg] of the lanes' conv histories */
    float* const* const* S_host;    /* host [nlayers] of host arrays [nseg]: the same pointers, for the commit */
    float* const* const* hist_host;
    uint16_t* const* const* idx_ring_host; /* host [nlayers] of host arrays [nseg]: the lanes' raw-key rings of the attention
                                            * layers with an indexer (null without block selection) */
} FnxWindowLanes;
int fnx_window_stage_lanes(const FnxStackCfg* cfg, const FnxLayer* layers, const FnxHead* head, void* ws, const FnxWindowLanes* lanes, int stage,
                           void* st);
/* keeps the first n[s] rows of lane s (tags[s]: the lane's window tag, whose low bit says which history half was read) */
int fnx_window_commit_lanes(const FnxStackCfg* cfg, const FnxLayer* layers, void* ws, const FnxWindowLanes* lanes, const int* n, const int* tags,
                            void* host_jobs, void* st);

/* per-call timing of windows enqueued outside a graph (the reference's engine keeps per-window timers,
 * src/engine.hpp:182-187): between fnx_trace_begin and fnx_trace_end every C ABI call of fnx_window_stage is bracketed by
 * CUDA events on its stream; fnx_trace_end waits for them and returns each call's name, layer and milliseconds.
 * fnx_window_kernel_count: kernel launches this library has made so far, counted at each launch's check, whoever the
 * caller (reset != 0 reads and zeroes the count) */
int fnx_trace_begin(void);
int fnx_trace_end(float* ms, int* layer, const char** names, int cap);
long fnx_window_kernel_count(int reset);

/* ---- acceptance on the host (reference src/session.cpp:39-82, 469-510) */
typedef struct FnxSampling {
    float temperature, top_p, min_p;
    int top_k;
} FnxSampling;
/* rows[0] the last committed token, rows[1..T) the drafts, out[t] row t's argmax: 1 + the matching prefix */
int fnx_accept_greedy(const int* rows, const int* out, int T);
/* rejection sampling against fixed (one-hot) drafts over the rows' 64 candidates; rng: a std::mt19937_64 stream made
 * by fnx_rng_new(seed); o receives the emitted tokens; returns their number */
void* fnx_rng_new(unsigned long long seed);
void fnx_rng_free(void* rng);
int fnx_accept_sampled(const int* rows, int T, const float* cand_v, const int* cand_i, const FnxSampling* s, void* rng, int* o);
/* n-gram lookup drafts (reference src/session.hpp:48-51, src/session.cpp:377-394 lookup_drafts): ctx = the n tokens so far
 * (host), lk = the most drafts wanted, d1 = the token the first draft must be (the draft layer's, or -1 for any),
 * image_tok = the first image-cell id (the reference's Engine::IMAGE_TOK, 1 << 30).  Writes the drafts to out (room for lk)
 * and returns their number (0: none); negative on bad arguments */
int fnx_lookup_drafts(const int* ctx, int n, int lk, int d1, int image_tok, int* out);
/* merges nslice per-GPU candidate lists [nslice][T][64] into the rows' 64 best (reference src/engine_common.cu:640-653) */
int fnx_top_merge(const float* vs, const int* is, int nslice, int T, float* out_v, int* out_i);
/* the partition rule (reference src/card_split.hpp:12-26): FF slice, value-head owner, key heads of a GPU */
int fnx_ff_lo(int ff, int n, int c);
int fnx_vhead_card(int nkh, int nvh, int n, int v);
int fnx_khead_first(int nkh, int nvh, int n, int c);
int fnx_khead_count(int nkh, int nvh, int n, int c);

/* ---- load-time repacks (the reference's loader does the same kind of work, src/model.cpp:554-606) */
/* GGUF Q8_0 blocks [rows][cols / 32] -> split layout */
int fnx_repack_q8_0_split(const void* blocks, int8_t* q, uint16_t* d, size_t rows, size_t cols, void* st);
/* GGUF Q6_K rows of src_cols -> 32-column units of columns [c0, c0 + cols): the same bytes regrouped so that the
 * FF width can be cut at any multiple of 32 */
int fnx_repack_q6k_units(const void* blocks, size_t rows, size_t src_cols, size_t c0, size_t cols, void* QL, void* QH, void* SC,
                         void* D, void* st);

/* ---- synthetic weights: counter-based N(0, sigma) values quantised on the device (seeded, reproducible) */
int fnx_synth_normal(float* out, size_t n, float sigma, unsigned long long seed, void* st);
int fnx_synth_quant(int type, void* blocks, size_t nvalues, float sigma, unsigned long long seed, void* st);

/* element-wise probes of the kernels' exact math (tests): op 0 exp, 1 log1p, 2 sigmoid, 3 silu, 4 rsqrt, 5 sin, 6 cos */
int fnx_math_probe(int op, const float* x, float* y, size_t n, void* st);

#ifdef __cplusplus
}
#endif
#endif
