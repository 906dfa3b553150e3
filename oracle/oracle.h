/* CPU ORACLE - test infrastructure, not product code.
 *
 * Plain-C restatement of the reference's verify-window arithmetic (johnfink8/sfnx: src/moe.cuh, src/moe_q4k.cuh,
 * src/dense.cuh, src/gdn_core.cuh, src/kernels.cu, src/topk.cuh, src/session.cpp).  Only the tests, the smoke check
 * and the bench's CPU-baseline leg may load it; the CUDA library never links or calls it.
 */
#ifndef ORACLE_H
#define ORACLE_H

#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#include "omath.h"

#define ORC_MAXT 16
#define ORC_TOPK_N 64

typedef struct { /* reference src/kernels.hpp:18-23 */
    int w;
    int n;
    int y[ORC_MAXT];
    int out[ORC_MAXT];
} OrcJob;

#define ORC_PF_JOB 64
typedef struct { /* reference src/kernels.hpp:25-32 (BigJob): up to 64 rows of one expert */
    int w;
    int n;
    int y[ORC_PF_JOB];
    int out[ORC_PF_JOB];
} OrcBigJob;

typedef struct { /* reference src/kernels.hpp:160-165; pt null: one contiguous run of local rows */
    const int* pt;
    size_t page; /* halves per page */
    int rows;    /* local rows per page */
    int cap;     /* rows of a cache without a page table (needed when q8) */
    int q8;      /* int8 rows with an f16 scale per group of 32: reference src/kernels.hpp:149-181 */
} OrcKvPages;

typedef struct { /* reference src/session.hpp:18-25 (the fields the distribution uses) */
    float temperature, top_p, min_p;
    int top_k;
} OrcSampling;

typedef struct {
    uint64_t mt[312];
    int idx;
} OrcMt;

/* formats */
void orc_q4k_scale_min(const uint8_t* sc12, int j, int* sc, int* m);
void orc_dequant_q4k(const uint8_t* blocks, float* out, size_t nblocks);
int orc_q6k_q(const uint8_t* blk, int i);
void orc_dequant_q6k(const uint8_t* blocks, float* out, size_t nblocks);
void orc_dequant_q8_0(const uint8_t* blocks, float* out, size_t nblocks);
void orc_quantize_q8_0(const float* x, uint8_t* blocks, size_t nblocks);
void orc_quantize_q4k(const float* x, uint8_t* blocks, size_t nblocks);
void orc_quantize_q6k(const float* x, uint8_t* blocks, size_t nblocks);
void orc_q8_0_to_split(const uint8_t* blocks, int8_t* q, o_half* d, size_t rows, size_t cols);
void orc_q6k_to_planes(const uint8_t* blocks, size_t rows, size_t src_cols, size_t c0, size_t cols, uint8_t* QL, uint8_t* QH,
                       int8_t* SC, o_half* D);
int orc_q6p_q(const uint8_t* ql16, const uint8_t* qh8, int i);
void orc_quantize_q8_1(const float* x, uint8_t* q, int n, int rows);

/* MoE FFN */
void orc_gemv_f32(const float* W, const float* x, float* y, int rows, int n, int T, int parts, int y_stride);
void orc_router_route(const float* W, const float* x, float* logits, int T, int n, int nexp, int topk, int* topi, float* topw,
                      OrcJob* gu, OrcJob* dn, int* njobs);
void orc_moe_gate_up_q4k(const uint8_t* A, size_t sa, const OrcJob* jobs, int njobs, const uint8_t* xq, float* gu, int n,
                         int nrows);
float orc_q8s_row_dot(const int8_t* wq, const o_half* wd, const int8_t* a, const float* da, int cols);
void orc_q8_1_unpack(const uint8_t* yq, int cols, int rows, int8_t* a, float* da);
void orc_q8s_gemv(const int8_t* wq, const o_half* wd, int rows, int cols, const uint8_t* yq, float* out, int out_stride, int T);
void orc_q8s_gemv_blocks(const int8_t* wq, const o_half* wd, int rows, int cols, const uint8_t* yq, float* out, int out_stride, int T);
void orc_moe_gate_up_q8(const int8_t* wq, size_t sq, const o_half* wd, size_t sd, const OrcJob* jobs, int njobs,
                        const uint8_t* xq, int T, float* gu, int n, int nrows);
void orc_swiglu_q8(const float* gu_row, int ffs, int8_t* hq, float* hd);
void orc_moe_down_q6p(const uint8_t* QL, const uint8_t* QH, const int8_t* SC, const o_half* D, size_t expert_units,
                      const OrcJob* jobs, int njobs, const float* gu, float* part, int nrows, int ffs);
void orc_moe_down_q8(const int8_t* wq, size_t sq, const o_half* wd, size_t sd, const OrcJob* jobs, int njobs, const float* gu,
                     float* part, int nrows, int ffs);
void orc_shared_expert(const int8_t* guq, const o_half* gud, const int8_t* dnq, const o_half* dnd, const uint8_t* xq, int T,
                       int n, int ffs, float* sh_gu, float* out);
void orc_moe_combine(const float* part, const float* topw, const float* sh, const float* logits, int logit_stride, int sh_col,
                     float* out, int T, int n, int topk);
/* the prompt path's experts: f16 weights with one rounding, sums in double (omma.c) */
o_half orc_d2h(double x);
void orc_mma_weights_q4k(const uint8_t* A, int rows, int n, o_half* w);
void orc_mma_weights_q8(const int8_t* wq, const o_half* wd, int rows, int n, o_half* w);
void orc_mma_weights_q6p(const uint8_t* QL, const uint8_t* QH, const int8_t* SC, const o_half* D, int rows, int n, o_half* w);
void orc_moe_mma(const o_half* w, const OrcBigJob* jobs, int njobs, const o_half* x, int nrows, int n, double* out, double* mag);
void orc_swiglu_h16(const float* gu, int ffs, int P, o_half* h);
void orc_rms_norm_rows(const float* x, const float* w, float* y, int rows, int n, float eps);

/* Gated DeltaNet */
void orc_gdn_core(const float* qkvz, const float* ab, float* hist, const float* convw, const float* dt, const float* a,
                  const float* nw, float* S, uint8_t* yq, const int* ctl, float* snap, float* hsnap, int nk, int nv,
                  const int* vmap, int T, float eps, float* y32);
void orc_gdn_rollback(float* S, float* hist, const float* snap, const float* hsnap, const int* ctl, int nk, int nv, int T, int n);

/* attention */
int orc_kv_owned(int p, int card, int ncard);
void orc_rope_freqs(float base, int nrot, float* freq);
void orc_attn_prep_append(float* qg, float* k, const float* v, const float* q_norm, const float* k_norm, o_half* kc, o_half* vc,
                          const OrcKvPages* g, int card, int ncard, int T, int pos0, float eps, float rope_base, int nq, int nkv,
                          int hd, int nrot);
void orc_attn_partial(const float* qg, const o_half* kc, const o_half* vc, const OrcKvPages* g, float* part, int card, int ncard,
                      int T, int pos0, int nq, int nkv, int hd);
void orc_attn_partial_cells(const float* qg, const o_half* kc, const o_half* vc, const OrcKvPages* g, float* part, int card, int ncard,
                            int T, int pos0, int nq, int nkv, int hd, const int* cells, const int* n_cells, int maxsel);
void orc_attn_merge(const float* const* parts, const float* qg, float* out, int ncard, int T, int nq, int hd);

/* the attention layers' block selection (oqsa.c) */
void orc_qsa_proj(const uint16_t* wq, const uint16_t* wk, const float* x, float* y, int T, int n);
void orc_qsa_index(const float* y, const float* qn, const float* kn, o_half* ring, int ring_rows, o_half* pooled, const OrcKvPages* g,
                   int ncard, float* q, int pos0, int T, float eps, float rope_base);
void orc_qsa_select(const float* q, const o_half* pooled, const OrcKvPages* g, float* scores, int* cells, int* n_cells, int max_pools,
                    const int* pos, const int* const* pts, int T, int card, int ncard, int top);

/* hyper-connections (ohc.c) */
void orc_hc_write(float* R, const float* bo, const float* inj, int T, int n, int hc);
void orc_hc_read(float* R, const float* bo_prev, const float* inj_prev, const float* w_norm, const int8_t* down_q, const o_half* down_d,
                 const int8_t* up_q, const o_half* up_d, const uint16_t* w_inj, float eps, float* mixed, float* inject, uint8_t* q8, int T,
                 int n, int hc, int lr);

/* head, acceptance, ring order */
unsigned orc_argmax(const float* logits, int rows, int T, int v0, float* best_v, int* best_i);
void orc_argmax_merge(const float* best_v, const int* best_i, int nslice, int T, int* out);
unsigned orc_top_tokens(float* logits, int n, int T, int v0, const int* pen_tok, const int* pen_cnt, const int* pen_n,
                        int pen_stride, const float* pen_par, float* out_v, int* out_i);
void orc_top_merge(const float* vs, const int* is, int nslice, int T, float* out_v, int* out_i);
void orc_make_dist(const float* cv, const int* ci, int ncand, const OrcSampling* s, int* n_out, int* ids, double* p);
void orc_mt_seed(OrcMt* g, uint64_t seed);
uint64_t orc_mt_next(OrcMt* g);
double orc_mt_unif(OrcMt* g);
int orc_accept_greedy(const int* rows, const int* out, int T);
int orc_lookup_drafts(const int* ctx, int n, int lk, int d1, int image_tok, int* out);
int orc_accept_sampled(const int* rows, int T, const float* cand_v, const int* cand_i, const OrcSampling* s, OrcMt* rng, int* o);
void orc_ring_sum(const float* const* x, float* out, int nrank, int T, int row_len);

/* scalar probes for the math tests */
void orc_math_probe(int op, const float* x, float* y, size_t n);

#endif
