/*
 * CPU oracle for the GPT-OSS MoE FFN block.  TEST INFRASTRUCTURE ONLY: the product library never
 * links, loads or calls anything in this directory.  Every function states the reference file:line
 * whose arithmetic it restates (paths relative to the reference project root).
 *
 * Parity status: PINNED.  The restatement is checked against outputs of the reference's own
 * forward() (run.cpp:501) executed on a seeded gpt-oss-7m-shaped checkpoint; the vectors are
 * committed under tests/golden/ together with the script that produced them.
 */
#ifndef MOE_ORACLE_H
#define MOE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Rounding contract of the block. */
enum {
  ORACLE_MODE_CPU = 0,      /* run.cpp:622-709 verbatim arithmetic: fp32 data, double accumulation   */
  ORACLE_MODE_GPU_BF16 = 1  /* same, but the SwiGLU output is rounded to bf16 before the down        */
                            /* projection, as the reference GPU path stores it (matrix_core.cpp:1674) */
};

/* Which top-k tie rule / softmax formula to follow. */
enum {
  ORACLE_TOPK_SELECTION = 0, /* selection sort with swap, strict '>' (layer_hip_batch.cpp:1119-1140)  */
  ORACLE_TOPK_QSORT = 1      /* libc qsort on (value,index) pairs (run.cpp:371-402); ties unspecified */
};

typedef struct {
  int hidden;        /* H  */
  int intermediate;  /* I  */
  int n_experts;     /* E  */
  int top_k;         /* k  */
  float swiglu_limit;
} oracle_dims;

/* bf16 helpers (round to nearest even), used to build bf16-representable fp32 inputs. */
uint16_t oracle_f32_to_bf16(float f);
float oracle_bf16_to_f32(uint16_t h);
void oracle_round_bf16(float *x, long long n);

/* scores[T,E] = t[T,H] . Wr[E,H]^T + br   (run.cpp:627-634; double accumulation as run.cpp:339-352) */
void oracle_router_scores(const float *t, const float *w_router, const float *b_router, int T, int H,
                          int E, float *scores);

/* Top-k of each row of scores[T,E] in descending order + softmax over the selected raw scores.
 *   rule = ORACLE_TOPK_SELECTION: layer_hip_batch.cpp:1119-1153 (weights by the GPU formula)
 *   rule = ORACLE_TOPK_QSORT    : run.cpp:371-402 + run.cpp:319-337 (weights by the CPU formula)
 * topk_raw (optional) receives the selected raw scores.  Returns the number of rows in which two
 * of the k+1 largest scores are exactly equal (ties make the reference's own two paths disagree). */
int oracle_topk_softmax(const float *scores, int T, int E, int k, int rule, float *topk_w,
                        int *topk_i, float *topk_raw);

/* margin[t] = smallest gap between consecutive entries of the k+1 largest scores of row t. */
void oracle_topk_margin(const float *scores, int T, int E, int k, float *margin);

/* Counting sort of pair ids by expert (kernel.cpp:504-542 executed serially => stable order).
 * offsets[E+1], sorted[P]; pairs with an id outside [0,E) are skipped (kernel.cpp:519,537).
 * Returns the number of pairs placed. */
int oracle_counting_sort(const int *topk_i, int P, int E, int *offsets, int *sorted);

/* x_packed[p,:] = t[sorted[p]/k,:]  (kernel.cpp:560) */
void oracle_gather(const float *t, const int *sorted, int n_rows, int k, int H, float *x_packed);

/* One expert applied to one token row: mlp1 + bias, de-interleave, clamp, SwiGLU, (optional bf16),
 * mlp2 + bias  (run.cpp:655-697).  h_out[I] and y_out[H] are optional taps. */
void oracle_expert_row(const oracle_dims *d, int mode, const float *t_row, const float *w_mlp1_e,
                       const float *b_mlp1_e, const float *w_mlp2_e, const float *b_mlp2_e,
                       float *h_out, float *y_out);

/* The whole block for T rows (run.cpp:622-709 minus the rmsnorm and the residual):
 *   out[T,H] = sum over selected experts (ascending expert id, as run.cpp:642) of w * expert(t).
 * Only experts in [e_begin,e_end) contribute (expert-parallel partial, model.cpp:342-426);
 * pass 0,E for the full block.  topk_w/topk_i [T,k] come from oracle_topk_softmax.
 * h_pairs (optional) [T*k, I]: SwiGLU output of pair b*k+j;  y_pairs (optional) [T*k, H]: unweighted
 * expert output of pair b*k+j.  Threads over experts with OpenMP when compiled with -fopenmp. */
void oracle_moe_block(const oracle_dims *d, int mode, const float *t, int T, const float *topk_w,
                      const int *topk_i, const float *w_mlp1, const float *b_mlp1,
                      const float *w_mlp2, const float *b_mlp2, int e_begin, int e_end, float *out,
                      float *h_pairs, float *y_pairs);

/* Convenience: router -> top-k -> block -> residual, x[T,H] += out (run.cpp:707-709). */
void oracle_moe_forward(const oracle_dims *d, int mode, int rule, const float *t, int T,
                        const float *w_router, const float *b_router, const float *w_mlp1,
                        const float *b_mlp1, const float *w_mlp2, const float *b_mlp2, float *x);

/* The slot-ordered combine the CUDA path uses: out[b] = ((s0+s1)+s2)+s3 with s_j = w_j*y_(b,j),
 * fp32.  Differs from run.cpp:699-702 only in summation order (slot order instead of expert id
 * order); provided so tests can bound that difference separately. */
void oracle_combine_slots(const float *y_pairs, const float *topk_w, int T, int k, int H, float *out);

/* out[i] = element start+i of the seeded stream (seed, tensor_id): N(0,sigma) rounded to bf16, as fp32.
 * Same bits as the Python module `synth` and the CUDA generator; multithreaded. */
void oracle_synth_normal_f32(uint64_t seed, uint64_t tensor_id, uint64_t start, uint64_t n, float sigma,
                             float *out);

int oracle_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
