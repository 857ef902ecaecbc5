/*
 * CPU oracle for the GPT-OSS MoE FFN block (see moe_oracle.h).  TEST INFRASTRUCTURE ONLY.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -fPIC -shared moe_oracle.c -lm
 * (-ffp-contract=off keeps every multiply and add a separately rounded IEEE operation, so the
 *  result does not depend on whether the host has FMA.)
 *
 * The arithmetic follows the reference CPU model exactly: fp32 products accumulated into a double
 * in ascending input index (run.cpp:339-352), fp32 bias adds, fp32 SwiGLU with expf
 * (run.cpp:670-686), fp32 weighted aggregation in ascending expert id (run.cpp:642,699-702).
 * Tokens are processed in blocks per expert for speed; each output element still sees the same
 * sequence of operations as the token-at-a-time reference loop.
 */
#include "moe_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TOK_BLOCK 64

uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float oracle_bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

void oracle_round_bf16(float *x, long long n) {
  for (long long i = 0; i < n; ++i) x[i] = oracle_bf16_to_f32(oracle_f32_to_bf16(x[i]));
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* out[d] = W[d,n] . x[n] for a block of tokens held transposed (xt[n][mb]); double accumulation in
 * ascending n with fp32 products, exactly the per-element sequence of run.cpp:339-352. */
static void matmul_block(const float *w, const float *xt, int n, int d, int mb, float *out_t) {
  double acc[TOK_BLOCK];
  for (int i = 0; i < d; ++i) {
    const float *wr = w + (long long)i * n;
    for (int m = 0; m < mb; ++m) acc[m] = 0.0;
    for (int j = 0; j < n; ++j) {
      const float wv = wr[j];
      const float *xr = xt + (long long)j * TOK_BLOCK;
      for (int m = 0; m < mb; ++m) {
        float prod = wv * xr[m];
        acc[m] += prod;
      }
    }
    float *o = out_t + (long long)i * TOK_BLOCK;
    for (int m = 0; m < mb; ++m) o[m] = (float)acc[m];
  }
}

void oracle_router_scores(const float *t, const float *w_router, const float *b_router, int T, int H,
                          int E, float *scores) {
#pragma omp parallel for schedule(static)
  for (int b = 0; b < T; ++b) {
    const float *x = t + (long long)b * H;
    for (int e = 0; e < E; ++e) {
      const float *w = w_router + (long long)e * H;
      double val = 0.0;
      for (int j = 0; j < H; ++j) {
        float prod = w[j] * x[j];
        val += prod;
      }
      float s = (float)val;
      s += b_router[e];
      scores[(long long)b * E + e] = s;
    }
  }
}

typedef struct {
  float value;
  int index;
} score_pair;

static int cmp_desc(const void *a, const void *b) {
  float diff = ((const score_pair *)b)->value - ((const score_pair *)a)->value;
  if (diff > 0) return 1;
  if (diff < 0) return -1;
  return 0;
}

int oracle_topk_softmax(const float *scores, int T, int E, int k, int rule, float *topk_w,
                        int *topk_i, float *topk_raw) {
  int tie_rows = 0;
  if (E <= 0 || k <= 0 || k > E) return -1;
  float *vals = (float *)malloc(sizeof(float) * (size_t)E);
  int *idx = (int *)malloc(sizeof(int) * (size_t)E);
  score_pair *pairs = (score_pair *)malloc(sizeof(score_pair) * (size_t)E);
  float *sel = (float *)malloc(sizeof(float) * (size_t)(k + 1));
  for (int b = 0; b < T; ++b) {
    const float *r = scores + (long long)b * E;
    /* selection of the k+1 largest with the GPU rule; used for tie detection in both modes */
    for (int i = 0; i < E; ++i) {
      vals[i] = r[i];
      idx[i] = i;
    }
    int kk = (k + 1 <= E) ? k + 1 : E;
    for (int i = 0; i < kk; ++i) {
      int max_idx = i;
      for (int j = i + 1; j < E; ++j)
        if (vals[j] > vals[max_idx]) max_idx = j;
      if (max_idx != i) {
        float tv = vals[i];
        vals[i] = vals[max_idx];
        vals[max_idx] = tv;
        int ti = idx[i];
        idx[i] = idx[max_idx];
        idx[max_idx] = ti;
      }
      /* the reference stops after k rounds; the extra (k+1)-th round run here (for tie detection)
       * only swaps positions >= k and so never changes the first k entries */
    }
    int tie = 0;
    for (int i = 0; i + 1 < kk; ++i)
      if (vals[i] == vals[i + 1]) tie = 1;
    tie_rows += tie;

    float *w_out = topk_w + (long long)b * k;
    int *i_out = topk_i + (long long)b * k;
    if (rule == ORACLE_TOPK_SELECTION) {
      for (int i = 0; i < k; ++i) sel[i] = vals[i];
      for (int i = 0; i < k; ++i) i_out[i] = idx[i];
      /* layer_hip_batch.cpp:1143-1153 */
      double max_val = (double)sel[0];
      double denom = 0.0;
      for (int i = 0; i < k; ++i) denom += expf(sel[i] - (float)max_val);
      for (int i = 0; i < k; ++i) w_out[i] = expf(sel[i] - (float)max_val) / (float)denom;
      if (topk_raw)
        for (int i = 0; i < k; ++i) topk_raw[(long long)b * k + i] = sel[i];
    } else {
      for (int i = 0; i < E; ++i) {
        pairs[i].value = r[i];
        pairs[i].index = i;
      }
      qsort(pairs, (size_t)E, sizeof(score_pair), cmp_desc);
      for (int i = 0; i < k; ++i) {
        w_out[i] = pairs[i].value;
        i_out[i] = pairs[i].index;
        if (topk_raw) topk_raw[(long long)b * k + i] = pairs[i].value;
      }
      /* run.cpp:319-337 */
      double max_val = w_out[0];
      for (int i = 1; i < k; ++i)
        if (w_out[i] > max_val) max_val = w_out[i];
      double sum = 0.0;
      for (int i = 0; i < k; ++i) {
        w_out[i] = expf((float)(w_out[i] - max_val));
        sum += w_out[i];
      }
      for (int i = 0; i < k; ++i) w_out[i] = (float)(w_out[i] / sum);
    }
  }
  free(vals);
  free(idx);
  free(pairs);
  free(sel);
  return tie_rows;
}

void oracle_topk_margin(const float *scores, int T, int E, int k, float *margin) {
  float *top = (float *)malloc(sizeof(float) * (size_t)(k + 2));
  int kk = (k + 1 <= E) ? k + 1 : E;
  for (int b = 0; b < T; ++b) {
    const float *r = scores + (long long)b * E;
    for (int i = 0; i < kk; ++i) top[i] = -INFINITY;
    for (int e = 0; e < E; ++e) { /* insertion into a descending list of the kk largest */
      float v = r[e];
      int p = kk;
      while (p > 0 && v > top[p - 1]) --p;
      if (p < kk) {
        for (int q = kk - 1; q > p; --q) top[q] = top[q - 1];
        top[p] = v;
      }
    }
    float m = INFINITY;
    for (int i = 0; i + 1 < kk; ++i) {
      float g = top[i] - top[i + 1];
      if (g < m) m = g;
    }
    margin[b] = m;
  }
  free(top);
}

int oracle_counting_sort(const int *topk_i, int P, int E, int *offsets, int *sorted) {
  int *cnt = (int *)calloc((size_t)E, sizeof(int));
  for (int p = 0; p < P; ++p) {
    int e = topk_i[p];
    if (0 <= e && e < E) cnt[e]++;
  }
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + cnt[e];
  memset(cnt, 0, sizeof(int) * (size_t)E);
  for (int p = 0; p < P; ++p) {
    int e = topk_i[p];
    if (0 <= e && e < E) sorted[offsets[e] + cnt[e]++] = p;
  }
  int placed = offsets[E];
  free(cnt);
  return placed;
}

void oracle_gather(const float *t, const int *sorted, int n_rows, int k, int H, float *x_packed) {
  for (int p = 0; p < n_rows; ++p)
    memcpy(x_packed + (long long)p * H, t + (long long)(sorted[p] / k) * H, sizeof(float) * (size_t)H);
}

/* clamp + SwiGLU on de-interleaved gate/up values (run.cpp:664-686) */
static inline float swiglu_one(float gate, float up, float limit) {
  const float alpha = 1.702f;
  float val = gate;
  float up_val = up;
  if (val > limit) val = limit;
  if (up_val > limit) up_val = limit;
  if (up_val < -limit) up_val = -limit;
  val *= (1.0f / (1.0f + expf(-alpha * val)));
  val *= (up_val + 1.0f);
  return val;
}

/* Applies expert e to mb token rows given transposed (xt[H][TOK_BLOCK]); writes ht[I][TOK_BLOCK] and
 * yt[H][TOK_BLOCK].  g_t is scratch [2I][TOK_BLOCK]. */
static void expert_block(const oracle_dims *d, int mode, const float *xt, int mb, const float *w1,
                         const float *b1, const float *w2, const float *b2, float *g_t, float *ht,
                         float *yt) {
  const int H = d->hidden, I = d->intermediate;
  matmul_block(w1, xt, H, 2 * I, mb, g_t);
  for (int i = 0; i < 2 * I; ++i)
    for (int m = 0; m < mb; ++m) g_t[(long long)i * TOK_BLOCK + m] += b1[i];
  for (int c = 0; c < I; ++c)
    for (int m = 0; m < mb; ++m) {
      float v = swiglu_one(g_t[(long long)(2 * c) * TOK_BLOCK + m],
                           g_t[(long long)(2 * c + 1) * TOK_BLOCK + m], d->swiglu_limit);
      if (mode == ORACLE_MODE_GPU_BF16) v = oracle_bf16_to_f32(oracle_f32_to_bf16(v));
      ht[(long long)c * TOK_BLOCK + m] = v;
    }
  matmul_block(w2, ht, I, H, mb, yt);
  for (int i = 0; i < H; ++i)
    for (int m = 0; m < mb; ++m) yt[(long long)i * TOK_BLOCK + m] += b2[i];
}

void oracle_expert_row(const oracle_dims *d, int mode, const float *t_row, const float *w_mlp1_e,
                       const float *b_mlp1_e, const float *w_mlp2_e, const float *b_mlp2_e,
                       float *h_out, float *y_out) {
  const int H = d->hidden, I = d->intermediate;
  float *xt = (float *)calloc((size_t)H * TOK_BLOCK, sizeof(float));
  float *g_t = (float *)malloc(sizeof(float) * (size_t)2 * I * TOK_BLOCK);
  float *ht = (float *)malloc(sizeof(float) * (size_t)I * TOK_BLOCK);
  float *yt = (float *)malloc(sizeof(float) * (size_t)H * TOK_BLOCK);
  for (int j = 0; j < H; ++j) xt[(long long)j * TOK_BLOCK] = t_row[j];
  expert_block(d, mode, xt, 1, w_mlp1_e, b_mlp1_e, w_mlp2_e, b_mlp2_e, g_t, ht, yt);
  if (h_out)
    for (int c = 0; c < I; ++c) h_out[c] = ht[(long long)c * TOK_BLOCK];
  if (y_out)
    for (int i = 0; i < H; ++i) y_out[i] = yt[(long long)i * TOK_BLOCK];
  free(xt);
  free(g_t);
  free(ht);
  free(yt);
}

void oracle_moe_block(const oracle_dims *d, int mode, const float *t, int T, const float *topk_w,
                      const int *topk_i, const float *w_mlp1, const float *b_mlp1,
                      const float *w_mlp2, const float *b_mlp2, int e_begin, int e_end, float *out,
                      float *h_pairs, float *y_pairs) {
  const int H = d->hidden, I = d->intermediate, E = d->n_experts, k = d->top_k;
  const int P = T * k;
  int *offsets = (int *)malloc(sizeof(int) * (size_t)(E + 1));
  int *sorted = (int *)malloc(sizeof(int) * (size_t)(P > 0 ? P : 1));
  oracle_counting_sort(topk_i, P, E, offsets, sorted);
  float *y_all = y_pairs ? y_pairs : (float *)malloc(sizeof(float) * (size_t)(P > 0 ? P : 1) * H);

  /* work items = (expert, token block) so that a hot expert does not serialise the run */
  int n_items = 0;
  for (int e = e_begin; e < e_end; ++e)
    n_items += (offsets[e + 1] - offsets[e] + TOK_BLOCK - 1) / TOK_BLOCK;
  int *item_e = (int *)malloc(sizeof(int) * (size_t)(n_items > 0 ? n_items : 1));
  int *item_r = (int *)malloc(sizeof(int) * (size_t)(n_items > 0 ? n_items : 1));
  n_items = 0;
  for (int e = e_begin; e < e_end; ++e)
    for (int r = offsets[e]; r < offsets[e + 1]; r += TOK_BLOCK) {
      item_e[n_items] = e;
      item_r[n_items] = r;
      ++n_items;
    }

#pragma omp parallel
  {
    float *xt = (float *)malloc(sizeof(float) * (size_t)H * TOK_BLOCK);
    float *g_t = (float *)malloc(sizeof(float) * (size_t)2 * I * TOK_BLOCK);
    float *ht = (float *)malloc(sizeof(float) * (size_t)I * TOK_BLOCK);
    float *yt = (float *)malloc(sizeof(float) * (size_t)H * TOK_BLOCK);
#pragma omp for schedule(dynamic, 1)
    for (int it = 0; it < n_items; ++it) {
      const int e = item_e[it], r0 = item_r[it];
      const int mb = (offsets[e + 1] - r0 < TOK_BLOCK) ? offsets[e + 1] - r0 : TOK_BLOCK;
      for (int m = 0; m < mb; ++m) {
        const float *row = t + (long long)(sorted[r0 + m] / k) * H;
        for (int j = 0; j < H; ++j) xt[(long long)j * TOK_BLOCK + m] = row[j];
      }
      expert_block(d, mode, xt, mb, w_mlp1 + (long long)e * 2 * I * H, b_mlp1 + (long long)e * 2 * I,
                   w_mlp2 + (long long)e * H * I, b_mlp2 + (long long)e * H, g_t, ht, yt);
      for (int m = 0; m < mb; ++m) {
        const int pair = sorted[r0 + m];
        float *yo = y_all + (long long)pair * H;
        for (int i = 0; i < H; ++i) yo[i] = yt[(long long)i * TOK_BLOCK + m];
        if (h_pairs) {
          float *ho = h_pairs + (long long)pair * I;
          for (int c = 0; c < I; ++c) ho[c] = ht[(long long)c * TOK_BLOCK + m];
        }
      }
    }
    free(xt);
    free(g_t);
    free(ht);
    free(yt);
  }

  /* weighted aggregation in ascending expert id (run.cpp:642-652, 699-702): for each expert the
   * reference takes the FIRST slot holding it */
#pragma omp parallel for schedule(static)
  for (int b = 0; b < T; ++b) {
    float *o = out + (long long)b * H;
    for (int i = 0; i < H; ++i) o[i] = 0.0f;
    for (int e = e_begin; e < e_end; ++e) {
      int slot = -1;
      for (int j = 0; j < k; ++j)
        if (topk_i[(long long)b * k + j] == e) {
          slot = j;
          break;
        }
      if (slot < 0) continue;
      const float w = topk_w[(long long)b * k + slot];
      const float *y = y_all + ((long long)b * k + slot) * H;
      for (int i = 0; i < H; ++i) {
        float prod = y[i] * w;
        o[i] += prod;
      }
    }
  }
  if (!y_pairs) free(y_all);
  free(item_e);
  free(item_r);
  free(offsets);
  free(sorted);
}

void oracle_moe_forward(const oracle_dims *d, int mode, int rule, const float *t, int T,
                        const float *w_router, const float *b_router, const float *w_mlp1,
                        const float *b_mlp1, const float *w_mlp2, const float *b_mlp2, float *x) {
  const int H = d->hidden, E = d->n_experts, k = d->top_k;
  float *scores = (float *)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1) * E);
  float *tw = (float *)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1) * k);
  int *ti = (int *)malloc(sizeof(int) * (size_t)(T > 0 ? T : 1) * k);
  float *out = (float *)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1) * H);
  oracle_router_scores(t, w_router, b_router, T, H, E, scores);
  oracle_topk_softmax(scores, T, E, k, rule, tw, ti, NULL);
  oracle_moe_block(d, mode, t, T, tw, ti, w_mlp1, b_mlp1, w_mlp2, b_mlp2, 0, E, out, NULL, NULL);
  for (long long i = 0; i < (long long)T * H; ++i) x[i] += out[i];
  free(scores);
  free(tw);
  free(ti);
  free(out);
}

void oracle_combine_slots(const float *y_pairs, const float *topk_w, int T, int k, int H, float *out) {
  for (int b = 0; b < T; ++b)
    for (int i = 0; i < H; ++i) {
      float acc = 0.0f;
      for (int j = 0; j < k; ++j) {
        float s = topk_w[(long long)b * k + j] * y_pairs[((long long)b * k + j) * H + i];
        acc = (j == 0) ? s : acc + s;
      }
      out[(long long)b * H + i] = acc;
    }
}

/* ---- seeded synthetic tensors (same stream definition as the Python module `synth`) ------------- */
static inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

void oracle_synth_normal_f32(uint64_t seed, uint64_t tensor_id, uint64_t start, uint64_t n, float sigma,
                             float *out) {
  const uint64_t key = splitmix64(seed * 0x100000001B3ull + tensor_id);
  const float scale = (float)((double)sigma / 53509.91992145008); /* sqrt(8 (65536^2 - 1) / 12) */
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)n; ++i) {
    const uint64_t a = splitmix64(key + 2ull * (start + (uint64_t)i));
    const uint64_t b = splitmix64(key + 2ull * (start + (uint64_t)i) + 1ull);
    int s = 0;
    for (int sh = 0; sh < 64; sh += 16) s += (int)((a >> sh) & 0xFFFFull) + (int)((b >> sh) & 0xFFFFull);
    const float z = (float)(s - 4 * 65535) * scale;
    out[i] = oracle_bf16_to_f32(oracle_f32_to_bf16(z));
  }
}
