// C entry points around the UNMODIFIED reference CPU model.  TEST INFRASTRUCTURE ONLY.
//
// This file is not a translation unit of its own: the recipe in oracle/Makefile streams the
// reference's run.cpp (read where it lies, with the two `#include "getp-csrc/..."` lines that pull in
// the HIP engine dropped, and -DTESTING so that its main() is compiled out) into the compiler and
// appends this file, so everything here sees the reference's own Transformer/Config types and calls
// the reference's own build_transformer(), forward(), matmul(), topk(), softmax() and
// sample_argmax().  No reference source is copied into this repository; only the resulting
// shared object is written (to oracle/_ref/).

#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// ---- whole-model access: run.cpp:283 (build_transformer), :501 (forward), :739 (sample_argmax) ----

void *ref_open(const char *bin_path) {
  Transformer *tr = new Transformer();
  build_transformer(tr, const_cast<char *>(bin_path));
  return tr;
}

void ref_close(void *h) {
  Transformer *tr = static_cast<Transformer *>(h);
  free_transformer(tr);
  delete tr;
}

void ref_config(void *h, int *out15) {
  // 15 four-byte header fields in file order (run.cpp:25-45); the three floats are bit-copied
  memcpy(out15, &static_cast<Transformer *>(h)->config, sizeof(Config));
}

// Runs one position through the reference forward(); returns the greedy next token and, if asked,
// copies the logits.
int ref_forward(void *h, int token, int pos, float *logits_out) {
  Transformer *tr = static_cast<Transformer *>(h);
  float *logits = forward(tr, token, pos);
  if (logits_out) memcpy(logits_out, logits, sizeof(float) * tr->config.vocab_size);
  return sample_argmax(logits, tr->config.vocab_size);
}

// forward() through the first n_layers layers only (the loop bound is the configuration's layer count, run.cpp:519;
// the per-layer weight pointers were laid out for the full model when it was opened, so the prefix sees the same
// weights).  Afterwards ref_last_moe_state describes layer n_layers - 1.  The KV rows it writes for `pos` are the
// ones the full forward() writes, so calling it before ref_forward at the same position changes nothing.
void ref_forward_prefix(void *h, int token, int pos, int n_layers) {
  Transformer *tr = static_cast<Transformer *>(h);
  const int full = tr->config.n_layers;
  if (n_layers < 1 || n_layers > full) return;
  tr->config.n_layers = n_layers;
  forward(tr, token, pos);
  tr->config.n_layers = full;
}

// State left behind by the LAST layer's MoE block after a forward() call: the block input t
// (run.cpp:623), the routing result (run.cpp:636-638; topk_v already softmaxed) and the block
// output e_agg (run.cpp:641-704).  None of these buffers is written again before forward() returns.
void ref_last_moe_state(void *h, float *t, float *topk_v, int *topk_i, float *e_agg,
                        float *router_score) {
  Transformer *tr = static_cast<Transformer *>(h);
  const Config &c = tr->config;
  const RunState &s = tr->state;
  if (t) memcpy(t, s.t, sizeof(float) * c.hidden_dim);
  if (topk_v) memcpy(topk_v, s.topk_v, sizeof(float) * c.experts_per_token);
  if (topk_i) memcpy(topk_i, s.topk_i, sizeof(int) * c.experts_per_token);
  if (e_agg) memcpy(e_agg, s.e_agg, sizeof(float) * c.hidden_dim);
  if (router_score) memcpy(router_score, s.router_score, sizeof(float) * c.n_experts);
}

// ---- the MoE block on a batch of rows, built on the reference's own matmul/topk/softmax ----------
// Sequence of run.cpp:626-704 for each of the T rows of t[T,H]; weights in the .bin layouts
// (gate.weight [E,H], mlp1 [E,2I,H], mlp2 [E,H,I]).  Outputs: e_agg[T,H]; optional topk_v[T,k]
// (softmaxed) and topk_i[T,k].  Rows in [row_begin,row_end) only, so that a timed sample can be
// bounded.  Returns the number of rows processed.
int ref_moe_rows(const float *t, int row_begin, int row_end, const float *w_router,
                 const float *b_router, const float *w_mlp1, const float *b_mlp1,
                 const float *w_mlp2, const float *b_mlp2, int H, int I, int E, int k, float limit,
                 float *e_agg, float *topk_v_out, int *topk_i_out) {
  std::vector<float> score(E), tv(k), mlp1(2 * (size_t)I), act(I), y(H);
  std::vector<int> ti(k);
  for (int b = row_begin; b < row_end; ++b) {
    float *x = const_cast<float *>(t) + (long long)b * H;
    matmul(score.data(), x, const_cast<float *>(w_router), H, E);
    for (int e = 0; e < E; ++e) score[e] += b_router[e];
    topk(tv.data(), ti.data(), score.data(), E, k);
    softmax(tv.data(), k);
    if (topk_v_out) memcpy(topk_v_out + (long long)b * k, tv.data(), sizeof(float) * k);
    if (topk_i_out) memcpy(topk_i_out + (long long)b * k, ti.data(), sizeof(int) * k);

    float *agg = e_agg + (long long)b * H;
    for (int i = 0; i < H; ++i) agg[i] = 0.0f;
    for (int e = 0; e < E; ++e) {  // ascending expert id, first matching slot (run.cpp:642-652)
      int slot = -1;
      for (int j = 0; j < k && slot < 0; ++j)
        if (ti[j] == e) slot = j;
      if (slot < 0) continue;
      const float gate_weight = tv[slot];
      matmul(mlp1.data(), x, const_cast<float *>(w_mlp1) + (long long)e * 2 * I * H, H, 2 * I);
      const float *b1 = b_mlp1 + (long long)e * 2 * I;
      for (int i = 0; i < 2 * I; ++i) mlp1[i] += b1[i];
      for (int c = 0; c < I; ++c) {  // run.cpp:664-686
        float g = mlp1[2 * c], u = mlp1[2 * c + 1];
        if (g > limit) g = limit;
        if (u > limit) u = limit;
        if (u < -limit) u = -limit;
        g *= (1.0f / (1.0f + expf(-1.702f * g)));
        g *= (u + 1.0f);
        act[c] = g;
      }
      matmul(y.data(), act.data(), const_cast<float *>(w_mlp2) + (long long)e * H * I, I, H);
      const float *b2 = b_mlp2 + (long long)e * H;
      for (int i = 0; i < H; ++i) y[i] += b2[i];
      for (int i = 0; i < H; ++i) agg[i] += y[i] * gate_weight;
    }
  }
  return row_end - row_begin;
}

// ---- tokenizer: read_tokenizer (tokenizer.cpp:49) + encode (tokenizer.cpp:268) ---------------------------------
int ref_encode(const char *tokenizer_path, int vocab_size, const char *text, int *out, int max_tokens) {
  Tokenizer t;
  read_tokenizer(&t, tokenizer_path, vocab_size);
  int n = 0;
  encode(&t, text, -1, -1, out, &n, max_tokens);
  free_tokenizer(&t);
  return n;
}

int ref_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
