// Whole-model decode step around the MoE block: the B200 counterpart of forward_gpu_20b_batched /
// forward_gpu_120b_batched (getp-csrc/src/model.cpp:6-151, 153-489) and of the CPU forward() (run.cpp:501-717).
//
// One GPU holds the whole model, or `world` GPUs (one model object each) split the work: the sequences of the
// batch are dealt out in contiguous slices (attention, dense GEMMs, KV cache and residual stream of a sequence live
// on its rank only: data-parallel attention, no attention-side all-reduce) and the experts are sharded by rank;
// per layer the ranks exchange the routing of their tokens, the normalised rows (each row only to the ranks whose
// experts it selected) and the expert outputs (stored to the token's owner from the down-GEMM epilogue), all over
// peer memory.
//
// Per step (all sequences at the same position, prompt tokens force-fed by the caller — the reference's
// lock-step decode): embedding -> per layer [RMSNorm -> QKV GEMM -> RoPE + KV store -> single-query attention
// with sinks / sliding window -> o-proj GEMM -> residual + RMSNorm -> MoE block] -> final RMSNorm ->
// classifier GEMM -> argmax.  The dense GEMMs (QKV, o-proj, classifier) run on the same tcgen05 kernel as the
// expert down-projection: one "expert" holding every row, identity permutation, weight 1.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "kernels.cuh"

using namespace gptoss;

struct gptoss_model {
  gptoss_model_config c;
  int device = 0, max_batch = 0, S = 0, sm_count = kSmCountFallback;
  int rank = 0, world = 1;
  int max_local = 0;                    // sequences this rank can hold: max_batch, or its slice of it
  int step_B = 0, step_pos = 0, step_first = 0, step_n = 0;  // the step in progress: global batch, position, own slice
  gptoss_ctx *moe = nullptr;
  // weights
  __nv_bfloat16 *emb = nullptr, *unemb = nullptr, *w_qkv = nullptr, *w_o = nullptr;
  float *attn_norm = nullptr, *mlp_norm = nullptr, *final_norm = nullptr, *b_qkv = nullptr, *b_o = nullptr, *sinks = nullptr;
  std::vector<CUtensorMap> map_qkv, map_o;
  CUtensorMap map_unemb, map_t, map_att;
  CUtensorMap map_t_as_w, map_unemb_rows;  // fused classifier + argmax: the batch as the MMA's M side, the vocabulary as its N side
  float *amax_val = nullptr;            // [vocab blocks][sequences] largest logit of the block
  int *amax_at = nullptr;               //                           and its vocabulary id
  int *amax_sched = nullptr;            // offsets {0, V}, token-block prefix {0, vocab blocks}; then {0, 1}, {0, 1} for one row
  int n_vocab_blocks = 0;
  float *cos_t = nullptr, *sin_t = nullptr;
  __nv_bfloat16 *k_cache = nullptr, *v_cache = nullptr;
  // scratch
  float *x = nullptr, *qkv = nullptr, *q = nullptr, *proj = nullptr, *logits = nullptr, *ones = nullptr, *staging = nullptr;
  __nv_bfloat16 *t = nullptr, *att = nullptr;
  int *tokens_dev = nullptr, *next_dev = nullptr, *iota = nullptr, *dense_off = nullptr, *dense_tbp = nullptr, *status = nullptr;
  int *rows_dev = nullptr;              // cache row of each sequence of a compacted step
  const int *step_rows = nullptr;       // rows_dev during such a step, else null (sequence i lives in cache row i)
  int *pos_dev = nullptr;               // position of each sequence of a step whose sequences started at different times
  const int *step_pos_rows = nullptr;   // pos_dev during such a step, else null (every sequence at step_pos)
  // such a step keeps its sequences ordered by position; [class_end[c-1], class_end[c]) are those with a position below
  // kPosClassEnd[c], and class_pos[c] the largest position among them
  int class_end[3] = {0, 0, 0}, class_pos[3] = {0, 0, 0};
  std::vector<int> perm, sorted_in, sorted_out;  // host scratch of the ordering: [3][max_batch] and [max_batch]
  std::vector<char> row_taken;          // host scratch: cache rows named by the step's sequences (they must be distinct)
  std::vector<int> place;               // after such a step: where the caller's sequence i stands in that order
  bool last_step_ordered = false;       // the last step was one (gptoss_model_read_logits translates its row)
  int cur_B = -1;
  cudaStream_t stream = nullptr;
  bool weights_ready = false;
  std::string err;
  int fail(int code, const char *what, cudaError_t e = cudaSuccess) {
    char buf[512];
    if (e != cudaSuccess)
      snprintf(buf, sizeof buf, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    else
      snprintf(buf, sizeof buf, "%s", what);
    err = buf;
    return code;
  }
  int qkv_dim() const { return c.head_dim * (c.n_attn_heads + 2 * c.n_kv_heads); }
};

#define MK(call)                                                       \
  do {                                                                 \
    cudaError_t e_ = (call);                                           \
    if (e_ != cudaSuccess) return m->fail(GPTOSS_ERR_CUDA, #call, e_); \
  } while (0)

namespace {

constexpr size_t kStagingElems = 16u << 20;  // 64 MiB of fp32

template <typename T>
cudaError_t dalloc(T **p, size_t n) {
  return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(T));
}

// host fp32 -> device bf16 / fp32 through the staging buffer
int upload_bf16(gptoss_model *m, __nv_bfloat16 *dst, const float *src, size_t n) {
  for (size_t o = 0; o < n; o += kStagingElems) {
    const size_t c = n - o < kStagingElems ? n - o : kStagingElems;
    MK(cudaMemcpy(m->staging, src + o, c * sizeof(float), cudaMemcpyHostToDevice));
    MK(launch_f32_to_bf16(m->staging, dst + o, c, 0));
  }
  return GPTOSS_OK;
}
int upload_f32(gptoss_model *m, float *dst, const float *src, size_t n, bool round_bf16) {
  MK(cudaMemcpy(dst, src, n * sizeof(float), cudaMemcpyHostToDevice));
  if (round_bf16) MK(launch_round_bf16_f32(dst, dst, n, 0));
  return GPTOSS_OK;
}

// cos/sin table with YaRN scaling (run.cpp:404-470), float arithmetic as in the reference
void rope_tables(const gptoss_model_config &c, int S, std::vector<float> &cs, std::vector<float> &sn) {
  const int half = c.head_dim / 2;
  std::vector<float> inv(half);
  float concentration = 1.0f;
  const float base = c.rope_theta, scaling = c.rope_scaling_factor, init_ctx = (float)c.initial_context_length;
  const float ntk_beta = 32.0f, ntk_alpha = 1.0f;
  if (scaling > 1.0f) {
    concentration = 0.1f * logf(scaling) + 1.0f;
    const float low = half * logf(init_ctx / (ntk_beta * 2.0f * (float)M_PI)) / logf(base);
    const float high = half * logf(init_ctx / (ntk_alpha * 2.0f * (float)M_PI)) / logf(base);
    for (int i = 0; i < half; ++i) {
      const float freq = powf(base, ((float)(2 * i)) / (float)c.head_dim);
      const float interpolation = 1.0f / (scaling * freq), extrapolation = 1.0f / freq;
      float ramp = ((float)i - low) / (high - low);
      ramp = ramp < 0 ? 0 : (ramp > 1 ? 1 : ramp);
      const float mask = 1.0f - ramp;
      inv[i] = interpolation * (1.0f - mask) + extrapolation * mask;
    }
  } else {
    for (int i = 0; i < half; ++i) inv[i] = 1.0f / powf(base, ((float)(2 * i)) / (float)c.head_dim);
  }
  cs.resize((size_t)S * half);
  sn.resize((size_t)S * half);
  for (int p = 0; p < S; ++p)
    for (int j = 0; j < half; ++j) {
      const float v = (float)p * inv[j];
      cs[(size_t)p * half + j] = cosf(v) * concentration;
      sn[(size_t)p * half + j] = sinf(v) * concentration;
    }
}

// out[B, n_out] (fp32) = act[B, K] (bf16) . W[n_out, K]^T + bias — the down-GEMM kernel with one "expert"
enum { kDenseQkv = 0, kDenseOut = 1, kDenseVocab = 2 };  // which token-block split (dense_tbp) a dense GEMM uses

int dense(gptoss_model *m, int which, const CUtensorMap &map_w, const CUtensorMap &map_act, int K, int n_out,
          const float *bias, float *out) {
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.map_w = map_w;
  a.map_act = map_act;
  a.offsets = m->dense_off;
  a.tb_prefix = m->dense_tbp + 2 * which;
  a.e_begin = 0;
  a.n_local = 1;
  a.n_feat = n_out;
  a.n_feat_tiles = (n_out + kTileF - 1) / kTileF;
  a.k_blocks = (K + kBlockK - 1) / kBlockK;
  a.bias_a = bias;
  a.y_pairs = out;
  a.sorted = m->iota;
  a.topk_w = m->ones;
  a.status = m->status;
  a.n_owners = 1;
  a.top_k = 1;
  a.slice_tokens = m->max_local;
  MK(launch_grouped_mlp2(a, m->sm_count, m->stream));
  return GPTOSS_OK;
}

// Number of token blocks for a dense GEMM of B rows and n_out features: work items = feature tiles x token blocks
// go round-robin over the persistent CTAs, so the time is (rounds of items) x (time of one item).  An item costs
// about its block's rows (at least 64: below that the weight tile's shared-memory reads bound the MMA) plus a
// fixed part (pipeline fill, epilogue), here 32 rows' worth.  More, smaller blocks can fill the last round.
int pick_token_blocks(int B, int n_out, int sm_count) {
  const int nft = n_out <= kTileF ? 1 : (n_out + 2 * kTileF - 1) / (2 * kTileF);  // the dense GEMM works on 256-feature tiles
  const int nb_min = (B + kMaxTileTokens - 1) / kMaxTileTokens;
  int best = nb_min > 0 ? nb_min : 1;
  long best_cost = -1;
  for (int nb = best; nb <= 4 * best && nb <= 64; ++nb) {
    const int blk = (((B + nb - 1) / nb) + 15) & ~15;
    const long rounds = ((long)nft * nb + sm_count - 1) / sm_count;
    const long cost = rounds * ((blk < 64 ? 64 : blk) + 32);
    if (best_cost < 0 || cost < best_cost) best_cost = cost, best = nb;
  }
  return best;
}

int set_batch(gptoss_model *m, int B) {
  if (m->cur_B == B) return GPTOSS_OK;
  const gptoss_model_config &c = m->c;
  const int qkvd = c.head_dim * (c.n_attn_heads + 2 * c.n_kv_heads);
  const int off[2] = {0, B};
  const int tbp[6] = {0, pick_token_blocks(B, qkvd, m->sm_count), 0, pick_token_blocks(B, c.hidden_dim, m->sm_count),
                      0, pick_token_blocks(B, c.vocab_size, m->sm_count)};
  MK(cudaMemcpyAsync(m->dense_off, off, sizeof off, cudaMemcpyHostToDevice, m->stream));
  MK(cudaMemcpyAsync(m->dense_tbp, tbp, sizeof tbp, cudaMemcpyHostToDevice, m->stream));
  MK(cudaStreamSynchronize(m->stream));
  MK(encode_map_2d(&m->map_t, m->t, m->c.hidden_dim, B, (uint32_t)kTokChunk));
  MK(encode_weight_map(&m->map_t_as_w, m->t, m->c.hidden_dim, B, 1));
  MK(encode_map_2d(&m->map_att, m->att, (uint64_t)m->c.head_dim * m->c.n_attn_heads, B, (uint32_t)kTokChunk));
  m->cur_B = B;
  return GPTOSS_OK;
}

}  // namespace

extern "C" {

int gptoss_model_create(const gptoss_model_config *cfg, int device, int max_batch, int max_seq, gptoss_model **out) {
  return gptoss_model_create_ep(cfg, device, 0, 1, max_batch, max_seq, out);
}

int gptoss_model_create_ep(const gptoss_model_config *cfg, int device, int rank, int world, int max_batch, int max_seq,
                           gptoss_model **out) {
  if (!cfg || !out) return GPTOSS_ERR_BAD_ARG;
  *out = nullptr;
  const gptoss_model_config &c = *cfg;
  if (c.vocab_size <= 0 || c.hidden_dim <= 0 || c.hidden_dim % 8 || c.n_layers <= 0 || (c.head_dim != 32 && c.head_dim != 64) ||
      c.n_attn_heads <= 0 || c.n_kv_heads <= 0 || c.n_attn_heads % c.n_kv_heads ||
      (c.n_attn_heads / c.n_kv_heads != 1 && c.n_attn_heads / c.n_kv_heads != 2 && c.n_attn_heads / c.n_kv_heads != 4 &&
       c.n_attn_heads / c.n_kv_heads != 8) || max_batch <= 0 || max_seq <= 0 || max_seq > c.seq_len || world <= 0 ||
      rank < 0 || rank >= world)
    return GPTOSS_ERR_BAD_ARG;
  gptoss_model *m = new (std::nothrow) gptoss_model();
  if (!m) return GPTOSS_ERR_CUDA;
  m->c = c;
  m->device = device;
  m->max_batch = max_batch;
  m->rank = rank;
  m->world = world;
  m->max_local = slice_rows(max_batch, world) < max_batch ? slice_rows(max_batch, world) : max_batch;
  m->S = max_seq;
  gptoss_moe_dims d{c.hidden_dim, c.intermediate_dim, c.n_experts, c.experts_per_token, c.n_layers, c.swiglu_limit};
  int rc = gptoss_ctx_create(&d, device, rank, world, max_batch, GPTOSS_WIRE_F32, &m->moe);
  if (rc) {
    delete m;
    return rc;
  }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, device);
  m->sm_count = prop.multiProcessorCount;
  const size_t L = c.n_layers, H = c.hidden_dim, V = c.vocab_size, B = m->max_local, S = max_seq;
  const size_t qd = (size_t)c.head_dim * c.n_attn_heads, kvd = (size_t)c.head_dim * c.n_kv_heads, qkvd = qd + 2 * kvd;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) {
    if (e == cudaSuccess) e = r;
  };
  A(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  A(dalloc(&m->emb, V * H));
  A(dalloc(&m->unemb, V * H));
  A(dalloc(&m->attn_norm, L * H));
  A(dalloc(&m->mlp_norm, L * H));
  A(dalloc(&m->final_norm, H));
  A(dalloc(&m->w_qkv, L * qkvd * H));
  A(dalloc(&m->b_qkv, L * qkvd));
  A(dalloc(&m->w_o, L * H * qd));
  A(dalloc(&m->b_o, L * H));
  A(dalloc(&m->sinks, L * c.n_attn_heads));
  A(dalloc(&m->cos_t, S * (c.head_dim / 2)));
  A(dalloc(&m->sin_t, S * (c.head_dim / 2)));
  A(dalloc(&m->k_cache, L * B * S * kvd));
  A(dalloc(&m->v_cache, L * B * S * kvd));
  A(dalloc(&m->x, B * H));
  A(dalloc(&m->t, B * H));
  A(dalloc(&m->qkv, B * qkvd));
  A(dalloc(&m->q, B * qd));
  A(dalloc(&m->att, B * qd));
  A(dalloc(&m->proj, B * H));
  m->n_vocab_blocks = (int)((V + kMaxTileTokens - 1) / kMaxTileTokens);
  A(dalloc(&m->logits, V));  // one row, filled on demand by gptoss_model_read_logits
  A(dalloc(&m->amax_val, (size_t)m->n_vocab_blocks * B));
  A(dalloc(&m->amax_at, (size_t)m->n_vocab_blocks * B));
  A(dalloc(&m->amax_sched, 8));
  A(dalloc(&m->tokens_dev, B));
  A(dalloc(&m->next_dev, B));
  A(dalloc(&m->iota, B));
  A(dalloc(&m->rows_dev, B));
  A(dalloc(&m->pos_dev, B));
  A(dalloc(&m->ones, B));
  A(dalloc(&m->dense_off, 2));
  A(dalloc(&m->dense_tbp, 6));
  A(dalloc(&m->status, kStatusWords));
  A(dalloc(&m->staging, kStagingElems));
  if (e == cudaSuccess) A(cudaMemset(m->status, 0, kStatusWords * sizeof(int)));
  if (e == cudaSuccess) A(cudaMemset(m->k_cache, 0, L * B * S * kvd * sizeof(__nv_bfloat16)));
  if (e == cudaSuccess) A(cudaMemset(m->v_cache, 0, L * B * S * kvd * sizeof(__nv_bfloat16)));
  if (e == cudaSuccess) A(launch_iota_ones(m->iota, m->ones, (int)B, 0));
  m->map_qkv.resize(L);
  m->map_o.resize(L);
  for (size_t l = 0; l < L && e == cudaSuccess; ++l) {
    A(encode_weight_map(&m->map_qkv[l], m->w_qkv + l * qkvd * H, H, qkvd, 1));
    A(encode_weight_map(&m->map_o[l], m->w_o + l * H * qd, qd, H, 1));
  }
  if (e == cudaSuccess) A(encode_weight_map(&m->map_unemb, m->unemb, H, V, 1));
  if (e == cudaSuccess) A(encode_map_2d(&m->map_unemb_rows, m->unemb, H, V, (uint32_t)kTokChunk));
  if (e == cudaSuccess) {
    const int sched[8] = {0, (int)V, 0, m->n_vocab_blocks, 0, 1, 0, 1};
    A(cudaMemcpy(m->amax_sched, sched, sizeof sched, cudaMemcpyHostToDevice));
  }
  if (e == cudaSuccess) {
    std::vector<float> cs, sn;
    rope_tables(c, (int)S, cs, sn);
    A(cudaMemcpy(m->cos_t, cs.data(), cs.size() * sizeof(float), cudaMemcpyHostToDevice));
    A(cudaMemcpy(m->sin_t, sn.data(), sn.size() * sizeof(float), cudaMemcpyHostToDevice));
  }
  if (e == cudaSuccess) A(cudaDeviceSynchronize());
  if (e != cudaSuccess) {
    gptoss_model_destroy(m);
    return GPTOSS_ERR_CUDA;
  }
  *out = m;
  return GPTOSS_OK;
}

int gptoss_model_destroy(gptoss_model *m) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  cudaSetDevice(m->device);
  cudaDeviceSynchronize();
  if (m->moe) gptoss_ctx_destroy(m->moe);
  void *ptrs[] = {m->emb, m->unemb, m->attn_norm, m->mlp_norm, m->final_norm, m->w_qkv, m->b_qkv, m->w_o, m->b_o, m->sinks,
                  m->cos_t, m->sin_t, m->k_cache, m->v_cache, m->x, m->t, m->qkv, m->q, m->att, m->proj, m->logits,
                  m->tokens_dev, m->next_dev, m->iota, m->rows_dev, m->pos_dev, m->amax_val, m->amax_at, m->amax_sched, m->ones, m->dense_off, m->dense_tbp, m->status, m->staging};
  for (void *p : ptrs) cudaFree(p);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
  return GPTOSS_OK;
}

const char *gptoss_model_last_error(const gptoss_model *m) {
  if (!m) return "null model";
  if (!m->err.empty()) return m->err.c_str();
  return gptoss_last_error(m->moe);
}

// Loads every tensor of a flat checkpoint image already in host memory (header + fp32 tensors in the order of
// run.cpp:194-233), e.g. the mapping the reference's load_checkpoint made (Transformer::data, run.cpp:274);
// the header must match the configuration the model was created with.
int gptoss_model_load_mem(gptoss_model *m, const void *image, uint64_t bytes) {
  if (!m || !image) return GPTOSS_ERR_BAD_ARG;
  MK(cudaSetDevice(m->device));
  int rc = GPTOSS_OK;
  const gptoss_model_config &c = m->c;
  gptoss_model_config hdr;
  if (bytes < sizeof hdr) return m->fail(GPTOSS_ERR_BAD_ARG, "checkpoint image shorter than its header");
  memcpy(&hdr, image, sizeof hdr);
  const size_t L = c.n_layers, H = c.hidden_dim, V = c.vocab_size, E = c.n_experts, I = c.intermediate_dim;
  const size_t qd = (size_t)c.head_dim * c.n_attn_heads, kvd = (size_t)c.head_dim * c.n_kv_heads, qkvd = qd + 2 * kvd;
  const size_t need = sizeof hdr + 4 * (2 * V * H + 2 * L * H + H + L * qkvd * H + L * qkvd + L * H * qd + L * H +
                                        L * c.n_attn_heads + L * E * H + L * E + L * E * 2 * I * H + L * E * 2 * I +
                                        L * E * H * I + L * E * H);
  if (memcmp(&hdr, &c, 9 * sizeof(int)) != 0 || hdr.sliding_window != c.sliding_window || bytes != need)
    return m->fail(GPTOSS_ERR_BAD_ARG, "checkpoint header or size does not match the model configuration");
  const float *p = reinterpret_cast<const float *>(static_cast<const char *>(image) + sizeof hdr);
  auto take = [&](size_t n) {
    const float *r = p;
    p += n;
    return r;
  };
  const float *emb = take(V * H), *unemb = take(V * H), *an = take(L * H), *mn = take(L * H), *fn = take(H);
  const float *wqkv = take(L * qkvd * H), *bqkv = take(L * qkvd), *wo = take(L * H * qd), *bo = take(L * H);
  const float *sinks = take(L * c.n_attn_heads), *wr = take(L * E * H), *br = take(L * E);
  const float *w1 = take(L * E * 2 * I * H), *b1 = take(L * E * 2 * I), *w2 = take(L * E * H * I), *b2 = take(L * E * H);
  if (!rc) rc = upload_bf16(m, m->emb, emb, V * H);
  if (!rc) rc = upload_bf16(m, m->unemb, unemb, V * H);
  if (!rc) rc = upload_f32(m, m->attn_norm, an, L * H, false);  // norm scales stay fp32 (alloc.cpp:17)
  if (!rc) rc = upload_f32(m, m->mlp_norm, mn, L * H, false);
  if (!rc) rc = upload_f32(m, m->final_norm, fn, H, false);
  if (!rc) rc = upload_bf16(m, m->w_qkv, wqkv, L * qkvd * H);
  if (!rc) rc = upload_f32(m, m->b_qkv, bqkv, L * qkvd, true);
  if (!rc) rc = upload_bf16(m, m->w_o, wo, L * H * qd);
  if (!rc) rc = upload_f32(m, m->b_o, bo, L * H, true);
  if (!rc) rc = upload_f32(m, m->sinks, sinks, L * c.n_attn_heads, true);
  for (size_t l = 0; l < L && !rc; ++l) {
    rc = gptoss_upload_layer(m->moe, (int)l, wr + l * E * H, br + l * E, w1 + l * E * 2 * I * H, b1 + l * E * 2 * I,
                             w2 + l * E * H * I, b2 + l * E * H);
    if (rc) m->fail(rc, gptoss_last_error(m->moe));
  }
  cudaDeviceSynchronize();
  if (!rc) m->weights_ready = true;
  return rc;
}

// load_checkpoint (run.cpp:235-281): maps the file and loads it.
int gptoss_model_load_bin(gptoss_model *m, const char *path) {
  if (!m || !path) return GPTOSS_ERR_BAD_ARG;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return m->fail(GPTOSS_ERR_BAD_ARG, "cannot open checkpoint");
  struct stat st;
  fstat(fd, &st);
  void *map = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return m->fail(GPTOSS_ERR_BAD_ARG, "mmap of checkpoint failed");
  const int rc = gptoss_model_load_mem(m, map, (uint64_t)st.st_size);
  munmap(map, st.st_size);
  return rc;
}

// Random-init weights generated on the device (N(0, sigma) rounded to bf16, RMSNorm scales 1.0); meant for
// throughput runs of architectures whose checkpoint would not fit on the host.
int gptoss_model_fill_synthetic(gptoss_model *m, uint64_t seed, float sigma) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  MK(cudaSetDevice(m->device));
  const gptoss_model_config &c = m->c;
  const size_t L = c.n_layers, H = c.hidden_dim, V = c.vocab_size;
  const size_t qd = (size_t)c.head_dim * c.n_attn_heads, kvd = (size_t)c.head_dim * c.n_kv_heads, qkvd = qd + 2 * kvd;
  MK(launch_synth_normal(m->emb, V * H, seed, 64, 0, sigma, 0));
  MK(launch_synth_normal(m->unemb, V * H, seed, 65, 0, sigma, 0));
  std::vector<float> ones((L * H > H ? L * H : H), 1.0f);
  MK(cudaMemcpy(m->attn_norm, ones.data(), L * H * sizeof(float), cudaMemcpyHostToDevice));
  MK(cudaMemcpy(m->mlp_norm, ones.data(), L * H * sizeof(float), cudaMemcpyHostToDevice));
  MK(cudaMemcpy(m->final_norm, ones.data(), H * sizeof(float), cudaMemcpyHostToDevice));
  MK(launch_synth_normal(m->w_qkv, L * qkvd * H, seed, 69, 0, sigma, 0));
  MK(launch_synth_normal_f32(m->b_qkv, L * qkvd, seed, 70, 0, sigma, 0));
  MK(launch_synth_normal(m->w_o, L * H * qd, seed, 71, 0, sigma, 0));
  MK(launch_synth_normal_f32(m->b_o, L * H, seed, 72, 0, sigma, 0));
  MK(launch_synth_normal_f32(m->sinks, L * c.n_attn_heads, seed, 73, 0, sigma, 0));
  for (size_t l = 0; l < L; ++l) {
    int rc = gptoss_fill_layer_synthetic(m->moe, (int)l, seed, sigma);
    if (rc) return m->fail(rc, gptoss_last_error(m->moe));
  }
  MK(cudaDeviceSynchronize());
  m->weights_ready = true;
  return GPTOSS_OK;
}

// ---- one lock-step decode step, in phases -------------------------------------------------------------------
// gptoss_model_step runs them in order; they are separate entry points so that a host can interleave the ranks of
// an expert-parallel group itself (several model objects driven by one thread, e.g. on one device in a test).
//   step_begin         tokens of this rank's sequences -> embedding rows (the residual stream)
//   layer_attention    RMSNorm -> QKV GEMM -> RoPE + KV store -> attention -> o-proj GEMM -> residual + RMSNorm
//                      (expert-parallel: then the routing of this rank's rows, shared with every rank)
//   layer_moe_dispatch expert-parallel only: grouping of the whole batch from everybody's routing rows; this rank's
//                      rows go to the ranks whose experts they selected
//   layer_moe_push     one GPU: the whole MoE block.  Expert-parallel: expert GEMMs of this rank's experts on the rows
//                      it received, outputs pushed to the tokens' owners
//   layer_moe_combine  expert-parallel only: slot-ordered sum of the pushed rows into this rank's residual rows
//   step_end           final RMSNorm -> classifier GEMM -> argmax -> next tokens of this rank's sequences
int gptoss_model_slice(const gptoss_model *m, int B, int *first, int *count) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  return gptoss_moe_slice_bounds(m->moe, B, first, count);
}

gptoss_ctx *gptoss_model_moe_ctx(gptoss_model *m) { return m ? m->moe : nullptr; }

int gptoss_model_step_begin(gptoss_model *m, const int *tokens_host, int pos, int B) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (B <= 0 || B > m->max_batch || pos < 0 || pos >= m->S) return m->fail(GPTOSS_ERR_BAD_ARG, "batch or position out of range");
  if (!m->weights_ready) return m->fail(GPTOSS_ERR_STATE, "model has no weights yet");
  MK(cudaSetDevice(m->device));
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(m->moe, B, &first, &n);
  if (n > 0 && !tokens_host) return m->fail(GPTOSS_ERR_BAD_ARG, "null token pointer");
  m->step_B = B, m->step_pos = pos, m->step_first = first, m->step_n = n;
  m->step_rows = nullptr;
  m->step_pos_rows = nullptr;
  m->last_step_ordered = false;
  if (n == 0) return GPTOSS_OK;
  int rc = set_batch(m, n);
  if (rc) return rc;
  MK(cudaMemcpyAsync(m->tokens_dev, tokens_host, n * sizeof(int), cudaMemcpyHostToDevice, m->stream));
  MK(launch_embed(m->tokens_dev, m->emb, n, m->c.hidden_dim, m->c.vocab_size, m->x, m->stream));
  return GPTOSS_OK;
}

int gptoss_model_layer_attention(gptoss_model *m, int layer) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (layer < 0 || layer >= m->c.n_layers || m->step_B <= 0) return m->fail(GPTOSS_ERR_STATE, "no step in progress or bad layer");
  MK(cudaSetDevice(m->device));
  const gptoss_model_config &c = m->c;
  const size_t l = layer, H = c.hidden_dim, S = m->S;
  const int nq = c.n_attn_heads, nkv = c.n_kv_heads, hd = c.head_dim, B = m->step_n, pos = m->step_pos;
  const size_t qd = (size_t)hd * nq, kvd = (size_t)hd * nkv, qkvd = qd + 2 * kvd;
  cudaStream_t s = m->stream;
  int rc;
  if (B > 0) {
    MK(launch_residual_rmsnorm(m->x, nullptr, m->attn_norm + l * H, B, (int)H, m->t, s));
    if ((rc = dense(m, kDenseQkv, m->map_qkv[l], m->map_t, (int)H, (int)qkvd, m->b_qkv + l * qkvd, m->qkv))) return rc;
    __nv_bfloat16 *kc = m->k_cache + l * (size_t)m->max_local * S * kvd, *vc = m->v_cache + l * (size_t)m->max_local * S * kvd;
    MK(launch_qkv_rope_store(m->qkv, m->cos_t, m->sin_t, pos, B, nq, nkv, hd, (int)S, m->q, kc, vc, m->step_rows,
                             m->step_pos_rows, s));
    const bool windowed = c.sliding_window > 0 && (l % 2 == 0);  // run.cpp:582
    const int window = windowed ? c.sliding_window : 0;
    if (!m->step_pos_rows) {
      const int t_lo = windowed && pos - window + 1 > 0 ? pos - window + 1 : 0;
      MK(launch_attention(m->q, kc, vc, m->sinks + l * nq, pos, t_lo, B, nq, nkv, hd, (int)S, m->att, m->step_rows, nullptr, 0, s));
    } else {
      // sequences at their own positions, ordered by position: one launch per run of sequences whose contexts (the
      // window applied) ask for the same number of warps per problem, so every sequence is summed in the order a
      // lock-step batch at its position would use
      int b0 = 0;
      while (b0 < B) {
        int cls = 0;
        while (m->class_end[cls] <= b0) ++cls;
        const auto span_of = [&](int p) { return windowed && p > window - 1 ? window - 1 : p; };
        const int warps = attention_warps_per_problem(span_of(m->class_pos[cls]));
        int b1 = m->class_end[cls], span = span_of(m->class_pos[cls]);
        for (int nx = cls + 1; nx < 3; ++nx) {  // following classes that the window folds into the same split
          if (m->class_end[nx] == b1) continue;
          if (attention_warps_per_problem(span_of(m->class_pos[nx])) != warps) break;
          b1 = m->class_end[nx];
          span = span_of(m->class_pos[nx]);
        }
        MK(launch_attention(m->q + (size_t)b0 * qd, kc, vc, m->sinks + l * nq, span, 0, b1 - b0, nq, nkv, hd, (int)S,
                            m->att + (size_t)b0 * qd, m->step_rows + b0, m->step_pos_rows + b0, window, s));
        b0 = b1;
      }
    }
    if ((rc = dense(m, kDenseOut, m->map_o[l], m->map_att, (int)qd, (int)H, m->b_o + l * H, m->proj))) return rc;
  }
  if (m->world == 1) {
    MK(launch_residual_rmsnorm(m->x, m->proj, m->mlp_norm + l * H, B, (int)H, m->t, s));
  } else {  // this rank normalises and routes its own rows and shares the routing rows with every rank
    if (B > 0) MK(launch_residual_rmsnorm(m->x, m->proj, m->mlp_norm + l * H, B, (int)H, m->t, s));
    if ((rc = gptoss_moe_dispatch_route(m->moe, layer, m->step_B, m->t, s))) return m->fail(rc, gptoss_last_error(m->moe));
  }
  return GPTOSS_OK;
}

int gptoss_model_layer_moe_dispatch(gptoss_model *m, int layer) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (layer < 0 || layer >= m->c.n_layers || m->step_B <= 0) return m->fail(GPTOSS_ERR_STATE, "no step in progress or bad layer");
  if (m->world == 1) return GPTOSS_OK;
  const int rc = gptoss_moe_dispatch_rows(m->moe, layer, m->step_B, m->t, m->stream);
  return rc ? m->fail(rc, gptoss_last_error(m->moe)) : GPTOSS_OK;
}

int gptoss_model_layer_moe_push(gptoss_model *m, int layer) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (layer < 0 || layer >= m->c.n_layers || m->step_B <= 0) return m->fail(GPTOSS_ERR_STATE, "no step in progress or bad layer");
  const int rc = m->world == 1 ? gptoss_moe_forward(m->moe, layer, m->step_B, m->t, m->x, m->stream)
                               : gptoss_moe_dispatch_push(m->moe, layer, m->stream);
  return rc ? m->fail(rc, gptoss_last_error(m->moe)) : GPTOSS_OK;
}

int gptoss_model_layer_moe_combine(gptoss_model *m, int layer) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (layer < 0 || layer >= m->c.n_layers || m->step_B <= 0) return m->fail(GPTOSS_ERR_STATE, "no step in progress or bad layer");
  if (m->world == 1) return GPTOSS_OK;
  const int rc = gptoss_moe_sliced_combine(m->moe, m->x, m->stream);
  return rc ? m->fail(rc, gptoss_last_error(m->moe)) : GPTOSS_OK;
}

int gptoss_model_step_end(gptoss_model *m, int *next_tokens_host) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (m->step_B <= 0) return m->fail(GPTOSS_ERR_STATE, "no step in progress");
  MK(cudaSetDevice(m->device));
  const gptoss_model_config &c = m->c;
  const int B = m->step_n, H = c.hidden_dim;
  cudaStream_t s = m->stream;
  int rc;
  if (next_tokens_host && B > 0) {  // a step whose outputs are all overridden by prompt tokens needs no logits
    MK(launch_residual_rmsnorm(m->x, nullptr, m->final_norm, B, H, m->t, s));
    // classifier + greedy argmax in one GEMM (layer_hip_batch.cpp:1465-1712 + sample_argmax, run.cpp:739-750): the
    // sequences are the MMA's M side, blocks of 256 vocabulary rows its N side, and the epilogue keeps one
    // (max, id) per (vocabulary block, sequence) instead of storing B x V logits; a small kernel merges the blocks
    GemmArgs a;
    memset(&a, 0, sizeof a);
    a.map_w = m->map_t_as_w;
    a.map_act = m->map_unemb_rows;
    a.offsets = m->amax_sched;
    a.tb_prefix = m->amax_sched + 2;
    a.n_local = 1;
    a.n_feat = B;
    a.k_blocks = (H + kBlockK - 1) / kBlockK;
    a.status = m->status;
    a.n_owners = 1;
    a.top_k = 1;
    a.slice_tokens = m->max_local;
    // (the argmax kernel orders its items with the sequence tile fastest: the tiles of one vocabulary block run side
    // by side and share its rows in L2)
    a.amax_val = m->amax_val;
    a.amax_at = m->amax_at;
    MK(launch_grouped_amax(a, m->sm_count, s));
    MK(launch_argmax_partials(m->amax_val, m->amax_at, m->n_vocab_blocks, B, m->next_dev, s));
    MK(cudaMemcpyAsync(next_tokens_host, m->next_dev, B * sizeof(int), cudaMemcpyDeviceToHost, s));
  }
  int st[kStatusWords];
  MK(cudaMemcpyAsync(st, m->status, sizeof st, cudaMemcpyDeviceToHost, s));
  MK(cudaStreamSynchronize(s));
  m->step_B = 0;
  if (st[0] != 0) {
    cudaMemset(m->status, 0, sizeof st);
    return m->fail(GPTOSS_ERR_TIMEOUT, "device-side bounded wait gave up in a dense GEMM");
  }
  rc = gptoss_ctx_status(m->moe);
  return rc ? m->fail(rc, gptoss_last_error(m->moe)) : GPTOSS_OK;
}

// One lock-step decode step: tokens of this rank's sequences at position `pos` -> their greedy next tokens
// (forward_gpu_20b_batched / forward_gpu_120b_batched, getp-csrc/src/model.cpp:6-151,153-489; CPU: forward +
// sample_argmax, run.cpp:501,739).  B is the batch of the whole group.
int gptoss_model_step(gptoss_model *m, const int *tokens_host, int pos, int B, int *next_tokens_host) {
  int rc = gptoss_model_step_begin(m, tokens_host, pos, B);
  for (int l = 0; !rc && l < m->c.n_layers; ++l) {
    if ((rc = gptoss_model_layer_attention(m, l))) break;
    if ((rc = gptoss_model_layer_moe_dispatch(m, l))) break;
    if ((rc = gptoss_model_layer_moe_push(m, l))) break;
    rc = gptoss_model_layer_moe_combine(m, l);
  }
  if (rc) {
    if (m) m->step_B = 0;
    return rc;
  }
  return gptoss_model_step_end(m, next_tokens_host);
}

// The same step for a batch from which finished sequences were dropped (dead-sequence compaction of the lock-step
// scheduler): n live sequences, sequence i keeps the KV-cache row rows_host[i] it has had since position 0.  Every
// kernel of the step works on n rows; only the cache accesses go through the row map.
int gptoss_model_step_rows(gptoss_model *m, const int *tokens_host, const int *rows_host, int pos, int n, int *next_tokens_host) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (m->world != 1) return m->fail(GPTOSS_ERR_UNSUPPORTED, "compacted steps are for a single-GPU model (a group keeps its slices)");
  if (!rows_host) return m->fail(GPTOSS_ERR_BAD_ARG, "null row map");
  if (n <= 0 || n > m->max_batch) return m->fail(GPTOSS_ERR_BAD_ARG, "batch out of range");
  m->row_taken.assign(m->max_batch, 0);
  for (int i = 0; i < n; ++i) {
    if (rows_host[i] < 0 || rows_host[i] >= m->max_batch) return m->fail(GPTOSS_ERR_BAD_ARG, "cache row out of range");
    if (m->row_taken[rows_host[i]]++) return m->fail(GPTOSS_ERR_BAD_ARG, "two sequences name the same cache row");
  }
  int rc = gptoss_model_step_begin(m, tokens_host, pos, n);
  if (rc) return rc;
  MK(cudaMemcpyAsync(m->rows_dev, rows_host, n * sizeof(int), cudaMemcpyHostToDevice, m->stream));
  m->step_rows = m->rows_dev;
  for (int l = 0; !rc && l < m->c.n_layers; ++l) {
    if ((rc = gptoss_model_layer_attention(m, l))) break;
    rc = gptoss_model_layer_moe_push(m, l);
  }
  if (rc) {
    m->step_B = 0;
    m->step_rows = nullptr;
    return rc;
  }
  rc = gptoss_model_step_end(m, next_tokens_host);
  m->step_rows = nullptr;
  return rc;
}

// The same step for sequences that did not start together (continuous batching: a sequence that finished hands its
// cache row to a waiting request, which starts at position 0 while its batch mates carry on): sequence i holds cache row
// rows_host[i] and is at position pos_host[i].  Only RoPE and attention look at positions; they take them per sequence.
// Internally the sequences are ordered by position, so that attention runs each class of context lengths with the
// warp split a lock-step batch of that length gets; a sequence's result does not depend on who shares the batch.
int gptoss_model_step_seqs(gptoss_model *m, const int *tokens_host, const int *rows_host, const int *pos_host, int n,
                           int *next_tokens_host) {
  if (!m) return GPTOSS_ERR_BAD_ARG;
  if (m->world != 1) return m->fail(GPTOSS_ERR_UNSUPPORTED, "per-sequence positions are for a single-GPU model (a group steps in lock-step)");
  if (!tokens_host || !rows_host || !pos_host) return m->fail(GPTOSS_ERR_BAD_ARG, "null token, row or position pointer");
  if (n <= 0 || n > m->max_batch) return m->fail(GPTOSS_ERR_BAD_ARG, "batch out of range");
  // class c: positions whose full-context attention uses 1, 2, 4 warps per problem
  const auto class_of = [](int p) { const int w = attention_warps_per_problem(p); return w == 1 ? 0 : (w == 2 ? 1 : 2); };
  int count[3] = {0, 0, 0}, max_pos = 0;
  m->row_taken.assign(m->max_batch, 0);
  for (int i = 0; i < n; ++i) {
    if (rows_host[i] < 0 || rows_host[i] >= m->max_batch) return m->fail(GPTOSS_ERR_BAD_ARG, "cache row out of range");
    if (m->row_taken[rows_host[i]]++) return m->fail(GPTOSS_ERR_BAD_ARG, "two sequences name the same cache row");
    if (pos_host[i] < 0 || pos_host[i] >= m->S) return m->fail(GPTOSS_ERR_BAD_ARG, "position out of range");
    ++count[class_of(pos_host[i])];
    if (pos_host[i] > max_pos) max_pos = pos_host[i];
  }
  const size_t B = (size_t)m->max_batch;
  m->perm.resize(B), m->sorted_in.resize(3 * B), m->sorted_out.resize(B);
  int at[3] = {0, count[0], count[0] + count[1]};
  m->class_end[0] = count[0], m->class_end[1] = count[0] + count[1], m->class_end[2] = n;
  m->class_pos[0] = m->class_pos[1] = m->class_pos[2] = 0;
  int *tok_s = m->sorted_in.data(), *row_s = tok_s + B, *pos_s = row_s + B;
  for (int i = 0; i < n; ++i) {
    const int c = class_of(pos_host[i]), j = at[c]++;
    m->perm[j] = i;
    tok_s[j] = tokens_host[i], row_s[j] = rows_host[i], pos_s[j] = pos_host[i];
    if (pos_host[i] > m->class_pos[c]) m->class_pos[c] = pos_host[i];
  }
  int rc = gptoss_model_step_begin(m, tok_s, max_pos, n);
  if (rc) return rc;
  MK(cudaMemcpyAsync(m->rows_dev, row_s, n * sizeof(int), cudaMemcpyHostToDevice, m->stream));
  MK(cudaMemcpyAsync(m->pos_dev, pos_s, n * sizeof(int), cudaMemcpyHostToDevice, m->stream));
  m->step_rows = m->rows_dev;
  m->step_pos_rows = m->pos_dev;
  for (int l = 0; !rc && l < m->c.n_layers; ++l) {
    if ((rc = gptoss_model_layer_attention(m, l))) break;
    rc = gptoss_model_layer_moe_push(m, l);
  }
  if (!rc) rc = gptoss_model_step_end(m, next_tokens_host ? m->sorted_out.data() : nullptr);
  m->step_B = 0;
  m->step_rows = nullptr;
  m->step_pos_rows = nullptr;
  if (rc) return rc;
  if (next_tokens_host)
    for (int j = 0; j < n; ++j) next_tokens_host[m->perm[j]] = m->sorted_out[j];
  m->place.assign(B, -1);
  for (int j = 0; j < n; ++j) m->place[m->perm[j]] = j;
  m->last_step_ordered = true;
  return GPTOSS_OK;
}

// Logits of one sequence of the last step that produced tokens (debug/parity tap).  The step itself never stores
// logits (the classifier's epilogue keeps only the argmax), so they are computed here for the one row asked for:
// the classifier GEMM on that row of the final-norm output, which the step left in place.
int gptoss_model_read_logits(gptoss_model *m, int row, float *host_out) {
  if (!m || !host_out) return GPTOSS_ERR_BAD_ARG;
  if (row < 0 || row >= m->max_local) return m->fail(GPTOSS_ERR_BAD_ARG, "row out of range");
  if (m->last_step_ordered && (row = m->place[row]) < 0) return m->fail(GPTOSS_ERR_BAD_ARG, "row was not part of the last step");
  MK(cudaSetDevice(m->device));
  const int H = m->c.hidden_dim, V = m->c.vocab_size;
  CUtensorMap map_row;
  MK(encode_map_2d(&map_row, m->t + (size_t)row * H, H, 1, (uint32_t)kTokChunk));
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.map_w = m->map_unemb;
  a.map_act = map_row;
  a.offsets = m->amax_sched + 4;
  a.tb_prefix = m->amax_sched + 6;
  a.n_local = 1;
  a.n_feat = V;
  a.n_feat_tiles = (V + kTileF - 1) / kTileF;
  a.k_blocks = (H + kBlockK - 1) / kBlockK;
  a.y_pairs = m->logits;
  a.sorted = m->iota;
  a.topk_w = m->ones;
  a.status = m->status;
  a.n_owners = 1;
  a.top_k = 1;
  a.slice_tokens = m->max_local;
  MK(launch_grouped_mlp2(a, m->sm_count, m->stream));
  MK(cudaMemcpyAsync(host_out, m->logits, (size_t)V * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
  MK(cudaStreamSynchronize(m->stream));
  return GPTOSS_OK;
}

}  // extern "C"
