// extern "C" entry points of gptoss_b200 (declared in include/gptoss_b200.h): context, weights, the
// per-layer MoE operator and its stages, taps.  No call aborts or throws; every failure is a status
// code plus a message retrievable with gptoss_last_error().
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "kernels.cuh"

using namespace gptoss;

namespace {

// tensor-stream ids of the synthetic generator (kind + 16 * layer), shared with the Python module `synth`
enum { kTidRouterW = 2, kTidRouterB = 3, kTidMlp1W = 4, kTidMlp1B = 5, kTidMlp2W = 6, kTidMlp2B = 7 };

struct LayerWeights {
  __nv_bfloat16 *router_w = nullptr;  // [E,H]
  float *router_b = nullptr;          // [E]
  __nv_bfloat16 *w1 = nullptr;        // [E_local][2][I][H]   gate rows, then up rows
  float *b1g = nullptr, *b1u = nullptr;  // [E_local][I]
  __nv_bfloat16 *w2 = nullptr;        // [E_local][H][I]
  float *b2 = nullptr;                // [E_local][H]
  CUtensorMap map_w1, map_w2, map_wr;
  bool ready = false;
};

}  // namespace

struct gptoss_ctx {
  gptoss_moe_dims dims;
  Dims d;
  int device = 0, rank = 0, world = 1, max_tokens = 0, wire = 0;
  int n_local = 0, sm_count = kSmCountFallback;
  int cur_T = 0;
  RouteBuffers rb{};
  __nv_bfloat16 *x_packed = nullptr;  // [P,H]   (inside `sym`: peers dispatch token rows into it)
  __nv_bfloat16 *gate_up = nullptr;   // [P,I]
  float *y_pairs = nullptr;           // [P,H]   (inside `sym`)
  // symmetric buffer: same layout on every rank, exported to the peers over CUDA IPC
  //   [flags: 4*kMaxRanks ints, padded to 1 KiB][delta: T*H fp32][y_pairs: P*H fp32][topk_w: P fp32][topk_i: P i32]
  //   [blk_hist: n_route_blocks*E i32][x_packed: P*H bf16]
  uint8_t *sym = nullptr;
  size_t sym_bytes = 0, sym_delta_off = 0, sym_y_off = 0, sym_tw_off = 0, sym_ti_off = 0, sym_hist_off = 0, sym_xp_off = 0, sym_sorted_off = 0;
  RowDispatch rows_self{};            // token rows go to this rank's x_packed (its own experts only) ...
  RowDispatch rows_all{};             // ... or to the x_packed of the expert's owner (filled when peers are attached)
  TileBalance balance{};              // how expert_scan_kernel cuts the experts' rows into token blocks
  bool pair_policy = false;           // expert GEMMs on pairs of CTAs (GPTOSS_PAIR=1)
  int balance_pushing_gemm = -1;      // size the token blocks of a group's down GEMM too: -1 by the number of local experts, 0 / 1 forced
  bool pair_mode = false;             // the routed batch's GEMMs run on pairs (decided when the batch is grouped)
  bool pushed_bf16 = false;           // the rows of the last push travelled as bf16 (token-sliced forms on the bf16 wire)
  bool group_broken = false;          // a wait on a peer gave up: the ranks' step counters no longer match
  RouteShare share_self{};            // where routing rows go: this rank alone ...
  RouteShare share{};                 // ... or every rank of the group (filled when peers are attached)
  int route_step = 0;                 // number of shared routings so far (flag D carries it)
  bool share_routing = false;         // GPTOSS_SHARED_ROUTING=1: each rank routes its token slice only and shares the rows
                                      // (off by default: measured neutral, the replicated scatter/gather dominates the stage)
  int *comm_counter = nullptr;        // last-block counter of the owner combine
  void *peer_base[kMaxRanks] = {};    // opened IPC mappings (nullptr for the own rank / not attached)
  PeerTable peers{};
  bool attached = false;
  int comm_step = 0;
  int gather_step = 0;  // token-sliced form: number of slice gathers so far (flag C carries it)
  int pending_gather = 0;  // gather step the next route_finish has to wait for (0 = none)
  int *status = nullptr;              // [kStatusWords]
  // Host-buffer entry points: two sets of device copies, so that a second call can be submitted (its uploads and
  // kernels running) while the first one's result is still on its way back to the host
  struct HostSlot {
    __nv_bfloat16 *t = nullptr;       // [max_tokens,H]
    float *x = nullptr;               // [max_tokens,H]
    int *status_host = nullptr;       // pinned copy of the status words, read back behind the result
    cudaEvent_t ev_t = nullptr, ev_x = nullptr, ev_done = nullptr, ev_out = nullptr;
    bool busy = false;
  } hslot[2];
  int h_head = 0, h_tail = 0;         // slot of the next submit / of the oldest call not yet waited for
  cudaStream_t s_out = nullptr;       // device -> host copies of the results
  float *router_partials = nullptr;   // [kRouterMaxSplits][max_tokens][E] split-K partial scores
  CUtensorMap map_t;                  // tensor map of the caller's activations (re-encoded when they move)
  const void *map_t_base = nullptr;
  int map_t_rows = -1;
  cudaStream_t s_main = nullptr, s_copy = nullptr;  // kernels / host -> device copies of the host-buffer entry points (created on first use)
  float *staging = nullptr;           // fp32 scratch for weight conversion
  size_t staging_elems = 0;
  CUtensorMap map_x, map_h;
  std::vector<LayerWeights> layers;
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
};

#define CK(call)                                                          \
  do {                                                                    \
    cudaError_t e_ = (call);                                              \
    if (e_ != cudaSuccess) return ctx->fail(GPTOSS_ERR_CUDA, #call, e_); \
  } while (0)

namespace {

template <typename T>
cudaError_t dev_alloc(T **p, size_t n) {
  return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(T));
}

int ensure_staging(gptoss_ctx *ctx, size_t elems) {
  if (ctx->staging_elems >= elems) return GPTOSS_OK;
  if (ctx->staging) cudaFree(ctx->staging);
  ctx->staging = nullptr;
  ctx->staging_elems = 0;
  CK(dev_alloc(&ctx->staging, elems));
  ctx->staging_elems = elems;
  return GPTOSS_OK;
}

int check_layer(gptoss_ctx *ctx, int layer, bool need_ready) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (layer < 0 || layer >= ctx->dims.n_layers) return ctx->fail(GPTOSS_ERR_BAD_ARG, "layer index out of range");
  if (need_ready && !ctx->layers[layer].ready) return ctx->fail(GPTOSS_ERR_STATE, "layer has no weights yet");
  return GPTOSS_OK;
}

int alloc_layer(gptoss_ctx *ctx, LayerWeights &w) {
  if (w.router_w) return GPTOSS_OK;
  const size_t H = ctx->d.H, I = ctx->d.I, E = ctx->d.E, EL = ctx->n_local;
  CK(dev_alloc(&w.router_w, E * H));
  CK(dev_alloc(&w.router_b, E));
  CK(dev_alloc(&w.w1, EL * 2 * I * H));
  CK(dev_alloc(&w.b1g, EL * I));
  CK(dev_alloc(&w.b1u, EL * I));
  CK(dev_alloc(&w.w2, EL * H * I));
  CK(dev_alloc(&w.b2, EL * H));
  CK(encode_weight_map(&w.map_w1, w.w1, H, I, EL * 2));
  CK(encode_weight_map(&w.map_w2, w.w2, I, H, EL));
  CK(encode_map_2d(&w.map_wr, w.router_w, H, E, (uint32_t)((E + 15) & ~(size_t)15)));
  return GPTOSS_OK;
}

void free_layer(LayerWeights &w) {
  cudaFree(w.router_w);
  cudaFree(w.router_b);
  cudaFree(w.w1);
  cudaFree(w.b1g);
  cudaFree(w.b1u);
  cudaFree(w.w2);
  cudaFree(w.b2);
  w = LayerWeights();
}

int check_T(gptoss_ctx *ctx, int T) {
  if (T < 0 || T > ctx->max_tokens) return ctx->fail(GPTOSS_ERR_BAD_ARG, "T outside [0, max_tokens]");
  return GPTOSS_OK;
}

// Fixes, for the batch about to be grouped, whether its expert GEMMs run on pairs of CTAs, and returns the parameters
// with which expert_scan_kernel sizes the token blocks for that choice.  The pair kernels (tcgen05 cta_group::2) give
// the same bits and, measured from 128 to 1024 rows per expert, the same time or a few per cent more than one CTA per
// item (the GEMMs are bound by the tensor pipe under the board's power cap, not by what a CTA stages), so they run
// only on request: GPTOSS_PAIR=1.
TileBalance balance_for(gptoss_ctx *ctx) {
  ctx->pair_mode = ctx->pair_policy && ctx->d.H > kTileF;  // the one-tile down GEMM has no pair form
  TileBalance b = ctx->balance;
  const int H = ctx->d.H, I = ctx->d.I;
  if (ctx->pair_mode) {
    b.ctas = ctx->sm_count / 2;
    b.nft1 = (I + 2 * kTileF - 1) / (2 * kTileF);
    b.nft2 = (H + 4 * kTileF - 1) / (4 * kTileF);
    b.fixed_rows = 2 * kMaxTileTokens;  // a CTA stages two weight tiles (as many bytes as 256 token rows) and HALF the block's rows
  } else {
    b.ctas = ctx->sm_count;
    b.nft1 = (I + kTileF - 1) / kTileF;
    b.nft2 = H <= kTileF ? 1 : (H + 2 * kTileF - 1) / (2 * kTileF);
    b.fixed_rows = kMaxTileTokens;
  }
  // The down GEMM of a group of GPUs stores its rows to their owners over NVLink from its epilogue, which makes more,
  // smaller items dearer than the model knows.  Measured on real GPUs: with 16 local experts (2 GPUs) the balanced
  // blocks lose (96 us against 92.5, although they win without the push: 86 against 97), with 4 local experts (8
  // GPUs), where the fill of the rounds matters most, they win (gate/up + down with push 198 us against 207), with 8
  // (4 GPUs) it makes no difference (213-214 against 216).  So the down GEMM is balanced up to 4 local experts and keeps
  // blocks of 256 rows beyond (no items: every size costs the same, the largest wins).  GPTOSS_BALANCE_PUSH=0/1 forces
  // either for measurements.
  const bool balance_down = ctx->balance_pushing_gemm >= 0 ? ctx->balance_pushing_gemm != 0 : ctx->n_local <= 4;
  if (ctx->world > 1 && !balance_down) b.nft2 = 0;
  return b;
}

GemmArgs gemm_args(gptoss_ctx *ctx, const LayerWeights &w, bool mlp1) {
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.map_w = mlp1 ? w.map_w1 : w.map_w2;
  a.map_act = mlp1 ? ctx->map_x : ctx->map_h;
  a.offsets = ctx->rb.offsets;
  a.tb_prefix = mlp1 ? ctx->rb.tb_prefix : ctx->rb.tb_prefix2;
  a.e_begin = ctx->d.e_begin;
  a.n_local = ctx->n_local;
  a.n_feat = mlp1 ? ctx->d.I : ctx->d.H;
  a.n_feat_tiles = (a.n_feat + kTileF - 1) / kTileF;
  a.k_blocks = ((mlp1 ? ctx->d.H : ctx->d.I) + kBlockK - 1) / kBlockK;
  a.limit = ctx->d.limit;
  a.bias_a = mlp1 ? w.b1g : w.b2;
  a.bias_b = mlp1 ? w.b1u : nullptr;
  a.gate_up = ctx->gate_up;
  a.y_pairs = ctx->y_pairs;
  a.sorted = ctx->rb.sorted;
  a.topk_w = ctx->rb.topk_w;
  a.status = ctx->status;
  a.n_owners = 1;
  a.top_k = ctx->d.k;
  a.slice_tokens = ctx->max_tokens;
  return a;
}

}  // namespace

extern "C" {

const char *gptoss_version(void) { return "gptoss_b200 0.2 sm_100a"; }

uint64_t gptoss_launch_count(void) { return launch_counter().load(); }

int gptoss_ctx_create(const gptoss_moe_dims *dims, int device, int rank, int world, int max_tokens,
                      int wire_dtype, gptoss_ctx **out) {
  if (!dims || !out) return GPTOSS_ERR_BAD_ARG;
  *out = nullptr;
  if (dims->hidden <= 0 || dims->hidden % 8 || dims->intermediate <= 0 || dims->intermediate % 8 ||
      dims->n_experts <= 0 || dims->n_experts > kMaxExperts || dims->top_k <= 0 || dims->top_k > kMaxTopK ||
      dims->top_k > dims->n_experts || dims->n_layers <= 0 || world <= 0 || rank < 0 || rank >= world ||
      dims->n_experts % world || max_tokens <= 0 || (wire_dtype != GPTOSS_WIRE_F32 && wire_dtype != GPTOSS_WIRE_BF16))
    return GPTOSS_ERR_BAD_ARG;
  if ((long long)max_tokens * dims->top_k > (1ll << 30)) return GPTOSS_ERR_BAD_ARG;
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) return GPTOSS_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return GPTOSS_ERR_CUDA;
  if (prop.major != 10) return GPTOSS_ERR_UNSUPPORTED;
  if (cudaSetDevice(device) != cudaSuccess) return GPTOSS_ERR_CUDA;

  gptoss_ctx *ctx = new (std::nothrow) gptoss_ctx();
  if (!ctx) return GPTOSS_ERR_CUDA;
  ctx->dims = *dims;
  ctx->device = device;
  ctx->rank = rank;
  ctx->world = world;
  ctx->max_tokens = max_tokens;
  ctx->wire = wire_dtype;
  ctx->n_local = dims->n_experts / world;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->d = Dims{dims->hidden, dims->intermediate, dims->n_experts, dims->top_k, rank * ctx->n_local,
                (rank + 1) * ctx->n_local, dims->swiglu_limit};
  ctx->layers.resize(dims->n_layers);
  ctx->peers.timeout_ns = 2000000000ull;
  if (const char *e = getenv("GPTOSS_SHARED_ROUTING")) ctx->share_routing = world > 1 && e[0] == '1';
  if (const char *e = getenv("GPTOSS_TOKEN_BLOCK")) ctx->balance.force_rows = atoi(e);  // measurement aid: fixed token-block size
  if (const char *e = getenv("GPTOSS_BALANCE_PUSH")) ctx->balance_pushing_gemm = atoi(e) != 0 ? 1 : 0;
  if (const char *e = getenv("GPTOSS_PAIR")) ctx->pair_policy = atoi(e) != 0;           // expert GEMMs on pairs of CTAs

  const size_t T = max_tokens, H = dims->hidden, I = dims->intermediate, E = dims->n_experts, k = dims->top_k;
  const size_t P = T * k, nblk = (T + kTokensPerRouteBlock - 1) / kTokensPerRouteBlock;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) {
    if (e == cudaSuccess) e = r;
  };
  A(dev_alloc(&ctx->rb.scores, T * E));
  A(dev_alloc(&ctx->rb.blk_base, nblk * E));
  A(dev_alloc(&ctx->rb.offsets, E + 1));
  A(dev_alloc(&ctx->rb.tb_prefix, E + 1));
  A(dev_alloc(&ctx->rb.tb_prefix2, E + 1));
  A(dev_alloc(&ctx->gate_up, P * I));
  ctx->sym_delta_off = 1024;
  ctx->sym_y_off = ctx->sym_delta_off + ((T * H * sizeof(float) + 1023) & ~(size_t)1023);
  auto up = [](size_t v) { return (v + 1023) & ~(size_t)1023; };
  ctx->sym_tw_off = up(ctx->sym_y_off + P * H * sizeof(float));
  ctx->sym_ti_off = up(ctx->sym_tw_off + P * sizeof(float));
  ctx->sym_hist_off = up(ctx->sym_ti_off + P * sizeof(int));
  ctx->sym_xp_off = up(ctx->sym_hist_off + nblk * E * sizeof(int));
  ctx->sym_sorted_off = up(ctx->sym_xp_off + P * H * sizeof(__nv_bfloat16));
  ctx->sym_bytes = up(ctx->sym_sorted_off + P * sizeof(int));
  A(cudaMalloc(reinterpret_cast<void **>(&ctx->sym), ctx->sym_bytes));
  if (e == cudaSuccess) A(cudaMemset(ctx->sym, 0, 1024));
  if (e == cudaSuccess) {
    ctx->y_pairs = reinterpret_cast<float *>(ctx->sym + ctx->sym_y_off);
    ctx->rb.topk_w = reinterpret_cast<float *>(ctx->sym + ctx->sym_tw_off);
    ctx->rb.topk_i = reinterpret_cast<int *>(ctx->sym + ctx->sym_ti_off);
    ctx->rb.blk_hist = reinterpret_cast<int *>(ctx->sym + ctx->sym_hist_off);
    ctx->x_packed = reinterpret_cast<__nv_bfloat16 *>(ctx->sym + ctx->sym_xp_off);
    ctx->rb.sorted = reinterpret_cast<int *>(ctx->sym + ctx->sym_sorted_off);
    ctx->rows_self.n = 1;
    ctx->rows_self.experts_per_rank = ctx->n_local;
    ctx->rows_self.xp[0] = ctx->x_packed;
    ctx->share_self.n = 1;
    ctx->share_self.topk_w[0] = ctx->rb.topk_w;
    ctx->share_self.topk_i[0] = ctx->rb.topk_i;
    ctx->share_self.blk_hist[0] = ctx->rb.blk_hist;
  }
  A(dev_alloc(&ctx->comm_counter, 4));  // [0] exchange kernels, [1] shared routing, [2] row dispatch
  if (e == cudaSuccess) A(cudaMemset(ctx->comm_counter, 0, 4 * sizeof(int)));
  A(dev_alloc(&ctx->status, kStatusWords));
  for (auto &hs : ctx->hslot) {
    A(dev_alloc(&hs.t, T * H));
    A(dev_alloc(&hs.x, T * H));
  }
  A(dev_alloc(&ctx->router_partials, (size_t)kRouterMaxSplits * T * E));
  if (e == cudaSuccess) A(cudaMemset(ctx->status, 0, kStatusWords * sizeof(int)));
  // rows never written by the gather are still read by TMA (their columns are discarded): keep them finite
  if (e == cudaSuccess) A(cudaMemset(ctx->x_packed, 0, P * H * sizeof(__nv_bfloat16)));
  if (e == cudaSuccess) A(cudaMemset(ctx->gate_up, 0, P * I * sizeof(__nv_bfloat16)));
  if (e == cudaSuccess) A(encode_act_map(&ctx->map_x, ctx->x_packed, H, P));
  if (e == cudaSuccess) A(encode_act_map(&ctx->map_h, ctx->gate_up, I, P));
  if (e != cudaSuccess) {
    gptoss_ctx_destroy(ctx);
    return GPTOSS_ERR_CUDA;
  }
  *out = ctx;
  return GPTOSS_OK;
}

int gptoss_ctx_destroy(gptoss_ctx *ctx) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  for (auto &w : ctx->layers) free_layer(w);
  cudaFree(ctx->rb.scores);
  cudaFree(ctx->rb.blk_base);
  cudaFree(ctx->rb.offsets);
  cudaFree(ctx->rb.tb_prefix);
  cudaFree(ctx->rb.tb_prefix2);
  cudaFree(ctx->gate_up);
  for (int r = 0; r < kMaxRanks; ++r)
    if (ctx->peer_base[r]) cudaIpcCloseMemHandle(ctx->peer_base[r]);
  cudaFree(ctx->sym);
  cudaFree(ctx->comm_counter);
  cudaFree(ctx->status);
  for (auto &hs : ctx->hslot) {
    cudaFree(hs.t);
    cudaFree(hs.x);
    for (cudaEvent_t ev : {hs.ev_t, hs.ev_x, hs.ev_done, hs.ev_out})
      if (ev) cudaEventDestroy(ev);
    if (hs.status_host) cudaFreeHost(hs.status_host);
  }
  if (ctx->s_out) cudaStreamDestroy(ctx->s_out);
  cudaFree(ctx->router_partials);
  cudaFree(ctx->staging);
  if (ctx->s_main) cudaStreamDestroy(ctx->s_main);
  if (ctx->s_copy) cudaStreamDestroy(ctx->s_copy);
  delete ctx;
  return GPTOSS_OK;
}

const char *gptoss_last_error(const gptoss_ctx *ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int gptoss_ctx_status(gptoss_ctx *ctx) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  CK(cudaSetDevice(ctx->device));
  CK(cudaDeviceSynchronize());
  int st[kStatusWords];
  CK(cudaMemcpy(st, ctx->status, sizeof st, cudaMemcpyDeviceToHost));
  if (st[0] != 0) {
    CK(cudaMemset(ctx->status, 0, sizeof st));
    // a wait on a peer flag (sites 0x21xx..0x26xx) that gave up leaves this rank's step counters ahead of the silent
    // rank's: later exchanges of this group could never match again
    if (st[0] == kDevErrTimeout && ctx->attached && st[1] >= 0x2100 && st[1] < 0x2700) ctx->group_broken = true;
    char buf[160];
    snprintf(buf, sizeof buf, "device-side bounded wait gave up: code %d site 0x%x block %d", st[0], st[1], st[2]);
    return ctx->fail(st[0] == kDevErrTimeout ? GPTOSS_ERR_TIMEOUT : GPTOSS_ERR_CUDA, buf);
  }
  return GPTOSS_OK;
}

// ---- weights ------------------------------------------------------------------------------------------
int gptoss_upload_layer(gptoss_ctx *ctx, int layer, const float *router_w, const float *router_b,
                        const float *mlp1_w, const float *mlp1_b, const float *mlp2_w, const float *mlp2_b) {
  int rc = check_layer(ctx, layer, false);
  if (rc) return rc;
  if (!router_w || !router_b || !mlp1_w || !mlp1_b || !mlp2_w || !mlp2_b)
    return ctx->fail(GPTOSS_ERR_BAD_ARG, "null weight pointer");
  CK(cudaSetDevice(ctx->device));
  LayerWeights &w = ctx->layers[layer];
  if ((rc = alloc_layer(ctx, w))) return rc;
  const size_t H = ctx->d.H, I = ctx->d.I, E = ctx->d.E, EL = ctx->n_local, e0 = ctx->d.e_begin;
  size_t need = 2 * I * H;
  if (E * H > need) need = E * H;
  if (EL * 2 * I > need) need = EL * 2 * I;
  if ((rc = ensure_staging(ctx, need))) return rc;
  float *st = ctx->staging;

  CK(cudaMemcpy(st, router_w, E * H * sizeof(float), cudaMemcpyHostToDevice));
  CK(launch_f32_to_bf16(st, w.router_w, E * H, 0));
  CK(cudaMemcpy(st, router_b, E * sizeof(float), cudaMemcpyHostToDevice));
  CK(launch_round_bf16_f32(st, w.router_b, E, 0));
  for (size_t el = 0; el < EL; ++el) {
    CK(cudaMemcpy(st, mlp1_w + (e0 + el) * 2 * I * H, 2 * I * H * sizeof(float), cudaMemcpyHostToDevice));
    CK(launch_mlp1_deinterleave(st, w.w1 + el * 2 * I * H, (int)I, (int)H, 0));
  }
  for (size_t el = 0; el < EL; ++el) {
    CK(cudaMemcpy(st, mlp2_w + (e0 + el) * H * I, H * I * sizeof(float), cudaMemcpyHostToDevice));
    CK(launch_f32_to_bf16(st, w.w2 + el * H * I, H * I, 0));
  }
  CK(cudaMemcpy(st, mlp1_b + e0 * 2 * I, EL * 2 * I * sizeof(float), cudaMemcpyHostToDevice));
  CK(launch_bias_split(st, w.b1g, w.b1u, EL * I, 0));
  CK(cudaMemcpy(st, mlp2_b + e0 * H, EL * H * sizeof(float), cudaMemcpyHostToDevice));
  CK(launch_round_bf16_f32(st, w.b2, EL * H, 0));
  CK(cudaDeviceSynchronize());
  w.ready = true;
  return GPTOSS_OK;
}

int gptoss_fill_layer_synthetic(gptoss_ctx *ctx, int layer, uint64_t seed, float sigma) {
  int rc = check_layer(ctx, layer, false);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  LayerWeights &w = ctx->layers[layer];
  if ((rc = alloc_layer(ctx, w))) return rc;
  const size_t H = ctx->d.H, I = ctx->d.I, E = ctx->d.E, EL = ctx->n_local, e0 = ctx->d.e_begin;
  if ((rc = ensure_staging(ctx, EL * 2 * I))) return rc;
  const uint64_t lo = 16ull * (uint64_t)layer;
  CK(launch_synth_normal(w.router_w, E * H, seed, kTidRouterW + lo, 0, sigma, 0));
  CK(launch_synth_normal_f32(w.router_b, E, seed, kTidRouterB + lo, 0, sigma, 0));
  for (size_t el = 0; el < EL; ++el)
    CK(launch_synth_mlp1(w.w1 + el * 2 * I * H, (int)I, (int)H, seed, kTidMlp1W + lo, (e0 + el) * 2 * I * H, sigma, 0));
  CK(launch_synth_normal(w.w2, EL * H * I, seed, kTidMlp2W + lo, e0 * H * I, sigma, 0));
  CK(launch_synth_normal_f32(ctx->staging, EL * 2 * I, seed, kTidMlp1B + lo, e0 * 2 * I, sigma, 0));
  CK(launch_bias_split(ctx->staging, w.b1g, w.b1u, EL * I, 0));
  CK(launch_synth_normal_f32(w.b2, EL * H, seed, kTidMlp2B + lo, e0 * H, sigma, 0));
  CK(cudaDeviceSynchronize());
  w.ready = true;
  return GPTOSS_OK;
}

int gptoss_set_router_bias(gptoss_ctx *ctx, int layer, const float *router_b) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  if (!router_b) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null router bias");
  CK(cudaSetDevice(ctx->device));
  if ((rc = ensure_staging(ctx, ctx->d.E))) return rc;
  CK(cudaMemcpy(ctx->staging, router_b, ctx->d.E * sizeof(float), cudaMemcpyHostToDevice));
  CK(launch_round_bf16_f32(ctx->staging, ctx->layers[layer].router_b, ctx->d.E, 0));
  CK(cudaDeviceSynchronize());
  return GPTOSS_OK;
}

int gptoss_download_layer(gptoss_ctx *ctx, int layer, float *router_w, float *router_b, float *mlp1_w,
                          float *mlp1_b, float *mlp2_w, float *mlp2_b) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  const LayerWeights &w = ctx->layers[layer];
  const size_t H = ctx->d.H, I = ctx->d.I, E = ctx->d.E, EL = ctx->n_local;
  size_t need = 2 * I * H;
  if (E * H > need) need = E * H;
  if (EL * 2 * I > need) need = EL * 2 * I;
  if ((rc = ensure_staging(ctx, need))) return rc;
  float *st = ctx->staging;
  if (router_w) {
    CK(launch_bf16_to_f32(w.router_w, st, E * H, 0));
    CK(cudaMemcpy(router_w, st, E * H * sizeof(float), cudaMemcpyDeviceToHost));
  }
  if (router_b) CK(cudaMemcpy(router_b, w.router_b, E * sizeof(float), cudaMemcpyDeviceToHost));
  if (mlp1_w)
    for (size_t el = 0; el < EL; ++el) {
      CK(launch_mlp1_interleave(w.w1 + el * 2 * I * H, st, (int)I, (int)H, 0));
      CK(cudaMemcpy(mlp1_w + el * 2 * I * H, st, 2 * I * H * sizeof(float), cudaMemcpyDeviceToHost));
    }
  if (mlp1_b) {
    CK(launch_bias_merge(w.b1g, w.b1u, st, EL * I, 0));
    CK(cudaMemcpy(mlp1_b, st, EL * 2 * I * sizeof(float), cudaMemcpyDeviceToHost));
  }
  if (mlp2_w)
    for (size_t el = 0; el < EL; ++el) {
      CK(launch_bf16_to_f32(w.w2 + el * H * I, st, H * I, 0));
      CK(cudaMemcpy(mlp2_w + el * H * I, st, H * I * sizeof(float), cudaMemcpyDeviceToHost));
    }
  if (mlp2_b) CK(cudaMemcpy(mlp2_b, w.b2, EL * H * sizeof(float), cudaMemcpyDeviceToHost));
  return GPTOSS_OK;
}

// ---- stages ---------------------------------------------------------------------------------------------
static int check_attached(gptoss_ctx *ctx);

// Router GEMM + top-k + softmax + block histograms for rows [first, first + n) of a batch of T tokens (rows = their
// bf16 activations, 16-byte aligned), results stored to every rank of `sh`.
static int route_rows(gptoss_ctx *ctx, int layer, int T, const void *rows, int first, int n, const RouteShare &sh,
                      cudaStream_t s) {
  const LayerWeights &w = ctx->layers[layer];
  const int k_blocks = (ctx->d.H + kBlockK - 1) / kBlockK;
  if (n > 0) {
    if (reinterpret_cast<uintptr_t>(rows) & 15u) return ctx->fail(GPTOSS_ERR_BAD_ARG, "activations must be 16-byte aligned");
    if (ctx->map_t_base != rows || ctx->map_t_rows != n) {
      CK(encode_map_2d(&ctx->map_t, rows, ctx->d.H, n, 128));
      ctx->map_t_base = rows;
      ctx->map_t_rows = n;
    }
    RouterArgs ra;
    memset(&ra, 0, sizeof ra);
    ra.map_t = ctx->map_t;
    ra.map_wr = w.map_wr;
    ra.partials = ctx->router_partials;
    ra.T = n;
    ra.split_T = T;  // split K as a rank that routes the whole batch would: same bits whoever routes a token
    ra.E = ctx->d.E;
    ra.n_cols = (ctx->d.E + 15) & ~15;
    ra.k_blocks = k_blocks;
    ra.status = ctx->status;
    CK(launch_router_gemm(ra, kRouterMaxSplits, s));
  }
  CK(launch_router_topk(ctx->router_partials, router_splits_for(T, k_blocks, kRouterMaxSplits), w.router_b, n, first, ctx->d,
                        ctx->rb, sh, s));
  return GPTOSS_OK;
}

// Counting sort of the whole batch from the routing rows present in this rank's buffers + gather of the token rows
// of this rank's experts.
static int route_group(gptoss_ctx *ctx, int T, const void *t_full, cudaStream_t s) {
  CK(launch_expert_scan(ctx->rb, T, ctx->d, balance_for(ctx), FlagWait{}, s));
  CK(launch_scatter_gather(static_cast<const __nv_bfloat16 *>(t_full), 0, T, ctx->rb.topk_i, T, ctx->d, ctx->rb.blk_base,
                           ctx->rb.sorted, ctx->rows_self, s));
  return GPTOSS_OK;
}

int gptoss_moe_route(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (!t_dev_bf16) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null activation pointer");
  CK(cudaSetDevice(ctx->device));
  ctx->cur_T = T;
  if (T == 0) return GPTOSS_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((rc = route_rows(ctx, layer, T, t_dev_bf16, 0, T, ctx->share_self, s))) return rc;
  return route_group(ctx, T, t_dev_bf16, s);
}

// Shared routing: this rank routes only its token slice and stores the rows to every rank (flag D); route_finish
// waits for every rank's rows (and, in the token-sliced form, for the gathered activations) and groups the batch.
int gptoss_moe_route_local(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  CK(cudaSetDevice(ctx->device));
  ctx->cur_T = T;
  if (T == 0 || !ctx->share_routing) return GPTOSS_OK;  // small groups: route_finish routes the whole batch here
  const uint8_t *t = static_cast<const uint8_t *>(t_dev_bf16 ? t_dev_bf16 : ctx->sym + ctx->sym_delta_off);
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n);
  ctx->share.step = ++ctx->route_step;
  return route_rows(ctx, layer, T, t + (size_t)first * ctx->d.H * 2, first, n, ctx->share, static_cast<cudaStream_t>(stream));
}

int gptoss_moe_route_finish(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (T != ctx->cur_T || (ctx->share_routing && ctx->route_step == 0))
    return ctx->fail(GPTOSS_ERR_STATE, "route_finish without a matching route_local");
  CK(cudaSetDevice(ctx->device));
  if (T == 0) return GPTOSS_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void *t = t_dev_bf16 ? t_dev_bf16 : ctx->sym + ctx->sym_delta_off;
  if (ctx->pending_gather > 0 || ctx->share_routing)
    CK(launch_wait_flags(ctx->peers, ctx->pending_gather, ctx->share_routing ? ctx->route_step : 0, ctx->status, s));
  ctx->pending_gather = 0;
  if (!ctx->share_routing) return gptoss_moe_route(ctx, layer, T, t, stream);
  return route_group(ctx, T, t, s);
}

int gptoss_moe_mlp1_swiglu(gptoss_ctx *ctx, int layer, void *stream) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK((ctx->pair_mode ? launch_grouped_mlp1_pair : launch_grouped_mlp1)(gemm_args(ctx, ctx->layers[layer], true), ctx->sm_count,
                                                                       static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_mlp2(gptoss_ctx *ctx, int layer, void *stream) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK((ctx->pair_mode ? launch_grouped_mlp2_pair : launch_grouped_mlp2)(gemm_args(ctx, ctx->layers[layer], false), ctx->sm_count,
                                                                       static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_combine(gptoss_ctx *ctx, int T, float *x_dev, int residual, void *stream) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  int rc = check_T(ctx, T);
  if (rc) return rc;
  if (!x_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null output pointer");
  if (T != ctx->cur_T) return ctx->fail(GPTOSS_ERR_STATE, "combine: T differs from the routed batch");
  CK(cudaSetDevice(ctx->device));
  if (T == 0) return GPTOSS_OK;
  CK(launch_combine(ctx->y_pairs, ctx->rb.topk_i, T, ctx->d, x_dev, residual, ctx->sm_count,
                    static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

// ---- stages of the fused cross-GPU combine -------------------------------------------------------------------
static int check_attached(gptoss_ctx *ctx) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (ctx->world < 2 || !ctx->attached) return ctx->fail(GPTOSS_ERR_STATE, "no peers attached");
  if (ctx->group_broken)
    return ctx->fail(GPTOSS_ERR_STATE, "an earlier wait on a peer timed out: the group's step counters no longer match, "
                                       "destroy and re-create the contexts of all ranks");
  return GPTOSS_OK;
}

// Down GEMM whose epilogue stores each gate-weighted row into the y_pairs buffer of the token's owner; bf16: the rows
// travel (and are kept) as bf16, the owner still sums them in fp32.
static int push_rows(gptoss_ctx *ctx, int layer, bool bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int step = ++ctx->comm_step;
  GemmArgs a = gemm_args(ctx, ctx->layers[layer], false);
  a.out_bf16 = bf16 ? 1 : 0;
  ctx->pushed_bf16 = bf16;
  a.n_owners = ctx->world;
  a.slice_tokens = slice_rows(ctx->cur_T, ctx->world);
  for (int r = 0; r < ctx->world; ++r) {
    a.y_owner[r] = ctx->peers.y[r];
    a.signal_flags[r] = ctx->peers.flags[r] + ctx->rank;  // flag A of this rank on rank r
  }
  a.signal_step = step;
  a.signal_counter = ctx->comm_counter;
  CK((ctx->pair_mode ? launch_grouped_mlp2_pair : launch_grouped_mlp2)(a, ctx->sm_count, s));
  return GPTOSS_OK;
}

int gptoss_moe_push_to_owners(gptoss_ctx *ctx, int layer, void *stream) { return push_rows(ctx, layer, false, stream); }

int gptoss_moe_owner_combine(gptoss_ctx *ctx, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK(launch_combine_owner(ctx->peers, ctx->wire == GPTOSS_WIRE_BF16, ctx->cur_T, ctx->d.H, ctx->d.k, ctx->comm_step, ctx->status,
                          ctx->comm_counter, ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_add_delta(gptoss_ctx *ctx, float *x_dev, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if (!x_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null residual pointer");
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK(launch_add_delta(ctx->peers, ctx->wire == GPTOSS_WIRE_BF16, ctx->cur_T, ctx->d.H, ctx->comm_step, x_dev, ctx->status, ctx->sm_count,
                      static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

// ---- token-sliced form: every rank keeps only its slice of the residual stream ------------------------------
int gptoss_moe_slice_bounds(const gptoss_ctx *ctx, int T, int *first, int *count) {
  if (!ctx || T < 0) return GPTOSS_ERR_BAD_ARG;
  const int slice = slice_rows(T, ctx->world);
  int b0 = ctx->rank * slice, n = T - b0;
  n = n < 0 ? 0 : (n > slice ? slice : n);
  if (n == 0) b0 = T;
  if (first) *first = b0;
  if (count) *count = n;
  return GPTOSS_OK;
}

int gptoss_moe_gather_slice(gptoss_ctx *ctx, int T, float *x_slice_dev, const float *add_dev, const float *norm_w_dev,
                            void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (T == 0) return GPTOSS_OK;
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n);  // a rank without tokens still takes part (it raises its flag)
  if ((n > 0 && !x_slice_dev) || !norm_w_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null slice or norm-weight pointer");
  CK(cudaSetDevice(ctx->device));
  const int step = ctx->pending_gather = ++ctx->gather_step;
  CK(launch_slice_norm_gather(ctx->peers, T, ctx->d.H, x_slice_dev, add_dev, norm_w_dev, step, ctx->comm_counter,
                              static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_gather_rows(gptoss_ctx *ctx, int T, const void *t_slice_dev_bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (T == 0) return GPTOSS_OK;
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n);
  if (n > 0 && !t_slice_dev_bf16) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null slice pointer");
  if (n > 0 && (reinterpret_cast<uintptr_t>(t_slice_dev_bf16) & 15)) return ctx->fail(GPTOSS_ERR_BAD_ARG, "slice must be 16-byte aligned");
  CK(cudaSetDevice(ctx->device));
  const int step = ctx->pending_gather = ++ctx->gather_step;
  CK(launch_slice_copy_gather(ctx->peers, T, ctx->d.H, t_slice_dev_bf16, step, ctx->comm_counter, ctx->sm_count,
                              static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_comm_rendezvous(gptoss_ctx *ctx, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  CK(cudaSetDevice(ctx->device));
  CK(launch_rendezvous(ctx->peers, ++ctx->gather_step, ctx->status, static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_sliced_route(gptoss_ctx *ctx, int layer, int T, void *stream) {
  if (ctx && ctx->gather_step == 0) return ctx->fail(GPTOSS_ERR_STATE, "sliced route before any gather");
  return gptoss_moe_route_local(ctx, layer, T, nullptr, stream);  // this rank's rows of its own gathered buffer
}

int gptoss_moe_sliced_push(gptoss_ctx *ctx, int layer, int T, void *stream) {
  int rc = gptoss_moe_route_finish(ctx, layer, T, nullptr, stream);
  if (rc) return rc;
  if (T == 0) return GPTOSS_OK;
  if ((rc = gptoss_moe_mlp1_swiglu(ctx, layer, stream))) return rc;
  return push_rows(ctx, layer, ctx->wire == GPTOSS_WIRE_BF16, stream);
}

// ---- dispatch form of the token-sliced block: only the rows an expert needs cross NVLink ------------------------
int gptoss_moe_dispatch_route(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  CK(cudaSetDevice(ctx->device));
  ctx->cur_T = T;
  if (T == 0) return GPTOSS_OK;
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n);
  if (n > 0 && !t_slice_dev_bf16) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null slice pointer");
  ctx->share.step = ++ctx->route_step;
  return route_rows(ctx, layer, T, t_slice_dev_bf16, first, n, ctx->share, static_cast<cudaStream_t>(stream));
}

int gptoss_moe_dispatch_rows(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (T != ctx->cur_T || ctx->route_step == 0) return ctx->fail(GPTOSS_ERR_STATE, "dispatch_rows without a matching dispatch_route");
  CK(cudaSetDevice(ctx->device));
  if (T == 0) return GPTOSS_OK;
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n);
  if (n > 0 && !t_slice_dev_bf16) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null slice pointer");
  if (n > 0 && (reinterpret_cast<uintptr_t>(t_slice_dev_bf16) & 15)) return ctx->fail(GPTOSS_ERR_BAD_ARG, "slice must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the prefix-sum kernel first waits until every rank's routing rows have arrived (flag D)
  const FlagWait fw{ctx->peers.flags[ctx->rank] + 3 * kMaxRanks, ctx->world, ctx->route_step, ctx->peers.timeout_ns, ctx->status, 0x2600};
  CK(launch_expert_scan(ctx->rb, T, ctx->d, balance_for(ctx), fw, s));
  RowDispatch rd = ctx->rows_all;
  rd.step = ctx->pending_gather = ++ctx->gather_step;
  // every rank places the pairs of ITS tokens: row and pair id go to the rank of the pair's expert (a rank without
  // tokens only raises its flag)
  CK(launch_scatter_gather(n > 0 ? static_cast<const __nv_bfloat16 *>(t_slice_dev_bf16) : nullptr, first, n, ctx->rb.topk_i, T, ctx->d,
                           ctx->rb.blk_base, ctx->rb.sorted, rd, s));
  return GPTOSS_OK;
}

int gptoss_moe_dispatch_push(gptoss_ctx *ctx, int layer, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if (ctx->cur_T > 0 && ctx->pending_gather == 0) return ctx->fail(GPTOSS_ERR_STATE, "dispatch_push without a matching dispatch_rows");
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK(launch_wait_flags(ctx->peers, ctx->pending_gather, 0, ctx->status, static_cast<cudaStream_t>(stream)));  // every rank's rows have arrived
  ctx->pending_gather = 0;
  if ((rc = gptoss_moe_mlp1_swiglu(ctx, layer, stream))) return rc;
  return push_rows(ctx, layer, ctx->wire == GPTOSS_WIRE_BF16, stream);
}

int gptoss_moe_forward_dispatch(gptoss_ctx *ctx, int layer, int T, const void *t_slice_dev_bf16, float *x_slice_dev, void *stream) {
  int rc = gptoss_moe_dispatch_route(ctx, layer, T, t_slice_dev_bf16, stream);
  if (rc || T == 0) return rc;
  if ((rc = gptoss_moe_dispatch_rows(ctx, layer, T, t_slice_dev_bf16, stream))) return rc;
  if ((rc = gptoss_moe_dispatch_push(ctx, layer, stream))) return rc;
  return gptoss_moe_sliced_combine(ctx, x_slice_dev, stream);
}

int gptoss_moe_sliced_combine(gptoss_ctx *ctx, float *x_slice_dev, void *stream) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  int first = 0, n = 0;
  gptoss_moe_slice_bounds(ctx, ctx->cur_T, &first, &n);
  if (n > 0 && !x_slice_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null slice pointer");
  CK(cudaSetDevice(ctx->device));
  if (ctx->cur_T == 0) return GPTOSS_OK;
  CK(launch_combine_owner_slice(ctx->peers, ctx->pushed_bf16, ctx->cur_T, ctx->d.H, ctx->d.k, ctx->comm_step, x_slice_dev, ctx->status,
                                ctx->sm_count, static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_forward_sliced(gptoss_ctx *ctx, int layer, int T, float *x_slice_dev, void *stream) {
  int rc = gptoss_moe_sliced_route(ctx, layer, T, stream);
  if (rc) return rc;
  if ((rc = gptoss_moe_sliced_push(ctx, layer, T, stream))) return rc;
  return gptoss_moe_sliced_combine(ctx, x_slice_dev, stream);
}

// ---- the per-layer operator --------------------------------------------------------------------------------
static int forward_common(gptoss_ctx *ctx, int layer, int T, const void *t, float *out, int residual, void *stream) {
  int rc;
  if ((rc = gptoss_moe_route(ctx, layer, T, t, stream))) return rc;
  if ((rc = gptoss_moe_mlp1_swiglu(ctx, layer, stream))) return rc;
  if ((rc = gptoss_moe_mlp2(ctx, layer, stream))) return rc;
  return gptoss_moe_combine(ctx, T, out, residual, stream);
}

int gptoss_moe_forward(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, float *x_dev, void *stream) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!x_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null residual pointer");
  if (ctx->world == 1) return forward_common(ctx, layer, T, t_dev_bf16, x_dev, 1, stream);
  if (!ctx->attached)
    return ctx->fail(GPTOSS_ERR_STATE, "world > 1 without attached peers: use gptoss_moe_forward_partial");
  // expert-parallel with peer memory: push rows to their owners from the down-GEMM epilogue, owners
  // combine their token slice and deliver it to every rank, every rank adds it to its residual
  int rc;
  if (!t_dev_bf16) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null activation pointer");
  if ((rc = gptoss_moe_route_local(ctx, layer, T, t_dev_bf16, stream))) return rc;  // each rank routes its token slice
  if (T == 0) return GPTOSS_OK;
  if ((rc = gptoss_moe_route_finish(ctx, layer, T, t_dev_bf16, stream))) return rc;
  if ((rc = gptoss_moe_mlp1_swiglu(ctx, layer, stream))) return rc;
  if ((rc = gptoss_moe_push_to_owners(ctx, layer, stream))) return rc;
  if ((rc = gptoss_moe_owner_combine(ctx, stream))) return rc;
  return gptoss_moe_add_delta(ctx, x_dev, stream);
}

int gptoss_moe_forward_partial(gptoss_ctx *ctx, int layer, int T, const void *t_dev_bf16, float *partial_dev,
                               void *stream) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!partial_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null output pointer");
  return forward_common(ctx, layer, T, t_dev_bf16, partial_dev, 0, stream);
}

// ---- host buffers ---------------------------------------------------------------------------------------------
// A call is submitted (uploads on the copy stream, kernels on the main stream, the result's way back on a third
// stream, all chained by events) and waited for separately; two calls may be in flight, so that the second one's upload
// and kernels run while the first one's result crosses PCIe in the other direction.  The plain entry points are a
// submit followed by a wait.
static int host_streams(gptoss_ctx *ctx) {
  if (ctx->s_main) return GPTOSS_OK;
  CK(cudaStreamCreateWithFlags(&ctx->s_main, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&ctx->s_copy, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&ctx->s_out, cudaStreamNonBlocking));
  for (auto &hs : ctx->hslot) {
    for (cudaEvent_t *ev : {&hs.ev_t, &hs.ev_x, &hs.ev_done, &hs.ev_out}) CK(cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
    CK(cudaHostAlloc(reinterpret_cast<void **>(&hs.status_host), kStatusWords * sizeof(int), cudaHostAllocDefault));
  }
  return GPTOSS_OK;
}

// rows: token rows this rank moves over PCIe (all T of them, or its slice of a group's batch)
static int host_submit(gptoss_ctx *ctx, int layer, int T, int rows, const uint16_t *t_host, float *x_host, bool sliced) {
  int rc = host_streams(ctx);
  if (rc) return rc;
  gptoss_ctx::HostSlot &hs = ctx->hslot[ctx->h_head];
  if (hs.busy) return ctx->fail(GPTOSS_ERR_STATE, "two host-buffer calls are already in flight: wait for the older one first");
  const size_t n = (size_t)rows * ctx->d.H;
  // activations first (the routing needs them at once); the residual is needed only by the last kernel, so its
  // upload follows on the same copy stream and runs beside the routing and the GEMMs
  if (n) CK(cudaMemcpyAsync(hs.t, t_host, n * sizeof(uint16_t), cudaMemcpyHostToDevice, ctx->s_copy));
  CK(cudaEventRecord(hs.ev_t, ctx->s_copy));
  if (n) CK(cudaMemcpyAsync(hs.x, x_host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->s_copy));
  CK(cudaEventRecord(hs.ev_x, ctx->s_copy));
  CK(cudaStreamWaitEvent(ctx->s_main, hs.ev_t, 0));
  if (T > 0 && !sliced) {
    if ((rc = gptoss_moe_route(ctx, layer, T, hs.t, ctx->s_main))) return rc;
    if ((rc = gptoss_moe_mlp1_swiglu(ctx, layer, ctx->s_main))) return rc;
    if ((rc = gptoss_moe_mlp2(ctx, layer, ctx->s_main))) return rc;
    CK(cudaStreamWaitEvent(ctx->s_main, hs.ev_x, 0));
    if ((rc = gptoss_moe_combine(ctx, T, hs.x, 1, ctx->s_main))) return rc;
  } else if (T > 0) {
    if ((rc = gptoss_moe_dispatch_route(ctx, layer, T, hs.t, ctx->s_main))) return rc;
    if ((rc = gptoss_moe_dispatch_rows(ctx, layer, T, hs.t, ctx->s_main))) return rc;
    if ((rc = gptoss_moe_dispatch_push(ctx, layer, ctx->s_main))) return rc;
    CK(cudaStreamWaitEvent(ctx->s_main, hs.ev_x, 0));
    if ((rc = gptoss_moe_sliced_combine(ctx, hs.x, ctx->s_main))) return rc;
  }
  CK(cudaEventRecord(hs.ev_done, ctx->s_main));
  CK(cudaStreamWaitEvent(ctx->s_out, hs.ev_done, 0));
  if (n) CK(cudaMemcpyAsync(x_host, hs.x, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->s_out));
  CK(cudaMemcpyAsync(hs.status_host, ctx->status, kStatusWords * sizeof(int), cudaMemcpyDeviceToHost, ctx->s_out));
  CK(cudaEventRecord(hs.ev_out, ctx->s_out));
  hs.busy = true;
  ctx->h_head ^= 1;
  return GPTOSS_OK;
}

int gptoss_moe_forward_host_submit(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host, float *x_host) {
  int rc = check_layer(ctx, layer, true);
  if (rc) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  if (ctx->world > 1) return ctx->fail(GPTOSS_ERR_STATE, "world > 1: use gptoss_moe_forward_host_sliced_submit");
  if (T > 0 && (!t_host || !x_host)) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null host pointer");
  CK(cudaSetDevice(ctx->device));
  return host_submit(ctx, layer, T, T, t_host, x_host, false);
}

// Token-sliced form through host buffers: this rank's rows of t and x only (the host -> device traffic of a step is
// then the batch once over all GPUs instead of once per GPU); the rows of the other ranks arrive over NVLink.
int gptoss_moe_forward_host_sliced_submit(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host_slice, float *x_host_slice) {
  int rc = check_attached(ctx);
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, true))) return rc;
  if ((rc = check_T(ctx, T))) return rc;
  int first = 0, n_rows = 0;
  gptoss_moe_slice_bounds(ctx, T, &first, &n_rows);
  if (n_rows > 0 && (!t_host_slice || !x_host_slice)) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null host pointer");
  CK(cudaSetDevice(ctx->device));
  return host_submit(ctx, layer, T, n_rows, t_host_slice, x_host_slice, true);
}

int gptoss_moe_forward_host_wait(gptoss_ctx *ctx) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  gptoss_ctx::HostSlot &hs = ctx->hslot[ctx->h_tail];
  if (!hs.busy) return ctx->fail(GPTOSS_ERR_STATE, "no host-buffer call in flight");
  CK(cudaSetDevice(ctx->device));
  CK(cudaEventSynchronize(hs.ev_out));
  hs.busy = false;
  ctx->h_tail ^= 1;
  if (hs.status_host[0] != 0) return gptoss_ctx_status(ctx);  // formats the message and clears the word
  return GPTOSS_OK;
}

int gptoss_moe_forward_host(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host, float *x_host) {
  if (ctx && ctx->world > 1) {  // a group: every rank passes the whole batch and gets the whole result
    int rc = check_layer(ctx, layer, true);
    if (rc) return rc;
    if ((rc = check_T(ctx, T))) return rc;
    if (!t_host || !x_host) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null host pointer");
    if (T == 0) return GPTOSS_OK;
    if (ctx->hslot[0].busy || ctx->hslot[1].busy) return ctx->fail(GPTOSS_ERR_STATE, "host-buffer calls in flight");
    CK(cudaSetDevice(ctx->device));
    if ((rc = host_streams(ctx))) return rc;
    gptoss_ctx::HostSlot &hs = ctx->hslot[0];
    const size_t n = (size_t)T * ctx->d.H;
    CK(cudaMemcpyAsync(hs.t, t_host, n * sizeof(uint16_t), cudaMemcpyHostToDevice, ctx->s_main));
    CK(cudaMemcpyAsync(hs.x, x_host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->s_main));
    if ((rc = gptoss_moe_forward(ctx, layer, T, hs.t, hs.x, ctx->s_main))) return rc;
    CK(cudaMemcpyAsync(x_host, hs.x, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->s_main));
    CK(cudaMemcpyAsync(hs.status_host, ctx->status, kStatusWords * sizeof(int), cudaMemcpyDeviceToHost, ctx->s_main));
    CK(cudaStreamSynchronize(ctx->s_main));
    if (hs.status_host[0] != 0) return gptoss_ctx_status(ctx);
    return GPTOSS_OK;
  }
  int rc = gptoss_moe_forward_host_submit(ctx, layer, T, t_host, x_host);
  return rc ? rc : gptoss_moe_forward_host_wait(ctx);
}

int gptoss_moe_forward_host_sliced(gptoss_ctx *ctx, int layer, int T, const uint16_t *t_host_slice, float *x_host_slice) {
  int rc = gptoss_moe_forward_host_sliced_submit(ctx, layer, T, t_host_slice, x_host_slice);
  return rc ? rc : gptoss_moe_forward_host_wait(ctx);
}

// ---- peer memory ----------------------------------------------------------------------------------------------
// rank r's routing buffers and this rank's "routed" flag on rank r, inside r's symmetric buffer at `base`
static void set_share(gptoss_ctx *ctx, int r, uint8_t *base) {
  RouteShare &sh = ctx->share;
  sh.n = ctx->world;
  sh.counter = ctx->comm_counter + 1;
  sh.topk_w[r] = reinterpret_cast<float *>(base + ctx->sym_tw_off);
  sh.topk_i[r] = reinterpret_cast<int *>(base + ctx->sym_ti_off);
  sh.blk_hist[r] = reinterpret_cast<int *>(base + ctx->sym_hist_off);
  sh.flags[r] = reinterpret_cast<int *>(base) + 3 * kMaxRanks + ctx->rank;
  RowDispatch &rd = ctx->rows_all;
  rd.n = ctx->world;
  rd.experts_per_rank = ctx->n_local;
  rd.counter = ctx->comm_counter + 2;
  rd.xp[r] = reinterpret_cast<__nv_bfloat16 *>(base + ctx->sym_xp_off);
  rd.sorted[r] = reinterpret_cast<int *>(base + ctx->sym_sorted_off);
  rd.flags[r] = reinterpret_cast<int *>(base) + 2 * kMaxRanks + ctx->rank;  // flag C of this rank on rank r
}

int gptoss_comm_export(gptoss_ctx *ctx, void *handle_out) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!handle_out) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null handle buffer");
  static_assert(sizeof(cudaIpcMemHandle_t) == GPTOSS_IPC_HANDLE_BYTES, "IPC handle size");
  CK(cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  CK(cudaIpcGetMemHandle(&h, ctx->sym));
  memcpy(handle_out, &h, sizeof h);
  return GPTOSS_OK;
}

int gptoss_comm_attach(gptoss_ctx *ctx, const void *handles) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!handles) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null handle buffer");
  if (ctx->world > kMaxRanks) return ctx->fail(GPTOSS_ERR_BAD_ARG, "world larger than 16");
  if (ctx->attached) return ctx->fail(GPTOSS_ERR_STATE, "peers already attached");
  CK(cudaSetDevice(ctx->device));
  ctx->peers.rank = ctx->rank;
  ctx->peers.world = ctx->world;
  for (int r = 0; r < ctx->world; ++r) {
    uint8_t *base = ctx->sym;
    if (r != ctx->rank) {
      cudaIpcMemHandle_t h;
      memcpy(&h, static_cast<const uint8_t *>(handles) + (size_t)r * GPTOSS_IPC_HANDLE_BYTES, sizeof h);
      void *p = nullptr;
      CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
      ctx->peer_base[r] = p;
      base = static_cast<uint8_t *>(p);
    }
    ctx->peers.flags[r] = reinterpret_cast<int *>(base);
    ctx->peers.delta[r] = reinterpret_cast<float *>(base + ctx->sym_delta_off);
    ctx->peers.y[r] = reinterpret_cast<float *>(base + ctx->sym_y_off);
    set_share(ctx, r, base);
  }
  ctx->attached = true;
  return GPTOSS_OK;
}

int gptoss_comm_attach_local(gptoss_ctx *ctx, gptoss_ctx *const *all) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!all) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null context array");
  if (ctx->world > kMaxRanks) return ctx->fail(GPTOSS_ERR_BAD_ARG, "world larger than 16");
  if (ctx->attached) return ctx->fail(GPTOSS_ERR_STATE, "peers already attached");
  CK(cudaSetDevice(ctx->device));
  ctx->peers.rank = ctx->rank;
  ctx->peers.world = ctx->world;
  for (int r = 0; r < ctx->world; ++r) {
    const gptoss_ctx *p = all[r];
    if (!p || p->world != ctx->world || p->rank != r || p->sym_bytes != ctx->sym_bytes)
      return ctx->fail(GPTOSS_ERR_BAD_ARG, "context array does not hold ranks 0..world-1 of the same shape");
    if (p->device != ctx->device) {
      cudaError_t e = cudaDeviceEnablePeerAccess(p->device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) return ctx->fail(GPTOSS_ERR_CUDA, "cudaDeviceEnablePeerAccess", e);
    }
    ctx->peers.flags[r] = reinterpret_cast<int *>(p->sym);
    ctx->peers.delta[r] = reinterpret_cast<float *>(p->sym + p->sym_delta_off);
    ctx->peers.y[r] = reinterpret_cast<float *>(p->sym + p->sym_y_off);
    set_share(ctx, r, p->sym);
  }
  ctx->attached = true;
  return GPTOSS_OK;
}

int gptoss_comm_set_timeout_ms(gptoss_ctx *ctx, int ms) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (ms <= 0 || ms > 60000) return ctx->fail(GPTOSS_ERR_BAD_ARG, "timeout must be in 1..60000 ms");
  ctx->peers.timeout_ns = (unsigned long long)ms * 1000000ull;
  return GPTOSS_OK;
}

// ---- stand-alone routing operators ---------------------------------------------------------------------------
int gptoss_topk_softmax(gptoss_ctx *ctx, int T, const float *scores_dev, float *topk_w_dev, int *topk_i_dev,
                        void *stream) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (T < 0) return ctx->fail(GPTOSS_ERR_BAD_ARG, "negative T");
  if (T == 0) return GPTOSS_OK;  // empty batch: nothing to read or write, pointers may be null
  if (!scores_dev || !topk_w_dev || !topk_i_dev) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null pointer");
  CK(cudaSetDevice(ctx->device));
  CK(launch_topk_softmax(scores_dev, T, ctx->d.E, ctx->d.k, topk_w_dev, topk_i_dev, static_cast<cudaStream_t>(stream)));
  return GPTOSS_OK;
}

int gptoss_moe_build_offsets(gptoss_ctx *ctx, int T, const int *topk_i_dev, int *offsets_dev, int *sorted_pair_ids_dev,
                             void *stream) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  int rc = check_T(ctx, T);
  if (rc) return rc;
  if (!offsets_dev || (T > 0 && (!topk_i_dev || !sorted_pair_ids_dev)))
    return ctx->fail(GPTOSS_ERR_BAD_ARG, "null pointer");
  CK(cudaSetDevice(ctx->device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 0) {  // empty batch: all offsets are zero, nothing else is touched
    CK(cudaMemsetAsync(offsets_dev, 0, (ctx->d.E + 1) * sizeof(int), s));
    return GPTOSS_OK;
  }
  RouteBuffers rb = ctx->rb;  // block histograms/bases live in the context scratch; results go to the caller
  rb.offsets = offsets_dev;
  rb.sorted = sorted_pair_ids_dev;
  rb.tb_prefix = nullptr;  // the token-block prefix of the context's own batch stays as it is
  CK(launch_pair_hist(topk_i_dev, T, ctx->d, rb.blk_hist, s));
  CK(launch_expert_scan(rb, T, ctx->d, ctx->balance, FlagWait{}, s));
  CK(launch_scatter_gather(nullptr, 0, 0, topk_i_dev, T, ctx->d, rb.blk_base, rb.sorted, RowDispatch{}, s));
  return GPTOSS_OK;
}

// sample_argmax (run.cpp:739-750) on caller-supplied device rows
int gptoss_argmax_rows(const float *logits_dev, int B, int V, int *next_dev, void *stream) {
  if (B < 0 || V <= 0) return GPTOSS_ERR_BAD_ARG;
  if (B == 0) return GPTOSS_OK;
  if (!logits_dev || !next_dev) return GPTOSS_ERR_BAD_ARG;
  return launch_argmax(logits_dev, B, V, next_dev, static_cast<cudaStream_t>(stream)) == cudaSuccess ? GPTOSS_OK : GPTOSS_ERR_CUDA;
}

// ---- taps --------------------------------------------------------------------------------------------------------
int gptoss_read_tap(gptoss_ctx *ctx, int tap, void *host_dst, uint64_t bytes) {
  if (!ctx) return GPTOSS_ERR_BAD_ARG;
  if (!host_dst) return ctx->fail(GPTOSS_ERR_BAD_ARG, "null destination");
  const size_t T = ctx->max_tokens, H = ctx->d.H, I = ctx->d.I, E = ctx->d.E, k = ctx->d.k, P = T * k;
  const void *src = nullptr;
  size_t cap = 0;
  switch (tap) {
    case GPTOSS_TAP_SCORES: src = ctx->rb.scores; cap = T * E * 4; break;
    case GPTOSS_TAP_TOPK_W: src = ctx->rb.topk_w; cap = P * 4; break;
    case GPTOSS_TAP_TOPK_I: src = ctx->rb.topk_i; cap = P * 4; break;
    case GPTOSS_TAP_OFFSETS: src = ctx->rb.offsets; cap = (E + 1) * 4; break;
    case GPTOSS_TAP_SORTED: src = ctx->rb.sorted; cap = P * 4; break;
    case GPTOSS_TAP_X_PACKED: src = ctx->x_packed; cap = P * H * 2; break;
    case GPTOSS_TAP_GATE_UP: src = ctx->gate_up; cap = P * I * 2; break;
    case GPTOSS_TAP_Y_PAIRS: src = ctx->y_pairs; cap = P * H * 4; break;
    case GPTOSS_TAP_GATHERED: src = ctx->sym + ctx->sym_delta_off; cap = T * H * 2; break;
    default: return ctx->fail(GPTOSS_ERR_BAD_ARG, "unknown tap");
  }
  if (bytes > cap) return ctx->fail(GPTOSS_ERR_BAD_ARG, "tap read larger than the buffer");
  CK(cudaSetDevice(ctx->device));
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost));
  return GPTOSS_OK;
}

int gptoss_synth_normal_bf16(void *dst_dev_bf16, uint64_t n, uint64_t seed, uint64_t tensor_id, uint64_t start,
                             float sigma, void *stream) {
  if (!dst_dev_bf16) return GPTOSS_ERR_BAD_ARG;
  if (n == 0) return GPTOSS_OK;
  cudaError_t e = launch_synth_normal(static_cast<__nv_bfloat16 *>(dst_dev_bf16), n, seed, tensor_id, start, sigma,
                                      static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? GPTOSS_OK : GPTOSS_ERR_CUDA;
}

}  // extern "C"
