// Host-callable launchers of the gptoss_b200 kernels (internal to the library).
#pragma once

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <utility>

#include "common.cuh"

namespace gptoss {

// Launch with the programmatic-serialization attribute (see pdl_wait in common.cuh); GPTOSS_NO_PDL=1 in the
// environment falls back to plain stream order.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char *v = std::getenv("GPTOSS_NO_PDL");
    return !(v && v[0] == '1');
  }();
  return on;
}
// Kernels this library has launched in this process (every launch goes through launch_chain or count_launch).
inline std::atomic<uint64_t> &launch_counter() {
  static std::atomic<uint64_t> n{0};
  return n;
}
inline void count_launch() { launch_counter().fetch_add(1, std::memory_order_relaxed); }

template <typename... KArgs, typename... Args>
cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// routing.cu
// T rows of partial scores (local row b = token first_token + b of the batch); results to every rank of `share`
cudaError_t launch_router_topk(const float *partials, int n_splits, const float *br, int T, int first_token, const Dims &d,
                               const RouteBuffers &rb, const RouteShare &share, cudaStream_t s);
cudaError_t launch_topk_softmax(const float *scores, int T, int E, int k, float *topk_w, int *topk_i,
                                cudaStream_t s);
cudaError_t launch_pair_hist(const int *topk_i, int T, const Dims &d, int *blk_hist, cudaStream_t s);
// fw.step > 0: the kernel first waits for that flag of every rank (dispatch form: the routing rows of all ranks)
cudaError_t launch_expert_scan(const RouteBuffers &rb, int T, const Dims &d, const TileBalance &tb, const FlagWait &fw,
                               cudaStream_t s);
// t: rows of tokens [t_first, t_first + t_count) (null: pair ids only)
cudaError_t launch_scatter_gather(const __nv_bfloat16 *t, int t_first, int t_count, const int *topk_i, int T, const Dims &d,
                                  const int *blk_base, int *sorted, const RowDispatch &rd, cudaStream_t s);
cudaError_t launch_combine(const float *y_pairs, const int *topk_i, int T, const Dims &d, float *x,
                           int residual, int sm_count, cudaStream_t s);

// comm.cu — peer-memory combine across the ranks of one box
constexpr int kMaxRanks = 16;
struct PeerTable {
  int rank, world;
  unsigned long long timeout_ns;  // limit of every wait on a peer flag
  float *y[kMaxRanks];      // every rank's y_pairs  [P,H] fp32 (index = own rank: local memory)
  float *delta[kMaxRanks];  // every rank's delta    [T,H] fp32, or bf16 in the same storage (bf16 wire); in the token-sliced
                            //                       form the same storage holds the gathered activations [T,H] bf16
  int *flags[kMaxRanks];    // every rank's flags    [4][kMaxRanks]: A = "rank r pushed", B = "owner r delivered",
                            //                       C = "rank r stored its slice of the gathered activations",
                            //                       D = "rank r stored the routing of its token slice"
};
cudaError_t launch_combine_owner(const PeerTable &pt, bool bf16_wire, int T, int H, int k, int step, int *status,
                                 int *counter, int sm_count, cudaStream_t s);
cudaError_t launch_add_delta(const PeerTable &pt, bool bf16_wire, int T, int H, int step, float *x, int *status,
                             int sm_count, cudaStream_t s);

cudaError_t launch_slice_norm_gather(const PeerTable &pt, int T, int H, float *x_slice, const float *add, const float *w,
                                     int step, int *counter, cudaStream_t s);
cudaError_t launch_slice_copy_gather(const PeerTable &pt, int T, int H, const void *t_slice, int step, int *counter,
                                     int sm_count, cudaStream_t s);
// waits for flag C >= gather_step and flag D >= route_step of every rank (a step of 0 skips that flag)
cudaError_t launch_wait_flags(const PeerTable &pt, int gather_step, int route_step, int *status, cudaStream_t s);
cudaError_t launch_rendezvous(const PeerTable &pt, int step, int *status, cudaStream_t s);
cudaError_t launch_combine_owner_slice(const PeerTable &pt, bool bf16_rows, int T, int H, int k, int step, float *x_slice,
                                       int *status, int sm_count, cudaStream_t s);

// router.cu
struct RouterArgs {
  CUtensorMap map_t;   // activations t [T,H]: 2-D (k, token), box {64,128}
  CUtensorMap map_wr;  // router weight [E,H]: 2-D (k, expert), box {64, n_cols}
  float *partials;     // [splits][T][E]
  int split_T;         // batch size the split-K factor is derived from (0 = T): a rank that routes only its slice
                       // of a batch must split K like a rank that routes all of it, or the scores' bits differ
  int T, E;
  int n_cols;          // E rounded up to a multiple of 16 (UMMA N)
  int k_blocks;        // ceil(H / 64)
  int *status;
  // filled by launch_router_gemm
  int k_blocks_per_split, stages, stage_bytes, tmem_cols;
};
constexpr int kRouterMaxSplits = 8;
cudaError_t launch_router_gemm(RouterArgs a, int max_splits, cudaStream_t s);
int router_splits_for(int T, int k_blocks, int max_splits);
// 2-D bf16 map with the 128-byte swizzle and an arbitrary box height (<= 256 rows)
cudaError_t encode_map_2d(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows, uint32_t box_rows);

// grouped_gemm.cu
struct GemmArgs {
  CUtensorMap map_w;    // weights: 3-D (k, feature, expert-slab), bf16, 128-byte swizzle, box {64,128,1}
  CUtensorMap map_act;  // activations: 2-D (k, row), bf16, 128-byte swizzle, box {64,32}
  const int *offsets;    // [E+1] global expert offsets
  const int *tb_prefix;  // [E_local+1]
  int e_begin, n_local;  // local expert range
  int n_feat;            // output features per expert (I for mlp1, H for mlp2)
  int n_feat_tiles;      // ceil(n_feat / 128)
  int k_blocks;          // ceil(K / 64)
  float limit;           // swiglu clamp (mlp1)
  const float *bias_a;   // mlp1: gate bias [E_local, I];  mlp2: bias [E_local, H]
  const float *bias_b;   // mlp1: up bias   [E_local, I];  mlp2: unused
  __nv_bfloat16 *gate_up;  // mlp1 out [P, I]
  float *y_pairs;          // mlp2 out [P, H] by pair id (local)
  int out_bf16;            // mlp2: rows are stored as bf16 (same row/element indexing, half the bytes)
  float *y_owner[kMaxRanks];  // mlp2 with n_owners > 1: y_pairs of the rank that owns the token slice
  int n_owners;            // 1 = store locally; > 1 = push each row to its owner
  int slice_tokens;        // tokens per owner slice
  int *signal_flags[kMaxRanks];  // mlp2 pushing to owners: this rank's "pushed" flag on every rank, raised to
  int signal_step;               // signal_step by the last CTA to finish (0 = no signalling)
  int *signal_counter;           // CTAs finished so far (left at 0)
  int top_k;
  float *amax_val;         // argmax epilogue (launch_grouped_amax): per (token block, feature) the largest product over
  int *amax_at;            // the block's rows, and the id of the row that gave it (first one on ties)
  const int *sorted;       // mlp2: [P]
  const float *topk_w;     // mlp2: [P] by pair id
  int *status;             // device status words
};
cudaError_t launch_grouped_mlp1(const GemmArgs &a, int sm_count, cudaStream_t s);
cudaError_t launch_grouped_mlp2(const GemmArgs &a, int sm_count, cudaStream_t s);
// grouped_gemm_pair.cu — the same two GEMMs with a pair of CTAs (tcgen05 cta_group::2) per work item
cudaError_t launch_grouped_mlp1_pair(const GemmArgs &a, int sm_count, cudaStream_t s);
cudaError_t launch_grouped_mlp2_pair(const GemmArgs &a, int sm_count, cudaStream_t s);
cudaError_t launch_grouped_amax(const GemmArgs &a, int sm_count, cudaStream_t s);
// Encodes the two tensor maps (driver entry point resolved at run time; no link-time libcuda).
// weights: base of [slabs][rows][K] bf16;  activations: base of [rows][K] bf16.
cudaError_t encode_weight_map(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows, uint64_t slabs);
cudaError_t encode_act_map(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows);

// model_kernels.cu — the kernels around the MoE block that a decode step needs
cudaError_t launch_embed(const int *tokens, const __nv_bfloat16 *table, int B, int H, int vocab, float *x, cudaStream_t s);
cudaError_t launch_residual_rmsnorm(float *x, const float *add, const float *w, int B, int H, __nv_bfloat16 *out,
                                    cudaStream_t s);
cudaError_t launch_qkv_rope_store(const float *qkv, const float *cos_t, const float *sin_t, int pos, int B, int nq, int nkv,
                                  int hd, int S, float *q_out, __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache,
                                  const int *cache_rows, const int *pos_rows, cudaStream_t s);
cudaError_t launch_attention(const float *q, const __nv_bfloat16 *k_cache, const __nv_bfloat16 *v_cache, const float *sinks,
                             int pos, int t_lo, int B, int nq, int nkv, int hd, int S, __nv_bfloat16 *out, const int *cache_rows,
                             const int *pos_rows, int window, cudaStream_t s);
// Warps that share one (sequence, kv head) problem of the attention kernel, by the number of cached positions it reads
// minus one (`span` = pos - t_lo): the split fixes the order of the softmax accumulation, so it follows the context
// length only.
inline int attention_warps_per_problem(int span) {
  const int n_chunks = span / 32 + 1;
  return n_chunks <= 16 ? 1 : (n_chunks <= 64 ? 2 : 4);
}
// pos_rows (both launchers above): null, or the position of each of the B sequences (a batch whose sequences started at
// different steps); `pos` is then ignored by the RoPE kernel, and the attention launcher takes the sequences of ONE
// class of attention_warps_per_problem per call, with pos / t_lo those of its longest context and `window` the
// sliding window of the layer (0 = none), from which the kernel derives each sequence's first position.
// cache_rows (both launchers above): null, or for each of the B sequences of the step the row of the KV cache that holds
// it (a batch from which finished sequences were dropped keeps the cache rows of the remaining ones)
cudaError_t launch_argmax(const float *logits, int B, int V, int *next, cudaStream_t s);
// next[b] = id of the first maximum over the (max, id) partials val/at [n_blocks][B] (blocks in ascending id order)
cudaError_t launch_argmax_partials(const float *val, const int *at, int n_blocks, int B, int *next, cudaStream_t s);
cudaError_t launch_iota_ones(int *iota, float *ones, int n, cudaStream_t s);

// convert.cu
cudaError_t launch_f32_to_bf16(const float *src, __nv_bfloat16 *dst, size_t n, cudaStream_t s);
cudaError_t launch_bf16_to_f32(const __nv_bfloat16 *src, float *dst, size_t n, cudaStream_t s);
// mlp1 rows: checkpoint order (gate row 2c, up row 2c+1) <-> device order [2][I][K] per expert
cudaError_t launch_mlp1_deinterleave(const float *src, __nv_bfloat16 *dst, int I, int K, cudaStream_t s);
cudaError_t launch_mlp1_interleave(const __nv_bfloat16 *src, float *dst, int I, int K, cudaStream_t s);
cudaError_t launch_bias_split(const float *src, float *g, float *u, size_t n_pairs, cudaStream_t s);
cudaError_t launch_bias_merge(const float *g, const float *u, float *dst, size_t n_pairs, cudaStream_t s);
cudaError_t launch_round_bf16_f32(const float *src, float *dst, size_t n, cudaStream_t s);
cudaError_t launch_synth_normal(__nv_bfloat16 *dst, uint64_t n, uint64_t seed, uint64_t tensor_id,
                                uint64_t start, float sigma, cudaStream_t s);
// synthetic mlp1 slab for one expert directly in device order; `start` = checkpoint-order index of the
// expert's first element
cudaError_t launch_synth_mlp1(__nv_bfloat16 *dst, int I, int K, uint64_t seed, uint64_t tensor_id,
                              uint64_t start, float sigma, cudaStream_t s);
cudaError_t launch_synth_normal_f32(float *dst, uint64_t n, uint64_t seed, uint64_t tensor_id,
                                    uint64_t start, float sigma, cudaStream_t s);

// ---- residual + RMSNorm of one row, shared by the single-GPU kernel and the peer-storing one ---------------------
//   if (add) x[:] += add[:]            (projection output incl. its bias)
//   store(i, w[i] * (x[i] * rsqrt(mean(x^2) + 1e-5)))   for every i, 4 consecutive elements at a time if H % 4 == 0
// Called by every thread of a 256-thread block (part: 8 doubles of shared memory).  The sum of squares is accumulated
// in fp32 per thread, added across the warp by shuffles and across warps in double, in this fixed order, so every
// caller gets the same bits for the same row.
template <class Store4, class Store1>
__device__ __forceinline__ void residual_rmsnorm_row(float *__restrict__ xr, const float *__restrict__ addr,
                                                     const float *__restrict__ w, int H, double *part, Store4 store4,
                                                     Store1 store1) {
  float ss = 0.f;
  const bool vec = (H & 3) == 0;
  if (vec) {
    float4 *x4 = reinterpret_cast<float4 *>(xr);
    const float4 *a4 = reinterpret_cast<const float4 *>(addr);
    for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
      float4 v = x4[i];
      if (addr) {
        const float4 a = a4[i];
        v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
        x4[i] = v;
      }
      ss += v.x * v.x;
      ss += v.y * v.y;
      ss += v.z * v.z;
      ss += v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (addr) {
        v += addr[i];
        xr[i] = v;
      }
      ss += v * v;
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = (double)ss;
  __syncthreads();
  double tot = 0.0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += part[i];
  const float inv = 1.0f / sqrtf((float)(tot / H + 1e-5));
  if (vec) {
    const float4 *x4 = reinterpret_cast<const float4 *>(xr), *w4 = reinterpret_cast<const float4 *>(w);
    for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
      const float4 v = x4[i], g = w4[i];
      const __nv_bfloat162 lo = __floats2bfloat162_rn(g.x * (inv * v.x), g.y * (inv * v.y));
      const __nv_bfloat162 hi = __floats2bfloat162_rn(g.z * (inv * v.z), g.w * (inv * v.w));
      store4(i, make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi)));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) store1(i, __float2bfloat16_rn(w[i] * (inv * xr[i])));
  }
}

}  // namespace gptoss
