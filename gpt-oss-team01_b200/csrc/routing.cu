// Routing side of the MoE block: router split-K reduction + top-k + softmax, expert histogram / prefix / stable
// scatter (counting sort of pair ids), row gather, and the slot-ordered combine.
//
// Everything here is bandwidth/latency-bound integer and fp32 work: one warp per token, 16-byte
// loads, warp shuffles, no global atomics, deterministic results (all ranks of an expert-parallel
// group must derive bit-identical routing from the replicated activations).
#include <climits>
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace gptoss {

namespace {

// Top-k of E scores spread over the warp (position p = s*32 + lane holds val[s]) in the exact order
// the reference kernel produces (layer_hip_batch.cpp:1119-1140): k rounds of "first maximum of
// positions [i,E) under strict '>', swapped into position i" — the swap moves the displaced element
// to the winner's old position, which decides later ties.  Then softmax over the selected raw
// scores (layer_hip_batch.cpp:1143-1153).  Lanes j < k return (weight_j, id_j).
template <int SLOTS>
__device__ __forceinline__ void warp_topk_softmax(float (&val)[SLOTS], int E, int k, int lane,
                                                  float &out_w, int &out_i) {
  int idx[SLOTS];
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) idx[s] = s * 32 + lane;

  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
#pragma unroll
  for (int i = 0; i < kMaxTopK; ++i) {
    sel_v[i] = 0.f;
    sel_i[i] = -1;
    if (i < k) {
      // position i's current content (the initial max_idx of the round)
      float vi = 0.f;
      int ii = 0;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s)
        if (s == i / 32) {
          vi = val[s];
          ii = idx[s];
        }
      vi = __shfl_sync(0xffffffffu, vi, i & 31);
      ii = __shfl_sync(0xffffffffu, ii, i & 31);

      // best strictly-greater candidate among positions (i, E): lowest position among the maxima
      float bv = vi;
      int bp = i;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s) {
        const int p = s * 32 + lane;
        if (p > i && p < E && (val[s] > bv)) {
          bv = val[s];
          bp = p;
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int op = __shfl_xor_sync(0xffffffffu, bp, off);
        if (ov > bv || (ov == bv && op < bp)) {
          bv = ov;
          bp = op;
        }
      }
      // id stored at the winning position
      int bi = 0;
#pragma unroll
      for (int s = 0; s < SLOTS; ++s)
        if (s == bp / 32) bi = idx[s];
      bi = __shfl_sync(0xffffffffu, bi, bp & 31);

      if (bp != i) {  // swap positions i and bp
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
          const int p = s * 32 + lane;
          if (p == bp) {
            val[s] = vi;
            idx[s] = ii;
          } else if (p == i) {
            val[s] = bv;
            idx[s] = bi;
          }
        }
      }
      sel_v[i] = bv;
      sel_i[i] = bi;
    }
  }

  const float mx = sel_v[0];
  double denom = 0.0;
#pragma unroll
  for (int i = 0; i < kMaxTopK; ++i)
    if (i < k) denom += (double)expf(sel_v[i] - mx);
  out_w = 0.f;
  out_i = -1;
#pragma unroll
  for (int i = 0; i < kMaxTopK; ++i)
    if (i < k && lane == i) {
      out_w = expf(sel_v[i] - mx) / (float)denom;
      out_i = sel_i[i];
    }
}

}  // namespace

// ---- split-K reduction of the router GEMM + bias + top-k + softmax + per-block expert histogram ---------
// One warp per token.  scores[b,e] = (partial[0][b,e] + partial[1][b,e] + ...) + br[e], summed in split order.
// Local row b is token first + b of the batch (first is a multiple of the block's 8 tokens); the gate weights, expert
// ids and the block's histogram go to the routing buffers of every rank in `sh`.
template <int GROUPS>
__global__ void __launch_bounds__(256) router_topk_kernel(const float *__restrict__ partials, int n_splits,
                                                          const float *__restrict__ br, int T, int first, Dims d,
                                                          RouteBuffers rb, RouteShare sh) {
  __shared__ int hist[kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kTokensPerRouteBlock + warp;
  for (int e = threadIdx.x; e < d.E; e += blockDim.x) hist[e] = 0;
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  if (b < T) {
    float score[GROUPS];
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const int eg = g * 32 + lane;
      float s = -INFINITY;
      if (eg < d.E) {
        s = partials[(size_t)b * d.E + eg];
        for (int sp = 1; sp < n_splits; ++sp) s += partials[((size_t)sp * T + b) * d.E + eg];
        s += br[eg];
        rb.scores[(size_t)(first + b) * d.E + eg] = s;
      }
      score[g] = s;
    }
    float w;
    int id;
    warp_topk_softmax<GROUPS>(score, d.E, d.k, lane, w, id);
    if (lane < d.k) {
      const size_t o = (size_t)(first + b) * d.k + lane;
      for (int r = 0; r < sh.n; ++r) {
        sh.topk_w[r][o] = w;
        sh.topk_i[r][o] = id;
      }
      atomicAdd(&hist[id], 1);
    }
  }
  __syncthreads();
  if (blockIdx.x * kTokensPerRouteBlock < T) {
    const size_t blk = (size_t)(first / kTokensPerRouteBlock + blockIdx.x) * d.E;
    for (int e = threadIdx.x; e < d.E; e += blockDim.x)
      for (int r = 0; r < sh.n; ++r) sh.blk_hist[r][blk + e] = hist[e];
  }
  if (sh.step > 0) {  // stores ordered before the count by the barrier plus one system-scope fence (cumulative)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int *>(sh.counter), 1u);
      if (prev == gridDim.x - 1) {
        *sh.counter = 0;
        __threadfence_system();
        for (int r = 0; r < sh.n; ++r) st_relaxed_sys(sh.flags[r], sh.step);
      }
    }
  }
}

// ---- stand-alone top-k + softmax on a score matrix ---------------------------------------------------
template <int GROUPS>
__global__ void __launch_bounds__(256) topk_softmax_kernel(const float *__restrict__ scores, int T, int E,
                                                           int k, float *__restrict__ topk_w,
                                                           int *__restrict__ topk_i) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kTokensPerRouteBlock + warp;
  if (b >= T) return;
  float score[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int eg = g * 32 + lane;
    score[g] = (eg < E) ? scores[(size_t)b * E + eg] : -INFINITY;
  }
  float w;
  int id;
  warp_topk_softmax<GROUPS>(score, E, k, lane, w, id);
  if (lane < k) {
    topk_w[(size_t)b * k + lane] = w;
    topk_i[(size_t)b * k + lane] = id;
  }
}

// ---- per-block expert histogram of caller-supplied ids (stand-alone build_offsets) --------------------
__global__ void __launch_bounds__(256) pair_hist_kernel(const int *__restrict__ topk_i, int T, int k, int E,
                                                        int *__restrict__ blk_hist) {
  __shared__ int hist[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int first = blockIdx.x * kTokensPerRouteBlock * k;
  const int n = min(kTokensPerRouteBlock, T - blockIdx.x * kTokensPerRouteBlock) * k;
  for (int q = threadIdx.x; q < n; q += blockDim.x) {
    const int e = topk_i[first + q];
    if (0 <= e && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) blk_hist[(size_t)blockIdx.x * E + e] = hist[e];
}

// ---- prefix sums: expert offsets, per-block bases, token-block prefix for the GEMM tile scheduler -----
// Token blocks of the expert GEMMs: expert e is cut into ceil(rows_e / size) blocks of equal size (a multiple of 16
// rows), size <= 256, the widest MMA.  The persistent CTAs of a GEMM take the (block, feature tile) items round-robin,
// so a launch lasts about `rounds` = ceil(items / CTAs) items, and an item of b rows takes about as long as
// (tb.fixed_rows + b) rows' worth of work (measured 27 / 32 / 37 us at 128 / 176 / 256 rows on both GEMMs: fixed part
// 256).  With few local experts the size decides how full the last round is.  The kernel evaluates
// rounds x (fixed + largest block) for the sizes 256, 240, .., 128 on the row counts at hand, separately for the two
// GEMMs (they differ in items per block; a GEMM given no items keeps 256), and keeps the cheapest (the larger size on
// a tie).  Beyond 8 rounds at size 256 it keeps 256: there the CTAs drift apart, rounds mean little, and fewer, larger
// items win.  tb.force_rows > 0 forces one size for both GEMMs (measurements).
constexpr int kBlockSizeCandidates = 9;  // 256 - 16 c
constexpr int kBalanceMaxRounds = 8;
__device__ __forceinline__ int blocks_of(int rows, int size) { return (rows + size - 1) / size; }

// fw: in the dispatch form the block histograms come from every rank; the kernel first waits for their "routed" flags
// (and only then lets its successor start: a kernel that became resident behind a pending flag wait would sit in its
// own waits for as long as the slowest peer takes).
__global__ void __launch_bounds__(1024) expert_scan_kernel(RouteBuffers rb, int n_blocks, Dims d, TileBalance tb, FlagWait fw) {
  __shared__ __align__(16) int seg_sum4[4096];  // per (team or segment, expert) sums, then their exclusive prefixes
  int *const seg_sum = seg_sum4;
  __shared__ int chunk_sum[1024];
  __shared__ int off_s[kMaxExperts + 1];
  const int E = d.E;
  const int nseg = 1024 / E;
  const int tid = threadIdx.x;
  pdl_wait();
  if (fw.step > 0) wait_all_ranks(fw.flags, fw.world, fw.step, fw.timeout_ns, fw.status, fw.site);
  pdl_launch_dependents();
  if ((E & 3) == 0) {
    // E a multiple of 4 (every real configuration): E/4 threads read one block's histogram row as 16-byte pieces, the
    // 1024 threads form 1024 / (E/4) such teams, and each team owns a contiguous run of blocks, so a pass over all
    // blocks is n_blocks / teams iterations of independent 16-byte loads (8 for 8192 tokens and 32 experts).
    int *const team_sum = seg_sum4;
    const int G = E >> 2, teams = 1024 / G;
    const int team = tid / G, g = tid - team * G;
    const bool active = team < teams;
    const int per = (n_blocks + teams - 1) / teams;
    const int b0 = min(n_blocks, team * per), b1 = min(n_blocks, b0 + per);
    if (active) {
      int4 sum = make_int4(0, 0, 0, 0);
#pragma unroll 4
      for (int b = b0; b < b1; ++b) {
        const int4 h = reinterpret_cast<const int4 *>(rb.blk_hist + (size_t)b * E)[g];
        sum.x += h.x, sum.y += h.y, sum.z += h.z, sum.w += h.w;
      }
      reinterpret_cast<int4 *>(team_sum + team * E)[g] = sum;
    }
    __syncthreads();
    // exclusive prefix over the teams, per expert, in two levels with consecutive lanes on consecutive experts (no
    // bank conflicts): runs of teams ("chunks") are summed by one thread per (chunk, expert), E threads walk the
    // 1024 / E chunk sums, and the chunk threads turn their teams' sums into prefixes
    {
      const int chunks = 1024 / E, tpc = (teams + chunks - 1) / chunks;
      const int chunk = tid / E, e = tid - chunk * E;
      const int c0 = min(teams, chunk * tpc), c1 = min(teams, c0 + tpc);
      const bool has = chunk < chunks;
      if (has) {
        int csum = 0;
        for (int t = c0; t < c1; ++t) csum += team_sum[t * E + e];
        chunk_sum[chunk * E + e] = csum;
      }
      __syncthreads();
      if (tid < E) {
        int run = 0;
        for (int c = 0; c < chunks; ++c) {
          const int v = chunk_sum[c * E + tid];
          chunk_sum[c * E + tid] = run;
          run += v;
        }
        off_s[tid + 1] = run;  // count of expert tid
      }
      __syncthreads();
      if (has) {
        int run = chunk_sum[chunk * E + e];
        for (int t = c0; t < c1; ++t) {
          const int v = team_sum[t * E + e];
          team_sum[t * E + e] = run;
          run += v;
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      off_s[0] = 0;
      for (int x = 0; x < E; ++x) off_s[x + 1] += off_s[x];
    }
    __syncthreads();
    if (tid <= E) rb.offsets[tid] = off_s[tid];
    if (active) {
      const int4 p = reinterpret_cast<const int4 *>(team_sum + team * E)[g];
      int4 run = make_int4(off_s[4 * g] + p.x, off_s[4 * g + 1] + p.y, off_s[4 * g + 2] + p.z, off_s[4 * g + 3] + p.w);
#pragma unroll 4
      for (int b = b0; b < b1; ++b) {
        const int4 h = reinterpret_cast<const int4 *>(rb.blk_hist + (size_t)b * E)[g];
        reinterpret_cast<int4 *>(rb.blk_base + (size_t)b * E)[g] = run;
        run.x += h.x, run.y += h.y, run.z += h.z, run.w += h.w;
      }
    }
  } else {
    const int seg = tid / E, e = tid % E;
    const bool active = seg < nseg;
    const int per = (n_blocks + nseg - 1) / nseg;
    const int b0 = min(n_blocks, seg * per), b1 = min(n_blocks, b0 + per);
    if (active) {
      int sum = 0;
      for (int b = b0; b < b1; ++b) sum += rb.blk_hist[(size_t)b * E + e];
      seg_sum[seg * E + e] = sum;
    }
    __syncthreads();
    if (tid < E) {
      int run = 0;
      for (int s = 0; s < nseg; ++s) {
        const int v = seg_sum[s * E + tid];
        seg_sum[s * E + tid] = run;
        run += v;
      }
      off_s[tid + 1] = run;  // count of expert tid
    }
    __syncthreads();
    if (tid == 0) {
      off_s[0] = 0;
      for (int x = 0; x < E; ++x) off_s[x + 1] += off_s[x];
    }
    __syncthreads();
    if (tid <= E) rb.offsets[tid] = off_s[tid];
    if (active) {
      int run = off_s[e] + seg_sum[seg * E + e];
      for (int b = b0; b < b1; ++b) {
        rb.blk_base[(size_t)b * E + e] = run;
        run += rb.blk_hist[(size_t)b * E + e];
      }
    }
  }
  // token-block prefix of the local experts for the GEMM tile schedulers
  if (rb.tb_prefix == nullptr) return;
  __shared__ int cost_s[2][kBlockSizeCandidates];
  __shared__ int rounds_s[2];  // rounds at the largest size
  const int warp = tid >> 5, lane = tid & 31;
  const bool choose = tb.force_rows <= 0 && tb.ctas > 0;
  if (choose && warp < 2 * kBlockSizeCandidates) {  // one warp per (GEMM, candidate size)
    const int g = warp / kBlockSizeCandidates, c = warp - g * kBlockSizeCandidates;
    const int size = kMaxTileTokens - 16 * c;
    int blocks = 0, largest = 0;
    for (int x = d.e_begin + lane; x < d.e_end; x += 32) {
      const int rows = off_s[x + 1] - off_s[x], nb = blocks_of(rows, size);
      blocks += nb;
      if (nb > 0) largest = max(largest, (blocks_of(rows, nb) + 15) & ~15);
    }
    for (int o = 16; o > 0; o >>= 1) {
      blocks += __shfl_xor_sync(0xffffffffu, blocks, o);
      largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, o));
    }
    if (lane == 0) {
      const long long items = (long long)blocks * (g == 0 ? tb.nft1 : tb.nft2);
      const long long rounds = (items + tb.ctas - 1) / tb.ctas;
      cost_s[g][c] = (int)min(rounds * (tb.fixed_rows + largest), (long long)INT_MAX);
      if (c == 0) rounds_s[g] = (int)min(rounds, (long long)INT_MAX);
    }
  }
  __syncthreads();
  if (lane == 0 && warp < 2) {  // warp 0: gate/up GEMM, warp 1: down GEMM
    int size = kMaxTileTokens;
    if (tb.force_rows > 0) {
      size = min(kMaxTileTokens, max(16, tb.force_rows & ~15));
    } else if (choose && rounds_s[warp] <= kBalanceMaxRounds) {
      int best = cost_s[warp][0];
      for (int c = 1; c < kBlockSizeCandidates; ++c)
        if (cost_s[warp][c] < best) best = cost_s[warp][c], size = kMaxTileTokens - 16 * c;
    }
    int *prefix = warp == 0 ? rb.tb_prefix : rb.tb_prefix2;
    if (prefix != nullptr) {
      int n = 0;
      prefix[0] = 0;
      for (int x = d.e_begin; x < d.e_end; ++x) {
        n += blocks_of(off_s[x + 1] - off_s[x], size);
        prefix[x - d.e_begin + 1] = n;
      }
    }
  }
}

// ---- stable scatter of pair ids (+ optional gather / dispatch of the token rows) ----------------------
// Every block places the pair ids of its 8 tokens.  rd.n == 1: all tokens of the batch, so `sorted` is complete on this
// rank.  Rows: `t` holds the bf16 rows of tokens [t_first, t_first + t_count) (null = ids only); the row of each pair
// of those tokens is copied to its position in x_packed — of this rank, for slots of its own experts (rd.n == 1), or,
// together with its pair id, of the rank that owns the slot's expert (rd.n > 1: the dispatch half of the
// expert-parallel exchange, peer stores; a rank then holds the sorted order of its own experts' rows only).
__global__ void __launch_bounds__(1024) scatter_gather_kernel(const __nv_bfloat16 *__restrict__ t, int t_first, int t_count,
                                                             const int *__restrict__ topk_i, int T, Dims d,
                                                             const int *__restrict__ blk_base,
                                                             int *__restrict__ sorted, RowDispatch rd) {
  __shared__ int ids[kTokensPerRouteBlock * kMaxTopK];
  __shared__ int pos_s[kTokensPerRouteBlock * kMaxTopK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k = d.k;
  // rd.n == 1: one block per 8 tokens of the whole batch (this rank keeps the complete sorted order).  rd.n > 1
  // (dispatch): one block per 8 tokens of this rank's slice only — the pairs of the other tokens are placed by their
  // owners, which store row and pair id straight into this rank's buffers.  (t_first is a multiple of 8.)
  const bool own_only = rd.n > 1;
  const int blk = own_only ? t_first / kTokensPerRouteBlock + (int)blockIdx.x : (int)blockIdx.x;
  const int first = blk * kTokensPerRouteBlock * k;
  const int n = max(0, min(kTokensPerRouteBlock, (own_only ? t_first + t_count : T) - blk * kTokensPerRouteBlock)) * k;
  pdl_wait();
  pdl_launch_dependents();
  for (int q = threadIdx.x; q < kTokensPerRouteBlock * k; q += blockDim.x)
    ids[q] = (q < n) ? topk_i[first + q] : -1;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    const int q = threadIdx.x, e = ids[q];
    int pos = -1;
    if (0 <= e && e < d.E) {
      int rank = 0;
      for (int r = 0; r < q; ++r) rank += (ids[r] == e);
      pos = blk_base[(size_t)blk * d.E + e] + rank;
      (own_only ? rd.sorted[min(rd.n - 1, e / rd.experts_per_rank)] : sorted)[pos] = first + q;
    }
    pos_s[q] = pos;
  }
  __syncthreads();
  // gather: blockDim.x / 256 warps share one token row (its 16-byte chunks interleaved), so that a block
  // keeps enough loads in flight; the row is read once and written to each slot that wants it
  const int wpt = blockDim.x >> 8;            // warps per token
  const int tok = warp / wpt, part = warp - tok * wpt;
  const int b = blk * kTokensPerRouteBlock + tok;
  if (t != nullptr && b < T && b >= t_first && b < t_first + t_count) {
    const int nchunk = d.H >> 3;
    const uint4 *src = reinterpret_cast<const uint4 *>(t + (size_t)(b - t_first) * d.H);
    uint4 *dst[kMaxTopK];
#pragma unroll
    for (int j = 0; j < kMaxTopK; ++j) {
      dst[j] = nullptr;
      if (j < k) {
        const int e = ids[tok * k + j], pos = pos_s[tok * k + j];
        if (pos >= 0) {
          if (rd.n > 1) dst[j] = reinterpret_cast<uint4 *>(rd.xp[min(rd.n - 1, e / rd.experts_per_rank)]) + (size_t)pos * nchunk;
          else if (e >= d.e_begin && e < d.e_end) dst[j] = reinterpret_cast<uint4 *>(rd.xp[0]) + (size_t)pos * nchunk;
        }
      }
    }
#pragma unroll 4
    for (int c = part * 32 + lane; c < nchunk; c += 32 * wpt) {
      const uint4 v = __ldg(src + c);
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j)
        if (dst[j] != nullptr) dst[j][c] = v;
    }
  }
  if (rd.step > 0) {  // stores ordered before the count by the barrier plus one system-scope fence (cumulative)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int *>(rd.counter), 1u);
      if (prev == gridDim.x - 1) {
        *rd.counter = 0;
        __threadfence_system();
        for (int r = 0; r < rd.n; ++r) st_relaxed_sys(rd.flags[r], rd.step);
      }
    }
  }
}

// ---- combine: x[b,:] (+)= sum over this rank's slots j = 0..k-1 (ascending) of y_pairs[b*k+j,:] --------
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ y_pairs,
                                                      const int *__restrict__ topk_i, int T, Dims d,
                                                      float *__restrict__ x, int residual) {
  const int h4 = d.H >> 2;
  const size_t total = (size_t)T * h4;
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int b = (int)(i / h4), c = (int)(i % h4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool first = true;
    for (int j = 0; j < d.k; ++j) {
      const int e = topk_i[(size_t)b * d.k + j];
      if (e >= d.e_begin && e < d.e_end) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(y_pairs) + ((size_t)b * d.k + j) * h4 + c);
        if (first) {
          acc = v;
          first = false;
        } else {
          acc.x += v.x;
          acc.y += v.y;
          acc.z += v.z;
          acc.w += v.w;
        }
      }
    }
    float4 *xp = reinterpret_cast<float4 *>(x) + i;
    if (residual) {
      float4 o = *xp;
      o.x += acc.x;
      o.y += acc.y;
      o.z += acc.z;
      o.w += acc.w;
      *xp = o;
    } else {
      *xp = acc;
    }
  }
}

// ---- launchers -------------------------------------------------------------------------------------------
static inline int route_blocks(int T) { return (T + kTokensPerRouteBlock - 1) / kTokensPerRouteBlock; }

cudaError_t launch_router_topk(const float *partials, int n_splits, const float *br, int T, int first_token, const Dims &d,
                               const RouteBuffers &rb, const RouteShare &share, cudaStream_t s) {
  const int groups = (d.E + 31) / 32;
  const int nb = route_blocks(T);
  const dim3 grid(nb > 0 ? nb : 1), block(256);  // a rank without tokens still raises its flag
  cudaError_t err = cudaSuccess;
#define GPTOSS_ROUTER_CASE(G)                                                            \
  case G:                                                                                \
    err = launch_chain(router_topk_kernel<G>, grid, block, 0, s, partials, n_splits, br, T, first_token, d, rb, share); \
    break;
  switch (groups) {
    GPTOSS_ROUTER_CASE(1)
    GPTOSS_ROUTER_CASE(2)
    GPTOSS_ROUTER_CASE(3)
    GPTOSS_ROUTER_CASE(4)
    GPTOSS_ROUTER_CASE(5)
    GPTOSS_ROUTER_CASE(6)
    GPTOSS_ROUTER_CASE(7)
    GPTOSS_ROUTER_CASE(8)
    default:
      return cudaErrorInvalidValue;
  }
#undef GPTOSS_ROUTER_CASE
  return err;
}

cudaError_t launch_topk_softmax(const float *scores, int T, int E, int k, float *topk_w, int *topk_i,
                                cudaStream_t s) {
  const int groups = (E + 31) / 32;
  const dim3 grid(route_blocks(T)), block(256);
#define GPTOSS_TOPK_CASE(G)                                                   \
  case G:                                                                     \
    topk_softmax_kernel<G><<<grid, block, 0, s>>>(scores, T, E, k, topk_w, topk_i); \
    break;
  count_launch();
  switch (groups) {
    GPTOSS_TOPK_CASE(1)
    GPTOSS_TOPK_CASE(2)
    GPTOSS_TOPK_CASE(3)
    GPTOSS_TOPK_CASE(4)
    GPTOSS_TOPK_CASE(5)
    GPTOSS_TOPK_CASE(6)
    GPTOSS_TOPK_CASE(7)
    GPTOSS_TOPK_CASE(8)
    default:
      return cudaErrorInvalidValue;
  }
#undef GPTOSS_TOPK_CASE
  return cudaGetLastError();
}

cudaError_t launch_pair_hist(const int *topk_i, int T, const Dims &d, int *blk_hist, cudaStream_t s) {
  count_launch();
  pair_hist_kernel<<<route_blocks(T), 256, 0, s>>>(topk_i, T, d.k, d.E, blk_hist);
  return cudaGetLastError();
}

cudaError_t launch_expert_scan(const RouteBuffers &rb, int T, const Dims &d, const TileBalance &tb, const FlagWait &fw,
                               cudaStream_t s) {
  return launch_chain(expert_scan_kernel, dim3(1), dim3(1024), 0, s, rb, route_blocks(T), d, tb, fw);
}

cudaError_t launch_scatter_gather(const __nv_bfloat16 *t, int t_first, int t_count, const int *topk_i, int T, const Dims &d,
                                  const int *blk_base, int *sorted, const RowDispatch &rd, cudaStream_t s) {
  const int blocks = rd.n > 1 ? (t_count + kTokensPerRouteBlock - 1) / kTokensPerRouteBlock : route_blocks(T);
  return launch_chain(scatter_gather_kernel, dim3(blocks > 0 ? blocks : 1), dim3(t ? 1024 : 256), 0, s, t, t_first, t_count,
                      topk_i, T, d, blk_base, sorted, rd);
}

cudaError_t launch_combine(const float *y_pairs, const int *topk_i, int T, const Dims &d, float *x,
                           int residual, int sm_count, cudaStream_t s) {
  const size_t total = (size_t)T * (d.H >> 2);
  int blocks = (int)((total + 255) / 256);
  const int cap = sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return launch_chain(combine_kernel, dim3(blocks), dim3(256), 0, s, y_pairs, topk_i, T, d, x, residual);
}

// ---- allocation-free grouping -----------------------------------------------------------------------------
// Scratch of gptoss_moe_build_offsets_noalloc: per-block expert histograms, per-block bases and the
// token-block prefix, in one statically allocated device array (every device that loads the library holds
// these 1 MiB + 1 KiB until the process exits).  In host code `g_noalloc_scratch` is only a handle: the
// device address is obtained with cudaGetSymbolAddress, once per device, below.
constexpr int kNoAllocMaxEntries = 128 * 1024;  // route blocks x experts
static __device__ __align__(256) int g_noalloc_scratch[2 * kNoAllocMaxEntries + kMaxExperts + 1];

}  // namespace gptoss

namespace {
thread_local char g_noalloc_error[256] = "";
int noalloc_fail(int code, const char *msg) {
  snprintf(g_noalloc_error, sizeof g_noalloc_error, "%s", msg);
  return code;
}
constexpr int kMaxDevices = 64;
int *g_noalloc_ptr[kMaxDevices];  // device address of g_noalloc_scratch, per device (0 = not resolved yet)
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" const char *gptoss_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int gptoss_moe_build_offsets_noalloc(int T, int n_experts, int top_k, const int *topk_i_dev,
                                                 int *offsets_dev, int *sorted_pair_ids_dev, void *stream) {
  using namespace gptoss;
  if (T < 0 || n_experts <= 0 || n_experts > kMaxExperts || top_k <= 0 || top_k > kMaxTopK)
    return noalloc_fail(GPTOSS_ERR_BAD_ARG, "T, n_experts (1..256) or top_k (1..8) out of range");
  if (!offsets_dev || (T > 0 && (!topk_i_dev || !sorted_pair_ids_dev)))
    return noalloc_fail(GPTOSS_ERR_BAD_ARG, "null pointer");
  const long long n_blocks = ((long long)T + kTokensPerRouteBlock - 1) / kTokensPerRouteBlock;
  if (n_blocks * n_experts > kNoAllocMaxEntries)
    return noalloc_fail(GPTOSS_ERR_BAD_ARG,
                        "batch too large for the static scratch: ceil(T/8) * n_experts must not exceed 131072 "
                        "(use gptoss_moe_build_offsets with a context instead)");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    if (cudaMemsetAsync(offsets_dev, 0, (n_experts + 1) * sizeof(int), s) != cudaSuccess)
      return noalloc_fail(GPTOSS_ERR_CUDA, "cudaMemsetAsync failed");
    return GPTOSS_OK;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return noalloc_fail(GPTOSS_ERR_CUDA, "cudaGetDevice failed or device index above 63");
  int *scratch;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {  // first call on this device: resolve the symbol with this device current
      void *p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p) return noalloc_fail(GPTOSS_ERR_CUDA, "cudaGetSymbolAddress failed");
      g_noalloc_ptr[dev] = static_cast<int *>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  Dims d{0, 0, n_experts, top_k, 0, n_experts, 0.f};
  RouteBuffers rb{};
  rb.blk_hist = scratch;
  rb.blk_base = scratch + kNoAllocMaxEntries;
  rb.tb_prefix = nullptr;  // no GEMM follows: the token-block prefix is not computed
  rb.offsets = offsets_dev;
  rb.sorted = sorted_pair_ids_dev;
  // every entry of the scratch that the scan and the scatter read is first written by this call, so
  // nothing has to start at zero
  if (launch_pair_hist(topk_i_dev, T, d, rb.blk_hist, s) != cudaSuccess ||
      launch_expert_scan(rb, T, d, TileBalance{0}, FlagWait{}, s) != cudaSuccess ||
      launch_scatter_gather(nullptr, 0, 0, topk_i_dev, T, d, rb.blk_base, rb.sorted, RowDispatch{}, s) != cudaSuccess)
    return noalloc_fail(GPTOSS_ERR_CUDA, "kernel launch failed");
  return GPTOSS_OK;
}
