// Bandwidth-bound kernels around the MoE block that a decode step needs end to end: embedding gather,
// RMSNorm (with the residual add fused), QKV split + rotary embedding + KV-cache store, single-query
// attention with learned sinks and a sliding window, and the per-row argmax of the logits.
//
// Each restates a piece of the reference CPU model (run.cpp) with the rounding points of the reference GPU
// engine: activations that feed a GEMM are bf16, the residual stream, norms, softmax and accumulations fp32,
// the KV cache bf16 (config.hpp KV16).
#include <cfloat>

#include "kernels.cuh"

namespace gptoss {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// x[b,:] = float(embedding[token_b,:])   (run.cpp:515-517)
__global__ void __launch_bounds__(256) embed_kernel(const int *__restrict__ tokens, const __nv_bfloat16 *__restrict__ table,
                                                    int H, int vocab, float *__restrict__ x) {
  const int b = blockIdx.x;
  pdl_wait();
  int tok = tokens[b];
  tok = min(max(tok, 0), vocab - 1);
  const uint16_t *row = reinterpret_cast<const uint16_t *>(table) + (size_t)tok * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) x[(size_t)b * H + i] = bf16_bits_to_f32(row[i]);
  pdl_launch_dependents();  // at the end: the next kernel's blocks should not take room from this one's
}

// Optional residual update followed by RMSNorm (run.cpp:304-317, 611-623), one block per row:
//   if (add) x[b,:] += add[b,:];   out[b,:] = bf16( w[:] * (x[b,:] * rsqrt(mean(x^2) + 1e-5)) )
__global__ void __launch_bounds__(256) residual_rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ add,
                                                               const float *__restrict__ w, int H,
                                                               __nv_bfloat16 *__restrict__ out) {
  __shared__ double part[8];
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * H;
  __nv_bfloat16 *o = out + row;
  residual_rmsnorm_row(
      x + row, add ? add + row : nullptr, w, H, part, [&](int i, uint2 v) { reinterpret_cast<uint2 *>(o)[i] = v; },
      [&](int i, __nv_bfloat16 v) { o[i] = v; });
  pdl_launch_dependents();
}

// qkv[b, :] = (q heads | k heads | v heads), bias already added (run.cpp:534-557).  Rotates q and k with the
// cos/sin of position `pos` (half-split pairs: element i pairs with i + hd/2), writes q as fp32 and k, v as
// bf16 into the caches at [b, kv_head, pos, i]: the rows that one (sequence, kv head) attends to are contiguous.
__global__ void __launch_bounds__(256) qkv_rope_store_kernel(const float *__restrict__ qkv, const float *__restrict__ cos_t,
                                                             const float *__restrict__ sin_t, int pos, int nq, int nkv,
                                                             int hd, int S, float *__restrict__ q_out,
                                                             __nv_bfloat16 *__restrict__ k_cache,
                                                             __nv_bfloat16 *__restrict__ v_cache,
                                                             const int *__restrict__ cache_rows,
                                                             const int *__restrict__ pos_rows) {
  pdl_wait();
  const int b = blockIdx.x;
  const int cb = cache_rows ? cache_rows[b] : b;  // cache row of sequence b (a compacted batch keeps its rows)
  if (pos_rows) pos = pos_rows[b];                // sequences that joined the batch later are at their own positions
  const int half = hd >> 1, hp = half >> 1;  // hp: pairs of adjacent rotation indices per head (hd is 32 or 64)
  const int qdim = nq * hd, kvdim = nkv * hd;
  const float *row = qkv + (size_t)b * (qdim + 2 * kvdim);
  const float2 *cs = reinterpret_cast<const float2 *>(cos_t + (size_t)pos * half);
  const float2 *sn = reinterpret_cast<const float2 *>(sin_t + (size_t)pos * half);
  for (int i = threadIdx.x; i < (nq + nkv) * hp; i += blockDim.x) {
    const int h = i / hp, j = 2 * (i - h * hp);  // heads 0..nq-1 are q, nq.. are k; elements j, j+1 and their partners
    const float *src = row + (size_t)h * hd;
    const float2 x1 = *reinterpret_cast<const float2 *>(src + j), x2 = *reinterpret_cast<const float2 *>(src + j + half);
    const float2 c = cs[j >> 1], s = sn[j >> 1];
    const float2 o1 = make_float2(x1.x * c.x - x2.x * s.x, x1.y * c.y - x2.y * s.y);
    const float2 o2 = make_float2(x2.x * c.x + x1.x * s.x, x2.y * c.y + x1.y * s.y);
    if (h < nq) {
      float *dst = q_out + (size_t)b * qdim + h * hd + j;
      *reinterpret_cast<float2 *>(dst) = o1;
      *reinterpret_cast<float2 *>(dst + half) = o2;
    } else {
      __nv_bfloat16 *dst = k_cache + (((size_t)cb * nkv + (h - nq)) * S + pos) * hd + j;
      *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(o1.x, o1.y);
      *reinterpret_cast<__nv_bfloat162 *>(dst + half) = __floats2bfloat162_rn(o2.x, o2.y);
    }
  }
  const float *vsrc = row + qdim + kvdim;
  for (int i = threadIdx.x; i < (kvdim >> 2); i += blockDim.x) {
    const int h = (4 * i) / hd, j = 4 * i - h * hd;
    const float4 v = reinterpret_cast<const float4 *>(vsrc)[i];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(v_cache + (((size_t)cb * nkv + h) * S + pos) * hd + j) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
  }
  pdl_launch_dependents();
}

// ---- single-query attention (run.cpp:565-607) -------------------------------------------------------------------
// One "problem" is one (sequence, kv head): the KVM query heads of the group against the K/V rows [t_lo, pos]
// of that head.  The op is bound by reading the cache (every K and V row once), so all per-position arithmetic
// runs on the tensor cores with warp-level mma.sync m16n8k16 (the M = 128 tcgen05 shapes have no use for 8 query
// rows): rows of the A operand = query heads (8 of 16 used), and
//   scores  S[head, pos]  = Q[head, dim] . K[pos, dim]      (B operand = K rows as they lie in the cache)
//   output  O[head, dim] += P[head, pos] . V[pos, dim]      (A = the probabilities, taken from the S accumulators
//                                                            in registers; B = V rows, pairs of positions packed
//                                                            with one byte-permute each)
// Q and P are fp32 values: each is split into a bf16 head (tile rows 0..7) and a bf16 remainder (rows 8..15, which 8
// query heads leave free), and the two accumulator halves are added, so the products carry ~16 mantissa bits and
// accumulate in fp32 at no extra MMA (K and V are bf16 in the cache, exactly).  The order of
// the contraction index is free, which is used to give every thread 16-byte contiguous loads: thread (g = lane/4,
// c = lane%4) owns the dims [HD/4*c, HD/4*(c+1)) of K row g of each 8-position tile, and the dims
// [HD/8*g, HD/8*(g+1)) of the four V rows {2c, 2c+1, 2c+8, 2c+9} of each 16-position step.
// A block's 4 warps serve G problems with 4/G warps each (positions dealt out in chunks of 32); online softmax per
// head; the partial (max, sum, accumulator) are merged through shared memory, where the learned sink joins the
// denominator only (run.cpp:588-591).
// a0/a2: rows 0..7 (k 0..7 / 8..15 of the step), a1/a3: rows 8..15; c[0..1]: rows 0..7, c[2..3]: rows 8..15
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (x, y) -> bf16 pair of the rounded values (hi) and of the remainders (lo); x in the low half
__device__ __forceinline__ void split_pair(float x, float y, uint32_t &hi, uint32_t &lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  const __nv_bfloat16 xl = __float2bfloat16_rn(x - __bfloat162float(xh)), yl = __float2bfloat16_rn(y - __bfloat162float(yh));
  hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
  lo = (uint32_t)__bfloat16_as_ushort(xl) | ((uint32_t)__bfloat16_as_ushort(yl) << 16);
}

template <int HD, int G>
__global__ void __launch_bounds__(128) attention_kernel(const float *__restrict__ q, const __nv_bfloat16 *__restrict__ k_cache,
                                                        const __nv_bfloat16 *__restrict__ v_cache,
                                                        const float *__restrict__ sinks, int pos, int t_lo, int nq,
                                                        int nkv, int kvm, int S, int n_problems,
                                                        __nv_bfloat16 *__restrict__ out,
                                                        const int *__restrict__ cache_rows,
                                                        const int *__restrict__ pos_rows, int window) {
  constexpr int PS = 4 / G;    // warps (position groups) per problem
  constexpr int D4 = HD / 4;   // K dims per thread
  constexpr int KS = HD / 16;  // k-steps of the score MMA
  constexpr int DV = HD / 8;   // V dims per thread = n-tiles of the output MMA
  __shared__ float m_s[4][8], l_s[4][8], f_s[4][8];
  __shared__ __align__(16) float acc_s[4][8][HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int grp = warp / PS, ps = warp % PS;
  const int prob = blockIdx.x * G + grp;
  const bool active = prob < n_problems;
  const int b = active ? prob / nkv : 0, kvh = active ? prob % nkv : 0;
  pdl_wait();  // q and this position's K/V rows come from the kernel before
  const int cb = cache_rows ? cache_rows[b] : b;  // cache row of sequence b
  if (pos_rows) {  // every sequence at its own position (and the window that ends there)
    pos = pos_rows[b];
    t_lo = window > 0 && pos - window + 1 > 0 ? pos - window + 1 : 0;
  }
  uint32_t qh[KS][2], ql[KS][2];
#pragma unroll
  for (int s = 0; s < KS; ++s) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active && g < kvm) v = *reinterpret_cast<const float4 *>(q + ((size_t)b * nq + (size_t)kvh * kvm + g) * HD + D4 * c + 4 * s);
    split_pair(v.x, v.y, qh[s][0], ql[s][0]);
    split_pair(v.z, v.w, qh[s][1], ql[s][1]);
  }
  const float scale = 1.0f / sqrtf((float)HD);
  // cache rows of this problem: [b, kvh, t, :], contiguous over t
  const uint16_t *kbase = reinterpret_cast<const uint16_t *>(k_cache) + ((size_t)cb * nkv + kvh) * S * HD + D4 * c;
  const uint16_t *vbase = reinterpret_cast<const uint16_t *>(v_cache) + ((size_t)cb * nkv + kvh) * S * HD + DV * g;

  float m_run = -FLT_MAX, l_part = 0.f;  // l_part: this thread's share of the denominator (its own positions)
  float o[DV][4];
#pragma unroll
  for (int i = 0; i < DV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // The loads run one step ahead of their use: the K rows of the next chunk are requested as soon as the scores
  // of this one have left the K registers, the V rows once the output MMAs have left the V registers, so that a
  // warp always has a chunk's worth of rows in flight while it computes.  Rows past `pos` re-read row `pos` (their
  // scores are masked).
  uint32_t kr[4][D4 / 2], vr[2][4][DV / 2];
  auto load_k = [&](int t0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 *src = reinterpret_cast<const uint4 *>(kbase + (size_t)min(t0 + 8 * j + g, pos) * HD);
#pragma unroll
      for (int u = 0; u < D4 / 8; ++u) {
        const uint4 x = src[u];
        kr[j][4 * u] = x.x, kr[j][4 * u + 1] = x.y, kr[j][4 * u + 2] = x.z, kr[j][4 * u + 3] = x.w;
      }
    }
  };
  auto load_v = [&](int t0) {
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = 16 * s + 2 * c + (r & 1) + 8 * (r >> 1);
        const uint16_t *src = vbase + (size_t)min(t0 + row, pos) * HD;
        if (DV == 8) {
          const uint4 x = *reinterpret_cast<const uint4 *>(src);
          vr[s][r][0] = x.x, vr[s][r][1] = x.y, vr[s][r][DV / 2 - 2] = x.z, vr[s][r][DV / 2 - 1] = x.w;
        } else {
          const uint2 x = *reinterpret_cast<const uint2 *>(src);
          vr[s][r][0] = x.x, vr[s][r][1] = x.y;
        }
      }
  };
  const int t_first = t_lo + 32 * ps;
  if (active && t_first <= pos) {
    load_k(t_first);
    load_v(t_first);
    for (int t0 = t_first; t0 <= pos; t0 += 32 * PS) {
      const int t_next = t0 + 32 * PS;
      // scores of head g at positions t0 + 8j + 2c + {0,1}: rows 0..7 of the tile carry the bf16 heads of the
      // queries, rows 8..15 their remainders, so that the sum of the two accumulator halves is the fp32-query product
      float p[4][2];
      float cmax = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KS; ++s) mma_bf16_16816(acc, qh[s][0], ql[s][0], qh[s][1], ql[s][1], kr[j][2 * s], kr[j][2 * s + 1]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[j][e] = (t0 + 8 * j + 2 * c + e <= pos) ? (acc[e] + acc[2 + e]) * scale : -FLT_MAX;
          cmax = fmaxf(cmax, p[j][e]);
        }
      }
      if (t_next <= pos) load_k(t_next);
      cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 1));
      cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 2));
      const float m_new = fmaxf(m_run, cmax);  // finite: every chunk holds at least position t0 <= pos
      const float corr = __expf(m_run - m_new);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[j][e] = (t0 + 8 * j + 2 * c + e <= pos) ? __expf(p[j][e] - m_new) : 0.f;
          psum += p[j][e];
        }
      l_part = l_part * corr + psum;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < DV; ++i) o[i][0] *= corr, o[i][1] *= corr, o[i][2] *= corr, o[i][3] *= corr;
#pragma unroll
      for (int s = 0; s < 2; ++s) {  // probabilities: heads in rows 0..7, remainders in rows 8..15, as for the queries
        uint32_t a0h, a0l, a2h, a2l;
        split_pair(p[2 * s][0], p[2 * s][1], a0h, a0l);
        split_pair(p[2 * s + 1][0], p[2 * s + 1][1], a2h, a2l);
#pragma unroll
        for (int i = 0; i < DV; ++i) {  // n-tile i, column g = dim DV*g + i
          const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
          const uint32_t b0 = __byte_perm(vr[s][0][i >> 1], vr[s][1][i >> 1], sel);
          const uint32_t b1 = __byte_perm(vr[s][2][i >> 1], vr[s][3][i >> 1], sel);
          mma_bf16_16816(o[i], a0h, a0l, a2h, a2l, b0, b1);
        }
      }
      if (t_next <= pos) load_v(t_next);
    }
  }
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 1);
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 2);
  pdl_launch_dependents();  // after the main loop: the next kernel's blocks should not take room from this one's
  if (PS == 1) {
    // one warp per problem: nothing to merge.  Thread (g, c) holds head g, dims [2*DV*c, 2*DV*(c+1)) (accumulator
    // columns 2c and 2c+1 of n-tile i are dims DV*2c + i and DV*(2c+1) + i); the sink joins the denominator only
    if (active && g < kvm) {
      const float sink = sinks[kvh * kvm + g];
      const float mx = fmaxf(sink, m_run);
      const float cw = __expf(m_run - mx);
      const float inv = cw / (__expf(sink - mx) + l_part * cw);
      uint32_t pk[DV];
#pragma unroll
      for (int i = 0; i < DV; i += 2) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn((o[i][0] + o[i][2]) * inv, (o[i + 1][0] + o[i + 1][2]) * inv);
        const __nv_bfloat162 hi = __floats2bfloat162_rn((o[i][1] + o[i][3]) * inv, (o[i + 1][1] + o[i + 1][3]) * inv);
        pk[i >> 1] = *reinterpret_cast<const uint32_t *>(&lo);
        pk[(DV >> 1) + (i >> 1)] = *reinterpret_cast<const uint32_t *>(&hi);
      }
      uint32_t *dst = reinterpret_cast<uint32_t *>(out + (size_t)b * nq * HD + (size_t)(kvh * kvm + g) * HD + 2 * DV * c);
      if (DV == 8) {
        reinterpret_cast<uint4 *>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        reinterpret_cast<uint4 *>(dst)[1] = make_uint4(pk[DV - 4], pk[DV - 3], pk[DV - 2], pk[DV - 1]);
      } else {
        reinterpret_cast<uint4 *>(dst)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
    return;
  }
  if (c == 0) {
    m_s[warp][g] = m_run;
    l_s[warp][g] = l_part;
  }
#pragma unroll
  for (int i = 0; i < DV; ++i) {  // accumulator columns 2c, 2c+1 of n-tile i = dims DV*2c + i, DV*(2c+1) + i
    acc_s[warp][g][DV * (2 * c) + i] = o[i][0] + o[i][2];
    acc_s[warp][g][DV * (2 * c + 1) + i] = o[i][1] + o[i][3];
  }
  __syncthreads();
  // merge of the position groups: per (problem, head) the common maximum and denominator (with the sink), folded into
  // one factor per position group; then every thread scales and adds 4 dims of one head
  if (threadIdx.x < G * 8) {
    const int gr = threadIdx.x >> 3, h = threadIdx.x & 7;
    const int pr = blockIdx.x * G + gr;
    if (pr < n_problems && h < kvm) {
      const float sink = sinks[(pr % nkv) * kvm + h];
      float mx = sink;
#pragma unroll
      for (int w = 0; w < PS; ++w) mx = fmaxf(mx, m_s[gr * PS + w][h]);
      float denom = __expf(sink - mx);
      float cw[PS];
#pragma unroll
      for (int w = 0; w < PS; ++w) {
        cw[w] = __expf(m_s[gr * PS + w][h] - mx);
        denom += l_s[gr * PS + w][h] * cw[w];
      }
#pragma unroll
      for (int w = 0; w < PS; ++w) f_s[gr * PS + w][h] = cw[w] / denom;
    }
  }
  __syncthreads();
  constexpr int HD4 = HD / 4;
  for (int idx = threadIdx.x; idx < G * 8 * HD4; idx += blockDim.x) {
    const int gr = idx / (8 * HD4), h = (idx / HD4) & 7, d4 = idx % HD4;
    const int pr = blockIdx.x * G + gr;
    if (pr >= n_problems || h >= kvm) continue;
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < PS; ++w) {
      const float f = f_s[gr * PS + w][h];
      const float4 v = *reinterpret_cast<const float4 *>(&acc_s[gr * PS + w][h][4 * d4]);
      num.x = fmaf(v.x, f, num.x), num.y = fmaf(v.y, f, num.y), num.z = fmaf(v.z, f, num.z), num.w = fmaf(v.w, f, num.w);
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(num.x, num.y), hi = __floats2bfloat162_rn(num.z, num.w);
    *reinterpret_cast<uint2 *>(out + (size_t)(pr / nkv) * nq * HD + (size_t)((pr % nkv) * kvm + h) * HD + 4 * d4) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
  }
}

// next[b] = index of the FIRST maximum of logits[b,:]   (run.cpp:739-750).  Like the reference's scan (which starts
// from element 0 and replaces it only on a strict '>'), a row without any comparable maximum (all -inf or NaN, or a
// NaN in front) yields index 0, never an index outside [0, V).
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ next) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int b = blockIdx.x;
  pdl_wait();
  const float *row = logits + (size_t)b * V;
  float best = -FLT_MAX;
  int idx = 0x7fffffff;
  const int v4 = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) ? (V >> 2) : 0;  // 16-byte loads where the row allows
  for (int i = threadIdx.x; i < v4; i += blockDim.x) {
    const float4 q = reinterpret_cast<const float4 *>(row)[i];
    const float vals[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (vals[e] > best) {  // ascending index per thread: strict '>' keeps the lowest index
        best = vals[e];
        idx = 4 * i + e;
      }
  }
  for (int i = 4 * v4 + threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) {
      best = v;
      idx = i;
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    bv[threadIdx.x >> 5] = best;
    bi[threadIdx.x >> 5] = idx;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = (threadIdx.x < (blockDim.x >> 5)) ? bv[threadIdx.x] : -FLT_MAX;
    idx = (threadIdx.x < (blockDim.x >> 5)) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
      }
    }
    if (threadIdx.x == 0) next[b] = (idx == 0x7fffffff || row[0] != row[0]) ? 0 : idx;
  }
}

// Second stage of the fused classifier argmax: per sequence the first maximum over the per-vocabulary-block partials
// (blocks ascend in vocabulary id, so among equal values the one from the lower block — the lower id — wins).  A
// block of 32 warps serves 32 sequences: lane = sequence (coalesced reads of val/at [block][sequence]), the warps share
// out the vocabulary blocks and merge through shared memory.  A sequence without any comparable logit gets 0.
__global__ void __launch_bounds__(1024) argmax_partials_kernel(const float *__restrict__ val, const int *__restrict__ at,
                                                               int n_blocks, int B, int *__restrict__ next) {
  __shared__ float best_s[32][33];
  __shared__ int idx_s[32][33];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.x * 32 + lane;
  float best = -FLT_MAX;
  int idx = 0x7fffffff;
  if (b < B)
    for (int i = warp; i < n_blocks; i += 32) {  // ascending blocks per warp: strict '>' keeps the first maximum
      const float v = val[(size_t)i * B + b];
      if (v > best) best = v, idx = at[(size_t)i * B + b];
    }
  best_s[warp][lane] = best;
  idx_s[warp][lane] = idx;
  __syncthreads();
  if (warp == 0 && b < B) {
    for (int w = 1; w < 32; ++w) {
      const float v = best_s[w][lane];
      const int j = idx_s[w][lane];
      if (v > best || (v == best && j < idx)) best = v, idx = j;
    }
    next[b] = idx == 0x7fffffff ? 0 : idx;
  }
  pdl_launch_dependents();
}

__global__ void iota_ones_kernel(int *__restrict__ iota, float *__restrict__ ones, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    iota[i] = i;
    ones[i] = 1.0f;
  }
}

}  // namespace

cudaError_t launch_embed(const int *tokens, const __nv_bfloat16 *table, int B, int H, int vocab, float *x, cudaStream_t s) {
  return launch_chain(embed_kernel, dim3(B), dim3(256), 0, s, tokens, table, H, vocab, x);
}
cudaError_t launch_residual_rmsnorm(float *x, const float *add, const float *w, int B, int H, __nv_bfloat16 *out,
                                    cudaStream_t s) {
  return launch_chain(residual_rmsnorm_kernel, dim3(B), dim3(256), 0, s, x, add, w, H, out);
}
cudaError_t launch_qkv_rope_store(const float *qkv, const float *cos_t, const float *sin_t, int pos, int B, int nq, int nkv,
                                  int hd, int S, float *q_out, __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache,
                                  const int *cache_rows, const int *pos_rows, cudaStream_t s) {
  return launch_chain(qkv_rope_store_kernel, dim3(B), dim3(256), 0, s, qkv, cos_t, sin_t, pos, nq, nkv, hd, S, q_out, k_cache,
                      v_cache, cache_rows, pos_rows);
}
cudaError_t launch_attention(const float *q, const __nv_bfloat16 *k_cache, const __nv_bfloat16 *v_cache, const float *sinks,
                             int pos, int t_lo, int B, int nq, int nkv, int hd, int S, __nv_bfloat16 *out, const int *cache_rows,
                             const int *pos_rows, int window, cudaStream_t s) {
  const int kv_mul = nq / nkv;
  if (kv_mul < 1 || kv_mul > 8 || kv_mul * nkv != nq) return cudaErrorInvalidValue;  // query rows of one MMA tile
  const int n_prob = B * nkv;
  // Warps per problem by the context length alone (1 up to 512 positions: a warp streams its problem's rows front
  // to back with the loads one chunk ahead, which beats sharing them out; 2 up to 2048; else 4): the split fixes the
  // order of the softmax accumulation, so it must not depend on the batch, or a sequence would get different
  // low-order bits in a large batch, a small one, or a slice of one on another GPU.  With per-sequence positions the
  // caller passes sequences of one length class per launch, and `pos` / `t_lo` are those of the longest context.
  const int g = 4 / attention_warps_per_problem(pos - t_lo);
  const int grid = (n_prob + g - 1) / g;
#define GPTOSS_ATT_CASE(HD, G)                                                                                             \
  if (hd == HD && g == G) {                                                                                                \
    return launch_chain(attention_kernel<HD, G>, dim3(grid), dim3(128), 0, s, q, k_cache, v_cache, sinks, pos, t_lo, nq, nkv,   \
                        kv_mul, S, n_prob, out, cache_rows, pos_rows, window);                                             \
  }
  GPTOSS_ATT_CASE(64, 4)
  GPTOSS_ATT_CASE(64, 2)
  GPTOSS_ATT_CASE(64, 1)
  GPTOSS_ATT_CASE(32, 4)
  GPTOSS_ATT_CASE(32, 2)
  GPTOSS_ATT_CASE(32, 1)
#undef GPTOSS_ATT_CASE
  return cudaErrorInvalidValue;  // head_dim must be 32 or 64
}
cudaError_t launch_argmax(const float *logits, int B, int V, int *next, cudaStream_t s) {
  return launch_chain(argmax_kernel, dim3(B), dim3(1024), 0, s, logits, V, next);
}
cudaError_t launch_argmax_partials(const float *val, const int *at, int n_blocks, int B, int *next, cudaStream_t s) {
  return launch_chain(argmax_partials_kernel, dim3((B + 31) / 32), dim3(1024), 0, s, val, at, n_blocks, B, next);
}
cudaError_t launch_iota_ones(int *iota, float *ones, int n, cudaStream_t s) {
  iota_ones_kernel<<<(n + 255) / 256, 256, 0, s>>>(iota, ones, n);
  return cudaGetLastError();
}

}  // namespace gptoss
