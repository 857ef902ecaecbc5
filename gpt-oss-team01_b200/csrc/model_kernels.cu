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
  int tok = tokens[b];
  tok = min(max(tok, 0), vocab - 1);
  const uint16_t *row = reinterpret_cast<const uint16_t *>(table) + (size_t)tok * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) x[(size_t)b * H + i] = bf16_bits_to_f32(row[i]);
}

// Optional residual update followed by RMSNorm (run.cpp:304-317, 611-623):
//   if (add) x[b,:] += add[b,:]            (projection output incl. its bias)
//   out[b,:] = bf16( w[:] * (x[b,:] * rsqrt(mean(x^2) + 1e-5)) )
// One block per row; the sum of squares is accumulated in fp32 per thread and reduced in double.
__global__ void __launch_bounds__(256) residual_rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ add,
                                                               const float *__restrict__ w, int H,
                                                               __nv_bfloat16 *__restrict__ out) {
  __shared__ double part[8];
  const int b = blockIdx.x;
  float *xr = x + (size_t)b * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = xr[i];
    if (add) {
      v += add[(size_t)b * H + i];
      xr[i] = v;
    }
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = (double)ss;
  __syncthreads();
  double tot = 0.0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += part[i];
  const float inv = 1.0f / sqrtf((float)(tot / H + 1e-5));
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)b * H + i] = __float2bfloat16_rn(w[i] * (inv * xr[i]));
}

// qkv[b, :] = (q heads | k heads | v heads), bias already added (run.cpp:534-557).  Rotates q and k with the
// cos/sin of position `pos` (half-split pairs: element i pairs with i + hd/2), writes q as fp32 and k, v as
// bf16 into the caches at [b, pos, kv_head*hd + i].
__global__ void __launch_bounds__(256) qkv_rope_store_kernel(const float *__restrict__ qkv, const float *__restrict__ cos_t,
                                                             const float *__restrict__ sin_t, int pos, int nq, int nkv,
                                                             int hd, int S, float *__restrict__ q_out,
                                                             __nv_bfloat16 *__restrict__ k_cache,
                                                             __nv_bfloat16 *__restrict__ v_cache) {
  const int b = blockIdx.x;
  const int half = hd >> 1;
  const int qdim = nq * hd, kvdim = nkv * hd;
  const float *row = qkv + (size_t)b * (qdim + 2 * kvdim);
  const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
  for (int i = threadIdx.x; i < (nq + nkv) * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;  // heads 0..nq-1 are q, nq.. are k
    const float *src = row + (size_t)h * hd;
    const float x1 = src[j], x2 = src[j + half], c = cs[j], s = sn[j];
    const float o1 = x1 * c - x2 * s, o2 = x2 * c + x1 * s;
    if (h < nq) {
      q_out[(size_t)b * qdim + h * hd + j] = o1;
      q_out[(size_t)b * qdim + h * hd + j + half] = o2;
    } else {
      __nv_bfloat16 *dst = k_cache + ((size_t)b * S + pos) * kvdim + (h - nq) * hd;
      dst[j] = __float2bfloat16_rn(o1);
      dst[j + half] = __float2bfloat16_rn(o2);
    }
  }
  const float *vsrc = row + qdim + kvdim;
  __nv_bfloat16 *vdst = v_cache + ((size_t)b * S + pos) * kvdim;
  for (int i = threadIdx.x; i < kvdim; i += blockDim.x) vdst[i] = __float2bfloat16_rn(vsrc[i]);
}

// Single-query attention for one (sequence, kv head) (run.cpp:565-607).  Memory-bound: every K and V row of
// the cache is read once per kv head and serves the query heads of the group from registers.  The block's
// 4 warps are laid out as HS head groups x (4/HS) position groups: with a long context (HS = 1) every warp
// serves all KVM query heads and the positions [t_lo, pos] are dealt out in chunks of 32; with a short one the
// heads are split over the warps instead, so that no warp idles.  Within a chunk one lane owns one position
// for the scores (its K row in registers, the queries broadcast from shared memory) and the lanes own the head
// dimension for the values; online softmax per head; the partial (max, sum, accumulator) of the position
// groups are merged through shared memory, where the learned sink joins the denominator only
// (run.cpp:588-591).  HD = head_dim (32 or 64), KVM = query heads per kv head.
template <int HD, int KVM, int HS>
__global__ void __launch_bounds__(128) attention_kernel(const float *__restrict__ q, const __nv_bfloat16 *__restrict__ k_cache,
                                                        const __nv_bfloat16 *__restrict__ v_cache,
                                                        const float *__restrict__ sinks, int pos, int t_lo, int nq,
                                                        int nkv, int S, __nv_bfloat16 *__restrict__ out) {
  constexpr int DPL = HD / 32;   // output dims per lane
  constexpr int NW = 4;
  constexpr int PS = NW / HS;    // position groups
  constexpr int HPW = KVM / HS;  // query heads per warp
  __shared__ __align__(16) float q_s[KVM * HD];
  __shared__ float m_s[PS][KVM], l_s[PS][KVM], acc_s[PS][KVM][HD];
  const int b = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = warp % HS, ps = warp / HS, h0 = hs * HPW;
  const int kvdim = nkv * HD;
  for (int i = threadIdx.x; i < KVM * HD; i += blockDim.x) q_s[i] = q[(size_t)b * nq * HD + (size_t)kvh * KVM * HD + i];
  __syncthreads();
  const float scale = 1.0f / sqrtf((float)HD);
  const uint16_t *kbase = reinterpret_cast<const uint16_t *>(k_cache) + (size_t)b * S * kvdim + kvh * HD;
  const uint16_t *vbase = reinterpret_cast<const uint16_t *>(v_cache) + (size_t)b * S * kvdim + kvh * HD;

  float m[HPW], l[HPW], acc[HPW][DPL];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    m[h] = -FLT_MAX;
    l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }
  for (int t0 = t_lo + 32 * ps; t0 <= pos; t0 += 32 * PS) {
    const int t = t0 + lane;
    const bool valid = t <= pos;
    const int n_here = min(32, pos - t0 + 1);
    float kf[HD];
    if (valid) {
      const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)t * kvdim);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        const uint4 kv4 = kr[c];
        const uint32_t w[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          kf[c * 8 + 2 * e] = __uint_as_float(w[e] << 16);
          kf[c * 8 + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < HD; ++i) kf[i] = 0.f;
    }
    // values: all rows of the chunk are requested before the first is used (the loads are independent; issued
    // one by one behind their uses they would serialise on memory latency)
    uint32_t vv[32];
#pragma unroll
    for (int tt = 0; tt < 32; ++tt) {
      const uint16_t *vr = vbase + (size_t)(t0 + min(tt, n_here - 1)) * kvdim;
      vv[tt] = (DPL == 2) ? *reinterpret_cast<const uint32_t *>(vr + 2 * lane) : (uint32_t)vr[lane];
    }
    float p[HPW];
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
      const float4 *q4 = reinterpret_cast<const float4 *>(q_s + (h0 + h) * HD);
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < HD / 4; ++c) {
        const float4 qv = q4[c];
        dot = fmaf(qv.x, kf[4 * c], dot);
        dot = fmaf(qv.y, kf[4 * c + 1], dot);
        dot = fmaf(qv.z, kf[4 * c + 2], dot);
        dot = fmaf(qv.w, kf[4 * c + 3], dot);
      }
      const float sc = valid ? dot * scale : -FLT_MAX;
      const float m_new = fmaxf(m[h], warp_max(sc));
      const float corr = __expf(m[h] - m_new);
      p[h] = valid ? __expf(sc - m_new) : 0.f;
      l[h] = l[h] * corr + warp_sum(p[h]);
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[h][d] *= corr;
      m[h] = m_new;
    }
#pragma unroll
    for (int tt = 0; tt < 32; ++tt) {
      if (tt < n_here) {
        float v[DPL];
        v[0] = __uint_as_float(vv[tt] << 16);
        if (DPL == 2) v[DPL - 1] = __uint_as_float(vv[tt] & 0xffff0000u);
#pragma unroll
        for (int h = 0; h < HPW; ++h) {
          const float pt = __shfl_sync(0xffffffffu, p[h], tt);
#pragma unroll
          for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(pt, v[d], acc[h][d]);
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    if (lane == 0) {
      m_s[ps][h0 + h] = m[h];
      l_s[ps][h0 + h] = l[h];
    }
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc_s[ps][h0 + h][DPL * lane + d] = acc[h][d];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < KVM * HD; i += blockDim.x) {
    const int h = i / HD, d = i - h * HD;
    const float sink = sinks[kvh * KVM + h];
    float mx = sink;
#pragma unroll
    for (int w = 0; w < PS; ++w) mx = fmaxf(mx, m_s[w][h]);
    float denom = __expf(sink - mx), num = 0.f;
#pragma unroll
    for (int w = 0; w < PS; ++w) {
      const float c = __expf(m_s[w][h] - mx);
      denom += l_s[w][h] * c;
      num += acc_s[w][h][d] * c;
    }
    out[(size_t)b * nq * HD + (size_t)(kvh * KVM + h) * HD + d] = __float2bfloat16_rn(num / denom);
  }
}

// next[b] = index of the FIRST maximum of logits[b,:]   (run.cpp:739-750)
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ next) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int b = blockIdx.x;
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
    if (threadIdx.x == 0) next[b] = idx;
  }
}

__global__ void iota_ones_kernel(int *__restrict__ iota, float *__restrict__ ones, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    iota[i] = i;
    ones[i] = 1.0f;
  }
}

}  // namespace

cudaError_t launch_embed(const int *tokens, const __nv_bfloat16 *table, int B, int H, int vocab, float *x, cudaStream_t s) {
  embed_kernel<<<B, 256, 0, s>>>(tokens, table, H, vocab, x);
  return cudaGetLastError();
}
cudaError_t launch_residual_rmsnorm(float *x, const float *add, const float *w, int B, int H, __nv_bfloat16 *out,
                                    cudaStream_t s) {
  residual_rmsnorm_kernel<<<B, 256, 0, s>>>(x, add, w, H, out);
  return cudaGetLastError();
}
cudaError_t launch_qkv_rope_store(const float *qkv, const float *cos_t, const float *sin_t, int pos, int B, int nq, int nkv,
                                  int hd, int S, float *q_out, __nv_bfloat16 *k_cache, __nv_bfloat16 *v_cache,
                                  cudaStream_t s) {
  qkv_rope_store_kernel<<<B, 256, 0, s>>>(qkv, cos_t, sin_t, pos, nq, nkv, hd, S, q_out, k_cache, v_cache);
  return cudaGetLastError();
}
cudaError_t launch_attention(const float *q, const __nv_bfloat16 *k_cache, const __nv_bfloat16 *v_cache, const float *sinks,
                             int pos, int t_lo, int B, int nq, int nkv, int hd, int S, __nv_bfloat16 *out, cudaStream_t s) {
  const int kv_mul = nq / nkv;
  const int n_chunks = (pos - t_lo) / 32 + 1;
  int hs = n_chunks >= 4 ? 1 : (n_chunks >= 2 ? 2 : 4);  // short context: split the heads over the warps
  if (hs > kv_mul) hs = kv_mul;
  const dim3 grid(B, nkv);
#define GPTOSS_ATT_CASE(HD, KVM, HS)                                                                                 \
  if (hd == HD && kv_mul == KVM && hs == HS) {                                                                       \
    attention_kernel<HD, KVM, HS><<<grid, 128, 0, s>>>(q, k_cache, v_cache, sinks, pos, t_lo, nq, nkv, S, out);      \
    return cudaGetLastError();                                                                                       \
  }
#define GPTOSS_ATT_HD(HD)    \
  GPTOSS_ATT_CASE(HD, 8, 1)  \
  GPTOSS_ATT_CASE(HD, 8, 2)  \
  GPTOSS_ATT_CASE(HD, 8, 4)  \
  GPTOSS_ATT_CASE(HD, 4, 1)  \
  GPTOSS_ATT_CASE(HD, 4, 2)  \
  GPTOSS_ATT_CASE(HD, 4, 4)  \
  GPTOSS_ATT_CASE(HD, 2, 1)  \
  GPTOSS_ATT_CASE(HD, 2, 2)  \
  GPTOSS_ATT_CASE(HD, 1, 1)
  GPTOSS_ATT_HD(64)
  GPTOSS_ATT_HD(32)
#undef GPTOSS_ATT_HD
#undef GPTOSS_ATT_CASE
  return cudaErrorInvalidValue;  // head_dim must be 32 or 64, 1/2/4/8 query heads per kv head
}
cudaError_t launch_argmax(const float *logits, int B, int V, int *next, cudaStream_t s) {
  argmax_kernel<<<B, 1024, 0, s>>>(logits, V, next);
  return cudaGetLastError();
}
cudaError_t launch_iota_ones(int *iota, float *ones, int n, cudaStream_t s) {
  iota_ones_kernel<<<(n + 255) / 256, 256, 0, s>>>(iota, ones, n);
  return cudaGetLastError();
}

}  // namespace gptoss
