// Grouped expert GEMMs of the MoE block on the 5th-generation tensor cores (sm_100a):
//   mlp1:  gate_up[p, c] = SwiGLU( W1g_e[c,:] . x[p,:] + b1g_e[c],  W1u_e[c,:] . x[p,:] + b1u_e[c] )   (bf16 out)
//   mlp2:  y_pairs[pair(p), f] = gate_weight(pair) * ( W2_e[f,:] . gate_up[p,:] + b2_e[f] )           (fp32 out)
// for the rows p of each local expert e (rows are contiguous per expert after the counting sort).
//
// Decode-first orientation: the WEIGHT tile is the UMMA "A" operand (M = 128 output features, one per
// TMEM lane) and the TOKENS are the "B" operand (N = 16..256 in steps of 16), so an expert with few
// rows wastes at most 15 columns instead of most of a 128-row tile, and every weight byte is read
// from HBM exactly once per token block.  Both operands are K-major bf16 (the checkpoint stores
// weights out-feature-major, i.e. already K-contiguous), staged by TMA with the 128-byte swizzle.
//
// One persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (one elected
// thread) and TMEM owner, warps 2-5 = epilogue (one TMEM lane quadrant each).  Tiles are
// (expert, token block of <= 256 rows, 128-feature tile), enumerated from the device-built
// token-block prefix, so no row count ever travels to the host.
//
// Every mbarrier wait is bounded: when a wait gives up the CTA raises an abort flag, records a
// time-out in the status words, drains its outstanding copies, frees its TMEM and returns.
#include "kernels.cuh"

namespace gptoss {

namespace {

constexpr int kATileBytes = kTileF * kBlockK * 2;           // 16 KiB: 128 features x 64 k
constexpr int kBChunkBytes = kTokChunk * kBlockK * 2;       //  8 KiB: 64 tokens x 64 k
constexpr int kBTileBytes = kMaxTileTokens * kBlockK * 2;   // 32 KiB
constexpr int kGemmThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 20;

template <int NA>
struct TileCfg {
  static constexpr int kStages = (NA == 2) ? 3 : 4;
  static constexpr int kStageBytes = NA * kATileBytes + kBTileBytes;
  static constexpr int kAccBuffers = (NA == 2) ? 1 : 2;
};

struct Ctrl {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int tbp[kMaxExperts + 1];
  int off[kMaxExperts + 1];
  int pair_s[2][kMaxTileTokens];
  float w_s[2][kMaxTileTokens];
};

struct Tile {
  int e;        // local expert
  int f0;       // first output feature
  int row0;     // first row (sorted order)
  int n_valid;  // rows in the tile
};

// ---- PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA abort flag + the global status) on time-out or
// if the CTA is already aborting.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctrl *ctrl, int *status, int site) {
  volatile int *ab = &ctrl->abort;
  if (*ab) return false;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *ab) return false;
  }
  *ab = 1;
  if (atomicCAS(status, 0, kDevErrTimeout) == 0) {
    status[1] = site;
    status[2] = (int)blockIdx.x;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, bf16 x bf16 -> fp32, M = 128, K = 16, N from the instruction descriptor
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrive once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 64 bf16 x R rows writes): 8-row groups 1024 bytes apart (SBO), LBO unused
// (=1), descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).  Stepping K by 16 elements inside
// the swizzle row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor: fp32 accumulate, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileF >> 4) << 24);
}

__device__ __forceinline__ bool decode_tile(int idx, const Ctrl *c, int n_local, int nft, int &cur, Tile &t) {
  while (cur < n_local && idx >= c->tbp[cur + 1] * nft) ++cur;
  if (cur >= n_local) return false;
  const int r = idx - c->tbp[cur] * nft;
  const int nb = c->tbp[cur + 1] - c->tbp[cur];
  const int ft = r / nb, tb = r - ft * nb;
  t.e = cur;
  t.f0 = ft * kTileF;
  t.row0 = c->off[cur] + tb * kMaxTileTokens;
  t.n_valid = min(kMaxTileTokens, c->off[cur + 1] - t.row0);
  return true;
}

__device__ __forceinline__ float swiglu(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
}

template <int NA>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmArgs a) {
  using Cfg = TileCfg<NA>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  Ctrl *ctrl = reinterpret_cast<Ctrl *>(smem_raw + (tiles_base - raw) + Cfg::kStages * Cfg::kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_local = a.n_local, nft = a.n_feat_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), kEpilogueThreads);
    }
    ctrl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i <= n_local; i += blockDim.x) {
    ctrl->tbp[i] = a.tb_prefix[i];
    ctrl->off[i] = a.offsets[a.e_begin + i];
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->tbp[n_local] * nft;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int cur = 0;
      uint32_t armed = 0, last_par = 0;  // per-stage: was it armed, and with which phase parity
      Tile t;
      for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
        if (!decode_tile(idx, ctrl, n_local, nft, cur, t)) break;
        const int n_mma = max(16, (t.n_valid + 15) & ~15);
        const int n_chunks = (n_mma + kTokChunk - 1) / kTokChunk;
        const uint32_t tx = NA * kATileBytes + n_chunks * kBChunkBytes;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1u, ctrl, a.status, 0x100 | stage);
          const uint32_t bar = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = tiles_base + stage * Cfg::kStageBytes;
          armed |= 1u << stage;
          last_par = (last_par & ~(1u << stage)) | (phase << stage);
          mbar_expect_tx(bar, tx);
          tma_load_3d(sa, &a.map_w, bar, kb * kBlockK, t.f0, t.e * NA);
          if (NA == 2) tma_load_3d(sa + kATileBytes, &a.map_w, bar, kb * kBlockK, t.f0, t.e * NA + 1);
          const uint32_t sb = sa + NA * kATileBytes;
          for (int c = 0; c < n_chunks; ++c)
            tma_load_2d(sb + c * kBChunkBytes, &a.map_act, bar, kb * kBlockK, t.row0 + c * kTokChunk);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // drain: every armed stage must have landed before the CTA may exit (bounded)
      for (int s = 0; s < Cfg::kStages; ++s) {
        if (armed & (1u << s)) {
          const uint32_t par = (last_par >> s) & 1u;
          for (uint32_t i = 0; i < kSpinLimit; ++i)
            if (mbar_try_wait(smem_u32(&ctrl->full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int cur = 0, acc = 0;
      uint32_t acc_phase = 0;
      Tile t;
      for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
        if (!decode_tile(idx, ctrl, n_local, nft, cur, t)) break;
        const int n_mma = max(16, (t.n_valid + 15) & ~15);
        const uint32_t idesc = umma_idesc(n_mma);
        mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1u, ctrl, a.status, 0x200 | acc);
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(acc * kMaxTileTokens);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->full[stage]), phase, ctrl, a.status, 0x300 | stage);
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * Cfg::kStageBytes;
          const uint64_t da0 = smem_desc_sw128(sa);
          const uint64_t da1 = smem_desc_sw128(sa + kATileBytes);
          const uint64_t db = smem_desc_sw128(sa + NA * kATileBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            umma_bf16(d0, da0 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            if (NA == 2) umma_bf16(d0 + kMaxTileTokens, da1 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          umma_commit(smem_u32(&ctrl->empty[stage]));
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit(smem_u32(&ctrl->tmem_full[acc]));
        if (++acc == Cfg::kAccBuffers) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int et = threadIdx.x - 64;        // 0..127
    int cur = 0, acc = 0;
    uint32_t acc_phase = 0;
    Tile t;
    for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
      if (!decode_tile(idx, ctrl, n_local, nft, cur, t)) break;
      const int f = t.f0 + q * 32 + lane;
      const bool f_ok = f < a.n_feat;
      if (NA == 1) {
        for (int n = et; n < t.n_valid; n += kEpilogueThreads) {
          const int pair = a.sorted[t.row0 + n];
          ctrl->pair_s[acc][n] = pair;
          ctrl->w_s[acc][n] = a.topk_w[pair];
        }
        epilogue_bar_sync();
      }
      const float bias0 = f_ok ? a.bias_a[(size_t)t.e * a.n_feat + f] : 0.f;
      const float bias1 = (NA == 2 && f_ok) ? a.bias_b[(size_t)t.e * a.n_feat + f] : 0.f;
      mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, ctrl, a.status, 0x400 | acc);
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kMaxTileTokens);
      for (int c0 = 0; c0 < t.n_valid; c0 += 16) {
        uint32_t r0[16], r1[16];
        tmem_ld16(tbase + c0, r0);
        if (NA == 2) tmem_ld16(tbase + kMaxTileTokens + c0, r1);
        tmem_ld_wait();
        if (f_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = c0 + j;
            if (n < t.n_valid) {
              if (NA == 2) {
                const float v = swiglu(__uint_as_float(r0[j]) + bias0, __uint_as_float(r1[j]) + bias1, a.limit);
                a.gate_up[(size_t)(t.row0 + n) * a.n_feat + f] = __float2bfloat16_rn(v);
              } else {
                const float v = (__uint_as_float(r0[j]) + bias0) * ctrl->w_s[acc][n];
                a.y_pairs[(size_t)ctrl->pair_s[acc][n] * a.n_feat + f] = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
      if (++acc == Cfg::kAccBuffers) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int NA>
cudaError_t launch_grouped(const GemmArgs &a, int sm_count, cudaStream_t s) {
  using Cfg = TileCfg<NA>;
  const size_t smem = (size_t)Cfg::kStages * Cfg::kStageBytes + 1024 + sizeof(Ctrl);
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<NA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  grouped_gemm_kernel<NA><<<sm_count, kGemmThreads, smem, s>>>(a);
  return cudaGetLastError();
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

cudaError_t get_encode_fn(EncodeTiledFn *fn) {
  static EncodeTiledFn cached = nullptr;
  if (!cached) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (q != cudaDriverEntryPointSuccess || !p) return cudaErrorNotSupported;
    cached = reinterpret_cast<EncodeTiledFn>(p);
  }
  *fn = cached;
  return cudaSuccess;
}

}  // namespace

cudaError_t launch_grouped_mlp1(const GemmArgs &a, int sm_count, cudaStream_t s) {
  return launch_grouped<2>(a, sm_count, s);
}
cudaError_t launch_grouped_mlp2(const GemmArgs &a, int sm_count, cudaStream_t s) {
  return launch_grouped<1>(a, sm_count, s);
}

cudaError_t encode_weight_map(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows, uint64_t slabs) {
  EncodeTiledFn fn;
  cudaError_t e = get_encode_fn(&fn);
  if (e != cudaSuccess) return e;
  const cuuint64_t dims[3] = {K, rows, slabs};
  const cuuint64_t strides[2] = {K * 2, K * rows * 2};
  const cuuint32_t box[3] = {(cuuint32_t)kBlockK, (cuuint32_t)kTileF, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t encode_act_map(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows) {
  EncodeTiledFn fn;
  cudaError_t e = get_encode_fn(&fn);
  if (e != cudaSuccess) return e;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)kTokChunk};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace gptoss
