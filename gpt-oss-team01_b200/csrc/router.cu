// Router GEMM on the tensor cores: partial[s][b][e] = sum over the k-blocks of split s of t[b,:] . Wr[e,:]
// (bf16 x bf16 -> fp32).  Tokens are the UMMA M side (128 per CTA, one TMEM lane each), experts the N side
// (E rounded up to 16, at most 256), K is split over gridDim.y CTAs (4 or 8, by the size of the whole batch) so that
// even 1024 tokens keep 32 to 64 SMs streaming; the splits are summed in a fixed order by the top-k kernel, so the scores are
// bit-identical on every launch and on every rank.  Same warp roles and bounded waits as the expert GEMMs.  A CTA computes one tile:
// when a wait gives up, every later wait of the CTA returns at once, the loops run out (their copies and MMAs touch only
// this CTA's ring and accumulator; the single-thread loops do not branch on the result of a wait, which was measured
// to slow the expert GEMMs by 8-15 %), the MMA thread waits for what it has issued, and the host sees the time-out; the
// scores of that tile are then meaningless.
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace gptoss {

namespace {

constexpr int kRouterThreads = 192;
constexpr int kRouterATile = 128 * kBlockK * 2;  // 16 KiB: 128 tokens x 64 k
constexpr int kRouterMaxStages = 8;
constexpr int kRouterSmemBudget = 200 * 1024;

struct RouterCtrl {
  uint64_t full[kRouterMaxStages];
  uint64_t empty[kRouterMaxStages];
  uint64_t tmem_full;
  uint64_t mma_done;  // abort path only: completion of every MMA issued so far
  uint32_t tmem_base;
  int abort;
};

__global__ void __launch_bounds__(kRouterThreads, 1) router_gemm_kernel(const __grid_constant__ RouterArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  RouterCtrl *ctrl = reinterpret_cast<RouterCtrl *>(smem_raw + (tiles_base - raw) + a.stages * a.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb0 = blockIdx.y * a.k_blocks_per_split;
  const int kb1 = min(a.k_blocks, kb0 + a.k_blocks_per_split);
  const int row0 = blockIdx.x * 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctrl->tmem_full), 1);
    mbar_init(smem_u32(&ctrl->mma_done), 1);
    ctrl->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), a.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();  // the activations may come from the kernel just before this one
      pdl_launch_dependents();
      int stage = 0;
      uint32_t phase = 0, armed = 0, last_par = 0;
      const uint32_t tx = kRouterATile + a.n_cols * kBlockK * 2;
      for (int kb = kb0; kb < kb1; ++kb) {
        mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1u, &ctrl->abort, a.status, 0x1100 | stage);
        const uint32_t bar = smem_u32(&ctrl->full[stage]);
        const uint32_t sa = tiles_base + stage * a.stage_bytes;
        armed |= 1u << stage;
        last_par = (last_par & ~(1u << stage)) | (phase << stage);
        mbar_expect_tx(bar, tx);
        tma_load_2d(sa, &a.map_t, bar, kb * kBlockK, row0);
        tma_load_2d(sa + kRouterATile, &a.map_wr, bar, kb * kBlockK, 0);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      for (int s = 0; s < a.stages; ++s)
        if (armed & (1u << s)) {
          const uint32_t par = (last_par >> s) & 1u;
          for (uint32_t i = 0; i < kSpinLimit; ++i)
            if (mbar_try_wait(smem_u32(&ctrl->full[s]), par)) break;
        }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t idesc = umma_idesc(a.n_cols);
      for (int kb = kb0; kb < kb1; ++kb) {
        mbar_wait(smem_u32(&ctrl->full[stage]), phase, &ctrl->abort, a.status, 0x1300 | stage);
        tc_fence_after();
        const uint32_t sa = tiles_base + stage * a.stage_bytes;
        const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + kRouterATile);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k)
          umma_bf16(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(smem_u32(&ctrl->empty[stage]));
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (*reinterpret_cast<volatile int *>(&ctrl->abort)) {
        // aborting: the MMAs issued so far must have retired before TMEM and the ring are given up (bounded)
        umma_commit(smem_u32(&ctrl->mma_done));
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(smem_u32(&ctrl->mma_done), 0)) break;
      } else {
        umma_commit(smem_u32(&ctrl->tmem_full));
      }
    }
  } else {
    const int q = warp & 3;
    const int b = row0 + q * 32 + lane;
    mbar_wait(smem_u32(&ctrl->tmem_full), 0, &ctrl->abort, a.status, 0x1400);
    tc_fence_after();
    float *dst = a.partials + ((size_t)blockIdx.y * a.T + b) * a.E;
    const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16);
    for (int c0 = 0; c0 < a.n_cols; c0 += 16) {
      uint32_t r[16];
      tmem_ld16(tbase + c0, r);
      tmem_ld_wait();
      if (b < a.T) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < a.E) dst[c0 + j] = __uint_as_float(r[j]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, a.tmem_cols);
  }
}

}  // namespace

// Fills the launch geometry of `a` (splits, stages, shared memory) for T tokens and launches.
cudaError_t launch_router_gemm(RouterArgs a, int max_splits, cudaStream_t s) {
  const int n_tiles = (a.T + 127) / 128;
  const int splits = router_splits_for(a.split_T > 0 ? a.split_T : a.T, a.k_blocks, max_splits);
  a.k_blocks_per_split = (a.k_blocks + splits - 1) / splits;
  a.stage_bytes = kRouterATile + ((a.n_cols * kBlockK * 2 + 1023) & ~1023);
  a.stages = kRouterSmemBudget / a.stage_bytes;
  if (a.stages > kRouterMaxStages) a.stages = kRouterMaxStages;
  if (a.stages > a.k_blocks_per_split) a.stages = a.k_blocks_per_split < 2 ? 2 : a.k_blocks_per_split;
  a.tmem_cols = 32;
  while (a.tmem_cols < a.n_cols) a.tmem_cols <<= 1;
  const size_t smem = (size_t)a.stages * a.stage_bytes + 1024 + sizeof(RouterCtrl);
  cudaError_t e = cudaFuncSetAttribute(router_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_chain(router_gemm_kernel, dim3(n_tiles, splits), dim3(kRouterThreads), smem, s, a);
}

// Split-K factor of the router GEMM, from the size of the WHOLE batch (a rank that routes only its slice of a batch
// passes the batch size, so that a token's partial sums are added in the same order whoever routes it: otherwise the
// scores would differ in their last bits and a slice-routing rank could pick another expert than a rank routing
// everything).  Up to 2048 tokens: 8 splits (1024 tokens: 64 CTAs with 6 k-blocks each).  Beyond: 4 — a CTA's fixed
// cost (TMEM allocation, barrier set-up) then outweighs shorter k-loops for a full batch (8192 tokens: 91 us with 8
// splits, 79 us with 1), while a 1024-token slice of such a batch still gets 32 CTAs with 12 k-blocks each instead
// of 8 CTAs walking all 45.
int router_splits_for(int T, int k_blocks, int max_splits) {
  int splits = T <= 2048 ? 8 : 4;
  if (splits > max_splits) splits = max_splits;
  if (splits > k_blocks) splits = k_blocks;
  if (splits < 1) splits = 1;
  const int per = (k_blocks + splits - 1) / splits;
  return (k_blocks + per - 1) / per;
}

}  // namespace gptoss
