// The grouped expert GEMMs of grouped_gemm.cu with a PAIR of CTAs (a cluster of two SMs) per work item:
// tcgen05.mma with cta_group::2, M = 256.
//
// What it changes: one CTA per item stages 2 weight tiles and ALL token rows of the block per k-block; in a pair each
// CTA stages its own 2 weight tiles and only HALF of the token rows, and the tensor cores of both SMs read both halves:
// the same MMA work per SM for a quarter less staged bytes at 256 rows, and a ring that is one stage deeper.
// What it gives: identical results (tests compare the two kernels bit for bit), and no speed: with 128 to 1024 rows per
// expert both GEMMs take the same time or 2-8 % more than with one CTA per item (4 experts x 1024 rows: 116 + 68 us
// against 115 + 65; 32 x 1024: 986 + 478 against 919 + 462; 32 x 128: 220 + 112 against 199 + 108).  At hundreds of rows
// per expert the one-CTA GEMMs already run at 0.85 of the sustained cuBLAS bf16 rate under the power cap, so staging is
// not what bounds them; at few rows the weights are streamed from HBM and 148 independent streams beat 74.  The kernels
// therefore run only on request (GPTOSS_PAIR=1).
//
// Work split: an item is (expert, token block, pair of feature tiles).  CTA r of the pair owns the features
// f0 + r * kTileFeat ..: its weight tiles are rows of the A operand that only it loads, and its 128 TMEM lanes receive
// exactly its features for ALL token columns, so the epilogue is the one-CTA epilogue with a shifted feature index.
// Token rows: CTA r loads rows [r * n/2, (r + 1) * n/2) of the block (n = rows rounded up to 32).
//
// Protocol (all waits bounded, as in the one-CTA kernel):
//   full[s]    (leader's)  1 arrival (the leader's expect_tx of BOTH CTAs' bytes) + the bytes of both CTAs' copies
//   empty[s]   (each CTA's own)  the leader's tcgen05.commit, multicast to both CTAs
//   tmem_full  (each CTA's own)  the leader's tcgen05.commit after the last k-block, multicast
//   tmem_empty (leader's)  one arrival per epilogue thread of BOTH CTAs (the peer's arrive over the cluster)
// A CTA that gives up raises its peer's abort flag as well; both CTAs meet at a cluster barrier before TMEM is freed, so
// neither leaves while the other may still read its shared memory or signal its barriers.
#include <cstdlib>

#include "gemm_tile.cuh"

namespace gptoss {

using namespace gemm;

namespace {

template <bool GLU, bool OUT16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    grouped_gemm_pair_kernel(const __grid_constant__ GemmArgs a) {
  static_assert(!OUT16 || !GLU, "bf16 rows are an option of the row GEMM only");
  using Cfg = TileCfg<2, GLU>;
  using CtrlT = Ctrl<2, GLU>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t ring = smem_u32(smem_raw);
  CtrlT *ctrl = reinterpret_cast<CtrlT *>(smem_raw + kRingBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_local = a.n_local, nft = a.n_feat_tiles;  // nft: PAIRS of feature tiles
  const uint32_t cta_rank = cluster_cta_rank();
  const bool leader = cta_rank == 0;
  const int pair_id = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
  const uint32_t peer_abort = map_to_cta(smem_u32(&ctrl->abort), cta_rank ^ 1u);

  if (threadIdx.x == 0) {
    ctrl->max_rows = 0;
    if (ring & 1023u) {  // the ring must be 1024-byte aligned for the 128-byte swizzle
      ctrl->abort = 1;
      if (atomicCAS(a.status, 0, kDevErrTimeout) == 0) a.status[1] = 0x901;
    } else {
      ctrl->abort = 0;
    }
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), 2 * kEpilogueThreads);
    }
    mbar_init(smem_u32(&ctrl->mma_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  {
    int mx = 0;
    for (int i = threadIdx.x; i <= n_local; i += blockDim.x) {
      ctrl->tbp[i] = a.tb_prefix[i];
      const int o = a.offsets[a.e_begin + i];
      ctrl->off[i] = o;
      if (i < n_local) {  // rows of this expert's largest tile (see decode_tile)
        const int rows = a.offsets[a.e_begin + i + 1] - o, nb = a.tb_prefix[i + 1] - a.tb_prefix[i];
        if (nb > 0) mx = max(mx, min(kMaxTileTokens, (((rows + nb - 1) / nb) + 15) & ~15));
      }
    }
    if (mx > 0) atomicMax(&ctrl->max_rows, mx);
  }
  if (warp == 1) {  // the same warp of both CTAs
    tmem_alloc_pair(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers exist, both have their TMEM, before anything crosses between them
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->abort ? 0 : ctrl->tbp[n_local] * nft;
  // ring geometry of this launch: two weight tiles + this CTA's half of the token rows of the largest block
  const int half_rows_max = ((ctrl->max_rows + 31) & ~31) >> 1;
  const int b_rows = max(kTokChunk, (half_rows_max + kTokChunk - 1) / kTokChunk * kTokChunk);
  const int stage_bytes = Cfg::kAStageBytes + b_rows * kBlockK * 2;
  const int n_stages = min(kMaxStages, kRingBytes / stage_bytes);
  const int f_shift = (int)cta_rank * Cfg::kTileFeat;  // this CTA's features inside the pair's item

  if (warp == 0) {
    // ===================== TMA producer (each CTA: its weight tiles, its half of the token rows) ==============
    if (lane == 0) {
      int stage = 0, cur = 0;
      uint32_t phase = 0, armed = 0, last_par = 0;
      Tile t;
      const uint64_t pol_w = l2_policy_evict_first();
      pdl_wait();
      pdl_launch_dependents();
      for (int idx = pair_id; idx < total_tiles; idx += n_pairs) {
        if (aborting(&ctrl->abort) || !decode_tile<2 * Cfg::kTileFeat, false>(idx, ctrl, n_local, nft, cur, t)) break;
        const int f0 = t.f0 + f_shift;
        const int n_mma = max(32, (t.n_valid + 31) & ~31);
        const int half = n_mma >> 1;
        const int n_chunks = (half + kTokChunk - 1) / kTokChunk;
        const uint32_t tx = Cfg::kAStageBytes + n_chunks * kBChunkBytes;  // bytes of ONE CTA's copies
        const int row_first = t.row0 + (int)cta_rank * half;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1u, &ctrl->abort, a.status, 0x500 | stage);
          const uint32_t sa = ring + stage * stage_bytes;
          const uint32_t bar = map_to_cta(smem_u32(&ctrl->full[stage]), 0);  // the leader counts both CTAs' bytes
          if (leader) {
            armed |= 1u << stage;
            last_par = (last_par & ~(1u << stage)) | (phase << stage);
            mbar_expect_tx(smem_u32(&ctrl->full[stage]), 2 * tx);
          }
          tma_load_3d_hint_pair(sa, &a.map_w, bar, kb * kBlockK, f0, t.e * Cfg::kSlabs, pol_w);
          // GLU: the up rows of the same features (next slab); else the next 128 features (zero-filled past the end)
          tma_load_3d_hint_pair(sa + kATileBytes, &a.map_w, bar, kb * kBlockK, GLU ? f0 : f0 + kTileF,
                                GLU ? t.e * Cfg::kSlabs + 1 : t.e * Cfg::kSlabs, pol_w);
          const uint32_t sb = sa + Cfg::kAStageBytes;
          for (int c = 0; c < n_chunks; ++c)
            tma_load_2d_pair(sb + c * kBChunkBytes, &a.map_act, bar, kb * kBlockK, row_first + c * kTokChunk);
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (aborting(&ctrl->abort)) st_cluster_u32(peer_abort, 1u);
      // drain (leader: its barriers count the copies of both CTAs): every armed stage must have landed before the
      // CTAs may exit (bounded); the peer is held by the cluster barrier below
      for (int s = 0; s < n_stages; ++s)
        if (armed & (1u << s)) {
          const uint32_t par = (last_par >> s) & 1u;
          for (uint32_t i = 0; i < kSpinLimit; ++i)
            if (mbar_try_wait(smem_u32(&ctrl->full[s]), par)) break;
        }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader only) =====================
    if (lane == 0 && leader) {
      int stage = 0, cur = 0;
      uint32_t phase = 0, acc_phase = 0;
      Tile t;
      for (int idx = pair_id; idx < total_tiles; idx += n_pairs) {
        if (aborting(&ctrl->abort) || !decode_tile<2 * Cfg::kTileFeat, false>(idx, ctrl, n_local, nft, cur, t)) break;
        const int n_mma = max(32, (t.n_valid + 31) & ~31);
        const uint32_t idesc = umma_idesc_pair(n_mma);
        mbar_wait(smem_u32(&ctrl->tmem_empty[0]), acc_phase ^ 1u, &ctrl->abort, a.status, 0x600);
        tc_fence_after();
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->full[stage]), phase, &ctrl->abort, a.status, 0x700 | stage);
          tc_fence_after();
          const uint32_t sa = ring + stage * stage_bytes;
          const uint64_t da0 = smem_desc_sw128(sa);
          const uint64_t da1 = smem_desc_sw128(sa + kATileBytes);
          const uint64_t db = smem_desc_sw128(sa + Cfg::kAStageBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            umma_bf16_pair(tmem_base, da0 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            umma_bf16_pair(tmem_base + kMaxTileTokens, da1 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          umma_commit_pair(smem_u32(&ctrl->empty[stage]), 3);
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit_pair(smem_u32(&ctrl->tmem_full[0]), 3);
        acc_phase ^= 1u;
      }
      if (aborting(&ctrl->abort)) {  // the MMAs issued so far must have retired before TMEM and the rings are given up
        st_cluster_u32(peer_abort, 1u);
        umma_commit_pair(smem_u32(&ctrl->mma_done), 1);
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(smem_u32(&ctrl->mma_done), 0)) break;
      }
    }
  } else {
    // ===================== epilogue (warps 2..9 of each CTA: its own features, all token columns) ============
    const int q = warp & 3;                                   // TMEM lane quadrant this warp may read
    const int half = (warp - kFirstEpilogueWarp) >> 2;        // which of the two warps of the quadrant
    const int et = threadIdx.x - kFirstEpilogueWarp * 32;     // 0..255
    int cur = 0;
    uint32_t acc_phase = 0;
    Tile t;
    const uint64_t pol_keep = l2_policy_evict_last();  // the outputs are read again by the next kernel
    const uint32_t leader_tmem_empty = map_to_cta(smem_u32(&ctrl->tmem_empty[0]), 0);
    for (int idx = pair_id; idx < total_tiles; idx += n_pairs) {
      if (!decode_tile<2 * Cfg::kTileFeat, false>(idx, ctrl, n_local, nft, cur, t)) break;
      if constexpr (GLU) {
        if (aborting(&ctrl->abort)) break;  // no named barrier in this loop: each thread may leave on its own
      } else {
        // all epilogue threads meet, learn whether any role gave up and leave together; the meeting also means that
        // every thread has left the previous tile before its staging slots (dst_s / w_s) are overwritten below
        if (epilogue_any(aborting(&ctrl->abort))) break;
      }
      const int f = t.f0 + f_shift + q * 32 + lane;
      const bool f_ok = f < a.n_feat;
      if constexpr (!GLU) {
        for (int n = et; n < t.n_valid; n += kEpilogueThreads) {
          const int pair = a.sorted[t.row0 + n];
          char *base = reinterpret_cast<char *>(a.y_pairs);
          if (a.n_owners > 1) base = reinterpret_cast<char *>(a.y_owner[min(a.n_owners - 1, (pair / a.top_k) / a.slice_tokens)]);
          ctrl->dst_s[0][n] = base + (size_t)pair * a.n_feat * (OUT16 ? 2 : 4);
          ctrl->w_s[0][n] = a.topk_w[pair];
        }
        epilogue_bar_sync();
      }
      const float bias0 = (f_ok && a.bias_a) ? a.bias_a[(size_t)t.e * a.n_feat + f] : 0.f;  // a null bias means none
      const bool f1_ok = !GLU && f + kTileF < a.n_feat;  // second tile of the down projection: feature f + 128
      const float bias1 = (GLU && f_ok)            ? a.bias_b[(size_t)t.e * a.n_feat + f]
                          : (f1_ok && a.bias_a) ? a.bias_a[(size_t)t.e * a.n_feat + f + kTileF]
                                                : 0.f;
      mbar_wait(smem_u32(&ctrl->tmem_full[0]), acc_phase, &ctrl->abort, a.status, 0x800);
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16);
      for (int c0 = half * 16; c0 < t.n_valid; c0 += 32) {
        uint32_t r0[16], r1[16];
        tmem_ld16(tbase + c0, r0);
        tmem_ld16(tbase + kMaxTileTokens + c0, r1);
        tmem_ld_wait();
        float v[16];
        if constexpr (GLU) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            v[j] = swiglu(__uint_as_float(r0[j]) + bias0, __uint_as_float(r1[j]) + bias1, a.limit);
          __nv_bfloat16 *dst = a.gate_up + (size_t)(t.row0 + c0) * a.n_feat + f;
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const __nv_bfloat162 pk = __floats2bfloat162_rn(v[j], v[j + 1]);
            if (f_ok && c0 + j < t.n_valid) st_b16_hint(dst + (size_t)j * a.n_feat, __bfloat16_as_ushort(pk.x), pol_keep);
            if (f_ok && c0 + j + 1 < t.n_valid) st_b16_hint(dst + (size_t)(j + 1) * a.n_feat, __bfloat16_as_ushort(pk.y), pol_keep);
          }
        } else if constexpr (OUT16) {
          char *pr[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pr[j] = ctrl->dst_s[0][c0 + j];
            v[j] = (__uint_as_float(r0[j]) + bias0) * ctrl->w_s[0][c0 + j];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (f_ok && c0 + j < t.n_valid)
              st_b16_hint(pr[j] + (size_t)f * 2, __bfloat16_as_ushort(__float2bfloat16_rn(v[j])), pol_keep);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (f1_ok && c0 + j < t.n_valid)
              st_b16_hint(pr[j] + (size_t)(f + kTileF) * 2,
                          __bfloat16_as_ushort(__float2bfloat16_rn((__uint_as_float(r1[j]) + bias1) * ctrl->w_s[0][c0 + j])), pol_keep);
        } else {
          float *pr[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pr[j] = reinterpret_cast<float *>(ctrl->dst_s[0][c0 + j]);
            v[j] = (__uint_as_float(r0[j]) + bias0) * ctrl->w_s[0][c0 + j];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (f_ok && c0 + j < t.n_valid) st_f32_hint(pr[j] + f, v[j], pol_keep);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (f1_ok && c0 + j < t.n_valid)
              st_f32_hint(pr[j] + f + kTileF, (__uint_as_float(r1[j]) + bias1) * ctrl->w_s[0][c0 + j], pol_keep);
        }
      }
      tc_fence_before();
      mbar_arrive_cluster(leader_tmem_empty);  // the leader's MMA thread waits for the epilogues of both CTAs
      acc_phase ^= 1u;
    }
    if (aborting(&ctrl->abort) && et == 0) st_cluster_u32(peer_abort, 1u);
  }

  tc_fence_before();
  cluster_sync_all();  // nobody frees TMEM or leaves while its peer may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if constexpr (!GLU) {
    // pushing to owners: as in the one-CTA kernel, the last CTA to finish raises this rank's "pushed" flag on every rank
    if (a.signal_step > 0 && threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int *>(a.signal_counter), 1u);
      if (prev == gridDim.x - 1) {
        *a.signal_counter = 0;
        __threadfence_system();
        for (int r = 0; r < a.n_owners; ++r) st_relaxed_sys(a.signal_flags[r], a.signal_step);
      }
    }
  }
}

template <bool GLU, bool OUT16>
cudaError_t launch_pair(const GemmArgs &a, int sm_count, cudaStream_t s) {
  const size_t smem = (size_t)kRingBytes + sizeof(Ctrl<2, GLU>);
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_pair_kernel<GLU, OUT16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_chain(grouped_gemm_pair_kernel<GLU, OUT16>, dim3(sm_count & ~1), dim3(kGemmThreads), smem, s, a);
}

}  // namespace

// Feature tiles per token block when a pair of CTAs shares an item: pairs of 128-feature tiles (gate/up GEMM), pairs of
// 256-feature double tiles (down GEMM).
cudaError_t launch_grouped_mlp1_pair(const GemmArgs &a, int sm_count, cudaStream_t s) {
  GemmArgs b = a;
  b.n_feat_tiles = (a.n_feat + 2 * kTileF - 1) / (2 * kTileF);
  return launch_pair<true, false>(b, sm_count, s);
}

cudaError_t launch_grouped_mlp2_pair(const GemmArgs &a, int sm_count, cudaStream_t s) {
  GemmArgs b = a;
  b.n_feat_tiles = (a.n_feat + 4 * kTileF - 1) / (4 * kTileF);
  return a.out_bf16 ? launch_pair<false, true>(b, sm_count, s) : launch_pair<false, false>(b, sm_count, s);
}

}  // namespace gptoss
