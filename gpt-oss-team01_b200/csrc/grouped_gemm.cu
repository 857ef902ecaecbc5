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
// One persistent CTA per SM, 10 warps: warp 0 = TMA producer, warp 1 = MMA issuer (one elected thread) and
// TMEM owner, warps 2-9 = epilogue (two warps per TMEM lane quadrant, alternating 16-column chunks).
// Tiles are (expert, token block of <= 256 rows, feature tile), enumerated from the device-built
// token-block prefix, so no row count ever travels to the host.  A ring stage carries two weight tiles that
// multiply the same token rows: the gate and up rows of 128 features (mlp1), or two adjacent 128-feature tiles
// (mlp2 and the dense GEMMs; a one-tile variant remains for outputs of at most 128 features).
//
// The block is bound by streaming weights, so what matters is the number of weight bytes in flight per SM:
// a ring stage holds the weight tile(s) of one k-block plus the activation rows of the largest token block
// of this launch (read from the expert offsets, rounded to 32 rows), and the ring takes as many stages as
// fit into shared memory (decode: 4 x 52 KiB).
//
// Every mbarrier wait is bounded: when a wait gives up the CTA raises an abort flag and records a time-out in the
// status words.  Every later wait of the CTA returns at once, and every role looks at the flag at the top of each tile
// and leaves its loop there (the epilogue warps of the row GEMM agree on it through a barrier reduction, so that their
// named-barrier counts stay equal).  Then the producer waits (bounded) for the copies it has armed, the MMA thread for
// the MMAs it has issued, and the CTA frees its TMEM and returns.  The flag is deliberately NOT tested per ring stage:
// making the single-thread producer / MMA loops branch on the result of each wait was measured 8-15 % slower (both
// GEMMs, T = 1024 and T = 8192), so a role may still issue the rest of ONE tile's copies or MMAs after a time-out; they
// touch only this CTA's ring and accumulator, and the drain below waits for them.
#include <cstdlib>

#include "gemm_tile.cuh"

namespace gptoss {

using namespace gemm;

namespace {

template <int NA, bool GLU, bool AMAX = false, bool OUT16 = false>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmArgs a) {
  static_assert(!AMAX || (NA == 2 && !GLU), "the argmax epilogue exists for the two-tile row GEMM only");
  static_assert(!OUT16 || (!GLU && !AMAX), "bf16 rows are an option of the row GEMM only");
  using Cfg = TileCfg<NA, GLU>;
  using CtrlT = Ctrl<NA, GLU>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t ring = smem_u32(smem_raw);
  CtrlT *ctrl = reinterpret_cast<CtrlT *>(smem_raw + kRingBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_local = a.n_local, nft = a.n_feat_tiles;

  if (threadIdx.x == 0) {
    ctrl->max_rows = 0;
    if (ring & 1023u) {  // the ring must be 1024-byte aligned for the 128-byte swizzle
      ctrl->abort = 1;
      if (atomicCAS(a.status, 0, kDevErrTimeout) == 0) a.status[1] = 0x900;
    } else {
      ctrl->abort = 0;
    }
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[b]), kEpilogueThreads);
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
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->abort ? 0 : ctrl->tbp[n_local] * nft;
  // ring geometry of this launch
  const int b_rows = max(kTokChunk, (ctrl->max_rows + kTokChunk - 1) / kTokChunk * kTokChunk);
  const int stage_bytes = Cfg::kAStageBytes + b_rows * kBlockK * 2;
  const int n_stages = min(kMaxStages, kRingBytes / stage_bytes);

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int stage = 0, cur = 0;
      uint32_t phase = 0, armed = 0, last_par = 0;
      Tile t;
      // each weight byte is used once per launch; with the roles swapped (AMAX) the "weights" are the small operand
      // that every item reads again
      const uint64_t pol_w = AMAX ? l2_policy_evict_last() : l2_policy_evict_first();
      // Head start: the weights do not depend on the kernel before this one, so the weight tiles of the first
      // ring fill are requested before waiting for it; its outputs (the activation rows) are loaded after.
      int pre = 0;
      if ((int)blockIdx.x < total_tiles && decode_tile<Cfg::kTileFeat, AMAX>(blockIdx.x, ctrl, n_local, nft, cur, t)) {
        const int n_chunks = (max(16, (t.n_valid + 15) & ~15) + kTokChunk - 1) / kTokChunk;
        pre = min(n_stages, a.k_blocks);
        for (int kb = 0; kb < pre; ++kb) {
          const uint32_t bar = smem_u32(&ctrl->full[kb]);
          const uint32_t sa = ring + kb * stage_bytes;
          armed |= 1u << kb;
          mbar_expect_tx(bar, Cfg::kAStageBytes + n_chunks * kBChunkBytes);
          tma_load_3d_hint(sa, &a.map_w, bar, kb * kBlockK, t.f0, t.e * Cfg::kSlabs, pol_w);
          if (NA == 2)  // GLU: the up rows of the same features (next slab); else the next 128 features (zero-filled past the end)
            tma_load_3d_hint(sa + kATileBytes, &a.map_w, bar, kb * kBlockK, GLU ? t.f0 : t.f0 + kTileF,
                             GLU ? t.e * Cfg::kSlabs + 1 : t.e * Cfg::kSlabs, pol_w);
        }
        pdl_wait();
        pdl_launch_dependents();
        for (int kb = 0; kb < pre; ++kb)
          for (int c = 0; c < n_chunks; ++c)
            tma_load_2d(ring + kb * stage_bytes + Cfg::kAStageBytes + c * kBChunkBytes, &a.map_act,
                        smem_u32(&ctrl->full[kb]), kb * kBlockK, t.row0 + c * kTokChunk);
        stage = pre % n_stages;
        phase = (pre == n_stages) ? 1u : 0u;
        cur = 0;
      } else {
        pdl_wait();
        pdl_launch_dependents();
      }
      for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
        if (aborting(&ctrl->abort) || !decode_tile<Cfg::kTileFeat, AMAX>(idx, ctrl, n_local, nft, cur, t)) break;
        const int n_mma = max(16, (t.n_valid + 15) & ~15);
        const int n_chunks = (n_mma + kTokChunk - 1) / kTokChunk;
        const uint32_t tx = Cfg::kAStageBytes + n_chunks * kBChunkBytes;
        for (int kb = (idx == (int)blockIdx.x) ? pre : 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1u, &ctrl->abort, a.status, 0x100 | stage);
          const uint32_t bar = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = ring + stage * stage_bytes;
          armed |= 1u << stage;
          last_par = (last_par & ~(1u << stage)) | (phase << stage);
          mbar_expect_tx(bar, tx);
          tma_load_3d_hint(sa, &a.map_w, bar, kb * kBlockK, t.f0, t.e * Cfg::kSlabs, pol_w);
          if (NA == 2)  // GLU: the up rows of the same features (next slab); else the next 128 features (zero-filled past the end)
            tma_load_3d_hint(sa + kATileBytes, &a.map_w, bar, kb * kBlockK, GLU ? t.f0 : t.f0 + kTileF,
                             GLU ? t.e * Cfg::kSlabs + 1 : t.e * Cfg::kSlabs, pol_w);
          const uint32_t sb = sa + Cfg::kAStageBytes;
          for (int c = 0; c < n_chunks; ++c)
            tma_load_2d(sb + c * kBChunkBytes, &a.map_act, bar, kb * kBlockK, t.row0 + c * kTokChunk);
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // drain: every armed stage must have landed before the CTA may exit (bounded)
      for (int s = 0; s < n_stages; ++s)
        if (armed & (1u << s)) {
          const uint32_t par = (last_par >> s) & 1u;
          for (uint32_t i = 0; i < kSpinLimit; ++i)
            if (mbar_try_wait(smem_u32(&ctrl->full[s]), par)) break;
        }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int stage = 0, cur = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      Tile t;
      for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
        if (aborting(&ctrl->abort) || !decode_tile<Cfg::kTileFeat, AMAX>(idx, ctrl, n_local, nft, cur, t)) break;
        const int n_mma = max(16, (t.n_valid + 15) & ~15);
        const uint32_t idesc = umma_idesc(n_mma);
        mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1u, &ctrl->abort, a.status, 0x200 | acc);
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(acc * kMaxTileTokens);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          mbar_wait(smem_u32(&ctrl->full[stage]), phase, &ctrl->abort, a.status, 0x300 | stage);
          tc_fence_after();
          const uint32_t sa = ring + stage * stage_bytes;
          const uint64_t da0 = smem_desc_sw128(sa);
          const uint64_t da1 = smem_desc_sw128(sa + kATileBytes);
          const uint64_t db = smem_desc_sw128(sa + Cfg::kAStageBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            umma_bf16(d0, da0 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
            if (NA == 2) umma_bf16(d0 + kMaxTileTokens, da1 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accum);
          }
          umma_commit(smem_u32(&ctrl->empty[stage]));
          if (++stage == n_stages) {
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
      if (aborting(&ctrl->abort)) {  // the MMAs issued so far must have retired before TMEM and the ring are given up
        umma_commit(smem_u32(&ctrl->mma_done));
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(smem_u32(&ctrl->mma_done), 0)) break;
      }
    }
  } else {
    // ===================== epilogue (warps 2..9) =====================
    const int q = warp & 3;                                   // TMEM lane quadrant this warp may read
    const int half = (warp - kFirstEpilogueWarp) >> 2;        // which of the two warps of the quadrant
    const int et = threadIdx.x - kFirstEpilogueWarp * 32;     // 0..255
    int cur = 0, acc = 0;
    uint32_t acc_phase = 0;
    Tile t;
    const uint64_t pol_keep = l2_policy_evict_last();  // the outputs are read again by the next kernel
    for (int idx = blockIdx.x; idx < total_tiles; idx += gridDim.x) {
      if (!decode_tile<Cfg::kTileFeat, AMAX>(idx, ctrl, n_local, nft, cur, t)) break;
      if constexpr (GLU) {
        if (aborting(&ctrl->abort)) break;  // no named barrier in this loop: each thread may leave on its own
      } else {
        // all epilogue threads meet, learn whether any role gave up and leave together; the meeting also means that
        // every thread has left the previous tile before its staging slots (dst_s / w_s) are overwritten below
        if (epilogue_any(aborting(&ctrl->abort))) break;
      }
      const int f = t.f0 + q * 32 + lane;
      const bool f_ok = f < a.n_feat;
      if constexpr (AMAX) {
        // running first maximum of this thread's columns for its two features (f: first tile, f + 128: second tile)
        float best0 = -3.402823466e+38f, best1 = -3.402823466e+38f;
        int at0 = 0x7fffffff, at1 = 0x7fffffff;
        mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, &ctrl->abort, a.status, 0x400 | acc);
        tc_fence_after();
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kMaxTileTokens);
        for (int c0 = half * 16; c0 < t.n_valid; c0 += 32) {
          uint32_t r0[16], r1[16];
          tmem_ld16(tbase + c0, r0);
          tmem_ld16(tbase + kMaxTileTokens + c0, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int id = t.row0 + c0 + j;
            float v0 = __uint_as_float(r0[j]), v1 = __uint_as_float(r1[j]);
            // a scan that starts from element 0 never leaves it when it is NaN (every '>' fails): rank it above all
            if (id == 0 && v0 != v0) v0 = __int_as_float(0x7f800000);
            if (id == 0 && v1 != v1) v1 = __int_as_float(0x7f800000);
            const bool in = c0 + j < t.n_valid;
            if (in && v0 > best0) best0 = v0, at0 = id;  // ascending ids, strict '>': the first maximum stays
            if (in && v1 > best1) best1 = v1, at1 = id;
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&ctrl->tmem_empty[acc]));
        if (++acc == Cfg::kAccBuffers) {
          acc = 0;
          acc_phase ^= 1u;
        }
        // the two warps of a quadrant saw alternate 16-column chunks: merge through shared memory (first maximum)
        int *at_s = reinterpret_cast<int *>(ctrl->w_s[1]);
        const int lane_f = q * 32 + lane;
        if (half == 1) {
          ctrl->w_s[0][lane_f] = best0, ctrl->w_s[0][kTileF + lane_f] = best1;
          at_s[lane_f] = at0, at_s[kTileF + lane_f] = at1;
        }
        epilogue_bar_sync();
        if (half == 0) {
          const float o0 = ctrl->w_s[0][lane_f], o1 = ctrl->w_s[0][kTileF + lane_f];
          const int p0 = at_s[lane_f], p1 = at_s[kTileF + lane_f];
          if (o0 > best0 || (o0 == best0 && p0 < at0)) best0 = o0, at0 = p0;
          if (o1 > best1 || (o1 == best1 && p1 < at1)) best1 = o1, at1 = p1;
          const size_t o = (size_t)t.tb * a.n_feat;
          if (f_ok) a.amax_val[o + f] = best0, a.amax_at[o + f] = at0;
          if (f + kTileF < a.n_feat) a.amax_val[o + f + kTileF] = best1, a.amax_at[o + f + kTileF] = at1;
        }
        continue;
      }
      if constexpr (!GLU) {
        for (int n = et; n < t.n_valid; n += kEpilogueThreads) {
          const int pair = a.sorted[t.row0 + n];
          char *base = reinterpret_cast<char *>(a.y_pairs);
          if (a.n_owners > 1) base = reinterpret_cast<char *>(a.y_owner[min(a.n_owners - 1, (pair / a.top_k) / a.slice_tokens)]);
          ctrl->dst_s[acc][n] = base + (size_t)pair * a.n_feat * (OUT16 ? 2 : 4);
          ctrl->w_s[acc][n] = a.topk_w[pair];
        }
        epilogue_bar_sync();
      }
      const float bias0 = (f_ok && a.bias_a) ? a.bias_a[(size_t)t.e * a.n_feat + f] : 0.f;  // a null bias means none
      const bool f1_ok = NA == 2 && !GLU && f + kTileF < a.n_feat;  // second tile of the down projection: feature f + 128
      const float bias1 = (GLU && f_ok)            ? a.bias_b[(size_t)t.e * a.n_feat + f]
                          : (f1_ok && a.bias_a) ? a.bias_a[(size_t)t.e * a.n_feat + f + kTileF]
                                                : 0.f;
      mbar_wait(smem_u32(&ctrl->tmem_full[acc]), acc_phase, &ctrl->abort, a.status, 0x400 | acc);
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kMaxTileTokens);
      // 16 token columns at a time, alternating between the two warps of the quadrant; the 16 values of a
      // chunk are independent chains, computed branch-free so that they overlap
      for (int c0 = half * 16; c0 < t.n_valid; c0 += 32) {
        uint32_t r0[16], r1[16];
        tmem_ld16(tbase + c0, r0);
        if (NA == 2) tmem_ld16(tbase + kMaxTileTokens + c0, r1);
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
        } else {
          if constexpr (OUT16) {
            char *pr[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              pr[j] = ctrl->dst_s[acc][c0 + j];
              v[j] = (__uint_as_float(r0[j]) + bias0) * ctrl->w_s[acc][c0 + j];
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f_ok && c0 + j < t.n_valid)
                st_b16_hint(pr[j] + (size_t)f * 2, __bfloat16_as_ushort(__float2bfloat16_rn(v[j])), pol_keep);
            if constexpr (NA == 2) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (f1_ok && c0 + j < t.n_valid)
                  st_b16_hint(pr[j] + (size_t)(f + kTileF) * 2,
                              __bfloat16_as_ushort(__float2bfloat16_rn((__uint_as_float(r1[j]) + bias1) * ctrl->w_s[acc][c0 + j])), pol_keep);
            }
          } else {
            float *pr[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              pr[j] = reinterpret_cast<float *>(ctrl->dst_s[acc][c0 + j]);
              v[j] = (__uint_as_float(r0[j]) + bias0) * ctrl->w_s[acc][c0 + j];
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f_ok && c0 + j < t.n_valid) st_f32_hint(pr[j] + f, v[j], pol_keep);
            if constexpr (NA == 2) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (f1_ok && c0 + j < t.n_valid)
                  st_f32_hint(pr[j] + f + kTileF, (__uint_as_float(r1[j]) + bias1) * ctrl->w_s[acc][c0 + j], pol_keep);
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
  if constexpr (!GLU) {
    // pushing to owners: every row this CTA stored (possibly into a peer's memory) is ordered before the count by
    // the barrier above plus this thread's system-scope fence; the last CTA to finish raises this rank's "pushed"
    // flag on every rank
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

template <int NA, bool GLU, bool AMAX = false, bool OUT16 = false>
cudaError_t launch_grouped(const GemmArgs &a, int sm_count, cudaStream_t s) {
  const size_t smem = (size_t)kRingBytes + sizeof(Ctrl<NA, GLU>);
  static_assert(kRingBytes + sizeof(Ctrl<NA, GLU>) <= 232448, "exceeds the 227 KiB dynamic shared memory of an SM");
  static_assert(kRingBytes >= 2 * (2 * kATileBytes + kMaxTileTokens * kBlockK * 2), "ring must hold two full stages");
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<NA, GLU, AMAX, OUT16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_chain(grouped_gemm_kernel<NA, GLU, AMAX, OUT16>, dim3(sm_count), dim3(kGemmThreads), smem, s, a);
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
  return launch_grouped<2, true>(a, sm_count, s);
}
// Down projection / dense GEMM: two adjacent 128-feature tiles per ring stage (one pass over the token rows feeds
// 256 output features) unless there are at most 128 features, or GPTOSS_MLP2_SINGLE=1 asks for the one-tile kernel
// (A/B measurements).  The feature-tile count of the arguments is recomputed for the tile width used.
cudaError_t launch_grouped_mlp2(const GemmArgs &a, int sm_count, cudaStream_t s) {
  static const bool single = [] {
    const char *e = getenv("GPTOSS_MLP2_SINGLE");
    return e && e[0] == '1';
  }();
  GemmArgs b = a;
  if (single || a.n_feat <= kTileF) {
    b.n_feat_tiles = (a.n_feat + kTileF - 1) / kTileF;
    return a.out_bf16 ? launch_grouped<1, false, false, true>(b, sm_count, s) : launch_grouped<1, false>(b, sm_count, s);
  }
  b.n_feat_tiles = (a.n_feat + 2 * kTileF - 1) / (2 * kTileF);
  return a.out_bf16 ? launch_grouped<2, false, false, true>(b, sm_count, s) : launch_grouped<2, false>(b, sm_count, s);
}

// Row GEMM with the (max, argmax)-over-rows epilogue: amax_val / amax_at [token blocks][n_feat]
cudaError_t launch_grouped_amax(const GemmArgs &a, int sm_count, cudaStream_t s) {
  if (!a.amax_val || !a.amax_at || a.n_local != 1) return cudaErrorInvalidValue;
  GemmArgs b = a;
  b.n_feat_tiles = (a.n_feat + 2 * kTileF - 1) / (2 * kTileF);
  return launch_grouped<2, false, true>(b, sm_count, s);
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

cudaError_t encode_map_2d(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn;
  cudaError_t e = get_encode_fn(&fn);
  if (e != cudaSuccess) return e;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t encode_act_map(CUtensorMap *m, const void *base, uint64_t K, uint64_t rows) {
  return encode_map_2d(m, base, K, rows, (uint32_t)kTokChunk);
}

}  // namespace gptoss
