// Pieces shared by the grouped GEMM kernels (one CTA per item: grouped_gemm.cu; a pair of CTAs per item:
// grouped_gemm_pair.cu): tile geometry, the per-CTA control block, the item decoder and the epilogue helpers.
#pragma once

#include "kernels.cuh"
#include "tcgen05.cuh"

namespace gptoss {
namespace gemm {

constexpr int kATileBytes = kTileF * kBlockK * 2;           // 16 KiB: 128 features x 64 k
constexpr int kBChunkBytes = kTokChunk * kBlockK * 2;       //  4 KiB: 32 tokens x 64 k
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kGemmThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
constexpr int kTmemCols = 512;
constexpr int kMaxStages = 8;
constexpr int kRingBytes = 216 * 1024;

// NA = weight tiles per ring stage (both multiply the same token rows); GLU = the two tiles are the gate and up
// halves of the same 128 features (SwiGLU epilogue, bf16 out), otherwise they are two adjacent 128-feature tiles
// of the down projection (fp32 rows by pair id).  Two tiles per stage double the MMA work and the weight bytes
// in flight per byte of token rows staged.
template <int NA, bool GLU>
struct TileCfg {
  static constexpr int kAStageBytes = NA * kATileBytes;
  static constexpr int kAccBuffers = (NA == 2) ? 1 : 2;   // two tiles fill all 512 TMEM columns at 256 tokens
  static constexpr int kMetaTokens = GLU ? 1 : kMaxTileTokens;  // pair/weight staging only for the down projection
  static constexpr int kTileFeat = (NA == 2 && !GLU) ? 2 * kTileF : kTileF;  // output features per tile
  static constexpr int kSlabs = GLU ? 2 : 1;                // weight slabs per expert in the tensor map
};

template <int NA, bool GLU>
struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t mma_done;  // abort path only: completion of every MMA issued so far
  uint32_t tmem_base;
  int abort;
  int max_rows;
  int tbp[kMaxExperts + 1];
  int off[kMaxExperts + 1];
  char *dst_s[2][TileCfg<NA, GLU>::kMetaTokens];   // mlp2: destination row of each token column (local or peer)
  float w_s[2][TileCfg<NA, GLU>::kMetaTokens];     // mlp2: gate weight of each token column
};

struct Tile {
  int e;        // local expert
  int f0;       // first output feature
  int row0;     // first row (sorted order)
  int n_valid;  // rows in the tile
  int tb;       // index of the token block within the expert
};

// Items of an expert are ordered feature tile by feature tile with the token block fastest (concurrently running
// CTAs then share a weight tile in L2), or, with FT_FASTEST, token block by token block with the feature tile fastest
// (they share the token rows instead: right when the "token" side is the large streamed operand).
template <int TILE_FEAT, bool FT_FASTEST, class C>
__device__ __forceinline__ bool decode_tile(int idx, const C *c, int n_local, int nft, int &cur, Tile &t) {
  while (cur < n_local && idx >= c->tbp[cur + 1] * nft) ++cur;
  if (cur >= n_local) return false;
  const int r = idx - c->tbp[cur] * nft;
  const int nb = c->tbp[cur + 1] - c->tbp[cur];
  const int ft = FT_FASTEST ? r % nft : r / nb, tb = FT_FASTEST ? r / nft : r - ft * nb;
  // an expert with more than 256 rows is cut into nb blocks of (almost) equal size, a multiple of 16 rows
  const int rows = c->off[cur + 1] - c->off[cur];
  const int blk = (((rows + nb - 1) / nb) + 15) & ~15;
  t.e = cur;
  t.f0 = ft * TILE_FEAT;
  t.row0 = c->off[cur] + tb * blk;
  t.n_valid = min(blk, rows - tb * blk);
  t.tb = tb;
  return true;
}

// clamp + SwiGLU (alpha 1.702); exp and the reciprocal use the fast hardware approximations (relative
// error ~1e-6, far below the bf16 rounding of the result)
__device__ __forceinline__ float swiglu(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return __fdividef(g, 1.0f + __expf(-1.702f * g)) * (u + 1.0f);
}

// OUT16 (with !GLU): the output rows are bf16 instead of fp32 (same row and element indexing).
// AMAX (with !GLU): instead of storing the products, the epilogue keeps for every output feature (a TMEM lane) the
// largest value over the token columns of the tile and the row id it came from, i.e. one (max, argmax) partial per
// (token block, feature), and the items are ordered feature tile fastest.  With the operand roles swapped — the
// batch's activations as the "weights", a vocabulary-sized matrix as the "tokens" — this is the classifier with the
// greedy argmax fused: the logits never reach memory.
// OR of `pred` over the eight epilogue warps (named barrier 1): every epilogue thread gets the same answer
__device__ __forceinline__ bool epilogue_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, 256, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ bool aborting(const int *flag) { return *reinterpret_cast<const volatile int *>(flag) != 0; }

}  // namespace gemm
}  // namespace gptoss
