// Shared definitions of the gptoss_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gptoss_b200.h"

namespace gptoss {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;
constexpr int kTokensPerRouteBlock = 8;  // one warp per token, 8 warps per block
constexpr int kSmCountFallback = 148;

// GEMM tiling (shared by host launch code and kernels)
constexpr int kBlockK = 64;        // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kTileF = 128;        // output features per accumulator tile (UMMA M)
constexpr int kTokChunk = 32;      // token rows per TMA box of the activation operand
constexpr int kMaxTileTokens = 256;  // token rows per tile (UMMA N max)

// device status word layout (int[8] in global memory)
//   [0] sticky error code (0 = ok)   [1] where (kernel id << 16 | site)   [2..3] detail
constexpr int kStatusWords = 8;
constexpr int kDevErrTimeout = 3;

// Device scratch shared by the routing kernels and read by the GEMM kernels.
struct RouteBuffers {
  float *scores;        // [T,E]
  float *topk_w;        // [T,k]
  int *topk_i;          // [T,k]
  int *blk_hist;        // [n_route_blocks, E]
  int *blk_base;        // [n_route_blocks, E]   global start row of each block's pairs per expert
  int *offsets;         // [E+1]
  int *sorted;          // [T*k]
  int *tb_prefix;       // [E_local+1]   cumulative count of token blocks (at most kMaxTileTokens rows each) of the local
                        //               experts, as the gate/up GEMM cuts them; null = not wanted (grouping only)
  int *tb_prefix2;      // [E_local+1]   the same for the down GEMM (its own block size)
};

// How the prefix-sum kernel cuts the experts' rows into token blocks (see expert_scan_kernel).
struct TileBalance {
  int force_rows;  // > 0: blocks of at most this many rows instead of a size chosen per GEMM (measurement aid)
  int ctas;        // CTAs (or pairs of CTAs) that share out the items of a GEMM launch; 0: blocks of at most
                   // kMaxTileTokens rows, no balancing
  int nft1, nft2;  // work items per token block (feature tiles, or pairs of them) of the gate/up and of the down GEMM
  int fixed_rows;  // an item of b rows costs (fixed_rows + b): the weight tiles it stages, in units of staged token rows
};

// Where the gathered token rows go.  n == 1: into this rank's own x_packed, rows of its experts only.  n > 1 (dispatch
// of a token slice): the row of pair (token, slot) goes to the x_packed of the rank that owns the slot's expert, at its
// position in the global sorted order; the last block raises flags[r] = step on every rank when step > 0.
struct RowDispatch {
  int n;
  int experts_per_rank;
  int step;
  int *counter;
  __nv_bfloat16 *xp[16];
  int *sorted[16];  // n > 1: the pair id of a dispatched row goes with it, into the sorted order of the expert's owner
  int *flags[16];
};

// Tokens per owner slice of a batch of T tokens over `world` ranks: contiguous slices of equal size, a multiple of the
// routing block so that a block of the per-block expert histogram never straddles two ranks.
__host__ __device__ inline int slice_rows(int T, int world) {
  const int per = (T + world - 1) / world;
  return (per + kTokensPerRouteBlock - 1) / kTokensPerRouteBlock * kTokensPerRouteBlock;
}

// Where the routing result of a token goes: the routing buffers of every rank of the group (this rank's alone when
// the context has no peers).  Every rank routes its own token slice and stores the rows to all; the last block raises
// this rank's "routed" flag (flags[r], value step) on every rank when step > 0.
constexpr int kMaxShareRanks = 16;
struct RouteShare {
  int n;         // ranks to store to
  int step;      // 0 = no flag
  int *counter;  // blocks finished so far (left at 0)
  float *topk_w[kMaxShareRanks];
  int *topk_i[kMaxShareRanks];
  int *blk_hist[kMaxShareRanks];
  int *flags[kMaxShareRanks];
};

struct Dims {
  int H, I, E, k;
  int e_begin, e_end;  // local experts
  float limit;
};

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start
// while its predecessor in the stream is still running; pdl_wait() returns once the predecessor has
// completed and its writes are visible (a no-op for a normal launch), pdl_launch_dependents() lets the
// successor's blocks be scheduled as soon as resources free up.  Every kernel of the chain waits BEFORE it
// releases its successor, so completion of all earlier kernels is implied transitively.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Flags that another GPU (or this one) polls: acquire load, and a relaxed system-scope store that is meant to follow
// ONE __threadfence_system() covering every flag of a batch (fence once, then store the flags back to back: a
// release store per flag would pay the round trip to each peer in turn).
__device__ __forceinline__ int ld_acquire_sys(const int *p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(int *p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---- waits on flags that peers raise ---------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Threads 0..world-1 of the block each wait until flags[r] >= step; then the block synchronises.  The wait is bounded
// by wall time; a wait that gives up records a time-out (with `site`) in the status words and returns.
__device__ __forceinline__ void wait_all_ranks(const int *flags, int world, int step, unsigned long long limit_ns,
                                               int *status, int site) {
  if ((int)threadIdx.x < world) {
    const unsigned long long t0 = global_ns();
    while (ld_acquire_sys(flags + threadIdx.x) < step) {
      if (*reinterpret_cast<volatile int *>(status) != 0) break;  // some wait already gave up
      if (global_ns() - t0 > limit_ns) {
        if (atomicCAS(status, 0, kDevErrTimeout) == 0) {
          status[1] = site;
          status[2] = (int)threadIdx.x;
        }
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
}
// A wait on one kind of flag of every rank, to be done at the start of a kernel (step == 0: nothing to wait for).
struct FlagWait {
  const int *flags;  // this rank's copy of the flags of that kind, one per rank
  int world, step;
  unsigned long long timeout_ns;
  int *status;
  int site;
};

}  // namespace gptoss
