// Cross-GPU combine of the expert-parallel MoE block over NVLink peer memory (no NCCL, no TMA multicast).
//
// Every rank owns a contiguous slice of the tokens.  The down-GEMM epilogue of each rank stores its
// gate-weighted expert outputs, row by row as the tiles finish, straight into the OWNER's y_pairs buffer
// (plain peer stores, addressed by pair id = token*k + slot, so every row has exactly one writer).  When a
// rank has pushed everything it raises flag A on every peer.  The owner waits for flag A of all ranks, sums
// the k slots of each of its tokens in slot order (the same fixed order as the single-GPU combine, so the
// result is bit-identical for any number of GPUs), stores the sum into the `delta` buffer of EVERY rank
// (the all-gather, again by peer stores) and raises flag B everywhere.  Each rank finally waits for flag B
// of all owners and adds `delta` to its replicated residual stream.
//
// Token-sliced variant (each rank keeps only its own slice of the residual stream, e.g. behind data-parallel
// attention): a rank normalises its slice and stores the bf16 rows into the gathered activation buffer of EVERY
// rank (flag C), all ranks route the full batch and push to the owners as above, and the owner adds the slot-ordered
// sum to its own residual slice: no delivery step, half the NVLink traffic of the replicated form.
//
// A rank's "pushed" flag is raised by its down GEMM itself: the last CTA to finish stores it on every rank.
// Flags carry the step number (monotonic), so nothing is ever reset.  All waits are bounded by wall time;
// a wait that gives up records a time-out in the status words and the kernel carries on without waiting.
#include "kernels.cuh"

namespace gptoss {

namespace {

// The last block of the grid to get here raises flag `which` (0 = A, 1 = B, 2 = C) of this rank on every rank.  The
// block's stores are ordered before its count by the barrier plus ONE thread's system-scope fence (the fence is
// cumulative over what the barrier made visible to that thread); a fence by every thread would make each of them
// wait out the round trip of the block's peer stores.
__device__ __forceinline__ void signal_all_ranks(const PeerTable &pt, int which, int step, int *counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int *>(counter), 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      *counter = 0;
      __threadfence_system();
      for (int r = 0; r < pt.world; ++r) st_relaxed_sys(pt.flags[r] + which * kMaxRanks + pt.rank, step);
    }
  }
}

}  // namespace

__device__ __forceinline__ uint2 pack_bf16x4(const float4 &v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  return make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
}
__device__ __forceinline__ float4 unpack_bf16x4(const uint2 &u) {
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}

// Owner: delta[b,:] = ((s0+s1)+s2)+s3 for the tokens of this rank's slice, stored to every rank (fp32, or
// rounded to bf16 when the wire format is bf16 — the owner then reads back the rounded value like everyone
// else, so the replicated residual streams stay bit-identical).
template <bool BF16>
__global__ void __launch_bounds__(256) combine_owner_kernel(PeerTable pt, int T, int H, int k, int step,
                                                            int *status, int *counter) {
  pdl_wait();
  wait_all_ranks(pt.flags[pt.rank], pt.world, step, pt.timeout_ns, status, 0x2100);
  const int slice = slice_rows(T, pt.world);
  const int b0 = pt.rank * slice, b1 = min(T, b0 + slice);
  const int h8 = H >> 3;  // 8 elements per thread: two float4 loads per slot, one 16-byte (bf16) or two (fp32) stores per rank
  const size_t total = (size_t)max(0, b1 - b0) * h8;
  const float4 *y = reinterpret_cast<const float4 *>(pt.y[pt.rank]);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int b = b0 + (int)(i / h8), c = (int)(i % h8);
    const size_t row4 = (size_t)b * k * (2 * h8) + 2 * c;
    float4 a0 = y[row4], a1 = y[row4 + 1];
    for (int j = 1; j < k; ++j) {
      const float4 v0 = y[row4 + (size_t)j * 2 * h8], v1 = y[row4 + (size_t)j * 2 * h8 + 1];
      a0.x += v0.x; a0.y += v0.y; a0.z += v0.z; a0.w += v0.w;
      a1.x += v1.x; a1.y += v1.y; a1.z += v1.z; a1.w += v1.w;
    }
    const size_t o = (size_t)b * h8 + c;
    if (BF16) {
      const uint2 p0 = pack_bf16x4(a0), p1 = pack_bf16x4(a1);
      const uint4 pk = make_uint4(p0.x, p0.y, p1.x, p1.y);
      for (int r = 0; r < pt.world; ++r) reinterpret_cast<uint4 *>(pt.delta[r])[o] = pk;
    } else {
      for (int r = 0; r < pt.world; ++r) {
        reinterpret_cast<float4 *>(pt.delta[r])[2 * o] = a0;
        reinterpret_cast<float4 *>(pt.delta[r])[2 * o + 1] = a1;
      }
    }
  }
  pdl_launch_dependents();
  signal_all_ranks(pt, 1, step, counter);
}

// Every rank: x += delta once all owners have delivered their slices.
template <bool BF16>
__global__ void __launch_bounds__(256) add_delta_kernel(PeerTable pt, int T, int H, int step, float *x, int *status) {
  pdl_wait();
  wait_all_ranks(pt.flags[pt.rank] + kMaxRanks, pt.world, step, pt.timeout_ns, status, 0x2200);
  const size_t total = (size_t)T * (H >> 2);
  float4 *xp = reinterpret_cast<float4 *>(x);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float4 o = xp[i];
    const float4 v = BF16 ? unpack_bf16x4(reinterpret_cast<const uint2 *>(pt.delta[pt.rank])[i])
                          : reinterpret_cast<const float4 *>(pt.delta[pt.rank])[i];
    o.x += v.x;
    o.y += v.y;
    o.z += v.z;
    o.w += v.w;
    xp[i] = o;
  }
  pdl_launch_dependents();
}

// Token-sliced form, producer side.  Residual update + RMSNorm of the rows of this rank's slice (one block per row,
// the same row routine as the single-GPU kernel, hence the same bits), each bf16 row stored into the gathered
// activation buffer of every rank; the last block raises flag C.
__global__ void __launch_bounds__(256) slice_norm_gather_kernel(PeerTable pt, int T, int H, float *__restrict__ x_slice,
                                                                const float *__restrict__ add, const float *__restrict__ w,
                                                                int step, int *counter) {
  __shared__ double part[8];
  pdl_wait();
  const int slice = slice_rows(T, pt.world);
  const int b0 = pt.rank * slice, n_rows = max(0, min(T, b0 + slice) - b0);
  const int i_row = blockIdx.x;
  if (i_row < n_rows) {
    const size_t row = (size_t)(b0 + i_row) * H;
    residual_rmsnorm_row(
        x_slice + (size_t)i_row * H, add ? add + (size_t)i_row * H : nullptr, w, H, part,
        [&](int i, uint2 v) {
          for (int r = 0; r < pt.world; ++r) reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(pt.delta[r]) + row)[i] = v;
        },
        [&](int i, __nv_bfloat16 v) {
          for (int r = 0; r < pt.world; ++r) reinterpret_cast<__nv_bfloat16 *>(pt.delta[r])[row + i] = v;
        });
  }
  pdl_launch_dependents();
  signal_all_ranks(pt, 2, step, counter);
}

// Token-sliced form, producer side, for rows that are already normalised: copies this rank's bf16 rows into the
// gathered activation buffer of every rank (16 bytes per thread and peer); the last block raises flag C.
__global__ void __launch_bounds__(256) slice_copy_gather_kernel(PeerTable pt, int T, int H, const uint4 *__restrict__ t_slice,
                                                                int step, int *counter) {
  pdl_wait();
  const int slice = slice_rows(T, pt.world);
  const int b0 = pt.rank * slice, n_rows = max(0, min(T, b0 + slice) - b0);
  const size_t total = (size_t)n_rows * H / 8, first = (size_t)b0 * H / 8;  // H % 8 == 0
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = t_slice[i];
    for (int r = 0; r < pt.world; ++r) reinterpret_cast<uint4 *>(pt.delta[r])[first + i] = v;
  }
  pdl_launch_dependents();
  signal_all_ranks(pt, 2, step, counter);
}

// Returns once every rank has raised flag C to gather_step (its slice of the gathered activations has arrived) and
// flag D to route_step (the routing of its token slice has arrived); a step of 0 skips that flag.
//
// The successor is released only AFTER the waits: a kernel that became resident while this one still polled would
// sit in its own (poll-count bounded) mbarrier waits for as long as the slowest peer takes, and could give up there
// although the peer is well inside the wall-time limit of the flag wait.
__global__ void wait_flags_kernel(PeerTable pt, int gather_step, int route_step, int *status) {
  pdl_wait();
  if (gather_step > 0) wait_all_ranks(pt.flags[pt.rank] + 2 * kMaxRanks, pt.world, gather_step, pt.timeout_ns, status, 0x2300);
  if (route_step > 0) wait_all_ranks(pt.flags[pt.rank] + 3 * kMaxRanks, pt.world, route_step, pt.timeout_ns, status, 0x2600);
  pdl_launch_dependents();
}

// Device-side rendezvous of the ranks (no data): raises this rank's flag C everywhere, then waits for everyone's.
__global__ void rendezvous_kernel(PeerTable pt, int step, int *status) {
  pdl_wait();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < pt.world; ++r) st_relaxed_sys(pt.flags[r] + 2 * kMaxRanks + pt.rank, step);
  }
  __syncthreads();
  wait_all_ranks(pt.flags[pt.rank] + 2 * kMaxRanks, pt.world, step, pt.timeout_ns, status, 0x2500);
  pdl_launch_dependents();  // after the wait, like wait_flags_kernel
}

// Token-sliced form, owner side: x_slice[i,:] += ((s0+s1)+s2)+s3 for the rows of this rank's slice, slots in order.
// BF16: the pushed rows are bf16 (same indexing, half the bytes); the sum is fp32 either way.
template <bool BF16>
__global__ void __launch_bounds__(256) combine_owner_slice_kernel(PeerTable pt, int T, int H, int k, int step,
                                                                  float *__restrict__ x_slice, int *status) {
  pdl_wait();
  wait_all_ranks(pt.flags[pt.rank], pt.world, step, pt.timeout_ns, status, 0x2400);
  const int slice = slice_rows(T, pt.world);
  const int b0 = pt.rank * slice, b1 = min(T, b0 + slice);
  const int h4 = H >> 2;
  const size_t total = (size_t)max(0, b1 - b0) * h4;
  const float4 *y = reinterpret_cast<const float4 *>(pt.y[pt.rank]);
  const uint2 *yb = reinterpret_cast<const uint2 *>(pt.y[pt.rank]);
  float4 *xp = reinterpret_cast<float4 *>(x_slice);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int b = b0 + (int)(i / h4), c = (int)(i % h4);
    const size_t row4 = (size_t)b * k * h4 + c;
    float4 a = BF16 ? unpack_bf16x4(yb[row4]) : y[row4];
    for (int j = 1; j < k; ++j) {
      const float4 v = BF16 ? unpack_bf16x4(yb[row4 + (size_t)j * h4]) : y[row4 + (size_t)j * h4];
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    float4 o = xp[i];
    o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
    xp[i] = o;
  }
  pdl_launch_dependents();
}

cudaError_t launch_combine_owner(const PeerTable &pt, bool bf16_wire, int T, int H, int k, int step, int *status,
                                 int *counter, int sm_count, cudaStream_t s) {
  const int slice = slice_rows(T, pt.world);
  const size_t total = (size_t)slice * (H >> 3);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count * 4) blocks = sm_count * 4;  // few, long-lived blocks: each ends with a system-scope fence
  if (blocks < 1) blocks = 1;
  return launch_chain(bf16_wire ? combine_owner_kernel<true> : combine_owner_kernel<false>, dim3(blocks), dim3(256), 0, s, pt,
                      T, H, k, step, status, counter);
}

cudaError_t launch_add_delta(const PeerTable &pt, bool bf16_wire, int T, int H, int step, float *x, int *status,
                             int sm_count, cudaStream_t s) {
  const size_t total = (size_t)T * (H >> 2);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count * 16) blocks = sm_count * 16;
  if (blocks < 1) blocks = 1;
  return launch_chain(bf16_wire ? add_delta_kernel<true> : add_delta_kernel<false>, dim3(blocks), dim3(256), 0, s, pt, T, H,
                      step, x, status);
}

cudaError_t launch_slice_norm_gather(const PeerTable &pt, int T, int H, float *x_slice, const float *add, const float *w,
                                     int step, int *counter, cudaStream_t s) {
  const int slice = slice_rows(T, pt.world);
  int rows = T - pt.rank * slice;
  rows = rows < 0 ? 0 : (rows > slice ? slice : rows);
  return launch_chain(slice_norm_gather_kernel, dim3(rows > 0 ? rows : 1), dim3(256), 0, s, pt, T, H, x_slice, add, w, step,
                      counter);
}

cudaError_t launch_slice_copy_gather(const PeerTable &pt, int T, int H, const void *t_slice, int step, int *counter,
                                     int sm_count, cudaStream_t s) {
  const int slice = slice_rows(T, pt.world);
  const size_t total = (size_t)slice * H / 8;
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count * 4) blocks = sm_count * 4;
  if (blocks < 1) blocks = 1;
  return launch_chain(slice_copy_gather_kernel, dim3(blocks), dim3(256), 0, s, pt, T, H, static_cast<const uint4 *>(t_slice), step,
                      counter);
}

cudaError_t launch_wait_flags(const PeerTable &pt, int gather_step, int route_step, int *status, cudaStream_t s) {
  return launch_chain(wait_flags_kernel, dim3(1), dim3(32), 0, s, pt, gather_step, route_step, status);
}

cudaError_t launch_rendezvous(const PeerTable &pt, int step, int *status, cudaStream_t s) {
  return launch_chain(rendezvous_kernel, dim3(1), dim3(32), 0, s, pt, step, status);
}

cudaError_t launch_combine_owner_slice(const PeerTable &pt, bool bf16_rows, int T, int H, int k, int step, float *x_slice,
                                       int *status, int sm_count, cudaStream_t s) {
  const int slice = slice_rows(T, pt.world);
  const size_t total = (size_t)slice * (H >> 2);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count * 16) blocks = sm_count * 16;
  if (blocks < 1) blocks = 1;
  return launch_chain(bf16_rows ? combine_owner_slice_kernel<true> : combine_owner_slice_kernel<false>, dim3(blocks), dim3(256), 0, s,
                      pt, T, H, k, step, x_slice, status);
}

}  // namespace gptoss
