// Weight format conversion (checkpoint fp32 layouts <-> device bf16 layouts) and the seeded synthetic
// generator.  All kernels are plain grid-stride element-wise passes, used at load time only.
#include "kernels.cuh"

namespace gptoss {

namespace {

constexpr double kIrwinHallStd = 53509.91992145008;  // sqrt(8 * (65536^2 - 1) / 12)
constexpr int kIrwinHallMean = 4 * 65535;

__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ uint16_t bf16_bits_rne(float f) {
  uint32_t u = __float_as_uint(f);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// element i of the stream: Irwin-Hall sum of eight 16-bit uniforms, centred, one fp32 multiply, bf16 RNE
__device__ __forceinline__ uint16_t synth_bits(uint64_t key, uint64_t i, float scale) {
  const uint64_t a = splitmix64(key + 2ull * i), b = splitmix64(key + 2ull * i + 1ull);
  int s = 0;
#pragma unroll
  for (int sh = 0; sh < 64; sh += 16) s += (int)((a >> sh) & 0xFFFFull) + (int)((b >> sh) & 0xFFFFull);
  return bf16_bits_rne(__fmul_rn((float)(s - kIrwinHallMean), scale));
}

inline uint64_t stream_key(uint64_t seed, uint64_t tensor_id) {
  return splitmix64(seed * 0x100000001B3ull + tensor_id);
}
inline float stream_scale(float sigma) { return (float)((double)sigma / kIrwinHallStd); }

inline int grid_for(size_t n) {
  size_t b = (n + 255) / 256;
  if (b > 148u * 16u) b = 148u * 16u;
  if (b < 1) b = 1;
  return (int)b;
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = bf16_bits_rne(src[i]);
}
__global__ void bf16_to_f32_kernel(const uint16_t *__restrict__ src, float *__restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __uint_as_float((uint32_t)src[i] << 16);
}
__global__ void round_bf16_f32_kernel(const float *__restrict__ src, float *__restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __uint_as_float((uint32_t)bf16_bits_rne(src[i]) << 16);
}
// src: one expert's mlp1 in checkpoint order [2I][K] (row 2c = gate c, row 2c+1 = up c), fp32
// dst: the same expert in device order [2][I][K] (all gate rows, then all up rows), bf16
__global__ void mlp1_deinterleave_kernel(const float *__restrict__ src, uint16_t *__restrict__ dst, int I, int K) {
  const size_t n = (size_t)2 * I * K;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / K, col = i % K;
    const size_t c = row >> 1, half = row & 1;
    dst[(half * I + c) * K + col] = bf16_bits_rne(src[i]);
  }
}
__global__ void mlp1_interleave_kernel(const uint16_t *__restrict__ src, float *__restrict__ dst, int I, int K) {
  const size_t n = (size_t)2 * I * K;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / K, col = i % K;
    const size_t c = row >> 1, half = row & 1;
    dst[i] = __uint_as_float((uint32_t)src[(half * I + c) * K + col] << 16);
  }
}
__global__ void synth_normal_kernel(uint16_t *__restrict__ dst, uint64_t n, uint64_t key, uint64_t start, float scale) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = synth_bits(key, start + i, scale);
}
__global__ void synth_normal_f32_kernel(float *__restrict__ dst, uint64_t n, uint64_t key, uint64_t start, float scale) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = __uint_as_float((uint32_t)synth_bits(key, start + i, scale) << 16);
}
__global__ void synth_mlp1_kernel(uint16_t *__restrict__ dst, int I, int K, uint64_t key, uint64_t start, float scale) {
  const uint64_t n = (uint64_t)2 * I * K;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t row = i / K, col = i % K;
    const uint64_t c = row >> 1, half = row & 1;
    dst[(half * I + c) * K + col] = synth_bits(key, start + i, scale);
  }
}

// interleaved bias [n_exp][2I] (gate 2c, up 2c+1) <-> split [n_exp][I] + [n_exp][I]; values rounded to bf16
__global__ void bias_split_kernel(const float *__restrict__ src, float *__restrict__ g, float *__restrict__ u,
                                  size_t n_pairs) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += (size_t)gridDim.x * blockDim.x) {
    g[i] = __uint_as_float((uint32_t)bf16_bits_rne(src[2 * i]) << 16);
    u[i] = __uint_as_float((uint32_t)bf16_bits_rne(src[2 * i + 1]) << 16);
  }
}
__global__ void bias_merge_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ dst,
                                  size_t n_pairs) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += (size_t)gridDim.x * blockDim.x) {
    dst[2 * i] = g[i];
    dst[2 * i + 1] = u[i];
  }
}

}  // namespace

cudaError_t launch_bias_split(const float *src, float *g, float *u, size_t n_pairs, cudaStream_t s) {
  bias_split_kernel<<<grid_for(n_pairs), 256, 0, s>>>(src, g, u, n_pairs);
  return cudaGetLastError();
}
cudaError_t launch_bias_merge(const float *g, const float *u, float *dst, size_t n_pairs, cudaStream_t s) {
  bias_merge_kernel<<<grid_for(n_pairs), 256, 0, s>>>(g, u, dst, n_pairs);
  return cudaGetLastError();
}

cudaError_t launch_f32_to_bf16(const float *src, __nv_bfloat16 *dst, size_t n, cudaStream_t s) {
  f32_to_bf16_kernel<<<grid_for(n), 256, 0, s>>>(src, reinterpret_cast<uint16_t *>(dst), n);
  return cudaGetLastError();
}
cudaError_t launch_bf16_to_f32(const __nv_bfloat16 *src, float *dst, size_t n, cudaStream_t s) {
  bf16_to_f32_kernel<<<grid_for(n), 256, 0, s>>>(reinterpret_cast<const uint16_t *>(src), dst, n);
  return cudaGetLastError();
}
cudaError_t launch_round_bf16_f32(const float *src, float *dst, size_t n, cudaStream_t s) {
  round_bf16_f32_kernel<<<grid_for(n), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}
cudaError_t launch_mlp1_deinterleave(const float *src, __nv_bfloat16 *dst, int I, int K, cudaStream_t s) {
  mlp1_deinterleave_kernel<<<grid_for((size_t)2 * I * K), 256, 0, s>>>(src, reinterpret_cast<uint16_t *>(dst), I, K);
  return cudaGetLastError();
}
cudaError_t launch_mlp1_interleave(const __nv_bfloat16 *src, float *dst, int I, int K, cudaStream_t s) {
  mlp1_interleave_kernel<<<grid_for((size_t)2 * I * K), 256, 0, s>>>(reinterpret_cast<const uint16_t *>(src), dst, I, K);
  return cudaGetLastError();
}
cudaError_t launch_synth_normal(__nv_bfloat16 *dst, uint64_t n, uint64_t seed, uint64_t tensor_id, uint64_t start,
                                float sigma, cudaStream_t s) {
  synth_normal_kernel<<<grid_for(n), 256, 0, s>>>(reinterpret_cast<uint16_t *>(dst), n, stream_key(seed, tensor_id),
                                                   start, stream_scale(sigma));
  return cudaGetLastError();
}
cudaError_t launch_synth_normal_f32(float *dst, uint64_t n, uint64_t seed, uint64_t tensor_id, uint64_t start,
                                    float sigma, cudaStream_t s) {
  synth_normal_f32_kernel<<<grid_for(n), 256, 0, s>>>(dst, n, stream_key(seed, tensor_id), start, stream_scale(sigma));
  return cudaGetLastError();
}
cudaError_t launch_synth_mlp1(__nv_bfloat16 *dst, int I, int K, uint64_t seed, uint64_t tensor_id, uint64_t start,
                              float sigma, cudaStream_t s) {
  synth_mlp1_kernel<<<grid_for((size_t)2 * I * K), 256, 0, s>>>(reinterpret_cast<uint16_t *>(dst), I, K,
                                                                 stream_key(seed, tensor_id), start, stream_scale(sigma));
  return cudaGetLastError();
}

}  // namespace gptoss
