// Shared device helpers for the sm_100a kernels: status word, bounded waits, small math.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_API extern "C" __attribute__((visibility("default")))

// Status word written by kernels instead of trapping.  0 = ok; any other value names the first failure.
// Every in-kernel wait gives up after SB_WAIT_CYCLES clock cycles (about a second), records where, and lets
// the kernel run to its normal end (barriers passed, tensor memory freed) so the context stays usable.
enum SbStatus : int {
  SB_OK = 0,
  SB_TIMEOUT_SMEM_EMPTY = 1,
  SB_TIMEOUT_SMEM_FULL = 2,
  SB_TIMEOUT_TMEM_EMPTY = 3,
  SB_TIMEOUT_TMEM_FULL = 4,
  SB_TIMEOUT_PEER_FLAG = 5,
  SB_BAD_ARGUMENT = 6,
};

#ifndef SB_WAIT_CYCLES
#define SB_WAIT_CYCLES 2000000000ll
#endif

// The wait limit can be changed at run time (sb_set_wait_cycles in status.cu): ints 4-5 of the status array hold it as one
// 64-bit cycle count, 0 meaning the compile-time default.  Kernels read it only on the slow path of a wait.
__device__ __forceinline__ long long sb_wait_cycles(const int* status) {
  const long long v = *reinterpret_cast<const volatile long long*>(status + 4);
  return v > 0 ? v : SB_WAIT_CYCLES;
}

// The status word lives in status.cu; host code fetches its device address once per device with
// sb_status_ptr() and passes it to every kernel that can wait.
SB_API int* sb_status_ptr();
SB_API int sb_reserved_sms();   // SMs persistent kernels leave to concurrent kernels (status.cu)

__device__ __forceinline__ void sb_set_status(int* status, int code, int detail) {
  if (atomicCAS(&status[0], 0, code) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = detail;
  }
}
__device__ __forceinline__ bool sb_failed(const int* status) { return *((volatile const int*)status) != 0; }

// Stateless dropout mask.  One 32-bit hash serves FOUR consecutive elements: element `idx` of the tensor drawn with `seed` takes
// byte (idx & 3) of hash(seed, idx >> 2) and is kept iff that byte is >= thresh, an 8-bit threshold (p * 256, rounded; the
// effective drop probability is thresh / 256 and the keep scale 256 / (256 - thresh)).  Forward kernels and the backward kernels
// that rebuild the mask call these with the same (seed, row * N + col), so no mask tensor is ever stored; kernels that own four
// aligned elements call sb_dropout_hash4 once and test the bytes.
__device__ __forceinline__ unsigned int sb_dropout_hash4(unsigned long long seed, unsigned long long group) {
  unsigned int h = (unsigned int)group * 0x9E3779B1u ^ (unsigned int)(group >> 32) * 0x85EBCA77u ^ (unsigned int)seed;
  h ^= h >> 16; h *= 0x7FEB352Du; h ^= h >> 15; h *= 0x846CA68Bu; h ^= h >> 16;
  h ^= (unsigned int)(seed >> 32); h *= 0x9E3779B1u; h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12;
  return h;
}
__device__ __forceinline__ bool sb_dropout_keep_in(unsigned int h, int k, unsigned int thresh) {
  return ((h >> (8 * k)) & 255u) >= thresh;
}
__device__ __forceinline__ bool sb_dropout_keep(unsigned long long seed, unsigned long long idx, unsigned int thresh) {
  return sb_dropout_keep_in(sb_dropout_hash4(seed, idx >> 2), (int)(idx & 3ull), thresh);
}
static inline unsigned int sb_dropout_threshold(float p) {
  if (p <= 0.f) return 0u;
  const unsigned int t = (unsigned int)(p * 256.f + 0.5f);
  return t > 255u ? 255u : t;
}
static inline float sb_dropout_scale(float p) {
  const unsigned int t = sb_dropout_threshold(p);
  return t ? 256.f / (256.f - (float)t) : 1.f;
}

// rcp.approx instead of an IEEE division: the full-precision divide costs more than the rest of an epilogue put together
__device__ __forceinline__ float sb_sigmoid(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float sb_swish(float x) { return x * sb_sigmoid(x); }
__device__ __forceinline__ float sb_dswish(float z) {
  float s = sb_sigmoid(z);
  return s + z * s * (1.f - s);
}
__device__ __forceinline__ float sb_gelu(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118f)); }
__device__ __forceinline__ float sb_dgelu(float x) {
  float cdf = 0.5f * (1.f + erff(x * 0.70710678118f));
  float pdf = 0.39894228040f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32); `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : -3.0e38f;
  if (w == 0) r = warp_max(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ float log_add(float a, float b) {
  float m = fmaxf(a, b);
  if (m < -1.0e29f) return -1.0e30f;
  return m + log1pf(__expf(-fabsf(a - b)));
}

static inline int sb_num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
