// Allocation-free gradient norm + clip coefficient; the contract is in grad_norm_static.h.
#include "grad_norm_static.h"
#include <mutex>
#include <stdio.h>

// The scratch itself: block partial sums.  Lives in the module's device data segment, one instance per device.
static __device__ __align__(256) float g_static_partials[SB_GRAD_NORM_STATIC_MAX_PARTS];

namespace {

constexpr int kMaxDevices = 64;

// Host-side cache of the device address of g_static_partials for each device ordinal.
float* g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

__global__ void sumsq_static_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  const bool vec_ok = (reinterpret_cast<unsigned long long>(g) & 15ull) == 0;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (vec_ok && i + 4 <= n) {
      const float4 a = *reinterpret_cast<const float4*>(g + i);
      s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    } else {
      const long long e = i + 4 < n ? i + 4 : n;
      for (long long j = i; j < e; ++j) s += g[j] * g[j];
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void clip_coef_static_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ scalars,
                                        float max_norm, float grad_scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float norm = sqrtf(s) * grad_scale;
    scalars[0] = norm;
    const float c = max_norm / (norm + 1e-6f);
    scalars[1] = grad_scale * (c < 1.f ? c : 1.f);
    if (!isfinite(norm)) scalars[2] = 1.f;
  }
}

// Device address of the scratch array on the current device; resolved once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return SB_GRAD_NORM_STATIC_E_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_partials_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_partials);
    if (e != cudaSuccess) {
      fprintf(stderr, "sb_grad_norm_clip_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return (int)e;
    }
    g_partials_addr[dev] = ptr;
  }
  *out = g_partials_addr[dev];
  return 0;
}

}  // namespace

SB_API int sb_grad_norm_static_max_parts() { return SB_GRAD_NORM_STATIC_MAX_PARTS; }

SB_API int sb_grad_norm_clip_static(const float* g, long long n, float* scalars, float max_norm, float grad_scale, int nparts,
                                    cudaStream_t stream) {
  if (g == nullptr || scalars == nullptr || n < 0 || nparts < 0) return SB_GRAD_NORM_STATIC_E_BAD_ARG;
  if (nparts == 0) {   // default: eight blocks per SM, clamped to what the static array holds
    nparts = sb_num_sms() * 8;
    if (nparts > SB_GRAD_NORM_STATIC_MAX_PARTS) nparts = SB_GRAD_NORM_STATIC_MAX_PARTS;
  }
  if (nparts > SB_GRAD_NORM_STATIC_MAX_PARTS) {
    fprintf(stderr,
            "sb_grad_norm_clip_static: %d partial sums requested but the static scratch holds %d; "
            "pass a smaller nparts or use sb_grad_norm_clip with a caller-provided buffer\n",
            nparts, SB_GRAD_NORM_STATIC_MAX_PARTS);
    return SB_GRAD_NORM_STATIC_E_TOO_LARGE;
  }
  float* partials = nullptr;
  const int rc = scratch_for_current_device(&partials);
  if (rc != 0) return rc;
  sumsq_static_kernel<<<nparts, 256, 0, stream>>>(g, n, partials);
  clip_coef_static_kernel<<<1, 256, 0, stream>>>(partials, nparts, scalars, max_norm, grad_scale);
  return (int)cudaGetLastError();
}
