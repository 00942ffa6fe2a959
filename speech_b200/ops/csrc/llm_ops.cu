// Memory-bound kernels of the decoder-only LLM block: RMSNorm forward / backward, SwiGLU forward / backward, rotary position
// embedding (forward and, with the sine negated, backward).  bf16 activations, fp32 parameters and statistics; every tensor is
// read and written once with 16-byte accesses.
#include "common.cuh"

namespace {

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    float2 v = __bfloat1622float2(h[u]);
    f[2 * u] = v.x;
    f[2 * u + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  __align__(16) __nv_bfloat162 o[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) o[u] = __floats2bfloat162_rn(f[2 * u], f[2 * u + 1]);
  return *reinterpret_cast<uint4*>(o);
}

// ------------------------------------------------------------------------------------------------ RMSNorm
// One warp per row.  y = x * rstd * gamma, rstd = 1 / sqrt(mean(x^2) + eps); rstd is saved for backward.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, __nv_bfloat16* __restrict__ y,
                                   float* __restrict__ rstd_out, long long rows, int D, float eps) {
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += (long long)gridDim.x * wpb) {
    const __nv_bfloat16* xr = x + row * D;
    float ss = 0.f;
    for (int i = lane * 8; i < D; i += 256) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + i), f);
#pragma unroll
      for (int u = 0; u < 8; ++u) ss += f[u] * f[u];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    __nv_bfloat16* yr = y + row * D;
    for (int i = lane * 8; i < D; i += 256) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + i), f);
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + i), g1 = *reinterpret_cast<const float4*>(gamma + i + 4);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int u = 0; u < 8; ++u) f[u] = f[u] * rstd * g[u];
      *reinterpret_cast<uint4*>(yr + i) = pack8(f);
    }
  }
}

// dx = rstd * (g*dy - xhat * mean(g*dy*xhat)), xhat = x * rstd;  dgamma += sum_rows dy * xhat.
// A lane touches the same columns (lane*8 + k*256 ...) in every row, so for D <= NCH*256 its share of dgamma lives in NCH*8
// registers across all rows of the block and reaches shared memory once; NCH = 0 is the generic form with one shared-memory
// atomic per element.  Shared memory (fp32 [D]) is added to global memory once per block.
template <int NCH>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                                   long long rows, int D) {
  extern __shared__ float sdg[];
  for (int i = threadIdx.x; i < D; i += blockDim.x) sdg[i] = 0.f;
  __syncthreads();
  const int wpb = blockDim.x >> 5, lane = threadIdx.x & 31;
  constexpr int NA = NCH > 0 ? NCH : 1;
  float acc[NA][8];
#pragma unroll
  for (int k = 0; k < NA; ++k)
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[k][u] = 0.f;
  for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += (long long)gridDim.x * wpb) {
    const __nv_bfloat16 *xr = x + row * D, *dyr = dy + row * D;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = lane * 8; i < D; i += 256) {
      float fx[8], fd[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + i), fx);
      unpack8(*reinterpret_cast<const uint4*>(dyr + i), fd);
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + i), g1 = *reinterpret_cast<const float4*>(gamma + i + 4);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int u = 0; u < 8; ++u) dot += g[u] * fd[u] * fx[u] * rstd;
    }
    dot = warp_sum(dot) / D;
    __nv_bfloat16* dxr = dx + row * D;
    if (NCH > 0) {
#pragma unroll
      for (int k = 0; k < NA; ++k) {
        const int i = lane * 8 + k * 256;
        if (i < D) {
          float fx[8], fd[8], o[8];
          unpack8(*reinterpret_cast<const uint4*>(xr + i), fx);
          unpack8(*reinterpret_cast<const uint4*>(dyr + i), fd);
          const float4 g0 = *reinterpret_cast<const float4*>(gamma + i), g1 = *reinterpret_cast<const float4*>(gamma + i + 4);
          const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float xh = fx[u] * rstd;
            o[u] = rstd * (g[u] * fd[u] - xh * dot);
            acc[k][u] += fd[u] * xh;
          }
          *reinterpret_cast<uint4*>(dxr + i) = pack8(o);
        }
      }
    } else {
      for (int i = lane * 8; i < D; i += 256) {
        float fx[8], fd[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + i), fx);
        unpack8(*reinterpret_cast<const uint4*>(dyr + i), fd);
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + i), g1 = *reinterpret_cast<const float4*>(gamma + i + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float xh = fx[u] * rstd;
          o[u] = rstd * (g[u] * fd[u] - xh * dot);
          if (dgamma) atomicAdd(&sdg[i + u], fd[u] * xh);
        }
        *reinterpret_cast<uint4*>(dxr + i) = pack8(o);
      }
    }
  }
  if (NCH > 0 && dgamma) {
#pragma unroll
    for (int k = 0; k < NA; ++k) {
      const int i = lane * 8 + k * 256;
      if (i < D) {
#pragma unroll
        for (int u = 0; u < 8; ++u) atomicAdd(&sdg[i + u], acc[k][u]);
      }
    }
  }
  __syncthreads();
  if (dgamma)
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dgamma[i], sdg[i]);
}

// ------------------------------------------------------------------------------------------------ SwiGLU
// y = silu(g) * u;  dg = dy * u * silu'(g), du = dy * silu(g).  Flat over n elements (n % 8 == 0).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ y,
                                  long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float fg[8], fu[8];
    unpack8(reinterpret_cast<const uint4*>(g)[i], fg);
    unpack8(reinterpret_cast<const uint4*>(u)[i], fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) fg[k] = sb_swish(fg[k]) * fu[k];
    reinterpret_cast<uint4*>(y)[i] = pack8(fg);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                  __nv_bfloat16* __restrict__ dg, __nv_bfloat16* __restrict__ du, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float fd[8], fg[8], fu[8], og[8], ou[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], fd);
    unpack8(reinterpret_cast<const uint4*>(g)[i], fg);
    unpack8(reinterpret_cast<const uint4*>(u)[i], fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      og[k] = fd[k] * fu[k] * sb_dswish(fg[k]);
      ou[k] = fd[k] * sb_swish(fg[k]);
    }
    reinterpret_cast<uint4*>(dg)[i] = pack8(og);
    reinterpret_cast<uint4*>(du)[i] = pack8(ou);
  }
}

// ------------------------------------------------------------------------------------------------ rotary embedding
// x: [B, T, H, D] bf16 (D % 16 == 0), cos / sin: fp32 [B, T, D] with both halves equal (rotate-half convention):
// y[:d] = x[:d] cos - x[d:] sin, y[d:] = x[d:] cos + x[:d] sin, d = D / 2.  sign = -1 gives the transpose (backward).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            __nv_bfloat16* __restrict__ y, long long rows, int H, int D, float sign) {
  const int d = D / 2, per_row = d / 8;                       // 8-element groups of the first half; each also handles its partner
  const long long total = rows * per_row;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / per_row;                      // (b, t, h)
    const int c = (int)(idx % per_row) * 8;
    const long long bt = row / H;
    const __nv_bfloat16* xr = x + row * D;
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c), a);
    unpack8(*reinterpret_cast<const uint4*>(xr + d + c), b);
    const float* cr = cs + bt * D + c;
    const float* sr = sn + bt * D + c;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float co = cr[k], si = sign * sr[k];
      oa[k] = a[k] * co - b[k] * si;
      ob[k] = b[k] * co + a[k] * si;
    }
    __nv_bfloat16* yr = y + row * D;
    *reinterpret_cast<uint4*>(yr + c) = pack8(oa);
    *reinterpret_cast<uint4*>(yr + d + c) = pack8(ob);
  }
}

int grid_for(long long work_items, int per_block) {
  long long nb = (work_items + per_block - 1) / per_block;
  const long long cap = 148ll * 8;
  return (int)(nb < 1 ? 1 : (nb > cap ? cap : nb));
}

}  // namespace

SB_API int sb_rmsnorm_fwd(const void* x, const float* gamma, void* y, float* rstd, long long rows, int D, float eps, cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0) return SB_BAD_ARGUMENT;
  const int warps = 8;
  rmsnorm_fwd_kernel<<<grid_for(rows, warps), warps * 32, 0, stream>>>((const __nv_bfloat16*)x, gamma, (__nv_bfloat16*)y, rstd, rows, D, eps);
  return (int)cudaGetLastError();
}

SB_API int sb_rmsnorm_bwd(const void* dy, const void* x, const float* gamma, const float* rstd, void* dx, float* dgamma, long long rows, int D,
                          cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0 || D > 12288) return SB_BAD_ARGUMENT;
  const int warps = 8;
  long long nb = (rows + warps - 1) / warps;
  // few blocks for short rows (many rows per block amortise the per-block flush of dgamma), at most two waves
  const long long cap = 148ll * 2;
  const int grid = (int)(nb > cap ? cap : nb);
  const __nv_bfloat16 *pdy = (const __nv_bfloat16*)dy, *px = (const __nv_bfloat16*)x;
  __nv_bfloat16* pdx = (__nv_bfloat16*)dx;
  const size_t smem = D * sizeof(float);
  if (D <= 256) rmsnorm_bwd_kernel<1><<<grid, warps * 32, smem, stream>>>(pdy, px, gamma, rstd, pdx, dgamma, rows, D);
  else if (D <= 512) rmsnorm_bwd_kernel<2><<<grid, warps * 32, smem, stream>>>(pdy, px, gamma, rstd, pdx, dgamma, rows, D);
  else if (D <= 1024) rmsnorm_bwd_kernel<4><<<grid, warps * 32, smem, stream>>>(pdy, px, gamma, rstd, pdx, dgamma, rows, D);
  else if (D <= 2048) rmsnorm_bwd_kernel<8><<<grid, warps * 32, smem, stream>>>(pdy, px, gamma, rstd, pdx, dgamma, rows, D);
  else rmsnorm_bwd_kernel<0><<<grid, warps * 32, smem, stream>>>(pdy, px, gamma, rstd, pdx, dgamma, rows, D);
  return (int)cudaGetLastError();
}

SB_API int sb_swiglu_fwd(const void* g, const void* u, void* y, long long n, cudaStream_t stream) {
  if (n % 8 != 0 || n <= 0) return SB_BAD_ARGUMENT;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)y, n / 8);
  return (int)cudaGetLastError();
}

SB_API int sb_swiglu_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, long long n, cudaStream_t stream) {
  if (n % 8 != 0 || n <= 0) return SB_BAD_ARGUMENT;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u,
                                                               (__nv_bfloat16*)dg, (__nv_bfloat16*)du, n / 8);
  return (int)cudaGetLastError();
}

SB_API int sb_rope(const void* x, const float* cos_t, const float* sin_t, void* y, long long rows, int H, int D, int inverse, cudaStream_t stream) {
  if (D % 16 != 0 || rows <= 0 || H <= 0) return SB_BAD_ARGUMENT;
  rope_kernel<<<grid_for(rows * (D / 16), 256), 256, 0, stream>>>((const __nv_bfloat16*)x, cos_t, sin_t, (__nv_bfloat16*)y, rows, H, D,
                                                                   inverse ? -1.f : 1.f);
  return (int)cudaGetLastError();
}
