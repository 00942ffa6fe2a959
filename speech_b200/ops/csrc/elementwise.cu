// Memory-bound kernels: LayerNorm forward/backward, fused AdamW over flat buffers, gradient-norm reduction,
// column sums (bias gradients), dtype casts.  Each is written to touch every byte once with 16-byte accesses.
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------ LayerNorm
// One warp per row; the row (D <= 8192) is read once into registers-by-loop and written once.
// x, y: bf16 [rows, D]; gamma/beta: fp32 [D]; mean/rstd: fp32 [rows] (saved for backward).
template <int VEC>
__global__ void layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int D, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (long long)row * D;
  float s = 0.f, ss = 0.f;
  for (int i = lane * 8; i < D; i += 32 * 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float2 f = __bfloat1622float2(h[u]);
      s += f.x + f.y;
      ss += f.x * f.x + f.y * f.y;
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const float mean = s / D;
  const float var = fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + (long long)row * D;
  for (int i = lane * 8; i < D; i += 32 * 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float2 f = __bfloat1622float2(h[u]);
      const int c = i + 2 * u;
      float a = (f.x - mean) * rstd * gamma[c] + (beta ? beta[c] : 0.f);
      float b = (f.y - mean) * rstd * gamma[c + 1] + (beta ? beta[c + 1] : 0.f);
      o[u] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<uint4*>(yr + i) = *reinterpret_cast<uint4*>(o);
  }
}

// Register-resident forward for D = NCH * 256 (NCH <= 4): the row is read once, gamma / beta come in as float4.
template <int NCH>
__global__ void __launch_bounds__(256) layernorm_fwd_reg_kernel(
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
    __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, float eps) {
  constexpr int D = NCH * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (long long)row * D;
  float v[NCH][8];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + j * 256 + lane * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float2 f = __bfloat1622float2(h[u]);
      v[j][2 * u] = f.x;
      v[j][2 * u + 1] = f.y;
      s += f.x + f.y;
    }
  }
  const float mean = warp_sum(s) * (1.f / D);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      v[j][u] -= mean;
      ss += v[j][u] * v[j][u];
    }
  const float rstd = rsqrtf(warp_sum(ss) * (1.f / D) + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + (long long)row * D;
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = j * 256 + lane * 8;
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
    if (beta) {
      b0 = *reinterpret_cast<const float4*>(beta + c);
      b1 = *reinterpret_cast<const float4*>(beta + c + 4);
    }
    __align__(16) __nv_bfloat162 o[4];
    o[0] = __floats2bfloat162_rn(v[j][0] * rstd * g0.x + b0.x, v[j][1] * rstd * g0.y + b0.y);
    o[1] = __floats2bfloat162_rn(v[j][2] * rstd * g0.z + b0.z, v[j][3] * rstd * g0.w + b0.w);
    o[2] = __floats2bfloat162_rn(v[j][4] * rstd * g1.x + b1.x, v[j][5] * rstd * g1.y + b1.y);
    o[3] = __floats2bfloat162_rn(v[j][6] * rstd * g1.z + b1.z, v[j][7] * rstd * g1.w + b1.w);
    *reinterpret_cast<uint4*>(yr + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// dx for one row per warp; per-block partial dgamma/dbeta accumulated in shared memory then atomically added
// to fp32 [D] outputs (which the caller zeroes or which already hold earlier gradient contributions).
__global__ void layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                     const float* __restrict__ gamma, const float* __restrict__ mean,
                                     const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int D,
                                     int rows_per_block, const __nv_bfloat16* __restrict__ dres) {
  extern __shared__ float sh[];  // [2*D]
  float* sg = sh;
  float* sb = sh + D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) sh[i] = 0.f;
  __syncthreads();
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  for (int row = row0 + w; row < row1; row += warps) {
    const __nv_bfloat16* xr = x + (long long)row * D;
    const __nv_bfloat16* gr = dy + (long long)row * D;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int i = lane * 8; i < D; i += 256) {
      uint4 rx = *reinterpret_cast<const uint4*>(xr + i);
      uint4 rg = *reinterpret_cast<const uint4*>(gr + i);
      const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
      const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float2 fx = __bfloat1622float2(hx[u]), fg = __bfloat1622float2(hg[u]);
        const int c = i + 2 * u;
        float xh0 = (fx.x - mu) * rs, xh1 = (fx.y - mu) * rs;
        float g0 = fg.x * gamma[c], g1 = fg.y * gamma[c + 1];
        s1 += g0 + g1;
        s2 += g0 * xh0 + g1 * xh1;
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    __nv_bfloat16* dr = dx + (long long)row * D;
    for (int i = lane * 8; i < D; i += 256) {
      uint4 rx = *reinterpret_cast<const uint4*>(xr + i);
      uint4 rg = *reinterpret_cast<const uint4*>(gr + i);
      const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
      const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
      __align__(16) __nv_bfloat162 o[4];
      uint4 rr = make_uint4(0u, 0u, 0u, 0u);  // bf16 zeros
      if (dres) rr = *reinterpret_cast<const uint4*>(dres + (long long)row * D + i);
      const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float2 fx = __bfloat1622float2(hx[u]), fg = __bfloat1622float2(hg[u]);
        const float2 fr = __bfloat1622float2(hr[u]);
        const int c = i + 2 * u;
        float xh0 = (fx.x - mu) * rs, xh1 = (fx.y - mu) * rs;
        float g0 = fg.x * gamma[c], g1 = fg.y * gamma[c + 1];
        o[u] = __floats2bfloat162_rn(rs * (g0 - s1 - xh0 * s2) + fr.x, rs * (g1 - s1 - xh1 * s2) + fr.y);
        atomicAdd(&sg[c], fg.x * xh0);
        atomicAdd(&sg[c + 1], fg.y * xh1);
        atomicAdd(&sb[c], fg.x);
        atomicAdd(&sb[c + 1], fg.y);
      }
      *reinterpret_cast<uint4*>(dr + i) = *reinterpret_cast<uint4*>(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    atomicAdd(&dgamma[i], sg[i]);
    if (dbeta) atomicAdd(&dbeta[i], sb[i]);
  }
}

// Register-resident variant for D = NCH * 256 (NCH <= 4): a lane owns the same 8*NCH columns in every row its warp
// visits, so x / dy are read once and the dgamma / dbeta partial sums live in registers until the end of the block.
template <int NCH>
__global__ void __launch_bounds__(256) layernorm_bwd_reg_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
    const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
    float* __restrict__ dbeta, int rows, int rows_per_block, const __nv_bfloat16* __restrict__ dres) {
  constexpr int D = NCH * 256;
  __shared__ float sg[D];
  __shared__ float sb[D];
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    sg[i] = 0.f;
    sb[i] = 0.f;
  }
  __syncthreads();
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float gam[NCH][8], ag[NCH][8], ab[NCH][8];
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      gam[j][u] = gamma[j * 256 + lane * 8 + u];
      ag[j][u] = 0.f;
      ab[j][u] = 0.f;
    }
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  for (int row = row0 + w; row < row1; row += warps) {
    const __nv_bfloat16* xr = x + (long long)row * D;
    const __nv_bfloat16* gr = dy + (long long)row * D;
    const float mu = mean[row], rs = rstd[row];
    float xh[NCH][8], g[NCH][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const uint4 rx = *reinterpret_cast<const uint4*>(xr + j * 256 + lane * 8);
      const uint4 rg = *reinterpret_cast<const uint4*>(gr + j * 256 + lane * 8);
      const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
      const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 fx = __bfloat1622float2(hx[u]), fg = __bfloat1622float2(hg[u]);
        xh[j][2 * u] = (fx.x - mu) * rs;
        xh[j][2 * u + 1] = (fx.y - mu) * rs;
        g[j][2 * u] = fg.x;
        g[j][2 * u + 1] = fg.y;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float gg = g[j][u] * gam[j][u];
        s1 += gg;
        s2 += gg * xh[j][u];
        ag[j][u] += g[j][u] * xh[j][u];
        ab[j][u] += g[j][u];
      }
    }
    s1 = warp_sum(s1) * (1.f / D);
    s2 = warp_sum(s2) * (1.f / D);
    __nv_bfloat16* dr = dx + (long long)row * D;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      __align__(16) __nv_bfloat162 o[4];
      uint4 rr = make_uint4(0u, 0u, 0u, 0u);  // bf16 zeros
      if (dres) rr = *reinterpret_cast<const uint4*>(dres + (long long)row * D + j * 256 + lane * 8);
      const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 fr = __bfloat1622float2(hr[u]);
        const float a = rs * (g[j][2 * u] * gam[j][2 * u] - s1 - xh[j][2 * u] * s2) + fr.x;
        const float b = rs * (g[j][2 * u + 1] * gam[j][2 * u + 1] - s1 - xh[j][2 * u + 1] * s2) + fr.y;
        o[u] = __floats2bfloat162_rn(a, b);
      }
      *reinterpret_cast<uint4*>(dr + j * 256 + lane * 8) = *reinterpret_cast<const uint4*>(o);
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      atomicAdd(&sg[j * 256 + lane * 8 + u], ag[j][u]);
      atomicAdd(&sb[j * 256 + lane * 8 + u], ab[j][u]);
    }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    atomicAdd(&dgamma[i], sg[i]);
    if (dbeta) atomicAdd(&dbeta[i], sb[i]);
  }
}

// ------------------------------------------------------------------------------------------------ AdamW
// scalars[1] = gradient multiplier (clip coefficient x loss scale), read from device memory.
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ lowp, long long n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float rsqrt_bc2, const float* __restrict__ scalars,
                             const int* __restrict__ status) {
  // The update is skipped as a whole when the gradient norm of this step was not finite (scalars[2], set by the clip kernel
  // after the gradients were reduced over ranks, hence identical on all of them) or when a kernel of this step gave up a wait
  // (status word): the gradients may then be incomplete.  The host learns of either through its own reads.
  if ((scalars && scalars[2] != 0.f) || (status && *((volatile const int*)status) != 0)) return;
  const float gs = scalars ? scalars[1] : 1.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 pp = *reinterpret_cast<float4*>(p + i);
      float4 gg = *reinterpret_cast<const float4*>(g + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* pa = &pp.x; float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float gr = ga[u] * gs;
        ma[u] = beta1 * ma[u] + (1.f - beta1) * gr;
        va[u] = beta2 * va[u] + (1.f - beta2) * gr * gr;
        float denom = sqrtf(va[u]) * rsqrt_bc2 + eps;
        pa[u] = pa[u] * (1.f - lr * wd) - (lr / bc1) * (ma[u] / denom);
      }
      *reinterpret_cast<float4*>(p + i) = pp;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (lowp) {
        __align__(8) __nv_bfloat162 o[2] = {__floats2bfloat162_rn(pp.x, pp.y), __floats2bfloat162_rn(pp.z, pp.w)};
        *reinterpret_cast<uint2*>(lowp + i) = *reinterpret_cast<uint2*>(o);
      }
    } else {
      for (long long j = i; j < n; ++j) {
        float gr = g[j] * gs;
        float mj = beta1 * m[j] + (1.f - beta1) * gr;
        float vj = beta2 * v[j] + (1.f - beta2) * gr * gr;
        m[j] = mj; v[j] = vj;
        float pj = p[j] * (1.f - lr * wd) - (lr / bc1) * (mj / (sqrtf(vj) * rsqrt_bc2 + eps));
        p[j] = pj;
        if (lowp) lowp[j] = __float2bfloat16(pj);
      }
    }
  }
}

// Sum of squares of an fp32 buffer into partial[blockIdx]; a second tiny kernel finishes and computes the clip coefficient.
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 a = *reinterpret_cast<const float4*>(g + i);
      s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    } else {
      for (long long j = i; j < n; ++j) s += g[j] * g[j];
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void clip_coef_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ scalars, float max_norm,
                                 float grad_scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    float norm = sqrtf(s) * grad_scale;
    scalars[0] = norm;
    float c = max_norm / (norm + 1e-6f);
    scalars[1] = grad_scale * (c < 1.f ? c : 1.f);
    scalars[2] = isfinite(norm) ? 0.f : 1.f;
  }
}

// Column sums of a bf16 [rows, N] matrix into fp32 out[N] (out = beta*out + sum): bias gradients.
// Block handles 64 columns x a slab of rows; partial sums go through shared memory then one atomicAdd per column.
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int rows, int N, float* __restrict__ out,
                              int rows_per_block) {
  __shared__ float acc[8][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int rgroup = threadIdx.x >> 6;  // 0..7 with 512 threads
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float s = 0.f;
  if (c < N)
    for (int r = row0 + rgroup; r < row1; r += 8) s += __bfloat162float(x[(long long)r * ld + c]);
  acc[rgroup][threadIdx.x & 63] = s;
  __syncthreads();
  if (threadIdx.x < 64 && c < N) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += acc[i][threadIdx.x];
    atomicAdd(&out[c], t);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 a = *reinterpret_cast<const float4*>(in + i);
      __align__(8) __nv_bfloat162 o[2] = {__floats2bfloat162_rn(a.x * scale, a.y * scale), __floats2bfloat162_rn(a.z * scale, a.w * scale)};
      *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<uint2*>(o);
    } else {
      for (long long j = i; j < n; ++j) out[j] = __float2bfloat16(in[j] * scale);
    }
  }
}

float g_partial_host_unused;
}  // namespace

SB_API int sb_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, int rows,
                            int D, float eps, cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0) return -1;
  const int warps = 8;
  if (D % 256 == 0 && D <= 1024 && (reinterpret_cast<uintptr_t>(gamma) & 15) == 0 && (!beta || (reinterpret_cast<uintptr_t>(beta) & 15) == 0)) {
    const int nb = (rows + warps - 1) / warps;
    const __nv_bfloat16* gx = (const __nv_bfloat16*)x;
    __nv_bfloat16* gy = (__nv_bfloat16*)y;
    switch (D / 256) {
      case 1: layernorm_fwd_reg_kernel<1><<<nb, warps * 32, 0, stream>>>(gx, gamma, beta, gy, mean, rstd, rows, eps); break;
      case 2: layernorm_fwd_reg_kernel<2><<<nb, warps * 32, 0, stream>>>(gx, gamma, beta, gy, mean, rstd, rows, eps); break;
      case 3: layernorm_fwd_reg_kernel<3><<<nb, warps * 32, 0, stream>>>(gx, gamma, beta, gy, mean, rstd, rows, eps); break;
      default: layernorm_fwd_reg_kernel<4><<<nb, warps * 32, 0, stream>>>(gx, gamma, beta, gy, mean, rstd, rows, eps); break;
    }
    return (int)cudaGetLastError();
  }
  layernorm_fwd_kernel<8><<<(rows + warps - 1) / warps, warps * 32, 0, stream>>>(
      (const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, rows, D, eps);
  return (int)cudaGetLastError();
}

// dx = LayerNorm backward (+ dres when given: the gradient that reaches the same tensor through the residual branch).
SB_API int sb_layernorm_bwd_res(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx,
                                float* dgamma, float* dbeta, const void* dres, int rows, int D, cudaStream_t stream) {
  if (D % 8 != 0 || rows <= 0 || D > 5632) return -1;  // 2*D floats of shared memory
  // the register-resident kernel runs one 256-thread block per SM (246 registers at D = 1024): exactly one wave of blocks
  const bool reg_path = D % 256 == 0 && D <= 1024;
  const int blocks = min(rows, (reg_path ? 1 : 2) * sb_num_sms());
  const int rpb = (rows + blocks - 1) / blocks;
  const int nblocks = (rows + rpb - 1) / rpb;
  if (reg_path) {
    const __nv_bfloat16 *gdy = (const __nv_bfloat16*)dy, *gx = (const __nv_bfloat16*)x;
    __nv_bfloat16* gdx = (__nv_bfloat16*)dx;
    const __nv_bfloat16* gres = (const __nv_bfloat16*)dres;
    switch (D / 256) {
      case 1: layernorm_bwd_reg_kernel<1><<<nblocks, 256, 0, stream>>>(gdy, gx, gamma, mean, rstd, gdx, dgamma, dbeta, rows, rpb, gres); break;
      case 2: layernorm_bwd_reg_kernel<2><<<nblocks, 256, 0, stream>>>(gdy, gx, gamma, mean, rstd, gdx, dgamma, dbeta, rows, rpb, gres); break;
      case 3: layernorm_bwd_reg_kernel<3><<<nblocks, 256, 0, stream>>>(gdy, gx, gamma, mean, rstd, gdx, dgamma, dbeta, rows, rpb, gres); break;
      default: layernorm_bwd_reg_kernel<4><<<nblocks, 256, 0, stream>>>(gdy, gx, gamma, mean, rstd, gdx, dgamma, dbeta, rows, rpb, gres); break;
    }
    return (int)cudaGetLastError();
  }
  layernorm_bwd_kernel<<<nblocks, 256, 2 * D * sizeof(float), stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, mean, rstd, (__nv_bfloat16*)dx, dgamma, dbeta, rows, D, rpb,
      (const __nv_bfloat16*)dres);
  return (int)cudaGetLastError();
}

SB_API int sb_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx,
                            float* dgamma, float* dbeta, int rows, int D, cudaStream_t stream) {
  return sb_layernorm_bwd_res(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, nullptr, rows, D, stream);
}

SB_API int sb_adamw(float* p, const float* g, float* m, float* v, void* lowp, long long n, float lr, float beta1, float beta2,
                    float eps, float wd, int step, const float* scalars, cudaStream_t stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  const int threads = 256;
  long long blocks = (n / 4 + threads - 1) / threads;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  adamw_kernel<<<(int)blocks, threads, 0, stream>>>(p, g, m, v, (__nv_bfloat16*)lowp, n, lr, beta1, beta2, eps, wd, bc1,
                                                   1.f / sqrtf(bc2), scalars, sb_status_ptr());
  return (int)cudaGetLastError();
}

// partial must hold at least sb_grad_norm_partials() floats.
SB_API int sb_grad_norm_partials() { return sb_num_sms() * 8; }

SB_API int sb_grad_norm_clip(const float* g, long long n, float* partial, float* scalars, float max_norm, float grad_scale,
                             cudaStream_t stream) {
  const int blocks = sb_num_sms() * 8;
  sumsq_kernel<<<blocks, 256, 0, stream>>>(g, n, partial);
  clip_coef_kernel<<<1, 256, 0, stream>>>(partial, blocks, scalars, max_norm, grad_scale);
  return (int)cudaGetLastError();
}

// out[N] += column sums of x[rows, N]   (caller zeroes `out` when it wants a plain sum)
SB_API int sb_colsum_bf16(const void* x, long long ld, int rows, int N, float* out, cudaStream_t stream) {
  if (rows <= 0 || N <= 0) return 0;
  const int col_blocks = (N + 63) / 64;
  int row_blocks = (4 * sb_num_sms() + col_blocks - 1) / col_blocks;
  if (row_blocks > (rows + 63) / 64) row_blocks = (rows + 63) / 64;
  if (row_blocks < 1) row_blocks = 1;
  const int rpb = (rows + row_blocks - 1) / row_blocks;
  dim3 grid(col_blocks, (rows + rpb - 1) / rpb);
  colsum_kernel<<<grid, 512, 0, stream>>>((const __nv_bfloat16*)x, ld, rows, N, out, rpb);
  return (int)cudaGetLastError();
}

SB_API int sb_cast_f32_bf16(const float* in, void* out, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cast_f32_to_bf16_kernel<<<(int)blocks, 256, 0, stream>>>(in, (__nv_bfloat16*)out, n, scale);
  return (int)cudaGetLastError();
}

namespace {
// dz = alpha * mask * dy * act'(z) for bf16 [rows, N] (dy may have a row stride; z (optional) and dz are dense).  The
// dropout mask (thresh != 0) is rebuilt from (seed, r * N + c), matching the GEMM epilogue that applied it.
__global__ void scale_dact_kernel(const __nv_bfloat16* __restrict__ dy, long long ld_dy, const __nv_bfloat16* __restrict__ z,
                                  __nv_bfloat16* __restrict__ dz, int rows, int N, int act, float alpha, unsigned int thresh,
                                  float drop_scale, unsigned long long seed) {
  const long long total8 = (long long)rows * (N / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / (N / 8)), c = (int)(i % (N / 8)) * 8;
    uint4 rg = *reinterpret_cast<const uint4*>(dy + (long long)r * ld_dy + c);
    uint4 rz = z ? *reinterpret_cast<const uint4*>(z + (long long)r * N + c) : make_uint4(0, 0, 0, 0);
    const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
    const __nv_bfloat162* hz = reinterpret_cast<const __nv_bfloat162*>(&rz);
    __align__(16) __nv_bfloat162 o[4];
    // N is a multiple of 8 and c of 8: the eight elements are two aligned groups of four, one hash each
    const unsigned long long grp = ((unsigned long long)r * N + c) >> 2;
    const unsigned int h0 = thresh ? sb_dropout_hash4(seed, grp) : 0u, h1 = thresh ? sb_dropout_hash4(seed, grp + 1) : 0u;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float2 g = __bfloat1622float2(hg[u]), zz = __bfloat1622float2(hz[u]);
      float d0, d1;
      if (act == 1) { d0 = zz.x > 0.f ? 1.f : 0.f; d1 = zz.y > 0.f ? 1.f : 0.f; }
      else if (act == 2) { d0 = sb_dswish(zz.x); d1 = sb_dswish(zz.y); }
      else if (act == 3) { d0 = sb_dgelu(zz.x); d1 = sb_dgelu(zz.y); }
      else { d0 = d1 = 1.f; }
      if (thresh) {
        const unsigned int h = u < 2 ? h0 : h1;
        d0 = sb_dropout_keep_in(h, (2 * u) & 3, thresh) ? d0 * drop_scale : 0.f;
        d1 = sb_dropout_keep_in(h, (2 * u + 1) & 3, thresh) ? d1 * drop_scale : 0.f;
      }
      o[u] = __floats2bfloat162_rn(alpha * g.x * d0, alpha * g.y * d1);
    }
    *reinterpret_cast<uint4*>(dz + (long long)r * N + c) = *reinterpret_cast<uint4*>(o);
  }
}
}  // namespace

namespace {
// The same element-wise work with the bias gradient folded in: a thread keeps ONE group of eight columns and walks down the rows,
// so that it can also accumulate the column sums of dz (= the gradient of the linear layer's bias, which the caller would
// otherwise compute with a second pass over dz).  Block = 256 threads = CG column groups x RL row lanes; the block's row lanes
// meet in shared memory and one atomic per column and block reaches gb (which is accumulated into).
__global__ void __launch_bounds__(256) scale_dact_colsum_kernel(const __nv_bfloat16* __restrict__ dy, long long ld_dy,
                                                               const __nv_bfloat16* __restrict__ z, __nv_bfloat16* __restrict__ dz, int rows,
                                                               int N, int act, float alpha, unsigned int thresh, float drop_scale,
                                                               unsigned long long seed, float* __restrict__ gb, int cgs, int rows_per_block) {
  __shared__ float red[256 * 8];
  const int rl_n = 256 / cgs;                               // row lanes of the block
  const int cg = blockIdx.x * cgs + (threadIdx.x % cgs);    // this thread's column group
  const int rl = threadIdx.x / cgs;
  const int c = cg * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < N) {
    for (int r = r0 + rl; r < r1; r += rl_n) {
      const uint4 rg = *reinterpret_cast<const uint4*>(dy + (long long)r * ld_dy + c);
      const uint4 rz = z ? *reinterpret_cast<const uint4*>(z + (long long)r * N + c) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
      const __nv_bfloat162* hz = reinterpret_cast<const __nv_bfloat162*>(&rz);
      const unsigned long long grp = ((unsigned long long)r * N + c) >> 2;
      const unsigned int h0 = thresh ? sb_dropout_hash4(seed, grp) : 0u, h1 = thresh ? sb_dropout_hash4(seed, grp + 1) : 0u;
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 g = __bfloat1622float2(hg[u]), zz = __bfloat1622float2(hz[u]);
        float d0, d1;
        if (act == 1) { d0 = zz.x > 0.f ? 1.f : 0.f; d1 = zz.y > 0.f ? 1.f : 0.f; }
        else if (act == 2) { d0 = sb_dswish(zz.x); d1 = sb_dswish(zz.y); }
        else if (act == 3) { d0 = sb_dgelu(zz.x); d1 = sb_dgelu(zz.y); }
        else { d0 = d1 = 1.f; }
        if (thresh) {
          const unsigned int h = u < 2 ? h0 : h1;
          d0 = sb_dropout_keep_in(h, (2 * u) & 3, thresh) ? d0 * drop_scale : 0.f;
          d1 = sb_dropout_keep_in(h, (2 * u + 1) & 3, thresh) ? d1 * drop_scale : 0.f;
        }
        o[u] = __floats2bfloat162_rn(alpha * g.x * d0, alpha * g.y * d1);
        const float2 w = __bfloat1622float2(o[u]);          // the sums see the rounded values, as a separate pass over dz would
        acc[2 * u] += w.x;
        acc[2 * u + 1] += w.y;
      }
      *reinterpret_cast<uint4*>(dz + (long long)r * N + c) = *reinterpret_cast<uint4*>(o);
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[threadIdx.x * 8 + k] = acc[k];
  __syncthreads();
  if (rl == 0 && c < N) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float sum = 0.f;
      for (int q = 0; q < rl_n; ++q) sum += red[(q * cgs + (threadIdx.x % cgs)) * 8 + k];
      atomicAdd(gb + c + k, sum);
    }
  }
}
}  // namespace

// dz = alpha * mask * dy * act'(z) and gb[N] += column sums of dz, in one pass.
SB_API int sb_scale_dact_dropout_bias(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                                      float drop_p, unsigned long long seed, float* gb, cudaStream_t stream) {
  if (N % 8 != 0 || rows <= 0 || !gb) return -1;
  if (z == nullptr) act = 0;
  const int ngroups = N / 8;
  int cgs = ngroups >= 128 ? 128 : (ngroups >= 64 ? 64 : (ngroups >= 32 ? 32 : 16));   // column groups per block (divides 256)
  const int col_blocks = (ngroups + cgs - 1) / cgs;
  int row_blocks = (4 * sb_num_sms() + col_blocks - 1) / col_blocks;
  const int rl_n = 256 / cgs;
  if (row_blocks > (rows + 8 * rl_n - 1) / (8 * rl_n)) row_blocks = (rows + 8 * rl_n - 1) / (8 * rl_n);
  if (row_blocks < 1) row_blocks = 1;
  const int rpb = (rows + row_blocks - 1) / row_blocks;
  dim3 grid(col_blocks, (rows + rpb - 1) / rpb);
  scale_dact_colsum_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, ld_dy, (const __nv_bfloat16*)z, (__nv_bfloat16*)dz, rows, N,
                                                    act, alpha, sb_dropout_threshold(drop_p), sb_dropout_scale(drop_p), seed, gb, cgs, rpb);
  return (int)cudaGetLastError();
}

SB_API int sb_scale_dact_dropout(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                                 float drop_p, unsigned long long seed, cudaStream_t stream);

SB_API int sb_scale_dact(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                         cudaStream_t stream) {
  return sb_scale_dact_dropout(dy, ld_dy, z, dz, rows, N, act, alpha, 0.f, 0ull, stream);
}

SB_API int sb_scale_dact_dropout(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                                 float drop_p, unsigned long long seed, cudaStream_t stream) {
  if (N % 8 != 0 || rows <= 0) return -1;
  if (z == nullptr) act = 0;
  long long total8 = (long long)rows * (N / 8);
  long long blocks = (total8 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  scale_dact_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)dy, ld_dy, (const __nv_bfloat16*)z,
                                                    (__nv_bfloat16*)dz, rows, N, act, alpha, sb_dropout_threshold(drop_p),
                                                    sb_dropout_scale(drop_p), seed);
  return (int)cudaGetLastError();
}
