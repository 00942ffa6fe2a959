// Conformer convolution module core, channels-last: GLU -> pad mask -> depthwise conv (K taps) -> BatchNorm -> SiLU,
// forward and backward, for activations laid out [B, T, C] so that the surrounding pointwise convolutions are plain
// GEMMs on the same buffers (reference math: nemo/collections/asr/parts/submodules/conformer_modules.py:338-368).
//
// Forward:  A) glu_dwconv_fwd: y = dwconv(mask(glu(g))) (bf16) and per-channel sum / sum-of-squares of y (fp32 atomics)
//           B) bn_silu_fwd:    s = silu(gamma * (y - mean) * rstd + beta); training statistics come from (A) (possibly
//                              all-reduced across ranks in between), evaluation uses the running statistics.
// Backward: C) bn_silu_bwd_stats: per-channel sums of dz and dz*xhat, dz = ds * silu'(z)
//           D) dwconv_glu_bwd:    dy (BatchNorm backward) -> dx (transposed depthwise conv) -> GLU backward -> dg, plus
//                                 depthwise weight / bias gradients accumulated per thread and added atomically.
// A thread owns a few adjacent channels and walks along time with a register sliding window, so each activation is
// read once (plus a K-1 halo per time tile).
#include "common.cuh"

namespace {

constexpr int TT = 16;  // time steps per block in the sliding-window kernels

template <int K>
__global__ void glu_dwconv_fwd_kernel(const __nv_bfloat16* __restrict__ g, const uint8_t* __restrict__ pad,
                                      const float* __restrict__ w, const float* __restrict__ bias,
                                      __nv_bfloat16* __restrict__ y, float* __restrict__ stats, int T, int C, int left) {
  // grid: (ceil(C/4/blockDim), ceil(T/TT), B)
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * TT;
  float wk[K][4], bs[4];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int u = 0; u < 4; ++u) wk[k][u] = w[(c + u) * K + k];
#pragma unroll
  for (int u = 0; u < 4; ++u) bs[u] = bias ? bias[c + u] : 0.f;
  float win[K][4];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int u = 0; u < 4; ++u) win[k][u] = 0.f;
  float s1[4] = {0, 0, 0, 0}, s2[4] = {0, 0, 0, 0};
  const __nv_bfloat16* gb = g + (long long)b * T * 2 * C;
  const uint8_t* pb = pad ? pad + (long long)b * T : nullptr;
  // input position needed for output t: t - left + k, k in [0,K).  Stream input positions ti = t0-left .. t0+TT-1-left+K-1.
  for (int step = 0; step < TT + K - 1; ++step) {
    const int ti = t0 - left + step;
    float x[4] = {0, 0, 0, 0};
    if (ti >= 0 && ti < T && !(pb && pb[ti])) {
      uint2 ra = *reinterpret_cast<const uint2*>(gb + (long long)ti * 2 * C + c);
      uint2 rb = *reinterpret_cast<const uint2*>(gb + (long long)ti * 2 * C + C + c);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb);
      float2 a0 = __bfloat1622float2(ha[0]), a1 = __bfloat1622float2(ha[1]);
      float2 b0 = __bfloat1622float2(hb[0]), b1 = __bfloat1622float2(hb[1]);
      x[0] = a0.x * sb_sigmoid(b0.x); x[1] = a0.y * sb_sigmoid(b0.y);
      x[2] = a1.x * sb_sigmoid(b1.x); x[3] = a1.y * sb_sigmoid(b1.y);
    }
#pragma unroll
    for (int k = 0; k < K - 1; ++k)
#pragma unroll
      for (int u = 0; u < 4; ++u) win[k][u] = win[k + 1][u];
#pragma unroll
    for (int u = 0; u < 4; ++u) win[K - 1][u] = x[u];
    const int t = t0 + step - (K - 1);
    if (step >= K - 1 && t < T) {
      float o[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float acc = bs[u];
#pragma unroll
        for (int k = 0; k < K; ++k) acc += wk[k][u] * win[k][u];
        o[u] = acc;
        s1[u] += acc;
        s2[u] += acc * acc;
      }
      __align__(8) __nv_bfloat162 ob[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
      *reinterpret_cast<uint2*>(y + ((long long)b * T + t) * C + c) = *reinterpret_cast<uint2*>(ob);
    }
  }
  if (stats) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      atomicAdd(&stats[c + u], s1[u]);
      atomicAdd(&stats[C + c + u], s2[u]);
    }
  }
}

// mean / rstd per channel from sums (training) or running statistics (evaluation); also the running-stat update.
__global__ void bn_finalize_kernel(const float* __restrict__ stats, float count_arg, const float* __restrict__ count_ptr,
                                   float* __restrict__ mean_rstd,
                                   float* __restrict__ running_mean, float* __restrict__ running_var, int C, float eps,
                                   float momentum, int training) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float count = count_ptr ? *count_ptr : count_arg;
  float mean, var;
  if (training) {
    mean = stats[c] / count;
    var = fmaxf(stats[C + c] / count - mean * mean, 0.f);
    if (running_mean) {
      const float unb = var * (count / fmaxf(count - 1.f, 1.f));
      running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
      running_var[c] = (1.f - momentum) * running_var[c] + momentum * unb;
    }
  } else {
    mean = running_mean[c];
    var = running_var[c];
  }
  mean_rstd[c] = mean;
  mean_rstd[C + c] = rsqrtf(var + eps);
}

__global__ void bn_silu_fwd_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ mean_rstd,
                                   const float* __restrict__ gamma, const float* __restrict__ beta,
                                   __nv_bfloat16* __restrict__ s, long long rows, int C) {
  const long long total8 = rows * (C / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % (C / 8)) * 8;
    uint4 raw = reinterpret_cast<const uint4*>(y)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float2 f = __bfloat1622float2(h[u]);
      const int cc = c + 2 * u;
      float z0 = (f.x - mean_rstd[cc]) * mean_rstd[C + cc] * gamma[cc] + beta[cc];
      float z1 = (f.y - mean_rstd[cc + 1]) * mean_rstd[C + cc + 1] * gamma[cc + 1] + beta[cc + 1];
      o[u] = __floats2bfloat162_rn(sb_swish(z0), sb_swish(z1));
    }
    reinterpret_cast<uint4*>(s)[i] = *reinterpret_cast<uint4*>(o);
  }
}

// sums[c] += sum dz, sums[C+c] += sum dz*xhat over a slab of rows.  Thread owns 4 channels.
__global__ void bn_silu_bwd_stats_kernel(const __nv_bfloat16* __restrict__ ds, const __nv_bfloat16* __restrict__ y,
                                         const float* __restrict__ mean_rstd, const float* __restrict__ gamma,
                                         const float* __restrict__ beta, float* __restrict__ sums, long long rows, int C,
                                         int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float mu[4], rs[4], ga[4], be[4], a1[4] = {0, 0, 0, 0}, a2[4] = {0, 0, 0, 0};
#pragma unroll
  for (int u = 0; u < 4; ++u) { mu[u] = mean_rstd[c + u]; rs[u] = mean_rstd[C + c + u]; ga[u] = gamma[c + u]; be[u] = beta[c + u]; }
  for (long long r = r0; r < r1; ++r) {
    uint2 rd = *reinterpret_cast<const uint2*>(ds + r * C + c);
    uint2 ry = *reinterpret_cast<const uint2*>(y + r * C + c);
    const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&rd);
    const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry);
    float d[4], yy[4];
    float2 t0 = __bfloat1622float2(hd[0]), t1 = __bfloat1622float2(hd[1]);
    d[0] = t0.x; d[1] = t0.y; d[2] = t1.x; d[3] = t1.y;
    t0 = __bfloat1622float2(hy[0]); t1 = __bfloat1622float2(hy[1]);
    yy[0] = t0.x; yy[1] = t0.y; yy[2] = t1.x; yy[3] = t1.y;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float xh = (yy[u] - mu[u]) * rs[u];
      float dz = d[u] * sb_dswish(xh * ga[u] + be[u]);
      a1[u] += dz;
      a2[u] += dz * xh;
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    atomicAdd(&sums[c + u], a1[u]);
    atomicAdd(&sums[C + c + u], a2[u]);
  }
}

// BatchNorm backward -> transposed depthwise conv -> GLU backward, plus dw / dbias accumulation.
// sums: [2C] = (sum dz, sum dz*xhat) over `count` positions (already all-reduced when statistics are synchronised);
// with training == 0 (frozen statistics) the mean terms vanish.
template <int K>
__global__ void dwconv_glu_bwd_kernel(const __nv_bfloat16* __restrict__ ds, const __nv_bfloat16* __restrict__ y,
                                      const __nv_bfloat16* __restrict__ g, const uint8_t* __restrict__ pad,
                                      const float* __restrict__ w, const float* __restrict__ mean_rstd,
                                      const float* __restrict__ gamma, const float* __restrict__ beta,
                                      const float* __restrict__ sums, float count_arg,
                                      const float* __restrict__ count_ptr, int training, __nv_bfloat16* __restrict__ dg, float* __restrict__ dw, float* __restrict__ dbias, int T,
                                      int C, int left) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * TT;
  const int right = K - 1 - left;
  const float count = count_ptr ? *count_ptr : count_arg;
  float wk[K][4], mu[4], rs[4], ga[4], be[4], m1[4], m2[4];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int u = 0; u < 4; ++u) wk[k][u] = w[(c + u) * K + k];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    mu[u] = mean_rstd[c + u]; rs[u] = mean_rstd[C + c + u]; ga[u] = gamma[c + u]; be[u] = beta[c + u];
    m1[u] = training ? sums[c + u] / count : 0.f;
    m2[u] = training ? sums[C + c + u] / count : 0.f;
  }
  // dx[ti] = sum_k w[k] * dy[ti + left - k]; stream output positions to = ti+left-k, i.e. to from t0-right .. t0+TT-1+left.
  // Window slot j holds dy[to] with to = (current ti) + left - j.
  float win[K][4], dwacc[K][4], dbacc[4] = {0, 0, 0, 0};
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int u = 0; u < 4; ++u) { win[k][u] = 0.f; dwacc[k][u] = 0.f; }
  const long long base = (long long)b * T;
  for (int step = 0; step < TT + K - 1; ++step) {
    const int to = t0 - right + step;  // newest dy position entering the window (slot 0 after the shift)
    float dy[4] = {0, 0, 0, 0};
    if (to >= 0 && to < T) {
      uint2 rd = *reinterpret_cast<const uint2*>(ds + (base + to) * C + c);
      uint2 ry = *reinterpret_cast<const uint2*>(y + (base + to) * C + c);
      const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&rd);
      const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry);
      float d[4], yy[4];
      float2 q0 = __bfloat1622float2(hd[0]), q1 = __bfloat1622float2(hd[1]);
      d[0] = q0.x; d[1] = q0.y; d[2] = q1.x; d[3] = q1.y;
      q0 = __bfloat1622float2(hy[0]); q1 = __bfloat1622float2(hy[1]);
      yy[0] = q0.x; yy[1] = q0.y; yy[2] = q1.x; yy[3] = q1.y;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float xh = (yy[u] - mu[u]) * rs[u];
        float dz = d[u] * sb_dswish(xh * ga[u] + be[u]);
        dy[u] = ga[u] * rs[u] * (dz - m1[u] - xh * m2[u]);
      }
      // bias gradient: count each output position once (only by the block that owns it as an input position tile)
      if (to >= t0 && to < t0 + TT) {
#pragma unroll
        for (int u = 0; u < 4; ++u) dbacc[u] += dy[u];
      }
    }
#pragma unroll
    for (int k = K - 1; k > 0; --k)
#pragma unroll
      for (int u = 0; u < 4; ++u) win[k][u] = win[k - 1][u];
#pragma unroll
    for (int u = 0; u < 4; ++u) win[0][u] = dy[u];
    // after this shift, slot j holds dy[to - j]; input position ti satisfies to = ti + left  ->  ti = to - left,
    // and slot k holds dy[ti + left - k] as required.
    const int ti = to - left;
    if (step >= K - 1 && ti < T && ti >= 0) {
      float x[4] = {0, 0, 0, 0}, sa[4], aa[4];
      const bool masked = pad && pad[base + ti];
      uint2 ra = *reinterpret_cast<const uint2*>(g + (base + ti) * 2 * C + c);
      uint2 rb = *reinterpret_cast<const uint2*>(g + (base + ti) * 2 * C + C + c);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb);
      float2 a0 = __bfloat1622float2(ha[0]), a1 = __bfloat1622float2(ha[1]);
      float2 b0 = __bfloat1622float2(hb[0]), b1 = __bfloat1622float2(hb[1]);
      aa[0] = a0.x; aa[1] = a0.y; aa[2] = a1.x; aa[3] = a1.y;
      sa[0] = sb_sigmoid(b0.x); sa[1] = sb_sigmoid(b0.y); sa[2] = sb_sigmoid(b1.x); sa[3] = sb_sigmoid(b1.y);
      float da[4], db[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        x[u] = masked ? 0.f : aa[u] * sa[u];
        float dx = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          dx += wk[k][u] * win[k][u];
          dwacc[k][u] += x[u] * win[k][u];
        }
        if (masked) dx = 0.f;
        da[u] = dx * sa[u];
        db[u] = dx * aa[u] * sa[u] * (1.f - sa[u]);
      }
      __align__(8) __nv_bfloat162 oa[2] = {__floats2bfloat162_rn(da[0], da[1]), __floats2bfloat162_rn(da[2], da[3])};
      __align__(8) __nv_bfloat162 ob[2] = {__floats2bfloat162_rn(db[0], db[1]), __floats2bfloat162_rn(db[2], db[3])};
      *reinterpret_cast<uint2*>(dg + (base + ti) * 2 * C + c) = *reinterpret_cast<uint2*>(oa);
      *reinterpret_cast<uint2*>(dg + (base + ti) * 2 * C + C + c) = *reinterpret_cast<uint2*>(ob);
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
#pragma unroll
    for (int k = 0; k < K; ++k) atomicAdd(&dw[(c + u) * K + k], dwacc[k][u]);
    if (dbias) atomicAdd(&dbias[c + u], dbacc[u]);
  }
}

template <int K>
int launch_fwd(const void* g, const uint8_t* pad, const float* w, const float* bias, void* y, float* stats, int B, int T,
               int C, int left, cudaStream_t stream) {
  const int threads = 128;
  dim3 grid((C / 4 + threads - 1) / threads, (T + TT - 1) / TT, B);
  glu_dwconv_fwd_kernel<K><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)g, pad, w, bias, (__nv_bfloat16*)y, stats, T, C, left);
  return (int)cudaGetLastError();
}
template <int K>
int launch_bwd(const void* ds, const void* y, const void* g, const uint8_t* pad, const float* w, const float* mean_rstd,
               const float* gamma, const float* beta, const float* sums, float count, const float* count_ptr, int training,
               void* dg, float* dw, float* dbias, int B, int T, int C, int left, cudaStream_t stream) {
  const int threads = 128;
  dim3 grid((C / 4 + threads - 1) / threads, (T + TT - 1) / TT, B);
  dwconv_glu_bwd_kernel<K><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)ds, (const __nv_bfloat16*)y,
                                                        (const __nv_bfloat16*)g, pad, w, mean_rstd, gamma, beta, sums, count,
                                                        count_ptr, training, (__nv_bfloat16*)dg, dw, dbias, T, C, left);
  return (int)cudaGetLastError();
}

}  // namespace

SB_API int sb_glu_dwconv_fwd(const void* g, const uint8_t* pad, const float* w, const float* bias, void* y, float* stats,
                             int B, int T, int C, int K, int left, cudaStream_t stream) {
  if (C % 4 != 0 || B <= 0 || T <= 0) return -1;
  switch (K) {
    case 5: return launch_fwd<5>(g, pad, w, bias, y, stats, B, T, C, left, stream);
    case 9: return launch_fwd<9>(g, pad, w, bias, y, stats, B, T, C, left, stream);
    case 15: return launch_fwd<15>(g, pad, w, bias, y, stats, B, T, C, left, stream);
    default: return -2;
  }
}

SB_API int sb_bn_finalize(const float* stats, float count, const float* count_ptr, float* mean_rstd, float* running_mean,
                          float* running_var, int C, float eps, float momentum, int training, cudaStream_t stream) {
  bn_finalize_kernel<<<(C + 255) / 256, 256, 0, stream>>>(stats, count, count_ptr, mean_rstd, running_mean, running_var, C, eps,
                                                         momentum, training);
  return (int)cudaGetLastError();
}

SB_API int sb_bn_silu_fwd(const void* y, const float* mean_rstd, const float* gamma, const float* beta, void* s, long long rows,
                          int C, cudaStream_t stream) {
  if (C % 8 != 0 || rows <= 0) return -1;
  long long total8 = rows * (C / 8), blocks = (total8 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  bn_silu_fwd_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)y, mean_rstd, gamma, beta, (__nv_bfloat16*)s, rows, C);
  return (int)cudaGetLastError();
}

SB_API int sb_bn_silu_bwd_stats(const void* ds, const void* y, const float* mean_rstd, const float* gamma, const float* beta,
                                float* sums, long long rows, int C, cudaStream_t stream) {
  if (C % 4 != 0 || rows <= 0) return -1;
  const int threads = 128;
  const int cblocks = (C / 4 + threads - 1) / threads;
  int rblocks = (4 * sb_num_sms() + cblocks - 1) / cblocks;
  if (rblocks > rows) rblocks = (int)rows;
  const int rpb = (int)((rows + rblocks - 1) / rblocks);
  dim3 grid(cblocks, (unsigned)((rows + rpb - 1) / rpb));
  bn_silu_bwd_stats_kernel<<<grid, threads, 0, stream>>>((const __nv_bfloat16*)ds, (const __nv_bfloat16*)y, mean_rstd, gamma,
                                                        beta, sums, rows, C, rpb);
  return (int)cudaGetLastError();
}

SB_API int sb_dwconv_glu_bwd(const void* ds, const void* y, const void* g, const uint8_t* pad, const float* w,
                             const float* mean_rstd, const float* gamma, const float* beta, const float* sums, float count,
                             const float* count_ptr, int training, void* dg, float* dw, float* dbias, int B, int T, int C, int K, int left,
                             cudaStream_t stream) {
  if (C % 4 != 0 || B <= 0 || T <= 0) return -1;
  switch (K) {
    case 5: return launch_bwd<5>(ds, y, g, pad, w, mean_rstd, gamma, beta, sums, count, count_ptr, training, dg, dw, dbias, B, T, C, left, stream);
    case 9: return launch_bwd<9>(ds, y, g, pad, w, mean_rstd, gamma, beta, sums, count, count_ptr, training, dg, dw, dbias, B, T, C, left, stream);
    case 15: return launch_bwd<15>(ds, y, g, pad, w, mean_rstd, gamma, beta, sums, count, count_ptr, training, dg, dw, dbias, B, T, C, left, stream);
    default: return -2;
  }
}
