// Depthwise-striding convolutional sub-sampling (the FastConformer 8x front end) as channels-last kernels.
//
// The reference runs this front end as a chain of library convolutions in NCHW with a masking multiply before every layer
// (nemo/collections/asr/parts/submodules/subsampling.py:184-257, MaskedConvSequential :697-731).  On bucketed ~300 s batches
// that chain costs more than eight milliseconds per training step: the depthwise 3x3 / stride-2 backward kernels of the
// library alone take 2.8 ms.  Everything here is memory-bound by design instead:
//   * activations are [B, T, F, C] bf16 with the channel innermost: a thread owns 8 channels (one 16-byte vector) of one
//     (t, f) position, 32 threads cover C = 256, every load and store is a full coalesced line;
//   * the length masks are folded into the kernels (inputs are read as zero beyond the utterance's length, outputs are
//     written as zero beyond it), so no masking pass exists;
//   * first layer (1 -> C, 3x3, stride 2) + ReLU is one kernel; its backward (weight / bias gradients only, the input is
//     the feature matrix) is fused into the data-gradient kernel of the depthwise layer that follows, so the gradient of the
//     largest activation of the model ([B, T/2, F/2, C]) is never written;
//   * the depthwise backward kernel produces the data gradient, the weight gradient and the bias gradient in one pass over
//     the input positions (per-thread register accumulators, one block-level reduction, one atomic per value and block);
//   * the pointwise 1x1 convolutions are plain GEMMs over [B*T*F, C] rows and run on the tcgen05 GEMM with its fused
//     bias + ReLU epilogue; the final flatten is a masked [F, C] -> [C, F] transpose feeding the output projection GEMM.
// Padding: `pad` rows / columns before the first element (1 for the symmetric layers, 2 for the causal ones); the output
// extent is supplied by the caller.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  __align__(16) __nv_bfloat162 o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return *reinterpret_cast<const uint4*>(o);
}

// y[b, to, fo, c] = (to < Lout[b]) * relu(bias[c] + sum_ij w[c, i, j] * x[b, 2 to - pad + i, 2 fo - pad + j]),  x read as 0 outside
// [0, min(T, Lin[b])) x [0, F).  x is fp32 with arbitrary strides (the feature matrix is usually a transposed view).
__global__ void __launch_bounds__(THREADS) conv1_fwd_kernel(const float* __restrict__ x, long long sb, long long st, long long sf,
                                                           const long long* __restrict__ Lin, const long long* __restrict__ Lout,
                                                           const float* __restrict__ w, const float* __restrict__ bias,
                                                           __nv_bfloat16* __restrict__ y, int B, int T, int F, int To, int Fo, int C,
                                                           int pad) {
  const int tpp = C >> 3;                        // threads per position
  const int slot = threadIdx.x / tpp, cg = threadIdx.x - slot * tpp;
  const int slots = THREADS / tpp;
  float wr[8][9], br[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    br[c] = bias ? bias[cg * 8 + c] : 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) wr[c][k] = w[(cg * 8 + c) * 9 + k];
  }
  const long long npos = (long long)B * To * Fo;
  for (long long p = (long long)blockIdx.x * slots + slot; p < npos; p += (long long)gridDim.x * slots) {
    const int fo = (int)(p % Fo);
    const long long r = p / Fo;
    const int to = (int)(r % To), b = (int)(r / To);
    float acc[8];
    const bool live = to < (int)Lout[b];
    if (live) {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = br[c];
      const int tlim = min(T, (int)Lin[b]);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int t = 2 * to - pad + i;
        if (t < 0 || t >= tlim) continue;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int f = 2 * fo - pad + j;
          if (f < 0 || f >= F) continue;
          const float xv = __ldg(x + b * sb + t * st + f * sf);
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] = fmaf(wr[c][i * 3 + j], xv, acc[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = fmaxf(acc[c], 0.f);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.f;
    }
    *reinterpret_cast<uint4*>(y + p * C + cg * 8) = pack8(acc);
  }
}

// z[b, to, fo, c] = (to < Lout[b]) * (bias[c] + sum_ij w[c, i, j] * yin[b, 2 to - pad + i, 2 fo - pad + j, c]),  yin read as 0 outside
// [0, min(Ti, Lin[b])) x [0, Fi)
__global__ void __launch_bounds__(THREADS) dw_fwd_kernel(const __nv_bfloat16* __restrict__ yin, const long long* __restrict__ Lin,
                                                        const long long* __restrict__ Lout, const float* __restrict__ w,
                                                        const float* __restrict__ bias, __nv_bfloat16* __restrict__ z, int B, int Ti,
                                                        int Fi, int To, int Fo, int C, int pad) {
  const int tpp = C >> 3;
  const int slot = threadIdx.x / tpp, cg = threadIdx.x - slot * tpp;
  const int slots = THREADS / tpp;
  float wr[8][9], br[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    br[c] = bias ? bias[cg * 8 + c] : 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) wr[c][k] = w[(cg * 8 + c) * 9 + k];
  }
  const long long npos = (long long)B * To * Fo;
  for (long long p = (long long)blockIdx.x * slots + slot; p < npos; p += (long long)gridDim.x * slots) {
    const int fo = (int)(p % Fo);
    const long long r = p / Fo;
    const int to = (int)(r % To), b = (int)(r / To);
    float acc[8];
    if (to < (int)Lout[b]) {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = br[c];
      const int tlim = min(Ti, (int)Lin[b]);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int t = 2 * to - pad + i;
        if (t < 0 || t >= tlim) continue;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int f = 2 * fo - pad + j;
          if (f < 0 || f >= Fi) continue;
          float v[8];
          unpack8(*reinterpret_cast<const uint4*>(yin + (((long long)b * Ti + t) * Fi + f) * C + cg * 8), v);
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] = fmaf(wr[c][i * 3 + j], v[c], acc[c]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.f;
    }
    *reinterpret_cast<uint4*>(z + p * C + cg * 8) = pack8(acc);
  }
}

// Sum `v` over the position slots of the block (threads that own the same channel group) and add it to *dst for slot 0's threads.
__device__ __forceinline__ void slot_reduce_add(float v, float* red, int tpp, int slots, float* dst) {
  red[threadIdx.x] = v;
  __syncthreads();
  if ((int)threadIdx.x < tpp) {
    float s = 0.f;
    for (int q = 0; q < slots; ++q) s += red[q * tpp + threadIdx.x];
    if (s != 0.f) atomicAdd(dst, s);
  }
  __syncthreads();
}

// Backward of dw_fwd over INPUT positions.  dz is the gradient of z (zero beyond Lout by construction of the caller's graph).
//   dyin[b, ti, fi, c] = (ti < Lin[b]) * sum over the outputs (to, fo) that read this position through tap (i, j) of dz * w[c, i, j]
//   gw[c, i, j]       += sum dz[b, to, fo, c] * yin[b, ti, fi, c]          gb[c] += sum of dz over output positions (centre tap)
// FIRST = true: yin is the output of conv1_fwd (ReLU, masked).  dyin is not stored; instead dz1 = dyin * (yin > 0) feeds the
// first layer's gradients:  gw0[c, i, j] += dz1 * x[b, 2 ti - pad0 + i, 2 fi - pad0 + j],  gb0[c] += dz1.
template <bool FIRST>
__global__ void __launch_bounds__(THREADS) dw_bwd_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ yin,
                                                        const long long* __restrict__ Lin, const long long* __restrict__ Lout,
                                                        const float* __restrict__ w, __nv_bfloat16* __restrict__ dyin,
                                                        float* __restrict__ gw, float* __restrict__ gb, int B, int Ti, int Fi, int To,
                                                        int Fo, int C, int pad,
                                                        // first layer (FIRST only)
                                                        const float* __restrict__ x, long long sb, long long st, long long sf,
                                                        const long long* __restrict__ L0, int T0, int F0, int pad0,
                                                        float* __restrict__ gw0, float* __restrict__ gb0) {
  __shared__ float red[THREADS];
  __shared__ __align__(16) float ws[9 * 512];     // weights as [tap][channel]: the register file is needed for the accumulators
  const int tpp = C >> 3;
  const int slot = threadIdx.x / tpp, cg = threadIdx.x - slot * tpp;
  const int slots = THREADS / tpp;
  for (int i = threadIdx.x; i < C * 9; i += THREADS) ws[(i % 9) * C + i / 9] = w[i];
  __syncthreads();
  float aw[8][9], ab[8];
  float aw0[FIRST ? 8 : 1][9], ab0[FIRST ? 8 : 1];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    ab[c] = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) aw[c][k] = 0.f;
  }
#pragma unroll
  for (int c = 0; c < (FIRST ? 8 : 1); ++c) {
    ab0[c] = 0.f;
#pragma unroll
    for (int k = 0; k < 9; ++k) aw0[c][k] = 0.f;
  }
  const long long npos = (long long)B * Ti * Fi;
  for (long long p = (long long)blockIdx.x * slots + slot; p < npos; p += (long long)gridDim.x * slots) {
    const int fi = (int)(p % Fi);
    const long long r = p / Fi;
    const int ti = (int)(r % Ti), b = (int)(r / Ti);
    float dy[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) dy[c] = 0.f;
    const bool live = ti < (int)Lin[b];
    float yv[8];
    if (live) {
      unpack8(*reinterpret_cast<const uint4*>(yin + p * C + cg * 8), yv);
      const int olim = min(To, (int)Lout[b]);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int t2 = ti + pad - i;
        if (t2 < 0 || (t2 & 1)) continue;
        const int to = t2 >> 1;
        if (to >= olim) continue;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int f2 = fi + pad - j;
          if (f2 < 0 || (f2 & 1)) continue;
          const int fo = f2 >> 1;
          if (fo >= Fo) continue;
          float g[8];
          unpack8(*reinterpret_cast<const uint4*>(dz + (((long long)b * To + to) * Fo + fo) * C + cg * 8), g);
          const float4 w0 = *reinterpret_cast<const float4*>(ws + (i * 3 + j) * C + cg * 8);
          const float4 w1 = *reinterpret_cast<const float4*>(ws + (i * 3 + j) * C + cg * 8 + 4);
          const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            dy[c] = fmaf(g[c], wv[c], dy[c]);
            aw[c][i * 3 + j] = fmaf(g[c], yv[c], aw[c][i * 3 + j]);
          }
        }
      }
    }
    if (!FIRST) {
      *reinterpret_cast<uint4*>(dyin + p * C + cg * 8) = pack8(dy);
    } else if (live) {
      float d1[8];
      bool any = false;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        d1[c] = yv[c] > 0.f ? dy[c] : 0.f;
        any |= d1[c] != 0.f;
      }
      if (any) {
        const int tlim = min(T0, (int)L0[b]);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const int t = 2 * ti - pad0 + i;
          if (t < 0 || t >= tlim) continue;
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            const int f = 2 * fi - pad0 + j;
            if (f < 0 || f >= F0) continue;
            const float xv = __ldg(x + b * sb + t * st + f * sf);
#pragma unroll
            for (int c = 0; c < 8; ++c) aw0[c][i * 3 + j] = fmaf(d1[c], xv, aw0[c][i * 3 + j]);
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) ab0[c] += d1[c];
      }
    }
  }
  // bias gradient of the depthwise layer: sum of dz over output positions, walked by the same threads
  {
    const long long nout = (long long)B * To * Fo;
    for (long long p = (long long)blockIdx.x * slots + slot; p < nout; p += (long long)gridDim.x * slots) {
      const long long r = p / Fo;
      const int to = (int)(r % To), b = (int)(r / To);
      if (to >= (int)Lout[b]) continue;
      float g[8];
      unpack8(*reinterpret_cast<const uint4*>(dz + p * C + cg * 8), g);
#pragma unroll
      for (int c = 0; c < 8; ++c) ab[c] += g[c];
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    slot_reduce_add(ab[c], red, tpp, slots, gb + cg * 8 + c);
#pragma unroll
    for (int k = 0; k < 9; ++k) slot_reduce_add(aw[c][k], red, tpp, slots, gw + (cg * 8 + c) * 9 + k);
  }
  if (FIRST) {
#pragma unroll
    for (int c = 0; c < (FIRST ? 8 : 1); ++c) {
      slot_reduce_add(ab0[c], red, tpp, slots, gb0 + cg * 8 + c);
#pragma unroll
      for (int k = 0; k < 9; ++k) slot_reduce_add(aw0[c][k], red, tpp, slots, gw0 + (cg * 8 + c) * 9 + k);
    }
  }
}

// One block per (b, t) row: out[b, t, q, p] = (t < L[b]) * in[b, t, p, q] for in of shape [B, T, P, Q] (bf16).  Forward flatten:
// (P, Q) = (F, C) gives the reference's channel-major feature order; the backward pass calls it with (P, Q) = (C, F).
__global__ void __launch_bounds__(THREADS) mask_transpose_kernel(const __nv_bfloat16* __restrict__ in, const long long* __restrict__ L,
                                                                __nv_bfloat16* __restrict__ out, int T, int P, int Q) {
  extern __shared__ __nv_bfloat16 tile[];
  const long long row = blockIdx.x;
  const int b = (int)(row / T), t = (int)(row % T);
  const int n = P * Q;
  const bool live = t < (int)L[b];
  if (live) {
    for (int i = threadIdx.x; i < n; i += THREADS) tile[i] = in[row * n + i];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < n; o += THREADS) {
    const int q = o / P, p = o - q * P;
    out[row * n + o] = live ? tile[p * Q + q] : __float2bfloat16(0.f);
  }
}

inline int conv_grid(long long npos, int slots) {
  long long blocks = (npos + slots - 1) / slots;
  const long long cap = (long long)sb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}
inline bool channels_ok(int C) { return C >= 8 && C <= 512 && C % 8 == 0 && THREADS % (C / 8) == 0; }

}  // namespace

SB_API int sb_subs_conv1_fwd(const float* x, long long sb, long long st, long long sf, const long long* Lin, const long long* Lout,
                             const float* w, const float* bias, void* y, int B, int T, int F, int To, int Fo, int C, int pad,
                             cudaStream_t stream) {
  if (!channels_ok(C) || B <= 0 || To <= 0 || Fo <= 0) return -1;
  conv1_fwd_kernel<<<conv_grid((long long)B * To * Fo, THREADS / (C / 8)), THREADS, 0, stream>>>(
      x, sb, st, sf, Lin, Lout, w, bias, (__nv_bfloat16*)y, B, T, F, To, Fo, C, pad);
  return (int)cudaGetLastError();
}

SB_API int sb_subs_dw_fwd(const void* yin, const long long* Lin, const long long* Lout, const float* w, const float* bias, void* z, int B,
                          int Ti, int Fi, int To, int Fo, int C, int pad, cudaStream_t stream) {
  if (!channels_ok(C) || B <= 0 || To <= 0 || Fo <= 0) return -1;
  dw_fwd_kernel<<<conv_grid((long long)B * To * Fo, THREADS / (C / 8)), THREADS, 0, stream>>>(
      (const __nv_bfloat16*)yin, Lin, Lout, w, bias, (__nv_bfloat16*)z, B, Ti, Fi, To, Fo, C, pad);
  return (int)cudaGetLastError();
}

// gw [C * 9] and gb [C] are ACCUMULATED into (fp32).  dyin may be null only with the first-layer arguments (x != null), in which
// case gw0 / gb0 are accumulated as well.
SB_API int sb_subs_dw_bwd(const void* dz, const void* yin, const long long* Lin, const long long* Lout, const float* w, void* dyin,
                          float* gw, float* gb, int B, int Ti, int Fi, int To, int Fo, int C, int pad, const float* x, long long sb,
                          long long st, long long sf, const long long* L0, int T0, int F0, int pad0, float* gw0, float* gb0,
                          cudaStream_t stream) {
  if (!channels_ok(C) || B <= 0 || To <= 0 || Fo <= 0 || !gw || !gb) return -1;
  // fewer, longer-lived blocks than the forward kernels: every block ends with a reduction of its 80 (160) accumulators
  long long blocks = (long long)sb_num_sms() * 2;
  const int slots = THREADS / (C / 8);
  const long long need = ((long long)B * Ti * Fi + slots - 1) / slots;
  if (blocks > need) blocks = need;
  if (blocks < 1) blocks = 1;
  if (x) {
    if (!gw0 || !gb0 || !L0) return -1;
    dw_bwd_kernel<true><<<(int)blocks, THREADS, 0, stream>>>((const __nv_bfloat16*)dz, (const __nv_bfloat16*)yin, Lin, Lout, w, nullptr,
                                                            gw, gb, B, Ti, Fi, To, Fo, C, pad, x, sb, st, sf, L0, T0, F0, pad0, gw0,
                                                            gb0);
  } else {
    if (!dyin) return -1;
    dw_bwd_kernel<false><<<(int)blocks, THREADS, 0, stream>>>((const __nv_bfloat16*)dz, (const __nv_bfloat16*)yin, Lin, Lout, w,
                                                             (__nv_bfloat16*)dyin, gw, gb, B, Ti, Fi, To, Fo, C, pad, nullptr, 0, 0, 0,
                                                             nullptr, 0, 0, 0, nullptr, nullptr);
  }
  return (int)cudaGetLastError();
}

SB_API int sb_subs_mask_transpose(const void* in, const long long* L, void* out, int B, int T, int P, int Q, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || P <= 0 || Q <= 0 || (long long)P * Q * 2 > 96 * 1024) return -1;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(mask_transpose_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr_set = true;
  }
  mask_transpose_kernel<<<B * T, THREADS, (size_t)P * Q * 2, stream>>>((const __nv_bfloat16*)in, L, (__nv_bfloat16*)out, T, P, Q);
  return (int)cudaGetLastError();
}
