// Relative-position (Transformer-XL) attention: the softmax stage between the tcgen05 score GEMMs and the PV GEMM.
//
//   scores[i,j] = (AC[i,j] + BD[i, j + Tq-1-i]) / sqrt(dk)        AC = (q+u) k^T,  BD = (q+v) p^T
//
// The Transformer-XL "rel_shift" is never materialised: it is the column offset (Tq-1-i) applied when BD is read
// (forward) or when the gradient is scattered back (backward).  Masked positions are filled with -10000 before
// the softmax and their probabilities are zeroed afterwards, as the reference does
// (nemo/collections/asr/parts/submodules/multi_head_attention.py:127-148,266-277).  Dropout on the probabilities
// uses a counter-based hash so the backward pass regenerates the same keep-mask from (seed, element index).
//
// Layouts: AC fp32 [B,H,Tq,ldac]; BD fp32 [B,H,Tq,ldbd]; P / Pd bf16 [B,H,Tq,ldp] (ldp >= Tk, multiple of 8, padding
// columns written as zero); mask uint8 [Bm,Tq,Tk] with Bm in {1,B}, non-zero = hidden.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t hash_u32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return (uint32_t)x;
}
__device__ __forceinline__ bool keep_elem(uint64_t seed, uint64_t idx, float p) {
  return (hash_u32(seed + idx * 0x9E3779B97F4A7C15ULL) >> 8) * (1.0f / 16777216.0f) >= p;
}

// q_u = q + u, q_v = q + v for q given with a row stride (q may be a slice of a fused qkv tensor).
__global__ void add_pos_bias_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, const float* __restrict__ u,
                                    const float* __restrict__ v, __nv_bfloat16* __restrict__ qu, __nv_bfloat16* __restrict__ qv,
                                    long long rows, int HD) {
  const long long total8 = rows * (HD / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (HD / 8);
    const int c = (int)(i % (HD / 8)) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(q + r * q_row_stride + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    __align__(16) __nv_bfloat162 ou[4], ov[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      ou[k] = __floats2bfloat162_rn(f.x + u[c + 2 * k], f.y + u[c + 2 * k + 1]);
      ov[k] = __floats2bfloat162_rn(f.x + v[c + 2 * k], f.y + v[c + 2 * k + 1]);
    }
    *reinterpret_cast<uint4*>(qu + r * HD + c) = *reinterpret_cast<uint4*>(ou);
    *reinterpret_cast<uint4*>(qv + r * HD + c) = *reinterpret_cast<uint4*>(ov);
  }
}

// One warp per (b,h,i) row.
__global__ void relpos_softmax_fwd_kernel(const float* __restrict__ AC, const float* __restrict__ BD,
                                          const uint8_t* __restrict__ mask, int mask_bstride, __nv_bfloat16* __restrict__ P,
                                          __nv_bfloat16* __restrict__ Pd, int H, int Tq, int Tk, int ldac, int ldbd, int ldp,
                                          float scale, float drop_p, unsigned long long seed, long long rows) {
  extern __shared__ float sh[];
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sh + (size_t)w * ldp;
  const long long row = (long long)blockIdx.x * warps + w;
  if (row >= rows) return;
  const int i = (int)(row % Tq);
  const long long bh = row / Tq;
  const int b = (int)(bh / H);
  const float* ac = AC + row * ldac;
  const float* bd = BD ? BD + row * ldbd + (Tq - 1 - i) : nullptr;
  const uint8_t* mk = mask ? mask + ((long long)b * mask_bstride + i) * Tk : nullptr;
  float mx = -3.0e38f;
  for (int j = lane; j < Tk; j += 32) {
    float s = (ac[j] + (bd ? bd[j] : 0.f)) * scale;
    if (mk && mk[j]) s = -10000.f;
    buf[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < Tk; j += 32) {
    float e = __expf(buf[j] - mx);
    buf[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  const float keep_scale = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  __nv_bfloat16* pr = P + row * ldp;
  __nv_bfloat16* pdr = Pd ? Pd + row * ldp : nullptr;
  for (int j = lane; j < ldp; j += 32) {
    float pj = 0.f;
    if (j < Tk) {
      pj = buf[j] * inv;
      if (mk && mk[j]) pj = 0.f;
    }
    pr[j] = __float2bfloat16(pj);
    if (pdr) {
      float d = (j < Tk && keep_elem(seed, (uint64_t)row * Tk + j, drop_p)) ? pj * keep_scale : 0.f;
      pdr[j] = __float2bfloat16(d);
    }
  }
}

// dS = P * (dP - sum_j P*dP) * scale with dP = keep ? dPd/(1-p) : 0;   dAC = dS,  dBD[i, j+Tq-1-i] = dS[i,j] (others 0).
__global__ void relpos_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ P, const float* __restrict__ dPd,
                                          __nv_bfloat16* __restrict__ dAC, __nv_bfloat16* __restrict__ dBD, int H, int Tq,
                                          int Tk, int ldp, int lddp, int lddbd, float scale, float drop_p,
                                          unsigned long long seed, long long rows) {
  extern __shared__ float sh[];
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sh + (size_t)w * ldp;
  const long long row = (long long)blockIdx.x * warps + w;
  if (row >= rows) return;
  const int i = (int)(row % Tq);
  const __nv_bfloat16* pr = P + row * ldp;
  const float* dp = dPd + row * lddp;
  const float keep_scale = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  float dot = 0.f;
  for (int j = lane; j < Tk; j += 32) {
    float g = dp[j];
    if (drop_p > 0.f) g = keep_elem(seed, (uint64_t)row * Tk + j, drop_p) ? g * keep_scale : 0.f;
    const float pj = __bfloat162float(pr[j]);
    buf[j] = g;
    dot += pj * g;
  }
  dot = warp_sum(dot);
  __nv_bfloat16* ac = dAC + row * ldp;
  __nv_bfloat16* bd = dBD ? dBD + row * lddbd : nullptr;
  const int shift = Tq - 1 - i;
  if (bd) {
    for (int r = lane; r < lddbd; r += 32)
      if (r < shift || r >= shift + Tk) bd[r] = __float2bfloat16(0.f);
  }
  for (int j = lane; j < ldp; j += 32) {
    float ds = 0.f;
    if (j < Tk) ds = __bfloat162float(pr[j]) * (buf[j] - dot) * scale;
    const __nv_bfloat16 o = __float2bfloat16(ds);
    ac[j] = o;
    if (bd && j < Tk) bd[shift + j] = o;
  }
}

// out = a + b (bf16, dense), used to merge the two query-gradient branches when they cannot be fused.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 ra = reinterpret_cast<const uint4*>(a)[i], rb = reinterpret_cast<const uint4*>(b)[i];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb);
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = __hadd2(ha[k], hb[k]);
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<uint4*>(o);
  }
}

}  // namespace

SB_API int sb_add_pos_bias(const void* q, long long q_row_stride, const float* u, const float* v, void* qu, void* qv,
                           long long rows, int HD, cudaStream_t stream) {
  if (HD % 8 != 0 || rows <= 0) return -1;
  long long total8 = rows * (HD / 8);
  long long blocks = (total8 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  add_pos_bias_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)q, q_row_stride, u, v, (__nv_bfloat16*)qu,
                                                      (__nv_bfloat16*)qv, rows, HD);
  return (int)cudaGetLastError();
}

SB_API int sb_relpos_softmax_fwd(const float* AC, const float* BD, const uint8_t* mask, int mask_bstride, void* P, void* Pd,
                                 int B, int H, int Tq, int Tk, int ldac, int ldbd, int ldp, float scale, float drop_p,
                                 unsigned long long seed, cudaStream_t stream) {
  const long long rows = (long long)B * H * Tq;
  if (rows <= 0 || ldp < Tk) return -1;
  int warps = 8;
  while (warps > 1 && (size_t)warps * ldp * sizeof(float) > 96 * 1024) warps >>= 1;
  const size_t smem = (size_t)warps * ldp * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(relpos_softmax_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  relpos_softmax_fwd_kernel<<<(unsigned)((rows + warps - 1) / warps), warps * 32, smem, stream>>>(
      AC, BD, mask, mask_bstride, (__nv_bfloat16*)P, (__nv_bfloat16*)Pd, H, Tq, Tk, ldac, ldbd, ldp, scale, drop_p, seed, rows);
  return (int)cudaGetLastError();
}

SB_API int sb_relpos_softmax_bwd(const void* P, const float* dPd, void* dAC, void* dBD, int B, int H, int Tq, int Tk, int ldp,
                                 int lddp, int lddbd, float scale, float drop_p, unsigned long long seed, cudaStream_t stream) {
  const long long rows = (long long)B * H * Tq;
  if (rows <= 0) return -1;
  int warps = 8;
  while (warps > 1 && (size_t)warps * ldp * sizeof(float) > 96 * 1024) warps >>= 1;
  const size_t smem = (size_t)warps * ldp * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(relpos_softmax_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  relpos_softmax_bwd_kernel<<<(unsigned)((rows + warps - 1) / warps), warps * 32, smem, stream>>>(
      (const __nv_bfloat16*)P, dPd, (__nv_bfloat16*)dAC, (__nv_bfloat16*)dBD, H, Tq, Tk, ldp, lddp, lddbd, scale, drop_p, seed,
      rows);
  return (int)cudaGetLastError();
}

SB_API int sb_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n % 8 != 0 || n <= 0) return -1;
  long long n8 = n / 8, blocks = (n8 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  add_bf16_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n8);
  return (int)cudaGetLastError();
}
