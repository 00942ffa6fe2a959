// LSTM prediction network (the transducer decoder): recurrent part of one layer, forward and backward.
//
// The input projection x W_ih^T + b for all time steps and all weight gradients are tcgen05 GEMMs issued by the host
// wrapper; the kernels here are the strictly sequential part.  One launch per time step (the host entry point issues
// the whole sequence), so there is no cross-block spinning and nothing can hang.
//
//   forward step t:   gates = xproj[t] + h_{t-1} W_hh^T ; (i,f,g,o) = (sig,sig,tanh,sig) ; c = f c + i g ; h = o tanh(c)
//   backward step t:  (a) dgates from dh, dc and the saved activations;  (b) dh_{t-1} = dgates W_hh
// Gate order follows torch.nn.LSTM (i, f, g, o).  Shapes: xproj, acts: [U, B, 4H] fp32; c_all, h_all: [U, B, H];
// W_hh: bf16 [4H, H].
#include "common.cuh"

namespace {

constexpr int JB = 8;  // hidden units per block in the forward step

// Block = (32 batch lanes) x (JB hidden units).  Thread (b, jl) accumulates the 4 gate pre-activations of unit j.
__global__ void lstm_fwd_step_kernel(const float* __restrict__ xproj_t, const float* __restrict__ h_prev,
                                     const float* __restrict__ c_prev, const __nv_bfloat16* __restrict__ whh,
                                     float* __restrict__ acts_t, float* __restrict__ c_t, float* __restrict__ h_t,
                                     __nv_bfloat16* __restrict__ y_t, int B, int H) {
  extern __shared__ float hT[];  // [H][32] : h_prev transposed, batch padded to 32
  const int b = threadIdx.x & 31;
  const int jl = threadIdx.x >> 5;
  const int j = blockIdx.x * JB + jl;
  for (int bstart = 0; bstart < B; bstart += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < H * 32; i += blockDim.x) {
      const int k = i >> 5, bb = i & 31;
      hT[i] = (bstart + bb < B && h_prev) ? h_prev[(long long)(bstart + bb) * H + k] : 0.f;
    }
    __syncthreads();
    const int bg = bstart + b;
    if (j < H) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < H; k += 8) {
        float hv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) hv[u] = hT[(k + u) * 32 + b];
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          uint4 raw = *reinterpret_cast<const uint4*>(whh + ((long long)gi * H + j) * H + k);
          const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float2 wf = __bfloat1622float2(w2[u]);
            acc[gi] += wf.x * hv[2 * u] + wf.y * hv[2 * u + 1];
          }
        }
      }
      if (bg < B) {
        const long long gbase = (long long)bg * 4 * H;
        const float gi_ = sb_sigmoid(acc[0] + xproj_t[gbase + j]);
        const float gf_ = sb_sigmoid(acc[1] + xproj_t[gbase + H + j]);
        const float gg_ = tanhf(acc[2] + xproj_t[gbase + 2 * H + j]);
        const float go_ = sb_sigmoid(acc[3] + xproj_t[gbase + 3 * H + j]);
        const float cp = c_prev ? c_prev[(long long)bg * H + j] : 0.f;
        const float c = gf_ * cp + gi_ * gg_;
        const float h = go_ * tanhf(c);
        acts_t[gbase + j] = gi_;
        acts_t[gbase + H + j] = gf_;
        acts_t[gbase + 2 * H + j] = gg_;
        acts_t[gbase + 3 * H + j] = go_;
        c_t[(long long)bg * H + j] = c;
        h_t[(long long)bg * H + j] = h;
        y_t[(long long)bg * H + j] = __float2bfloat16(h);
      }
    }
  }
}

// (a) gate gradients for step t.  dh_in = upstream dy[t] (+ recurrent dh carried in dh_rec), dc carried in dc_rec.
__global__ void lstm_bwd_gates_kernel(const __nv_bfloat16* __restrict__ dy_t, const float* __restrict__ dh_rec,
                                      float* __restrict__ dc_rec, const float* __restrict__ acts_t,
                                      const float* __restrict__ c_t, const float* __restrict__ c_prev,
                                      float* __restrict__ dgates_t, __nv_bfloat16* __restrict__ dgates_bf16_t, int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx % H;
  const long long gbase = (long long)b * 4 * H;
  const float gi_ = acts_t[gbase + j], gf_ = acts_t[gbase + H + j], gg_ = acts_t[gbase + 2 * H + j], go_ = acts_t[gbase + 3 * H + j];
  const float tc = tanhf(c_t[idx]);
  const float dh = (dy_t ? __bfloat162float(dy_t[idx]) : 0.f) + (dh_rec ? dh_rec[idx] : 0.f);
  const float dct = dc_rec[idx] + dh * go_ * (1.f - tc * tc);
  const float cp = c_prev ? c_prev[idx] : 0.f;
  const float di = dct * gg_ * gi_ * (1.f - gi_);
  const float df = dct * cp * gf_ * (1.f - gf_);
  const float dg = dct * gi_ * (1.f - gg_ * gg_);
  const float dout = dh * tc * go_ * (1.f - go_);
  dc_rec[idx] = dct * gf_;
  dgates_t[gbase + j] = di;
  dgates_t[gbase + H + j] = df;
  dgates_t[gbase + 2 * H + j] = dg;
  dgates_t[gbase + 3 * H + j] = dout;
  dgates_bf16_t[gbase + j] = __float2bfloat16(di);
  dgates_bf16_t[gbase + H + j] = __float2bfloat16(df);
  dgates_bf16_t[gbase + 2 * H + j] = __float2bfloat16(dg);
  dgates_bf16_t[gbase + 3 * H + j] = __float2bfloat16(dout);
}

// (b) dh_rec[b, k] = sum_r dgates[b, r] * W_hh[r, k].  Block covers 128 columns k; dgates rows staged in shared memory.
__global__ void lstm_bwd_dh_kernel(const float* __restrict__ dgates_t, const __nv_bfloat16* __restrict__ whh,
                                   float* __restrict__ dh_rec, int B, int H) {
  extern __shared__ float dg[];  // [BB][4H] for a group of BB batch rows
  constexpr int BB = 4;
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  const int R = 4 * H;
  for (int b0 = blockIdx.y * BB; b0 < B; b0 += gridDim.y * BB) {
    __syncthreads();
    for (int i = threadIdx.x; i < BB * R; i += blockDim.x) {
      const int bb = i / R, r = i % R;
      dg[i] = (b0 + bb < B) ? dgates_t[(long long)(b0 + bb) * R + r] : 0.f;
    }
    __syncthreads();
    if (k < H) {
      float acc[BB] = {0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < R; ++r) {
        const float w = __bfloat162float(whh[(long long)r * H + k]);
#pragma unroll
        for (int bb = 0; bb < BB; ++bb) acc[bb] += w * dg[bb * R + r];
      }
#pragma unroll
      for (int bb = 0; bb < BB; ++bb)
        if (b0 + bb < B) dh_rec[(long long)(b0 + bb) * H + k] = acc[bb];
    }
  }
}

}  // namespace

// Runs all U forward steps of one layer.  h0/c0 may be null (zeros).  Outputs: acts [U,B,4H], c_all [U,B,H], h_all [U,B,H]
// (fp32) and y [U,B,H] (bf16).
SB_API int sb_lstm_forward(const float* xproj, const float* h0, const float* c0, const void* whh, float* acts, float* c_all,
                           float* h_all, void* y, int U, int B, int H, cudaStream_t stream) {
  if (H % 8 != 0 || U <= 0 || B <= 0) return -1;
  const size_t smem = (size_t)H * 32 * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(lstm_fwd_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int blocks = (H + JB - 1) / JB;
  for (int t = 0; t < U; ++t) {
    const float* hp = t == 0 ? h0 : h_all + (long long)(t - 1) * B * H;
    const float* cp = t == 0 ? c0 : c_all + (long long)(t - 1) * B * H;
    lstm_fwd_step_kernel<<<blocks, 32 * JB, smem, stream>>>(xproj + (long long)t * B * 4 * H, hp, cp, (const __nv_bfloat16*)whh,
                                                           acts + (long long)t * B * 4 * H, c_all + (long long)t * B * H,
                                                           h_all + (long long)t * B * H,
                                                           (__nv_bfloat16*)y + (long long)t * B * H, B, H);
  }
  return (int)cudaGetLastError();
}

// Runs all U backward steps of one layer.  dy: bf16 [U,B,H] upstream gradient of the outputs (may be null);
// dh_rec / dc_rec: fp32 [B,H] scratch holding the gradient flowing into the final state on entry (zeros or d(h_n), d(c_n))
// and the gradient w.r.t. (h0, c0) on exit.  Outputs dgates fp32 + bf16 [U,B,4H].
SB_API int sb_lstm_backward(const void* dy, float* dh_rec, float* dc_rec, const float* acts, const float* c_all, const float* c0,
                            const void* whh, float* dgates, void* dgates_bf16, int U, int B, int H, cudaStream_t stream) {
  if (U <= 0 || B <= 0) return -1;
  const size_t smem = (size_t)4 * 4 * H * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(lstm_bwd_dh_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int n = B * H;
  dim3 grid_dh((H + 127) / 128, (B + 3) / 4);
  for (int t = U - 1; t >= 0; --t) {
    const float* cp = t == 0 ? c0 : c_all + (long long)(t - 1) * B * H;
    lstm_bwd_gates_kernel<<<(n + 255) / 256, 256, 0, stream>>>(
        dy ? (const __nv_bfloat16*)dy + (long long)t * B * H : nullptr, dh_rec, dc_rec, acts + (long long)t * B * 4 * H,
        c_all + (long long)t * B * H, cp, dgates + (long long)t * B * 4 * H,
        (__nv_bfloat16*)dgates_bf16 + (long long)t * B * 4 * H, B, H);
    lstm_bwd_dh_kernel<<<grid_dh, 128, smem, stream>>>(dgates + (long long)t * B * 4 * H, (const __nv_bfloat16*)whh, dh_rec, B, H);
  }
  return (int)cudaGetLastError();
}
