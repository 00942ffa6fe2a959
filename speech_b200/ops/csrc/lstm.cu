// LSTM prediction network (the transducer decoder): recurrent part of one layer, forward and backward.
//
// The input projection x W_ih^T + b for all time steps and all weight gradients are tcgen05 GEMMs issued by the Python
// wrapper.  The recurrence itself is, per time step, one small tcgen05 GEMM (h_{t-1} W_hh^T accumulated onto the input
// projection with the beta = 1 epilogue, or dgates W_hh in the backward pass) followed by one pointwise kernel.  The host
// entry points issue the whole sequence of launches, so there is no cross-block spinning and nothing can hang.
//
//   forward step t:   gates = xproj[t] + h_{t-1} W_hh^T ; (i,f,g,o) = (sig,sig,tanh,sig) ; c = f c + i g ; h = o tanh(c)
//   backward step t:  (a) dgates from dh, dc and the saved activations;  (b) dh_{t-1} = dgates W_hh
// Gate order follows torch.nn.LSTM (i, f, g, o).  Shapes: xproj (overwritten with the gate pre-activations), acts:
// [U, B, 4H] fp32; c_all: [U, B, H] fp32; y: [U, B, H] bf16; W_hh: bf16 [4H, H].
#include "common.cuh"
#include "gemm_api.h"
#include <string.h>

namespace {

__global__ void lstm_fwd_pointwise_kernel(const float* __restrict__ pre_t, const float* __restrict__ c_prev,
                                          float* __restrict__ acts_t, float* __restrict__ c_t, __nv_bfloat16* __restrict__ y_t,
                                          int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx % H;
  const long long g = (long long)b * 4 * H;
  const float gi = sb_sigmoid(pre_t[g + j]);
  const float gf = sb_sigmoid(pre_t[g + H + j]);
  const float gg = tanhf(pre_t[g + 2 * H + j]);
  const float go = sb_sigmoid(pre_t[g + 3 * H + j]);
  const float cp = c_prev ? c_prev[idx] : 0.f;
  const float c = gf * cp + gi * gg;
  acts_t[g + j] = gi;
  acts_t[g + H + j] = gf;
  acts_t[g + 2 * H + j] = gg;
  acts_t[g + 3 * H + j] = go;
  c_t[idx] = c;
  y_t[idx] = __float2bfloat16(go * tanhf(c));
}

// (a) gate gradients for step t.  dh = upstream dy[t] + recurrent dh_rec; dc carried in dc_rec (updated in place).
__global__ void lstm_bwd_gates_kernel(const __nv_bfloat16* __restrict__ dy_t, const float* __restrict__ dh_rec,
                                      float* __restrict__ dc_rec, const float* __restrict__ acts_t,
                                      const float* __restrict__ c_t, const float* __restrict__ c_prev,
                                      __nv_bfloat16* __restrict__ dgates_t, int B, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * H) return;
  const int b = idx / H, j = idx % H;
  const long long g = (long long)b * 4 * H;
  const float gi = acts_t[g + j], gf = acts_t[g + H + j], gg = acts_t[g + 2 * H + j], go = acts_t[g + 3 * H + j];
  const float tc = tanhf(c_t[idx]);
  const float dh = (dy_t ? __bfloat162float(dy_t[idx]) : 0.f) + dh_rec[idx];
  const float dct = dc_rec[idx] + dh * go * (1.f - tc * tc);
  const float cp = c_prev ? c_prev[idx] : 0.f;
  dc_rec[idx] = dct * gf;
  dgates_t[g + j] = __float2bfloat16(dct * gg * gi * (1.f - gi));
  dgates_t[g + H + j] = __float2bfloat16(dct * cp * gf * (1.f - gf));
  dgates_t[g + 2 * H + j] = __float2bfloat16(dct * gi * (1.f - gg * gg));
  dgates_t[g + 3 * H + j] = __float2bfloat16(dh * tc * go * (1.f - go));
}

SbGemmArgs small_gemm(const void* A, const void* Bm, void* D, int M, int N, int K, int b_mn, long long ldb, float beta) {
  SbGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.A = A; a.B = Bm; a.M = M; a.N = N; a.K = K;
  a.a_mn_major = 0; a.b_mn_major = b_mn;
  a.lda = K; a.ldb = ldb;
  a.batch0 = 1; a.batch1 = 1;
  a.D = D; a.d_is_f32 = 1; a.ldd = N;
  a.alpha = 1.f; a.beta = beta;
  a.tile_n = 128;
  a.ksplit = -1;  // the recurrence GEMMs are tiny; never slice K
  return a;
}

}  // namespace

// Runs all U forward steps of one layer.  xproj [U,B,4H] holds x W_ih^T + b on entry and the gate pre-activations on exit.
// h0 (bf16 [B,H]) / c0 (fp32 [B,H]) may be null (zeros).  Outputs: acts [U,B,4H], c_all [U,B,H] (fp32), y [U,B,H] (bf16).
SB_API int sb_lstm_forward(float* xproj, const void* h0_bf16, const float* c0, const void* whh, float* acts, float* c_all, void* y,
                           int U, int B, int H, cudaStream_t stream) {
  if (H % 8 != 0 || U <= 0 || B <= 0) return -1;
  const int n = B * H;
  __nv_bfloat16* yb = (__nv_bfloat16*)y;
  for (int t = 0; t < U; ++t) {
    float* pre = xproj + (long long)t * B * 4 * H;
    const void* hp = t == 0 ? h0_bf16 : (const void*)(yb + (long long)(t - 1) * n);
    if (hp) {
      SbGemmArgs g = small_gemm(hp, whh, pre, B, 4 * H, H, 0, H, 1.f);
      int rc = sb_gemm_bf16(&g, stream);
      if (rc) return rc;
    }
    const float* cp = t == 0 ? c0 : c_all + (long long)(t - 1) * n;
    lstm_fwd_pointwise_kernel<<<(n + 255) / 256, 256, 0, stream>>>(pre, cp, acts + (long long)t * B * 4 * H,
                                                                  c_all + (long long)t * n, yb + (long long)t * n, B, H);
  }
  return (int)cudaGetLastError();
}

// Runs all U backward steps of one layer.  dy: bf16 [U,B,H] upstream gradient of the outputs (may be null);
// dh_rec / dc_rec: fp32 [B,H] holding the gradient flowing into the final state on entry (zeros or d(h_n), d(c_n)) and the
// gradient w.r.t. (h0, c0) on exit.  Output dgates bf16 [U,B,4H].
SB_API int sb_lstm_backward(const void* dy, float* dh_rec, float* dc_rec, const float* acts, const float* c_all, const float* c0,
                            const void* whh, void* dgates_bf16, int U, int B, int H, cudaStream_t stream) {
  if (H % 8 != 0 || U <= 0 || B <= 0) return -1;
  const int n = B * H;
  __nv_bfloat16* dg = (__nv_bfloat16*)dgates_bf16;
  for (int t = U - 1; t >= 0; --t) {
    const float* cp = t == 0 ? c0 : c_all + (long long)(t - 1) * n;
    lstm_bwd_gates_kernel<<<(n + 255) / 256, 256, 0, stream>>>(
        dy ? (const __nv_bfloat16*)dy + (long long)t * n : nullptr, dh_rec, dc_rec, acts + (long long)t * B * 4 * H,
        c_all + (long long)t * n, cp, dg + (long long)t * B * 4 * H, B, H);
    // dh_rec[B,H] = dgates_t[B,4H] W_hh[4H,H]   (W_hh read as the MN-major B operand)
    SbGemmArgs g = small_gemm(dg + (long long)t * B * 4 * H, whh, dh_rec, B, H, 4 * H, 1, H, 0.f);
    int rc = sb_gemm_bf16(&g, stream);
    if (rc) return rc;
  }
  return (int)cudaGetLastError();
}
