// CTC loss, forward and backward, one CTA per utterance.
//
// Extended label sequence l' = (blank, y_1, blank, ..., y_L, blank), S = 2L+1 states, one thread per state, a
// __syncthreads per frame.  Inputs are log-probabilities [B, T, V] (fp32, row stride ldv); the gradient is taken with
// respect to those log-probabilities (the convention of torch.nn.functional.ctc_loss, which the reference wraps:
// nemo/collections/asr/losses/ctc.py:24-80):
//     dL/dlp[t,v] = -sum_{s : l'_s = v} exp(alpha_t(s) + beta_t(s) - lp[t,v] - loglik)
// with alpha and beta both including the emission at t.  Utterances whose likelihood is zero give loss 0 and zero
// gradient when zero_infinity is set.
#include "common.cuh"

namespace {

constexpr float NEGINF = -1.0e30f;

__device__ __forceinline__ int ext_label(const long long* tgt, int s, int blank) { return (s & 1) ? (int)tgt[s >> 1] : blank; }

__global__ void ctc_alpha_beta_kernel(const float* __restrict__ lp, long long ldv, long long lp_bs,
                                      const long long* __restrict__ targets, int tgt_ld,
                                      const long long* __restrict__ in_len, const long long* __restrict__ tgt_len,
                                      float* __restrict__ alpha, float* __restrict__ beta, float* __restrict__ nll, int T, int Smax,
                                      int blank, int zero_infinity) {
  const int b = blockIdx.x;
  const int s = threadIdx.x;
  const int Tb = (int)in_len[b];
  const int L = (int)tgt_len[b];
  const int S = 2 * L + 1;
  const long long* tgt = targets + (long long)b * tgt_ld;
  const float* lpb = lp + (long long)b * lp_bs;
  float* al = alpha + (long long)b * T * Smax;
  float* be = beta + (long long)b * T * Smax;
  const bool on = s < S;
  const int lab = on ? ext_label(tgt, s, blank) : blank;
  const bool skip_ok = on && s >= 2 && (s & 1) && lab != ext_label(tgt, s - 2, blank);
  // ---- alpha
  for (int t = 0; t < Tb; ++t) {
    if (on) {
      float a;
      if (t == 0) {
        a = (s <= 1) ? lpb[lab] : NEGINF;
      } else {
        const float* prev = al + (long long)(t - 1) * Smax;
        a = prev[s];
        if (s >= 1) a = log_add(a, prev[s - 1]);
        if (skip_ok) a = log_add(a, prev[s - 2]);
        a = a > -1.0e29f ? a + lpb[(long long)t * ldv + lab] : NEGINF;
      }
      al[(long long)t * Smax + s] = a;
    }
    __syncthreads();
  }
  // ---- beta
  const bool skip_fwd = on && (s + 2 < S) && (s & 1) && lab != ext_label(tgt, s + 2, blank);
  for (int t = Tb - 1; t >= 0; --t) {
    if (on) {
      float v;
      if (t == Tb - 1) {
        v = (s >= S - 2) ? lpb[(long long)t * ldv + lab] : NEGINF;
      } else {
        const float* nxt = be + (long long)(t + 1) * Smax;
        v = nxt[s];
        if (s + 1 < S) v = log_add(v, nxt[s + 1]);
        if (skip_fwd) v = log_add(v, nxt[s + 2]);
        v = v > -1.0e29f ? v + lpb[(long long)t * ldv + lab] : NEGINF;
      }
      be[(long long)t * Smax + s] = v;
    }
    __syncthreads();
  }
  if (s == 0) {
    float ll = NEGINF;
    if (Tb > 0) {
      ll = al[(long long)(Tb - 1) * Smax + S - 1];
      if (S > 1) ll = log_add(ll, al[(long long)(Tb - 1) * Smax + S - 2]);
    }
    float loss = -ll;
    if (ll < -1.0e29f) loss = zero_infinity ? 0.f : INFINITY;
    nll[b] = loss;
  }
}

// grad[b,t,v] (pre-zeroed) -= upstream[b] * exp(alpha+beta-lp-ll) summed over the states that emit v.
__global__ void ctc_grad_kernel(const float* __restrict__ lp, long long ldv, long long lp_bs, const long long* __restrict__ targets,
                                int tgt_ld, const long long* __restrict__ in_len, const long long* __restrict__ tgt_len,
                                const float* __restrict__ alpha, const float* __restrict__ beta, const float* __restrict__ nll,
                                const float* __restrict__ upstream, float* __restrict__ grad, long long g_ldv, long long g_bs,
                                int T, int Smax, int blank) {
  const int b = blockIdx.y;
  const int Tb = (int)in_len[b];
  const int S = 2 * (int)tgt_len[b] + 1;
  const float loss = nll[b];
  if (!(loss > 0.f) || isinf(loss)) return;  // zero-likelihood (or empty) utterances contribute nothing
  const float up = upstream ? upstream[b] : 1.f;
  const long long* tgt = targets + (long long)b * tgt_ld;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)Tb * S; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / S), s = (int)(i % S);
    const int lab = ext_label(tgt, s, blank);
    const float a = alpha[((long long)b * T + t) * Smax + s], be = beta[((long long)b * T + t) * Smax + s];
    if (a < -1.0e29f || be < -1.0e29f) continue;
    const float l = lp[(long long)b * lp_bs + (long long)t * ldv + lab];
    atomicAdd(&grad[(long long)b * g_bs + (long long)t * g_ldv + lab], -up * __expf(a + be - l + loss));
  }
}

}  // namespace

SB_API int sb_ctc_forward(const float* lp, long long ldv, long long lp_bs, const long long* targets, int tgt_ld,
                          const long long* in_len, const long long* tgt_len, float* alpha, float* beta, float* nll, int B, int T,
                          int Smax, int blank, int zero_infinity, cudaStream_t stream) {
  if (Smax > 1024 || B <= 0 || T <= 0) return -1;
  const int threads = (Smax + 31) / 32 * 32;
  ctc_alpha_beta_kernel<<<B, threads, 0, stream>>>(lp, ldv, lp_bs, targets, tgt_ld, in_len, tgt_len, alpha, beta, nll, T, Smax, blank,
                                                  zero_infinity);
  return (int)cudaGetLastError();
}

SB_API int sb_ctc_backward(const float* lp, long long ldv, long long lp_bs, const long long* targets, int tgt_ld,
                           const long long* in_len, const long long* tgt_len, const float* alpha, const float* beta, const float* nll,
                           const float* upstream, float* grad, long long g_ldv, long long g_bs, int B, int T, int Smax, int blank,
                           cudaStream_t stream) {
  int bx = (int)(((long long)T * Smax + 255) / 256);
  if (bx > 64) bx = 64;
  dim3 grid(bx, B);
  ctc_grad_kernel<<<grid, 256, 0, stream>>>(lp, ldv, lp_bs, targets, tgt_ld, in_len, tgt_len, alpha, beta, nll, upstream, grad, g_ldv,
                                           g_bs, T, Smax, blank);
  return (int)cudaGetLastError();
}
