// RNNT / TDT loss without the B x T x U x V tensor.
//
// The joint output layer is evaluated chunk by chunk (a few utterances, sized to stay in L2) by the tcgen05 GEMM;
// the kernels here do everything around it:
//   joint_build_h      h[(b,t,u),:] = relu(f[b,t,:] + g[b,u,:])                           (GEMM A operand)
//   joint_lse_gather   per lattice node: log-sum-exp over token logits and over duration logits, and the log-probs the
//                      lattice needs (blank, next label, D durations); the chunk's logits are then dropped
//   transducer_alpha / transducer_beta   forward / backward variables on an anti-diagonal wavefront, one CTA per utterance
//   transducer_node_grads   d(-loglik)/d(log-prob) per node from alpha, beta
//   joint_dlogits      rebuilds softmax from recomputed logits + saved LSE and writes d(logits) in bf16 for the two
//                      gradient GEMMs (dH = dZ W, dW += dZ^T H)
//   joint_reduce_dh    df[b,t] = sum_u dH, dg[b,u] = sum_t dH
// Lattice (reference recursion: nemo/collections/asr/losses/rnnt_pytorch.py:178-247): blank arcs advance d > 0 frames,
// label arcs advance d >= 0 frames, token log-probs are under-normalised by sigma; with D == 0 it is plain RNNT
// (blank advances one frame, labels none).
#include "common.cuh"

namespace {

constexpr float NEG = -1.0e30f;
constexpr int MAXD = 8;

// Arc model of the lattice.  n == 0: plain RNNT.  n > 0, free_label == 0: TDT (every blank AND label arc carries a duration
// d[i] with log-prob lpd[., i]; blank arcs need d > 0).  n > 0, free_label == 1: multi-blank RNNT (reference kernels
// parts/numba/rnnt_loss/utils/cuda_utils/gpu_rnnt_kernel.py:411,570,720): blank symbol i advances d[i] > 0 frames with log-prob
// lpd[., i] (lpb is then all zero), label arcs advance u only and cost lpl.
struct Durations {
  int n;
  int free_label;
  int d[MAXD];
};
constexpr int SB_DURATIONS_FREE_LABEL = 256;   // flag added to the duration count in the C interface

__global__ void joint_build_h_kernel(const __nv_bfloat16* __restrict__ f, const __nv_bfloat16* __restrict__ g,
                                     __nv_bfloat16* __restrict__ h, int b0, int nb, int T, int U1, int Hj, long long f_bs,
                                     long long g_bs, unsigned int drop_thresh, float drop_scale, unsigned long long seed) {
  // rows of the chunk: (b - b0, t, u); f: [B,T,Hj] with batch stride f_bs, g: [B,U1,Hj] with batch stride g_bs.
  // Dropout of the joint network (after the activation, as in the reference's joint_net = [act, Dropout, Linear]): the mask is
  // a hash of (seed, element index in the full [B, T, U1, Hj] lattice), so the backward pass rebuilds the same hidden units
  // when it recomputes a chunk; dropped units are stored as zero, which also zeroes their ReLU derivative.
  const long long rows = (long long)nb * T * U1;
  const int h8 = Hj / 8;
  const long long total = rows * h8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / h8;
    const int c = (int)(i % h8) * 8;
    const int u = (int)(r % U1);
    const int t = (int)((r / U1) % T);
    const int b = b0 + (int)(r / ((long long)U1 * T));
    uint4 rf = *reinterpret_cast<const uint4*>(f + b * f_bs + (long long)t * Hj + c);
    uint4 rg = *reinterpret_cast<const uint4*>(g + b * g_bs + (long long)u * Hj + c);
    const __nv_bfloat162* hf = reinterpret_cast<const __nv_bfloat162*>(&rf);
    const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg);
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = __bfloat1622float2(hf[k]), bb = __bfloat1622float2(hg[k]);
      float v0 = fmaxf(a.x + bb.x, 0.f), v1 = fmaxf(a.y + bb.y, 0.f);
      if (drop_thresh) {
        // eight consecutive elements: groups (base >> 2) and (base >> 2) + 1 of the four-per-hash mask
        const unsigned long long base = ((((unsigned long long)b * T + t) * U1 + u) * (unsigned long long)Hj + c);
        const unsigned int hh = sb_dropout_hash4(seed, (base >> 2) + (k >> 1));
        v0 = sb_dropout_keep_in(hh, (2 * k) & 3, drop_thresh) ? v0 * drop_scale : 0.f;
        v1 = sb_dropout_keep_in(hh, (2 * k + 1) & 3, drop_thresh) ? v1 * drop_scale : 0.f;
      }
      o[k] = __floats2bfloat162_rn(v0, v1);
    }
    *reinterpret_cast<uint4*>(h + r * Hj + c) = *reinterpret_cast<uint4*>(o);
  }
}

// One warp per row.  logits: fp32 [rows, ldz]; token classes [0, V1) with blank = V1-1, durations [V1, V1+D).
// Outputs (indexed by global node id = ((b*T)+t)*U1+u): lse_tok, lse_dur, lp_blank, lp_label, lp_dur[D].
__global__ void joint_lse_gather_kernel(const float* __restrict__ z, int ldz, const long long* __restrict__ targets, int tgt_ld,
                                        float* __restrict__ lse_tok, float* __restrict__ lse_dur, float* __restrict__ lp_blank,
                                        float* __restrict__ lp_label, float* __restrict__ lp_dur, int b0, long long rows, int T,
                                        int U1, int V1, int D, int blank, float sigma) {
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * warps + w;
  if (r >= rows) return;
  const float* zr = z + r * ldz;
  float mx = -3.0e38f;
  for (int v = lane; v < V1; v += 32) mx = fmaxf(mx, zr[v]);
  mx = warp_max(mx);
  float s = 0.f;
  for (int v = lane; v < V1; v += 32) s += __expf(zr[v] - mx);
  s = warp_sum(s);
  const float lse = mx + __logf(s);
  float lsed = 0.f;
  if (D > 0) {
    float md = -3.0e38f;
    for (int d = 0; d < D; ++d) md = fmaxf(md, zr[V1 + d]);
    float sd = 0.f;
    for (int d = 0; d < D; ++d) sd += __expf(zr[V1 + d] - md);
    lsed = md + __logf(sd);
  }
  if (lane == 0) {
    const int u = (int)(r % U1);
    const int b = b0 + (int)(r / ((long long)U1 * T));
    const long long node = (long long)b0 * T * U1 + r;
    lse_tok[node] = lse;
    lp_blank[node] = zr[blank] - lse - sigma;
    float ll = NEG;
    if (u < U1 - 1) {
      const long long y = targets[(long long)b * tgt_ld + u];
      if (y >= 0 && y < V1) ll = zr[y] - lse - sigma;
    }
    lp_label[node] = ll;
    if (D > 0) {
      lse_dur[node] = lsed;
      for (int d = 0; d < D; ++d) lp_dur[node * D + d] = zr[V1 + d] - lsed;
    }
  }
}

// alpha(t,u): one CTA per utterance, thread per u, anti-diagonal wavefront.
__device__ __forceinline__ void transducer_alpha_body(int b, const float* __restrict__ lpb, const float* __restrict__ lpl,
                                                      const float* __restrict__ lpd, const long long* __restrict__ f_len,
                                                      const long long* __restrict__ y_len, float* __restrict__ alpha,
                                                      float* __restrict__ loglik, int T, int U1, const Durations& du) {
  const int u = threadIdx.x;
  const int Tb = (int)f_len[b], Ub = (int)y_len[b];  // valid t < Tb, u <= Ub
  const long long base = (long long)b * T * U1;
  const int D = du.n;
  for (int n = 0; n < Tb + Ub; ++n) {
    const int t = n - u;
    if (u <= Ub && t >= 0 && t < Tb) {
      float a = (t == 0 && u == 0) ? 0.f : NEG;
      if (D == 0) {
        if (t > 0) a = log_add(a, alpha[base + (long long)(t - 1) * U1 + u] + lpb[base + (long long)(t - 1) * U1 + u]);
        if (u > 0) a = log_add(a, alpha[base + (long long)t * U1 + u - 1] + lpl[base + (long long)t * U1 + u - 1]);
      } else {
        for (int i = 0; i < D; ++i) {
          const int d = du.d[i];
          const int tp = t - d;
          if (tp < 0) continue;
          if (d > 0) {
            const long long nd = base + (long long)tp * U1 + u;
            a = log_add(a, alpha[nd] + lpb[nd] + lpd[nd * D + i]);
          }
          if (u > 0 && !du.free_label) {
            const long long nd = base + (long long)tp * U1 + u - 1;
            a = log_add(a, alpha[nd] + lpl[nd] + lpd[nd * D + i]);
          }
        }
        if (du.free_label && u > 0) a = log_add(a, alpha[base + (long long)t * U1 + u - 1] + lpl[base + (long long)t * U1 + u - 1]);
      }
      alpha[base + (long long)t * U1 + u] = a;
    }
    __syncthreads();
  }
  if (u == 0) {
    float ll = NEG;
    if (D == 0) {
      const long long nd = base + (long long)(Tb - 1) * U1 + Ub;
      ll = alpha[nd] + lpb[nd];
    } else {
      for (int i = 0; i < D; ++i) {
        const int d = du.d[i];
        if (d <= 0 || Tb - d < 0) continue;
        const long long nd = base + (long long)(Tb - d) * U1 + Ub;
        ll = log_add(ll, alpha[nd] + lpb[nd] + lpd[nd * D + i]);
      }
    }
    loglik[b] = ll;
  }
}

// beta(t,u) = log-prob of finishing from node (t,u).
__device__ __forceinline__ void transducer_beta_body(int b, const float* __restrict__ lpb, const float* __restrict__ lpl,
                                                     const float* __restrict__ lpd, const long long* __restrict__ f_len,
                                                     const long long* __restrict__ y_len, float* __restrict__ beta, int T, int U1,
                                                     const Durations& du) {
  const int u = threadIdx.x;
  const int Tb = (int)f_len[b], Ub = (int)y_len[b];
  const long long base = (long long)b * T * U1;
  const int D = du.n;
  for (int n = Tb + Ub - 1; n >= 0; --n) {
    const int t = n - u;
    if (u <= Ub && t >= 0 && t < Tb) {
      const long long nd = base + (long long)t * U1 + u;
      float bt = NEG;
      if (D == 0) {
        if (t == Tb - 1 && u == Ub) bt = lpb[nd];
        if (t + 1 < Tb) bt = log_add(bt, lpb[nd] + beta[nd + U1]);
        if (u < Ub) bt = log_add(bt, lpl[nd] + beta[nd + 1]);
      } else {
        for (int i = 0; i < D; ++i) {
          const int d = du.d[i];
          const float ld = lpd[nd * D + i];
          if (d > 0) {
            if (t + d == Tb && u == Ub) bt = log_add(bt, lpb[nd] + ld);
            else if (t + d < Tb) bt = log_add(bt, lpb[nd] + ld + beta[nd + (long long)d * U1]);
          }
          if (!du.free_label && u < Ub && t + d < Tb) bt = log_add(bt, lpl[nd] + ld + beta[nd + (long long)d * U1 + 1]);
        }
        if (du.free_label && u < Ub) bt = log_add(bt, lpl[nd] + beta[nd + 1]);
      }
      beta[nd] = bt;
    }
    __syncthreads();
  }
}

// Both recursions in one launch: blocks [0, B) run the forward variables, blocks [B, 2B) the backward variables.  Each is a
// chain of T + U dependent steps per utterance (latency-bound, one block per utterance), so running them side by side halves
// the time of the pair.  beta == nullptr: forward variables only (grid B).
__global__ void transducer_alpha_beta_kernel(const float* __restrict__ lpb, const float* __restrict__ lpl, const float* __restrict__ lpd,
                                             const long long* __restrict__ f_len, const long long* __restrict__ y_len,
                                             float* __restrict__ alpha, float* __restrict__ beta, float* __restrict__ loglik, int B,
                                             int T, int U1, Durations du) {
  if ((int)blockIdx.x < B) transducer_alpha_body(blockIdx.x, lpb, lpl, lpd, f_len, y_len, alpha, loglik, T, U1, du);
  else transducer_beta_body(blockIdx.x - B, lpb, lpl, lpd, f_len, y_len, beta, T, U1, du);
}

// Per node: gradient of the loss (-loglik * upstream) w.r.t. lp_blank, lp_label, lp_dur[d]; thread per node.
__global__ void transducer_node_grads_kernel(const float* __restrict__ lpb, const float* __restrict__ lpl,
                                             const float* __restrict__ lpd, const float* __restrict__ alpha,
                                             const float* __restrict__ beta, const float* __restrict__ loglik,
                                             const float* __restrict__ upstream, const long long* __restrict__ f_len,
                                             const long long* __restrict__ y_len, float* __restrict__ gb, float* __restrict__ gl,
                                             float* __restrict__ gd, int B, int T, int U1, Durations du, float fastemit) {
  const long long total = (long long)B * T * U1;
  const int D = du.n;
  for (long long nd = (long long)blockIdx.x * blockDim.x + threadIdx.x; nd < total; nd += (long long)gridDim.x * blockDim.x) {
    const int u = (int)(nd % U1);
    const int t = (int)((nd / U1) % T);
    const int b = (int)(nd / ((long long)U1 * T));
    const int Tb = (int)f_len[b], Ub = (int)y_len[b];
    float g_b = 0.f, g_l = 0.f;
    float g_d[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; ++i) g_d[i] = 0.f;
    if (t < Tb && u <= Ub) {
      const float up = -(upstream ? upstream[b] : 1.f);
      const float ll = loglik[b];
      const float a = alpha[nd];
      if (D == 0) {
        float x = NEG;
        if (t == Tb - 1 && u == Ub) x = a + lpb[nd] - ll;
        else if (t + 1 < Tb) x = a + lpb[nd] + beta[nd + U1] - ll;
        g_b = up * __expf(x);
        if (u < Ub) g_l = up * (1.f + fastemit) * __expf(a + lpl[nd] + beta[nd + 1] - ll);
      } else {
        for (int i = 0; i < D; ++i) {
          const int d = du.d[i];
          const float ld = lpd[nd * D + i];
          float occ_b = 0.f, occ_l = 0.f;
          if (d > 0) {
            if (t + d == Tb && u == Ub) occ_b = __expf(a + lpb[nd] + ld - ll);
            else if (t + d < Tb) occ_b = __expf(a + lpb[nd] + ld + beta[nd + (long long)d * U1] - ll);
          }
          if (!du.free_label && u < Ub && t + d < Tb)
            occ_l = (1.f + fastemit) * __expf(a + lpl[nd] + ld + beta[nd + (long long)d * U1 + 1] - ll);
          g_b += up * occ_b;
          g_l += up * occ_l;
          g_d[i] = up * (occ_b + occ_l);
        }
        if (du.free_label && u < Ub) g_l = up * (1.f + fastemit) * __expf(a + lpl[nd] + beta[nd + 1] - ll);
      }
    }
    gb[nd] = g_b;
    gl[nd] = g_l;
    for (int i = 0; i < D; ++i) gd[nd * D + i] = g_d[i];
  }
}

// dZ for a chunk: token part dz_v = [v==blank] g_b + [v==label] g_l - softmax_v (g_b + g_l); duration part likewise.
// One warp per row; dz bf16 [rows, lddz] with padding columns zeroed.
__global__ void joint_dlogits_kernel(const float* __restrict__ z, int ldz, const long long* __restrict__ targets, int tgt_ld,
                                     const float* __restrict__ lse_tok, const float* __restrict__ lse_dur,
                                     const float* __restrict__ gb, const float* __restrict__ gl, const float* __restrict__ gd,
                                     __nv_bfloat16* __restrict__ dz, int lddz, int b0, long long rows, int T, int U1, int V1,
                                     int D, int blank, float clamp) {
  const int warps = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * warps + w;
  if (r >= rows) return;
  const long long node = (long long)b0 * T * U1 + r;
  const int u = (int)(r % U1);
  const int b = b0 + (int)(r / ((long long)U1 * T));
  const float g_b = gb[node], g_l = gl[node];
  const float G = g_b + g_l;
  const float lse = lse_tok[node];
  long long y = -1;
  if (u < U1 - 1) y = targets[(long long)b * tgt_ld + u];
  const float* zr = z + r * ldz;
  __nv_bfloat16* dr = dz + r * lddz;
  float Gd = 0.f, lsed = 0.f;
  if (D > 0) {
    for (int i = 0; i < D; ++i) Gd += gd[node * D + i];
    lsed = lse_dur[node];
  }
  for (int v = lane; v < lddz; v += 32) {
    float o = 0.f;
    if (v < V1) {
      if (G != 0.f) {
        o = -__expf(zr[v] - lse) * G;
        if (v == blank) o += g_b;
        if (v == y) o += g_l;
      }
    } else if (v < V1 + D) {
      o = gd[node * D + (v - V1)] - __expf(zr[v] - lsed) * Gd;
    }
    if (clamp > 0.f) o = fminf(fmaxf(o, -clamp), clamp);
    dr[v] = __float2bfloat16(o);
  }
}

// df[b,t,:] = sum_u dh[(b,t,u),:]; dg[b,u,:] = sum_t dh[(b,t,u),:]   (dh bf16 [nb*T*U1, Hj], outputs fp32).
// One block per output row (a (b,t) pair for df, a (b,u) pair for dg); a thread owns two adjacent channels.
__global__ void joint_reduce_dh_kernel(const __nv_bfloat16* __restrict__ dh, float* __restrict__ df, float* __restrict__ dg,
                                       int b0, int nb, int T, int U1, int Hj) {
  const int c = 2 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= Hj) return;
  const int n_df = nb * T;
  int row = blockIdx.x;
  float s0 = 0.f, s1 = 0.f;
  if (row < n_df) {
    const int bl = row / T, t = row % T;
    const __nv_bfloat16* p = dh + ((long long)bl * T + t) * U1 * Hj + c;
    for (int u = 0; u < U1; ++u) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + (long long)u * Hj));
      s0 += v.x; s1 += v.y;
    }
    float* o = df + ((long long)(b0 + bl) * T + t) * Hj + c;
    o[0] = s0; o[1] = s1;
  } else {
    row -= n_df;
    const int bl = row / U1, u = row % U1;
    const __nv_bfloat16* p = dh + ((long long)bl * T * U1 + u) * Hj + c;
    for (int t = 0; t < T; ++t) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + (long long)t * U1 * Hj));
      s0 += v.x; s1 += v.y;
    }
    float* o = dg + ((long long)(b0 + bl) * U1 + u) * Hj + c;
    o[0] = s0; o[1] = s1;
  }
}

// Same gather as joint_lse_gather but from already materialised logits of the whole batch (non-fused joint path).
Durations make_durations(const int* d, int n) {
  Durations du;
  du.free_label = (n & SB_DURATIONS_FREE_LABEL) ? 1 : 0;
  n &= SB_DURATIONS_FREE_LABEL - 1;
  du.n = n;
  for (int i = 0; i < MAXD; ++i) du.d[i] = i < n ? d[i] : 0;
  return du;
}

}  // namespace

SB_API int sb_joint_build_h(const void* f, const void* g, void* h, int b0, int nb, int T, int U1, int Hj, long long f_bs,
                            long long g_bs, float drop_p, unsigned long long seed, cudaStream_t stream) {
  if (Hj % 8 != 0 || nb <= 0) return -1;
  const long long total = (long long)nb * T * U1 * (Hj / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  joint_build_h_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)f, (const __nv_bfloat16*)g, (__nv_bfloat16*)h, b0, nb,
                                                       T, U1, Hj, f_bs, g_bs, sb_dropout_threshold(drop_p), sb_dropout_scale(drop_p),
                                                       seed);
  return (int)cudaGetLastError();
}

SB_API int sb_joint_lse_gather(const float* z, int ldz, const long long* targets, int tgt_ld, float* lse_tok, float* lse_dur,
                               float* lp_blank, float* lp_label, float* lp_dur, int b0, int nb, int T, int U1, int V1, int D,
                               int blank, float sigma, cudaStream_t stream) {
  const long long rows = (long long)nb * T * U1;
  if (rows <= 0 || D > MAXD) return -1;
  joint_lse_gather_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(z, ldz, targets, tgt_ld, lse_tok, lse_dur, lp_blank,
                                                                         lp_label, lp_dur, b0, rows, T, U1, V1, D, blank, sigma);
  return (int)cudaGetLastError();
}

SB_API int sb_transducer_alpha_beta(const float* lpb, const float* lpl, const float* lpd, const long long* f_len,
                                    const long long* y_len, float* alpha, float* beta, float* loglik, int B, int T, int U1,
                                    const int* durations, int D, cudaStream_t stream) {
  if (U1 > 1024 || (D & (SB_DURATIONS_FREE_LABEL - 1)) > MAXD || B <= 0) return -1;
  const Durations du = make_durations(durations, D);
  const int threads = (U1 + 31) / 32 * 32;
  transducer_alpha_beta_kernel<<<beta ? 2 * B : B, threads, 0, stream>>>(lpb, lpl, lpd, f_len, y_len, alpha, beta, loglik, B, T, U1, du);
  return (int)cudaGetLastError();
}

SB_API int sb_transducer_node_grads(const float* lpb, const float* lpl, const float* lpd, const float* alpha, const float* beta,
                                    const float* loglik, const float* upstream, const long long* f_len, const long long* y_len,
                                    float* gb, float* gl, float* gd, int B, int T, int U1, const int* durations, int D,
                                    float fastemit, cudaStream_t stream) {
  if ((D & (SB_DURATIONS_FREE_LABEL - 1)) > MAXD) return -1;
  const Durations du = make_durations(durations, D);
  const long long total = (long long)B * T * U1;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  transducer_node_grads_kernel<<<(int)blocks, 256, 0, stream>>>(lpb, lpl, lpd, alpha, beta, loglik, upstream, f_len, y_len, gb,
                                                               gl, gd, B, T, U1, du, fastemit);
  return (int)cudaGetLastError();
}

SB_API int sb_joint_dlogits(const float* z, int ldz, const long long* targets, int tgt_ld, const float* lse_tok,
                            const float* lse_dur, const float* gb, const float* gl, const float* gd, void* dz, int lddz, int b0,
                            int nb, int T, int U1, int V1, int D, int blank, float clamp, cudaStream_t stream) {
  const long long rows = (long long)nb * T * U1;
  if (rows <= 0) return -1;
  joint_dlogits_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(z, ldz, targets, tgt_ld, lse_tok, lse_dur, gb, gl, gd,
                                                                      (__nv_bfloat16*)dz, lddz, b0, rows, T, U1, V1, D, blank, clamp);
  return (int)cudaGetLastError();
}

SB_API int sb_joint_reduce_dh(const void* dh, float* df, float* dg, int b0, int nb, int T, int U1, int Hj, cudaStream_t stream) {
  if (Hj % 2 != 0) return -1;
  const int threads = 128;
  dim3 grid(nb * T + nb * U1, (Hj / 2 + threads - 1) / threads);
  joint_reduce_dh_kernel<<<grid, threads, 0, stream>>>((const __nv_bfloat16*)dh, df, dg, b0, nb, T, U1, Hj);
  return (int)cudaGetLastError();
}
