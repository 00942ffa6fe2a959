// Host-side executor for one Conformer layer: a single C call issues every kernel of the layer's forward pass (or of its
// backward pass) on one stream, so the Python interpreter is entered once per layer instead of once per kernel.
//
//   forward : x -> x + 1/2 FF1(LN x) -> + MHSA(LN .) -> + Conv(LN .) -> + 1/2 FF2(LN .) -> LN
//   backward: the same chain in reverse; parameter gradients are ACCUMULATED into fp32 buffers supplied by the caller
//             (the optimizer's flat gradient buffer), activation gradients live in a scratch buffer.
//
// All activations that the backward pass needs are written into one caller-owned "saved" buffer whose layout is computed
// here (sb_conformer_layer_sizes); transient tensors use a second "scratch" buffer that can be shared by all layers.
// Layer structure and parameter roles follow the reference ConformerLayer (conformer_modules.py:36-415: macaron
// feed-forward halves with factor 0.5, Transformer-XL relative-position attention, GLU + depthwise conv + BatchNorm +
// Swish convolution module, final LayerNorm).
#include "common.cuh"
#include "gemm_api.h"
#include "peer_small.h"

#include <cstdint>
#include <cstdio>
#include <cstring>

SB_API int sb_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, int rows,
                            int D, float eps, cudaStream_t stream);
SB_API int sb_layernorm_bwd_res(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx,
                                float* dgamma, float* dbeta, const void* dres, int rows, int D, cudaStream_t stream);
SB_API int sb_add_pos_bias(const void* q, long long q_row_stride, const float* u, const float* v, void* qu, void* qv,
                           long long rows, int HD, cudaStream_t stream);
SB_API int sb_relpos_softmax_fwd(const float* AC, const float* BD, const uint8_t* mask, int mask_bstride, void* P, void* Pd,
                                 int B, int H, int Tq, int Tk, int ldac, int ldbd, int ldp, float scale, float drop_p,
                                 unsigned long long seed, cudaStream_t stream);
SB_API int sb_relpos_softmax_bwd(const void* P, const float* dPd, void* dAC, void* dBD, int B, int H, int Tq, int Tk, int ldp,
                                 int lddp, int lddbd, float scale, float drop_p, unsigned long long seed, cudaStream_t stream);
SB_API int sb_glu_dwconv_fwd(const void* g, const uint8_t* pad, const float* w, const float* bias, void* y, float* stats,
                             int B, int T, int C, int K, int left, cudaStream_t stream);
SB_API int sb_bn_finalize(const float* stats, float count, const float* count_ptr, float* mean_rstd, float* running_mean,
                          float* running_var, int C, float eps, float momentum, int training, cudaStream_t stream);
SB_API int sb_bn_silu_fwd(const void* y, const float* mean_rstd, const float* gamma, const float* beta, void* s, long long rows,
                          int C, cudaStream_t stream);
SB_API int sb_bn_silu_bwd_stats(const void* ds, const void* y, const float* mean_rstd, const float* gamma, const float* beta,
                                float* sums, long long rows, int C, cudaStream_t stream);
SB_API int sb_dwconv_glu_bwd(const void* ds, const void* y, const void* g, const uint8_t* pad, const float* w,
                             const float* mean_rstd, const float* gamma, const float* beta, const float* sums, float count,
                             const float* count_ptr, int training, void* dg, float* dw, float* dbias, int B, int T, int C, int K,
                             int left, cudaStream_t stream);
SB_API int sb_scale_dact_dropout(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                                 float drop_p, unsigned long long seed, cudaStream_t stream);
SB_API int sb_colsum_bf16(const void* x, long long ld, int rows, int N, float* out, cudaStream_t stream);
SB_API int sb_scale_dact_dropout_bias(const void* dy, long long ld_dy, const void* z, void* dz, int rows, int N, int act, float alpha,
                                      float drop_p, unsigned long long seed, float* gb, cudaStream_t stream);

// One linear layer: bf16 weight [out, in], fp32 bias [out] (may be null), fp32 gradient accumulators (null in inference).
struct SbLinearParams {
  const void* w;
  const float* b;
  float* gw;
  float* gb;
};
struct SbNormParams {
  const float* w;
  const float* b;
  float* gw;
  float* gb;
  float eps;
  int pad_;
};

struct SbConformerLayerArgs {
  int B, T, P, d, dff, H, conv_k, conv_left;
  int training;     // BatchNorm uses batch statistics and updates the running ones; dropout sites are active
  float fc_factor;  // 0.5
  float drop_ff, drop_att, drop_out;
  float bn_eps, bn_momentum;
  unsigned long long seeds[7];  // ff1 inner, ff1 out, attention, attention out, conv out, ff2 inner, ff2 out
  // inputs
  const void* x;                    // [B*T, d] bf16
  const void* pos_emb;              // [P, d] bf16, P = 2T-1 relative positions
  const uint8_t* att_mask;          // [1 or B, T, T], non-zero = hidden (may be null)
  int att_mask_bstride;             // T when the mask has a batch dimension, 0 otherwise
  int launches;                     // out: number of kernels launched by the call
  const uint8_t* pad_mask;          // [B, T], non-zero = padding (may be null)
  // parameters
  SbNormParams ln_ff1, ln_att, ln_conv, ln_ff2, ln_out;
  SbLinearParams ff1a, ff1b, qkv, pos, out_proj, pw1, pw2, ff2a, ff2b;
  const float* pos_u;
  const float* pos_v;
  float* g_pos_u;
  float* g_pos_v;
  const float* dw_w;   // [d, conv_k] fp32
  const float* dw_b;
  float* g_dw_w;
  float* g_dw_b;
  const float* bn_w;
  const float* bn_b;
  float* g_bn_w;
  float* g_bn_b;
  float* bn_mean;      // running statistics
  float* bn_var;
  // buffers
  void* out;           // [B*T, d] bf16 (forward output)
  char* saved;
  long long saved_bytes;
  char* scratch;
  long long scratch_bytes;
  // backward only
  const void* dout;    // [B*T, d] bf16
  void* dx;            // [B*T, d] bf16 (null: the input needs no gradient)
  // synchronised BatchNorm (training on several GPUs): the layer's batch statistics are summed over all ranks with the
  // small-vector peer all-reduce; sync_world <= 1 keeps them local.  The forward call uses epoch sync_epoch, and so does the
  // backward call (the caller advances the counter once per call, identically on every rank).
  void* const* sync_buffers;
  long long sync_base_off;
  int sync_rank, sync_world;
  unsigned int sync_epoch;
  int pad2_;
  // profiling (host memory, optional): when prof_ms is set, the call records a CUDA event after every launch, waits for the
  // last one and stores the device time of launch i in prof_ms[i] (milliseconds); at most prof_cap entries
  float* prof_ms;
  int prof_cap;
  int pad_;
};

namespace {

typedef __nv_bfloat16 bf16;

inline long long round8(long long n) { return (n + 7) / 8 * 8; }

struct Bump {
  char* base;
  long long off;
  template <typename T>
  T* take(long long count) {
    const long long o = (off + 255) & ~255LL;
    off = o + count * (long long)sizeof(T);
    return base ? reinterpret_cast<T*>(base + o) : nullptr;
  }
};

struct Saved {
  float *mean[5], *rstd[5];
  bf16 *h1, *pre1, *a1, *res1;
  bf16 *h2, *qkv, *p, *qu, *qv, *Pm, *Pd, *ctx, *res2;
  bf16 *h3, *g, *y, *s, *res3;
  float* mean_rstd;
  float* gcount;   // number of (frame, batch) positions behind the BatchNorm statistics, summed over ranks
  bf16 *h4, *pre2, *a2, *res4;
};

long long layout_saved(const SbConformerLayerArgs& a, char* base, Saved& s) {
  Bump m{base, 0};
  const long long R = (long long)a.B * a.T, d = a.d, F = a.dff, ldp = round8(a.T);
  for (int i = 0; i < 5; ++i) {
    s.mean[i] = m.take<float>(R);
    s.rstd[i] = m.take<float>(R);
  }
  s.h1 = m.take<bf16>(R * d);
  s.pre1 = m.take<bf16>(R * F);
  s.a1 = m.take<bf16>(R * F);
  s.res1 = m.take<bf16>(R * d);
  s.h2 = m.take<bf16>(R * d);
  s.qkv = m.take<bf16>(R * 3 * d);
  s.p = m.take<bf16>((long long)a.P * d);
  s.qu = m.take<bf16>(R * d);
  s.qv = m.take<bf16>(R * d);
  s.Pm = m.take<bf16>((long long)a.B * a.H * a.T * ldp);
  s.Pd = (a.training && a.drop_att > 0.f) ? m.take<bf16>((long long)a.B * a.H * a.T * ldp) : nullptr;
  s.ctx = m.take<bf16>(R * d);
  s.res2 = m.take<bf16>(R * d);
  s.h3 = m.take<bf16>(R * d);
  s.g = m.take<bf16>(R * 2 * d);
  s.y = m.take<bf16>(R * d);
  s.s = m.take<bf16>(R * d);
  s.res3 = m.take<bf16>(R * d);
  s.mean_rstd = m.take<float>(2 * d);
  s.gcount = m.take<float>(1);
  s.h4 = m.take<bf16>(R * d);
  s.pre2 = m.take<bf16>(R * F);
  s.a2 = m.take<bf16>(R * F);
  s.res4 = m.take<bf16>(R * d);
  return (m.off + 255) & ~255LL;
}

struct FwdScratch {
  float *AC, *BD, *stats;
};
long long layout_fwd_scratch(const SbConformerLayerArgs& a, char* base, FwdScratch& s) {
  Bump m{base, 0};
  const long long BHT = (long long)a.B * a.H * a.T;
  s.AC = m.take<float>(BHT * round8(a.T));
  s.BD = m.take<float>(BHT * round8(a.P));
  s.stats = m.take<float>(2 * a.d + 8);
  return (m.off + 255) & ~255LL;
}

struct BwdScratch {
  bf16 *GA, *GB, *dzd, *big, *dh, *dqkv, *dAC, *dBD, *dQu, *dp;
  float *dPd, *su, *sq, *sums;
};
long long layout_bwd_scratch(const SbConformerLayerArgs& a, char* base, BwdScratch& s) {
  Bump m{base, 0};
  const long long R = (long long)a.B * a.T, d = a.d, F = a.dff, BHT = (long long)a.B * a.H * a.T;
  s.GA = m.take<bf16>(R * d);
  s.GB = m.take<bf16>(R * d);
  s.dzd = m.take<bf16>(R * d);
  s.big = m.take<bf16>(R * (F > 2 * d ? F : 2 * d));
  s.dh = m.take<bf16>(R * d);
  s.dqkv = m.take<bf16>(R * 3 * d);
  s.dAC = m.take<bf16>(BHT * round8(a.T));
  s.dBD = m.take<bf16>(BHT * round8(a.P));
  s.dQu = m.take<bf16>(R * d);
  s.dp = m.take<bf16>((long long)a.P * d);
  s.dPd = m.take<float>(BHT * round8(a.T));
  s.su = m.take<float>(2 * d);  // su and sq share one block so that a single memset clears both
  s.sq = s.su + d;
  s.sums = m.take<float>(2 * d);
  return (m.off + 255) & ~255LL;
}

// out[i] += ca * a[i] + cb * b[i]   (b may be null)
__global__ void axpby_accum_kernel(float* __restrict__ out, const float* __restrict__ a, float ca, const float* __restrict__ b,
                                   float cb, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] += ca * a[i] + (b ? cb * b[i] : 0.f);
}

SbGemmArgs gemm_defaults() {
  SbGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.batch0 = g.batch1 = 1;
  g.alpha = 1.f;
  return g;
}

constexpr int kMaxProf = 160;
char g_prof_names[kMaxProf][40];   // names of the launches of the last profiled call (profiling is a single-threaded debug aid)

struct Exec {
  cudaStream_t stream;
  int launches = 0;
  int step = 0;     // index of the call that failed, for the error code
  int rc = 0;
  bool prof = false;
  cudaEvent_t ev[kMaxProf + 1];
  int nev = 0;
  const char* tag = "";   // name of the layer part being issued (profile labels only)
  const char* sub = "";
  void begin(bool profile) {
    prof = profile;
    if (prof && cudaEventCreate(&ev[0]) == cudaSuccess) {
      cudaEventRecord(ev[0], stream);
      nev = 1;
    } else {
      prof = false;
    }
  }
  bool run(int code) {
    ++step;
    ++launches;
    if (prof && nev <= kMaxProf && cudaEventCreate(&ev[nev]) == cudaSuccess) {
      cudaEventRecord(ev[nev], stream);
      snprintf(g_prof_names[nev - 1], sizeof(g_prof_names[0]), "%s%s", tag, sub);
      ++nev;
    }
    sub = "";
    if (code != 0 && rc == 0) rc = code < 0 ? -(step * 1000 - code) : -(step * 1000 + 999);
    return rc == 0;
  }
  void finish(float* out_ms, int cap) {
    if (!prof) return;
    if (nev > 1) cudaEventSynchronize(ev[nev - 1]);
    for (int i = 1; i < nev; ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, ev[i - 1], ev[i]);
      if (out_ms && i - 1 < cap) out_ms[i - 1] = ms;
    }
    for (int i = 0; i < nev; ++i) cudaEventDestroy(ev[i]);
  }
  bool named(const char* label, int code) {
    sub = label;
    return run(code);
  }
  // y[M, N] = epilogue(x[M, K] @ w[N, K]^T)
  bool linear(const bf16* x, long long ldx, const SbLinearParams& p, bf16* y, int M, int N, int K, int act, bf16* pre,
              const bf16* residual, float alpha, float drop_p, unsigned long long seed) {
    SbGemmArgs g = gemm_defaults();
    g.A = x; g.B = p.w; g.M = M; g.N = N; g.K = K; g.lda = ldx; g.ldb = K;
    g.D = y; g.ldd = N;
    g.bias = p.b; g.bias_is_f32 = p.b ? 1 : 0;
    g.residual = residual; g.ldr = residual ? N : 0;
    g.D_pre = pre; g.ldp = pre ? N : 0;
    g.alpha = alpha; g.act = act;
    g.drop_p = drop_p; g.drop_seed = drop_p > 0.f ? seed : 0ull;
    char label[32];
    snprintf(label, sizeof(label), ".linear %dx%d", N, K);
    sub = label;
    return run(sb_gemm_bf16(&g, stream));
  }
  // dx[M, K] = dz[M, N] @ w[N, K];  gw[N, K] += dz^T x;  gb[N] += column sums of dz
  // The input gradient can leave its GEMM already multiplied by the previous activation's derivative and dropout mask:
  // dx = dropout(dz @ w) * act'(dx_pre)  (dx_pre = that activation's saved input, dx_seed = its forward dropout seed).
  bool linear_bwd(const bf16* dz, long long ld_dz, const bf16* x, long long ldx, const SbLinearParams& p, bf16* dx, int M, int N,
                  int K, const bf16* dx_pre = nullptr, int dx_dact = 0, float dx_drop = 0.f, unsigned long long dx_seed = 0,
                  bool bias_grad_done = false) {
    char label[32];
    if (dx) {
      SbGemmArgs g = gemm_defaults();
      g.A = dz; g.B = p.w; g.M = M; g.N = K; g.K = N; g.lda = ld_dz; g.b_mn_major = 1; g.ldb = K;
      g.D = dx; g.ldd = K;
      if (dx_pre) {
        g.aux = dx_pre; g.ldx = K; g.dact = dx_dact;
      }
      g.drop_p = dx_drop; g.drop_seed = dx_drop > 0.f ? dx_seed : 0ull;
      snprintf(label, sizeof(label), ".dgrad %dx%d", N, K);
      sub = label;
      if (!run(sb_gemm_bf16(&g, stream))) return false;
    }
    if (p.gw) {
      SbGemmArgs g = gemm_defaults();
      g.A = dz; g.B = x; g.M = N; g.N = K; g.K = M; g.a_mn_major = 1; g.lda = ld_dz; g.b_mn_major = 1; g.ldb = ldx;
      g.D = p.gw; g.d_is_f32 = 1; g.ldd = K; g.beta = 1.f;
      snprintf(label, sizeof(label), ".wgrad %dx%d", N, K);
      sub = label;
      if (!run(sb_gemm_bf16(&g, stream))) return false;
    }
    if (p.gb && !bias_grad_done) {   // otherwise the kernel that produced dz has already added its column sums to p.gb
      sub = ".bgrad";
      if (!run(sb_colsum_bf16(dz, ld_dz, M, N, p.gb, stream))) return false;
    }
    return true;
  }
  bool ln(const bf16* x, const SbNormParams& p, bf16* y, float* mean, float* rstd, int rows, int D) {
    sub = ".ln";
    return run(sb_layernorm_fwd(x, p.w, p.b, y, mean, rstd, rows, D, p.eps, stream));
  }
  bool ln_bwd(const bf16* dy, const bf16* x, const SbNormParams& p, const float* mean, const float* rstd, bf16* dx,
              const bf16* dres, int rows, int D) {
    sub = ".ln_bwd";
    return run(sb_layernorm_bwd_res(dy, x, p.w, mean, rstd, dx, p.gw, p.gb, dres, rows, D, stream));
  }
  bool zero(void* ptr, size_t bytes) { sub = ".memset"; return run((int)cudaMemsetAsync(ptr, 0, bytes, stream)); }
  bool accum(float* out, const float* a, float ca, const float* b, float cb, int n) {
    axpby_accum_kernel<<<(n + 255) / 256, 256, 0, stream>>>(out, a, ca, b, cb, n);
    sub = ".accum";
    return run((int)cudaGetLastError());
  }
};

bool shapes_ok(const SbConformerLayerArgs& a) {
  if (a.B <= 0 || a.T <= 0 || a.H <= 0 || a.d <= 0 || a.dff <= 0) return false;
  if (a.d % a.H != 0 || (a.d / a.H) % 8 != 0 || a.d % 8 != 0 || a.dff % 8 != 0) return false;
  if (a.P != 2 * a.T - 1) return false;
  if (a.conv_k != 5 && a.conv_k != 9 && a.conv_k != 15) return false;
  return true;
}

}  // namespace

// Bytes of the three work buffers for the problem described by `a` (only the shape / mode fields are read).
SB_API int sb_conformer_layer_sizes(const SbConformerLayerArgs* a, long long* saved, long long* fwd_scratch, long long* bwd_scratch) {
  if (!shapes_ok(*a)) return -1;
  Saved s;
  FwdScratch f;
  BwdScratch b;
  *saved = layout_saved(*a, nullptr, s);
  *fwd_scratch = layout_fwd_scratch(*a, nullptr, f);
  *bwd_scratch = layout_bwd_scratch(*a, nullptr, b);
  return 0;
}

// Label of launch i of the most recent profiled call ("" beyond its end).
SB_API const char* sb_conformer_layer_prof_name(int i) { return (i >= 0 && i < kMaxProf) ? g_prof_names[i] : ""; }

SB_API int sb_conformer_layer_args_size() { return (int)sizeof(SbConformerLayerArgs); }

SB_API int sb_conformer_layer_fwd(SbConformerLayerArgs* a, cudaStream_t stream) {
  if (!shapes_ok(*a)) return -1;
  if (a->sync_world > 1 && 2 * a->d + 1 > SB_SMALL_MAX) return -5;
  Saved s;
  FwdScratch f;
  if (layout_saved(*a, a->saved, s) > a->saved_bytes || !a->saved) return -2;
  if (layout_fwd_scratch(*a, a->scratch, f) > a->scratch_bytes || !a->scratch) return -3;
  Exec e;
  e.stream = stream;
  e.begin(a->prof_ms != nullptr);
  const int B = a->B, T = a->T, P = a->P, d = a->d, F = a->dff, H = a->H, dk = d / H;
  const int R = B * T;
  const bool tr = a->training != 0;
  const float p_ff = tr ? a->drop_ff : 0.f, p_att = tr ? a->drop_att : 0.f, p_out = tr ? a->drop_out : 0.f;
  const bf16* x = (const bf16*)a->x;
  const int ldac = (int)round8(T), ldbd = (int)round8(P), ldp = (int)round8(T);
  const long long HD = d, QS = 3LL * d;
  bool ok = true;
  // ---- feed-forward 1
  e.tag = "ff1";
  ok = ok && e.ln(x, a->ln_ff1, s.h1, s.mean[0], s.rstd[0], R, d);
  ok = ok && e.linear(s.h1, d, a->ff1a, s.a1, R, F, d, /*swish*/ 2, s.pre1, nullptr, 1.f, p_ff, a->seeds[0]);
  ok = ok && e.linear(s.a1, F, a->ff1b, s.res1, R, d, F, 0, nullptr, x, a->fc_factor, p_ff, a->seeds[1]);
  // ---- self-attention
  e.tag = "att";
  ok = ok && e.ln(s.res1, a->ln_att, s.h2, s.mean[1], s.rstd[1], R, d);
  ok = ok && e.linear(s.h2, d, a->qkv, s.qkv, R, 3 * d, d, 0, nullptr, nullptr, 1.f, 0.f, 0);
  ok = ok && e.linear((const bf16*)a->pos_emb, d, a->pos, s.p, P, d, d, 0, nullptr, nullptr, 1.f, 0.f, 0);
  ok = ok && e.named(".add_pos_bias", sb_add_pos_bias(s.qkv, QS, a->pos_u, a->pos_v, s.qu, s.qv, R, d, stream));
  if (ok) {  // AC = (q + u) k^T
    SbGemmArgs g = gemm_defaults();
    g.A = s.qu; g.B = s.qkv + d; g.M = T; g.N = T; g.K = dk; g.lda = HD; g.ldb = QS;
    g.batch0 = H; g.batch1 = B; g.a_bs0 = dk; g.a_bs1 = (long long)T * HD; g.b_bs0 = dk; g.b_bs1 = (long long)T * QS;
    g.D = f.AC; g.d_is_f32 = 1; g.ldd = ldac; g.d_bs0 = (long long)T * ldac; g.d_bs1 = (long long)H * T * ldac;
    ok = e.named(".gemm_AC", sb_gemm_bf16(&g, stream));
  }
  if (ok) {  // BD = (q + v) p^T
    SbGemmArgs g = gemm_defaults();
    g.A = s.qv; g.B = s.p; g.M = T; g.N = P; g.K = dk; g.lda = HD; g.ldb = HD;
    g.batch0 = H; g.batch1 = B; g.a_bs0 = dk; g.a_bs1 = (long long)T * HD; g.b_bs0 = dk; g.b_bs1 = 0;
    g.D = f.BD; g.d_is_f32 = 1; g.ldd = ldbd; g.d_bs0 = (long long)T * ldbd; g.d_bs1 = (long long)H * T * ldbd;
    ok = e.named(".gemm_BD", sb_gemm_bf16(&g, stream));
  }
  ok = ok && e.named(".relpos_softmax_fwd", sb_relpos_softmax_fwd(f.AC, f.BD, a->att_mask, a->att_mask_bstride, s.Pm, p_att > 0.f ? s.Pd : nullptr, B, H, T,
                                         T, ldac, ldbd, ldp, 1.f / sqrtf((float)dk), p_att, a->seeds[2], stream));
  if (ok) {  // ctx = P v
    const bf16* Pu = (p_att > 0.f) ? s.Pd : s.Pm;
    SbGemmArgs g = gemm_defaults();
    g.A = Pu; g.B = s.qkv + 2 * d; g.M = T; g.N = dk; g.K = T; g.lda = ldp; g.b_mn_major = 1; g.ldb = QS;
    g.batch0 = H; g.batch1 = B; g.a_bs0 = (long long)T * ldp; g.a_bs1 = (long long)H * T * ldp; g.b_bs0 = dk;
    g.b_bs1 = (long long)T * QS;
    g.D = s.ctx; g.ldd = HD; g.d_bs0 = dk; g.d_bs1 = (long long)T * HD;
    ok = e.named(".gemm_ctx", sb_gemm_bf16(&g, stream));
  }
  ok = ok && e.linear(s.ctx, d, a->out_proj, s.res2, R, d, d, 0, nullptr, s.res1, 1.f, p_out, a->seeds[3]);
  // ---- convolution module
  e.tag = "conv";
  ok = ok && e.ln(s.res2, a->ln_conv, s.h3, s.mean[2], s.rstd[2], R, d);
  ok = ok && e.linear(s.h3, d, a->pw1, s.g, R, 2 * d, d, 0, nullptr, nullptr, 1.f, 0.f, 0);
  if (tr) ok = ok && e.zero(f.stats, (2 * d + 1) * sizeof(float));
  ok = ok && e.named(".glu_dwconv_fwd", sb_glu_dwconv_fwd(s.g, a->pad_mask, a->dw_w, a->dw_b, s.y, tr ? f.stats : nullptr, B, T, d, a->conv_k,
                                     a->conv_left, stream));
  const bool sync_bn = tr && a->sync_world > 1 && a->sync_buffers;
  if (sync_bn) {  // batch statistics and element count summed over all ranks
    SbPeerSmallArgs sa;
    memset(&sa, 0, sizeof(sa));
    sa.data = f.stats; sa.buffers = a->sync_buffers; sa.base_off = a->sync_base_off; sa.n = 2 * d; sa.has_extra = 1; sa.extra = (float)R;
    sa.rank = a->sync_rank; sa.world = a->sync_world; sa.epoch = a->sync_epoch;
    ok = ok && e.named(".peer_small_allreduce", sb_peer_small_allreduce(&sa, stream));
    ok = ok && e.named(".copy_count", (int)cudaMemcpyAsync(s.gcount, f.stats + 2 * d, sizeof(float), cudaMemcpyDeviceToDevice, stream));
  }
  ok = ok && e.named(".bn_finalize", sb_bn_finalize(tr ? f.stats : nullptr, (float)R, sync_bn ? f.stats + 2 * d : nullptr, s.mean_rstd,
                                                    a->bn_mean, a->bn_var, d, a->bn_eps, a->bn_momentum, tr ? 1 : 0, stream));
  ok = ok && e.named(".bn_silu_fwd", sb_bn_silu_fwd(s.y, s.mean_rstd, a->bn_w, a->bn_b, s.s, R, d, stream));
  ok = ok && e.linear(s.s, d, a->pw2, s.res3, R, d, d, 0, nullptr, s.res2, 1.f, p_out, a->seeds[4]);
  // ---- feed-forward 2 and the output norm
  e.tag = "ff2";
  ok = ok && e.ln(s.res3, a->ln_ff2, s.h4, s.mean[3], s.rstd[3], R, d);
  ok = ok && e.linear(s.h4, d, a->ff2a, s.a2, R, F, d, 2, s.pre2, nullptr, 1.f, p_ff, a->seeds[5]);
  ok = ok && e.linear(s.a2, F, a->ff2b, s.res4, R, d, F, 0, nullptr, s.res3, a->fc_factor, p_ff, a->seeds[6]);
  e.tag = "out";
  ok = ok && e.ln(s.res4, a->ln_out, (bf16*)a->out, s.mean[4], s.rstd[4], R, d);
  e.finish(a->prof_ms, a->prof_cap);
  a->launches = e.launches;
  return e.rc;
}

SB_API int sb_conformer_layer_bwd(SbConformerLayerArgs* a, cudaStream_t stream) {
  if (!shapes_ok(*a)) return -1;
  if (a->sync_world > 1 && 2 * a->d + 1 > SB_SMALL_MAX) return -5;
  Saved s;
  BwdScratch w;
  if (layout_saved(*a, a->saved, s) > a->saved_bytes || !a->saved) return -2;
  if (layout_bwd_scratch(*a, a->scratch, w) > a->scratch_bytes || !a->scratch) return -3;
  if (!a->dout) return -4;
  Exec e;
  e.stream = stream;
  e.begin(a->prof_ms != nullptr);
  const int B = a->B, T = a->T, P = a->P, d = a->d, F = a->dff, H = a->H, dk = d / H;
  const int R = B * T;
  const bool tr = a->training != 0;
  const float p_ff = tr ? a->drop_ff : 0.f, p_att = tr ? a->drop_att : 0.f, p_out = tr ? a->drop_out : 0.f;
  const bf16* x = (const bf16*)a->x;
  const int ldbd = (int)round8(P), ldp = (int)round8(T), lddp = (int)round8(T);
  const long long HD = d, QS = 3LL * d;
  bool ok = true;

  // One macaron feed-forward half: y = res_in + fc * drop(lin_b(drop(swish(lin_a(LN res_in))))).
  // G_in = gradient of y; writes the gradient of res_in into G_out.
  // dz = alpha * dropout-mask * dy * act'(z), with the bias gradient of the linear layer that consumes dz folded into the same pass
  auto dact_bias = [&](const bf16* dy_, long long ld, const bf16* z_, bf16* dz_, int N_, int act_, float alpha_, float p_, unsigned long long sd,
                       float* gb_) {
    if (gb_) return e.named(".scale_dact_dropout_bias", sb_scale_dact_dropout_bias(dy_, ld, z_, dz_, R, N_, act_, alpha_, p_, sd, gb_, stream));
    return e.named(".scale_dact_dropout", sb_scale_dact_dropout(dy_, ld, z_, dz_, R, N_, act_, alpha_, p_, sd, stream));
  };
  auto ff_bwd = [&](const bf16* G_in, bf16* G_out, const bf16* res_in, const bf16* h, const bf16* pre, const bf16* act_out,
                    const SbNormParams& norm, const SbLinearParams& la, const SbLinearParams& lb, const float* mean,
                    const float* rstd, unsigned long long seed_inner, unsigned long long seed_out) {
    bool k = dact_bias(G_in, d, nullptr, w.dzd, d, 0, a->fc_factor, p_ff, seed_out, lb.gb);
    // (folding swish'(pre) and the inner dropout into this dgrad GEMM's epilogue was measured slower: with K = d the GEMM is
    // epilogue-bound and the per-row loads of `pre` more than double it; the separate pass below runs at HBM speed)
    k = k && e.linear_bwd(w.dzd, d, act_out, F, lb, w.big, R, d, F, nullptr, 0, 0.f, 0, true);
    k = k && dact_bias(w.big, F, pre, w.big, F, 2, 1.f, p_ff, seed_inner, la.gb);
    k = k && e.linear_bwd(w.big, F, h, d, la, w.dh, R, F, d, nullptr, 0, 0.f, 0, true);
    k = k && e.ln_bwd(w.dh, res_in, norm, mean, rstd, G_out, G_in, R, d);
    return k;
  };

  // ---- output norm and feed-forward 2
  e.tag = "out";
  ok = ok && e.ln_bwd((const bf16*)a->dout, s.res4, a->ln_out, s.mean[4], s.rstd[4], w.GA, nullptr, R, d);
  e.tag = "ff2";
  ok = ok && ff_bwd(w.GA, w.GB, s.res3, s.h4, s.pre2, s.a2, a->ln_ff2, a->ff2a, a->ff2b, s.mean[3], s.rstd[3], a->seeds[5],
                    a->seeds[6]);
  // ---- convolution module: gradient of res3 is in GB
  e.tag = "conv";
  {
    const bf16* dz = w.GB;
    bool bias_done = false;
    if (p_out > 0.f) {
      ok = ok && dact_bias(w.GB, d, nullptr, w.dzd, d, 0, 1.f, p_out, a->seeds[4], a->pw2.gb);
      dz = w.dzd;
      bias_done = a->pw2.gb != nullptr;
    }
    bf16* ds = w.dh;
    ok = ok && e.linear_bwd(dz, d, s.s, d, a->pw2, ds, R, d, d, nullptr, 0, 0.f, 0, bias_done);
    ok = ok && e.zero(w.sums, 2 * d * sizeof(float));
    ok = ok && e.named(".bn_silu_bwd_stats", sb_bn_silu_bwd_stats(ds, s.y, s.mean_rstd, a->bn_w, a->bn_b, w.sums, R, d, stream));
    bf16* dg = w.big;
    // the affine gradients are the LOCAL sums (the data-parallel gradient exchange adds the ranks up later) ...
    if (a->g_bn_w) ok = ok && e.accum(a->g_bn_w, w.sums + d, 1.f, nullptr, 0.f, d);
    if (a->g_bn_b) ok = ok && e.accum(a->g_bn_b, w.sums, 1.f, nullptr, 0.f, d);
    // ... while the input gradient of a synchronised BatchNorm needs the sums over all ranks
    const bool sync_bn = tr && a->sync_world > 1 && a->sync_buffers;
    if (sync_bn) {
      SbPeerSmallArgs sa;
      memset(&sa, 0, sizeof(sa));
      sa.data = w.sums; sa.buffers = a->sync_buffers; sa.base_off = a->sync_base_off; sa.n = 2 * d;
      sa.rank = a->sync_rank; sa.world = a->sync_world; sa.epoch = a->sync_epoch;
      ok = ok && e.named(".peer_small_allreduce", sb_peer_small_allreduce(&sa, stream));
    }
    ok = ok && e.named(".dwconv_glu_bwd", sb_dwconv_glu_bwd(ds, s.y, s.g, a->pad_mask, a->dw_w, s.mean_rstd, a->bn_w, a->bn_b, w.sums, (float)R,
                                                            sync_bn ? s.gcount : nullptr, tr ? 1 : 0, dg, a->g_dw_w, a->g_dw_b, B, T, d,
                                                            a->conv_k, a->conv_left, stream));
    ok = ok && e.linear_bwd(dg, 2 * d, s.h3, d, a->pw1, w.dzd, R, 2 * d, d);
    ok = ok && e.ln_bwd(w.dzd, s.res2, a->ln_conv, s.mean[2], s.rstd[2], w.GA, w.GB, R, d);
  }
  // ---- self-attention: gradient of res2 is in GA
  e.tag = "att";
  {
    const bf16* dz = w.GA;
    bool bias_done = false;
    if (p_out > 0.f) {
      ok = ok && dact_bias(w.GA, d, nullptr, w.dzd, d, 0, 1.f, p_out, a->seeds[3], a->out_proj.gb);
      dz = w.dzd;
      bias_done = a->out_proj.gb != nullptr;
    }
    bf16* dctx = w.dh;
    ok = ok && e.linear_bwd(dz, d, s.ctx, d, a->out_proj, dctx, R, d, d, nullptr, 0, 0.f, 0, bias_done);
    const bf16* Pu = (p_att > 0.f) ? s.Pd : s.Pm;
    bf16 *dQ = w.dqkv, *dK = w.dqkv + d, *dV = w.dqkv + 2 * d;
    const bf16 *kk = s.qkv + d, *vv = s.qkv + 2 * d;
    const long long pb0 = (long long)T * ldp, pb1 = (long long)H * T * ldp;
    const long long bb0 = (long long)T * ldbd, bb1 = (long long)H * T * ldbd;
    if (ok) {  // dV = P^T dO
      SbGemmArgs g = gemm_defaults();
      g.A = Pu; g.B = dctx; g.M = T; g.N = dk; g.K = T; g.a_mn_major = 1; g.lda = ldp; g.b_mn_major = 1; g.ldb = HD;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = pb0; g.a_bs1 = pb1; g.b_bs0 = dk; g.b_bs1 = (long long)T * HD;
      g.D = dV; g.ldd = QS; g.d_bs0 = dk; g.d_bs1 = (long long)T * QS;
      ok = e.named(".gemm_dV", sb_gemm_bf16(&g, stream));
    }
    if (ok) {  // dP = dO V^T
      SbGemmArgs g = gemm_defaults();
      g.A = dctx; g.B = vv; g.M = T; g.N = T; g.K = dk; g.lda = HD; g.ldb = QS;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = dk; g.a_bs1 = (long long)T * HD; g.b_bs0 = dk; g.b_bs1 = (long long)T * QS;
      g.D = w.dPd; g.d_is_f32 = 1; g.ldd = lddp; g.d_bs0 = (long long)T * lddp; g.d_bs1 = (long long)H * T * lddp;
      ok = e.named(".gemm_dP", sb_gemm_bf16(&g, stream));
    }
    ok = ok && e.named(".relpos_softmax_bwd", sb_relpos_softmax_bwd(s.Pm, w.dPd, w.dAC, w.dBD, B, H, T, T, ldp, lddp, ldbd, 1.f / sqrtf((float)dk), p_att,
                                           a->seeds[2], stream));
    if (ok) {  // dK = dAC^T (q + u)
      SbGemmArgs g = gemm_defaults();
      g.A = w.dAC; g.B = s.qu; g.M = T; g.N = dk; g.K = T; g.a_mn_major = 1; g.lda = ldp; g.b_mn_major = 1; g.ldb = HD;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = pb0; g.a_bs1 = pb1; g.b_bs0 = dk; g.b_bs1 = (long long)T * HD;
      g.D = dK; g.ldd = QS; g.d_bs0 = dk; g.d_bs1 = (long long)T * QS;
      ok = e.named(".gemm_dK", sb_gemm_bf16(&g, stream));
    }
    if (ok) {  // dQu = dAC K
      SbGemmArgs g = gemm_defaults();
      g.A = w.dAC; g.B = kk; g.M = T; g.N = dk; g.K = T; g.lda = ldp; g.b_mn_major = 1; g.ldb = QS;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = pb0; g.a_bs1 = pb1; g.b_bs0 = dk; g.b_bs1 = (long long)T * QS;
      g.D = w.dQu; g.ldd = HD; g.d_bs0 = dk; g.d_bs1 = (long long)T * HD;
      ok = e.named(".gemm_dQu", sb_gemm_bf16(&g, stream));
    }
    if (ok) {  // dQ = dBD p + dQu
      SbGemmArgs g = gemm_defaults();
      g.A = w.dBD; g.B = s.p; g.M = T; g.N = dk; g.K = P; g.lda = ldbd; g.b_mn_major = 1; g.ldb = HD;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = bb0; g.a_bs1 = bb1; g.b_bs0 = dk; g.b_bs1 = 0;
      g.D = dQ; g.ldd = QS; g.d_bs0 = dk; g.d_bs1 = (long long)T * QS;
      g.residual = w.dQu; g.ldr = HD; g.r_bs0 = dk; g.r_bs1 = (long long)T * HD;
      ok = e.named(".gemm_dQ", sb_gemm_bf16(&g, stream));
    }
    if (ok && a->pos.gw) {  // dp = sum over the batch of dBD^T (q + v), then the positional projection's weight gradient
      SbGemmArgs g = gemm_defaults();
      g.A = w.dBD; g.B = s.qv; g.M = P; g.N = dk; g.K = T; g.a_mn_major = 1; g.lda = ldbd; g.b_mn_major = 1; g.ldb = HD;
      g.batch0 = H; g.batch1 = B; g.a_bs0 = bb0; g.a_bs1 = bb1; g.b_bs0 = dk; g.b_bs1 = (long long)T * HD;
      g.D = w.dp; g.ldd = HD; g.d_bs0 = dk; g.d_bs1 = 0; g.fold_batch1 = 1;
      ok = e.named(".gemm_dp", sb_gemm_bf16(&g, stream));
      ok = ok && e.linear_bwd(w.dp, d, (const bf16*)a->pos_emb, d, a->pos, nullptr, P, d, d);
    }
    if (a->g_pos_u || a->g_pos_v) {  // d(u) = colsum(dQu);  d(v) = colsum(dQ) - colsum(dQu)
      ok = ok && e.zero(w.su, 2 * (size_t)d * sizeof(float));
      ok = ok && e.named(".colsum_bf16", sb_colsum_bf16(w.dQu, HD, R, d, w.su, stream));
      ok = ok && e.named(".colsum_bf16", sb_colsum_bf16(dQ, QS, R, d, w.sq, stream));
      if (a->g_pos_u) ok = ok && e.accum(a->g_pos_u, w.su, 1.f, nullptr, 0.f, d);
      if (a->g_pos_v) ok = ok && e.accum(a->g_pos_v, w.sq, 1.f, w.su, -1.f, d);
    }
    ok = ok && e.linear_bwd(w.dqkv, QS, s.h2, d, a->qkv, w.dzd, R, 3 * d, d);
    ok = ok && e.ln_bwd(w.dzd, s.res1, a->ln_att, s.mean[1], s.rstd[1], w.GB, w.GA, R, d);
  }
  // ---- feed-forward 1: gradient of res1 is in GB; the layer input's gradient goes to dx (or to scratch when unused)
  e.tag = "ff1";
  bf16* dx = a->dx ? (bf16*)a->dx : w.GA;
  ok = ok && ff_bwd(w.GB, dx, x, s.h1, s.pre1, s.a1, a->ln_ff1, a->ff1a, a->ff1b, s.mean[0], s.rstd[0], a->seeds[0], a->seeds[1]);
  e.finish(a->prof_ms, a->prof_cap);
  a->launches = e.launches;
  return e.rc;
}
