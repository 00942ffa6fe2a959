// Persistent bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with TMEM accumulators -> fused epilogue.
//
//   D[b] = epilogue( alpha * A[b] (M x K) * B[b]^T (K x N) )          fp32 accumulation
//
// Each operand may be stored K-major ("row" of the logical matrix is contiguous in K: A as [M,K], B as [N,K],
// i.e. nn.Linear's weight) or MN-major (stored transposed: A as [K,M], B as [K,N]); the four combinations cover
// forward (x W^T), input-gradient (dy W) and weight-gradient (dy^T x) GEMMs without any transposition pass.
// Batched problems (attention scores per (batch, head)) use two batch indices with arbitrary strides.
//
// CTA layout (320 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and issues the MMAs,
// warps 2-9 run the epilogue (two warps per 32-lane TMEM quarter, each draining half of the columns).  The CTA is
// persistent over output tiles; two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the MMAs
// of tile i+1.  Shared-memory stages hold a 128x64 A tile and a BNx64 B tile (BN = 128 or 256) in the 128-byte
// swizzled layout that both TMA and the tcgen05 shared-memory descriptors understand.
//
// Epilogue (all optional, applied in this order): v = acc + bias[n]; store pre-activation (bf16);
// v = alpha * act(v); v *= act'(aux[m,n]); v += residual[m,n]; v += beta * D_old[m,n] (fp32 D only); store D as bf16 or fp32.
//
// Every mbarrier wait is bounded (see common.cuh): on a timeout the kernel records a status code and all roles
// fall through to the common exit where tensor memory is released.
#include "gemm_kernel.cuh"

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// Operand as a 4-D tensor (inner, outer, batch0, batch1) with a {64, box_outer, 1, 1} box.
int make_operand_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long ld, int batch0,
                     int batch1, long long bs0, long long bs1, int box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -100;
  if ((((uintptr_t)ptr) & 15) != 0 || (ld * 2) % 16 != 0) return -101;
  if ((batch0 > 1 && (bs0 * 2) % 16 != 0) || (batch1 > 1 && (bs1 * 2) % 16 != 0)) return -102;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch0, (cuuint64_t)batch1};
  const cuuint64_t safe = (cuuint64_t)ld * 2;
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, batch0 > 1 ? (cuuint64_t)bs0 * 2 : safe, batch1 > 1 ? (cuuint64_t)bs1 * 2 : safe};
  cuuint32_t box[4] = {64, (cuuint32_t)box_outer, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(200 + (int)r);
}

// Output (D or D_pre) as a 4-D tensor (N, M, batch0, batch1) with a {32, 32, 1, 1} box: 64-byte swizzle for bf16 rows of 64
// bytes, 128-byte swizzle for fp32 rows of 128 bytes.  Returns 0, or non-zero when the layout does not meet the alignment rules
// of a tensor map (the epilogue then stores by lanes).
int make_out_map(CUtensorMap* map, const void* ptr, bool f32, long long n, long long m, long long ld, int batch0, int batch1,
                 long long bs0, long long bs1) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -100;
  const long long es = f32 ? 4 : 2;
  if ((((uintptr_t)ptr) & 15) != 0 || (ld * es) % 16 != 0 || ld < n) return -101;
  if ((batch0 > 1 && ((bs0 * es) % 16 != 0 || bs0 <= 0)) || (batch1 > 1 && ((bs1 * es) % 16 != 0 || bs1 <= 0))) return -102;
  cuuint64_t dims[4] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)batch0, (cuuint64_t)batch1};
  const cuuint64_t safe = (cuuint64_t)(ld * es);
  cuuint64_t strides[3] = {(cuuint64_t)(ld * es), batch0 > 1 ? (cuuint64_t)(bs0 * es) : safe, batch1 > 1 ? (cuuint64_t)(bs1 * es) : safe};
  cuuint32_t box[4] = {32, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(200 + (int)r);
}

#ifdef SB_GEMM_DIAG
long long* g_trace = nullptr;
#endif

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------------
// Small-M GEMMs with a bf16 output (inference with a few hundred tokens: streaming steps, decoding): the output has a handful of
// tiles, so a handful of blocks would each walk the whole K extent with at most NUM_STAGES loads in flight, and the kernel
// time is (K blocks / stages) x memory latency.  Splitting K over more blocks keeps every block's slice inside its pipeline
// depth; the partial sums meet in an fp32 workspace that the caller provides (vector reductions, L2-resident) and a small kernel
// applies the epilogue.  Without a workspace the GEMM runs as one pass.
__global__ void splitk_finish_kernel(const float* __restrict__ ws, int M, int N, __nv_bfloat16* __restrict__ D, long long ldd,
                                     const float* __restrict__ bias_f32, const __nv_bfloat16* __restrict__ bias_bf16,
                                     __nv_bfloat16* __restrict__ D_pre, long long ldp, const __nv_bfloat16* __restrict__ residual,
                                     long long ldr, float alpha, int act) {
  const int n4 = N >> 2;
  const long long total = (long long)M * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / n4), c = (int)(i % n4) * 4;
    const float4 w = __ldcg(reinterpret_cast<const float4*>(ws + (long long)m * N + c));
    float v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (bias_f32) v[j] += __ldg(bias_f32 + c + j);
      else if (bias_bf16) v[j] += __bfloat162float(bias_bf16[c + j]);
    }
    if (D_pre) {
#pragma unroll
      for (int j = 0; j < 4; ++j) D_pre[(long long)m * ldp + c + j] = __float2bfloat16(v[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (act == 2) v[j] = sb_swish(v[j]);
      else if (act == 1) v[j] = fmaxf(v[j], 0.f);
      else if (act == 3) v[j] = sb_gelu(v[j]);
      v[j] *= alpha;
      if (residual) v[j] += __bfloat162float(residual[(long long)m * ldr + c + j]);
      D[(long long)m * ldd + c + j] = __float2bfloat16(v[j]);
    }
  }
}

SB_API int sb_gemm_bf16(const SbGemmArgs* a, cudaStream_t stream);
#ifdef SB_GEMM_DIAG
// diagnostic builds: device buffer of 8 x 256 int64 that block 0 of the following GEMMs fills with clock64() stamps (null = off)
SB_API void sb_gemm_set_trace(long long* buf) { g_trace = buf; }
#endif

// 1 = handled (rc in *out_rc), 0 = not applicable
static int small_m_splitk(const SbGemmArgs* a, cudaStream_t stream, int* out_rc) {
  static const bool enabled = [] { const char* e = getenv("SPEECH_B200_SMALL_M_SPLITK"); return !(e && e[0] == '0'); }();
  if (!enabled || a->d_is_f32 || a->beta != 0.f || a->batch0 != 1 || a->batch1 != 1 || a->fold_batch1 || a->aux || a->drop_p > 0.f ||
      a->peer_D || a->peer_A || a->sig_flags || a->ksplit != 0 || a->a_mn_major || a->M > 1024 || (a->N & 3) || a->pair == 1)
    return 0;
  const int num_kb = (a->K + BLOCK_K - 1) / BLOCK_K;
  const long long tiles = (long long)((a->M + BLOCK_M - 1) / BLOCK_M) * ((a->N + 127) / 128);
  const int sms = sb_num_sms() - sb_reserved_sms();
  if (num_kb < 12 || tiles * 4 > sms || !a->splitk_ws || (long long)a->M * a->N * 4 > a->splitk_ws_bytes) return 0;
  int split = (int)(sms / tiles);
  if (split > num_kb / 4) split = num_kb / 4;     // a slice keeps at least four K blocks
  if (split > 16) split = 16;
  if (split < 2) return 0;
  float* ws = (float*)a->splitk_ws;   // the caller's scratch (stream-ordered allocation), M x N fp32
  cudaError_t ce = cudaMemsetAsync(ws, 0, (size_t)a->M * a->N * 4, stream);
  if (ce != cudaSuccess) { *out_rc = (int)ce; return 1; }
  SbGemmArgs g = *a;
  g.D = ws; g.d_is_f32 = 1; g.ldd = a->N; g.beta = 1.f;
  g.bias = nullptr; g.residual = nullptr; g.D_pre = nullptr; g.act = 0; g.alpha = 1.f;
  g.tile_n = 128; g.ksplit = split; g.pair = -1; g.splitk_ws = nullptr; g.splitk_ws_bytes = 0;
  int rc = sb_gemm_bf16(&g, stream);
  if (rc != 0) { *out_rc = rc; return 1; }
  const long long total = (long long)a->M * (a->N >> 2);
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)sms * 4) blocks = (long long)sms * 4;
  splitk_finish_kernel<<<(int)blocks, 256, 0, stream>>>(ws, a->M, a->N, (__nv_bfloat16*)a->D, a->ldd,
                                                       (a->bias && a->bias_is_f32) ? (const float*)a->bias : nullptr,
                                                       (a->bias && !a->bias_is_f32) ? (const __nv_bfloat16*)a->bias : nullptr,
                                                       (__nv_bfloat16*)a->D_pre, a->ldp, (const __nv_bfloat16*)a->residual, a->ldr, a->alpha,
                                                       a->act);
  *out_rc = (int)cudaGetLastError();
  return 1;
}

// Returns 0 on success, a negative code for invalid arguments, or a positive cudaError_t.
SB_API int sb_gemm_bf16(const SbGemmArgs* a, cudaStream_t stream) {
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch0 <= 0 || a->batch1 <= 0) return -1;
  {
    int rc = 0;
    if (small_m_splitk(a, stream, &rc)) return rc;
  }
  // split-K is possible when the epilogue is exactly D(fp32) += alpha * A B^T: weight gradients (long K, few output tiles)
  const bool can_split = a->d_is_f32 && a->beta == 1.f && !a->bias && !a->residual && !a->aux && !a->D_pre && a->act == 0 &&
                         a->drop_p <= 0.f && !a->fold_batch1 && a->ksplit >= 0;
  // Tile width: a tcgen05.mma of M = 128 takes the same 128 cycles for N = 128 and N = 256 (the A operand fetch bounds it), so
  // 256-wide tiles do twice the work per instruction; 128-wide tiles only serve outputs that are no wider than that.
  int bn = a->tile_n;
  if (bn != 128 && bn != 256) bn = a->N > 128 ? 256 : 128;
  // CTA pairs (cta_group::2, 256 x 256 tiles): each CTA stages half of B, which halves the operand traffic per SM and leaves
  // room for six stages; the main loop then runs at the tensor pipe's rate.  Used whenever the shape allows; SbGemmArgs.pair =
  // -1 (or SPEECH_B200_GEMM_PAIR=0) selects single-CTA tiles.
  static const bool env_pair = [] { const char* e = getenv("SPEECH_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  const bool pair = bn == 256 && a->M > 128 && !a->peer_A && (a->pair == 1 || (a->pair == 0 && env_pair));
  CUtensorMap ta, tb;
  int rc;
  if (a->a_mn_major)
    rc = make_operand_map(&ta, a->A, a->M, a->K, a->lda, a->batch0, a->batch1, a->a_bs0, a->a_bs1, BLOCK_K);
  else
    rc = make_operand_map(&ta, a->A, a->K, a->M, a->lda, a->batch0, a->batch1, a->a_bs0, a->a_bs1, BLOCK_M);
  if (rc) return rc;
  if (a->b_mn_major)
    rc = make_operand_map(&tb, a->B, a->N, a->K, a->ldb, a->batch0, a->batch1, a->b_bs0, a->b_bs1, BLOCK_K);
  else
    rc = make_operand_map(&tb, a->B, a->K, a->N, a->ldb, a->batch0, a->batch1, a->b_bs0, a->b_bs1, pair ? bn / 2 : bn);
  if (rc) return rc - 1000;
  GemmParams p;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.batch0 = a->batch0; p.batch1 = a->batch1;
  p.tiles_m = pair ? (a->M + 2 * BLOCK_M - 1) / (2 * BLOCK_M) : (a->M + BLOCK_M - 1) / BLOCK_M;
  p.tiles_n = (a->N + bn - 1) / bn;
  p.kfold = a->fold_batch1 ? a->batch1 : 1;
  {
    const long long nt = (long long)p.tiles_m * p.tiles_n * a->batch0 * (a->fold_batch1 ? 1 : a->batch1);
    if (nt > (1ll << 27)) return -3;   // work items are counted in 32 bits
    p.num_tiles = (int)nt;
  }
  p.ksplit = 1;
  {
    const int num_kb = (a->K + BLOCK_K - 1) / BLOCK_K;
    const int avail = sb_num_sms() - sb_reserved_sms();
    const int sms = pair ? avail / 2 : avail;   // parallel workers: CTA pairs or CTAs
    if (a->ksplit > 1 && can_split) {
      p.ksplit = a->ksplit < num_kb ? a->ksplit : num_kb;
    } else if (can_split && a->ksplit == 0 && p.num_tiles < (long long)sms * 3 / 4) {
      // pick the split whose work-item count fills whole waves best; a slice keeps at least 12 K blocks (768 elements)
      double best = (double)p.num_tiles / sms;  // efficiency of one partial wave
      for (int s = 2; s <= 8 && num_kb / s >= 12; ++s) {
        const long long items = (long long)p.num_tiles * s;
        const double eff = (double)items / ((double)((items + sms - 1) / sms) * sms) - 0.02 * (s - 1);
        if (eff > best + 1e-9) {
          best = eff;
          p.ksplit = s;
        }
      }
    }
    p.kb_per = (num_kb + p.ksplit - 1) / p.ksplit;
    p.ksplit = (num_kb + p.kb_per - 1) / p.kb_per;  // no empty slices
    p.num_work = p.num_tiles * p.ksplit;
  }
  p.a_peer_rows = 0;
  static PeerMaps pm_zero;
  PeerMaps pm = pm_zero;
  if (a->peer_A) {
    // all-gather + GEMM: A is row-sharded over `peer_world` ranks; peer_A[r] is rank r's shard [peer_a_rows, K] (K-major)
    if (pair || a->a_mn_major || a->peer_world < 1 || a->peer_world > 8 || a->peer_a_rows <= 0 || a->peer_a_rows % BLOCK_M != 0 ||
        (long long)a->peer_a_rows * a->peer_world < a->M || a->batch0 != 1 || a->batch1 != 1)
      return -7;
    for (int r = 0; r < a->peer_world; ++r) {
      rc = make_operand_map(&pm.m[r], a->peer_A[r], a->K, a->peer_a_rows, a->lda, 1, 1, 0, 0, BLOCK_M);
      if (rc) return rc - 2000;
    }
    p.a_peer_rows = a->peer_a_rows;
  }
  p.sig_flags = a->sig_flags; p.sig_counter = a->sig_counter;
  p.sig_world = a->sig_world; p.sig_rank = a->sig_rank; p.sig_epoch = a->sig_epoch;
  p.sig_head = (a->sig_flags && a->sig_head) ? 1 : 0;
  p.sig_tail = (a->sig_flags && a->sig_tail) ? 1 : 0;
  if ((p.sig_head || p.sig_tail) && (a->sig_world < 1 || a->sig_world > 8 || a->sig_rank < 0 || a->sig_rank >= a->sig_world)) return -8;
  if (p.sig_tail && !a->sig_counter) return -8;
  if (p.sig_head && !a->peer_A) return -8;
  p.stage_src = a->stage_src; p.stage_dst = a->stage_dst; p.stage_counter = a->stage_counter;
  p.stage_bytes = (a->stage_src && a->stage_dst && a->stage_counter) ? a->stage_bytes : 0;
  if (p.stage_bytes > 0 && (!p.sig_head || (p.stage_bytes & 15) != 0 || pair)) return -9;
  p.status = sb_status_ptr();
  if (!p.status) return -2;
#ifdef SB_GEMM_DIAG
  static const int env_debug = [] { const char* e = getenv("SPEECH_B200_GEMM_DEBUG"); return e ? atoi(e) : 0; }();
  p.debug = env_debug & 31;
  p.trace = g_trace;
#endif
  EpilogueArgs& e = p.ep;
  e.D = a->D; e.d_is_f32 = a->d_is_f32; e.ldd = a->ldd; e.d_bs0 = a->d_bs0; e.d_bs1 = a->d_bs1;
  e.bias_f32 = (a->bias && a->bias_is_f32) ? (const float*)a->bias : nullptr;
  e.bias_bf16 = (a->bias && !a->bias_is_f32) ? (const __nv_bfloat16*)a->bias : nullptr;
  e.residual = (const __nv_bfloat16*)a->residual; e.ldr = a->ldr; e.r_bs0 = a->r_bs0; e.r_bs1 = a->r_bs1;
  e.aux = (const __nv_bfloat16*)a->aux; e.ldx = a->ldx; e.x_bs0 = a->x_bs0; e.x_bs1 = a->x_bs1;
  e.D_pre = (__nv_bfloat16*)a->D_pre; e.ldp = a->ldp; e.p_bs0 = a->p_bs0; e.p_bs1 = a->p_bs1;
  e.alpha = a->alpha; e.beta = a->beta; e.act = a->act; e.dact = (a->aux ? a->dact : 0);
  e.peer_D = (float* const*)a->peer_D; e.peer_rows = a->peer_rows;
  if (a->peer_D) {
    if (!a->d_is_f32 || a->peer_rows <= 0 || a->bias || a->residual || a->aux || a->D_pre || a->act || a->drop_p > 0.f ||
        a->batch0 != 1 || a->batch1 != 1 || a->ldd % 4 != 0)
      return -6;   // the scattered output is a pure accumulation of fp32 partial products
  }
  // Outputs go through tensor maps (bulk stores from a swizzled shared-memory box) whenever their layout allows; an fp32 output
  // that accumulates (beta = 1, split-K partial sums) becomes a bulk add-reduction.  Anything else is stored by lanes.
  static PeerMaps om_zero;
  CUtensorMap td = om_zero.m[0], tp = om_zero.m[0];
  e.tma_d = 0; e.tma_p = 0;
  const int ob1 = a->fold_batch1 ? 1 : a->batch1;
  if (!a->peer_D && (a->beta == 0.f || (a->d_is_f32 && a->beta == 1.f) || !a->d_is_f32) &&
      make_out_map(&td, a->D, a->d_is_f32 != 0, a->N, a->M, a->ldd, a->batch0, ob1, a->d_bs0, a->d_bs1) == 0)
    e.tma_d = (a->d_is_f32 && (a->beta == 1.f || p.ksplit > 1)) ? 2 : 1;
  e.tma_ragged_d = (a->N % (a->d_is_f32 ? 4 : 8)) == 0 ? 1 : 0;
  e.tma_ragged_p = (a->N % 8) == 0 ? 1 : 0;
  if (a->D_pre && !a->d_is_f32 && make_out_map(&tp, a->D_pre, false, a->N, a->M, a->ldp, a->batch0, ob1, a->p_bs0, a->p_bs1) == 0)
    e.tma_p = 1;
  e.drop_thresh = sb_dropout_threshold(a->drop_p);
  e.drop_scale = sb_dropout_scale(a->drop_p);
  e.drop_seed = a->drop_seed;
  int grid = sb_num_sms() - sb_reserved_sms();
  if (grid < 8) grid = 8;
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (grid > p.num_work) grid = p.num_work;
  const int variant = (a->a_mn_major ? 2 : 0) | (a->b_mn_major ? 1 : 0) | (bn == 256 ? 4 : 0) | (pair ? 8 : 0);
  if (pair) {
    int pairs = (sb_num_sms() - sb_reserved_sms()) / 2;
    if (pairs < 4) pairs = 4;
    if (a->max_ctas > 1 && a->max_ctas / 2 < pairs) pairs = a->max_ctas / 2;
    if (pairs > p.num_work) pairs = p.num_work;
    grid = 2 * pairs;
  }
  // epilogue class: the leanest kernel that can execute what was asked for
  const bool fwd = a->act != 0 || a->D_pre != nullptr;
  const bool bwd = e.dact != 0;
  if (fwd && bwd) return -11;   // act(.) and act'(aux) never meet in one GEMM
  if (fwd) return sb_gemm_launch_fwd(variant, grid, pair, stream, ta, tb, p, pm, td, tp);
  if (bwd) return sb_gemm_launch_bwd(variant, grid, pair, stream, ta, tb, p, pm, td, tp);
  if (a->residual || a->drop_p > 0.f) return sb_gemm_launch_fwd(variant, grid, pair, stream, ta, tb, p, pm, td, tp);
  return sb_gemm_launch_lean(variant, grid, pair, stream, ta, tb, p, pm, td, tp);
}
