// Small memory-bound kernels beside the encoder and the decoders: SpecAugment masks applied in place, and one step of a
// back-off n-gram automaton for every (hypothesis, token) pair.
//
// SpecAugment (reference behaviour: parts/submodules/spectr_augment.py:25 and the Numba kernel
// parts/numba/spec_augment/spec_aug_numba.py:27-95): the masks are drawn on the device as start / width tensors; the
// kernel writes ONLY the masked elements (a masked frequency row entirely, otherwise the masked time ranges of the row), so
// the traffic is the masked fraction of the tensor instead of a read + write of all of it.
//
// N-gram advance (reference: parts/submodules/ngram_lm/ngram_lm_batched.py:1005-1129 and its Triton kernel
// ngram_advance_triton_kernel.py): arcs sorted by state * V + token, per-state back-off weight and state.  One block per
// hypothesis walks the back-off chain once (at most 16 levels), finds the arc range of every level with two binary
// searches, and then every thread resolves its tokens by a binary search inside those short ranges.
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ T cast_from(float v);
template <> __device__ __forceinline__ float cast_from<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cast_from<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

constexpr int kMaxMasks = 32;

template <typename T>
__global__ void specaugment_kernel(T* __restrict__ x, int F, int T_, const int* __restrict__ f_start, const int* __restrict__ f_width,
                                   int nf, const int* __restrict__ t_start, const int* __restrict__ t_width, int nt,
                                   const long long* __restrict__ length, float mask_value) {
  const int b = blockIdx.y, f = blockIdx.x;
  __shared__ int s_ts[kMaxMasks], s_tw[kMaxMasks];
  __shared__ int s_row;
  if (threadIdx.x == 0) {
    int row = 0;
    for (int i = 0; i < nf; ++i) {
      int s = f_start[b * nf + i], w = f_width[b * nf + i];
      row |= (f >= s && f < s + w);
    }
    s_row = row;
  }
  if (threadIdx.x < nt) {
    s_ts[threadIdx.x] = t_start[b * nt + threadIdx.x];
    s_tw[threadIdx.x] = t_width[b * nt + threadIdx.x];
  }
  __syncthreads();
  T* row = x + ((size_t)b * F + f) * T_;
  const T fill = cast_from<T>(mask_value);
  if (s_row) {
    for (int t = threadIdx.x; t < T_; t += blockDim.x) row[t] = fill;
    return;
  }
  (void)length;
  for (int i = 0; i < nt; ++i) {
    int lo = max(s_ts[i], 0), hi = min(s_ts[i] + s_tw[i], T_);
    for (int t = lo + threadIdx.x; t < hi; t += blockDim.x) row[t] = fill;
  }
}

constexpr int kMaxDepth = 16;

__device__ __forceinline__ int lower_bound(const long long* __restrict__ keys, int lo, int hi, long long key) {
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (keys[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void ngram_advance_kernel(const long long* __restrict__ states, const long long* __restrict__ arc_keys,
                                     const float* __restrict__ arc_w, const long long* __restrict__ arc_to,
                                     const float* __restrict__ backoff_w, const long long* __restrict__ backoff_to, int n_arcs,
                                     int n_states, int V, int depth, float default_score, long long start_state,
                                     float* __restrict__ scores, long long* __restrict__ next_states) {
  const int b = blockIdx.x;
  __shared__ long long s_state[kMaxDepth];
  __shared__ float s_acc[kMaxDepth + 1];
  __shared__ int s_lo[kMaxDepth], s_hi[kMaxDepth];
  if (threadIdx.x == 0) {
    long long cur = states[b];
    float acc = 0.f;
    for (int d = 0; d < depth; ++d) {
      if (cur < 0 || cur >= n_states) cur = start_state;   // a corrupt state id never indexes outside the tables
      s_state[d] = cur;
      s_acc[d] = acc;
      acc += backoff_w[cur];
      cur = backoff_to[cur];
    }
    s_acc[depth] = acc;
  }
  __syncthreads();
  if (threadIdx.x < depth) {
    long long base = s_state[threadIdx.x] * (long long)V;
    int lo = lower_bound(arc_keys, 0, n_arcs, base);
    s_lo[threadIdx.x] = lo;
    s_hi[threadIdx.x] = lower_bound(arc_keys, lo, n_arcs, base + V);
  }
  __syncthreads();
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    float sc = s_acc[depth] + default_score;
    long long nx = start_state;
    for (int d = 0; d < depth; ++d) {
      int lo = s_lo[d], hi = s_hi[d];
      if (lo == hi) continue;
      long long key = s_state[d] * (long long)V + v;
      int i = lower_bound(arc_keys, lo, hi, key);
      if (i < hi && arc_keys[i] == key) {
        sc = s_acc[d] + arc_w[i];
        nx = arc_to[i];
        break;
      }
    }
    scores[(size_t)b * V + v] = sc;
    next_states[(size_t)b * V + v] = nx;
  }
}

}  // namespace

// x: [B, F, T] contiguous (fp32 or bf16), masked in place.  f_start / f_width: int32 [B, nf]; t_start / t_width: int32 [B, nt].
SB_API int sb_specaugment(void* x, int is_bf16, int B, int F, int T, const int* f_start, const int* f_width, int nf,
                          const int* t_start, const int* t_width, int nt, const long long* length, float mask_value,
                          cudaStream_t stream) {
  if (B <= 0 || F <= 0 || T <= 0) return 0;
  if (nf < 0 || nt < 0 || nt > kMaxMasks || B > 65535) return -1;
  dim3 grid(F, B);
  if (is_bf16)
    specaugment_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((__nv_bfloat16*)x, F, T, f_start, f_width, nf, t_start, t_width, nt,
                                                               length, mask_value);
  else
    specaugment_kernel<float><<<grid, 128, 0, stream>>>((float*)x, F, T, f_start, f_width, nf, t_start, t_width, nt, length, mask_value);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// One automaton step for B hypotheses and all V tokens: scores [B, V] fp32, next_states [B, V] int64.
SB_API int sb_ngram_advance(const long long* states, const long long* arc_keys, const float* arc_w, const long long* arc_to,
                            const float* backoff_w, const long long* backoff_to, int n_arcs, int n_states, int B, int V, int depth,
                            float default_score, long long start_state, float* scores, long long* next_states,
                            cudaStream_t stream) {
  if (B <= 0 || V <= 0) return 0;
  if (depth < 1 || depth > kMaxDepth || n_states <= 0) return -1;
  ngram_advance_kernel<<<B, 256, 0, stream>>>(states, arc_keys, arc_w, arc_to, backoff_w, backoff_to, n_arcs, n_states, V, depth,
                                              default_score, start_state, scores, next_states);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
