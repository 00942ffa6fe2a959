// Log-mel front end in two kernels (fp32 throughout, as the reference's featurizer:
// nemo/collections/asr/parts/preprocessing/features.py:415-494):
//   logmel_frames:    dither -> pre-emphasis (+ length mask) -> centred framing with zero padding -> window ->
//                     512-point FFT in shared memory -> power spectrum -> mel filterbank -> log(x + guard)
//   logmel_normalize: per-utterance, per-feature mean / unbiased std over the valid frames, normalisation,
//                     padding value beyond the valid length
// Output layout [B, nfilt, T].  A block transforms FR consecutive frames of one utterance.
#include "common.cuh"

namespace {

constexpr int NFFT = 512;
constexpr int NBINS = NFFT / 2 + 1;
constexpr int FR = 8;

__device__ __forceinline__ uint32_t mix32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return (uint32_t)x;
}
__device__ __forceinline__ float gauss_noise(uint64_t seed, uint64_t idx) {
  const uint32_t a = mix32(seed + 2 * idx), b = mix32(seed + 2 * idx + 1);
  const float u1 = ((a >> 8) + 1) * (1.0f / 16777217.0f), u2 = (b >> 8) * (1.0f / 16777216.0f);
  return sqrtf(-2.f * __logf(u1)) * __cosf(6.2831853f * u2);
}

__device__ __forceinline__ float sample_at(const float* x, long long n, long long len, float dither, uint64_t seed, uint64_t base) {
  if (n < 0 || n >= len) return 0.f;
  float v = x[n];
  if (dither > 0.f) v += dither * gauss_noise(seed, base + (uint64_t)n);
  return v;
}

__global__ void logmel_frames_kernel(const float* __restrict__ wave, long long wave_ld, const long long* __restrict__ seq_len,
                                     const float* __restrict__ window, int win_len, const float* __restrict__ fb,
                                     const int* __restrict__ fb_range, int nfilt, int hop, float preemph, float guard,
                                     float dither, unsigned long long seed, float* __restrict__ out, int T) {
  __shared__ float re[NFFT], im[NFFT], tw_re[NFFT / 2], tw_im[NFFT / 2], pw[NBINS + 3];
  const int b = blockIdx.y;
  const int tid = threadIdx.x;  // 256 threads
  const long long len = seq_len[b];
  const float* x = wave + (long long)b * wave_ld;
  const uint64_t nbase = (uint64_t)b * (uint64_t)wave_ld;
  const int woff = (NFFT - win_len) / 2;
  {
    float s, c;
    sincospif(-2.0f * tid / NFFT, &s, &c);
    tw_re[tid] = c;
    tw_im[tid] = s;
  }
  for (int f = 0; f < FR; ++f) {
    const int t = blockIdx.x * FR + f;
    if (t >= T) break;
    __syncthreads();
    // two samples per thread, written at bit-reversed positions
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int i = tid + h * 256;
      const long long n = (long long)t * hop - NFFT / 2 + i;
      float v = 0.f;
      const int wi = i - woff;
      if (wi >= 0 && wi < win_len) {
        float cur = sample_at(x, n, len, dither, seed, nbase);
        if (preemph != 0.f && n > 0 && n < len) cur -= preemph * sample_at(x, n - 1, len, dither, seed, nbase);
        v = cur * window[wi];
      }
      const int r = __brev((unsigned)i) >> 23;  // 9-bit reversal
      re[r] = v;
      im[r] = 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int s = 1; s <= 9; ++s) {
      const int half = 1 << (s - 1);
      const int grp = tid / half, pos = tid % half;
      const int i0 = grp * (half << 1) + pos, i1 = i0 + half;
      const int tw = pos * (NFFT >> s);
      const float wr = tw_re[tw], wi = tw_im[tw];
      const float xr = re[i1] * wr - im[i1] * wi, xi = re[i1] * wi + im[i1] * wr;
      const float ar = re[i0], ai = im[i0];
      __syncthreads();
      re[i0] = ar + xr; im[i0] = ai + xi;
      re[i1] = ar - xr; im[i1] = ai - xi;
      __syncthreads();
    }
    for (int k = tid; k < NBINS; k += 256) pw[k] = re[k] * re[k] + im[k] * im[k];
    __syncthreads();
    if (tid < nfilt) {
      const int k0 = fb_range[2 * tid], k1 = fb_range[2 * tid + 1];
      float acc = 0.f;
      for (int k = k0; k < k1; ++k) acc += fb[tid * NBINS + k] * pw[k];
      out[((long long)b * nfilt + tid) * T + t] = __logf(acc + guard);
    }
  }
}

__global__ void logmel_normalize_kernel(float* __restrict__ mel, const long long* __restrict__ out_len, int nfilt, int T,
                                        int normalize, float pad_value) {
  __shared__ float red[32];
  const int b = blockIdx.y, j = blockIdx.x;
  float* row = mel + ((long long)b * nfilt + j) * T;
  const int n = (int)min((long long)T, out_len[b]);
  float mean = 0.f, rstd = 1.f;
  if (normalize) {
    float s = 0.f;
    for (int t = threadIdx.x; t < n; t += blockDim.x) s += row[t];
    s = block_sum(s, red);
    mean = n > 0 ? s / n : 0.f;
    float ss = 0.f;
    for (int t = threadIdx.x; t < n; t += blockDim.x) { const float d = row[t] - mean; ss += d * d; }
    ss = block_sum(ss, red);
    float sd = n > 1 ? sqrtf(ss / (n - 1)) : 0.f;
    rstd = 1.f / (sd + 1e-5f);
  }
  for (int t = threadIdx.x; t < T; t += blockDim.x) row[t] = t < n ? (row[t] - mean) * rstd : pad_value;
}

}  // namespace

// wave: fp32 [B, wave_ld]; out: fp32 [B, nfilt, T] with T >= 1 + max_len / hop; fb: [nfilt, 257]; fb_range: int [nfilt, 2]
SB_API int sb_logmel(const float* wave, long long wave_ld, const long long* seq_len, const long long* out_len, const float* window,
                     int win_len, const float* fb, const int* fb_range, int nfilt, int n_fft, int hop, float preemph, float guard,
                     float dither, unsigned long long seed, int normalize, float pad_value, float* out, int B, int T, int T_frames,
                     cudaStream_t stream) {
  if (n_fft != NFFT || nfilt > 256 || win_len > NFFT || B <= 0 || T <= 0) return -1;
  dim3 grid((T_frames + FR - 1) / FR, B);
  logmel_frames_kernel<<<grid, 256, 0, stream>>>(wave, wave_ld, seq_len, window, win_len, fb, fb_range, nfilt, hop, preemph, guard,
                                                dither, seed, out, T);
  dim3 g2(nfilt, B);
  logmel_normalize_kernel<<<g2, 256, 0, stream>>>(out, out_len, nfilt, T, normalize, pad_value);
  return (int)cudaGetLastError();
}
