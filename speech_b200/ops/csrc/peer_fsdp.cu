// Fully-sharded data parallelism over NVLink peer memory: parameter all-gather fused with the up-cast, and gradient
// reduce-scatter fused with the sliced AdamW update.
//
// The reference shards parameters with PyTorch FSDP2 (nemo/collections/speechlm2/models/salm.py:534-543, fully_shard per layer):
// NCCL all-gather before a layer's forward / backward, NCCL reduce-scatter after its backward, a separate optimizer pass over the
// local shards.  Here every rank keeps the bf16 working copy of ITS shard of every unit in a symmetric buffer that all ranks can
// address, and
//   * peer_gather_kernel builds a unit's full bf16 parameters (and, optionally, their fp32 image for code that reads
//     parameter.data) by plain peer loads of the other ranks' shards: no staging copy on the sender, no flags (shards only change
//     in the optimizer step, which ends with a barrier);
//   * peer_pack_kernel writes this rank's unit gradient, scaled and cast to bf16, into its symmetric gradient buffer;
//   * peer_rs_adamw_kernel waits for all ranks' gradient buffers of the unit (flags, bounded waits), sums the slice this rank
//     owns over all ranks by peer loads in a fixed rank order and either
//       - applies AdamW to the rank's fp32 master / moment slices at once and refreshes the bf16 shard (no global clipping), or
//       - stores the reduced fp32 slice and adds its sum of squares to a device scalar (global-norm clipping: the update then
//         runs after one small all-reduce of that scalar).
// CTA b of a rank only waits for CTA b of its peers, so no CTA depends on another CTA of its own GPU.
#include "common.cuh"

#define SB_FSDP_MAX_WORLD 16
#define SB_FSDP_MAX_CTAS 64

struct SbFsdpArgs {
  void* const* grad_bufs;       // device array [world]: every rank's symmetric gradient buffer (bf16 [slice * world] per parity)
  long long buf_off;            // byte offset of this launch's parity half inside the gradient buffers
  long long flags_off;          // byte offset of the flag block inside the gradient buffers
  long long slice;              // elements per rank of this unit (multiple of 8)
  int rank, world, ctas;
  unsigned int epoch;           // per-parity launch counter, starts at 1
  int* status;
  // outputs for this rank's slice
  float* grad_shard;            // mode 1: reduced fp32 gradient slice; may be null in mode 0
  float* sumsq;                 // mode 1: device scalar accumulating the sum of squares
  // mode 0: fused AdamW on the slice
  float* master;
  float* exp_avg;
  float* exp_avg_sq;
  __nv_bfloat16* lowp_shard;    // this rank's bf16 shard (in the symmetric parameter buffer)
  float lr, beta1, beta2, eps, wd, bc1, rsqrt_bc2;
  int mode;                     // 0 = reduce + AdamW, 1 = reduce + store + sum of squares
};

namespace {

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void add8(float* acc, const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// dst_bf16[r * slice + i] = shard of rank r, element i;  dst_f32 (optional) receives the same values as fp32.
__global__ void __launch_bounds__(512) peer_gather_kernel(void* const* __restrict__ bufs, long long src_off, long long slice, int world,
                                                         __nv_bfloat16* __restrict__ dst, float* __restrict__ dst_f32) {
  const long long n8 = slice >> 3;
  const long long total = n8 * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // four peer loads in flight per thread: the copy is bound by NVLink latency, not by the few blocks' arithmetic
  for (long long g0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; g0 < total; g0 += 4 * stride) {
    uint4 v[4];
    long long o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long g = g0 + u * stride;
      o[u] = -1;
      if (g < total) {
        const int r = (int)(g / n8);
        const long long i = (g - (long long)r * n8) << 3;
        v[u] = __ldcg(reinterpret_cast<const uint4*>((const char*)bufs[r] + src_off + i * 2));
        o[u] = (long long)r * slice + i;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (o[u] < 0) continue;
      *reinterpret_cast<uint4*>(dst + o[u]) = v[u];
      if (dst_f32) {
        float t[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        add8(t, v[u]);
        *reinterpret_cast<float4*>(dst_f32 + o[u]) = make_float4(t[0], t[1], t[2], t[3]);
        *reinterpret_cast<float4*>(dst_f32 + o[u] + 4) = make_float4(t[4], t[5], t[6], t[7]);
      }
    }
  }
}

__global__ void peer_fsdp_pack_kernel(const float* __restrict__ grad, __nv_bfloat16* __restrict__ send, long long n, float scale) {
  const long long n8 = n >> 3;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n8; g += (long long)gridDim.x * blockDim.x) {
    const long long e = g << 3;
    const float4 x = *reinterpret_cast<const float4*>(grad + e), y = *reinterpret_cast<const float4*>(grad + e + 4);
    __align__(16) __nv_bfloat162 o[4] = {__floats2bfloat162_rn(x.x * scale, x.y * scale), __floats2bfloat162_rn(x.z * scale, x.w * scale),
                                         __floats2bfloat162_rn(y.x * scale, y.y * scale), __floats2bfloat162_rn(y.z * scale, y.w * scale)};
    *reinterpret_cast<uint4*>(send + e) = *reinterpret_cast<const uint4*>(o);
  }
}

__device__ bool wait_flags(const unsigned int* my_flags, int b, int world, int rank, unsigned int want, int* s_fail, const int* status) {
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const unsigned int* f = my_flags + (long long)b * SB_FSDP_MAX_WORLD + threadIdx.x;
    const long long t0 = clock64();
    unsigned int probes = 0;
    while ((int)(ld_acquire_sys(f) - want) < 0) {
      if (clock64() - t0 > sb_wait_cycles(status) || ((++probes & 255u) == 0 && sb_failed(status))) {
        atomicExch(s_fail, 1);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return *s_fail == 0;
}
__device__ void raise_flags(const SbFsdpArgs& a, int b, unsigned int value) {
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < a.world && (int)threadIdx.x != a.rank) {
    unsigned int* f = reinterpret_cast<unsigned int*>((char*)a.grad_bufs[threadIdx.x] + a.flags_off) + (long long)b * SB_FSDP_MAX_WORLD + a.rank;
    st_release_sys(f, value);
  }
}

__global__ void __launch_bounds__(512) peer_rs_adamw_kernel(SbFsdpArgs a) {
  __shared__ int s_fail;
  __shared__ float red[32];
  const int b = blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned int* my_flags = reinterpret_cast<const unsigned int*>((const char*)a.grad_bufs[a.rank] + a.flags_off);
  // every rank's gradient buffer of this unit is packed (its pack kernel ran before this kernel on its stream)
  raise_flags(a, b, 2u * a.epoch + 1u);
  if (!wait_flags(my_flags, b, a.world, a.rank, 2u * a.epoch + 1u, &s_fail, a.status)) {
    if (threadIdx.x == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 11);
    return;
  }
  long long chunk = (a.slice + a.ctas - 1) / a.ctas;
  chunk = (chunk + 7) / 8 * 8;
  const long long c0 = (long long)b * chunk, c1 = min(a.slice, c0 + chunk);
  const long long base = (long long)a.rank * a.slice;
  float sq = 0.f;
  const long long step = (long long)blockDim.x * 8;
  long long i_begin = c0 + (long long)threadIdx.x * 8;
  if (a.mode == 1 && a.world <= 2) {
    // store-only form with few ranks: four positions (x world loads) in flight per thread; rank order of the sums is unchanged
    for (; i_begin + 3 * step < c1; i_begin += 4 * step) {
      uint4 v[4][2];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < a.world) v[u][q] = __ldcg(reinterpret_cast<const uint4*>((const char*)a.grad_bufs[q] + a.buf_off + (base + i_begin + u * step) * 2));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < a.world) add8(acc, v[u][q]);
        const long long i = i_begin + u * step;
        *reinterpret_cast<float4*>(a.grad_shard + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(a.grad_shard + i + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
        for (int k = 0; k < 8; ++k) sq += acc[k] * acc[k];
      }
    }
  }
  for (long long i = i_begin; i < c1; i += step) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // fixed order by rank: every run (and every world layout) sums in the same order; four peer loads in flight
    for (int q0 = 0; q0 < a.world; q0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q0 + q < a.world) v[q] = __ldcg(reinterpret_cast<const uint4*>((const char*)a.grad_bufs[q0 + q] + a.buf_off + (base + i) * 2));
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q0 + q < a.world) add8(acc, v[q]);
    }
    if (a.mode == 1) {
      *reinterpret_cast<float4*>(a.grad_shard + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(a.grad_shard + i + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int k = 0; k < 8; ++k) sq += acc[k] * acc[k];
    } else {
      float p[8], m[8], v2[8];
      *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(a.master + i);
      *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(a.master + i + 4);
      *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(a.exp_avg + i);
      *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(a.exp_avg + i + 4);
      *reinterpret_cast<float4*>(v2) = *reinterpret_cast<const float4*>(a.exp_avg_sq + i);
      *reinterpret_cast<float4*>(v2 + 4) = *reinterpret_cast<const float4*>(a.exp_avg_sq + i + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float g = acc[k];
        m[k] = a.beta1 * m[k] + (1.f - a.beta1) * g;
        v2[k] = a.beta2 * v2[k] + (1.f - a.beta2) * g * g;
        p[k] = p[k] * (1.f - a.lr * a.wd) - (a.lr / a.bc1) * (m[k] / (sqrtf(v2[k]) * a.rsqrt_bc2 + a.eps));
      }
      *reinterpret_cast<float4*>(a.master + i) = *reinterpret_cast<const float4*>(p);
      *reinterpret_cast<float4*>(a.master + i + 4) = *reinterpret_cast<const float4*>(p + 4);
      *reinterpret_cast<float4*>(a.exp_avg + i) = *reinterpret_cast<const float4*>(m);
      *reinterpret_cast<float4*>(a.exp_avg + i + 4) = *reinterpret_cast<const float4*>(m + 4);
      *reinterpret_cast<float4*>(a.exp_avg_sq + i) = *reinterpret_cast<const float4*>(v2);
      *reinterpret_cast<float4*>(a.exp_avg_sq + i + 4) = *reinterpret_cast<const float4*>(v2 + 4);
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(p[2 * k], p[2 * k + 1]);
      *reinterpret_cast<uint4*>(a.lowp_shard + i) = *reinterpret_cast<const uint4*>(o);
    }
  }
  if (a.mode == 1) {
    sq = block_sum(sq, red);
    if (threadIdx.x == 0 && sq != 0.f) atomicAdd(a.sumsq, sq);
  }
  // this rank has finished reading the peers' buffers of this parity: they may be packed again two units later
  raise_flags(a, b, 2u * a.epoch + 2u);
  if (!wait_flags(my_flags, b, a.world, a.rank, 2u * a.epoch + 2u, &s_fail, a.status)) {
    if (threadIdx.x == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 12);
  }
}

}  // namespace

SB_API long long sb_fsdp_flags_bytes() { return (long long)SB_FSDP_MAX_CTAS * SB_FSDP_MAX_WORLD * sizeof(unsigned int); }

// bufs: device array [world] of the ranks' symmetric PARAMETER buffers; slice elements (multiple of 8) from byte offset src_off of
// each are gathered into dst (bf16 [world * slice]) and, when dst_f32 is given, up-cast into it as well.
SB_API int sb_fsdp_gather(void* const* bufs, long long src_off, long long slice, int world, void* dst, float* dst_f32, int blocks,
                          cudaStream_t stream) {
  if (world < 1 || world > SB_FSDP_MAX_WORLD || slice <= 0 || (slice & 7) || (src_off & 15)) return -1;
  if (blocks <= 0) blocks = 32;
  peer_gather_kernel<<<blocks, 512, 0, stream>>>(bufs, src_off, slice, world, (__nv_bfloat16*)dst, dst_f32);
  return (int)cudaGetLastError();
}

// grad: this rank's fp32 unit gradient [slice * world]; my_grad_buf: this rank's symmetric gradient buffer.  Launches the pack
// kernel and the reduce(+AdamW) kernel on `stream`.
SB_API int sb_fsdp_reduce_scatter(SbFsdpArgs* a, const float* grad, void* my_grad_buf, float scale, int step, cudaStream_t stream) {
  if (a->world < 1 || a->world > SB_FSDP_MAX_WORLD || a->rank < 0 || a->rank >= a->world || a->ctas < 1 || a->ctas > SB_FSDP_MAX_CTAS) return -1;
  if (a->slice <= 0 || (a->slice & 7) || (a->buf_off & 15) || a->epoch == 0 || !my_grad_buf) return -1;
  if (a->mode == 0 && (!a->master || !a->exp_avg || !a->exp_avg_sq || !a->lowp_shard)) return -2;
  if (a->mode == 1 && (!a->grad_shard || !a->sumsq)) return -2;
  a->status = sb_status_ptr();
  if (!a->status) return -3;
  if (a->mode == 0) {
    a->bc1 = 1.f - powf(a->beta1, (float)step);
    a->rsqrt_bc2 = 1.f / sqrtf(1.f - powf(a->beta2, (float)step));
  }
  const long long n = a->slice * a->world;
  long long blocks = ((n >> 3) + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 4;
  if (blocks > cap) blocks = cap;
  peer_fsdp_pack_kernel<<<(int)blocks, 256, 0, stream>>>(grad, reinterpret_cast<__nv_bfloat16*>((char*)my_grad_buf + a->buf_off), n, scale);
  peer_rs_adamw_kernel<<<a->ctas, 512, 0, stream>>>(*a);
  return (int)cudaGetLastError();
}
