// Latency-bound all-reduce of a small fp32 vector (BatchNorm statistics: a few thousand floats) over NVLink peer memory in one
// single-CTA kernel: every rank stores its vector into a slot of every peer's symmetric buffer, raises a flag there, waits
// for the flags of all peers in its own buffer and sums the slots in rank order (bit-identical results on all ranks).
// Replaces the per-layer NCCL all-reduce that synchronised BatchNorm needs (the reference relies on torch's SyncBatchNorm,
// i.e. an NCCL all-gather of the statistics per layer).
//
// Symmetric buffer layout (per rank):  [ flags: 2 x MAX_WORLD u32 | slots: 2 x MAX_WORLD x SB_SMALL_MAX floats ].
// Call number `epoch` (1, 2, ... identical on all ranks) uses half `epoch & 1` of the flags and slots.  A rank can only start
// call e+2 after it has seen every peer's flag of call e+1, and a peer raises that flag only after it finished reading the
// slots of call e, so two halves are enough.  Plain P2P stores and loads only (no TMA, no multicast).  The wait is bounded:
// after the wait limit (common.cuh) the kernel records SB_TIMEOUT_PEER_FLAG in the status word and leaves `data` untouched.
#include "common.cuh"

#include "peer_small.h"

namespace {

__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr long long kFlagsBytes = 2LL * SB_SMALL_MAX_WORLD * sizeof(unsigned int);
constexpr long long kFlagsRegion = (kFlagsBytes + 255) / 256 * 256;

__global__ void __launch_bounds__(256) peer_small_allreduce_kernel(SbPeerSmallArgs a) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const int half = (int)(a.epoch & 1u);
  const int total = a.n + (a.has_extra ? 1 : 0);
  // 1. my vector into slot [half][rank] of every rank's buffer (my own included)
  for (int p = 0; p < a.world; ++p) {
    float* slot = reinterpret_cast<float*>((char*)a.buffers[p] + a.base_off + kFlagsRegion) +
                  ((long long)half * SB_SMALL_MAX_WORLD + a.rank) * SB_SMALL_MAX;
    for (int i = threadIdx.x; i < total; i += blockDim.x) slot[i] = (i < a.n) ? a.data[i] : a.extra;
  }
  __threadfence_system();
  __syncthreads();
  // 2. flag [half][rank] = epoch in every peer's buffer
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    unsigned int* f = reinterpret_cast<unsigned int*>((char*)a.buffers[threadIdx.x] + a.base_off) + half * SB_SMALL_MAX_WORLD + a.rank;
    st_release_sys_u32(f, a.epoch);
  }
  // 3. wait for every peer's flag of this call in my own buffer
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    const unsigned int* f = reinterpret_cast<const unsigned int*>((char*)a.buffers[a.rank] + a.base_off) + half * SB_SMALL_MAX_WORLD +
                            threadIdx.x;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys_u32(f) - a.epoch) < 0) {
      if (clock64() - t0 > sb_wait_cycles(a.status) || sb_failed(a.status)) {
        atomicExch(&s_fail, 1);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
  if (s_fail) {
    if (threadIdx.x == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, (int)a.epoch);
    return;
  }
  // 4. sum the slots of this half in rank order
  const float* mine = reinterpret_cast<const float*>((char*)a.buffers[a.rank] + a.base_off + kFlagsRegion) +
                      (long long)half * SB_SMALL_MAX_WORLD * SB_SMALL_MAX;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    float s = 0.f;
    for (int q = 0; q < a.world; ++q) s += __ldcg(mine + (long long)q * SB_SMALL_MAX + i);
    a.data[i] = s;
  }
}

}  // namespace

// Bytes of symmetric memory the protocol needs (per rank).
SB_API long long sb_peer_small_bytes() { return kFlagsRegion + 2LL * SB_SMALL_MAX_WORLD * SB_SMALL_MAX * (long long)sizeof(float); }
SB_API int sb_peer_small_max() { return SB_SMALL_MAX; }

SB_API int sb_peer_small_allreduce(const SbPeerSmallArgs* args, cudaStream_t stream) {
  SbPeerSmallArgs a = *args;
  if (a.world < 1 || a.world > SB_SMALL_MAX_WORLD || a.rank < 0 || a.rank >= a.world) return -1;
  if (a.n <= 0 || a.n + (a.has_extra ? 1 : 0) > SB_SMALL_MAX || !a.data || !a.buffers || a.epoch == 0) return -2;
  a.status = sb_status_ptr();
  if (!a.status) return -3;
  peer_small_allreduce_kernel<<<1, 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}
