// Gradient all-reduce over NVLink peer memory in ONE kernel per bucket: cast + scale, reduce-scatter by peer loads,
// all-gather by peer stores, unpack.  Replaces the c10d reducer + NCCL all-reduce of the reference's DDP strategy for
// buckets of the flat gradient arena.
//
// Every rank owns one symmetric buffer laid out as  [ flags | send (bf16) | recv (bf16) ]  and knows the base address of
// every peer's buffer (plain P2P pointers: ordinary loads and stores, no TMA, no multicast).  All ranks launch this kernel
// for the same bucket in the same order.  CTA b of rank r:
//   phase 0  casts its sub-chunk b of EVERY slice p of the local fp32 gradient (times `scale`) to bf16 in the local send
//            buffer, then raises flag (b, r) = 2*epoch+1 in every peer's flag block;
//   wait     until flags (b, q) >= 2*epoch+1 for all peers q                       (their sub-chunk b is ready);
//   phase A  sums sub-chunk b of slice r over all ranks' send buffers in fp32, rounds to bf16 once and stores the result into
//            EVERY rank's recv buffer (so all ranks hold bit-identical values), then raises flag (b, r) = 2*epoch+2;
//   wait     until flags (b, q) >= 2*epoch+2 for all peers q;
//   phase B  converts sub-chunk b of every slice of the local recv buffer to fp32 in the gradient arena.
// CTA b only ever waits for CTA b of the peers, so no CTA depends on another CTA of its own GPU and the grid needs no
// co-residency.  Flags only grow (epoch = launch counter, identical on all ranks), so they are never reset; a rank that is
// one bucket ahead cannot touch a buffer a slower rank still uses because each phase is gated by the slower rank's flag.
// Every wait is bounded: after the wait limit (common.cuh) the CTA records SB_TIMEOUT_PEER_FLAG in the status word and returns
// without touching peer memory again.
#include "common.cuh"
#include <stdlib.h>
#include <string.h>

#define SB_PEER_MAX_WORLD 16
#define SB_PEER_MAX_CTAS 128

struct SbPeerArgs {
  float* grad;                 // local fp32 gradient bucket [n], reduced in place
  void* const* buffers;        // device array [world]: base address of each rank's symmetric buffer
  long long flags_off;         // byte offsets inside a symmetric buffer
  long long send_off;
  long long recv_off;
  long long n;                 // elements in the bucket
  long long slice;             // elements per rank slice (multiple of 8, slice * world >= n)
  long long chunk;             // elements per CTA sub-chunk (multiple of 8, chunk * ctas >= slice)
  int rank, world, ctas;
  unsigned int epoch;          // launch counter, starts at 1
  float scale;
  int* status;                 // device status word (filled in by sb_peer_allreduce)
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

// Thread q < world waits for peer q's flag; everyone gets the verdict.  Returns false after a timeout.
__device__ bool wait_peers(const unsigned int* my_flags, int b, int world, int rank, unsigned int want, int* s_fail, const int* status) {
  if (threadIdx.x < world && threadIdx.x != rank) {
    const unsigned int* f = my_flags + (long long)b * SB_PEER_MAX_WORLD + threadIdx.x;
    const long long t0 = clock64();
    unsigned int probes = 0;
    while ((int)(ld_acquire_sys(f) - want) < 0) {
      // once any kernel has given up (status word set) later waits end at once: a lost rank costs one limit, not one per launch
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

__device__ void signal_peers(const SbPeerArgs& a, int b, unsigned int value) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    unsigned int* f = reinterpret_cast<unsigned int*>((char*)a.buffers[threadIdx.x] + a.flags_off) +
                      (long long)b * SB_PEER_MAX_WORLD + a.rank;
    st_release_sys(f, value);
  }
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

// LOCAL = false leaves out the two local phases (cast into the send region, unpack from the receive region): they are then run
// by the wide element-wise kernels below, so that the few blocks of this kernel only do what needs them, the peer traffic.
template <bool LOCAL>
__global__ void __launch_bounds__(512) peer_allreduce_kernel(SbPeerArgs a) {
  __shared__ int s_fail;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  char* my_base = (char*)a.buffers[a.rank];
  __nv_bfloat16* my_send = reinterpret_cast<__nv_bfloat16*>(my_base + a.send_off);
  __nv_bfloat16* my_recv = reinterpret_cast<__nv_bfloat16*>(my_base + a.recv_off);
  const unsigned int* my_flags = reinterpret_cast<const unsigned int*>(my_base + a.flags_off);
  const long long c0 = (long long)b * a.chunk;                 // sub-chunk range inside a slice
  const long long c1 = min(a.slice, c0 + a.chunk);

  // Every loop below keeps UNR independent 16/32-byte loads in flight per thread: with one load per iteration a 512-thread CTA has
  // 16 KB outstanding and moves ~17 GB/s, a quarter of what four loads give.
  constexpr int UNR = 4;
  const long long step = (long long)blockDim.x * 8;
  // ---- phase 0: local cast of sub-chunk b of every slice
  for (int p = 0; LOCAL && p < a.world; ++p) {
    const long long base = (long long)p * a.slice;
    for (long long i0 = c0 + (long long)threadIdx.x * 8; i0 < c1; i0 += step * UNR) {
      float4 x[UNR], y[UNR];
      bool vec[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * step, e = base + i;
        vec[u] = i < c1 && e + 8 <= a.n;
        if (vec[u]) {
          x[u] = *reinterpret_cast<const float4*>(a.grad + e);
          y[u] = *reinterpret_cast<const float4*>(a.grad + e + 4);
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * step, e = base + i;
        if (i >= c1) break;
        __align__(16) __nv_bfloat162 o[4];
        if (vec[u]) {
          o[0] = __floats2bfloat162_rn(x[u].x * a.scale, x[u].y * a.scale);
          o[1] = __floats2bfloat162_rn(x[u].z * a.scale, x[u].w * a.scale);
          o[2] = __floats2bfloat162_rn(y[u].x * a.scale, y[u].y * a.scale);
          o[3] = __floats2bfloat162_rn(y[u].z * a.scale, y[u].w * a.scale);
        } else {
          float t[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) t[k] = (e + k < a.n) ? a.grad[e + k] * a.scale : 0.f;
#pragma unroll
          for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(t[2 * k], t[2 * k + 1]);
        }
        *reinterpret_cast<uint4*>(my_send + e) = *reinterpret_cast<const uint4*>(o);
      }
    }
  }
  signal_peers(a, b, 2u * a.epoch + 1u);
  if (!wait_peers(my_flags, b, a.world, a.rank, 2u * a.epoch + 1u, &s_fail, a.status)) {
    if (threadIdx.x == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 1);
    return;
  }

  // ---- phase A: reduce my slice's sub-chunk over all ranks, broadcast the rounded result
  {
    const long long base = (long long)a.rank * a.slice;
    constexpr int UA = 2, QB = 4;   // 2 positions x 4 ranks = 8 independent 16-byte peer reads in flight per thread
    for (long long i0 = c0 + (long long)threadIdx.x * 8; i0 < c1; i0 += step * UA) {
      float acc[UA][8];
#pragma unroll
      for (int u = 0; u < UA; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      for (int q0 = 0; q0 < a.world; q0 += QB) {
        uint4 v[UA][QB];
#pragma unroll
        for (int u = 0; u < UA; ++u) {
          const long long i = i0 + u * step, e = base + i;
#pragma unroll
          for (int q = 0; q < QB; ++q)
            if (i < c1 && e < a.n && q0 + q < a.world)
              v[u][q] = *reinterpret_cast<const uint4*>((const char*)a.buffers[q0 + q] + a.send_off + e * 2);
        }
#pragma unroll
        for (int u = 0; u < UA; ++u) {
          const long long i = i0 + u * step, e = base + i;
#pragma unroll
          for (int q = 0; q < QB; ++q)
            if (i < c1 && e < a.n && q0 + q < a.world) add8(acc[u], v[u][q]);
        }
      }
#pragma unroll
      for (int u = 0; u < UA; ++u) {
        const long long i = i0 + u * step, e = base + i;
        if (i >= c1 || e >= a.n) break;
        __align__(16) __nv_bfloat162 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[u][2 * k], acc[u][2 * k + 1]);
        const uint4 r = *reinterpret_cast<const uint4*>(o);
        for (int q = 0; q < a.world; ++q) *reinterpret_cast<uint4*>((char*)a.buffers[q] + a.recv_off + e * 2) = r;
      }
    }
  }
  signal_peers(a, b, 2u * a.epoch + 2u);
  if (!wait_peers(my_flags, b, a.world, a.rank, 2u * a.epoch + 2u, &s_fail, a.status)) {
    if (threadIdx.x == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 2);
    return;
  }

  // ---- phase B: unpack sub-chunk b of every slice into the fp32 arena
  for (int p = 0; LOCAL && p < a.world; ++p) {
    const long long base = (long long)p * a.slice;
    for (long long i0 = c0 + (long long)threadIdx.x * 8; i0 < c1; i0 += step * UNR) {
      uint4 v[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * step, e = base + i;
        if (i < c1 && e < a.n) v[u] = *reinterpret_cast<const uint4*>(my_recv + e);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * step, e = base + i;
        if (i >= c1 || e >= a.n) break;
        float t[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        add8(t, v[u]);
        if (e + 8 <= a.n) {
          *reinterpret_cast<float4*>(a.grad + e) = make_float4(t[0], t[1], t[2], t[3]);
          *reinterpret_cast<float4*>(a.grad + e + 4) = make_float4(t[4], t[5], t[6], t[7]);
        } else {
          for (int k = 0; k < 8 && e + k < a.n; ++k) a.grad[e + k] = t[k];
        }
      }
    }
  }
}

// fp32 gradients * scale -> bf16 send region (elements beyond n are zero), whole GPU wide and short
__global__ void peer_pack_kernel(const float* __restrict__ grad, __nv_bfloat16* __restrict__ send, long long n, long long padded, float scale) {
  const long long n8 = padded >> 3;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n8; g += (long long)gridDim.x * blockDim.x) {
    const long long e = g << 3;
    float t[8];
    if (e + 8 <= n) {
      const float4 x = *reinterpret_cast<const float4*>(grad + e), y = *reinterpret_cast<const float4*>(grad + e + 4);
      t[0] = x.x; t[1] = x.y; t[2] = x.z; t[3] = x.w; t[4] = y.x; t[5] = y.y; t[6] = y.z; t[7] = y.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) t[k] = e + k < n ? grad[e + k] : 0.f;
    }
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(t[2 * k] * scale, t[2 * k + 1] * scale);
    *reinterpret_cast<uint4*>(send + e) = *reinterpret_cast<const uint4*>(o);
  }
}

// bf16 receive region -> fp32 gradients
__global__ void peer_unpack_kernel(const __nv_bfloat16* __restrict__ recv, float* __restrict__ grad, long long n,
                                   const int* __restrict__ status) {
  // after a give-up of the peer kernel the receive region holds an earlier bucket: leave the gradients alone
  if (sb_failed(status)) return;
  const long long n8 = (n + 7) >> 3;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n8; g += (long long)gridDim.x * blockDim.x) {
    const long long e = g << 3;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(recv + e));     // written by other GPUs
    float t[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    add8(t, v);
    if (e + 8 <= n) {
      *reinterpret_cast<float4*>(grad + e) = make_float4(t[0], t[1], t[2], t[3]);
      *reinterpret_cast<float4*>(grad + e + 4) = make_float4(t[4], t[5], t[6], t[7]);
    } else {
      for (int k = 0; k < 8 && e + k < n; ++k) grad[e + k] = t[k];
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------------------
// Peer phase with bulk copies (opt-in, see sb_peer_allreduce_split).
//
// CTA b owns sub-chunk b of THIS rank's slice.  It walks the sub-chunk in tiles of `tile` bytes through a ring of STAGES
// shared-memory stages; a stage holds the tile of every rank's send region (fetched with cp.async.bulk, an untiled bulk copy
// from peer memory that completes on an mbarrier; no multicast) plus the reduced tile.  The 256 threads sum the `world` tiles
// in fp32, round once to bf16, and thread 0 sends the result to every rank's receive region with bulk stores.  Loads of the
// following STAGES - 1 tiles are in flight while a tile is summed, so a CTA has (STAGES - 1) * (world - 1) * tile bytes on
// the links; four CTAs cover what a 12-CTA register-staged kernel could not.  Same flag protocol as above (CTA b only ever
// waits for CTA b of its peers), same bounded waits.
constexpr int BULK_THREADS = 256;
constexpr int BULK_SMEM = 200 * 1024;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

__global__ void __launch_bounds__(BULK_THREADS) peer_allreduce_bulk_kernel(SbPeerArgs a, int tile_bytes, int stages) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_fail;
  __shared__ __align__(8) unsigned long long bars[16];
  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_fail = 0;
    for (int s = 0; s < stages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  char* my_base = (char*)a.buffers[a.rank];
  const unsigned int* my_flags = reinterpret_cast<const unsigned int*>(my_base + a.flags_off);
  const long long c0 = (long long)b * a.chunk;                              // elements inside the slice
  const long long c1 = min(a.slice, c0 + a.chunk);
  const long long base = (long long)a.rank * a.slice;
  const int tile_elems = tile_bytes / 2;
  const long long ntiles = c1 > c0 ? (c1 - c0 + tile_elems - 1) / tile_elems : 0;
  const int stage_bytes = tile_bytes * (a.world + 1);
  const uint32_t smem0 = (smem_addr(smem_raw) + 127u) & ~127u;

  // the send regions of all ranks are complete (their pack kernels ran before this kernel on their streams)
  signal_peers(a, b, 2u * a.epoch + 1u);
  if (!wait_peers(my_flags, b, a.world, a.rank, 2u * a.epoch + 1u, &s_fail, a.status)) {
    if (tid == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 1);
    return;
  }

  auto issue_loads = [&](long long t) {       // thread 0: fetch tile t of every rank into stage t % stages
    const int s = (int)(t % stages);
    const long long e0 = c0 + t * tile_elems;
    const uint32_t bytes = (uint32_t)(min((long long)tile_elems, c1 - e0) * 2);   // multiple of 16: chunk and slice are of 8
    const uint32_t bar = smem_addr(&bars[s]);
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes * a.world)
                 : "memory");
    for (int q = 0; q < a.world; ++q) {
      const int src_rank = (a.rank + q) % a.world;      // start with the local copy, then walk the ring
      const char* src = (const char*)a.buffers[src_rank] + a.send_off + (base + e0) * 2;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem0 + s * stage_bytes + q * tile_bytes), "l"(src), "r"(bytes), "r"(bar) : "memory");
    }
  };

  long long issued = 0;                       // thread 0: tiles whose loads have been issued
  if (tid == 0)
    for (long long t = 0; t < ntiles && t < stages - 1; ++t, ++issued) issue_loads(t);
  bool ok = true;
  long long done = 0;
  for (long long t = 0; t < ntiles; ++t) {
    const int s = (int)(t % stages);
    const uint32_t par = (uint32_t)((t / stages) & 1);
    // (1) the stage that tile t + stages - 1 will use was consumed in iteration t - 1 (all threads passed its barrier below) and
    //     its result tile has been read by the bulk stores issued then
    if (tid == 0 && t + stages - 1 < ntiles) {
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      issue_loads(t + stages - 1);
      ++issued;
    }
    // (2) wait for tile t (bounded)
    {
      const uint32_t bar = smem_addr(&bars[s]);
      if (!mbar_try(bar, par)) {
        const long long t0 = clock64();
        unsigned int probes = 0;
        while (!mbar_try(bar, par)) {
          if ((++probes & 63u) == 0 && (clock64() - t0 > sb_wait_cycles(a.status) || sb_failed(a.status))) {
            atomicExch(&s_fail, 1);
            break;
          }
        }
      }
    }
    if (__syncthreads_or(s_fail)) { ok = false; break; }
    // (3) sum the world tiles: a thread owns 16 bytes at a time
    const long long e0 = c0 + t * tile_elems;
    const int n16 = (int)(min((long long)tile_elems, c1 - e0) / 8);
    const unsigned char* st = smem_raw + (smem0 - smem_addr(smem_raw)) + (size_t)s * stage_bytes;
    unsigned char* out = const_cast<unsigned char*>(st) + (size_t)a.world * tile_bytes;
    for (int i = tid; i < n16; i += BULK_THREADS) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // fixed summation order by RANK (not by ring position), so that every rank rounds identical sums
      for (int r = 0; r < a.world; ++r) {
        const int q = (r - a.rank + a.world) % a.world;
        add8(acc, *reinterpret_cast<const uint4*>(st + (size_t)q * tile_bytes + (size_t)i * 16));
      }
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      *reinterpret_cast<uint4*>(out + (size_t)i * 16) = *reinterpret_cast<const uint4*>(o);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    // (4) the reduced tile goes to every rank's receive region
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)n16 * 16u;
      for (int q = 0; q < a.world; ++q) {
        const int dst_rank = (a.rank + q) % a.world;
        char* dst = (char*)a.buffers[dst_rank] + a.recv_off + (base + e0) * 2;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     ::"l"(dst), "r"(smem0 + s * stage_bytes + a.world * tile_bytes), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    done = t + 1;
  }
  if (tid == 0) {
    if (!ok) {
      // after a give-up: copies that are still on their way into this CTA's shared memory get one more (bounded) wait each
      for (long long t = done; t < issued; ++t) {
        const uint32_t bar = smem_addr(&bars[t % stages]);
        const uint32_t par = (uint32_t)((t / stages) & 1);
        const long long t0 = clock64();
        while (!mbar_try(bar, par) && clock64() - t0 < sb_wait_cycles(a.status)) { }
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // every store of this CTA has been performed
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  __syncthreads();
  if (!ok) {
    if (tid == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 3);
    return;
  }
  signal_peers(a, b, 2u * a.epoch + 2u);
  if (!wait_peers(my_flags, b, a.world, a.rank, 2u * a.epoch + 2u, &s_fail, a.status)) {
    if (tid == 0) sb_set_status(a.status, SB_TIMEOUT_PEER_FLAG, 2);
    return;
  }
}

}  // namespace

// Bytes of the flag block at the start of a symmetric buffer.
SB_API long long sb_peer_flags_bytes() { return (long long)SB_PEER_MAX_CTAS * SB_PEER_MAX_WORLD * sizeof(unsigned int); }

// Fills the derived fields (slice, chunk) and launches.  `grad` must be 16-byte aligned; the send / recv regions must hold
// slice * world bf16 elements.  Returns 0, a negative code for bad arguments or a positive cudaError_t.
SB_API int sb_peer_allreduce(SbPeerArgs* a, cudaStream_t stream) {
  if (a->world < 1 || a->world > SB_PEER_MAX_WORLD || a->rank < 0 || a->rank >= a->world) return -1;
  if (a->ctas < 1 || a->ctas > SB_PEER_MAX_CTAS || a->n <= 0 || a->epoch == 0) return -1;
  if ((reinterpret_cast<unsigned long long>(a->grad) & 15ull) || (a->send_off & 15) || (a->recv_off & 15) || (a->flags_off & 3)) return -2;
  long long slice = (a->n + a->world - 1) / a->world;
  slice = (slice + 7) / 8 * 8;
  long long chunk = (slice + a->ctas - 1) / a->ctas;
  chunk = (chunk + 7) / 8 * 8;
  a->status = sb_status_ptr();
  if (a->status == nullptr) return -3;
  a->slice = slice;
  a->chunk = chunk;
  peer_allreduce_kernel<true><<<a->ctas, 512, 0, stream>>>(*a);
  return (int)cudaGetLastError();
}

// Same reduction as three launches on `stream`: a wide cast kernel, the peer kernel with its local phases left out, a wide unpack
// kernel.  With the local phases inside the few-block kernel those blocks spend most of their time on local memory at the
// bandwidth of a few SMs; as wide kernels the same bytes take a fraction of a millisecond, squeezed in between the GEMMs.
// `my_base` is this rank's symmetric buffer (the entry of `buffers` for this rank).
SB_API int sb_peer_allreduce_split(SbPeerArgs* a, void* my_base, cudaStream_t stream) {
  if (a->world < 1 || a->world > SB_PEER_MAX_WORLD || a->rank < 0 || a->rank >= a->world || !my_base) return -1;
  if (a->ctas < 1 || a->ctas > SB_PEER_MAX_CTAS || a->n <= 0 || a->epoch == 0) return -1;
  if ((reinterpret_cast<unsigned long long>(a->grad) & 15ull) || (a->send_off & 15) || (a->recv_off & 15) || (a->flags_off & 3)) return -2;
  long long slice = (a->n + a->world - 1) / a->world;
  slice = (slice + 7) / 8 * 8;
  long long chunk = (slice + a->ctas - 1) / a->ctas;
  chunk = (chunk + 7) / 8 * 8;
  a->status = sb_status_ptr();
  if (a->status == nullptr) return -3;
  a->slice = slice;
  a->chunk = chunk;
  const long long padded = slice * a->world;
  __nv_bfloat16* send = reinterpret_cast<__nv_bfloat16*>((char*)my_base + a->send_off);
  const __nv_bfloat16* recv = reinterpret_cast<const __nv_bfloat16*>((char*)my_base + a->recv_off);
  long long blocks = ((padded >> 3) + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  peer_pack_kernel<<<(int)blocks, 256, 0, stream>>>(a->grad, send, a->n, padded, a->scale);
  // The bulk-copy kernel is opt-in (SPEECH_B200_PEER_BULK=1): with its ring of 16 KB tiles a CTA keeps under 50 KB on the
  // links at two ranks, and measured end to end (TDT-0.6B, 2 GPUs) it is slower than the register-staged kernel on 12 CTAs.
  static const bool use_bulk = [] { const char* e = getenv("SPEECH_B200_PEER_BULK"); return e && e[0] == '1'; }();
  if (use_bulk) {
    // stage = (world + 1) tiles; at least three stages in 200 KB, tiles of 1-16 KB
    int tile = (BULK_SMEM - 256) / (4 * (a->world + 1));
    tile = tile >= 16384 ? 16384 : (tile / 1024) * 1024;
    if (tile < 1024) tile = 1024;
    int stages = (BULK_SMEM - 256) / (tile * (a->world + 1));
    if (stages > 8) stages = 8;
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t ae = cudaFuncSetAttribute(peer_allreduce_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BULK_SMEM);
      if (ae != cudaSuccess) return (int)ae;
      attr_set = true;
    }
    // Launched as clusters of two CTAs when their number is even (the cluster is used for nothing else): a cluster of two
    // occupies both SMs of one TPC, so that the persistent GEMMs running beside this kernel, which are themselves built from
    // CTA pairs, lose whole pairs and not one SM out of several pairs.
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(a->ctas, 1, 1);
    cfg.blockDim = dim3(BULK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = BULK_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (a->ctas % 2 == 0) ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, peer_allreduce_bulk_kernel, *a, tile, stages);
    if (le != cudaSuccess) return (int)le;
  } else {
    peer_allreduce_kernel<false><<<a->ctas, 512, 0, stream>>>(*a);
  }
  peer_unpack_kernel<<<(int)blocks, 256, 0, stream>>>(recv, a->grad, a->n, a->status);
  return (int)cudaGetLastError();
}

// Capacity (elements) the send and recv regions need for a bucket of n elements.
SB_API long long sb_peer_padded_elems(long long n, int world) {
  long long slice = (n + world - 1) / world;
  slice = (slice + 7) / 8 * 8;
  return slice * world;
}
