// Kernel template of the persistent bf16 tcgen05 GEMM (see gemm_tcgen05.cu for the interface and the host side).  The kernel is
// instantiated per epilogue class in its own translation unit (gemm_epi_*.cu) so that the classes compile in parallel and each
// kernel carries only the epilogue code it can execute: an epilogue with every feature compiled in is tens of thousands of
// instructions, far more than the instruction caches hold, and the epilogue warps then run at a fraction of their speed.
#pragma once
#include "common.cuh"
#include "gemm_api.h"
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>


constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int NUM_ACC = 2;
constexpr int TILE_BYTES = BLOCK_M * BLOCK_K * 2;  // 16 KiB per operand tile
constexpr int NUM_THREADS = 320;  // warp 0: TMA, warp 1: MMA, warps 2-9: epilogue (two per TMEM lane quarter)
// Tile width BN is a template parameter: 128 (6 stages) or 256 (4 stages; halves shared-memory traffic per flop).
// In pair mode (cta_group::2: two CTAs of a cluster compute one 256 x BN tile) a CTA stages its own 128 rows of A and HALF of
// the B tile, so a stage is 32 KiB at BN = 256 and six of them fit.
constexpr int num_stages(int bn, bool pair = false) { return pair ? 6 : (bn == 256 ? 4 : 6); }
constexpr int stage_bytes(int bn, bool pair = false) { return TILE_BYTES + (pair ? bn / 2 : bn) * BLOCK_K * 2; }
constexpr int EPI_WARPS = 8;
constexpr int EPI_STAGE_BYTES = 4096;   // per epilogue warp: one 32 x 32 fp32 box or two 32 x 32 bf16 boxes
constexpr int smem_bytes(int bn, bool pair = false) {
  return num_stages(bn, pair) * stage_bytes(bn, pair) + 1024 /*align*/ + 1024 /*barriers*/ + EPI_WARPS * EPI_STAGE_BYTES /*store staging*/;
}

// Diagnostic builds (-DSB_GEMM_DIAG) can record clock64() stamps of block 0 into GemmParams::trace: row r, entry i.
#ifdef SB_GEMM_DIAG
#define SB_TRACE_DECL(x) x
#define SB_TRACE(row, i)                                                                                  \
  do {                                                                                                    \
    if (p.trace && blockIdx.x == 0 && (i) < 256) p.trace[(row) * 256 + (i)] = clock64();                  \
  } while (0)
// stamps of the first tile's epilogue chunks (warp 2, lane 0): row 7, entries 8 + 8 * chunk + k
#define SB_TRACE_EPI(k)                                                                                               \
  do {                                                                                                                \
    if (p.trace && blockIdx.x == 0 && warp == 2 && lane == 0 && tr_t == 0)                                            \
      p.trace[7 * 256 + 8 + 8 * (c - half * (BLOCK_N / 64)) + (k)] = clock64();                                       \
  } while (0)
#else
#define SB_TRACE_DECL(x)
#define SB_TRACE(row, i) do { } while (0)
#define SB_TRACE_EPI(k) do { } while (0)
#endif

struct EpilogueArgs {
  void* D;
  const float* bias_f32;
  const __nv_bfloat16* bias_bf16;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* aux;
  __nv_bfloat16* D_pre;
  long long ldd, ldr, ldx, ldp;
  long long d_bs0, d_bs1, r_bs0, r_bs1, x_bs0, x_bs1, p_bs0, p_bs1;
  float alpha, beta;
  int act;       // 0 none, 1 relu, 2 swish, 3 gelu
  int dact;      // 0 none, 1 relu', 2 swish', 3 gelu'  (multiplies by act'(aux))
  int d_is_f32;  // output dtype
  int tma_d;     // D is written through its tensor map: 1 = bulk store, 2 = bulk fp32 add-reduction (beta = 1 / split-K); 0 = by lanes
  int tma_p;     // D_pre is written through its tensor map
  int tma_ragged_d, tma_ragged_p;  // the last, partial column block may also go through the map: its valid part is whole 16-byte
                                   // units (the copy engine clips columns in units of 16 bytes, not of elements)
  unsigned int drop_thresh;  // 0 = no dropout; otherwise the 8-bit threshold of sb_dropout_keep(seed, batch*M*N + m*N + n, thresh)
  float drop_scale;          // 1 / (1 - p)
  unsigned long long drop_seed;
  // GEMM + reduce-scatter: output row m belongs to rank m / peer_rows and is ADDED (fp32 reductions over NVLink peer stores)
  // into that rank's buffer peer_D[rank] at row m % peer_rows.  Null = ordinary local output.
  float* const* peer_D;
  int peer_rows;
};

struct GemmParams {
  int M, N, K;
  int batch0, batch1;
  int kfold;  // > 1: the K loop also runs over this many batch1 entries (sum over batch1 into one output)
  int tiles_m, tiles_n;
  int num_tiles;
  // split-K: every output tile is computed by `ksplit` work items of `kb_per` K blocks each, which add their partial sums to
  // the fp32 output with vector reductions (only for plain accumulating epilogues: D += alpha * A B^T)
  int ksplit, kb_per;
  int num_work;        // num_tiles * ksplit
  int a_peer_rows;     // > 0: all-gather + GEMM: rows [r * a_peer_rows, (r+1) * a_peer_rows) of A live in rank r's memory (peer_a.m[r])
#ifdef SB_GEMM_DIAG
  int debug;           // diagnostic builds only (wrong results): 1 = tensor core alone (operands loaded once), 2 = loads alone (no MMAs)
  long long* trace;    // diagnostic builds only: per-stage / per-tile clock64 stamps of block 0 (8 rows of 256 entries)
#endif
  // rank synchronisation inside the kernel (see SbGemmArgs): flag arrays of all ranks, this rank, the call's epoch
  unsigned int* const* sig_flags;
  unsigned int* sig_counter;
  int sig_world, sig_rank, sig_head, sig_tail;
  unsigned int sig_epoch;
  // staging of remote shards into local memory (all-gather + GEMM; see SbGemmArgs)
  const void* const* stage_src;
  void* stage_dst;
  long long stage_bytes;
  unsigned int* stage_counter;
  EpilogueArgs ep;
  int* status;
};

// Tensor maps of the A operand in every rank's memory (all-gather + GEMM): a tile's rows belong to one rank, and the producer
// simply loads them through that rank's map: an ordinary TMA tile load whose source happens to be peer memory (no multicast).
struct PeerMaps {
  CUtensorMap m[8];
};

namespace {


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false after SB_WAIT_CYCLES, with the status word set.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned int probes = 0;
  while (!mbar_try_wait(bar, parity)) {
    // The give-up test reads the status word from global memory (several hundred cycles): doing it after every failed probe
    // put that latency on the critical path of each producer / consumer hand-over.  Every 64th probe is plenty for a bound.
    if ((++probes & 63u) == 0 && (clock64() - t0 > sb_wait_cycles(status) || sb_failed(status))) {
      sb_set_status(status, code, (int)parity);
      return false;
    }
  }
  return true;
}

// One lane of a converged warp (elect.sync).  The TMA and tcgen05 instructions take their operands from uniform registers; when
// they sit behind `if (lane == 0)` the compiler must treat the branch as divergent and wraps every such instruction in a
// per-lane loop of moves (about 150 cycles per tcgen05.mma, which then bounds the main loop).  Behind elect.sync, in a loop that
// the whole warp runs, it knows that exactly one lane is active.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void flag_store_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int flag_load_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait for a rank's flag to reach `epoch` (flags only grow; the comparison survives wrap-around).
__device__ __forceinline__ bool flag_wait(const unsigned int* p, unsigned int epoch, int* status) {
  if ((int)(flag_load_acquire_sys(p) - epoch) >= 0) return true;
  const long long t0 = clock64();
  unsigned int probes = 0;
  while ((int)(flag_load_acquire_sys(p) - epoch) < 0) {
    if ((++probes & 15u) == 0 && (clock64() - t0 > sb_wait_cycles(status) || sb_failed(status))) {
      sb_set_status(status, SB_TIMEOUT_PEER_FLAG, (int)epoch);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---- CTA-pair helpers (cta_group::2).  The TMA loads carry no multicast: each CTA fetches its own operand slices and reports
// the bytes to the LEADER CTA's barrier (a shared::cluster address), which the .cta_group::2 form of the copy permits.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // relaxed: the arrival only hands a tensor-memory accumulator back (ordered by tcgen05.fence::before_thread_sync); a release
  // at cluster scope would first wait for every earlier global store of the thread to be acknowledged
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* tmap, uint32_t leader_bar, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// one arrival on the barrier at `cluster_addr` (own or peer CTA) once all MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

// Shared-memory matrix descriptor (tcgen05): 128-byte swizzle, version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return fmaxf(v, 0.f);
  if (act == 2) return sb_swish(v);
  if (act == 3) return sb_gelu(v);
  return v;
}
__device__ __forceinline__ float apply_dact(float g, float z, int dact) {
  if (dact == 1) return z > 0.f ? g : 0.f;
  if (dact == 2) return g * sb_dswish(z);
  if (dact == 3) return g * sb_dgelu(z);
  return g;
}

// ---- epilogue stores through the copy engine.  A warp stages a 32-row x 32-column block of its output in shared memory in the
// swizzled layout of the output tensor map (lane l writes row l with 16-byte stores; the XOR pattern makes the eight lanes of a
// store phase hit distinct bank groups), then one elected lane issues a bulk tensor store (or fp32 add-reduction).
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
// bf16 block: rows of 64 bytes, CU_TENSOR_MAP_SWIZZLE_64B (16-byte chunk index XOR bits 7-8 of the address)
__device__ __forceinline__ void stage_bf16_sw64(uint32_t buf, int lane, const float* v) {
  const uint32_t row = buf + (uint32_t)lane * 64u;
  const uint32_t x = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j)
    st_shared_v4(row + ((j ^ x) << 4), pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                 pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
}
// fp32 block: rows of 128 bytes, CU_TENSOR_MAP_SWIZZLE_128B (16-byte chunk index XOR bits 7-9 of the address)
__device__ __forceinline__ void stage_f32_sw128(uint32_t buf, int lane, const float* v) {
  const uint32_t row = buf + (uint32_t)lane * 128u;
  const uint32_t x = (uint32_t)lane & 7u;
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j)
    st_shared_v4(row + ((j ^ x) << 4), __float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                 __float_as_uint(v[4 * j + 3]));
}
// Before a staging buffer is rewritten: the elected lane (elect.sync names the same lane every time) waits until at most
// PENDING of its bulk stores still read shared memory.  The caller follows with __syncwarp().
template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() {
  if (elect_one()) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}
// All lanes: make the staged bytes visible to the copy engine, then one lane issues the store (reduce = fp32 add into the tensor).
__device__ __forceinline__ void bulk_store(const CUtensorMap* tmap, uint32_t src, int c0, int c1, int c2, int c3, bool reduce) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (elect_one()) {
    if (reduce)
      asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                   ::"l"(tmap), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    else
      asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                   ::"l"(tmap), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  }
}

// ---- outputs that cannot go through a tensor map (unaligned layouts, beta other than 0 / 1, peer accumulators).  The 32 x 32
// block is staged as fp32 in the warp's buffer (all bulk stores that read the buffer must have finished: wait 0) and written
// by a short loop in which a lane owns a COLUMN, so that every instruction writes one contiguous row segment.
__device__ __forceinline__ float ld_staged_f32(uint32_t buf, int r, int col) {
  float x;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(buf + (uint32_t)r * 128u + ((((uint32_t)col >> 2) ^ ((uint32_t)r & 7u)) << 4) + (((uint32_t)col & 3u) << 2)) : "memory");
  return x;
}
// mode 0: store; 1: D = v + beta * D (fp32); 2: atomic D += v (fp32)
template <typename T>
__device__ __forceinline__ void store_by_lanes(uint32_t buf, int lane, const float* v, T* dst, long long ld, int rows_valid, int cols_valid,
                                               int mode, float beta) {
  bulk_wait_read<0>();
  __syncwarp();
  stage_f32_sw128(buf, lane, v);
  __syncwarp();
  if (lane < cols_valid) {
#pragma unroll 2
    for (int r = 0; r < rows_valid; ++r) {
      const float x = ld_staged_f32(buf, r, lane);
      T* d = dst + (long long)r * ld + lane;
      if constexpr (sizeof(T) == 2) {
        *d = __float2bfloat16(x);
      } else {
        if (mode == 2) atomicAdd(d, x);
        else *d = (mode == 1 && beta != 0.f) ? x + beta * *d : x;
      }
    }
  }
  __syncwarp();
}
// rows [row_base, row_base + rows_valid) are added into the accumulator of the rank that owns them
__device__ __forceinline__ void add_rows_peer(uint32_t buf, int lane, const float* v, float* const* peer_D, int peer_rows, long long ld,
                                              int row_base, int rows_valid, int col0, int cols_valid) {
  bulk_wait_read<0>();
  __syncwarp();
  stage_f32_sw128(buf, lane, v);
  __syncwarp();
  if (cols_valid >= 32) {
    // four rows per instruction: eight lanes cover the 128 bytes of a row with one 16-byte reduction each
    const int cg = lane & 7;
#pragma unroll 2
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + (lane >> 3);
      if (r < rows_valid) {
        float4 x;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w)
                     : "r"(buf + (uint32_t)r * 128u + (((uint32_t)cg ^ ((uint32_t)r & 7u)) << 4)) : "memory");
        const int row = row_base + r;
        const int owner = row / peer_rows;
        float* d = peer_D[owner] + (long long)(row - owner * peer_rows) * ld + col0 + cg * 4;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
      }
    }
  } else if (lane < cols_valid) {
    for (int r = 0; r < rows_valid; ++r) {
      const int row = row_base + r;
      const int owner = row / peer_rows;
      atomicAdd(peer_D[owner] + (long long)(row - owner * peer_rows) * ld + col0 + lane, ld_staged_f32(buf, r, lane));
    }
  }
  __syncwarp();
}

// Rarely taken paths are kept out of line so that they do not bloat the unrolled epilogue.
__device__ __noinline__ float ld_bias_guard(const float* bf, const __nv_bfloat16* bh, int col, int n) {
  if (col >= n) return 0.f;
  return bf ? __ldg(bf + col) : __bfloat162float(bh[col]);
}
__device__ __noinline__ float ld_bf16_guard(const __nv_bfloat16* p, int j, int n) { return j < n ? __bfloat162float(p[j]) : 0.f; }
__device__ __noinline__ float gelu_call(float x) { return sb_gelu(x); }
__device__ __noinline__ float drop_call(float x, unsigned long long seed, unsigned long long idx, unsigned int thresh, float scale) {
  return sb_dropout_keep(seed, idx, thresh) ? x * scale : 0.f;
}
__device__ __noinline__ float dact_call(float g, float z, int dact) { return apply_dact(g, z, dact); }

// Epilogue classes: the kernel is compiled once per class and carries only that class's code.
//   LEAN: D = alpha * (acc + bias)                                                 (projections, attention, weight gradients)
//   FWD:  bias, pre-activation output, activation, dropout, alpha, residual          (forward linears)
//   BWD:  dropout mask, alpha, act'(aux), residual                                   (input gradients)
constexpr int EPI_LEAN = 0, EPI_FWD = 1, EPI_BWD = 2;

// PAIR = true: launched as clusters of two CTAs; CTA pair c works on 256 x BN tiles (CTA rank r owns rows r*128..r*128+127 of
// the tile in its tensor memory and stages columns r*BN/2.. of B); only rank 0 issues MMAs (tcgen05.mma.cta_group::2).


// Row tile / column tile of work item `rem` (index inside one batch entry).  Ordinary GEMMs walk the row tiles fastest.  With a
// row-sharded A (all-gather + GEMM) the tiles of THIS rank's rows come first, for all column tiles, then the other ranks' rows
// starting with the next rank: the multiplication starts on local data while remote shards are still on their way.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int rem, int tile_m_rows, int& tm, int& tn) {
  if (p.a_peer_rows <= 0 || !p.sig_head) {
    tm = rem % p.tiles_m;
    tn = rem / p.tiles_m;
    return;
  }
  const int own = p.a_peer_rows / tile_m_rows;            // row tiles per rank (shards are whole tiles)
  const int own_items = own * p.tiles_n;
  if (rem < own_items) {
    tm = p.sig_rank * own + rem % own;
    tn = rem / own;
  } else {
    const int r2 = rem - own_items;
    const int others = p.tiles_m - own;                   // row tiles of the other ranks, walked in rotated order
    const int k = r2 % others;
    tm = (p.sig_rank * own + own + k) % p.tiles_m;
    tn = r2 / others;
  }
}

template <bool A_MN, bool B_MN, int BN, bool PAIR, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const __grid_constant__ PeerMaps peer_a, const __grid_constant__ CUtensorMap tmap_d,
                 const __grid_constant__ CUtensorMap tmap_p) {
  constexpr int BLOCK_N = BN;
  constexpr bool HAS_RES = EPI != EPI_LEAN;
  constexpr int NUM_STAGES = num_stages(BN, PAIR);
  constexpr int STAGE_BYTES = stage_bytes(BN, PAIR);
  constexpr int TMEM_COLS = NUM_ACC * BN;
  constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;        // rows of an output tile
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                  // rows (= output columns) of B staged by this CTA
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar_base = base + NUM_STAGES * STAGE_BYTES;
  // barrier slots (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2]; then the TMEM address word
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NUM_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NUM_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NUM_STAGES + NUM_ACC + a); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + NUM_STAGES * STAGE_BYTES + 8 * (2 * NUM_STAGES + 2 * NUM_ACC));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb1 = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int num_kb = num_kb1 * p.kfold;
  const int k_extent = num_kb1 * BLOCK_K;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
#ifdef SB_GEMM_DIAG
  bool diag_once = false;
#endif

  if (threadIdx.x == 32) {
    // descriptor fetches of the first copies start now instead of at the first cp.async.bulk.tensor
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    if (p.ep.tma_d) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_d) : "memory");
    if (p.ep.tma_p) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_p) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < NUM_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), PAIR ? 16 : 8);   // in pair mode the leader's barrier also hears the peer's eight epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // both CTAs' barriers are initialised before either touches the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#ifdef SB_GEMM_DIAG
  if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    p.trace[7 * 256 + 0] = clock64();
    p.trace[7 * 256 + 1] = (long long)gt;
  }
#endif
  if (p.sig_head && blockIdx.x == 0 && threadIdx.x == 64) {
    // this rank's shard was written by earlier work on this stream: tell every rank (this one included) that it is in place
    __threadfence_system();
    for (int r = 0; r < p.sig_world; ++r) flag_store_release_sys(p.sig_flags[r] + p.sig_rank, p.sig_epoch);
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp runs the loop (uniform control flow) and one elected lane issues the copies.  The loop carries
    // (stage, phase) and the K coordinate as counters: no division or modulo per K block.
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      unsigned int ready = p.sig_head ? 0u : 0xffffffffu;   // ranks whose "in place" flag this producer has seen
      SB_TRACE_DECL(int tr_i = 0;)
      for (int w = worker; w < p.num_work && ok; w += num_workers) {
        int tile = w, kb_begin = 0, kb_end = num_kb;
        if (p.ksplit > 1) {
          tile = w / p.ksplit;
          kb_begin = (w - tile * p.ksplit) * p.kb_per;
          kb_end = min(num_kb, kb_begin + p.kb_per);
        }
        const int batch = tile / tiles_per_batch;
        const int rem = tile - batch * tiles_per_batch;
        int tm, tn;
        tile_coords(p, rem, TILE_M, tm, tn);
        const int b1_tile = batch / p.batch0;
        const int b0 = batch - b1_tile * p.batch0;
        const int a_row0 = tm * TILE_M + (int)cta_rank * BLOCK_M;      // first A row (output row) staged by this CTA
        const int b_row0 = tn * BLOCK_N + (int)cta_rank * B_ROWS;      // first B row (output column) staged by this CTA
        // a folded batch1 (kfold > 1) never meets split-K, so its K loop starts at block 0 of entry 0
        int b1 = p.kfold > 1 ? 0 : b1_tile;
        int k0 = kb_begin * BLOCK_K;
        const CUtensorMap* amap = &tmap_a;
        int a_row = a_row0;
        if (!A_MN && !PAIR && p.a_peer_rows > 0) {
          const int owner = a_row0 / p.a_peer_rows;
          amap = &peer_a.m[owner];
          a_row = a_row0 - owner * p.a_peer_rows;
          if (!((ready >> owner) & 1u) && lane == 0) {
            // on a time-out the loads are still issued (from a shard that may be stale; the status word tells the host), so that
            // the barriers complete and the kernel ends in its normal way
            if (p.stage_bytes > 0 && owner != p.sig_rank) {
              // staged mode: every block has copied its slice of the remote shards into local memory
              const long long t0 = clock64();
              unsigned int probes = 0;
              while (*((volatile unsigned int*)p.stage_counter) < gridDim.x) {
                if ((++probes & 15u) == 0 && (clock64() - t0 > sb_wait_cycles(p.status) || sb_failed(p.status))) {
                  sb_set_status(p.status, SB_TIMEOUT_PEER_FLAG, 1000 + owner);
                  break;
                }
              }
              __threadfence();
              asm volatile("fence.proxy.async;" ::: "memory");
              ready = 0xffffffffu;                              // all remote shards are staged at once
            } else {
              flag_wait(p.sig_flags[p.sig_rank] + owner, p.sig_epoch, p.status);
              ready |= 1u << owner;
            }
          }
          ready = __shfl_sync(0xffffffffu, ready, 0);
          // after a give-up no tile is loaded from a shard that may not be in place: the roles end through their bounded waits
          if (__any_sync(0xffffffffu, sb_failed(p.status) ? 1 : 0)) { ok = false; break; }
        }
        for (int n = kb_end - kb_begin; n > 0; --n) {
#ifdef SB_GEMM_DIAG
          if ((p.debug & 15) == 1 && (stage == 0 && phase != 0 || diag_once)) { diag_once = true; continue; }
#endif
          ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, p.status, SB_TIMEOUT_SMEM_EMPTY) ? 1 : 0) != 0;
          if (!ok) break;
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + TILE_BYTES;
          if (!elect_one()) {
            // the other lanes only keep the loop converged
          } else if (PAIR) {
            SB_TRACE(1, tr_i);
            // the leader's barrier counts the bytes of both CTAs; only the leader posts the expectation (and the arrival)
            const uint32_t lbar = mapa_shared(full_bar(stage), 0);
            if (cta_rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
            if (A_MN) {
              tma_load_4d_pair(sa, &tmap_a, lbar, a_row0, k0, b0, b1);
              tma_load_4d_pair(sa + TILE_BYTES / 2, &tmap_a, lbar, a_row0 + 64, k0, b0, b1);
            } else {
              tma_load_4d_pair(sa, &tmap_a, lbar, k0, a_row0, b0, b1);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j)
                tma_load_4d_pair(sb + j * (TILE_BYTES / 2), &tmap_b, lbar, b_row0 + 64 * j, k0, b0, b1);
            } else {
              tma_load_4d_pair(sb, &tmap_b, lbar, k0, b_row0, b0, b1);
            }
          } else {
            SB_TRACE(1, tr_i);
#ifdef SB_GEMM_DIAG
            if ((p.debug & 15) == 3) {   // A operand only (a third of the bytes)
              mbar_expect_tx(full_bar(stage), TILE_BYTES);
              tma_load_4d(sa, &tmap_a, full_bar(stage), k0, a_row0, b0, b1);
            } else
#endif
            {
              mbar_expect_tx(full_bar(stage), STAGE_BYTES);
              if (A_MN) {
                tma_load_4d(sa, &tmap_a, full_bar(stage), a_row0, k0, b0, b1);
                tma_load_4d(sa + TILE_BYTES / 2, &tmap_a, full_bar(stage), a_row0 + 64, k0, b0, b1);
              } else {
                tma_load_4d(sa, amap, full_bar(stage), k0, a_row, b0, b1);
              }
              if (B_MN) {
#pragma unroll
                for (int j = 0; j < BLOCK_N / 64; ++j)
                  tma_load_4d(sb + j * (TILE_BYTES / 2), &tmap_b, full_bar(stage), b_row0 + 64 * j, k0, b0, b1);
              } else {
                tma_load_4d(sb, &tmap_b, full_bar(stage), k0, b_row0, b0, b1);
              }
            }
          }
          if (lane == 0) SB_TRACE(0, tr_i);
          SB_TRACE_DECL(++tr_i;)
          __syncwarp();
          if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
          k0 += BLOCK_K;
          if (k0 >= k_extent) { k0 = 0; ++b1; }   // next entry of a folded batch1 (after the last block otherwise: unused)
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // the whole warp runs the loop; one elected lane issues the MMAs and the commits of a K block
    if (cta_rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                 ((uint32_t)(BLOCK_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
      // descriptors of stage 0; a stage adds STAGE_BYTES >> 4 to the address field and a 16-wide K step adds KADV
      // (K-major: 32 bytes inside the swizzle atom; MN-major: 16 rows of 128 bytes)
      const uint64_t adesc0 = A_MN ? make_desc(base, BLOCK_K * 128, 1024) : make_desc(base, 16, 1024);
      const uint64_t bdesc0 = B_MN ? make_desc(base + TILE_BYTES, BLOCK_K * 128, 1024) : make_desc(base + TILE_BYTES, 16, 1024);
      constexpr uint64_t A_KADV = A_MN ? ((UMMA_K * 128) >> 4) : ((UMMA_K * 2) >> 4);
      constexpr uint64_t B_KADV = B_MN ? ((UMMA_K * 128) >> 4) : ((UMMA_K * 2) >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t aph = 0;
      bool ok = true;
      SB_TRACE_DECL(int tr_i = 0; int tr_t = 0;)
      for (int w = worker; w < p.num_work && ok; w += num_workers) {
        int nkb = num_kb;
        if (p.ksplit > 1) {
          const int kb_begin = (w % p.ksplit) * p.kb_per;
          nkb = min(num_kb, kb_begin + p.kb_per) - kb_begin;
        }
        ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), aph ^ 1u, p.status, SB_TIMEOUT_TMEM_EMPTY) ? 1 : 0) != 0;
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) SB_TRACE(6, tr_t);
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
        uint32_t accumulate = 0u;
        for (int n = nkb; n > 0; --n) {
#ifdef SB_GEMM_DIAG
          if (!((p.debug & 15) == 1 && (stage == 0 && phase != 0 || diag_once)))
#endif
          {
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, p.status, SB_TIMEOUT_SMEM_FULL) ? 1 : 0) != 0;
            if (!ok) break;
          }
#ifdef SB_GEMM_DIAG
          if ((p.debug & 15) == 1 && stage == NUM_STAGES - 1) diag_once = true;
#endif
          tc_fence_after();
          if (lane == 0) SB_TRACE(2, tr_i);
          const uint64_t ad = adesc0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
          const uint64_t bd = bdesc0 + (uint64_t)(stage * (STAGE_BYTES >> 4));
          if (elect_one()) {
#ifdef SB_GEMM_DIAG
          if ((p.debug & 15) < 2)
#endif
          {
#pragma unroll
            for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
              if (PAIR) umma_bf16_pair(d_tmem, ad + k * A_KADV, bd + k * B_KADV, idesc, accumulate);
              else umma_bf16(d_tmem, ad + k * A_KADV, bd + k * B_KADV, idesc, accumulate);
              accumulate = 1u;
            }
          }
#ifdef SB_GEMM_DIAG
          if ((p.debug & 31) == 1) {
            // stages are never recycled in this mode
          } else
#endif
          if (PAIR) {  // the stage is free in BOTH CTAs once these MMAs have read it
            umma_commit_pair(mapa_shared(empty_bar(stage), 0));
            umma_commit_pair(mapa_shared(empty_bar(stage), 1));
          } else {
            umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          }
          }
          if (lane == 0) SB_TRACE(3, tr_i);
          SB_TRACE_DECL(++tr_i;)
          __syncwarp();
          if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok && elect_one()) {
          if (PAIR) {
            umma_commit_pair(mapa_shared(tfull_bar(acc), 0));
            umma_commit_pair(mapa_shared(tfull_bar(acc), 1));
          } else {
            umma_commit(tfull_bar(acc));
          }
        }
        SB_TRACE_DECL(++tr_t;)
        if (++acc == NUM_ACC) { acc = 0; aph ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;            // TMEM lane quarter owned by this warp
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    const EpilogueArgs& e = p.ep;
    if (p.stage_bytes > 0) {
      // Remote shards -> local staging, each byte once: this block copies its slice of every other rank's shard with plain
      // 16-byte peer loads, while the MMA pipeline already works on this rank's own rows.  The eight epilogue warps have
      // nothing else to do until the first accumulator is complete.
      const int te = (int)threadIdx.x - 64;                       // 0 .. 255
      const long long n16 = p.stage_bytes >> 4;
      const long long per = (n16 + gridDim.x - 1) / gridDim.x;
      const long long lo = (long long)blockIdx.x * per;
      const long long hi = lo + per < n16 ? lo + per : n16;
      for (int r = 0; r < p.sig_world; ++r) {
        if (r == p.sig_rank) continue;
        if (te == 0) flag_wait(p.sig_flags[p.sig_rank] + r, p.sig_epoch, p.status);   // rank r's shard is in place
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const uint4* src = reinterpret_cast<const uint4*>(p.stage_src[r]);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.stage_dst) + (long long)r * p.stage_bytes);
        long long i = lo + te;
        for (; i + 3 * 256 < hi; i += 4 * 256) {                   // four loads in flight per thread
          const uint4 v0 = __ldcg(src + i), v1 = __ldcg(src + i + 256), v2 = __ldcg(src + i + 512), v3 = __ldcg(src + i + 768);
          dst[i] = v0; dst[i + 256] = v1; dst[i + 512] = v2; dst[i + 768] = v3;
        }
        for (; i < hi; i += 256) dst[i] = __ldcg(src + i);
      }
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");              // the staged bytes are read back through TMA (async proxy)
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (te == 0) {
        unsigned int old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.stage_counter) : "memory");
        (void)old;
      }
    }
    // this warp's staging area for bulk tensor stores: 4 KiB, 1024-byte aligned (one 32 x 32 fp32 box or two bf16 boxes)
    const uint32_t ebuf = bar_base + 1024u + (uint32_t)(warp - 2) * EPI_STAGE_BYTES;
    int sbuf = 0;
    int acc = 0;
    uint32_t aph = 0;
    bool ok = true;
    SB_TRACE_DECL(int tr_t = 0;)
    for (int w = worker; w < p.num_work && ok; w += num_workers) {
      const int tile = p.ksplit > 1 ? w / p.ksplit : w;
      const int batch = tile / tiles_per_batch;
      const int rem = tile - batch * tiles_per_batch;
      int tm, tn;
      tile_coords(p, rem, TILE_M, tm, tn);
      const int b1 = batch / p.batch0, b0 = batch - b1 * p.batch0;
      const int tile_row0 = tm * TILE_M + (int)cta_rank * BLOCK_M;   // first output row held in this CTA's tensor memory
      // the decision to go on must be warp-uniform: tcgen05.ld below is a warp-collective instruction
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), aph, p.status, SB_TIMEOUT_TMEM_FULL) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) SB_TRACE(4, tr_t);
      const int row_base = tile_row0 + q * 32;                  // first row of this warp's 32-row slab (warp-uniform)
      const int row = row_base + lane;
      const bool row_ok = row < p.M;
      const long long slab_d = (long long)b0 * e.d_bs0 + (long long)b1 * e.d_bs1 + (long long)row_base * e.ldd;
      const long long slab_p = (long long)b0 * e.p_bs0 + (long long)b1 * e.p_bs1 + (long long)row_base * e.ldp;
      const long long r_off = (long long)b0 * e.r_bs0 + (long long)b1 * e.r_bs1 + (long long)row * e.ldr;
      const long long x_off = (long long)b0 * e.x_bs0 + (long long)b1 * e.x_bs1 + (long long)row * e.ldx;
      const int rows_valid = min(32, p.M - row_base);            // warp-uniform; <= 0 when the slab lies outside the output
#pragma unroll 1
      for (int c = half * (BLOCK_N / 64); c < (half + 1) * (BLOCK_N / 64); ++c) {
        const int col0 = tn * BLOCK_N + c * 32;
        if (col0 >= p.N || rows_valid <= 0) continue;             // chunk entirely outside the output (warp-uniform)
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BLOCK_N + c * 32);
        SB_TRACE_EPI(0);
        tmem_ld32(taddr, r);
        const bool full = (col0 + 32 <= p.N);
        // Operands of the epilogue are requested BEFORE the wait on the tensor-memory load, so that the two latencies overlap.
        const __nv_bfloat16* rp = (HAS_RES && e.residual) ? e.residual + r_off + col0 : nullptr;
        const __nv_bfloat16* xp = (EPI == EPI_BWD && e.dact) ? e.aux + x_off + col0 : nullptr;
        const bool vec_b = e.bias_f32 && full && ((((uintptr_t)(e.bias_f32 + col0)) & 15) == 0);
        const bool vec_r = rp && row_ok && full && ((((uintptr_t)rp) & 15) == 0);
        const bool vec_x = xp && row_ok && full && ((((uintptr_t)xp) & 15) == 0);
        float4 bq[8];
        uint4 rq[4], xq[4];
        if (vec_b) {
#pragma unroll
          for (int j = 0; j < 8; ++j) bq[j] = __ldg(reinterpret_cast<const float4*>(e.bias_f32 + col0) + j);
        }
        if (HAS_RES && vec_r) {
#pragma unroll
          for (int j = 0; j < 4; ++j) rq[j] = *(reinterpret_cast<const uint4*>(rp) + j);
        }
        if (EPI == EPI_BWD && vec_x) {
#pragma unroll
          for (int j = 0; j < 4; ++j) xq[j] = *(reinterpret_cast<const uint4*>(xp) + j);
        }
        tmem_ld_wait();
        SB_TRACE_EPI(1);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        // the bias depends on the column only
        if (vec_b) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[4 * j] += bq[j].x; v[4 * j + 1] += bq[j].y; v[4 * j + 2] += bq[j].z; v[4 * j + 3] += bq[j].w;
          }
        } else if (e.bias_f32 || e.bias_bf16) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += ld_bias_guard(e.bias_f32, e.bias_bf16, col0 + j, p.N);
        }
        if (EPI == EPI_FWD) {
          // pre-activation (acc + bias)
          if (e.D_pre) {
            if (e.tma_p && (full || e.tma_ragged_p)) {
              bulk_wait_read<1>(); __syncwarp();
              stage_bf16_sw64(ebuf + (uint32_t)sbuf * 2048u, lane, v);
              bulk_store(&tmap_p, ebuf + (uint32_t)sbuf * 2048u, col0, row_base, b0, b1, false);
              sbuf ^= 1;
            } else {
              store_by_lanes(ebuf, lane, v, e.D_pre + slab_p + col0, e.ldp, rows_valid, p.N - col0, 0, 0.f);
            }
          }
          if (e.act == 2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = sb_swish(v[j]);
          } else if (e.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          } else if (e.act == 3) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_call(v[j]);
          }
        }
        if (EPI != EPI_LEAN && e.drop_thresh) {
          const unsigned long long base = ((unsigned long long)batch * p.M + row) * (unsigned long long)p.N + col0;
          if ((p.N & 3) == 0) {
            // rows start on a multiple of four elements: one hash per group of four columns
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const unsigned int h = sb_dropout_hash4(e.drop_seed, (base >> 2) + g);
#pragma unroll
              for (int u = 0; u < 4; ++u) v[4 * g + u] = sb_dropout_keep_in(h, u, e.drop_thresh) ? v[4 * g + u] * e.drop_scale : 0.f;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = drop_call(v[j], e.drop_seed, base + j, e.drop_thresh, e.drop_scale);
          }
        }
        if (e.alpha != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
        }
        if (EPI == EPI_BWD) {
          if (vec_x) {
            if (e.dact == 2) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&xq[j]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 z = __bfloat1622float2(t[u]);
                  v[8 * j + 2 * u] *= sb_dswish(z.x);
                  v[8 * j + 2 * u + 1] *= sb_dswish(z.y);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&xq[j]);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 z = __bfloat1622float2(t[u]);
                  v[8 * j + 2 * u] = dact_call(v[8 * j + 2 * u], z.x, e.dact);
                  v[8 * j + 2 * u + 1] = dact_call(v[8 * j + 2 * u + 1], z.y, e.dact);
                }
              }
            }
          } else if (xp && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = dact_call(v[j], ld_bf16_guard(xp, j, p.N - col0), e.dact);
          }
        }
        if (HAS_RES) {
          if (vec_r) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&rq[j]);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 z = __bfloat1622float2(t[u]);
                v[8 * j + 2 * u] += z.x;
                v[8 * j + 2 * u + 1] += z.y;
              }
            }
          } else if (rp && row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += ld_bf16_guard(rp, j, p.N - col0);
          }
        }
        // ---- output
        SB_TRACE_EPI(2);
        if (e.tma_d && (full || e.tma_ragged_d)) {
          // registers -> swizzled shared-memory box -> one bulk tensor store (or reduction) per 32 x 32 block; the copy engine clips
          // rows beyond M and columns beyond N
          if (e.d_is_f32) {
            bulk_wait_read<0>(); __syncwarp();
            stage_f32_sw128(ebuf, lane, v);
            bulk_store(&tmap_d, ebuf, col0, row_base, b0, b1, e.tma_d == 2);
          } else {
            bulk_wait_read<1>(); __syncwarp();
            SB_TRACE_EPI(3);
            stage_bf16_sw64(ebuf + (uint32_t)sbuf * 2048u, lane, v);
            SB_TRACE_EPI(4);
            bulk_store(&tmap_d, ebuf + (uint32_t)sbuf * 2048u, col0, row_base, b0, b1, false);
            SB_TRACE_EPI(5);
            sbuf ^= 1;
          }
        } else if (e.peer_D) {
          // GEMM + reduce-scatter: rows of this block belong to their owner rank's accumulator; plain P2P reductions over NVLink,
          // 128 contiguous bytes per row and instruction
          add_rows_peer(ebuf, lane, v, e.peer_D, e.peer_rows, e.ldd, row_base, rows_valid, col0, p.N - col0);
        } else if (e.d_is_f32) {
          // mode 1: D = v + beta * D;  mode 2: D += v atomically (partial sums of K slices)
          store_by_lanes(ebuf, lane, v, reinterpret_cast<float*>(e.D) + slab_d + col0, e.ldd, rows_valid, p.N - col0,
                         p.ksplit > 1 ? 2 : 1, e.beta);
        } else {
          store_by_lanes(ebuf, lane, v, reinterpret_cast<__nv_bfloat16*>(e.D) + slab_d + col0, e.ldd, rows_valid, p.N - col0, 0, 0.f);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));   // the leader's MMA warp waits for both CTAs
        else mbar_arrive(tempty_bar(acc));
      }
      if (warp == 2 && lane == 0) SB_TRACE(5, tr_t);
      SB_TRACE_DECL(++tr_t;)
      if (++acc == NUM_ACC) { acc = 0; aph ^= 1u; }
    }
    // every bulk store of this warp has completed (not only released its staging buffer) before the block can exit
    if (elect_one()) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }

  // ------------------------------------------------------------------ common exit
  if (p.sig_tail && warp >= 2) __threadfence_system();   // this thread's reductions into peer memory are performed before the block reports
  tc_fence_before();
  __syncthreads();
  if (p.stage_bytes > 0 && threadIdx.x == 0) {
    // the last block out clears both staging counters for the next call
    unsigned int gone;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(gone) : "l"(p.stage_counter + 1) : "memory");
    if (gone == gridDim.x - 1) {
      *((volatile unsigned int*)p.stage_counter) = 0u;
      *((volatile unsigned int*)(p.stage_counter + 1)) = 0u;
      __threadfence();
    }
  }
  if (p.sig_tail && threadIdx.x == 0) {
    unsigned int done;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(done) : "l"(p.sig_counter) : "memory");
    if (done == gridDim.x - 1) {
      // last block of this rank: every block's reductions are ordered before this point; publish "landed" to every rank
      *((volatile unsigned int*)p.sig_counter) = 0u;
      __threadfence_system();
      for (int r = 0; r < p.sig_world; ++r) flag_store_release_sys(p.sig_flags[r] + 8 + p.sig_rank, p.sig_epoch);
    }
  }
#ifdef SB_GEMM_DIAG
  if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    p.trace[7 * 256 + 2] = clock64();
    p.trace[7 * 256 + 3] = (long long)gt;
  }
#endif
  if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while its partner may still reach into it
  tc_fence_after();
  if (warp == 1) {
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// Launches the kernel variant `variant` (bit 0: B MN-major, bit 1: A MN-major, bit 2: 256-wide tiles, bit 3: CTA pairs) of this
// translation unit's epilogue class.  `grid` counts CTAs (pairs are launched as clusters of two).
template <int EPI>
int launch_gemm_variant(int variant, int grid, bool pair, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                        const GemmParams& p, const PeerMaps& pm, const CUtensorMap& td, const CUtensorMap& tp) {
  void (*kern)(const CUtensorMap, const CUtensorMap, const GemmParams, const PeerMaps, const CUtensorMap, const CUtensorMap) = nullptr;
  switch (variant) {
    case 0: kern = gemm_bf16_kernel<false, false, 128, false, EPI>; break;
    case 1: kern = gemm_bf16_kernel<false, true, 128, false, EPI>; break;
    case 2: kern = gemm_bf16_kernel<true, false, 128, false, EPI>; break;
    case 3: kern = gemm_bf16_kernel<true, true, 128, false, EPI>; break;
    case 4: kern = gemm_bf16_kernel<false, false, 256, false, EPI>; break;
    case 5: kern = gemm_bf16_kernel<false, true, 256, false, EPI>; break;
    case 6: kern = gemm_bf16_kernel<true, false, 256, false, EPI>; break;
    case 7: kern = gemm_bf16_kernel<true, true, 256, false, EPI>; break;
    case 12: kern = gemm_bf16_kernel<false, false, 256, true, EPI>; break;
    case 13: kern = gemm_bf16_kernel<false, true, 256, true, EPI>; break;
    case 14: kern = gemm_bf16_kernel<true, false, 256, true, EPI>; break;
    case 15: kern = gemm_bf16_kernel<true, true, 256, true, EPI>; break;
    default: return -10;
  }
  const int bn = (variant & 4) ? 256 : 128;
  const int smem = smem_bytes(bn, pair);
  static bool attr_set[16] = {};
  if (!attr_set[variant]) {
    cudaError_t ae = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ae != cudaSuccess) return (int)ae;
    attr_set[variant] = true;
  }
  // Staged all-gather + GEMM: tiles of remote rows wait until EVERY block has copied its slice, a grid-wide dependency.  A
  // cooperative launch starts the grid only when all of its blocks can be resident together, whatever else runs on the device.
  const bool coop = p.stage_bytes > 0;
  if (pair || coop) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pair) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 2;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = 1;
      ++na;
    }
    if (coop) {
      attr[na].id = cudaLaunchAttributeCooperative;
      attr[na].val.cooperative = 1;
      ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, p, pm, td, tp);
  }
  kern<<<grid, NUM_THREADS, smem, stream>>>(ta, tb, p, pm, td, tp);
  return (int)cudaGetLastError();
}

}  // namespace

// One definition per epilogue class, each in its own translation unit (gemm_epi_lean.cu, gemm_epi_fwd.cu, gemm_epi_bwd.cu).
int sb_gemm_launch_lean(int variant, int grid, bool pair, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                        const GemmParams& p, const PeerMaps& pm, const CUtensorMap& td, const CUtensorMap& tp);
int sb_gemm_launch_fwd(int variant, int grid, bool pair, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                       const GemmParams& p, const PeerMaps& pm, const CUtensorMap& td, const CUtensorMap& tp);
int sb_gemm_launch_bwd(int variant, int grid, bool pair, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                       const GemmParams& p, const PeerMaps& pm, const CUtensorMap& td, const CUtensorMap& tp);
