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
#include "common.cuh"
#include "gemm_api.h"
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace {

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
constexpr int EPI_ROW_BYTES = 80;   // 32 bf16 (64 B) + 16 B pad: conflict-free 16-byte writes by row and reads by 4-lane groups
constexpr int EPI_STAGE_BYTES = 32 * EPI_ROW_BYTES;
constexpr int smem_bytes(int bn, bool pair = false) {
  return num_stages(bn, pair) * stage_bytes(bn, pair) + 1024 /*align*/ + 256 /*barriers*/ + EPI_WARPS * EPI_STAGE_BYTES /*store staging*/;
}

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
  int stage_d;   // 1: bf16 D rows are 16-byte aligned at every 32-column block: store through the shared-memory transpose
  int stage_p;   // same for D_pre
  unsigned int drop_thresh;  // 0 = no dropout; otherwise keep iff sb_dropout_keep(seed, batch*M*N + m*N + n, thresh)
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
  long long num_tiles;
  // split-K: every output tile is computed by `ksplit` work items of `kb_per` K blocks each, which add their partial sums to
  // the fp32 output with vector reductions (only for plain accumulating epilogues: D += alpha * A B^T)
  int ksplit, kb_per;
  long long num_work;  // num_tiles * ksplit
  int a_peer_rows;     // > 0: all-gather + GEMM: rows [r * a_peer_rows, (r+1) * a_peer_rows) of A live in rank r's memory (peer_a.m[r])
  int debug;           // diagnostics only (wrong results): 1 = tensor core alone (operands loaded once), 2 = loads alone (no MMAs)
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
    if ((++probes & 63u) == 0 && (clock64() - t0 > SB_WAIT_CYCLES || sb_failed(status))) {
      sb_set_status(status, code, (int)parity);
      return false;
    }
  }
  return true;
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
    if ((++probes & 15u) == 0 && (clock64() - t0 > SB_WAIT_CYCLES || sb_failed(status))) {
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
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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

// Warp-level store of a 32 x 32 bf16 block: lane l holds row l (32 values); the block is transposed through shared
// memory so that every store instruction writes 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
__device__ __forceinline__ void stage_store_32x32(uint8_t* st, int lane, const float* v, __nv_bfloat16* dst_row0, long long ld,
                                                  int rows_valid) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __align__(16) __nv_bfloat162 t[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) t[u] = __floats2bfloat162_rn(v[8 * j + 2 * u], v[8 * j + 2 * u + 1]);
    *reinterpret_cast<uint4*>(st + lane * EPI_ROW_BYTES + j * 16) = *reinterpret_cast<const uint4*>(t);
  }
  __syncwarp();
  const int ch = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2);
    const uint4 val = *reinterpret_cast<const uint4*>(st + r * EPI_ROW_BYTES + ch * 16);
    if (r < rows_valid) *reinterpret_cast<uint4*>(dst_row0 + (long long)r * ld + ch * 8) = val;
  }
  __syncwarp();
}

// PAIR = true: launched as clusters of two CTAs; CTA pair c works on 256 x BN tiles (CTA rank r owns rows r*128..r*128+127 of
// the tile in its tensor memory and stages columns r*BN/2.. of B); only rank 0 issues MMAs (tcgen05.mma.cta_group::2).
// Tensor maps of the A operand in every rank's memory (all-gather + GEMM): a tile's rows belong to one rank, and the producer
// simply loads them through that rank's map — an ordinary TMA tile load whose source happens to be peer memory (no multicast).
struct PeerMaps {
  CUtensorMap m[8];
};

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

template <bool A_MN, bool B_MN, int BN, bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const __grid_constant__ PeerMaps peer_a) {
  constexpr int BLOCK_N = BN;
  constexpr int NUM_STAGES = num_stages(BN, PAIR);
  constexpr int STAGE_BYTES = stage_bytes(BN, PAIR);
  constexpr int TMEM_COLS = NUM_ACC * BN;
  constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;        // rows of an output tile
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                  // rows (= output columns) of B staged by this CTA
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const long long worker = PAIR ? (long long)(blockIdx.x >> 1) : (long long)blockIdx.x;
  const long long num_workers = PAIR ? (long long)(gridDim.x >> 1) : (long long)gridDim.x;
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

  if (p.sig_head && blockIdx.x == 0 && threadIdx.x == 64) {
    // this rank's shard was written by earlier work on this stream: tell every rank (this one included) that it is in place
    __threadfence_system();
    for (int r = 0; r < p.sig_world; ++r) flag_store_release_sys(p.sig_flags[r] + p.sig_rank, p.sig_epoch);
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      unsigned int ready = p.sig_head ? 0u : 0xffffffffu;   // ranks whose "in place" flag this producer has seen
      for (long long w = worker; w < p.num_work && ok; w += num_workers) {
        const long long tile = p.ksplit > 1 ? w / p.ksplit : w;
        const int kb_begin = p.ksplit > 1 ? (int)(w % p.ksplit) * p.kb_per : 0;
        const int kb_end = p.ksplit > 1 ? min(num_kb, kb_begin + p.kb_per) : num_kb;
        const int batch = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
        const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
        int tm, tn;
        tile_coords(p, rem, TILE_M, tm, tn);
        const int b0 = batch % p.batch0;
        const int a_row0 = tm * TILE_M + (int)cta_rank * BLOCK_M;      // first A row (output row) staged by this CTA
        const int b_row0 = tn * BLOCK_N + (int)cta_rank * B_ROWS;      // first B row (output column) staged by this CTA
        for (int kbt = kb_begin; kbt < kb_end; ++kbt, ++it) {
          const int kb = kbt % num_kb1;
          const int b1 = p.kfold > 1 ? kbt / num_kb1 : batch / p.batch0;
          const int s = (int)(it % NUM_STAGES);
          const uint32_t ph = (uint32_t)((it / NUM_STAGES) & 1);
          if ((p.debug & 15) == 1 && it >= NUM_STAGES) continue;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, p.status, SB_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + TILE_BYTES;
          if (PAIR) {
            // the leader's barrier counts the bytes of both CTAs; only the leader posts the expectation (and the arrival)
            const uint32_t lbar = mapa_shared(full_bar(s), 0);
            if (cta_rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
            if (A_MN) {
              tma_load_4d_pair(sa, &tmap_a, lbar, a_row0, kb * BLOCK_K, b0, b1);
              tma_load_4d_pair(sa + TILE_BYTES / 2, &tmap_a, lbar, a_row0 + 64, kb * BLOCK_K, b0, b1);
            } else {
              tma_load_4d_pair(sa, &tmap_a, lbar, kb * BLOCK_K, a_row0, b0, b1);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j)
                tma_load_4d_pair(sb + j * (TILE_BYTES / 2), &tmap_b, lbar, b_row0 + 64 * j, kb * BLOCK_K, b0, b1);
            } else {
              tma_load_4d_pair(sb, &tmap_b, lbar, kb * BLOCK_K, b_row0, b0, b1);
            }
          } else if ((p.debug & 15) == 3) {   // diagnostics: A operand only (a third of the bytes), no MMAs
            mbar_expect_tx(full_bar(s), TILE_BYTES);
            tma_load_4d(sa, &tmap_a, full_bar(s), kb * BLOCK_K, a_row0, b0, b1);
          } else {
            mbar_expect_tx(full_bar(s), STAGE_BYTES);
            if (A_MN) {
              tma_load_4d(sa, &tmap_a, full_bar(s), a_row0, kb * BLOCK_K, b0, b1);
              tma_load_4d(sa + TILE_BYTES / 2, &tmap_a, full_bar(s), a_row0 + 64, kb * BLOCK_K, b0, b1);
            } else if (p.a_peer_rows > 0) {
              const int owner = a_row0 / p.a_peer_rows;
              if (!((ready >> owner) & 1u)) {
                // the expectation is already posted: on a time-out the load is still issued (from a shard that may be stale; the
                // status word tells the host), so that the barrier completes and the kernel ends in its normal way
                if (p.stage_bytes > 0 && owner != p.sig_rank) {
                  // staged mode: every block has copied its slice of the remote shards into local memory
                  const long long t0 = clock64();
                  unsigned int probes = 0;
                  while (*((volatile unsigned int*)p.stage_counter) < gridDim.x) {
                    if ((++probes & 15u) == 0 && (clock64() - t0 > SB_WAIT_CYCLES || sb_failed(p.status))) {
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
              tma_load_4d(sa, &peer_a.m[owner], full_bar(s), kb * BLOCK_K, a_row0 - owner * p.a_peer_rows, b0, b1);
            } else {
              tma_load_4d(sa, &tmap_a, full_bar(s), kb * BLOCK_K, a_row0, b0, b1);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BLOCK_N / 64; ++j)
                tma_load_4d(sb + j * (TILE_BYTES / 2), &tmap_b, full_bar(s), b_row0 + 64 * j, kb * BLOCK_K, b0, b1);
            } else {
              tma_load_4d(sb, &tmap_b, full_bar(s), kb * BLOCK_K, b_row0, b0, b1);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BLOCK_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
      long long it = 0;
      long long tcount = 0;
      bool ok = true;
      for (long long w = worker; w < p.num_work && ok; w += num_workers, ++tcount) {
        const int kb_begin = p.ksplit > 1 ? (int)(w % p.ksplit) * p.kb_per : 0;
        const int kb_end = p.ksplit > 1 ? min(num_kb, kb_begin + p.kb_per) : num_kb;
        const int acc = (int)(tcount % NUM_ACC);
        const uint32_t aph = (uint32_t)((tcount / NUM_ACC) & 1);
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u, p.status, SB_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = (int)(it % NUM_STAGES);
          const uint32_t ph = (uint32_t)((it / NUM_STAGES) & 1);
          if (!((p.debug & 15) == 1 && it >= NUM_STAGES)) {
            if (!mbar_wait(full_bar(s), ph, p.status, SB_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            // K-major: advance 32 bytes inside the swizzle atom; MN-major: advance 16 rows of 128 bytes.
            const uint64_t ad = A_MN ? make_desc(sa + k * (UMMA_K * 128), BLOCK_K * 128, 1024)
                                     : make_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_desc(sb + k * (UMMA_K * 128), BLOCK_K * 128, 1024)
                                     : make_desc(sb + k * (UMMA_K * 2), 16, 1024);
            if ((p.debug & 15) >= 2) continue;
            if (PAIR) umma_bf16_pair(d_tmem, ad, bd, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
            else umma_bf16(d_tmem, ad, bd, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          if ((p.debug & 31) == 1) {
            // stages are never recycled in this mode
          } else if (PAIR) {  // the stage is free in BOTH CTAs once these MMAs have read it
            umma_commit_pair(mapa_shared(empty_bar(s), 0));
            umma_commit_pair(mapa_shared(empty_bar(s), 1));
          } else {
            umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
          }
        }
        if (ok) {
          if (PAIR) {
            umma_commit_pair(mapa_shared(tfull_bar(acc), 0));
            umma_commit_pair(mapa_shared(tfull_bar(acc), 1));
          } else {
            umma_commit(tfull_bar(acc));
          }
        }
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
    uint8_t* stage = smem + NUM_STAGES * STAGE_BYTES + 256 + (warp - 2) * EPI_STAGE_BYTES;
    long long tcount = 0;
    bool ok = true;
    for (long long w = worker; w < p.num_work && ok; w += num_workers, ++tcount) {
      const long long tile = p.ksplit > 1 ? w / p.ksplit : w;
      const int batch = (int)(tile / ((long long)p.tiles_m * p.tiles_n));
      const int rem = (int)(tile % ((long long)p.tiles_m * p.tiles_n));
      int tm, tn;
      tile_coords(p, rem, TILE_M, tm, tn);
      const int b0 = batch % p.batch0, b1 = batch / p.batch0;
      const int tile_row0 = tm * TILE_M + (int)cta_rank * BLOCK_M;   // first output row held in this CTA's tensor memory
      const int acc = (int)(tcount % NUM_ACC);
      const uint32_t aph = (uint32_t)((tcount / NUM_ACC) & 1);
      // the decision to go on must be warp-uniform: tcgen05.ld below is a warp-collective instruction
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), aph, p.status, SB_TIMEOUT_TMEM_FULL) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int row = tile_row0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long d_off = e.peer_D ? (long long)(row % e.peer_rows) * e.ldd
                                       : (long long)b0 * e.d_bs0 + (long long)b1 * e.d_bs1 + (long long)row * e.ldd;
      // with a scattered output the owner's buffer replaces D (rows beyond M never store, so the index stays in range)
      float* const peer_base = (e.peer_D && row_ok) ? e.peer_D[row / e.peer_rows] : nullptr;
      const long long r_off = (long long)b0 * e.r_bs0 + (long long)b1 * e.r_bs1 + (long long)row * e.ldr;
      const long long x_off = (long long)b0 * e.x_bs0 + (long long)b1 * e.x_bs1 + (long long)row * e.ldx;
      const long long p_off = (long long)b0 * e.p_bs0 + (long long)b1 * e.p_bs1 + (long long)row * e.ldp;
#pragma unroll 1
      for (int c = half * (BLOCK_N / 64); c < (half + 1) * (BLOCK_N / 64); ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BLOCK_N + c * 32);
        tmem_ld32(taddr, r);
        tmem_ld_wait();
        const int col0 = tn * BLOCK_N + c * 32;
        const bool full = (col0 + 32 <= p.N);
        const int row_base = tile_row0 + q * 32;                  // first row of this warp's 32-row slab
        const int rows_valid = min(32, p.M - row_base);           // warp-uniform
        const long long slab_d = (long long)b0 * e.d_bs0 + (long long)b1 * e.d_bs1 + (long long)row_base * e.ldd;
        const long long slab_p = (long long)b0 * e.p_bs0 + (long long)b1 * e.p_bs1 + (long long)row_base * e.ldp;
        const bool st_d = e.stage_d && full && rows_valid > 0;    // warp-uniform decisions
        const bool st_p = e.stage_p && full && rows_valid > 0 && e.D_pre != nullptr;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        // the bias depends on the column only: add it once, for all lanes, before the stores and the activation
        if (col0 < p.N) {
          if (e.bias_f32) {
            if (full && ((((uintptr_t)(e.bias_f32 + col0)) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 bv = __ldg(reinterpret_cast<const float4*>(e.bias_f32 + col0) + j);
                v[4 * j] += bv.x; v[4 * j + 1] += bv.y; v[4 * j + 2] += bv.z; v[4 * j + 3] += bv.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (full || col0 + j < p.N) v[j] += __ldg(e.bias_f32 + col0 + j);
            }
          } else if (e.bias_bf16) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += __bfloat162float(e.bias_bf16[col0 + j]);
          }
        }
        // pre-activation (acc + bias) stored coalesced: all lanes take part, rows beyond M are masked in the helper
        if (st_p) stage_store_32x32(stage, lane, v, e.D_pre + slab_p + col0, e.ldp, rows_valid);
        if (row_ok && col0 < p.N) {
          if (e.D_pre && !st_p) {
            __nv_bfloat16* dp = e.D_pre + p_off + col0;
            if (full && ((((uintptr_t)dp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __align__(16) __nv_bfloat162 t[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) t[u] = __floats2bfloat162_rn(v[j + 2 * u], v[j + 2 * u + 1]);
                *reinterpret_cast<uint4*>(dp + j) = *reinterpret_cast<uint4*>(t);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dp[j] = __float2bfloat16(v[j]);
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
            for (int j = 0; j < 32; ++j) v[j] = sb_gelu(v[j]);
          }
          if (e.drop_thresh) {
            const unsigned long long base = ((unsigned long long)batch * p.M + row) * (unsigned long long)p.N + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = sb_dropout_keep(e.drop_seed, base + j, e.drop_thresh) ? v[j] * e.drop_scale : 0.f;
          }
          if (e.alpha != 1.f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= e.alpha;
          }
          if (e.dact) {
            const __nv_bfloat16* xp = e.aux + x_off + col0;
            if (full && ((((uintptr_t)xp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 raw4 = *reinterpret_cast<const uint4*>(xp + j);
                const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&raw4);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  float2 z = __bfloat1622float2(t[u]);
                  v[j + 2 * u] = apply_dact(v[j + 2 * u], z.x, e.dact);
                  v[j + 2 * u + 1] = apply_dact(v[j + 2 * u + 1], z.y, e.dact);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] = apply_dact(v[j], __bfloat162float(xp[j]), e.dact);
            }
          }
          if (e.residual) {
            const __nv_bfloat16* rp = e.residual + r_off + col0;
            if (full && ((((uintptr_t)rp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 raw4 = *reinterpret_cast<const uint4*>(rp + j);
                const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&raw4);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  float2 z = __bfloat1622float2(t[u]);
                  v[j + 2 * u] += z.x;
                  v[j + 2 * u + 1] += z.y;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
            }
          }
          if (e.d_is_f32 && (p.ksplit > 1 || e.peer_D)) {
            // partial sum of one K slice (or of one rank's K shard): D += v.  The host only takes this path for epilogues of
            // exactly this form; with peer_D the destination is another GPU's memory, reached by plain P2P reductions.
            float* dp = (e.peer_D ? peer_base : reinterpret_cast<float*>(e.D)) + d_off + col0;
            if (full && ((((uintptr_t)dp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dp + j), "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]),
                             "f"(v[j + 3])
                             : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) atomicAdd(dp + j, v[j]);
            }
          } else if (e.d_is_f32) {
            float* dp = reinterpret_cast<float*>(e.D) + d_off + col0;
            if (full && ((((uintptr_t)dp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (e.beta != 0.f) {
                  float4 old = *reinterpret_cast<const float4*>(dp + j);
                  o.x += e.beta * old.x; o.y += e.beta * old.y; o.z += e.beta * old.z; o.w += e.beta * old.w;
                }
                *reinterpret_cast<float4*>(dp + j) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dp[j] = v[j] + (e.beta != 0.f ? e.beta * dp[j] : 0.f);
            }
          } else if (!st_d) {
            __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(e.D) + d_off + col0;
            if (full && ((((uintptr_t)dp) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __align__(16) __nv_bfloat162 t[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) t[u] = __floats2bfloat162_rn(v[j + 2 * u], v[j + 2 * u + 1]);
                *reinterpret_cast<uint4*>(dp + j) = *reinterpret_cast<uint4*>(t);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dp[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if (st_d) stage_store_32x32(stage, lane, v, reinterpret_cast<__nv_bfloat16*>(e.D) + slab_d + col0, e.ldd, rows_valid);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));   // the leader's MMA warp waits for both CTAs
        else mbar_arrive(tempty_bar(acc));
      }
    }
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
  if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while its partner may still reach into it
  tc_fence_after();
  if (warp == 1) {
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

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

bool g_attr_set[16] = {};

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
  // 256-wide tiles when the problem has enough of them to fill the machine, else 128-wide
  // split-K is possible when the epilogue is exactly D(fp32) += alpha * A B^T: weight gradients (long K, few output tiles)
  const bool can_split = a->d_is_f32 && a->beta == 1.f && !a->bias && !a->residual && !a->aux && !a->D_pre && a->act == 0 &&
                         a->drop_p <= 0.f && !a->fold_batch1 && a->ksplit >= 0;
  int bn = a->tile_n;
  if (bn != 128 && bn != 256 && can_split && a->N >= 256 && a->K >= 24 * BLOCK_K) {
    bn = 256;  // K slices restore the parallelism that wide tiles give up
  } else if (bn != 128 && bn != 256) {
    const long long t256 = (long long)((a->M + BLOCK_M - 1) / BLOCK_M) * ((a->N + 255) / 256) * a->batch0 *
                           (a->fold_batch1 ? 1 : a->batch1);
    bn = (a->N >= 256 && t256 >= (long long)sb_num_sms() * 3 / 4) ? 256 : 128;
  }
  // CTA pairs (cta_group::2, 256 x 256 tiles, half the B traffic per SM) for large plain-layout problems; opt-in while the path
  // is being qualified: SbGemmArgs.pair = 1, or the environment variable SPEECH_B200_GEMM_PAIR=1 for every eligible GEMM
  static const bool env_pair = [] { const char* e = getenv("SPEECH_B200_GEMM_PAIR"); return e && e[0] == '1'; }();
  const bool pair = bn == 256 && a->M > 128 && (a->pair == 1 || (a->pair == 0 && env_pair));
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
  p.num_tiles = (long long)p.tiles_m * p.tiles_n * a->batch0 * (a->fold_batch1 ? 1 : a->batch1);
  p.ksplit = 1;
  {
    const int num_kb = (a->K + BLOCK_K - 1) / BLOCK_K;
    const int sms = pair ? sb_num_sms() / 2 : sb_num_sms();   // parallel workers: CTA pairs or CTAs
    if (a->ksplit > 1 && can_split) {
      p.ksplit = a->ksplit < num_kb ? a->ksplit : num_kb;
    } else if (can_split && a->ksplit == 0 && p.num_tiles < (long long)sms * 3 / 4) {
      // pick the split whose work-item count fills whole waves best; a slice keeps at least 12 K blocks (768 elements)
      double best = (double)p.num_tiles / sms;  // efficiency of one partial wave
      for (int s = 2; s <= 8 && num_kb / s >= 12; ++s) {
        const long long items = p.num_tiles * s;
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
  static const int env_debug = [] { const char* e = getenv("SPEECH_B200_GEMM_DEBUG"); return e ? atoi(e) : 0; }();
  p.debug = env_debug & 31;
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
  auto al8 = [](long long x) { return (x % 8) == 0; };
  e.stage_d = (!a->d_is_f32 && a->beta == 0.f && (((uintptr_t)a->D) & 15) == 0 && al8(a->ldd) && al8(a->d_bs0) && al8(a->d_bs1)) ? 1 : 0;
  e.stage_p = (a->D_pre && (((uintptr_t)a->D_pre) & 15) == 0 && al8(a->ldp) && al8(a->p_bs0) && al8(a->p_bs1)) ? 1 : 0;
  e.drop_thresh = sb_dropout_threshold(a->drop_p);
  e.drop_scale = a->drop_p > 0.f ? 1.f / (1.f - a->drop_p) : 1.f;
  e.drop_seed = a->drop_seed;
  int grid = sb_num_sms() - sb_reserved_sms();
  if (grid < 8) grid = 8;
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if ((long long)grid > p.num_work) grid = (int)p.num_work;
  const int variant = (a->a_mn_major ? 2 : 0) | (a->b_mn_major ? 1 : 0) | (bn == 256 ? 4 : 0) | (pair ? 8 : 0);
  void (*kern)(const CUtensorMap, const CUtensorMap, const GemmParams, const PeerMaps) = nullptr;
  switch (variant) {
    case 0: kern = gemm_bf16_kernel<false, false, 128, false>; break;
    case 1: kern = gemm_bf16_kernel<false, true, 128, false>; break;
    case 2: kern = gemm_bf16_kernel<true, false, 128, false>; break;
    case 3: kern = gemm_bf16_kernel<true, true, 128, false>; break;
    case 4: kern = gemm_bf16_kernel<false, false, 256, false>; break;
    case 5: kern = gemm_bf16_kernel<false, true, 256, false>; break;
    case 6: kern = gemm_bf16_kernel<true, false, 256, false>; break;
    case 7: kern = gemm_bf16_kernel<true, true, 256, false>; break;
    case 12: kern = gemm_bf16_kernel<false, false, 256, true>; break;
    case 13: kern = gemm_bf16_kernel<false, true, 256, true>; break;
    case 14: kern = gemm_bf16_kernel<true, false, 256, true>; break;
    default: kern = gemm_bf16_kernel<true, true, 256, true>; break;
  }
  const int smem = smem_bytes(bn, pair);
  if (!g_attr_set[variant]) {
    cudaError_t ae = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ae != cudaSuccess) return (int)ae;
    if (pair) {
      ae = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
      (void)ae;
    }
    g_attr_set[variant] = true;
  }
  if (pair) {
    int pairs = (sb_num_sms() - sb_reserved_sms()) / 2;
    if (pairs < 4) pairs = 4;
    if (a->max_ctas > 1 && a->max_ctas / 2 < pairs) pairs = a->max_ctas / 2;
    if ((long long)pairs > p.num_work) pairs = (int)p.num_work;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, p, pm);
  }
  kern<<<grid, NUM_THREADS, smem, stream>>>(ta, tb, p, pm);
  return (int)cudaGetLastError();
}
