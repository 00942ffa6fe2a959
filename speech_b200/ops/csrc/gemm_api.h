// C interface of the tcgen05 GEMM (implemented in gemm_tcgen05.cu); used by the Python bindings and by other kernels' host
// drivers in this library (the LSTM recurrence issues one small GEMM per time step).
#pragma once
#include "common.cuh"

struct SbGemmArgs {
  const void* A;
  const void* B;
  int M, N, K;
  int a_mn_major, b_mn_major;
  long long lda, ldb;
  int batch0, batch1;
  long long a_bs0, a_bs1, b_bs0, b_bs1;
  void* D;
  int d_is_f32;
  long long ldd, d_bs0, d_bs1;
  const void* bias;
  int bias_is_f32;
  const void* residual;
  long long ldr, r_bs0, r_bs1;
  const void* aux;
  long long ldx, x_bs0, x_bs1;
  void* D_pre;
  long long ldp, p_bs0, p_bs1;
  float alpha, beta;
  int act, dact;
  int max_ctas;  // 0 = one per SM
  int fold_batch1;  // 1: sum over batch1 inside the K loop; D then has no batch1 dimension
  int tile_n;       // 128 or 256 to force the tile width, anything else = automatic
  float drop_p;     // > 0: dropout applied to act(acc + bias) before alpha / residual; mask = sb_dropout_keep(seed, m * N + n)
  unsigned long long drop_seed;
  int ksplit;       // 0 = automatic, -1 = never split K, > 1 = that many K slices (only honoured for D(fp32) += alpha * A B^T)
  const void* const* peer_D;  // device array [world] of fp32 output buffers for GEMM + reduce-scatter (see gemm_tcgen05.cu); or null
  int peer_rows;    // rows of the full output owned by each rank
  const void* const* peer_A;  // HOST array [peer_world] of device pointers: rank r's row shard of A (all-gather + GEMM); or null
  int peer_a_rows;  // rows per shard (multiple of 128)
  int peer_world;
  int pair;         // 0 = default policy, 1 = use CTA pairs (cta_group::2) when the shape allows, -1 = never
  // In-kernel rank synchronisation for the fused collectives (all null / 0 = none).  sig_flags is a DEVICE array [sig_world] of
  // device pointers: entry r is rank r's flag array (16 x u32: slots 0..7 "shard of rank i is in place", slots 8..15
  // "contributions of rank i have landed").  Flags carry a per-call epoch that only grows.
  //   sig_head: block 0 publishes this rank's "in place" flag to every rank at kernel start, and the TMA producer waits (bounded)
  //             for the owner's flag before its first load from that rank's memory (all-gather + GEMM);
  //   sig_tail: the last block to finish publishes this rank's "landed" flag to every rank (GEMM + reduce-scatter).
  unsigned int* const* sig_flags;
  unsigned int* sig_counter;   // device word, zero between calls: blocks that have finished
  int sig_world, sig_rank;
  unsigned int sig_epoch;
  int sig_head, sig_tail, pad3_;
  // Staging for all-gather + GEMM (with sig_head): instead of loading A tiles from the owner's memory for every column tile
  // (the shard would cross NVLink once per column tile), the blocks first copy every remote shard ONCE into this rank's
  // staging area with plain peer loads, while the tiles of this rank's own rows are already being multiplied; tiles of remote
  // rows wait (bounded) until all blocks have finished copying.  peer_A[r] then names the LOCAL staging slot of rank r (and
  // this rank's own shard for r == sig_rank).  stage_src is a DEVICE array [sig_world] of the ranks' shard addresses.
  const void* const* stage_src;
  void* stage_dst;              // staging area: sig_world slots of stage_bytes each
  long long stage_bytes;        // bytes of one shard (multiple of 16); 0 = no staging
  unsigned int* stage_counter;  // device words, zero between calls: [0] blocks that finished copying, [1] blocks that exited
  // Optional fp32 scratch of at least M * N * 4 bytes for small-M GEMMs with a bf16 output: when given (and the shape has few
  // output tiles and a long K), K is split over more blocks through this scratch and a second small kernel applies the epilogue.
  void* splitk_ws;
  long long splitk_ws_bytes;
};


// Returns 0 on success, a negative code for invalid arguments, or a positive cudaError_t.
SB_API int sb_gemm_bf16(const SbGemmArgs* a, cudaStream_t stream);
