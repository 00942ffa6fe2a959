// C interface of the small-vector peer all-reduce (peer_small_allreduce.cu); also called by the Conformer layer executor for
// synchronised BatchNorm statistics.
#pragma once
#include "common.cuh"

#define SB_SMALL_MAX_WORLD 16
#define SB_SMALL_MAX 4096

struct SbPeerSmallArgs {
  float* data;              // local vector [n] (+ 1 when has_extra), reduced in place
  void* const* buffers;     // device array [world]: base address of each rank's symmetric buffer
  long long base_off;       // byte offset of this protocol's region inside the symmetric buffers
  int n;
  int has_extra;            // 1: element n of the exchanged vector is `extra` (e.g. the local element count); data[n] gets the sum
  float extra;
  int rank, world;
  unsigned int epoch;
  int* status;
};

SB_API long long sb_peer_small_bytes();
SB_API int sb_peer_small_max();
// All ranks call this with the same n / has_extra / epoch sequence.  Returns 0, a negative argument error or a cudaError_t.
SB_API int sb_peer_small_allreduce(const SbPeerSmallArgs* args, cudaStream_t stream);
