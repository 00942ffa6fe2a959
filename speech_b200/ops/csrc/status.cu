// Device status word shared by all kernels of the library, plus host accessors.
#include "common.cuh"
#include <stdio.h>

#define SB_MAX_DEVICES 16
// ints 0-3: status word (code, block, detail, spare); ints 4-5: run-time wait limit in cycles (0 = SB_WAIT_CYCLES)
static __device__ __align__(16) int g_sb_status[8];
static int* g_status_ptr[SB_MAX_DEVICES] = {nullptr};

SB_API int* sb_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= SB_MAX_DEVICES) return nullptr;
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sb_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = (int*)p;
  }
  return g_status_ptr[dev];
}

// Copies the 4-int status word to the host (synchronises the stream) and clears it when `clear` is set.
SB_API int sb_read_status(int* out4, int clear, cudaStream_t stream) {
  int* p = sb_status_ptr();
  if (!p) return -1;
  cudaError_t e = cudaMemcpyAsync(out4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return (int)e;
  if (clear && out4[0] != 0) {
    e = cudaMemsetAsync(p, 0, 4 * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// Sets the limit of every bounded in-kernel wait on the current device, in SM clock cycles (0 restores the compile-time
// default of about a second).  Training raises it so that ordinary skew between ranks (a rank that validates or logs longer)
// does not trip it; tests lower it to make a wait run out quickly.  Synchronises the device.
SB_API int sb_set_wait_cycles(long long cycles) {
  int* p = sb_status_ptr();
  if (!p) return -1;
  if (cycles < 0) cycles = 0;
  cudaError_t e = cudaMemcpy(p + 4, &cycles, sizeof(long long), cudaMemcpyHostToDevice);
  return (int)e;
}

// Enqueues a copy of the 4-int status word into pinned host memory on `stream` (no synchronisation); the caller records an
// event behind it and reads `host4` once the event has completed.
SB_API int sb_status_copy_async(int* host4, cudaStream_t stream) {
  int* p = sb_status_ptr();
  if (!p || !host4) return -1;
  return (int)cudaMemcpyAsync(host4, p, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream);
}

SB_API const char* sb_status_string(int code) {
  switch (code) {
    case SB_OK: return "ok";
    case SB_TIMEOUT_SMEM_EMPTY: return "timeout waiting for a free shared-memory stage";
    case SB_TIMEOUT_SMEM_FULL: return "timeout waiting for a TMA load to land";
    case SB_TIMEOUT_TMEM_EMPTY: return "timeout waiting for the epilogue to release an accumulator";
    case SB_TIMEOUT_TMEM_FULL: return "timeout waiting for the tensor core to finish a tile";
    case SB_TIMEOUT_PEER_FLAG: return "timeout waiting for a peer rank's flag";
    case SB_BAD_ARGUMENT: return "bad argument";
    default: return "unknown";
  }
}

SB_API int sb_last_cuda_error() { return (int)cudaGetLastError(); }

// SMs that persistent kernels leave free for kernels running beside them (gradient-exchange kernels on another stream).  A
// persistent GEMM whose grid exceeds the SMs actually available runs its displaced CTAs as a second wave and takes twice as long.
static int g_sb_reserved_sms = 0;
SB_API void sb_set_reserved_sms(int n) { g_sb_reserved_sms = n < 0 ? 0 : n; }
SB_API int sb_reserved_sms() { return g_sb_reserved_sms; }
