// Consumer side of GEMM + reduce-scatter: wait until every rank's reductions into this rank's accumulator have landed,
// then convert the accumulator to the output dtype and clear it for its next use.
//
// Every rank's GEMM publishes a "landed" flag (slot 8 + rank of this rank's flag array) with the call's epoch from its last
// block, after system-scope fences that order all of its reductions into peer memory before the flag.  This kernel is launched
// on the same stream after the local GEMM; each block polls the `world` flags (bounded: about a second, then the status word is
// set and the conversion goes ahead on whatever is there, so the stream keeps running and the host reads the failure).
// The accumulator is read with L1 bypassed: its lines are written by other GPUs, which the L1 does not see.
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <bool BF16>
__global__ void wait_reduce_out_kernel(float* __restrict__ acc, void* __restrict__ out, long long n4, const unsigned int* flags, int world,
                                       unsigned int epoch, int* status) {
  if (threadIdx.x < world) {
    const unsigned int* f = flags + 8 + threadIdx.x;
    const long long t0 = clock64();
    unsigned int probes = 0;
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if ((++probes & 15u) == 0 && (clock64() - t0 > sb_wait_cycles(status) || sb_failed(status))) {
        sb_set_status(status, SB_TIMEOUT_PEER_FLAG, (int)threadIdx.x);
        break;
      }
    }
  }
  __syncthreads();
  // After a give-up (here or in an earlier kernel of the step) the accumulator may still receive late contributions: it is
  // neither converted nor cleared, the output keeps its old contents and the host reads the status word.
  if (sb_failed(status)) return;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4* src = reinterpret_cast<float4*>(acc) + i;
    const float4 v = __ldcg(src);
    if (BF16) {
      __align__(8) __nv_bfloat162 t[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
      reinterpret_cast<uint2*>(out)[i] = *reinterpret_cast<uint2*>(t);
    } else {
      reinterpret_cast<float4*>(out)[i] = v;
    }
    __stcg(src, zero);
  }
}

}  // namespace

// acc: this rank's fp32 accumulator [n] (n % 4 == 0, 16-byte aligned); out: [n] bf16 or fp32; flags: this rank's flag array.
SB_API int sb_peer_wait_reduce_out(float* acc, void* out, int out_is_bf16, long long n, const unsigned int* flags, int world,
                                   unsigned int epoch, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0 || world < 1 || world > 8 || !flags || (((uintptr_t)acc) & 15) != 0 || (((uintptr_t)out) & 15) != 0) return -1;
  int* status = sb_status_ptr();
  if (!status) return -2;
  const long long n4 = n / 4;
  long long blocks = (n4 + 255) / 256;
  const long long cap = (long long)sb_num_sms() * 4;
  if (blocks > cap) blocks = cap;
  if (out_is_bf16)
    wait_reduce_out_kernel<true><<<(int)blocks, 256, 0, stream>>>(acc, out, n4, flags, world, epoch, status);
  else
    wait_reduce_out_kernel<false><<<(int)blocks, 256, 0, stream>>>(acc, out, n4, flags, world, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
