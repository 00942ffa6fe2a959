// tcgen05 GEMM kernels of the LEAN epilogue class (see gemm_kernel.cuh).
#include "gemm_kernel.cuh"

int sb_gemm_launch_lean(int variant, int grid, bool pair, cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb,
                        const GemmParams& p, const PeerMaps& pm, const CUtensorMap& td, const CUtensorMap& tp) {
  return launch_gemm_variant<EPI_LEAN>(variant, grid, pair, stream, ta, tb, p, pm, td, tp);
}
