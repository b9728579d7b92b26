// The tiled kernel's instantiations for double (templates in gemm_tiled.cuh).
#include "gemm_tiled.cuh"

namespace blb200 {

int launch_tiled_d(const GemmParams& p, cudaStream_t stream) {
  if (p.m <= 64 && p.n <= 64) return launch_ops<double, Tile<double, 64, 64, 16, 4, 4, 3>, 3>(p, stream);
  return launch_ops<double, Tile<double, 128, 64, 16, 8, 4, 3>, 2>(p, stream);
}

}  // namespace blb200
