// The tiled kernel's instantiations for complex<double> (templates in gemm_tiled.cuh).
#include "gemm_tiled.cuh"

namespace blb200 {

int launch_tiled_z(const GemmParams& p, cudaStream_t stream) {
  return launch_ops<double2, Tile<double2, 64, 64, 16, 4, 4, 3>, 2>(p, stream);
}

}  // namespace blb200
