// The tiled kernel's instantiations for float (templates in gemm_tiled.cuh).
#include "gemm_tiled.cuh"

namespace blb200 {

int launch_tiled_s(const GemmParams& p, cudaStream_t stream) {
  // The 64 x 64 tile (4 x 4 register blocks, three CTAs per SM) wastes less on shapes that are not
  // multiples of 128 and was at least as fast as the 128-wide one up to 512^3 (320^3: 38.6 against
  // 23.7 TFLOP/s), so the wide tile keeps only the largest problems.
  if (p.m >= 1024 && p.n >= 1024) return launch_ops<float, Tile<float, 128, 128, 16, 8, 8, 3>, 1>(p, stream);
  return launch_ops<float, Tile<float, 64, 64, 16, 4, 4, 3>, 3>(p, stream);
}

}  // namespace blb200
