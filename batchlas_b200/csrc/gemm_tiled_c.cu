// The tiled kernel's instantiations for complex<float> (templates in gemm_tiled.cuh).
#include "gemm_tiled.cuh"

namespace blb200 {

int launch_tiled_c(const GemmParams& p, cudaStream_t stream) {
  // The wide tile is about 5 % faster on full tiles (256^3: 50.0 against 47.4 TFLOP/s), so the small
  // one takes over when it saves more than that in padding (160^3: 32.3 against 25.6).
  auto padded = [](int m, int n, int bm, int bn) {
    return (long long)((m + bm - 1) / bm) * bm * ((n + bn - 1) / bn) * bn;
  };
  if ((p.m <= 64 && p.n <= 64) || 20 * padded(p.m, p.n, 128, 64) > 21 * padded(p.m, p.n, 64, 64))
    return launch_ops<float2, Tile<float2, 64, 64, 16, 4, 4, 3>, 3>(p, stream);
  return launch_ops<float2, Tile<float2, 128, 64, 16, 8, 4, 3>, 2>(p, stream);
}

}  // namespace blb200
