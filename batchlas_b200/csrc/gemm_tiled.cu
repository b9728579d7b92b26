// placeholder until the tiled kernels land
#include "common.cuh"
namespace blb200 {
bool tiled_supported(const GemmParams&, int) { return false; }
int launch_tiled(const GemmParams&, int, cudaStream_t) { return BLB200_E_UNSUPPORTED; }
}  // namespace blb200
