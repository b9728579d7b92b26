// Entry of the register-blocked tile kernels (templates and design notes in gemm_tiled.cuh): checks
// the preconditions and hands the problem to the translation unit of its element type.
#include "common.cuh"

namespace blb200 {
// One translation unit per element type (gemm_tiled_s.cu, _d.cu, _c.cu, _z.cu); each picks its tile size.
int launch_tiled_s(const GemmParams& p, cudaStream_t stream);
int launch_tiled_d(const GemmParams& p, cudaStream_t stream);
int launch_tiled_c(const GemmParams& p, cudaStream_t stream);
int launch_tiled_z(const GemmParams& p, cudaStream_t stream);

// Shapes the tile kernels take; operands must be element-aligned (16-byte aligned operands use the
// 16-byte copy policy, others the element-granular one; structure hints and split-K need the former).
bool tiled_supported(const GemmParams& p, int dtype) {
  const long long es = dtype_bytes(dtype);
  if (p.k < 1) return false;
  if (p.m <= 32 && p.n <= 32) return false;  // too small to fill a tile: generic 16x16 / 32x32 tiles
  if (!operands_aligned_to(p, es, es)) return false;
  if ((has_hints(p) || p.splits > 1) && !operands_aligned_to(p, es, 16)) return false;
  return true;
}

int launch_tiled(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!tiled_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  int rc;
  switch (dtype) {
    case BLB200_S: rc = launch_tiled_s(p, stream); break;
    case BLB200_D: rc = launch_tiled_d(p, stream); break;
    case BLB200_C: rc = launch_tiled_c(p, stream); break;
    case BLB200_Z: rc = launch_tiled_z(p, stream); break;
    default: return BLB200_E_DTYPE;
  }
  if (rc == BLB200_OK) note_launch("tiled");
  return rc;
}

}  // namespace blb200
