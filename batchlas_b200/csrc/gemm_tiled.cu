// Register-blocked shared-memory tiles for mid and large matrices, all four dtypes and all nine
// op pairs, fed by a multi-stage ring of 16-byte asynchronous copies.
//
// One CTA computes a BM x BN tile of one batch item.  Operands stay in their stored orientation
// in shared memory; only the fragment read pattern changes with the op:
//   M-major A (op N):   smem rows are k, BM elements each; a 16-byte read = V rows at one k.
//   K-major A (op T/C): smem rows are m, BK elements each (+16 B pitch pad); a read = V k's of one
//                       row.  Tile row r is stored at a permuted row slot so that the 8 lanes of a
//                       request read 8 consecutive slots -> 8 different 16-byte bank groups.
//   B is handled the same way with n in place of m (N-major for op T/C, K-major for op N).
// V = 16 / sizeof(T).  A warp is 8 (m) x 4 (n) lanes, so an A request touches 128 contiguous bytes
// and a B request 64, both conflict-free.  Conjugation is applied to fragments in registers.
//
// Preconditions (checked by tiled_supported, otherwise the generic kernel runs): 16-byte aligned
// bases, and ld * sizeof(T) and stride * sizeof(T) multiples of 16.  m, n, k are arbitrary: edge
// chunks are zero-filled through the copy's source-size operand and the epilogue is predicated.
//
// Algorithmic traffic per item: A and B once each, C written once and read once iff beta != 0;
// tiles of one item re-read A/B through L2 (BM x BN tiles: A is read N/BN times, B M/BM times).
#include "common.cuh"

namespace blb200 {
// One translation unit per element type (gemm_tiled_s.cu, _d.cu, _c.cu, _z.cu); each picks its tile size.
int launch_tiled_s(const GemmParams& p, cudaStream_t stream);
int launch_tiled_d(const GemmParams& p, cudaStream_t stream);
int launch_tiled_c(const GemmParams& p, cudaStream_t stream);
int launch_tiled_z(const GemmParams& p, cudaStream_t stream);

namespace {
inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }
}  // namespace

bool tiled_supported(const GemmParams& p, int dtype) {
  const long long es = (dtype == BLB200_S) ? 4 : (dtype == BLB200_Z ? 16 : 8);
  if (p.k < 1) return false;
  if (p.m <= 32 && p.n <= 32) return false;  // too small to fill a tile: generic 16x16 / 32x32 tiles
  if (!aligned16(p.a) || !aligned16(p.b) || !aligned16(p.c)) return false;
  if ((p.lda * es) % 16 || (p.ldb * es) % 16 || (p.ldc * es) % 16) return false;
  if ((p.sa * es) % 16 || (p.sb * es) % 16 || (p.sc * es) % 16) return false;
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
