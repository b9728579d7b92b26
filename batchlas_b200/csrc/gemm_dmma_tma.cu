// FP64 tensor-core tiles for real double, fed by TMA: the plain strided-batched DGEMM of the mid and
// large shapes (256^3, 1024^3).  Same CTA shape as the cp.async DMMA kernel — 64 x 64 output, four
// warps of 32 x 32 as 4 x 4 mma.sync m8n8k4 tiles, four CTAs per SM — but the operand tiles arrive by
// cp.async.bulk.tensor from 3-D tensor maps (rows x columns x batch item) over the caller's own
// column-major storage, complete on one mbarrier per stage, and are laid out by the 128-byte
// swizzle.  What that removes from the 128 threads of a CTA: every per-thread copy instruction with
// its address and edge arithmetic (edges are zero-filled by the tensor map's bounds), the
// cp.async group bookkeeping, and the row padding of the stages (a stage is 16 KiB for every op
// pair).  One thread issues two to eight box copies per k-tile.
//
// Stage layout (BK = 16 doubles = 128 bytes, the widest row the 128-byte swizzle allows):
//   K-major operand (A under op T, B under op N): one box of 16 k x 64 rows; stage row r holds the
//     16 k of matrix row r, its 16-byte chunks XORed with (r & 7).
//   M-major operand (A under op N, B under op T): four blocks of 16 rows x 16 k, 2 KiB each; block
//     row kk holds 16 consecutive matrix rows at k = kk, chunks XORed with (kk & 7).  When the
//     operand's row count is a multiple of 16 the four blocks come from ONE copy through a 4-D map
//     that splits the rows into (16, rows / 16) — box 16 x 16 x 4 x 1 — otherwise from four 3-D
//     copies whose row bound zero-fills the ragged edge (the 4-D view cannot bound a partial group
//     of 16 rows; measured: four small boxes per operand cost 1-2 % against the cp.async kernel,
//     one box gains).
// The DMMA fragment of lane (g = lane >> 2, t = lane & 3) is element (row g, k t) of an 8 x 4 tile.
// With all stage rows exactly 128 bytes apart, a half-warp request (4 g x 4 t) is conflict-free only
// if the XOR spreads it over all eight chunks, which fixes which matrix rows the eight g-lanes of a
// tile must own.  Both assignments are permutations of the warp's 32 rows over (g, tile i):
//   K-major:  row = 16 (i >> 1) + 8 (g >> 2) + 2 (g & 3) + (i & 1)        -> row & 7 = 2 (g & 3) + (i & 1)
//   M-major:  row = 16 (i >> 1) + 8 ((g >> 1) & 1) + 4 (i & 1) + 2 (g >> 2) + (g & 1)
// Every tile product still multiplies rows of op(A) with columns of op(B) over the same k, so the
// result is the same sum in the same order as the other DMMA kernel; only which lane holds which
// element of C differs, and the epilogue applies the same permutations.
//
// Epilogue of the real kernel, chosen per call: for k <= 128 the tile is staged through the (now idle)
// stage buffers and leaves as whole stored columns, 16 bytes per lane (C's prior values read the same
// way, all sixteen requests of a lane in flight at once); for longer k each lane writes its
// fragment elements directly and the C tile is asked into L2 before the main loop when beta != 0.
// Both compute alpha * acc, then fma(beta, prior, .): the same bits.
//
// Preconditions (dmma_tma_supported): real double, no structure hints / per-item dims / split-K,
// 16-byte aligned bases and even ld and batch strides for A and B (tensor-map strides are multiples
// of 16 bytes), positive batch strides; C needs element alignment only.  No load with cluster multicast is used; the maps cover this GPU's memory.
#include <string.h>

#include <atomic>

#include "common.cuh"
#include "tensor_map.cuh"

namespace blb200 {
namespace {

enum WaitCode { kDmmaTmaWaitFull = 401 };

constexpr int kBM = 64, kBN = 64, kBK = 16, kStages = 3, kThreads = 128;
constexpr int kOperandBytes = 64 * kBK * 8;       // 8 KiB
constexpr int kStageBytes = 2 * kOperandBytes;    // A tile + B tile
enum EpilogueFlags { kEpiPairs = 1, kEpiStaged = 2, kEpiPrefetch = 4 };

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// Row of the warp's 32 owned by lane group g in tile i (see the file comment).
__device__ __forceinline__ int perm_kmajor(int g, int i) { return 16 * (i >> 1) + 8 * (g >> 2) + 2 * (g & 3) + (i & 1); }
__device__ __forceinline__ int perm_mmajor(int g, int i) {
  return 16 * (i >> 1) + 8 * ((g >> 1) & 1) + 4 * (i & 1) + 2 * (g >> 2) + (g & 1);
}

// Byte offset, inside an operand tile, of this lane's fragment element for tile 0 and k-step 0 of
// warp row-block w; fragment_offset() below moves it to tile i and k-step k4.
template <bool KMAJOR>
__device__ __forceinline__ int fragment_base(int w, int g, int t) {
  if (KMAJOR) return (32 * w + 2 * (g & 3) + 8 * (g >> 2)) * 128 + ((((t >> 1) | ((g & 3) << 1))) << 4) + (t & 1) * 8;
  const int c0 = (g >> 2) + 4 * ((g >> 1) & 1);
  return 2 * w * 2048 + t * 128 + ((c0 ^ t) << 4) + (g & 1) * 8;
}
template <bool KMAJOR>
__device__ __forceinline__ int fragment_offset(int base, int i, int k4) {
  if (KMAJOR) return (base ^ ((i & 1) << 4) ^ (k4 << 5)) + (i & 1) * 128 + (i >> 1) * 2048;
  return (base ^ ((i & 1) << 5) ^ ((k4 & 1) << 6)) + (i >> 1) * 2048 + k4 * 512;
}

// Position swizzle of the staged C tile (see the epilogue): which 16-byte chunk positions the column
// bits that vary inside one store request must flip, given which row bits vary there.
template <bool AK>
__device__ __forceinline__ int c_swizzle(int col) {
  const int lo = ((col >> 1) ^ (col >> 2)) & 1, hi = (col >> 3) & 1;
  return AK ? ((lo << 1) | (hi << 2)) : (lo | (hi << 1));
}

template <int OPA, int OPB>
__global__ void __launch_bounds__(kThreads, 4)
    gemm_dmma_tma_d_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           double* __restrict__ C, long long sc, long long ldc, int m, int n, int k, int tiles_m,
                           int tiles_n, double alpha, double beta, int a_grouped, int b_grouped, int epi) {
  constexpr bool AK = (OPA != BLB200_N);   // A stored k x m: k fastest
  const bool c_vec = epi & kEpiPairs, staged = epi & kEpiStaged;
  constexpr bool BKM = (OPB == BLB200_N);  // B stored k x n: k fastest
  extern __shared__ unsigned char smem_raw[];
  // the swizzle is a function of the shared-memory address: tiles must start on 1024-byte boundaries
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const int item = (int)(tile / tiles_per_item);
  const int rem = (int)(tile - (long long)item * tiles_per_item);
  const int m0 = (rem % tiles_m) * kBM, n0 = (rem / tiles_m) * kBN;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // Programmatic dependent launch: the next kernel's first CTAs may take their places while this
  // grid drains; nothing here touches global memory before every earlier grid has finished.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if ((epi & kEpiPrefetch) && beta != 0.0) {  // the epilogue reads this tile of C: ask L2 for it now (two threads per column, 128-byte lines)
    const int col = n0 + (tid >> 1), r0 = m0 + 32 * (tid & 1);
    if (col < n && r0 < m) {
      const double* pc = C + (long long)item * sc + (long long)col * ldc + r0;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(pc));
      if (r0 + 16 < m) asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + 16));
    }
  }

  const int KT = (k + kBK - 1) / kBK;
  auto issue = [&](int s, int kt) {  // one thread: the copies of k-tile kt into stage s
    unsigned char* st = smem + (size_t)s * kStageBytes;
    const int k0 = kt * kBK;
    mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
    if (AK) {
      tma_load_3d(st, &map_a, k0, m0, item, &full_bar[s]);
    } else if (a_grouped) {
      tma_load_4d(st, &map_a, 0, k0, m0 >> 4, item, &full_bar[s]);
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b) tma_load_3d(st + b * 2048, &map_a, m0 + 16 * b, k0, item, &full_bar[s]);
    }
    if (BKM) {
      tma_load_3d(st + kOperandBytes, &map_b, k0, n0, item, &full_bar[s]);
    } else if (b_grouped) {
      tma_load_4d(st + kOperandBytes, &map_b, 0, k0, n0 >> 4, item, &full_bar[s]);
    } else {
#pragma unroll
      for (int b = 0; b < 4; ++b) tma_load_3d(st + kOperandBytes + b * 2048, &map_b, n0 + 16 * b, k0, item, &full_bar[s]);
    }
  };
  if (tid == 0)
    for (int s = 0; s < kStages - 1 && s < KT; ++s) issue(s, s);

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int a_base = fragment_base<AK>(wm, g, t);
  const int b_base = fragment_base<BKM>(wn, g, t);

  int issued = KT < kStages - 1 ? KT : kStages - 1;  // k-tiles whose copies have been issued (thread 0's view)
  int kt = 0;
  bool lost = false;
  for (; kt < KT; ++kt) {
    const int s = kt % kStages;
    const bool ok = mbar_wait(&full_bar[s], (uint32_t)(kt / kStages) & 1u, kDmmaTmaWaitFull);
    // one barrier: every warp has left stage (kt - 1) % kStages, and all threads agree on `ok`
    if (__syncthreads_or(!ok)) {
      lost = true;
      break;
    }
    if (tid == 0 && issued < KT) {
      fence_async_smem();
      issue(issued % kStages, issued);
      ++issued;
    }
    const unsigned char* as = smem + (size_t)s * kStageBytes;
    const unsigned char* bs = as + kOperandBytes;
#pragma unroll
    for (int k4 = 0; k4 < kBK / 4; ++k4) {
      double af[4], bf[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) af[i] = *reinterpret_cast<const double*>(as + fragment_offset<AK>(a_base, i, k4));
#pragma unroll
      for (int j = 0; j < 4; ++j) bf[j] = *reinterpret_cast<const double*>(bs + fragment_offset<BKM>(b_base, j, k4));
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma(acc[i][j][0], acc[i][j][1], af[i], bf[j]);
    }
  }
  if (lost) {
    // A copy never arrived (recorded in the status word).  Do not leave while later copies may still
    // land in this CTA's shared memory: give each issued stage a short, bounded chance to complete.
    if (tid == 0)
      for (int q = kt + 1; q < issued; ++q)
        mbar_wait_limit(&full_bar[q % kStages], (uint32_t)(q / kStages) & 1u, kDmmaTmaWaitFull, 1u << 12);
    return;
  }

  if (!staged) {  // long k: the epilogue is a small part of the tile's life; write straight from the fragment layout
    const bool bz = beta == 0.0;
    double* Ci = C + (long long)item * sc;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = n0 + 32 * wn + (BKM ? perm_kmajor(2 * t + e, j) : perm_mmajor(2 * t + e, j));
        if (col >= n) continue;
        double* ccol = Ci + (long long)col * ldc;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = m0 + 32 * wm + (AK ? perm_kmajor(g, i) : perm_mmajor(g, i));
          if (row >= m) continue;
          double out = alpha * acc[i][j][e];
          if (!bz) out = fma(beta, ccol[row], out);
          ccol[row] = out;
        }
      }
    return;
  }
  // Epilogue through shared memory: the accumulators of a lane are scattered over the tile (8-byte
  // pieces of many columns), so the tile is first laid down column by column in the stage buffers,
  // which no copy targets any more, and then read back so that a warp handles one whole stored column per
  // step: 512 contiguous bytes of C, 16 per lane, for the read of the prior value and for the store.
  // Column `col` keeps its 16-byte chunk `ch` (rows 2ch, 2ch+1) at position ch ^ c_swizzle(col): that
  // spreads every store request of the fragment layout over all banks, and a permutation inside a
  // column costs the read-back nothing.
  __syncthreads();  // every warp has left the last stage; every copy was waited for above
  double* cs = reinterpret_cast<double*>(smem);
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int cl = 32 * wn + (BKM ? perm_kmajor(2 * t + e, j) : perm_mmajor(2 * t + e, j));
      double* col_s = cs + cl * kBM;
      const int h = c_swizzle<AK>(cl);
      if (AK) {  // tiles 2ip and 2ip + 1 hold rows r and r + 1: one 16-byte chunk
#pragma unroll
        for (int ip = 0; ip < 2; ++ip) {
          const int ch = (32 * wm + perm_kmajor(g, 2 * ip)) >> 1;
          *reinterpret_cast<double2*>(col_s + ((ch ^ h) << 1)) = make_double2(acc[2 * ip][j][e], acc[2 * ip + 1][j][e]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = 32 * wm + perm_mmajor(g, i);
          col_s[(((row >> 1) ^ h) << 1) + (row & 1)] = acc[i][j][e];
        }
      }
    }
  const bool beta_zero = beta == 0.0;
  C += (long long)item * sc;
  const int row = m0 + 2 * lane;
  const bool pair = c_vec && row + 1 < m;
  // the reads of prior values go out first, sixteen independent requests, once the accumulators have left their registers, and fly across the barrier
  double2 prior[kBN / 4];
  if (!beta_zero) {
#pragma unroll
    for (int q = 0; q < kBN / 4; ++q) {
      const int col = n0 + warp + 4 * q;
      prior[q] = make_double2(0.0, 0.0);
      if (col >= n || row >= m) continue;
      const double* pc = C + (long long)col * ldc + row;
      if (pair) {
        prior[q] = *reinterpret_cast<const double2*>(pc);
      } else {
        prior[q].x = pc[0];
        if (row + 1 < m) prior[q].y = pc[1];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kBN / 4; ++q) {
    const int cl = warp + 4 * q, col = n0 + cl;
    if (col >= n || row >= m) continue;
    const double2 v = *reinterpret_cast<const double2*>(cs + cl * kBM + ((lane ^ c_swizzle<AK>(cl)) << 1));
    double2 out = make_double2(alpha * v.x, alpha * v.y);
    if (!beta_zero) {
      out.x = fma(beta, prior[q].x, out.x);
      out.y = fma(beta, prior[q].y, out.y);
    }
    double* pc = C + (long long)col * ldc + row;
    if (pair) {
      *reinterpret_cast<double2*>(pc) = out;
    } else {
      pc[0] = out.x;
      if (row + 1 < m) pc[1] = out.y;
    }
  }
}

enum MapKind { kMapKMajor = 0, kMapRows16 = 1, kMapRowGroups = 2 };

// Map over a column-major operand seen as doubles (a complex element is two), 128 bytes wide boxes,
// 128-byte swizzle, zero fill past the bounds.  rows / ld / stride are in doubles.
//   kMapKMajor    3-D (rows, cols, items), box 16 x 64: the contraction index runs along the rows
//   kMapRows16    3-D (rows, cols, items), box 16 x box_k: 16 doubles of a column at box_k k, any row count
//   kMapRowGroups 4-D (16, cols, rows / 16, items), box 16 x box_k x (64 * 16 / box_k / 16 ...) — all
//                 64 tile rows at box_k k in one copy; rows must be a multiple of 16 doubles (a
//                 partial group has no bound in this view)
int make_operand_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, long long stride,
                     int batch, int kind, int box_k, int groups) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return BLB200_E_INTERNAL;
  const cuuint64_t items = (cuuint64_t)(batch > 0 ? batch : 1);
  const long long item_stride = batch > 1 ? stride : ld * (long long)cols;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r;
  if (kind == kMapRowGroups) {
    const cuuint64_t dims[4] = {16, (cuuint64_t)cols, (cuuint64_t)(rows / 16), items};
    const cuuint64_t strides[3] = {(cuuint64_t)ld * 8, 128, (cuuint64_t)item_stride * 8};
    const cuuint32_t box[4] = {16, (cuuint32_t)box_k, (cuuint32_t)groups, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    const cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)cols, items};
    const cuuint64_t strides[2] = {(cuuint64_t)ld * 8, (cuuint64_t)item_stride * 8};
    const cuuint32_t box[3] = {16, kind == kMapKMajor ? 64u : (cuuint32_t)box_k, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? BLB200_OK : BLB200_E_INTERNAL;
}

// Tensor maps are pure functions of (base, shape, ld, stride, batch, box kind): a small per-thread
// cache saves the driver call when the same operand is multiplied again.
struct OperandMapCache {
  struct Entry {
    const void* base = nullptr;
    long long rows = 0;
    int cols = 0, batch = 0;
    long long ld = 0, stride = 0;
    int kind = 0, box_k = 0;
    bool valid = false;
    alignas(64) CUtensorMap map;
  };
  static constexpr int kEntries = 16;
  Entry e[kEntries];
  int next = 0;
  int get(CUtensorMap* out, const void* base, long long rows, int cols, long long ld, long long stride, int batch,
          int kind, int box_k = 16, int groups = 4) {
    for (int i = 0; i < kEntries; ++i) {
      const Entry& c = e[i];
      if (c.valid && c.base == base && c.rows == rows && c.cols == cols && c.ld == ld && c.stride == stride &&
          c.batch == batch && c.kind == kind && c.box_k == box_k) {
        memcpy(out, &c.map, sizeof(CUtensorMap));
        return BLB200_OK;
      }
    }
    Entry& slot = e[next];
    next = (next + 1) % kEntries;
    slot.valid = false;
    const int rc = make_operand_map(&slot.map, base, rows, cols, ld, stride, batch, kind, box_k, groups);
    if (rc != BLB200_OK) return rc;
    slot.base = base; slot.rows = rows; slot.cols = cols; slot.ld = ld; slot.stride = stride;
    slot.batch = batch; slot.kind = kind; slot.box_k = box_k; slot.valid = true;
    memcpy(out, &slot.map, sizeof(CUtensorMap));
    return BLB200_OK;
  }
};

template <int OPA, int OPB>
int launch_op(const GemmParams& p, cudaStream_t stream) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  const size_t smem = (size_t)kStages * kStageBytes + kStages * sizeof(uint64_t) + 1024;
  const int tiles_m = (p.m + kBM - 1) / kBM, tiles_n = (p.n + kBN - 1) / kBN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  alignas(64) CUtensorMap map_a, map_b;
  static thread_local OperandMapCache maps;
  const int a_rows = AK ? p.k : p.m, a_cols = AK ? p.m : p.k;
  const int b_rows = BKM ? p.k : p.n, b_cols = BKM ? p.n : p.k;
  // The grouped (4-D) view has a row-group stride (128 bytes) below its column stride; should a
  // driver refuse to encode that, the operand is fetched as four 16-row boxes from then on.
  static std::atomic<int> grouped_ok{1};
  int a_kind = AK ? kMapKMajor : (a_rows % 16 == 0 && grouped_ok.load() ? kMapRowGroups : kMapRows16);
  int b_kind = BKM ? kMapKMajor : (b_rows % 16 == 0 && grouped_ok.load() ? kMapRowGroups : kMapRows16);
  int rc = maps.get(&map_a, p.a, a_rows, a_cols, p.lda, p.sa, p.batch, a_kind);
  if (rc != BLB200_OK && a_kind == kMapRowGroups) {
    grouped_ok.store(0);
    a_kind = kMapRows16;
    if (b_kind == kMapRowGroups) b_kind = kMapRows16;
    rc = maps.get(&map_a, p.a, a_rows, a_cols, p.lda, p.sa, p.batch, a_kind);
  }
  if (rc != BLB200_OK) return rc;
  rc = maps.get(&map_b, p.b, b_rows, b_cols, p.ldb, p.sb, p.batch, b_kind);
  if (rc != BLB200_OK && b_kind == kMapRowGroups) {
    grouped_ok.store(0);
    b_kind = kMapRows16;
    rc = maps.get(&map_b, p.b, b_rows, b_cols, p.ldb, p.sb, p.batch, b_kind);
  }
  if (rc != BLB200_OK) return rc;
  // C read and written as 16-byte pairs of rows when every column of every item starts on a 16-byte boundary
  int epi = (reinterpret_cast<uintptr_t>(p.c) % 16 == 0 && p.ldc % 2 == 0 && p.sc % 2 == 0) ? kEpiPairs : 0;
  // Measured (B200, beta = 1): staging wins while the epilogue is a large part of a tile's life — k = 64: 20.3
  // against 16.5 TFLOP/s, k = 128: 29.1 against 26.9 — and loses 2 % at k = 256, where the direct
  // epilogue with the L2 prefetch of its C tile is the faster one (k = 192: 32.6 against 31.9).
  epi |= (p.k <= 128) ? kEpiStaged : kEpiPrefetch;
  auto kern = gemm_dmma_tma_d_kernel<OPA, OPB>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)total);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (double*)p.c, (long long)p.sc, (long long)p.ldc, p.m, p.n, p.k,
                                 tiles_m, tiles_n, p.alpha[0], p.beta[0], a_kind == kMapRowGroups ? 1 : 0,
                                 b_kind == kMapRowGroups ? 1 : 0, epi);
}


// ---- complex double ----------------------------------------------------------------------------------
// CTA 64 x 64, 8 warps as 2 (m) x 4 (n), warp tile 32 x 16 (4 x 2 DMMA tiles, re and im planes), two
// CTAs per SM (registers).  A stage holds kZSubs sub-tiles of 8 complex k = 128-byte rows each (the
// widest row the swizzle allows), so one barrier round covers 16 k.  A lane's fragment is one complex element (16 bytes = one
// swizzle chunk), a quarter-warp request is 2 rows x 4 k; it covers all eight chunks when the two
// rows differ in bit 2, so lane group g owns row 4 (g & 1) + (g >> 1) of each 8-row tile — the same
// assignment for both orientations.  M-major operands come as 8-row blocks of 1 KiB (one grouped
// 4-D copy when the row count is a multiple of 8, else eight 3-D copies).
constexpr int kZSubs = 2, kZBK = 8 * kZSubs, kZThreads = 256;
constexpr int kZStageBytes = kZSubs * kStageBytes;  // per sub-tile: A tile (8 KiB) then B tile (8 KiB)
__device__ __forceinline__ int perm_z(int g) { return 4 * (g & 1) + (g >> 1); }

template <bool KMAJOR>
__device__ __forceinline__ int z_fragment_base(int first_row, int g, int t) {  // first_row: of the warp, multiple of 8
  const int chunk = ((g >> 1) ^ t) + 4 * (g & 1);
  if (KMAJOR) return (first_row + perm_z(g)) * 128 + (chunk << 4);
  return (first_row >> 3) * 1024 + t * 128 + (chunk << 4);
}
template <bool KMAJOR>
__device__ __forceinline__ int z_fragment_offset(int base, int i, int k4) {
  if (KMAJOR) return (base ^ (k4 << 6)) + i * 1024;
  return (base ^ (k4 << 6)) + i * 1024 + k4 * 512;
}

template <int OPA, int OPB>
__global__ void __launch_bounds__(kZThreads, 2)
    gemm_dmma_tma_z_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           double2* __restrict__ C, long long sc, long long ldc, int m, int n, int k, int tiles_m,
                           int tiles_n, double2 alpha, double2 beta, int a_grouped, int b_grouped) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr bool CONJ_A = (OPA == BLB200_H), CONJ_B = (OPB == BLB200_H);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kZStageBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const int item = (int)(tile / tiles_per_item);
  const int rem = (int)(tile - (long long)item * tiles_per_item);
  const int m0 = (rem % tiles_m) * kBM, n0 = (rem / tiles_m) * kBN;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // Programmatic dependent launch: the next kernel's first CTAs may take their places while this
  // grid drains; nothing here touches global memory before every earlier grid has finished.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int KT = (k + kZBK - 1) / kZBK;
  auto issue = [&](int s, int kt) {  // one thread; map coordinates along a complex dimension count doubles
    mbar_arrive_expect_tx(&full_bar[s], kZStageBytes);
#pragma unroll
    for (int sub = 0; sub < kZSubs; ++sub) {
      unsigned char* st = smem + (size_t)s * kZStageBytes + (size_t)sub * kStageBytes;
      const int k0 = kt * kZBK + 8 * sub;  // sub-tiles wholly past k are zero-filled by the maps' bounds
      if (AK) {
        tma_load_3d(st, &map_a, 2 * k0, m0, item, &full_bar[s]);
      } else if (a_grouped) {
        tma_load_4d(st, &map_a, 0, k0, m0 >> 3, item, &full_bar[s]);
      } else {
#pragma unroll
        for (int b = 0; b < 8; ++b) tma_load_3d(st + b * 1024, &map_a, 2 * (m0 + 8 * b), k0, item, &full_bar[s]);
      }
      if (BKM) {
        tma_load_3d(st + kOperandBytes, &map_b, 2 * k0, n0, item, &full_bar[s]);
      } else if (b_grouped) {
        tma_load_4d(st + kOperandBytes, &map_b, 0, k0, n0 >> 3, item, &full_bar[s]);
      } else {
#pragma unroll
        for (int b = 0; b < 8; ++b) tma_load_3d(st + kOperandBytes + b * 1024, &map_b, 2 * (n0 + 8 * b), k0, item, &full_bar[s]);
      }
    }
  };
  if (tid == 0)
    for (int s = 0; s < kStages - 1 && s < KT; ++s) issue(s, s);

  double accr[4][2][2], acci[4][2][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) accr[i][j][0] = accr[i][j][1] = acci[i][j][0] = acci[i][j][1] = 0.0;

  const int a_base = z_fragment_base<AK>(32 * wm, g, t);
  const int b_base = z_fragment_base<BKM>(16 * wn, g, t);

  int issued = KT < kStages - 1 ? KT : kStages - 1;
  int kt = 0;
  bool lost = false;
  for (; kt < KT; ++kt) {
    const int s = kt % kStages;
    const bool ok = mbar_wait(&full_bar[s], (uint32_t)(kt / kStages) & 1u, kDmmaTmaWaitFull);
    if (__syncthreads_or(!ok)) {
      lost = true;
      break;
    }
    if (tid == 0 && issued < KT) {
      fence_async_smem();
      issue(issued % kStages, issued);
      ++issued;
    }
#pragma unroll
    for (int k4all = 0; k4all < kZBK / 4; ++k4all) {
      const int k4 = k4all & 1;
      const unsigned char* as = smem + (size_t)s * kZStageBytes + (size_t)(k4all >> 1) * kStageBytes;
      const unsigned char* bs = as + kOperandBytes;
      double2 af[4], bf[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        af[i] = *reinterpret_cast<const double2*>(as + z_fragment_offset<AK>(a_base, i, k4));
        if (CONJ_A) af[i].y = -af[i].y;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        bf[j] = *reinterpret_cast<const double2*>(bs + z_fragment_offset<BKM>(b_base, j, k4));
        if (CONJ_B) bf[j].y = -bf[j].y;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const double nai = -af[i].y;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          dmma(accr[i][j][0], accr[i][j][1], af[i].x, bf[j].x);
          dmma(accr[i][j][0], accr[i][j][1], nai, bf[j].y);
          dmma(acci[i][j][0], acci[i][j][1], af[i].x, bf[j].y);
          dmma(acci[i][j][0], acci[i][j][1], af[i].y, bf[j].x);
        }
      }
    }
  }
  if (lost) {
    if (tid == 0)
      for (int q = kt + 1; q < issued; ++q)
        mbar_wait_limit(&full_bar[q % kStages], (uint32_t)(q / kStages) & 1u, kDmmaTmaWaitFull, 1u << 12);
    return;
  }

  const bool beta_zero = beta.x == 0.0 && beta.y == 0.0;
  C += (long long)item * sc;
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = n0 + 16 * wn + 8 * j + perm_z(2 * t + e);
      if (col >= n) continue;
      double2* ccol = C + (long long)col * ldc;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m0 + 32 * wm + 8 * i + perm_z(g);
        if (row >= m) continue;
        ccol[row] = epilogue<double2>(alpha, make_double2(accr[i][j][e], acci[i][j][e]), beta, beta_zero, ccol + row);
      }
    }
}

template <int OPA, int OPB>
int launch_op_z(const GemmParams& p, cudaStream_t stream) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  const size_t smem = (size_t)kStages * kZStageBytes + kStages * sizeof(uint64_t) + 1024;
  const int tiles_m = (p.m + kBM - 1) / kBM, tiles_n = (p.n + kBN - 1) / kBN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  alignas(64) CUtensorMap map_a, map_b;
  static thread_local OperandMapCache maps;
  const int a_rows = AK ? p.k : p.m, a_cols = AK ? p.m : p.k;
  const int b_rows = BKM ? p.k : p.n, b_cols = BKM ? p.n : p.k;
  static std::atomic<int> grouped_ok{1};
  int a_kind = AK ? kMapKMajor : (a_rows % 8 == 0 && grouped_ok.load() ? kMapRowGroups : kMapRows16);
  int b_kind = BKM ? kMapKMajor : (b_rows % 8 == 0 && grouped_ok.load() ? kMapRowGroups : kMapRows16);
  // rows, ld and strides in doubles; M-major boxes span 8 k, a grouped copy takes 8 groups of 8 rows
  int rc = maps.get(&map_a, p.a, 2LL * a_rows, a_cols, 2 * p.lda, 2 * p.sa, p.batch, a_kind, 8, 8);
  if (rc != BLB200_OK && a_kind == kMapRowGroups) {
    grouped_ok.store(0);
    a_kind = kMapRows16;
    if (b_kind == kMapRowGroups) b_kind = kMapRows16;
    rc = maps.get(&map_a, p.a, 2LL * a_rows, a_cols, 2 * p.lda, 2 * p.sa, p.batch, a_kind, 8, 8);
  }
  if (rc != BLB200_OK) return rc;
  rc = maps.get(&map_b, p.b, 2LL * b_rows, b_cols, 2 * p.ldb, 2 * p.sb, p.batch, b_kind, 8, 8);
  if (rc != BLB200_OK && b_kind == kMapRowGroups) {
    grouped_ok.store(0);
    b_kind = kMapRows16;
    rc = maps.get(&map_b, p.b, 2LL * b_rows, b_cols, 2 * p.ldb, 2 * p.sb, p.batch, b_kind, 8, 8);
  }
  if (rc != BLB200_OK) return rc;
  auto kern = gemm_dmma_tma_z_kernel<OPA, OPB>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)total);
  cfg.blockDim = dim3(kZThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (double2*)p.c, (long long)p.sc, (long long)p.ldc, p.m, p.n, p.k,
                                 tiles_m, tiles_n, make_double2(p.alpha[0], p.alpha[1]), make_double2(p.beta[0], p.beta[1]),
                                 a_kind == kMapRowGroups ? 1 : 0, b_kind == kMapRowGroups ? 1 : 0);
}

}  // namespace

int dmma_tma_device_status(int* out) { return read_device_status_word(out); }
int dmma_tma_device_status_clear() { return clear_device_status_word(); }

bool dmma_tma_supported(const GemmParams& p, int dtype) {
  if (dtype != BLB200_D && dtype != BLB200_Z) return false;
  if (p.k < 1 || (p.m <= 32 && p.n <= 32)) return false;
  if (has_hints(p) || p.splits > 1) return false;
  // tensor maps need 16-byte aligned bases and strides for A and B (always true of element-aligned
  // complex operands); C is stored element by element
  const long long es = dtype == BLB200_D ? 8 : 16;
  auto map_ok = [es](const void* base, long long ld, long long stride) {
    return reinterpret_cast<uintptr_t>(base) % 16 == 0 && (ld * es) % 16 == 0 && (stride * es) % 16 == 0;
  };
  if (!map_ok(p.a, p.lda, p.sa) || !map_ok(p.b, p.ldb, p.sb)) return false;
  if (reinterpret_cast<uintptr_t>(p.c) % (uintptr_t)es != 0) return false;
  if (p.batch > 1 && (p.sa <= 0 || p.sb <= 0)) return false;  // a broadcast operand has no tensor-map stride
  return encode_tiled_fn() != nullptr;
}

int launch_dmma_tma(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!dmma_tma_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  int rc = BLB200_E_INTERNAL;
  if (dtype == BLB200_D) {
#define BLB_OP(A_, B_) \
  if (p.op_a == A_ && p.op_b == B_) rc = launch_op<A_, B_>(p, stream);
    BLB_OP(0, 0) BLB_OP(0, 1) BLB_OP(1, 0) BLB_OP(1, 1)
#undef BLB_OP
  } else {
#define BLB_OP(A_, B_) \
  if (p.op_a == A_ && p.op_b == B_) rc = launch_op_z<A_, B_>(p, stream);
    BLB_OP(0, 0) BLB_OP(0, 1) BLB_OP(0, 2) BLB_OP(1, 0) BLB_OP(1, 1) BLB_OP(1, 2) BLB_OP(2, 0) BLB_OP(2, 1) BLB_OP(2, 2)
#undef BLB_OP
  }
  if (rc == BLB200_OK) note_launch("dmma_tma");
  return rc;
}

}  // namespace blb200
