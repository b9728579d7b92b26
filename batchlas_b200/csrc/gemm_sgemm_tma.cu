// Large float GEMM for all four op pairs, fed by TMA (A^T B has a kernel of its own further down): the long-k form of the
// 128 x 128 x 32 float tile.  Four warps per CTA, each owning all 128 rows and 32 columns of the tile
// with a 16 x 8 register block per lane (64 packed FP32 FMAs, fma.rn.f32x2, per 8 duplicated B values
// and 6 fragment reads of 16 bytes — half the non-FMA instructions per FMA of the 8 x 8 block), two
// CTAs per SM.  The operand tiles arrive by cp.async.bulk.tensor from 3-D tensor maps (rows x
// columns x batch item) over the caller's column-major storage and complete on one mbarrier per
// stage; no thread computes a copy address and the tensor map's bounds zero-fill every edge.  There
// is no producer warp and no CTA-wide barrier in the main loop: a warp that has finished a stage
// counts itself off it (release/acquire counter in shared memory) and the warp that leaves last
// issues the stage's next copies, so the four warps drift apart by up to a stage instead of meeting
// after every k-tile.
//
// Stage layout (32 KiB, three stages):
//   A  [32 k][128 m]   one box 128 x 32, rows of 512 bytes, no swizzle: a lane reads rows
//                      4ti + 32g .. +3 (g = 0..3) as four 16-byte chunks per k, already the row pairs
//                      the packed FMA wants.
//   B  op N (K-major in memory): [128 n][32 k], one box 32 x 128 with the 128-byte swizzle (16-byte
//                      chunk index XOR (n & 7)); a lane owns columns tj + 4c of its warp's 32.
//      op T (N-major in memory): [32 k][128 n], one box 128 x 32, no swizzle; a lane owns columns
//                      8tj .. 8tj + 7.
// The products and their order per output element are those of the cp.async kernel of the same tile
// (k ascending, one FMA per k): the same bits.
// Op pair TT runs as the NN problem of the transposed product (C^T = B_stored A_stored: B as stored has
// n fastest, A as stored k fastest), and the epilogue transposes the tile through shared memory into
// whole stored columns of C.  For TN neither operand has an output dimension fastest, so no operand
// comes in the row pairs the packed FMA wants: sgemm_tma_tn_kernel pairs along k instead.
//
// Preconditions (sgemm_tma_supported): float, plain gemm (no structure hints, per-item dims
// or split-K), A, B and C 16-byte aligned (base, ld and batch stride), positive batch strides.  No
// load with cluster multicast is used; the maps cover this GPU's memory only.  Every wait is bounded;
// a wait that runs out records code 501, and the CTA leaves as a unit after giving the copies it
// still has in flight a bounded chance to land.
#include <string.h>

#include "common.cuh"
#include "tensor_map.cuh"

namespace blb200 {
namespace {

enum WaitCode { kSgemmTmaWaitFull = 501 };

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, THREADS = 128, WARPS = THREADS / 32;
constexpr int A_STAGE = BK * BM * 4, B_STAGE = BK * BN * 4, STAGE = A_STAGE + B_STAGE;  // 16 + 16 KiB
constexpr int RG = 4;  // groups of 4 rows per lane

// OUT_T: the kernel computes the transpose of the caller's C (see the file comment on op pair TT): its rows
// are the caller's columns, and the epilogue transposes the tile through shared memory.
template <bool B_KMAJOR, bool OUT_T = false>
__global__ void __launch_bounds__(THREADS, 2)
    sgemm_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     float* __restrict__ C, long long sc, long long ldc, int m, int n, int k, int tiles_m, int tiles_n,
                     float alpha, float beta) {
  extern __shared__ unsigned char smem_raw[];
  // the swizzle is a function of the shared-memory address: tiles must start on 1024-byte boundaries
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE);
  uint32_t* left = reinterpret_cast<uint32_t*>(full_bar + STAGES);   // warps that have left each stage, ever
  int* issued_kt = reinterpret_cast<int*>(left + STAGES);            // last k-tile whose copies went into each stage
  int* dead = issued_kt + STAGES;                                    // a wait ran out somewhere in this CTA

  const int tid = threadIdx.x, wn = tid >> 5, lane = tid & 31;
  const int ti = lane & 7, tj = lane >> 3;

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const int item = (int)(tile / tiles_per_item);
  const int rem = (int)(tile - (long long)item * tiles_per_item);
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      left[s] = 0;
      issued_kt[s] = -1;
    }
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // Programmatic dependent launch: the next kernel's first CTAs may take their places while this
  // grid drains; nothing here touches global memory before every earlier grid has finished.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  C += (long long)item * sc;
  if (beta != 0.f) {  // the epilogue reads this tile of C: ask L2 for its 128-byte lines now (one thread per stored column)
    const int col = (OUT_T ? m0 : n0) + tid, first_row = OUT_T ? n0 : m0;
    if (col < (OUT_T ? m : n)) {
      const float* pc = C + (long long)col * ldc + first_row;
#pragma unroll
      for (int l = 0; l < BM / 32; ++l)
        if (first_row + 32 * l < (OUT_T ? n : m)) asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + 32 * l));
    }
  }

  const int KT = (k + BK - 1) / BK;
  auto issue = [&](int s, int kt) {  // one thread: the copies of k-tile kt into stage s
    unsigned char* st = smem + (size_t)s * STAGE;
    const int k0 = kt * BK;
    issued_kt[s] = kt;
    mbar_arrive_expect_tx(&full_bar[s], STAGE);
    tma_load_3d(st, &map_a, m0, k0, item, &full_bar[s]);
    if (B_KMAJOR) {
      tma_load_3d(st + A_STAGE, &map_b, k0, n0, item, &full_bar[s]);
    } else {
      tma_load_3d(st + A_STAGE, &map_b, n0, k0, item, &full_bar[s]);
    }
  };
  if (tid == 0)
    for (int s = 0; s < STAGES && s < KT; ++s) issue(s, s);

  uint64_t accp[RG * 16];  // [row pair rp][col c]: rows (2rp, 2rp+1) of the lane's 16, column c of its 8
#pragma unroll
  for (int i = 0; i < RG * 16; ++i) accp[i] = 0ull;

  bool lost = false;
  for (int kt = 0; kt < KT; ++kt) {
    const int s = kt % STAGES;
    const bool ok = mbar_wait(&full_bar[s], (uint32_t)(kt / STAGES) & 1u, kSgemmTmaWaitFull);
    if (!__all_sync(0xffffffffu, ok)) {
      lost = true;
      break;
    }
    const unsigned char* st = smem + (size_t)s * STAGE;
    const ulonglong2* As2 = reinterpret_cast<const ulonglong2*>(st) + ti;
    const float4* Bs4 = reinterpret_cast<const float4*>(st + A_STAGE);

    if (B_KMAJOR) {
      float bf[2][8][4];  // [buffer][col][kk]
      auto load_bf = [&](int kc, float (&dst)[8][4]) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int j = wn * 32 + tj + 4 * c;
          const float4 v = Bs4[j * 8 + (kc ^ (j & 7))];
          dst[c][0] = v.x; dst[c][1] = v.y; dst[c][2] = v.z; dst[c][3] = v.w;
        }
      };
      load_bf(0, bf[0]);
#pragma unroll
      for (int kc = 0; kc < BK / 4; ++kc) {
        if (kc + 1 < BK / 4) load_bf(kc + 1, bf[(kc + 1) & 1]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint64_t a2[2 * RG];
#pragma unroll
          for (int g = 0; g < RG; ++g) {
            const ulonglong2 v = As2[(4 * kc + kk) * 32 + 8 * g];
            a2[2 * g] = v.x;
            a2[2 * g + 1] = v.y;
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint64_t bd = dup2(bf[kc & 1][c][kk]);
#pragma unroll
            for (int rp = 0; rp < 2 * RG; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
          }
        }
      }
    } else {
#pragma unroll 8
      for (int kq = 0; kq < BK; ++kq) {
        const float4 v0 = Bs4[kq * 32 + wn * 8 + 2 * tj];
        const float4 v1 = Bs4[kq * 32 + wn * 8 + 2 * tj + 1];
        const float bv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        uint64_t a2[2 * RG];
#pragma unroll
        for (int g = 0; g < RG; ++g) {
          const ulonglong2 v = As2[kq * 32 + 8 * g];
          a2[2 * g] = v.x;
          a2[2 * g + 1] = v.y;
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint64_t bd = dup2(bv[c]);
#pragma unroll
          for (int rp = 0; rp < 2 * RG; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
        }
      }
    }

    // leave the stage; the last warp out sends for the k-tile that will live here next
    __syncwarp();
    if (lane == 0) {
      const uint32_t before = smem_add_acq_rel(&left[s], 1u);
      if ((before & (WARPS - 1)) == WARPS - 1 && kt + STAGES < KT) {
        fence_async_smem();
        issue(s, kt + STAGES);
      }
    }
  }
  if (lost && lane == 0) atomicExch(dead, 1);
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(dead)) {
    // A copy never arrived (recorded in the status word).  Do not leave while copies may still land
    // in this CTA's shared memory: give the last copy sent into each stage a short, bounded chance.
    if (tid == 0)
      for (int s = 0; s < STAGES; ++s) {
        const int q = issued_kt[s];
        if (q >= 0) mbar_wait_limit(&full_bar[s], (uint32_t)(q / STAGES) & 1u, kSgemmTmaWaitFull, 1u << 12);
      }
    return;
  }

  const bool beta_zero = beta == 0.f;
  if constexpr (OUT_T) {
    // The tile in hand is the transpose of the caller's: lay it down in the stage buffers (idle now; every
    // copy was waited for by every warp) as [kernel row r][kernel column c], which is one stored column
    // of the caller's C per r, and write those out whole: 512 contiguous bytes per warp step, 16 per
    // lane, eight rows' prior values requested before the first of them is stored.
    constexpr int PITCH = BN + 4;  // floats; keeps every row 16-byte aligned
    float* S = reinterpret_cast<float*>(smem);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int cl = wn * 32 + tj + 4 * c;
#pragma unroll
      for (int g = 0; g < RG; ++g) {
        float o[4];
        unpack2(accp[(2 * g) * 8 + c], o[0], o[1]);
        unpack2(accp[(2 * g + 1) * 8 + c], o[2], o[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) S[(32 * g + 4 * ti + e) * PITCH + cl] = o[e];
      }
    }
    __syncthreads();
    const int urow = n0 + 4 * lane;  // caller's row = kernel column
#pragma unroll 1
    for (int rb = 0; rb < 32; rb += 8) {
      float4 pr[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        pr[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int ucol = m0 + wn * 32 + rb + q;  // caller's column = kernel row
        if (beta_zero || ucol >= m || urow >= n) continue;
        const float* pc = C + (long long)ucol * ldc + urow;
        if (urow + 4 <= n) {
          pr[q] = *reinterpret_cast<const float4*>(pc);
        } else {
          pr[q].x = pc[0];
          if (urow + 1 < n) pr[q].y = pc[1];
          if (urow + 2 < n) pr[q].z = pc[2];
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int r = wn * 32 + rb + q, ucol = m0 + r;
        if (ucol >= m || urow >= n) continue;
        const float4 v = *reinterpret_cast<const float4*>(S + r * PITCH + 4 * lane);
        float4 out = make_float4(alpha * v.x, alpha * v.y, alpha * v.z, alpha * v.w);
        if (!beta_zero) {
          out.x = fmaf(beta, pr[q].x, out.x);
          out.y = fmaf(beta, pr[q].y, out.y);
          out.z = fmaf(beta, pr[q].z, out.z);
          out.w = fmaf(beta, pr[q].w, out.w);
        }
        float* pc = C + (long long)ucol * ldc + urow;
        if (urow + 4 <= n) {
          *reinterpret_cast<float4*>(pc) = out;
        } else {
          pc[0] = out.x;
          if (urow + 1 < n) pc[1] = out.y;
          if (urow + 2 < n) pc[2] = out.z;
        }
      }
    }
    return;
  }

  // Epilogue: column by column of the lane's eight, the prior values of the next column requested
  // before the current one is stored (C's loads and stores may alias as far as the compiler knows, so
  // left to itself it would finish each column's round trip to L2 before starting the next).
  auto col_of = [&](int c) { return n0 + wn * 32 + (B_KMAJOR ? (tj + 4 * c) : (8 * tj + c)); };
  auto load_prior = [&](int c, float4 (&dst)[RG]) {
    const int col = col_of(c);
#pragma unroll
    for (int g = 0; g < RG; ++g) {
      dst[g] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int row = m0 + 32 * g + 4 * ti;
      if (col >= n || row >= m) continue;
      const float* pc = C + (long long)col * ldc + row;
      if (row + 4 <= m) {
        dst[g] = *reinterpret_cast<const float4*>(pc);
      } else {
        dst[g].x = pc[0];
        if (row + 1 < m) dst[g].y = pc[1];
        if (row + 2 < m) dst[g].z = pc[2];
      }
    }
  };
  float4 prior[2][RG];
  if (!beta_zero) load_prior(0, prior[0]);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    if (!beta_zero && c + 1 < 8) load_prior(c + 1, prior[(c + 1) & 1]);
    const int col = col_of(c);
    if (col >= n) continue;
    float* ccol = C + (long long)col * ldc;
#pragma unroll
    for (int g = 0; g < RG; ++g) {
      const int row = m0 + 32 * g + 4 * ti;
      if (row >= m) continue;
      float o[4];
      unpack2(accp[(2 * g) * 8 + c], o[0], o[1]);
      unpack2(accp[(2 * g + 1) * 8 + c], o[2], o[3]);
      float4 out = make_float4(alpha * o[0], alpha * o[1], alpha * o[2], alpha * o[3]);
      if (!beta_zero) {
        const float4 pr = prior[c & 1][g];
        out.x = fmaf(beta, pr.x, out.x);
        out.y = fmaf(beta, pr.y, out.y);
        out.z = fmaf(beta, pr.z, out.z);
        out.w = fmaf(beta, pr.w, out.w);
      }
      if (row + 4 <= m) {
        *reinterpret_cast<float4*>(ccol + row) = out;
      } else {
        ccol[row] = out.x;
        if (row + 1 < m) ccol[row + 1] = out.y;
        if (row + 2 < m) ccol[row + 2] = out.z;
      }
    }
  }
}

// ---- A^T B: both operands have k fastest ------------------------------------------------------------
// Neither operand offers pairs along an output dimension, but both offer pairs along k: a 64-bit
// register (a[i][k], a[i][k+1]) times (b[k][j], b[k+1][j]) accumulates the even-k and the odd-k partial
// sum of c[i][j] side by side, with nothing to duplicate; the two halves are added once, in the
// epilogue.  (So the sum is ordered as even k ascending plus odd k ascending, not k ascending: within
// the parity bound, not bit-identical to the other float kernels.)  An 8 x 8 block per lane is 128
// accumulator registers; per four k a lane reads eight 16-byte fragments of each operand for 128
// packed FMAs.  CTA 128 x 128 x 32 with 8 warps as 2 (m) x 4 (n), one CTA per SM, four stages.
//   A  [128 m][32 k], B [128 n][32 k]: one box 32 x 128 each with the 128-byte swizzle (16-byte chunk
//      index XOR (row & 7)).  A lane owns rows ti + 8i of its warp's 64 — the eight lanes of a
//      quarter-warp differ in (row & 7), so a fragment request covers all banks once — and columns
//      tj + 4j of its warp's 32 (one address per quarter-warp).
constexpr int TN_THREADS = 256, TN_WARPS = TN_THREADS / 32, TN_STAGES = 4;

__global__ void __launch_bounds__(TN_THREADS, 1)
    sgemm_tma_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        float* __restrict__ C, long long sc, long long ldc, int m, int n, int k, int tiles_m, int tiles_n,
                        float alpha, float beta) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)TN_STAGES * STAGE);
  uint32_t* left = reinterpret_cast<uint32_t*>(full_bar + TN_STAGES);
  int* issued_kt = reinterpret_cast<int*>(left + TN_STAGES);
  int* dead = issued_kt + TN_STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 1, wn = warp >> 1;
  const int ti = lane & 7, tj = lane >> 3;

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const int item = (int)(tile / tiles_per_item);
  const int rem = (int)(tile - (long long)item * tiles_per_item);
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;

  if (tid == 0) {
    for (int s = 0; s < TN_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      left[s] = 0;
      issued_kt[s] = -1;
    }
    *dead = 0;
    mbar_fence_init();
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  C += (long long)item * sc;
  if (beta != 0.f && tid < BN) {  // the epilogue reads this tile of C: ask L2 for its 128-byte lines now
    const int col = n0 + tid;
    if (col < n) {
      const float* pc = C + (long long)col * ldc + m0;
#pragma unroll
      for (int l = 0; l < BM / 32; ++l)
        if (m0 + 32 * l < m) asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + 32 * l));
    }
  }

  const int KT = (k + BK - 1) / BK;
  auto issue = [&](int s, int kt) {
    unsigned char* st = smem + (size_t)s * STAGE;
    issued_kt[s] = kt;
    mbar_arrive_expect_tx(&full_bar[s], STAGE);
    tma_load_3d(st, &map_a, kt * BK, m0, item, &full_bar[s]);
    tma_load_3d(st + A_STAGE, &map_b, kt * BK, n0, item, &full_bar[s]);
  };
  if (tid == 0)
    for (int s = 0; s < TN_STAGES && s < KT; ++s) issue(s, s);

  uint64_t acc[8][8];  // [row i][col j]: (even-k sum, odd-k sum) of element (ti + 8i, tj + 4j) of the warp tile
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0ull;

  const int a_row0 = wm * 64 + ti, b_col0 = wn * 32 + tj;
  bool lost = false;
  for (int kt = 0; kt < KT; ++kt) {
    const int s = kt % TN_STAGES;
    const bool ok = mbar_wait(&full_bar[s], (uint32_t)(kt / TN_STAGES) & 1u, kSgemmTmaWaitFull);
    if (!__all_sync(0xffffffffu, ok)) {
      lost = true;
      break;
    }
    const ulonglong2* As2 = reinterpret_cast<const ulonglong2*>(smem + (size_t)s * STAGE);
    const ulonglong2* Bs2 = reinterpret_cast<const ulonglong2*>(smem + (size_t)s * STAGE + A_STAGE);
#pragma unroll
    for (int kc = 0; kc < BK / 4; ++kc) {
      ulonglong2 af[8], bf[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = a_row0 + 8 * i;
        af[i] = As2[r * 8 + (kc ^ (r & 7))];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = b_col0 + 4 * j;
        bf[j] = Bs2[c * 8 + (kc ^ (c & 7))];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) ffma2(acc[i][j], af[i].x, bf[j].x);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) ffma2(acc[i][j], af[i].y, bf[j].y);
    }
    __syncwarp();
    if (lane == 0) {
      const uint32_t before = smem_add_acq_rel(&left[s], 1u);
      if ((before & (TN_WARPS - 1)) == TN_WARPS - 1 && kt + TN_STAGES < KT) {
        fence_async_smem();
        issue(s, kt + TN_STAGES);
      }
    }
  }
  if (lost && lane == 0) atomicExch(dead, 1);
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(dead)) {
    if (tid == 0)
      for (int s = 0; s < TN_STAGES; ++s) {
        const int q = issued_kt[s];
        if (q >= 0) mbar_wait_limit(&full_bar[s], (uint32_t)(q / TN_STAGES) & 1u, kSgemmTmaWaitFull, 1u << 12);
      }
    return;
  }

  // Epilogue: a quarter-warp holds 8 consecutive rows of a column (one 32-byte sector); the prior values
  // of the next column are requested before the current one is stored.
  const bool beta_zero = beta == 0.f;
  auto load_prior = [&](int j, float (&dst)[8]) {
    const int col = n0 + b_col0 + 4 * j;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = m0 + a_row0 + 8 * i;
      dst[i] = (col < n && row < m) ? C[(long long)col * ldc + row] : 0.f;
    }
  };
  float prior[2][8];
  if (!beta_zero) load_prior(0, prior[0]);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (!beta_zero && j + 1 < 8) load_prior(j + 1, prior[(j + 1) & 1]);
    const int col = n0 + b_col0 + 4 * j;
    if (col >= n) continue;
    float* ccol = C + (long long)col * ldc;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = m0 + a_row0 + 8 * i;
      if (row >= m) continue;
      float even, odd;
      unpack2(acc[i][j], even, odd);
      float out = alpha * (even + odd);
      if (!beta_zero) out = fmaf(beta, prior[j & 1][i], out);
      ccol[row] = out;
    }
  }
}

// 3-D map (rows, cols, items) over a column-major float operand, zero fill past the bounds.
//   k_major: box 32 x 128 (32 k of 128 columns), 128-byte swizzle
//   else:    box 128 x 32 (128 rows at 32 k), no swizzle
int make_float_map(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, long long stride, int batch,
                   bool k_major) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return BLB200_E_INTERNAL;
  const cuuint64_t items = (cuuint64_t)(batch > 0 ? batch : 1);
  const long long item_stride = batch > 1 ? stride : ld * (long long)cols;
  const cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)cols, items};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)item_stride * 4};
  const cuuint32_t box[3] = {k_major ? 32u : 128u, k_major ? 128u : 32u, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, k_major ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BLB200_OK : BLB200_E_INTERNAL;
}

// Tensor maps are pure functions of (base, shape, ld, stride, batch, orientation): a small per-thread
// cache saves the driver call when the same operand is multiplied again.
struct FloatMapCache {
  struct Entry {
    const void* base = nullptr;
    long long rows = 0, ld = 0, stride = 0;
    int cols = 0, batch = 0, k_major = 0;
    CUtensorMap map;
  };
  static constexpr int kEntries = 8;
  Entry e[kEntries];
  int next = 0;
  int get(CUtensorMap* out, const void* base, long long rows, int cols, long long ld, long long stride, int batch,
          bool k_major) {
    for (int i = 0; i < kEntries; ++i)
      if (e[i].base == base && e[i].rows == rows && e[i].cols == cols && e[i].ld == ld && e[i].stride == stride &&
          e[i].batch == batch && e[i].k_major == (int)k_major) {
        memcpy(out, &e[i].map, sizeof(CUtensorMap));
        return BLB200_OK;
      }
    Entry& slot = e[next];
    const int rc = make_float_map(&slot.map, base, rows, cols, ld, stride, batch, k_major);
    if (rc != BLB200_OK) {
      slot.base = nullptr;
      return rc;
    }
    slot.base = base; slot.rows = rows; slot.cols = cols; slot.ld = ld; slot.stride = stride;
    slot.batch = batch; slot.k_major = (int)k_major;
    memcpy(out, &slot.map, sizeof(CUtensorMap));
    next = (next + 1) % kEntries;
    return BLB200_OK;
  }
};

// OUT_T (op pair TT): C^T = op(B)^T op(A)^T = B_stored A_stored, which is the NN problem on swapped
// operands — B as stored (n x k, n fastest) is the M-major operand, A as stored (k x m, k fastest) the
// K-major one — with the kernel's m and n being the caller's n and m.
template <bool B_KMAJOR, bool OUT_T = false>
int launch_op(const GemmParams& q, cudaStream_t stream) {
  GemmParams p = q;
  if (OUT_T) {
    p.a = q.b; p.lda = q.ldb; p.sa = q.sb;
    p.b = q.a; p.ldb = q.lda; p.sb = q.sa;
    p.m = q.n; p.n = q.m;
  }
  constexpr size_t smem = (size_t)STAGES * STAGE + 1024 + 128;
  const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  alignas(64) CUtensorMap map_a, map_b;
  static thread_local FloatMapCache maps;
  int rc = maps.get(&map_a, p.a, p.m, p.k, p.lda, p.sa, p.batch, false);
  if (rc != BLB200_OK) return rc;
  rc = B_KMAJOR ? maps.get(&map_b, p.b, p.k, p.n, p.ldb, p.sb, p.batch, true)
                : maps.get(&map_b, p.b, p.n, p.k, p.ldb, p.sb, p.batch, false);
  if (rc != BLB200_OK) return rc;
  auto kern = sgemm_tma_kernel<B_KMAJOR, OUT_T>;
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
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (float*)p.c, (long long)p.sc, (long long)p.ldc, p.m, p.n, p.k,
                                 tiles_m, tiles_n, (float)p.alpha[0], (float)p.beta[0]);
}

int launch_tn(const GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)TN_STAGES * STAGE + 1024 + 128;
  const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  alignas(64) CUtensorMap map_a, map_b;
  static thread_local FloatMapCache maps;
  int rc = maps.get(&map_a, p.a, p.k, p.m, p.lda, p.sa, p.batch, true);
  if (rc != BLB200_OK) return rc;
  rc = maps.get(&map_b, p.b, p.k, p.n, p.ldb, p.sb, p.batch, true);
  if (rc != BLB200_OK) return rc;
  auto kern = sgemm_tma_tn_kernel;
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
  cfg.blockDim = dim3(TN_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (float*)p.c, (long long)p.sc, (long long)p.ldc, p.m, p.n, p.k,
                                 tiles_m, tiles_n, (float)p.alpha[0], (float)p.beta[0]);
}

}  // namespace

bool sgemm_tma_supported(const GemmParams& p, int dtype) {
  if (dtype != BLB200_S) return false;
  if (has_hints(p) || p.splits > 1) return false;
  if (p.m < 64 || p.n < 64 || p.k < 1) return false;
  if (p.batch > 1 && (p.sa <= 0 || p.sb <= 0)) return false;  // a broadcast operand has no item stride to map
  if (!operands_aligned_to(p, 4, 16)) return false;
  return tiled_supported(p, dtype);
}

int launch_sgemm_tma(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!sgemm_tma_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const int rc = (p.op_a != BLB200_N) ? (p.op_b == BLB200_N ? launch_tn(p, stream) : launch_op<true, true>(p, stream))
                                      : (p.op_b == BLB200_N) ? launch_op<true>(p, stream) : launch_op<false>(p, stream);
  if (rc == BLB200_OK) note_launch("sgemm_tma");
  return rc;
}

int sgemm_tma_device_status(int* out) { return read_device_status_word(out); }
int sgemm_tma_device_status_clear() { return clear_device_status_word(); }

}  // namespace blb200
