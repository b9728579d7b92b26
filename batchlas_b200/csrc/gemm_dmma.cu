// FP64 tensor-core tiles for double and complex<double>: mma.sync m8n8k4 (DMMA) fed from the same
// multi-stage ring of 16-byte asynchronous copies as the FFMA/DFMA tiled kernel.
//
// Why DMMA: on B200 the DMMA issue rate measured 37.2 TFLOP/s against 33.6 for DFMA, and a DMMA
// fragment load moves one double per lane for 8 FMAs per lane, where the register-blocked DFMA
// tile needs 12 doubles for 32 FMAs — the DFMA kernel is bound by shared-memory-to-register
// bandwidth (about 78 % of it busy for 61 % of the FP64 pipe), the DMMA kernel is not.  DMMA
// multiplies and accumulates in full binary64, so results stay within the same bound.
//
// Layout.  Operands stay in their stored orientation, laid out so that the 16 lanes of a half-warp
// request (4 fragment rows x 4 k) fall into 16 different 8-byte bank pairs:
//   M-major A (op N):   stage rows are k, BM doubles each, pitched 32 bytes past their length;
//                       fragment (m = g, k = t) at [k][m]
//   K-major A (op T/C): stage rows are m, BK doubles each.  Real double: rows of exactly 128 bytes
//                       whose four 32-byte groups (4 k each) are stored at group index
//                       (k / 4) ^ (row & 3) — no padding, so a stage is 8 KiB and four CTAs fit an
//                       SM for every op pair (with padded rows TN needed 61 KiB per CTA and only
//                       three fitted).  Complex: rows pitched 64 bytes past their length.
//   (g = lane >> 2, t = lane & 3; B likewise with n in place of m.)
// A warp owns a 32 x 32 block of C as 4 x 4 DMMA tiles (16 accumulator pairs); a CTA of 4 warps
// owns 64 x 64, four CTAs share an SM.  Complex operands keep (re, im) interleaved, one 16-byte fragment load per lane,
// and each complex tile product is four real DMMAs; conjugation flips the sign of the imaginary
// fragment in registers.
//
// Preconditions are those of the tiled kernel: element-aligned operands.  16-byte aligned bases, ld
// and stride take 16-byte copies (AL = true); a double operand that is only 8-byte aligned (a slice
// with an odd offset, ld = 257) is copied element by element into the same stage layout
// (AL = false).  Edges are zero-filled on load and predicated on store.
#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// Bytes added to every stage row.  A request must spread its fragment rows over all banks: 4 rows
// of 32 bytes (double, half-warp of 64-bit loads; complex M-major, quarter-warp of 4 k-rows x 2
// elements) want a 32-byte shift per row, 2 rows of 64 bytes (complex K-major) a 64-byte shift.
__host__ __device__ constexpr int pad_for(int es, bool kmajor) { return kmajor ? (es == 16 ? 64 : 0) : 32; }

// Asynchronous copy of one operand tile into a pitched stage.  ES = element bytes (8 or 16).
template <int ES, int BMN, int BK, int THREADS, bool KMAJOR, bool AL = true>
__device__ __forceinline__ void load_tile_pitched(unsigned char* smem, const unsigned char* __restrict__ base,
                                                  long long ld, int MN0, int MN, int k0, int K, int tid) {
  constexpr int V = 16 / ES;  // elements per 16-byte chunk
  if constexpr (!KMAJOR && !AL && ES == 8) {
    // A stage row is one stored column: BMN consecutive doubles that may start on an odd 8-byte
    // boundary.  Copy the 16-byte aligned superset of the run with 16-byte copies (one more chunk
    // than an aligned row; it fits the row's 32 bytes of padding) and let the fragment reads of that
    // row start 8 bytes further in (row_shift_bytes below: a per-lane constant).  The 8 bytes in front
    // of a shifted row are never read; src-size stops every copy at the row's last valid element.
    constexpr int CPR = BMN / 2 + 1, PITCH = BMN * ES + pad_for(ES, false);
    const unsigned char* aligned_dummy = reinterpret_cast<const unsigned char*>(reinterpret_cast<uintptr_t>(base) & ~(uintptr_t)15);
    const int left = MN - MN0;  // valid elements of a tile row (may exceed BMN)
    // THREADS / BK threads share a row and take every (THREADS / BK)-th chunk of it (no division by 33)
    constexpr int TPR = THREADS / BK;
    static_assert(THREADS % BK == 0, "whole thread groups per stage row");
    const int kk = tid / TPR, j0 = tid % TPR;
    const int gk = k0 + kk;
    const unsigned char* row = base + ((long long)gk * ld + MN0) * ES;
    const int sh = (int)(reinterpret_cast<uintptr_t>(row) & 8u);
    unsigned char* drow = smem + (size_t)kk * PITCH;
#pragma unroll
    for (int j = j0; j < CPR; j += TPR) {
      const int e0 = 2 * j - (sh >> 3);  // this chunk holds tile elements e0 and e0 + 1
      int bytes = 0;
      if (gk < K && e0 < BMN) bytes = (e0 + 1 < left) ? 16 : (e0 < left ? 8 : 0);
      cp_async16(drow + (size_t)j * 16, bytes ? row - sh + 16 * j : aligned_dummy, bytes);
    }
    return;
  }
  if (!KMAJOR) {
    constexpr int CH_PER_ROW = BMN / V, CHUNKS = BK * CH_PER_ROW, PITCH = BMN * ES + pad_for(ES, false);
#pragma unroll
    for (int c = tid; c < CHUNKS; c += THREADS) {
      const int kk = c / CH_PER_ROW, mc = c % CH_PER_ROW;
      const int gk = k0 + kk, gm = MN0 + mc * V;
      int valid = (gk < K) ? (MN - gm) : 0;
      valid = valid < 0 ? 0 : (valid > V ? V : valid);
      const unsigned char* src = valid ? base + ((long long)gk * ld + gm) * ES : base;
      unsigned char* dst = smem + (size_t)kk * PITCH + (size_t)mc * 16;
      if constexpr (AL) {
        cp_async16(dst, src, valid * ES);
      } else {
        cp_async_chunk_widest<ES>(dst, src, valid);  // a warp copies one stored column: a 16-byte copy where that column is aligned
      }
    }
  } else {
    constexpr int CH_PER_ROW = BK / V, CHUNKS = BMN * CH_PER_ROW, PITCH = BK * ES + pad_for(ES, true);
#pragma unroll
    for (int c = tid; c < CHUNKS; c += THREADS) {
      const int r = c / CH_PER_ROW, kc = c % CH_PER_ROW;
      const int gmn = MN0 + r, gk = k0 + kc * V;
      int valid = (gmn < MN) ? (K - gk) : 0;
      valid = valid < 0 ? 0 : (valid > V ? V : valid);
      const unsigned char* src = valid ? base + ((long long)gmn * ld + gk) * ES : base;
      // real double: 32-byte group kc / 2 of row r lives at group (kc / 2) ^ (r & 3)
      unsigned char* dst = smem + (size_t)r * PITCH + (ES == 8 ? (size_t)((((kc >> 1) ^ (r & 3)) << 5) + ((kc & 1) << 4)) : (size_t)kc * 16);
      if constexpr (AL) {
        cp_async16(dst, src, valid * ES);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) cp_async_elem<ES>(dst + e * ES, e < valid ? src + e * ES : src, e < valid ? ES : 0);
      }
    }
  }
}

template <int ES, int BMN, int BK, bool KMAJOR>
__host__ __device__ constexpr int pitched_stage_bytes() {
  return KMAJOR ? BMN * (BK * ES + pad_for(ES, true)) : BK * (BMN * ES + pad_for(ES, false));
}

constexpr int kStagesD = 3, kStagesZ = 3;  // copy-ring depth; 4 gains ~1 % on NN/NT and costs the second CTA per SM on TN/TT

// ---- real double -------------------------------------------------------------------------------
// HINTS = false is the plain gemm; HINTS = true reads the structure hints of GemmParams (a separate
// instantiation, so that the plain kernel's code and register allocation stay what they were).
// WM x WN warps of 32 x 32 each; 16 / (WM * WN) CTAs per SM.
template <int OPA, int OPB, bool HINTS, int WM, int WN, bool AL = true>
__global__ void __launch_bounds__(32 * WM * WN, 16 / (WM * WN)) gemm_dmma_d_kernel(GemmParams p, int tiles_m, int tiles_n) {
  constexpr int BM = 32 * WM, BN = 32 * WN, BK = 16, STAGES = kStagesD, THREADS = 32 * WM * WN;
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr int A_STAGE = pitched_stage_bytes<8, BM, BK, AK>(), B_STAGE = pitched_stage_bytes<8, BN, BK, BKM>();
  constexpr int A_PITCH = AK ? BK * 8 + pad_for(8, true) : BM * 8 + pad_for(8, false);
  constexpr int B_PITCH = BKM ? BK * 8 + pad_for(8, true) : BN * 8 + pad_for(8, false);

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* As = smem;
  unsigned char* Bs = smem + (size_t)STAGES * A_STAGE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = warp % WM, wn = warp / WM;  // WM x WN warps, 32 x 32 each

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const long long vitem = tile / tiles_per_item;
  const int rem = (int)(tile - vitem * tiles_per_item);
  const SplitView sv = resolve_split(p, vitem);
  const long long item = sv.item;
  p.k = sv.k;
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;
  const unsigned char* A = (const unsigned char*)p.a + (item * p.sa + sv.a_off) * 8;
  const unsigned char* B = (const unsigned char*)p.b + (item * p.sb + sv.b_off) * 8;
  double* C = (double*)p.c + vitem * p.sc;
  if constexpr (HINTS) {  // per-item dims; triangular operand: shorter k range; triangular output: maybe nothing
    p.m = item_dim(p.het_m, item, p.m);
    p.n = item_dim(p.het_n, item, p.n);
    p.k = item_dim(p.het_k, item, p.k);
    if (m0 >= p.m || n0 >= p.n) return;
    const TileWork w = tile_work(p, p.k, m0, BM, n0, BN, BK);
    if (w.skip) return;
    A += a_k_offset(p, w.k_lo) * 8;
    B += b_k_offset(p, w.k_lo) * 8;
    p.k = w.k_hi - w.k_lo;
  }

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int KT = (p.k + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) {
      load_tile_pitched<8, BM, BK, THREADS, AK, AL>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, s * BK, p.k, tid);
      load_tile_pitched<8, BN, BK, THREADS, BKM, AL>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, s * BK, p.k, tid);
    }
    cp_async_commit();
  }
  if (!HINTS && p.beta[0] != 0.0) {  // the epilogue reads this tile of C: ask L2 for its 128-byte lines now
    constexpr int LPC = BM / 16;     // lines per stored column of the tile
    for (int c = tid; c < BN * LPC; c += THREADS) {
      const int col = n0 + c / LPC, r0 = m0 + 16 * (c % LPC);
      if (col < p.n && r0 < p.m) asm volatile("prefetch.global.L2 [%0];" ::"l"(C + (long long)col * p.ldc + r0));
    }
  }

  // byte offsets of this lane's fragment element inside a stage, for k-step 0
  const int a_off = AK ? (wm * 32 + g) * A_PITCH + t * 8 : t * A_PITCH + (wm * 32 + g) * 8;
  const int b_off = BKM ? (wn * 32 + g) * B_PITCH + t * 8 : t * B_PITCH + (wn * 32 + g) * 8;
  constexpr int A_MB = AK ? 8 * A_PITCH : 64;       // next 8 rows of m
  constexpr int B_NB = BKM ? 8 * B_PITCH : 64;      // next 8 columns of n
  // element-aligned M-major rows are stored 8 bytes further in when their stored column starts on an
  // odd 8-byte boundary; the row of this lane's fragments is k = 4 k4 + t, whose parity is t's
  const int a_shift = (!AL && !AK) ? (int)(((reinterpret_cast<uintptr_t>(A) >> 3) + (unsigned long long)t * (unsigned long long)p.lda) & 1u) * 8 : 0;
  const int b_shift = (!AL && BKM == false) ? (int)(((reinterpret_cast<uintptr_t>(B) >> 3) + (unsigned long long)t * (unsigned long long)p.ldb) & 1u) * 8 : 0;
  constexpr int A_K4 = AK ? 0 : 4 * A_PITCH;        // next 4 k (K-major: the swizzled group below)
  constexpr int B_K4 = BKM ? 0 : 4 * B_PITCH;
  const int ksw = (g & 3) << 5;                      // K-major rows: 4-k group q is stored at q ^ (row & 3)

  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = kt + STAGES - 1;
      if (nxt < KT) {
        const int s = nxt % STAGES;
        load_tile_pitched<8, BM, BK, THREADS, AK, AL>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, nxt * BK, p.k, tid);
        load_tile_pitched<8, BN, BK, THREADS, BKM, AL>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, nxt * BK, p.k, tid);
      }
      cp_async_commit();
    }
    const unsigned char* as = As + (size_t)(kt % STAGES) * A_STAGE + a_off + a_shift;
    const unsigned char* bs = Bs + (size_t)(kt % STAGES) * B_STAGE + b_off + b_shift;
#pragma unroll
    for (int k4 = 0; k4 < BK / 4; ++k4) {
      double af[4], bf[4];
      const int kgrp = ksw ^ (k4 << 5);
#pragma unroll
      for (int i = 0; i < 4; ++i) af[i] = *reinterpret_cast<const double*>(as + k4 * A_K4 + (AK ? kgrp : 0) + i * A_MB);
#pragma unroll
      for (int j = 0; j < 4; ++j) bf[j] = *reinterpret_cast<const double*>(bs + k4 * B_K4 + (BKM ? kgrp : 0) + j * B_NB);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma(acc[i][j][0], acc[i][j][1], af[i], bf[j]);
    }
  }
  cp_async_wait<0>();

  const double alpha = p.alpha[0], beta = p.beta[0];
  const bool beta_zero = beta == 0.0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = n0 + wn * 32 + j * 8 + 2 * t + e;
      if (col >= p.n) continue;
      double* ccol = C + (long long)col * p.ldc;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m0 + wm * 32 + i * 8 + g;
        if (row >= p.m || (HINTS && out_masked(p, row, col))) continue;
        double out = alpha * acc[i][j][e];
        if (!beta_zero) out = fma(beta, ccol[row], out);
        ccol[row] = out;
      }
    }
}

// ---- complex double ------------------------------------------------------------------------------
// CTA 64 x 64, 8 warps as 2 (m) x 4 (n), warp tile 32 x 16: 4 x 2 DMMA tiles, re and im planes.
template <int OPA, int OPB, bool HINTS, int WM, int WN>
__global__ void __launch_bounds__(32 * WM * WN, 16 / (WM * WN)) gemm_dmma_z_kernel(GemmParams p, int tiles_m, int tiles_n) {
  constexpr int BM = 32 * WM, BN = 16 * WN, BK = 8, STAGES = kStagesZ, THREADS = 32 * WM * WN;
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr bool CONJ_A = (OPA == BLB200_H), CONJ_B = (OPB == BLB200_H);
  constexpr int A_STAGE = pitched_stage_bytes<16, BM, BK, AK>(), B_STAGE = pitched_stage_bytes<16, BN, BK, BKM>();
  constexpr int A_PITCH = AK ? BK * 16 + pad_for(16, true) : BM * 16 + pad_for(16, false);
  constexpr int B_PITCH = BKM ? BK * 16 + pad_for(16, true) : BN * 16 + pad_for(16, false);

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* As = smem;
  unsigned char* Bs = smem + (size_t)STAGES * A_STAGE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = warp % WM, wn = warp / WM;  // WM x WN warps, 32 x 16 each

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const long long vitem = tile / tiles_per_item;
  const int rem = (int)(tile - vitem * tiles_per_item);
  const SplitView sv = resolve_split(p, vitem);
  const long long item = sv.item;
  p.k = sv.k;
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;
  const unsigned char* A = (const unsigned char*)p.a + (item * p.sa + sv.a_off) * 16;
  const unsigned char* B = (const unsigned char*)p.b + (item * p.sb + sv.b_off) * 16;
  double2* C = (double2*)p.c + vitem * p.sc;
  if constexpr (HINTS) {
    p.m = item_dim(p.het_m, item, p.m);
    p.n = item_dim(p.het_n, item, p.n);
    p.k = item_dim(p.het_k, item, p.k);
    if (m0 >= p.m || n0 >= p.n) return;
    const TileWork w = tile_work(p, p.k, m0, BM, n0, BN, BK);
    if (w.skip) return;
    A += a_k_offset(p, w.k_lo) * 16;
    B += b_k_offset(p, w.k_lo) * 16;
    p.k = w.k_hi - w.k_lo;
  }

  double accr[4][2][2], acci[4][2][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) accr[i][j][0] = accr[i][j][1] = acci[i][j][0] = acci[i][j][1] = 0.0;

  const int KT = (p.k + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) {
      load_tile_pitched<16, BM, BK, THREADS, AK>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, s * BK, p.k, tid);
      load_tile_pitched<16, BN, BK, THREADS, BKM>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, s * BK, p.k, tid);
    }
    cp_async_commit();
  }

  const int a_off = AK ? (wm * 32 + g) * A_PITCH + t * 16 : t * A_PITCH + (wm * 32 + g) * 16;
  const int b_off = BKM ? (wn * 16 + g) * B_PITCH + t * 16 : t * B_PITCH + (wn * 16 + g) * 16;
  constexpr int A_MB = AK ? 8 * A_PITCH : 128;
  constexpr int B_NB = BKM ? 8 * B_PITCH : 128;
  constexpr int A_K4 = AK ? 64 : 4 * A_PITCH;
  constexpr int B_K4 = BKM ? 64 : 4 * B_PITCH;

  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = kt + STAGES - 1;
      if (nxt < KT) {
        const int s = nxt % STAGES;
        load_tile_pitched<16, BM, BK, THREADS, AK>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, nxt * BK, p.k, tid);
        load_tile_pitched<16, BN, BK, THREADS, BKM>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, nxt * BK, p.k, tid);
      }
      cp_async_commit();
    }
    const unsigned char* as = As + (size_t)(kt % STAGES) * A_STAGE + a_off;
    const unsigned char* bs = Bs + (size_t)(kt % STAGES) * B_STAGE + b_off;
#pragma unroll
    for (int k4 = 0; k4 < BK / 4; ++k4) {
      double2 af[4], bf[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        af[i] = *reinterpret_cast<const double2*>(as + k4 * A_K4 + i * A_MB);
        if (CONJ_A) af[i].y = -af[i].y;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        bf[j] = *reinterpret_cast<const double2*>(bs + k4 * B_K4 + j * B_NB);
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
  cp_async_wait<0>();

  const double2 alpha = make_double2(p.alpha[0], p.alpha[1]), beta = make_double2(p.beta[0], p.beta[1]);
  const bool beta_zero = beta.x == 0.0 && beta.y == 0.0;
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = n0 + wn * 16 + j * 8 + 2 * t + e;
      if (col >= p.n) continue;
      double2* ccol = C + (long long)col * p.ldc;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = m0 + wm * 32 + i * 8 + g;
        if (row >= p.m || (HINTS && out_masked(p, row, col))) continue;
        const double2 v = make_double2(accr[i][j][e], acci[i][j][e]);
        if (HINTS && p.out_herm && row == col) {  // Hermitian diagonal: real in, real out
          double2 o = Scalar<double2>::mul(alpha, v);
          if (!beta_zero) o.x = fma(beta.x, ccol[row].x, o.x);
          o.y = 0.0;
          ccol[row] = o;
          continue;
        }
        ccol[row] = epilogue<double2>(alpha, v, beta, beta_zero, ccol + row);
      }
    }
}

template <typename Kern>
int launch_kernel(Kern kern, size_t smem, const GemmParams& p, int BM, int BN, cudaStream_t stream, int* configured_for,
                  int threads = 256) {
  const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  int cur = 0;
  cudaGetDevice(&cur);
  if (*configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    *configured_for = cur;
  }
  kern<<<(unsigned)total, threads, smem, stream>>>(p, tiles_m, tiles_n);
  return (int)cudaGetLastError();
}

template <int OPA, int OPB, int WM, int WN>
int launch_d_tile(const GemmParams& p, cudaStream_t stream) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr size_t smem =
      kStagesD * (size_t)(pitched_stage_bytes<8, 32 * WM, 16, AK>() + pitched_stage_bytes<8, 32 * WN, 16, BKM>());
  static thread_local int configured_for = -1, configured_for_hints = -1, configured_for_elem = -1;
  if (!operands_aligned_to(p, 8, 16)) {  // element-granular copies (plain gemm only: tiled_supported saw to that)
    if (has_hints(p) || p.splits > 1) return BLB200_E_UNSUPPORTED;
    return launch_kernel(gemm_dmma_d_kernel<OPA, OPB, false, WM, WN, false>, smem, p, 32 * WM, 32 * WN, stream,
                         &configured_for_elem, 32 * WM * WN);
  }
  if (has_hints(p))
    return launch_kernel(gemm_dmma_d_kernel<OPA, OPB, true, WM, WN>, smem, p, 32 * WM, 32 * WN, stream,
                         &configured_for_hints, 32 * WM * WN);
  return launch_kernel(gemm_dmma_d_kernel<OPA, OPB, false, WM, WN>, smem, p, 32 * WM, 32 * WN, stream, &configured_for,
                       32 * WM * WN);
}

// 2 x 2 warps (CTA 64 x 64, four CTAs per SM).  Measured against 4 x 2 (128 x 64, two CTAs per SM),
// 2 x 4, 4 x 1 and 2 x 1: 256^3 b2048 31.7-32.0 TFLOP/s (TN 29.5) against 28.8-29.3, 1024^3 33.5
// against 32.0, and shapes that are not multiples of 128 gain more (160^3: 19.9 against 13.8).
template <int OPA, int OPB>
int launch_d(const GemmParams& p, cudaStream_t stream) {
  return launch_d_tile<OPA, OPB, 2, 2>(p, stream);
}

template <int OPA, int OPB, int WM, int WN>
int launch_z_tile(const GemmParams& p, cudaStream_t stream) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr size_t smem =
      kStagesZ * (size_t)(pitched_stage_bytes<16, 32 * WM, 8, AK>() + pitched_stage_bytes<16, 16 * WN, 8, BKM>());
  static thread_local int configured_for = -1, configured_for_hints = -1;
  if (has_hints(p))
    return launch_kernel(gemm_dmma_z_kernel<OPA, OPB, true, WM, WN>, smem, p, 32 * WM, 16 * WN, stream,
                         &configured_for_hints, 32 * WM * WN);
  return launch_kernel(gemm_dmma_z_kernel<OPA, OPB, false, WM, WN>, smem, p, 32 * WM, 16 * WN, stream, &configured_for,
                       32 * WM * WN);
}

// 2 x 4 warps of 32 x 16 (CTA 64 x 64); 2 x 2, 1 x 4 and 1 x 2 measured within 1 % of it.
template <int OPA, int OPB>
int launch_z(const GemmParams& p, cudaStream_t stream) {
  return launch_z_tile<OPA, OPB, 2, 4>(p, stream);
}

}  // namespace

bool dmma_supported(const GemmParams& p, int dtype) {
  return (dtype == BLB200_D || dtype == BLB200_Z) && tiled_supported(p, dtype);
}

int launch_dmma(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!dmma_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const int oa = p.op_a, ob = p.op_b;
  int rc = BLB200_E_INTERNAL;
  if (dtype == BLB200_D) {
#define BLB_OP(A_, B_) \
  if (oa == A_ && ob == B_) rc = launch_d<A_, B_>(p, stream);
    BLB_OP(0, 0) BLB_OP(0, 1) BLB_OP(1, 0) BLB_OP(1, 1)
#undef BLB_OP
  } else {
#define BLB_OP(A_, B_) \
  if (oa == A_ && ob == B_) rc = launch_z<A_, B_>(p, stream);
    BLB_OP(0, 0) BLB_OP(0, 1) BLB_OP(0, 2) BLB_OP(1, 0) BLB_OP(1, 1) BLB_OP(1, 2) BLB_OP(2, 0) BLB_OP(2, 1) BLB_OP(2, 2)
#undef BLB_OP
  }
  if (rc == BLB200_OK) note_launch("dmma");
  return rc;
}

}  // namespace blb200
