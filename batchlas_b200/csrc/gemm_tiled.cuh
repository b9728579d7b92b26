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
// Two load policies, one kernel body (as BatchLAS switches policy inside its tiled kernel,
// src/sycl/gemm/load_policies.hh:18-34): AL = true needs 16-byte aligned bases and ld * sizeof(T),
// stride * sizeof(T) multiples of 16, and moves 16 bytes per copy; AL = false needs only element
// alignment (a slice with an odd offset, ld = 258) and moves one element per copy into the same
// shared-memory layout, with scalar C accesses in the epilogue.  m, n, k are arbitrary: edge
// chunks are zero-filled through the copy's source-size operand and the epilogue is predicated.
//
// Algorithmic traffic per item: A and B once each, C written once and read once iff beta != 0;
// tiles of one item re-read A/B through L2 (BM x BN tiles: A is read N/BN times, B M/BM times).
// This header holds the kernel and launcher templates; one translation unit per element type
// instantiates them (gemm_tiled_s.cu, _d.cu, _c.cu, _z.cu), so that the types compile in parallel.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

template <typename T, int BM_, int BN_, int BK_, int TM_, int TN_, int STAGES_>
struct Tile {
  static constexpr int BM = BM_, BN = BN_, BK = BK_, TM = TM_, TN = TN_, STAGES = STAGES_;
  static constexpr int V = 16 / (int)sizeof(T);
  static constexpr int GM = BM / TM, GN = BN / TN;  // thread groups along m and n
  static constexpr int THREADS = GM * GN;
  static constexpr int WX = GM / 8;                  // warps along m (a warp is 8 x 4 lanes)
  static_assert(GM % 8 == 0 && GN % 4 == 0, "warp shape is 8 x 4 lanes");
  static_assert(TM % V == 0 && TN % V == 0 && BK % V == 0, "thread tile must be whole 16-byte vectors");
};

// Bytes of one operand stage.  `kmajor`: rows are the m (or n) index and hold BK elements + pad.
template <typename T>
__host__ __device__ constexpr int stage_bytes(int rows_mn, int bk, bool kmajor) {
  return kmajor ? rows_mn * (bk * (int)sizeof(T) + 16) : bk * rows_mn * (int)sizeof(T);
}

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, T (&out)[16 / sizeof(T)]) {
  union {
    uint4 u;
    T t[16 / sizeof(T)];
  } cvt;
  cvt.u = raw;
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) out[i] = cvt.t[i];
}

// Issue the async copies of one operand tile.
//   MN0: first m (or n) index of the tile, MN: matrix extent along it, BMN: tile extent,
//   k0: first k of the tile, K: extent along k, G: thread groups along this dimension.
template <int ES>
__device__ __forceinline__ void copy_chunk_by_elements(unsigned char* dst, const unsigned char* src, int valid) {
  constexpr int V = 16 / ES;
#pragma unroll
  for (int e = 0; e < V; ++e) cp_async_elem<ES>(dst + e * ES, e < valid ? src + e * ES : src, e < valid ? ES : 0);
}

template <typename T, int BMN, int BK, int G, int THREADS, bool KMAJOR, bool AL = true>
__device__ __forceinline__ void load_tile(unsigned char* smem, const T* __restrict__ base, long long ld,
                                          int MN0, int MN, int k0, int K, int tid) {
  constexpr int V = 16 / (int)sizeof(T);
  if (!KMAJOR) {
    constexpr int CH_PER_ROW = BMN / V, CHUNKS = BK * CH_PER_ROW;
#pragma unroll
    for (int c = tid; c < CHUNKS; c += THREADS) {
      const int kk = c / CH_PER_ROW, mc = c % CH_PER_ROW;
      const int gk = k0 + kk, gm = MN0 + mc * V;
      int valid = (gk < K) ? (MN - gm) : 0;
      valid = valid < 0 ? 0 : (valid > V ? V : valid);
      const T* src = valid ? base + (long long)gk * ld + gm : base;
      unsigned char* dst = smem + (size_t)kk * (BMN * sizeof(T)) + (size_t)mc * 16;
      if constexpr (AL) cp_async16(dst, src, valid * (int)sizeof(T));
      else cp_async_chunk_widest<(int)sizeof(T)>(dst, (const unsigned char*)src, valid);  // a warp copies one stored column: uniform choice
    }
  } else {
    constexpr int CH_PER_ROW = BK / V, CHUNKS = BMN * CH_PER_ROW, PITCH = BK * (int)sizeof(T) + 16;
#pragma unroll
    for (int c = tid; c < CHUNKS; c += THREADS) {
      const int r = c / CH_PER_ROW, kc = c % CH_PER_ROW;
      const int gmn = MN0 + r, gk = k0 + kc * V;
      int valid = (gmn < MN) ? (K - gk) : 0;
      valid = valid < 0 ? 0 : (valid > V ? V : valid);
      // tile row r = v*(G*V) + g*V + e  ->  slot (v*V + e)*G + g
      const int v = r / (G * V), rem = r % (G * V), g = rem / V, e = rem % V;
      const int slot = (v * V + e) * G + g;
      const T* src = valid ? base + (long long)gmn * ld + gk : base;
      unsigned char* dst = smem + (size_t)slot * PITCH + (size_t)kc * 16;
      if constexpr (AL) cp_async16(dst, src, valid * (int)sizeof(T));
      else copy_chunk_by_elements<(int)sizeof(T)>(dst, (const unsigned char*)src, valid);
    }
  }
}

// Read this thread's TMN x V fragment for k-offsets [kk0, kk0+KSTEP) of the current stage.
//   frag[t][kv]: t-th row (or column) of the thread tile at k = kk0 + kv.
template <typename T, int BMN, int BK, int G, int TMN, int KSTEP, bool KMAJOR>
__device__ __forceinline__ void read_frag(const unsigned char* smem, int g, int kk0, T (&frag)[TMN][KSTEP]) {
  constexpr int V = 16 / (int)sizeof(T);
  if (!KMAJOR) {
#pragma unroll
    for (int kv = 0; kv < KSTEP; ++kv)
#pragma unroll
      for (int v = 0; v < TMN / V; ++v) {
        const uint4 raw = *reinterpret_cast<const uint4*>(smem + (size_t)(kk0 + kv) * (BMN * sizeof(T)) +
                                                          (size_t)(v * G + g) * 16);
        T tmp[V];
        unpack16<T>(raw, tmp);
#pragma unroll
        for (int e = 0; e < V; ++e) frag[v * V + e][kv] = tmp[e];
      }
  } else {
    static_assert(!KMAJOR || KSTEP == V, "a K-major read brings V consecutive k");
    constexpr int PITCH = BK * (int)sizeof(T) + 16;
#pragma unroll
    for (int t = 0; t < TMN; ++t) {
      const uint4 raw =
          *reinterpret_cast<const uint4*>(smem + (size_t)(t * G + g) * PITCH + (size_t)(kk0 / V) * 16);
      T tmp[V];
      unpack16<T>(raw, tmp);
#pragma unroll
      for (int kv = 0; kv < KSTEP; ++kv) frag[t][kv] = tmp[kv];
    }
  }
}

// HINTS = false is the plain gemm; HINTS = true reads the structure hints of GemmParams (a separate
// instantiation, so that the plain kernel's code and register allocation stay what they were).
template <typename T, typename Cfg, int OPA, int OPB, int MIN_BLOCKS, bool HINTS, bool AL = true>
__global__ void __launch_bounds__(Cfg::THREADS, MIN_BLOCKS)
    gemm_tiled_kernel(GemmParams p, int tiles_m, int tiles_n) {
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN, V = Cfg::V;
  constexpr int GM = Cfg::GM, GN = Cfg::GN, THREADS = Cfg::THREADS, STAGES = Cfg::STAGES;
  constexpr bool AK = (OPA != BLB200_N);   // A stored k x m: k fastest
  constexpr bool BKM = (OPB == BLB200_N);  // B stored k x n: k fastest
  constexpr bool CONJ_A = Scalar<T>::is_complex && OPA == BLB200_H;
  constexpr bool CONJ_B = Scalar<T>::is_complex && OPB == BLB200_H;
  constexpr int KSTEP = (AK || BKM) ? V : 1;
  constexpr int A_STAGE = stage_bytes<T>(BM, BK, AK), B_STAGE = stage_bytes<T>(BN, BK, BKM);

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* As = smem;
  unsigned char* Bs = smem + (size_t)STAGES * A_STAGE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = (warp % Cfg::WX) * 8 + (lane & 7);   // m group
  const int h = (warp / Cfg::WX) * 4 + (lane >> 3);  // n group

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const long long vitem = tile / tiles_per_item;
  const int rem = (int)(tile - vitem * tiles_per_item);
  const SplitView sv = resolve_split(p, vitem);
  const long long item = sv.item;
  p.k = sv.k;
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;
  const T* A = (const T*)p.a + item * p.sa + sv.a_off;
  const T* B = (const T*)p.b + item * p.sb + sv.b_off;
  T* C = (T*)p.c + vitem * p.sc;
  if constexpr (HINTS) {  // per-item dims; triangular operand: shorter k range; triangular output: maybe nothing
    p.m = item_dim(p.het_m, item, p.m);
    p.n = item_dim(p.het_n, item, p.n);
    p.k = item_dim(p.het_k, item, p.k);
    if (m0 >= p.m || n0 >= p.n) return;
    const TileWork w = tile_work(p, p.k, m0, BM, n0, BN, BK);
    if (w.skip) return;
    A += a_k_offset(p, w.k_lo);
    B += b_k_offset(p, w.k_lo);
    p.k = w.k_hi - w.k_lo;
  }

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = Scalar<T>::zero();

  const int KT = (p.k + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) {
      load_tile<T, BM, BK, GM, THREADS, AK, AL>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, s * BK, p.k, tid);
      load_tile<T, BN, BK, GN, THREADS, BKM, AL>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, s * BK, p.k, tid);
    }
    cp_async_commit();
  }

  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = kt + STAGES - 1;
      if (nxt < KT) {
        const int s = nxt % STAGES;
        load_tile<T, BM, BK, GM, THREADS, AK, AL>(As + (size_t)s * A_STAGE, A, p.lda, m0, p.m, nxt * BK, p.k, tid);
        load_tile<T, BN, BK, GN, THREADS, BKM, AL>(Bs + (size_t)s * B_STAGE, B, p.ldb, n0, p.n, nxt * BK, p.k, tid);
      }
      cp_async_commit();
    }
    const unsigned char* as = As + (size_t)(kt % STAGES) * A_STAGE;
    const unsigned char* bs = Bs + (size_t)(kt % STAGES) * B_STAGE;
#pragma unroll
    for (int kk0 = 0; kk0 < BK; kk0 += KSTEP) {
      T af[TM][KSTEP], bf[TN][KSTEP];
      read_frag<T, BM, BK, GM, TM, KSTEP, AK>(as, g, kk0, af);
      read_frag<T, BN, BK, GN, TN, KSTEP, BKM>(bs, h, kk0, bf);
      if (CONJ_A) {
#pragma unroll
        for (int t = 0; t < TM; ++t)
#pragma unroll
          for (int kv = 0; kv < KSTEP; ++kv) af[t][kv] = Scalar<T>::conj(af[t][kv]);
      }
      if (CONJ_B) {
#pragma unroll
        for (int t = 0; t < TN; ++t)
#pragma unroll
          for (int kv = 0; kv < KSTEP; ++kv) bf[t][kv] = Scalar<T>::conj(bf[t][kv]);
      }
#pragma unroll
      for (int kv = 0; kv < KSTEP; ++kv)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) Scalar<T>::fma(acc[i][j], af[i][kv], bf[j][kv]);
    }
  }
  cp_async_wait<0>();

  // Epilogue: V contiguous rows per 16-byte access; 8 lanes cover 128 contiguous bytes of a column.
  const T alpha = Scalar<T>::make(p.alpha[0], p.alpha[1]);
  const T beta = Scalar<T>::make(p.beta[0], p.beta[1]);
  const bool beta_zero = Scalar<T>::is_zero(beta);
#pragma unroll
  for (int j = 0; j < TN; ++j) {
    const int col = n0 + (j / V) * (GN * V) + h * V + (j % V);
    if (col >= p.n) continue;
    T* ccol = C + (long long)col * p.ldc;
#pragma unroll
    for (int v = 0; v < TM / V; ++v) {
      const int row = m0 + v * (GM * V) + g * V;
      // with a triangular output the vector access is used only strictly inside the wanted triangle
      const bool whole = !HINTS || p.out_tri == 0 || (p.out_tri == 1 ? row > col : row + V - 1 < col);
      if (AL && row + V <= p.m && whole) {
        union {
          uint4 u;
          T t[V];
        } io;
        if (!beta_zero) io.u = *reinterpret_cast<const uint4*>(ccol + row);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          T out = Scalar<T>::mul(alpha, acc[v * V + e][j]);
          if (!beta_zero) Scalar<T>::fma(out, beta, io.t[e]);
          io.t[e] = out;
        }
        *reinterpret_cast<uint4*>(ccol + row) = io.u;
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          if (row + e >= p.m || (HINTS && out_masked(p, row + e, col))) continue;
          if constexpr (HINTS && Scalar<T>::is_complex) {
            if (p.out_herm && row + e == col) {  // Hermitian diagonal: real in, real out
              T o = Scalar<T>::mul(alpha, acc[v * V + e][j]);
              if (!beta_zero) o.x += beta.x * ccol[row + e].x;
              o.y = 0;
              ccol[row + e] = o;
              continue;
            }
          }
          ccol[row + e] = epilogue<T>(alpha, acc[v * V + e][j], beta, beta_zero, ccol + row + e);
        }
      }
    }
  }
}

template <typename T, typename Cfg, int OPA, int OPB, int MIN_BLOCKS, bool HINTS, bool AL = true>
int launch_cfg(const GemmParams& p, cudaStream_t stream) {
  constexpr bool AK = (OPA != BLB200_N), BKM = (OPB == BLB200_N);
  constexpr size_t smem = (size_t)Cfg::STAGES * (stage_bytes<T>(Cfg::BM, Cfg::BK, AK) + stage_bytes<T>(Cfg::BN, Cfg::BK, BKM));
  const int tiles_m = (p.m + Cfg::BM - 1) / Cfg::BM, tiles_n = (p.n + Cfg::BN - 1) / Cfg::BN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  auto kern = gemm_tiled_kernel<T, Cfg, OPA, OPB, MIN_BLOCKS, HINTS, AL>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  kern<<<(unsigned)total, Cfg::THREADS, smem, stream>>>(p, tiles_m, tiles_n);
  return (int)cudaGetLastError();
}

template <typename T, typename Cfg, int MIN_BLOCKS>
int launch_ops(const GemmParams& p, cudaStream_t stream) {
  const int oa = p.op_a, ob = p.op_b;
  const bool hints = has_hints(p);
  // element-granular copies for operands that are not 16-byte aligned (plain gemm only; sizeof(T)
  // == 16 is always on the 16-byte policy)
  const bool al = sizeof(T) == 16 || operands_aligned_to(p, (long long)sizeof(T), 16);
  if (!al && (hints || p.splits > 1)) return BLB200_E_UNSUPPORTED;
#define BLB_OP(A_, B_)                                                                    \
  if (oa == A_ && ob == B_) {                                                             \
    if constexpr (sizeof(T) < 16) {                                                       \
      if (!al) return launch_cfg<T, Cfg, A_, B_, MIN_BLOCKS, false, false>(p, stream);    \
    }                                                                                     \
    return hints ? launch_cfg<T, Cfg, A_, B_, MIN_BLOCKS, true>(p, stream)                \
                 : launch_cfg<T, Cfg, A_, B_, MIN_BLOCKS, false>(p, stream);              \
  }
  BLB_OP(0, 0) BLB_OP(0, 1) BLB_OP(1, 0) BLB_OP(1, 1)
  if (Scalar<T>::is_complex) {
    BLB_OP(0, 2) BLB_OP(1, 2) BLB_OP(2, 0) BLB_OP(2, 1) BLB_OP(2, 2)
  }
#undef BLB_OP
  return BLB200_E_INTERNAL;
}

}  // namespace
}  // namespace blb200
