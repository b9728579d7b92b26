// Whole-matrix-per-warp gemm for large batches of small packed matrices of ANY of the four element
// types and any shape up to 32 x 32 (k up to 64): the general sibling of the float-only 32^3 / 64^3
// kernels.  Such problems are HBM-bound (a 32 x 32 x 32 double item moves 32 KiB for 64 Kflop), so the
// whole design is about streaming: a shared-memory ring is kept full with untiled TMA bulk copies
// of whole A, B (and C when beta != 0) items, one "full" mbarrier per slot, and each warp multiplies
// one item out of its slot.  A slot belongs to one warp for the whole launch; lane 0 of that warp
// issues the copies of the item that uses the slot next as soon as the bulk store of the result has
// read the slot (no producer warp, no "empty" barrier: a producer lane parked in a blocking barrier
// wait held up its warp's other lanes and every refill started late — double 32^3 4.0 -> 6.4 TB/s,
// float 16^3 2.6 -> 5.3).  Nothing but long sequential reads and the C stores reaches HBM.
//
// A lane owns rows ti + 8r and columns tj + 4c (ti = lane & 7, tj = lane >> 3; up to 4 x 8 outputs), so
// that an M-major A or an N-major B is read by consecutive lanes at consecutive addresses.  A K-major
// operand would put all lanes of a request into one bank (its rows are k elements apart), so with a
// K-major operand every lane walks k from its own starting offset: the same products in another
// order.  Conjugation is a sign flip on read.
//
// Preconditions (small_ring_supported): packed operands (ld == stored rows), item sizes multiples of
// 16 bytes, item starts on 16-byte boundaries, m, n <= 32 (complex<double>: 16), k <= 64, one slot at
// most 27 KiB, a batch large enough to keep a ring per SM busy.  Ring discipline as in the other ring kernels: the slot
// count is a multiple of the warp count, slot s always belongs to warp s % CW, and every wait
// is bounded (on expiry the waiter records a code in the device status word and returns).
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

enum WaitCode { kSmallRingWaitFull = 301 };
constexpr int kMaxMN = 32, kMaxK = 64, kMaxSlotBytes = 27648;

template <typename T>
__device__ __forceinline__ T maybe_conj(T v, bool conj) {
  if constexpr (Scalar<T>::is_complex) {
    if (conj) v.y = -v.y;
  }
  return v;
}

__device__ __forceinline__ void dmma884(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

// RB x CB: outputs per lane (4 x 8 covers 32 x 32; 2 x 4 covers 16 x 16 with a quarter of the registers).
// DMMA (double only; m, n multiples of 8, k a multiple of 4): the product runs on the FP64 tensor
// pipe instead.  RB x CB then counts 8 x 8 output tiles per warp; lane (g = lane >> 2, q = lane & 3)
// feeds A(8rb + g, k0 + q) and B(k0 + q, 8cb + g) and receives C(8rb + g, 8cb + 2q), C(.., 8cb + 2q + 1):
// two fragment doubles per lane for sixteen tile products per k-step of 4, where the scalar loop
// reads twelve per 32 multiply-adds and is bound by the latency of those reads.
template <typename T, int CW, bool A_KMAJOR, bool B_KMAJOR, bool HAS_C, int RB, int CB, bool DMMA = false>
__global__ void __launch_bounds__(32 * CW, 1)
    gemm_small_ring_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int m, int n, int k,
                           long long sa, long long sb, long long sc, int batch, T alpha, T beta, bool conj_a, bool conj_b,
                           int stages, int slot_bytes) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * slot_bytes);
  const uint32_t a_bytes = (uint32_t)(m * k * (int)sizeof(T)), b_bytes = (uint32_t)(k * n * (int)sizeof(T)),
                 c_bytes = (uint32_t)(m * n * (int)sizeof(T));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // Items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; the j-th one uses slot j % stages.
  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  auto issue = [&](int slot, int jj) {
    unsigned char* st = smem + (size_t)slot * slot_bytes;
    const long long it = (long long)blockIdx.x + (long long)jj * gridDim.x;
    mbar_arrive_expect_tx(&full_bar[slot], a_bytes + b_bytes + (HAS_C ? c_bytes : 0u));
    bulk_g2s(st, A + it * sa, a_bytes, &full_bar[slot]);
    bulk_g2s(st + a_bytes, B + it * sb, b_bytes, &full_bar[slot]);
    if (HAS_C) bulk_g2s(st + a_bytes + b_bytes, C + it * sc, c_bytes, &full_bar[slot]);
  };
  const int cw = warp;
  const int ti = lane & 7, tj = lane >> 3;
  const int rmax = (m - ti + 7) >> 3;  // rows ti + 8r < m
  const int cmax = (n - tj + 3) >> 2;  // columns tj + 4c < n
  // this lane's first k: only a K-major operand needs the stagger
  int k0 = (A_KMAJOR && B_KMAJOR) ? ti + 8 * tj : (A_KMAJOR ? ti : (B_KMAJOR ? tj : 0));
  k0 = k0 % k;

  if (lane == 0)
    for (int slot = cw; slot < stages && slot < my_items; slot += CW) issue(slot, slot);
  int s = cw;
  uint32_t round = 0;
  for (int j = cw; j < my_items; j += CW) {
    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    if (!mbar_wait(&full_bar[s], round & 1u, kSmallRingWaitFull)) return;
    const T* As = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes);
    const T* Bs = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes + a_bytes);
    const T* Cs = reinterpret_cast<const T*>(smem + (size_t)s * slot_bytes + a_bytes + b_bytes);

    if constexpr (DMMA) {
      constexpr int CBW = CB, cb0 = 0;  // column tiles of this warp, first one
      const int g = lane >> 2, q = lane & 3;
      const int mt = m >> 3, nt = n >> 3;
      double d0[RB][CBW], d1[RB][CBW];
#pragma unroll
      for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int cb = 0; cb < CBW; ++cb) d0[rb][cb] = d1[rb][cb] = 0.0;
      // tiles past the edge repeat the last valid one (read, multiplied nowhere, never stored)
      const double* ap[RB];
      const double* bp[CBW];
#pragma unroll
      for (int rb = 0; rb < RB; ++rb) {
        const int row = 8 * min(rb, mt - 1) + g;
        ap[rb] = As + (A_KMAJOR ? row * k + q : q * m + row);
      }
#pragma unroll
      for (int cb = 0; cb < CBW; ++cb) {
        const int col = 8 * min(cb0 + cb, nt - 1) + g;
        bp[cb] = Bs + (B_KMAJOR ? col * k + q : q * n + col);
      }
      const int a_step = A_KMAJOR ? 4 : 4 * m, b_step = B_KMAJOR ? 4 : 4 * n;
#pragma unroll 2
      for (int k0 = 0; k0 < k; k0 += 4) {
        double av[RB], bv[CBW];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) av[rb] = ap[rb][(k0 >> 2) * a_step];
#pragma unroll
        for (int cb = 0; cb < CBW; ++cb) bv[cb] = bp[cb][(k0 >> 2) * b_step];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
          for (int cb = 0; cb < CBW; ++cb)
            if (rb < mt && cb0 + cb < nt) dmma884(d0[rb][cb], d1[rb][cb], av[rb], bv[cb]);
      }
      __syncwarp();
      double* Os = const_cast<double*>(HAS_C ? Cs : As);
#pragma unroll
      for (int cb = 0; cb < CBW; ++cb)
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
          if (rb < mt && cb0 + cb < nt) {
            const int idx = (8 * (cb0 + cb) + 2 * q) * m + 8 * rb + g;
            double o0 = alpha * d0[rb][cb], o1 = alpha * d1[rb][cb];
            if (HAS_C) {
              o0 = fma(beta, Os[idx], o0);
              o1 = fma(beta, Os[idx + m], o1);
            }
            Os[idx] = o0;
            Os[idx + m] = o1;
          }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        // this warp's columns are one contiguous run of C
        const int c_first = 8 * cb0, c_last = min(n, 8 * (cb0 + CBW));
        if (c_last > c_first) {
          bulk_s2g(C + item * sc + (long long)c_first * m, Os + c_first * m,
                   (uint32_t)((c_last - c_first) * m * (int)sizeof(double)));
          bulk_commit();
          bulk_wait_read<0>();
        }
        if (j + stages < my_items) issue(s, j + stages);
      }
    } else {
    T acc[RB][CB];
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int c = 0; c < CB; ++c) acc[r][c] = Scalar<T>::zero();

    // Rows / columns past the edge are clamped to a valid element (read, multiplied, never stored),
    // which keeps the inner loop free of predicates.  Every operand is walked with one running
    // offset per operand; the lane-specific part of the address is folded into a base pointer.
    const T* ap[RB];
    const T* bp[CB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int row = min(ti + 8 * r, m - 1);
      ap[r] = As + (A_KMAJOR ? row * k : row);
    }
#pragma unroll
    for (int c = 0; c < CB; ++c) {
      const int col = min(tj + 4 * c, n - 1);
      bp[c] = Bs + (B_KMAJOR ? col * k : col);
    }
    const int a_step = A_KMAJOR ? 1 : m, b_step = B_KMAJOR ? 1 : n;
    // the k index of step t is computed from t alone (no value carried from step to step), so the
    // loads of the following steps can be issued while this step's multiply-adds are still running
#pragma unroll 4
    for (int t = 0; t < k; ++t) {
      int kk = k0 + t;
      kk -= kk >= k ? k : 0;
      const int a_off = kk * a_step, b_off = kk * b_step;
      T av[RB], bv[CB];
#pragma unroll
      for (int r = 0; r < RB; ++r) av[r] = maybe_conj(ap[r][a_off], conj_a);
#pragma unroll
      for (int c = 0; c < CB; ++c) bv[c] = maybe_conj(bp[c][b_off], conj_b);
#pragma unroll
      for (int r = 0; r < RB; ++r)
#pragma unroll
        for (int c = 0; c < CB; ++c) Scalar<T>::fma(acc[r][c], av[r], bv[c]);
    }

    // The result is assembled in the slot (over the old C, or over A when there is none: every lane
    // is past its reads of A and B after the warp barrier) and leaves as one bulk store; the slot
    // is handed back once that store has read it.
    __syncwarp();
    T* Os = const_cast<T*>(HAS_C ? Cs : As);
#pragma unroll
    for (int c = 0; c < CB; ++c) {
      if (c < cmax) {
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          if (r < rmax) {
            const int idx = (tj + 4 * c) * m + ti + 8 * r;
            T out = Scalar<T>::mul(alpha, acc[r][c]);
            if (HAS_C) Scalar<T>::fma(out, beta, Os[idx]);
            Os[idx] = out;
          }
        }
      }
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      bulk_s2g(C + item * sc, Os, c_bytes);
      bulk_commit();
      bulk_wait_read<0>();
      if (j + stages < my_items) issue(s, j + stages);
    }
    }  // scalar path
    s += CW;
    if (s >= stages) {
      s -= stages;
      ++round;
    }
  }
  if (lane == 0) bulk_wait<0>();  // the last stores have landed before the warp retires
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <typename T, int CW, bool AK, bool BK, bool HC, int RB, int CB, bool DMMA = false>
int launch_one(const GemmParams& p, int stages, int slot_bytes, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  const size_t smem = (size_t)stages * slot_bytes + (size_t)stages * sizeof(uint64_t);
  auto kern = gemm_small_ring_kernel<T, CW, AK, BK, HC, RB, CB, DMMA>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dev.smem_optin);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = p.batch < dev.sm_count ? p.batch : dev.sm_count;
  kern<<<grid, 32 * CW, smem, stream>>>((const T*)p.a, (const T*)p.b, (T*)p.c, p.m, p.n, p.k, p.sa, p.sb, p.sc,
                                            p.batch, Scalar<T>::make(p.alpha[0], p.alpha[1]),
                                            Scalar<T>::make(p.beta[0], p.beta[1]), p.op_a == BLB200_H,
                                            p.op_b == BLB200_H, stages, slot_bytes);
  return (int)cudaGetLastError();
}

template <typename T, int CW>
int launch_cw(const GemmParams& p, int stages, int slot_bytes, bool hc, cudaStream_t stream) {
  const bool ak = p.op_a != BLB200_N;  // op T / H stores A as k x m: k runs fastest
  const bool bk = p.op_b == BLB200_N;  // op N stores B as k x n: k runs fastest
  const bool quarter = p.m <= 16 && p.n <= 16;
  const bool dmma = std::is_same<T, double>::value && p.m % 8 == 0 && p.n % 8 == 0 && p.k % 4 == 0;
#define BLB_CASE(a, b)                                                                                     \
  if (ak == a && bk == b) {                                                                                \
    if constexpr (std::is_same<T, double>::value) {                                                        \
      if (dmma && quarter)                                                                                 \
        return hc ? launch_one<T, CW, a, b, true, 2, 2, true>(p, stages, slot_bytes, stream)               \
                  : launch_one<T, CW, a, b, false, 2, 2, true>(p, stages, slot_bytes, stream);             \
      if (dmma)                                                                                            \
        return hc ? launch_one<T, CW, a, b, true, 4, 4, true>(p, stages, slot_bytes, stream)               \
                  : launch_one<T, CW, a, b, false, 4, 4, true>(p, stages, slot_bytes, stream);             \
    }                                                                                                      \
    if (quarter)                                                                                           \
      return hc ? launch_one<T, CW, a, b, true, 2, 4>(p, stages, slot_bytes, stream)                       \
                : launch_one<T, CW, a, b, false, 2, 4>(p, stages, slot_bytes, stream);                     \
    if constexpr (sizeof(T) < 16)                                                                          \
      return hc ? launch_one<T, CW, a, b, true, 4, 8>(p, stages, slot_bytes, stream)                       \
                : launch_one<T, CW, a, b, false, 4, 8>(p, stages, slot_bytes, stream);                     \
    return BLB200_E_UNSUPPORTED;                                                                           \
  }
  BLB_CASE(false, false) BLB_CASE(false, true) BLB_CASE(true, false) BLB_CASE(true, true)
#undef BLB_CASE
  return BLB200_E_INTERNAL;
}

template <typename T>
int launch_typed(const GemmParams& p, cudaStream_t stream) {
  const bool hc = !(p.beta[0] == 0.0 && p.beta[1] == 0.0);
  // without an old C the result is assembled over A (and B): the slot must hold it
  int slot_elems = p.m * p.k + p.k * p.n + (hc ? p.m * p.n : 0);
  if (slot_elems < p.m * p.n) slot_elems = p.m * p.n;
  const int slot_bytes = slot_elems * (int)sizeof(T);
  const size_t budget = device_info().smem_optin > 8192 ? device_info().smem_optin - 4096 : 0;
  const int fit = (int)(budget / (size_t)slot_bytes);
  if constexpr (std::is_same<T, double>::value) {
    // Tensor-pipe path with 4 x 4 tiles per warp (about 135 registers): 8 warps with two or more slots
    // each where 16 slots fit (16 warps would cap a thread at 96 registers and spill: 24^3 ran at 2.4
    // instead of 3.5 TB/s); bigger items stay on four warps with two or three slots each, which
    // measured faster than eight warps with one (32^3: 4.0 against 3.9, beta = 0: 3.9 against 2.8 TB/s).
    const bool tiles4 = (p.m > 16 || p.n > 16) && p.m % 8 == 0 && p.n % 8 == 0 && p.k % 4 == 0;
    if (tiles4 && fit >= 16) return launch_cw<T, 8>(p, (fit >= 32 ? 32 : fit) / 8 * 8, slot_bytes, hc, stream);
  }
  // 16 warps with two slots each when that fits, else with one
  if (fit >= 32) return launch_cw<T, 16>(p, 32, slot_bytes, hc, stream);
  if (fit >= 16) return launch_cw<T, 16>(p, 16, slot_bytes, hc, stream);
  // big slots: four warps with two or three slots each measured 5-30 % faster than eight with one
  if (fit >= 8) return launch_cw<T, 4>(p, fit >= 12 ? 12 : 8, slot_bytes, hc, stream);
  return BLB200_E_UNSUPPORTED;
}

}  // namespace

int small_ring_device_status(int* out) { return read_device_status_word(out); }
int small_ring_device_status_clear() { return clear_device_status_word(); }

bool small_ring_supported(const GemmParams& p, int dtype) {
  const long long es = dtype == BLB200_S ? 4 : (dtype == BLB200_Z ? 16 : 8);
  if (p.m < 1 || p.n < 1 || p.k < 1 || p.m > kMaxMN || p.n > kMaxMN || p.k > kMaxK) return false;
  // complex<double>: 32 accumulators per lane do not fit, and from 16 x 16 on the generic kernel's
  // tiles measured faster than one warp per matrix (3.4 against 2.0 TB/s)
  if (dtype == BLB200_Z && (p.m > 8 || p.n > 8)) return false;
  if (p.splits > 1 || has_hints(p)) return false;
  const int a_rows = p.op_a == BLB200_N ? p.m : p.k, b_rows = p.op_b == BLB200_N ? p.k : p.n;
  if (p.lda != a_rows || p.ldb != b_rows || p.ldc != p.m) return false;  // packed
  const long long a_bytes = (long long)p.m * p.k * es, b_bytes = (long long)p.k * p.n * es,
                  c_bytes = (long long)p.m * p.n * es;
  if (a_bytes % 16 || b_bytes % 16 || c_bytes % 16) return false;
  const bool hc = !(p.beta[0] == 0.0 && p.beta[1] == 0.0);
  if (a_bytes + b_bytes + (hc ? c_bytes : 0) > kMaxSlotBytes || c_bytes > kMaxSlotBytes) return false;
  if (!aligned16(p.a) || !aligned16(p.b) || !aligned16(p.c)) return false;
  if ((p.sa * es) % 16 || (p.sb * es) % 16 || (p.sc * es) % 16) return false;
  if (p.batch > 1 && (p.sa < (long long)p.m * p.k || p.sb < (long long)p.k * p.n || p.sc < (long long)p.m * p.n))
    return false;  // overlapping or broadcast items: leave to the generic kernel
  return p.batch >= 8 * device_info().sm_count;
}

int launch_small_ring(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!small_ring_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  int rc;
  switch (dtype) {
    case BLB200_S: rc = launch_typed<float>(p, stream); break;
    case BLB200_D: rc = launch_typed<double>(p, stream); break;
    case BLB200_C: rc = launch_typed<float2>(p, stream); break;
    case BLB200_Z: rc = launch_typed<double2>(p, stream); break;
    default: return BLB200_E_DTYPE;
  }
  if (rc == BLB200_OK) note_launch("small_ring");
  return rc;
}

}  // namespace blb200
