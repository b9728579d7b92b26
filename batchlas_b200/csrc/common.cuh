// Shared device/host definitions for the sm_100a batched-GEMM kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/blb200.h"

namespace blb200 {

// Launch parameters in kernel-friendly form (passed by value in the kernel parameter space).
struct GemmParams {
  const void* a;
  const void* b;
  void* c;
  int m, n, k, batch;
  long long lda, ldb, ldc;
  long long sa, sb, sc;
  double alpha[2], beta[2];
  int op_a, op_b;
  // Split-K (splits > 1): the launch walks batch * splits virtual items; virtual item v is split
  // v % splits of item v / splits, covers k in [s*kchunk, min(k, (s+1)*kchunk)), reads A and B at
  // element offsets s*split_a / s*split_b past the item, and writes its own partial at c + v*sc.
  int splits, kchunk;
  long long split_a, split_b;
  // Structure hints, all 0 for a plain gemm (never combined with split-K).
  //   tri_a / tri_b: op(A) (m x k) / op(B) (k x n) is triangular WITH the zeros of its other triangle
  //     stored: 1 = lower (zero above the diagonal), 2 = upper.  A tile kernel trims each tile's k
  //     range to the non-zero part; a kernel that ignores the hint still computes the same product.
  //   out_tri: only the lower (1) / upper (2) triangle of a square C is computed and written.  A
  //     kernel handed out_tri must honour it.  out_herm: C is Hermitian — the imaginary part of its
  //     diagonal is neither read nor left non-zero.
  int tri_a = 0, tri_b = 0, out_tri = 0, out_herm = 0;
  // Heterogeneous batch: optional device-readable per-item dims (null = every item uses m / n / k,
  // which are then the capacities the tile grid is laid over).  Read by the same instantiations of
  // the tile kernels that read the structure hints.
  const int* het_m = nullptr;
  const int* het_n = nullptr;
  const int* het_k = nullptr;
};
__host__ __device__ inline bool has_hints(const GemmParams& p) {
  return (p.tri_a | p.tri_b | p.out_tri) != 0 || p.het_m || p.het_n || p.het_k;
}
// Per-item dims of a heterogeneous batch, clamped to [0, capacity].
__device__ __forceinline__ int item_dim(const int* dims, long long item, int cap) {
  if (!dims) return cap;
  const int v = dims[item];
  return v < 0 ? 0 : (v < cap ? v : cap);
}

// True when every operand's base, leading dimension and batch stride are multiples of `bytes`
// (es = element bytes): 16 selects the 16-byte copy policy of the tile kernels, es the
// element-granular one (how BatchLAS switches its own load policy inside one kernel,
// src/sycl/gemm/load_policies.hh:18-34).
inline bool operands_aligned_to(const GemmParams& p, long long es, long long bytes) {
  auto ok = [&](const void* base, long long ld, long long stride) {
    return reinterpret_cast<uintptr_t>(base) % (uintptr_t)bytes == 0 && (ld * es) % bytes == 0 && (stride * es) % bytes == 0;
  };
  return ok(p.a, p.lda, p.sa) && ok(p.b, p.ldb, p.sb) && ok(p.c, p.ldc, p.sc);
}
inline long long dtype_bytes(int dtype) { return dtype == BLB200_S ? 4 : (dtype == BLB200_Z ? 16 : 8); }

struct StructureHints {
  int tri_a, tri_b, out_tri, out_herm;
};

// What a CTA owning rows [m0, m0+BM) and columns [n0, n0+BN) has to do under the hints: the k range
// [k_lo, k_hi) (k_lo a multiple of BK, so 16-byte alignment of the operand rows survives the shift)
// or nothing at all when the tile lies wholly in the triangle of C that is not wanted.
struct TileWork {
  int k_lo, k_hi;
  bool skip;
};
__device__ __forceinline__ TileWork tile_work(const GemmParams& p, int k, int m0, int BM, int n0, int BN, int BK) {
  TileWork w{0, k, false};
  if (p.out_tri == 1) w.skip = m0 + BM - 1 < n0;
  if (p.out_tri == 2) w.skip = m0 > n0 + BN - 1;
  if (p.tri_a == 1) w.k_hi = min(w.k_hi, m0 + BM);          // op(A)(i, l) = 0 for l > i
  if (p.tri_a == 2) w.k_lo = max(w.k_lo, m0 / BK * BK);     // op(A)(i, l) = 0 for l < i
  if (p.tri_b == 1) w.k_lo = max(w.k_lo, n0 / BK * BK);     // op(B)(l, j) = 0 for l < j
  if (p.tri_b == 2) w.k_hi = min(w.k_hi, n0 + BN);          // op(B)(l, j) = 0 for l > j
  return w;
}
// Element offsets of k = k_lo inside the stored operands.
__device__ __forceinline__ long long a_k_offset(const GemmParams& p, int k_lo) {
  return p.op_a == BLB200_N ? (long long)k_lo * p.lda : (long long)k_lo;
}
__device__ __forceinline__ long long b_k_offset(const GemmParams& p, int k_lo) {
  return p.op_b == BLB200_N ? (long long)k_lo : (long long)k_lo * p.ldb;
}
// True when (row, col) lies outside the triangle of C that is wanted.
__device__ __forceinline__ bool out_masked(const GemmParams& p, int row, int col) {
  return p.out_tri == 1 ? row < col : (p.out_tri == 2 ? row > col : false);
}

// Resolves a virtual item into (real item, operand offsets in elements, K extent of this split).
struct SplitView {
  long long item, a_off, b_off;
  int k;
};
__host__ __device__ inline SplitView resolve_split(const GemmParams& p, long long vitem) {
  SplitView v{vitem, 0, 0, p.k};
  if (p.splits > 1) {
    const int s = (int)(vitem % p.splits);
    v.item = vitem / p.splits;
    v.a_off = (long long)s * p.split_a;
    v.b_off = (long long)s * p.split_b;
    const int left = p.k - s * p.kchunk;
    v.k = left < 0 ? 0 : (left < p.kchunk ? left : p.kchunk);
  }
  return v;
}

// Optional per-item dims of a heterogeneous batch (null pointer = every item uses the capacity).
struct HeteroDims {
  const int* m;
  const int* n;
  const int* k;
  int cap_m, cap_n, cap_k;
};

// ---- scalar traits ---------------------------------------------------------------------------
// Real types are float/double; complex types are float2/double2 with (x,y) = (re,im), which is
// the memory layout of std::complex<T>.
template <typename T>
struct Scalar;

template <>
struct Scalar<float> {
  using real_t = float;
  static constexpr bool is_complex = false;
  static constexpr int dtype = BLB200_S;
  __host__ __device__ static float zero() { return 0.f; }
  __host__ __device__ static float make(double re, double) { return (float)re; }
  __device__ static float conj(float v) { return v; }
  __device__ static bool is_zero(float v) { return v == 0.f; }
  // acc += a*b
  __device__ static void fma(float& acc, float a, float b) { acc = fmaf(a, b, acc); }
  __device__ static float mul(float a, float b) { return a * b; }
};

template <>
struct Scalar<double> {
  using real_t = double;
  static constexpr bool is_complex = false;
  static constexpr int dtype = BLB200_D;
  __host__ __device__ static double zero() { return 0.0; }
  __host__ __device__ static double make(double re, double) { return re; }
  __device__ static double conj(double v) { return v; }
  __device__ static bool is_zero(double v) { return v == 0.0; }
  __device__ static void fma(double& acc, double a, double b) { acc = ::fma(a, b, acc); }
  __device__ static double mul(double a, double b) { return a * b; }
};

template <>
struct Scalar<float2> {
  using real_t = float;
  static constexpr bool is_complex = true;
  static constexpr int dtype = BLB200_C;
  __host__ __device__ static float2 zero() { return float2{0.f, 0.f}; }
  __host__ __device__ static float2 make(double re, double im) { return float2{(float)re, (float)im}; }
  __device__ static float2 conj(float2 v) { return float2{v.x, -v.y}; }
  __device__ static bool is_zero(float2 v) { return v.x == 0.f && v.y == 0.f; }
  __device__ static void fma(float2& acc, float2 a, float2 b) {
    acc.x = fmaf(a.x, b.x, acc.x);
    acc.x = fmaf(-a.y, b.y, acc.x);
    acc.y = fmaf(a.x, b.y, acc.y);
    acc.y = fmaf(a.y, b.x, acc.y);
  }
  __device__ static float2 mul(float2 a, float2 b) {
    return float2{fmaf(a.x, b.x, -a.y * b.y), fmaf(a.x, b.y, a.y * b.x)};
  }
};

template <>
struct Scalar<double2> {
  using real_t = double;
  static constexpr bool is_complex = true;
  static constexpr int dtype = BLB200_Z;
  __host__ __device__ static double2 zero() { return double2{0.0, 0.0}; }
  __host__ __device__ static double2 make(double re, double im) { return double2{re, im}; }
  __device__ static double2 conj(double2 v) { return double2{v.x, -v.y}; }
  __device__ static bool is_zero(double2 v) { return v.x == 0.0 && v.y == 0.0; }
  __device__ static void fma(double2& acc, double2 a, double2 b) {
    acc.x = ::fma(a.x, b.x, acc.x);
    acc.x = ::fma(-a.y, b.y, acc.x);
    acc.y = ::fma(a.x, b.y, acc.y);
    acc.y = ::fma(a.y, b.x, acc.y);
  }
  __device__ static double2 mul(double2 a, double2 b) {
    return double2{::fma(a.x, b.x, -a.y * b.y), ::fma(a.x, b.y, a.y * b.x)};
  }
};

// C <- alpha*acc + beta*prior, with prior read only when beta != 0 (BLAS rule).
template <typename T>
__device__ __forceinline__ T epilogue(T alpha, T acc, T beta, bool beta_zero, const T* prior_ptr) {
  T out = Scalar<T>::mul(alpha, acc);
  if (!beta_zero) Scalar<T>::fma(out, beta, *prior_ptr);
  return out;
}

// ---- per-thread launch bookkeeping (diagnostics exposed through the C ABI) -----------------------
void note_launch(const char* kernel_name);
// Kernel selection for one descriptor; the second form passes structure hints to a tile kernel and
// answers BLB200_E_UNSUPPORTED when a triangular output is asked for and no tile kernel applies.
int dispatch(const blb200_gemm_desc* d, cudaStream_t stream);
int dispatch_structured(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream);

// ---- launchers implemented in the kernel translation units -------------------------------------
// Each returns BLB200_OK / a cudaError_t, or BLB200_E_UNSUPPORTED when the kernel's preconditions
// do not hold for `p` (the dispatcher then falls through to the next candidate).
int launch_generic(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_generic_hetero(const GemmParams& p, const HeteroDims& het, int dtype, cudaStream_t stream);
int launch_small32(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_small64(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_tiled(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_dmma(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_sgemm128(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_dmma_tma(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_sgemm_tma(const GemmParams& p, int dtype, cudaStream_t stream);
int launch_splitk_reduce(const GemmParams& orig, int dtype, const void* partials, int splits, long long part_ld,
                         long long part_stride, cudaStream_t stream);

bool small32_supported(const GemmParams& p, int dtype);
bool small64_supported(const GemmParams& p, int dtype);
bool small_ring_supported(const GemmParams& p, int dtype);
int launch_small_ring(const GemmParams& p, int dtype, cudaStream_t stream);
bool tiled_supported(const GemmParams& p, int dtype);
bool dmma_supported(const GemmParams& p, int dtype);
bool dmma_tma_supported(const GemmParams& p, int dtype);
bool sgemm_tma_supported(const GemmParams& p, int dtype);
bool sgemm128_supported(const GemmParams& p, int dtype);
bool sgemm128_preferred(const GemmParams& p);  // against the tiled kernel, by padded work

// Device properties cached per device.
struct DeviceInfo {
  int sm_count;
  int cc_major, cc_minor;
  size_t smem_optin;
};
const DeviceInfo& device_info();  // for the current device

}  // namespace blb200
