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
};

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
int launch_splitk_reduce(const GemmParams& orig, int dtype, const void* partials, int splits, long long part_ld,
                         long long part_stride, cudaStream_t stream);

bool small32_supported(const GemmParams& p, int dtype);
bool small64_supported(const GemmParams& p, int dtype);
bool tiled_supported(const GemmParams& p, int dtype);
bool dmma_supported(const GemmParams& p, int dtype);
bool sgemm128_supported(const GemmParams& p, int dtype);

// Device properties cached per device.
struct DeviceInfo {
  int sm_count;
  int cc_major, cc_minor;
  size_t smem_optin;
};
const DeviceInfo& device_info();  // for the current device

}  // namespace blb200
