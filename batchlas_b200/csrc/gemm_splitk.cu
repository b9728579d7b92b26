// Split-K for problems with too few output tiles to fill the GPU (small m x n, long k, small
// batch: Gram matrices of tall-skinny blocks are the typical caller).  The k range is cut into
// `splits` chunks; one launch of the ordinary tile kernel walks batch * splits virtual items and
// writes each chunk's product, unscaled, into its own partial in caller-provided scratch; a second
// kernel sums the partials and applies alpha / beta.  Same decomposition as BatchLAS's experimental
// split-K (src/sycl/gemm/split_k.hh:52-162: per-split launches into a temporary Matrix, then
// reduce_split_k_partials), generalised to every dtype, op pair and shape, with the scratch taken
// from the calling queue's workspace arena instead of a fresh allocation.
//
// A second entry point keeps the scratch in a fixed device array for callers that cannot allocate.
#include <mutex>

#include "common.cuh"

namespace blb200 {
int dispatch(const blb200_gemm_desc* d, cudaStream_t stream);
GemmParams to_params_public(const blb200_gemm_desc* d);

namespace {

size_t elem_bytes(int dtype) { return dtype == BLB200_S ? 4 : (dtype == BLB200_Z ? 16 : 8); }

struct SplitPlan {
  int splits, kchunk;
  long long ld, stride;  // partial layout, elements
  size_t bytes;
};

// splits_wanted == 0: choose; the answer is 1 when splitting would not help.
SplitPlan plan_split(const blb200_gemm_desc& d, int splits_wanted) {
  SplitPlan pl{1, d.k, 0, 0, 0};
  if (d.m <= 0 || d.n <= 0 || d.batch <= 0 || d.k <= 0) return pl;
  int splits = splits_wanted;
  if (splits <= 0) {
    const int bm = (d.dtype == BLB200_S) ? 128 : 64, bn = (d.dtype == BLB200_S) ? 128 : 64;  // CTA tiles of the kernels used
    const long long tiles = (long long)((d.m + bm - 1) / bm) * ((d.n + bn - 1) / bn) * d.batch;
    const long long sms = device_info().sm_count;
    if (tiles >= sms) return pl;
    long long s = (2 * sms + tiles - 1) / tiles;
    const long long by_k = d.k / 128;  // at least 128 k per chunk, or the reduce pass costs more than it saves
    if (s > by_k) s = by_k;
    if (s > 64) s = 64;
    splits = (int)s;
  }
  if (splits < 2) return pl;
  if (splits > d.k) splits = d.k;
  int kchunk = (d.k + splits - 1) / splits;
  kchunk = (kchunk + 15) / 16 * 16;  // keeps every chunk's first element 16-byte aligned
  splits = (d.k + kchunk - 1) / kchunk;
  if (splits < 2) return pl;
  const size_t es = elem_bytes(d.dtype);
  const long long vec = (long long)(16 / es);
  pl.splits = splits;
  pl.kchunk = kchunk;
  pl.ld = (d.m + vec - 1) / vec * vec;
  pl.stride = pl.ld * d.n;
  pl.bytes = (size_t)pl.stride * es * (size_t)d.batch * (size_t)splits;
  return pl;
}

// C <- alpha * sum_s partial[item*splits + s] + beta * C
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const T* __restrict__ partials, T* __restrict__ C, int m,
                                                            int n, int batch, int splits, long long part_ld,
                                                            long long part_stride, long long ldc, long long sc, T alpha,
                                                            T beta, bool beta_zero) {
  const long long per_item = (long long)m * n, total = per_item * batch;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long flat = (long long)blockIdx.x * blockDim.x + threadIdx.x; flat < total; flat += step) {
    const long long b = flat / per_item, rem = flat - b * per_item;
    const int col = (int)(rem / m), row = (int)(rem - (long long)col * m);
    const T* src = partials + b * splits * part_stride + (long long)col * part_ld + row;
    T sum = Scalar<T>::zero();
    for (int s = 0; s < splits; ++s) {
      const T v = src[(long long)s * part_stride];
      if constexpr (Scalar<T>::is_complex) {
        sum.x += v.x;
        sum.y += v.y;
      } else {
        sum += v;
      }
    }
    T* dst = C + b * sc + (long long)col * ldc + row;
    *dst = epilogue<T>(alpha, sum, beta, beta_zero, dst);
  }
}

template <typename T>
int reduce_typed(const GemmParams& o, const void* partials, int splits, long long part_ld, long long part_stride,
                 cudaStream_t stream) {
  const long long total = (long long)o.m * o.n * o.batch;
  const long long want = (total + 255) / 256;
  const long long cap = (long long)device_info().sm_count * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  const T alpha = Scalar<T>::make(o.alpha[0], o.alpha[1]), beta = Scalar<T>::make(o.beta[0], o.beta[1]);
  const bool beta_zero = o.beta[0] == 0.0 && o.beta[1] == 0.0;
  splitk_reduce_kernel<T><<<grid, 256, 0, stream>>>((const T*)partials, (T*)o.c, o.m, o.n, o.batch, splits, part_ld,
                                                    part_stride, o.ldc, o.sc, alpha, beta, beta_zero);
  return (int)cudaGetLastError();
}

int run_splitk(const blb200_gemm_desc* d, const SplitPlan& pl, void* scratch, cudaStream_t stream) {
  const GemmParams orig = to_params_public(d);
  GemmParams p = orig;
  p.c = scratch;
  p.ldc = pl.ld;
  p.sc = pl.stride;
  p.batch = orig.batch * pl.splits;
  p.alpha[0] = 1.0; p.alpha[1] = 0.0;
  p.beta[0] = 0.0; p.beta[1] = 0.0;
  p.splits = pl.splits;
  p.kchunk = pl.kchunk;
  p.split_a = (orig.op_a == BLB200_N) ? (long long)pl.kchunk * orig.lda : pl.kchunk;
  p.split_b = (orig.op_b == BLB200_N) ? pl.kchunk : (long long)pl.kchunk * orig.ldb;
  int rc;
  if (dmma_supported(p, d->dtype)) rc = launch_dmma(p, d->dtype, stream);
  else if (sgemm128_supported(p, d->dtype)) rc = launch_sgemm128(p, d->dtype, stream);
  else if (tiled_supported(p, d->dtype)) rc = launch_tiled(p, d->dtype, stream);
  else rc = launch_generic(p, d->dtype, stream);
  if (rc != BLB200_OK) return rc;
  rc = launch_splitk_reduce(orig, d->dtype, scratch, pl.splits, pl.ld, pl.stride, stream);
  if (rc == BLB200_OK) note_launch("splitk");
  return rc;
}

}  // namespace

int launch_splitk_reduce(const GemmParams& orig, int dtype, const void* partials, int splits, long long part_ld,
                         long long part_stride, cudaStream_t stream) {
  switch (dtype) {
    case BLB200_S: return reduce_typed<float>(orig, partials, splits, part_ld, part_stride, stream);
    case BLB200_D: return reduce_typed<double>(orig, partials, splits, part_ld, part_stride, stream);
    case BLB200_C: return reduce_typed<float2>(orig, partials, splits, part_ld, part_stride, stream);
    case BLB200_Z: return reduce_typed<double2>(orig, partials, splits, part_ld, part_stride, stream);
    default: return BLB200_E_DTYPE;
  }
}

// ---- fixed scratch for callers that must not allocate ----------------------------------------------
// The partials of blb200_gemm_splitk_static live in this array.  It is part of the library image:
// every GPU that loads the library sets the bytes aside until the process exits.
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_splitk_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, not something a kernel can dereference, so the address is asked for
// once per device (with that device current) and remembered.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cached[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return BLB200_E_NO_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_splitk_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!ptr) return BLB200_E_INTERNAL;
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return BLB200_OK;
}

}  // namespace blb200

extern "C" {

size_t blb200_gemm_splitk_static_capacity(void) { return blb200::kStaticScratchBytes; }

int blb200_gemm_splitk_static(const blb200_gemm_desc* desc, int32_t splits, void* cuda_stream) {
  int rc = blb200_gemm_validate(desc);
  if (rc != BLB200_OK) return rc;
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  const blb200::SplitPlan pl = blb200::plan_split(*desc, splits);
  if (pl.splits < 2) return blb200::dispatch(desc, (cudaStream_t)cuda_stream);  // needs no scratch at all
  if (pl.bytes > blb200::kStaticScratchBytes) return BLB200_E_TOO_LARGE;
  void* scratch = nullptr;
  rc = blb200::static_scratch_address(&scratch);
  if (rc != BLB200_OK) return rc;
  // Every element of every partial window is written by the tile kernel before the reduce pass
  // reads it, so nothing left over from an earlier call has to be cleared first.
  return blb200::run_splitk(desc, pl, scratch, (cudaStream_t)cuda_stream);
}

int32_t blb200_gemm_splitk_plan(const blb200_gemm_desc* desc, int32_t splits, size_t* workspace_bytes) {
  if (workspace_bytes) *workspace_bytes = 0;
  if (blb200_gemm_validate(desc) != BLB200_OK) return 1;
  const blb200::SplitPlan pl = blb200::plan_split(*desc, splits);
  if (workspace_bytes) *workspace_bytes = pl.bytes;
  return pl.splits;
}

int blb200_gemm_splitk(const blb200_gemm_desc* desc, int32_t splits, void* workspace, size_t workspace_bytes,
                       void* cuda_stream) {
  int rc = blb200_gemm_validate(desc);
  if (rc != BLB200_OK) return rc;
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  const blb200::SplitPlan pl = blb200::plan_split(*desc, splits);
  if (pl.splits < 2) return blb200::dispatch(desc, (cudaStream_t)cuda_stream);  // nothing to split
  if (!workspace) return BLB200_E_NULL;
  if (workspace_bytes < pl.bytes) return BLB200_E_TOO_LARGE;
  if (reinterpret_cast<uintptr_t>(workspace) & 15u) return BLB200_E_UNSUPPORTED;
  return blb200::run_splitk(desc, pl, workspace, (cudaStream_t)cuda_stream);
}

}  // extern "C"
