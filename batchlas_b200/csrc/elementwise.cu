// Elementwise helpers on batched column-major views: C <- A (op) B and C <- alpha*A + beta*B.
// Pure streaming work (two reads and one write per element), so the kernels are shaped for HBM:
// when the three views are packed and 16-byte aligned the whole batch is one flat array walked with
// 16-byte accesses; otherwise a thread block walks one item column by column, consecutive threads on
// consecutive rows, so that padded leading dimensions, slices and batch gaps cost nothing but the
// bytes they skip.  C may alias A or B: each element is read and written by the same thread.
#include "common.cuh"

namespace blb200 {
namespace {

enum { kAdd = 0, kSub = 1, kMul = 2, kDiv = 3, kAxpby = 4 };

template <typename T>
__device__ __forceinline__ T cdiv(T a, T b) {  // complex a / b, scaled by the larger part of b (Smith)
  using R = decltype(a.x);
  if (fabs(b.x) >= fabs(b.y)) {
    const R r = b.y / b.x, den = b.x + b.y * r;
    return T{(a.x + a.y * r) / den, (a.y - a.x * r) / den};
  }
  const R r = b.x / b.y, den = b.x * r + b.y;
  return T{(a.x * r + a.y) / den, (a.y * r - a.x) / den};
}

template <typename T, int OP>
__device__ __forceinline__ T apply(T a, T b, T alpha, T beta) {
  if constexpr (OP == kAxpby) {
    T out = Scalar<T>::mul(alpha, a);
    Scalar<T>::fma(out, beta, b);
    return out;
  } else if constexpr (Scalar<T>::is_complex) {
    if constexpr (OP == kAdd) return T{a.x + b.x, a.y + b.y};
    else if constexpr (OP == kSub) return T{a.x - b.x, a.y - b.y};
    else if constexpr (OP == kMul) return Scalar<T>::mul(a, b);
    else return cdiv(a, b);
  } else {
    if constexpr (OP == kAdd) return a + b;
    else if constexpr (OP == kSub) return a - b;
    else if constexpr (OP == kMul) return a * b;
    else return a / b;
  }
}

struct EwiseParams {
  const void* a;
  const void* b;
  void* c;
  int rows, cols, batch;
  long long lda, ldb, ldc, sa, sb, sc;
  double alpha[2], beta[2];
};

// Packed views: one flat array of `total` elements, V = 16 / sizeof(T) per access.
template <typename T, int OP>
__global__ void __launch_bounds__(256) ewise_flat_kernel(const T* a, const T* b, T* c,
                                                         long long total, T alpha, T beta) {
  constexpr int V = 16 / (int)sizeof(T);
  union Pack {
    uint4 u;
    T t[V];
  };
  const long long vecs = total / V, step = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long i = tid;
  for (; i + step < vecs; i += 2 * step) {  // two independent 16-byte triples in flight per thread
    Pack a0, b0, a1, b1;
    a0.u = reinterpret_cast<const uint4*>(a)[i];
    b0.u = reinterpret_cast<const uint4*>(b)[i];
    a1.u = reinterpret_cast<const uint4*>(a)[i + step];
    b1.u = reinterpret_cast<const uint4*>(b)[i + step];
#pragma unroll
    for (int e = 0; e < V; ++e) {
      a0.t[e] = apply<T, OP>(a0.t[e], b0.t[e], alpha, beta);
      a1.t[e] = apply<T, OP>(a1.t[e], b1.t[e], alpha, beta);
    }
    reinterpret_cast<uint4*>(c)[i] = a0.u;
    reinterpret_cast<uint4*>(c)[i + step] = a1.u;
  }
  for (; i < vecs; i += step) {
    Pack av, bv;
    av.u = reinterpret_cast<const uint4*>(a)[i];
    bv.u = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
    for (int e = 0; e < V; ++e) av.t[e] = apply<T, OP>(av.t[e], bv.t[e], alpha, beta);
    reinterpret_cast<uint4*>(c)[i] = av.u;
  }
  for (long long e = vecs * V + tid; e < total; e += step) c[e] = apply<T, OP>(a[e], b[e], alpha, beta);
}

// Any ld / stride: blockIdx.x walks (item, column block) pairs, threads run down the rows.
template <typename T, int OP>
__global__ void __launch_bounds__(256) ewise_strided_kernel(EwiseParams p, T alpha, T beta, int col_blocks,
                                                            int cols_per_block) {
  const long long work = (long long)col_blocks * p.batch;
  for (long long w = blockIdx.x; w < work; w += gridDim.x) {
    const long long item = w / col_blocks;
    const int c0 = (int)(w - item * col_blocks) * cols_per_block, c1 = min(p.cols, c0 + cols_per_block);
    const T* a = (const T*)p.a + item * p.sa;
    const T* b = (const T*)p.b + item * p.sb;
    T* c = (T*)p.c + item * p.sc;
    // (row, column) pairs of the block flattened, four independent triples in flight per thread
    const int n = (c1 - c0) * p.rows;
    for (int base = threadIdx.x; base < n; base += 4 * (int)blockDim.x) {
      T av[4], bv[4];
      long long oc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int f = base + u * (int)blockDim.x;
        oc[u] = -1;
        if (f < n) {
          const int jj = f / p.rows, i = f - jj * p.rows, j = c0 + jj;
          av[u] = a[(long long)j * p.lda + i];
          bv[u] = b[(long long)j * p.ldb + i];
          oc[u] = (long long)j * p.ldc + i;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (oc[u] >= 0) c[oc[u]] = apply<T, OP>(av[u], bv[u], alpha, beta);
    }
  }
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <typename T, int OP>
int launch_op(const EwiseParams& p, cudaStream_t stream) {
  const T alpha = Scalar<T>::make(p.alpha[0], p.alpha[1]), beta = Scalar<T>::make(p.beta[0], p.beta[1]);
  const long long per_item = (long long)p.rows * p.cols, total = per_item * p.batch;
  const long long cap = (long long)device_info().sm_count * 8;
  auto packed = [&](long long ld, long long st) { return (ld == p.rows || p.cols == 1) && (st == per_item || p.batch == 1); };
  if (packed(p.lda, p.sa) && packed(p.ldb, p.sb) && packed(p.ldc, p.sc) && aligned16(p.a) && aligned16(p.b) &&
      aligned16(p.c)) {
    const long long vecs = total / (16 / (long long)sizeof(T));
    const long long want = (vecs / 2 + 255) / 256 + 1;
    ewise_flat_kernel<T, OP><<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>((const T*)p.a, (const T*)p.b, (T*)p.c,
                                                                                    total, alpha, beta);
    return (int)cudaGetLastError();
  }
  // about 16 K elements per block visit, whole columns
  int cols_per_block = (int)((16384 + p.rows - 1) / p.rows);
  if (cols_per_block > p.cols) cols_per_block = p.cols;
  if (cols_per_block < 1) cols_per_block = 1;
  const int col_blocks = (p.cols + cols_per_block - 1) / cols_per_block;
  const long long work = (long long)col_blocks * p.batch;
  ewise_strided_kernel<T, OP><<<(unsigned)(work < cap ? work : cap), 256, 0, stream>>>(p, alpha, beta, col_blocks,
                                                                                      cols_per_block);
  return (int)cudaGetLastError();
}

template <typename T>
int launch_typed(const EwiseParams& p, int op, cudaStream_t stream) {
  switch (op) {
    case kAdd: return launch_op<T, kAdd>(p, stream);
    case kSub: return launch_op<T, kSub>(p, stream);
    case kMul: return launch_op<T, kMul>(p, stream);
    case kDiv: return launch_op<T, kDiv>(p, stream);
    case kAxpby: return launch_op<T, kAxpby>(p, stream);
    default: return BLB200_E_DTYPE;
  }
}

int run(const blb200_ewise_desc* d, int op, const double* alpha, const double* beta, cudaStream_t stream) {
  if (!d) return BLB200_E_NULL;
  if (d->dtype < BLB200_S || d->dtype > BLB200_Z || op < kAdd || op > kAxpby) return BLB200_E_DTYPE;
  if (d->rows < 0 || d->cols < 0 || d->batch < 0) return BLB200_E_SHAPE;
  const long long min_ld = d->rows > 1 ? d->rows : 1;
  if (d->lda < min_ld || d->ldb < min_ld || d->ldc < min_ld) return BLB200_E_SHAPE;
  if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0) return BLB200_E_SHAPE;
  if (d->rows == 0 || d->cols == 0 || d->batch == 0) return BLB200_OK;
  if (!d->a || !d->b || !d->c) return BLB200_E_NULL;
  EwiseParams p{};
  p.a = d->a; p.b = d->b; p.c = d->c;
  p.rows = d->rows; p.cols = d->cols; p.batch = d->batch;
  p.lda = d->lda; p.ldb = d->ldb; p.ldc = d->ldc;
  p.sa = d->stride_a; p.sb = d->stride_b; p.sc = d->stride_c;
  const bool cplx = d->dtype >= BLB200_C;
  if (alpha) { p.alpha[0] = alpha[0]; p.alpha[1] = cplx ? alpha[1] : 0.0; }
  if (beta) { p.beta[0] = beta[0]; p.beta[1] = cplx ? beta[1] : 0.0; }
  int rc;
  switch (d->dtype) {
    case BLB200_S: rc = launch_typed<float>(p, op, stream); break;
    case BLB200_D: rc = launch_typed<double>(p, op, stream); break;
    case BLB200_C: rc = launch_typed<float2>(p, op, stream); break;
    default: rc = launch_typed<double2>(p, op, stream); break;
  }
  if (rc == BLB200_OK) note_launch(op == kAxpby ? "axpby" : "elementwise");
  return rc;
}

}  // namespace
}  // namespace blb200

extern "C" {

int blb200_elementwise(const blb200_ewise_desc* desc, int32_t op, void* cuda_stream) {
  if (op < 0 || op > 3) return BLB200_E_DTYPE;
  return blb200::run(desc, op, nullptr, nullptr, (cudaStream_t)cuda_stream);
}

int blb200_axpby(const blb200_ewise_desc* desc, const double alpha[2], const double beta[2], void* cuda_stream) {
  if (!alpha || !beta) return BLB200_E_NULL;
  return blb200::run(desc, blb200::kAxpby, alpha, beta, (cudaStream_t)cuda_stream);
}

}  // extern "C"
