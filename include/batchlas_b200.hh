// batchlas_b200.hh — C++ host side of the B200 batched-GEMM path, header-only over the C ABI in
// blb200.h and the CUDA runtime.
//
// It keeps the spelling of BatchLAS's public surface for this one path, so code written as
//
//     Queue ctx(Device::default_device());
//     Matrix<float> A = ..., B = ..., C = ...;
//     gemm(ctx, A.view(), B.view(), C.view(), {.alpha = 2.0f, .transA = Transpose::Trans});
//     ctx.wait();
//
// compiles and runs unchanged.  Types mirrored (dense subset only), with the reference location of
// the interface each one replaces:
//   Device, Event, Queue           BatchLAS include/util/sycl-device-queue.hh:70-233 (global namespace
//                                  there too); a Queue is one in-order cudaStream_t on one device.
//   batchlas::WorkspaceLease       include/util/workspace.hh:70-162, arena src/queue.hh:41-226.
//   batchlas::Transpose/Backend/ComputePrecision/MatrixFormat   include/blas/enums.hh:37-82,269-276.
//   batchlas::Slice, MatrixView, Matrix    include/blas/matrix.hh:33-41,327-665,669-1196.
//   batchlas::GemmOptions, gemm(...)       include/blas/options.hh:39-46,210-222 and
//                                          include/blas/functions/gemm.hh:22-88.
//   batchlas::with_backend         include/blas/queue-dispatch.hh:29-57 (single CUDA arm here).
// Matrix storage is CUDA managed memory — host-visible like the reference's shared USM
// (src/util/sycl-util-impl.cc:36-46) — so tests can index elements on the host after ctx.wait().
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <complex>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <memory>
#include <random>
#include <span>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "blb200.h"

#define BATCHLAS_HAS_CUDA_BACKEND 1
#define BATCHLAS_HAS_ROCM_BACKEND 0
#define BATCHLAS_HAS_MKL_BACKEND 0
#define BATCHLAS_HAS_HOST_BACKEND 0

namespace batchlas {

enum class MatrixFormat { Dense, CSR, CSC, COO, SELL, BSR, BLOCKED_ELL };
enum class Backend { AUTO, CUDA, ROCM, MKL, MAGMA, SYCL, NETLIB };
enum class Transpose { NoTrans, Trans, ConjTrans };
enum class ComputePrecision { Default, F32, F64, F16, BF16, TF32 };

template <typename T>
struct base_type { using type = T; };
template <typename T>
struct base_type<std::complex<T>> { using type = T; };
template <typename T>
using float_t = typename base_type<T>::type;

class WorkspaceLease;

namespace detail {
inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void status_check(int status) {
  if (status != BLB200_OK) throw std::runtime_error(blb200_status_string(status));
}
template <typename T>
constexpr int dtype_code() {
  if constexpr (std::is_same_v<T, float>) return BLB200_S;
  else if constexpr (std::is_same_v<T, double>) return BLB200_D;
  else if constexpr (std::is_same_v<T, std::complex<float>>) return BLB200_C;
  else {
    static_assert(std::is_same_v<T, std::complex<double>>, "gemm supports float, double and their complex types");
    return BLB200_Z;
  }
}
}  // namespace detail
}  // namespace batchlas

// ---- Device / Event / Queue (global namespace, as in the reference) ------------------------------
enum class DeviceType { CPU, GPU, ACCELERATOR, HOST };

struct Device {
  static std::vector<Device> get_devices(DeviceType type) {
    std::vector<Device> out;
    if (type != DeviceType::GPU) return out;  // this build drives CUDA GPUs only
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0;
    for (int i = 0; i < n; ++i) out.emplace_back((size_t)i, DeviceType::GPU);
    return out;
  }
  Device() = default;
  Device(size_t idx, DeviceType type) : idx(idx), type(type) {}
  Device(std::string name) {
    std::transform(name.begin(), name.end(), name.begin(), ::tolower);
    if (name != "gpu") throw std::runtime_error(name == "cpu" || name == "accelerator" ? "No " + name + " device available"
                                                                                        : "Invalid device type: " + name);
    auto devs = get_devices(DeviceType::GPU);
    if (devs.empty()) throw std::runtime_error("No gpu device available");
    *this = devs.at(0);
  }
  Device(const char* name) : Device(std::string(name)) {}
  static Device default_device() {
    auto devs = get_devices(DeviceType::GPU);
    if (devs.empty()) throw std::runtime_error("No gpu device available");
    return devs.at(0);
  }
  std::string get_name() const {
    cudaDeviceProp prop;
    batchlas::detail::cuda_check(cudaGetDeviceProperties(&prop, (int)idx), "cudaGetDeviceProperties");
    return prop.name;
  }
  size_t idx = 0;
  DeviceType type = DeviceType::GPU;
};

struct Event {
  Event() = default;
  explicit Event(std::shared_ptr<CUevent_st> ev) : ev_(std::move(ev)) {}
  void wait() const {
    if (ev_) batchlas::detail::cuda_check(cudaEventSynchronize(ev_.get()), "Event::wait");
  }
  cudaEvent_t native() const { return ev_.get(); }

 private:
  std::shared_ptr<CUevent_st> ev_;
};

struct Queue {
  Queue() : Queue(Device::default_device()) {}
  Queue(Device device, bool in_order = true) : Queue(device, batchlas::Backend::AUTO, in_order) {}
  Queue(Device device, batchlas::Backend backend, bool in_order = true) : device_(device), in_order_(in_order) {
    if (device.type != DeviceType::GPU) throw std::runtime_error("Queue: only GPU devices are available in this build");
    set_backend(backend);
    make_current();
    batchlas::detail::cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    batchlas::detail::status_check(blb200_arena_create((int)device.idx, stream_, &arena_));
  }
  // A further queue on the same device (the reference shares the SYCL context; CUDA's primary
  // context is shared by construction).
  Queue(const Queue& base, bool in_order) : Queue(base.device_, base.backend_, in_order) {}
  Queue(const Queue&) = delete;
  Queue& operator=(const Queue&) = delete;
  Queue(Queue&& o) noexcept { steal(o); }
  Queue& operator=(Queue&& o) noexcept {
    if (this != &o) {
      destroy();
      steal(o);
    }
    return *this;
  }
  ~Queue() { destroy(); }

  void make_current() const { batchlas::detail::cuda_check(cudaSetDevice((int)device_.idx), "cudaSetDevice"); }
  cudaStream_t native_stream() const { return stream_; }

  void wait() const {
    make_current();
    batchlas::detail::cuda_check(cudaStreamSynchronize(stream_), "Queue::wait");
  }
  void wait_and_throw() const { wait(); }
  Event get_event() const { return record(); }
  // The launcher enqueues on this queue's own stream, so "after external work" is simply "now".
  Event create_event_after_external_work() { return record(); }
  void enqueue(Event& ev) {
    if (ev.native()) batchlas::detail::cuda_check(cudaStreamWaitEvent(stream_, ev.native(), 0), "cudaStreamWaitEvent");
  }

  [[nodiscard]] inline batchlas::WorkspaceLease workspace(size_t bytes);
  size_t workspace_capacity() const { return blb200_arena_capacity(arena_); }
  [[nodiscard]] bool trim_workspace() {
    int rc = blb200_arena_trim(arena_);
    if (rc < 0) batchlas::detail::status_check(rc);
    return rc == 1;
  }

  Device device() const { return device_; }
  bool in_order() const { return in_order_; }
  batchlas::Backend backend() const { return batchlas::Backend::CUDA; }  // AUTO resolves to the only arm
  batchlas::Backend requested_backend() const { return backend_; }
  void set_backend(batchlas::Backend b) {
    if (!backend_available(b)) throw std::runtime_error("Queue::set_backend: backend not compiled into this build");
    backend_ = b;
  }
  static bool backend_available(batchlas::Backend b) {
    return b == batchlas::Backend::AUTO || b == batchlas::Backend::CUDA;
  }
  blb200_arena* arena() const { return arena_; }

 private:
  Event record() const {
    make_current();
    cudaEvent_t ev = nullptr;
    batchlas::detail::cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    std::shared_ptr<CUevent_st> sp(ev, [](cudaEvent_t e) { cudaEventDestroy(e); });
    batchlas::detail::cuda_check(cudaEventRecord(ev, stream_), "cudaEventRecord");
    return Event(sp);
  }
  void steal(Queue& o) {
    device_ = o.device_;
    in_order_ = o.in_order_;
    backend_ = o.backend_;
    stream_ = o.stream_;
    arena_ = o.arena_;
    o.stream_ = nullptr;
    o.arena_ = nullptr;
  }
  void destroy() noexcept {
    if (!stream_ && !arena_) return;
    cudaSetDevice((int)device_.idx);
    if (stream_) cudaStreamSynchronize(stream_);  // enqueued kernels may still read arena blocks
    if (arena_) blb200_arena_destroy(arena_);
    if (stream_) cudaStreamDestroy(stream_);
    stream_ = nullptr;
    arena_ = nullptr;
  }
  Device device_;
  bool in_order_ = true;
  batchlas::Backend backend_ = batchlas::Backend::AUTO;
  cudaStream_t stream_ = nullptr;
  blb200_arena* arena_ = nullptr;
};

namespace batchlas {

// Scoped borrow of device scratch from a Queue's arena; move-only, releases on destruction.
class WorkspaceLease {
 public:
  WorkspaceLease() = default;
  WorkspaceLease(const WorkspaceLease&) = delete;
  WorkspaceLease& operator=(const WorkspaceLease&) = delete;
  WorkspaceLease(WorkspaceLease&& o) noexcept : arena_(o.arena_), lease_(o.lease_) { o.arena_ = nullptr; o.lease_ = {}; }
  WorkspaceLease& operator=(WorkspaceLease&& o) noexcept {
    if (this != &o) {
      release();  // necessarily out of order: `o` was acquired before this one is returned
      arena_ = o.arena_;
      lease_ = o.lease_;
      o.arena_ = nullptr;
      o.lease_ = {};
    }
    return *this;
  }
  ~WorkspaceLease() { release(); }
  std::byte* data() const { return static_cast<std::byte*>(lease_.ptr); }
  std::size_t size() const { return lease_.bytes; }
  void release() noexcept {
    if (arena_ && lease_.seq) blb200_arena_release(arena_, &lease_);
    arena_ = nullptr;
    lease_ = {};
  }

 private:
  friend struct ::Queue;
  WorkspaceLease(blb200_arena* a, const blb200_lease& l) : arena_(a), lease_(l) {}
  blb200_arena* arena_ = nullptr;
  blb200_lease lease_{};
};

struct SliceEnd {};
struct Slice {  // default selects everything
  int64_t start = std::numeric_limits<int64_t>::min();
  int64_t end = std::numeric_limits<int64_t>::max();
  Slice() = default;
  Slice(int64_t s, SliceEnd) : start(s) {}
  Slice(int64_t s, int64_t e) : start(s), end(e) {}
  Slice(int64_t s) : start(s) {}
};

namespace detail {
inline std::pair<int64_t, int64_t> normalize_slice(Slice s, int64_t extent) {
  int64_t b = s.start == std::numeric_limits<int64_t>::min() ? 0 : (s.start < 0 ? s.start + extent : s.start);
  int64_t e = s.end == std::numeric_limits<int64_t>::max() ? extent : (s.end < 0 ? s.end + extent : s.end);
  b = std::clamp<int64_t>(b, 0, extent);
  e = std::clamp<int64_t>(e, 0, extent);
  return {b, e - b};
}
}  // namespace detail

// Non-owning column-major view: element (i, j) of item b is data[b*stride + j*ld + i].
// The reference's optional per-item pointer array (data_ptrs, include/blas/matrix.hh:672-686) is not
// mirrored: nothing on the gemm path reads it (its users are the pointer-array solver calls such as
// batched trsm and getrs, src/backends/cublas.cc:1245,1503-1557).
template <typename T, MatrixFormat MType = MatrixFormat::Dense>
class MatrixView {
  static_assert(MType == MatrixFormat::Dense, "only dense views are on this path");

 public:
  MatrixView() = default;
  MatrixView(T* data, int rows, int cols, int ld = 0, int64_t stride = 0, int batch_size = 1)
      : data_(data), rows_(rows), cols_(cols), ld_(ld > 0 ? ld : rows),
        stride_(stride > 0 ? stride : (int64_t)(ld > 0 ? ld : rows) * cols), batch_size_(batch_size) {}
  T* data_ptr() const { return data_; }
  int rows() const { return rows_; }
  int cols() const { return cols_; }
  // Per-item active dimensions of a heterogeneous batch (device-readable int[batch], or null).
  int rows(int b) const { return active_rows_ ? active_rows_[b] : rows_; }
  int cols(int b) const { return active_cols_ ? active_cols_[b] : cols_; }
  bool is_heterogeneous() const { return active_rows_ || active_cols_; }
  const int* active_rows() const { return active_rows_; }
  const int* active_cols() const { return active_cols_; }
  MatrixView& set_active_dims(const int* active_rows, const int* active_cols) {
    active_rows_ = active_rows;
    active_cols_ = active_cols;
    return *this;
  }
  int ld() const { return ld_; }
  int64_t stride() const { return stride_; }
  int batch_size() const { return batch_size_; }
  T& at(int row, int col, int batch = 0) const { return data_[(int64_t)batch * stride_ + (int64_t)col * ld_ + row]; }
  T& operator()(int row, int col, int batch = 0) const { return at(row, col, batch); }
  MatrixView batch_item(int b) const {
    if (b < 0 || b >= batch_size_) throw std::out_of_range("Batch index out of range");
    return MatrixView(data_ + (int64_t)b * stride_, rows(b), cols(b), ld_);
  }
  MatrixView operator[](int b) const { return batch_item(b); }
  MatrixView operator()(Slice rows, Slice cols) const {
    auto [r0, rl] = detail::normalize_slice(rows, rows_);
    auto [c0, cl] = detail::normalize_slice(cols, cols_);
    if (rl <= 0 || cl <= 0)
      throw std::invalid_argument("Invalid slice dimensions: " + std::to_string(rl) + "x" + std::to_string(cl));
    return MatrixView(data_ + c0 * ld_ + r0, (int)rl, (int)cl, ld_, stride_, batch_size_);
  }
  MatrixView operator()(Slice rows) const { return (*this)(rows, {}); }

 private:
  T* data_ = nullptr;
  int rows_ = 0, cols_ = 0, ld_ = 0;
  int64_t stride_ = 0;
  int batch_size_ = 1;
  const int* active_rows_ = nullptr;
  const int* active_cols_ = nullptr;
};

// Owning batch of column-major matrices in managed (host-visible) memory.
template <typename T, MatrixFormat MType = MatrixFormat::Dense>
class Matrix {
  static_assert(MType == MatrixFormat::Dense, "only dense matrices are on this path");

 public:
  Matrix() = default;
  Matrix(int rows, int cols, int batch_size = 1, int ld = 0, int64_t stride = 0)
      : rows_(rows), cols_(cols), batch_size_(batch_size), ld_(ld > 0 ? ld : rows),
        stride_(stride > 0 ? stride : (int64_t)(ld > 0 ? ld : rows) * cols) {
    const size_t n = std::max<size_t>(1, (size_t)stride_ * (size_t)batch_size_);
    void* p = nullptr;
    detail::cuda_check(cudaMallocManaged(&p, n * sizeof(T)), "Matrix: cudaMallocManaged");
    data_.reset(static_cast<T*>(p), [](T* q) { cudaFree(q); });
    count_ = n;
  }
  Matrix(const Matrix&) = delete;
  Matrix& operator=(const Matrix&) = delete;
  Matrix(Matrix&&) noexcept = default;
  Matrix& operator=(Matrix&&) noexcept = default;

  static Matrix Zeros(int rows, int cols, int batch_size = 1) {
    Matrix m(rows, cols, batch_size);
    m.fill(T(0));
    return m;
  }
  static Matrix Identity(int n, int batch_size = 1) {
    Matrix m = Zeros(n, n, batch_size);
    for (int b = 0; b < batch_size; ++b)
      for (int i = 0; i < n; ++i) m(i, i, b) = T(1);
    return m;
  }
  // uniform[-1, 1]; the reference draws from a oneDPL minstd stream (src/matrix.cc:938-990) that
  // cannot be reproduced without oneDPL, so only the distribution is kept.
  static Matrix Random(int rows, int cols, bool hermitian = false, int batch_size = 1, unsigned seed = 42) {
    Matrix m(rows, cols, batch_size);
    std::mt19937_64 gen(seed);
    std::uniform_real_distribution<double> dist(-1.0, 1.0);
    for (int b = 0; b < batch_size; ++b)
      for (int j = 0; j < cols; ++j)
        for (int i = 0; i < rows; ++i) {
          if constexpr (std::is_floating_point_v<T>) m(i, j, b) = (T)dist(gen);
          else m(i, j, b) = T((float_t<T>)dist(gen), (float_t<T>)dist(gen));
        }
    if (hermitian && rows == cols)
      for (int b = 0; b < batch_size; ++b)
        for (int j = 0; j < cols; ++j)
          for (int i = 0; i <= j; ++i) {
            if constexpr (std::is_floating_point_v<T>) m(j, i, b) = m(i, j, b);
            else {
              if (i == j) m(i, i, b) = T(m(i, i, b).real(), 0);
              m(j, i, b) = std::conj(m(i, j, b));
            }
          }
    return m;
  }

  void fill(T v) { std::fill(data_.get(), data_.get() + count_, v); }
  Matrix clone() const {
    Matrix m(rows_, cols_, batch_size_, ld_, stride_);
    std::copy(data_.get(), data_.get() + count_, m.data_.get());
    return m;
  }
  MatrixView<T, MType> view() const {
    MatrixView<T, MType> v(data_.get(), rows_, cols_, ld_, stride_, batch_size_);
    if (active_) v.set_active_dims(active_.get(), active_.get() + batch_size_);
    return v;
  }
  // Per-item active dims (each <= the allocated rows/cols), kept in managed memory so that both the
  // host checks and the kernel can read them.  Empty vectors clear them.
  Matrix& set_active_dims(const std::vector<int>& active_rows, const std::vector<int>& active_cols) {
    if (active_rows.empty() && active_cols.empty()) {
      active_.reset();
      return *this;
    }
    if ((int)active_rows.size() != batch_size_ || (int)active_cols.size() != batch_size_)
      throw std::invalid_argument("active dims must have one entry per batch item");
    for (int b = 0; b < batch_size_; ++b)
      if (active_rows[b] < 0 || active_rows[b] > rows_ || active_cols[b] < 0 || active_cols[b] > cols_)
        throw std::invalid_argument("active dims exceed the matrix capacity");
    void* p = nullptr;
    detail::cuda_check(cudaMallocManaged(&p, sizeof(int) * 2 * (size_t)batch_size_), "Matrix: cudaMallocManaged");
    active_.reset(static_cast<int*>(p), [](int* q) { cudaFree(q); });
    std::copy(active_rows.begin(), active_rows.end(), active_.get());
    std::copy(active_cols.begin(), active_cols.end(), active_.get() + batch_size_);
    return *this;
  }
  bool is_heterogeneous() const { return (bool)active_; }
  int rows(int b) const { return active_ ? active_.get()[b] : rows_; }
  int cols(int b) const { return active_ ? active_.get()[batch_size_ + b] : cols_; }
  operator MatrixView<T, MType>() const { return view(); }
  T& operator()(int i, int j, int b = 0) const { return data_.get()[(int64_t)b * stride_ + (int64_t)j * ld_ + i]; }
  T* data_ptr() const { return data_.get(); }
  int rows() const { return rows_; }
  int cols() const { return cols_; }
  int ld() const { return ld_; }
  int64_t stride() const { return stride_; }
  int batch_size() const { return batch_size_; }

 private:
  std::shared_ptr<T> data_;
  std::shared_ptr<int> active_;
  size_t count_ = 0;
  int rows_ = 0, cols_ = 0, batch_size_ = 1, ld_ = 0;
  int64_t stride_ = 0;
};

template <typename T, MatrixFormat M>
inline std::pair<int, int> get_effective_dims(const MatrixView<T, M>& mat, Transpose trans) {
  return trans == Transpose::NoTrans ? std::make_pair(mat.rows(), mat.cols()) : std::make_pair(mat.cols(), mat.rows());
}

template <typename T>
struct GemmOptions {
  T alpha = T(1);
  T beta = T(0);
  Transpose transA = Transpose::NoTrans;
  Transpose transB = Transpose::NoTrans;
  ComputePrecision precision = ComputePrecision::Default;
};

template <typename F>
inline auto with_backend(Queue& ctx, F&& f) {
  switch (ctx.backend()) {
    case Backend::CUDA: return f(std::integral_constant<Backend, Backend::CUDA>{});
    default: break;
  }
  throw std::runtime_error("BatchLAS: this Queue's backend has no implementation in this build. "
                           "Check Queue::backend_available() before pinning a backend.");
}

namespace detail {
// A backend this build certainly has, used only to ask whether a positional call would compile.
inline constexpr Backend kProbeBackend = Backend::CUDA;
}  // namespace detail

// BATCHLAS_DISPATCH_ON_QUEUE(NAME): for an entry point declared as
//     template <Backend Back, typename T, ...> R NAME(Queue&, ...);
// defines NAME(queue, args...) that looks the backend up on the queue (BatchLAS
// include/blas/queue-dispatch.hh:103-113).  The arguments travel as a pack, so the primary's default
// arguments still apply, and the requires-clause admits only argument lists that the Backend-first
// form accepts — any other call leaves this overload out of resolution instead of failing inside it.
#define BATCHLAS_DISPATCH_ON_QUEUE(NAME)                                                        \
  template <typename... CallArgs>                                                                \
    requires requires(::Queue& probe_queue, CallArgs&&... probe_args) {                          \
      NAME<::batchlas::detail::kProbeBackend>(probe_queue, std::forward<CallArgs>(probe_args)...); \
    }                                                                                            \
  inline auto NAME(::Queue& queue, CallArgs&&... call_args) {                                    \
    return ::batchlas::with_backend(queue, [&](auto backend_tag) {                               \
      return NAME<backend_tag.value>(queue, std::forward<CallArgs>(call_args)...);               \
    });                                                                                          \
  }

// The seam: gemm<Backend::CUDA, T> (replaces BatchLAS src/backends/cublas.cc:1574-1585).
template <Backend Back, typename T>
Event gemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
           const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Transpose transA, Transpose transB,
           ComputePrecision precision = ComputePrecision::Default) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  constexpr bool is_f32 = std::is_same_v<float_t<T>, float>;
  // Reduced-precision requests change results; only the storage precision is accepted.
  if (!(precision == ComputePrecision::Default || (is_f32 && precision == ComputePrecision::F32) ||
        (!is_f32 && precision == ComputePrecision::F64)))
    throw std::runtime_error("GEMM: reduced compute precision is not available on this path");
  auto [m, k] = get_effective_dims(A, transA);
  auto [kb, n] = get_effective_dims(B, transB);
  if (A.batch_size() != B.batch_size() || A.batch_size() != C.batch_size() || k != kb || C.rows() != m ||
      C.cols() != n || m < 0 || n < 0 || k < 0)
    throw std::runtime_error("GEMM: incompatible matrix dimensions");
  const bool hetero = A.is_heterogeneous() || B.is_heterogeneous() || C.is_heterogeneous();
  if (hetero) {
    // per-item check on the host, as gemm_batch_dimensions_compatible does (gemm_variant.hh:29-41);
    // the arrays are managed memory, so the queue is drained first
    ctx.wait();
    for (int b = 0; b < A.batch_size(); ++b) {
      const int mi = transA == Transpose::NoTrans ? A.rows(b) : A.cols(b), ki = transA == Transpose::NoTrans ? A.cols(b) : A.rows(b);
      const int kj = transB == Transpose::NoTrans ? B.rows(b) : B.cols(b), ni = transB == Transpose::NoTrans ? B.cols(b) : B.rows(b);
      if (ki != kj || C.rows(b) != mi || C.cols(b) != ni || mi < 0 || ni < 0 || ki < 0)
        throw std::runtime_error("GEMM: incompatible matrix dimensions");
    }
  }
  blb200_gemm_desc d{};
  d.a = A.data_ptr();
  d.b = B.data_ptr();
  d.c = C.data_ptr();
  d.m = m; d.n = n; d.k = k; d.batch = A.batch_size();
  d.lda = A.ld(); d.ldb = B.ld(); d.ldc = C.ld();
  d.stride_a = A.stride(); d.stride_b = B.stride(); d.stride_c = C.stride();
  if constexpr (std::is_floating_point_v<T>) {
    d.alpha[0] = alpha; d.beta[0] = beta;
  } else {
    d.alpha[0] = alpha.real(); d.alpha[1] = alpha.imag();
    d.beta[0] = beta.real(); d.beta[1] = beta.imag();
  }
  d.dtype = detail::dtype_code<T>();
  d.op_a = (int)transA;
  d.op_b = (int)transB;
  ctx.make_current();
  if (hetero) {
    const int* mi = C.active_rows() ? C.active_rows() : (transA == Transpose::NoTrans ? A.active_rows() : A.active_cols());
    const int* ni = C.active_cols() ? C.active_cols() : (transB == Transpose::NoTrans ? B.active_cols() : B.active_rows());
    const int* ki = (transA == Transpose::NoTrans ? A.active_cols() : A.active_rows());
    if (!ki) ki = (transB == Transpose::NoTrans ? B.active_rows() : B.active_cols());
    detail::status_check(blb200_gemm_heterogeneous(&d, mi, ni, ki, ctx.native_stream()));
  } else {
    // Few output tiles and a long k: split k across the GPU, scratch leased from the queue's arena
    // for the duration of the call (the stream is in order, so the bytes may be re-lent afterwards).
    size_t ws_bytes = 0;
    const int splits = blb200_gemm_splitk_plan(&d, 0, &ws_bytes);
    if (splits > 1) {
      WorkspaceLease ws = ctx.workspace(ws_bytes);
      detail::status_check(blb200_gemm_splitk(&d, splits, ws.data(), ws.size(), ctx.native_stream()));
    } else {
      detail::status_check(blb200_gemm_strided_batched(&d, ctx.native_stream()));
    }
  }
  return ctx.create_event_after_external_work();
}

// gemm on views with per-item active dimensions; same call as gemm (the reference keeps both names,
// include/blas/functions/gemm.hh:48-78).
template <Backend Back, typename T>
inline Event gemm_heterogeneous(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A,
                                const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C,
                                T alpha, T beta, Transpose transA, Transpose transB,
                                ComputePrecision precision = ComputePrecision::Default) {
  return gemm<Back, T>(ctx, A, B, C, alpha, beta, transA, transB, precision);
}
template <typename T>
inline Event gemm_heterogeneous(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A,
                                const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C,
                                T alpha, T beta, Transpose transA, Transpose transB,
                                ComputePrecision precision = ComputePrecision::Default) {
  return gemm_heterogeneous<Backend::CUDA, T>(ctx, A, B, C, alpha, beta, transA, transB, precision);
}

template <Backend Back, typename T>
inline Event gemm(Queue& ctx, const Matrix<T>& A, const Matrix<T>& B, const Matrix<T>& C, T alpha, T beta,
                  Transpose transA, Transpose transB, ComputePrecision precision = ComputePrecision::Default) {
  return gemm<Back, T>(ctx, A.view(), B.view(), C.view(), alpha, beta, transA, transB, precision);
}

// Backend-deducing positional overloads.
template <typename T>
inline Event gemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Transpose transA, Transpose transB,
                  ComputePrecision precision = ComputePrecision::Default) {
  return with_backend(ctx, [&](auto Bk) { return gemm<Bk.value, T>(ctx, A, B, C, alpha, beta, transA, transB, precision); });
}
template <typename T>
inline Event gemm(Queue& ctx, const Matrix<T>& A, const Matrix<T>& B, const Matrix<T>& C, T alpha, T beta,
                  Transpose transA, Transpose transB, ComputePrecision precision = ComputePrecision::Default) {
  return gemm<T>(ctx, A.view(), B.view(), C.view(), alpha, beta, transA, transB, precision);
}

// Option-struct spellings; T comes from the matrix arguments so `{.alpha = 2.0f}` binds.
template <Backend Back, typename T>
inline Event gemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, const GemmOptions<std::type_identity_t<T>>& o) {
  return gemm<Back, T>(ctx, A, B, C, o.alpha, o.beta, o.transA, o.transB, o.precision);
}
template <typename T>
inline Event gemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, const GemmOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return gemm<Bk.value, T>(ctx, A, B, C, o); });
}
template <typename T>
inline Event gemm(Queue& ctx, const Matrix<T>& A, const Matrix<T>& B, const Matrix<T>& C,
                  const GemmOptions<std::type_identity_t<T>>& o = {}) {
  return gemm<T>(ctx, A.view(), B.view(), C.view(), o);
}

// gemm over several GPUs of the box with the operands in HOST memory (views over pinned or pageable
// host storage): the batch is cut into contiguous ranges, one per queue's device, each range runs
// its own copy / compute pipeline from a host thread of its own and writes its slice of C; nothing
// crosses between GPUs.  One Queue per GPU is how BatchLAS addresses a specific GPU
// (include/util/sycl-device-queue.hh:75); the reference itself has no multi-GPU call.  Synchronous.
template <typename T>
inline void gemm_host(std::span<Queue> queues, const MatrixView<T, MatrixFormat::Dense>& A,
                      const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C,
                      const GemmOptions<std::type_identity_t<T>>& o = {}) {
  if (queues.empty()) throw std::runtime_error("gemm_host: no queue given");
  if (o.precision != ComputePrecision::Default)
    throw std::runtime_error("GEMM: reduced compute precision is not available on this path");
  auto [m, k] = get_effective_dims(A, o.transA);
  auto [kb, n] = get_effective_dims(B, o.transB);
  if (A.batch_size() != B.batch_size() || A.batch_size() != C.batch_size() || k != kb || C.rows() != m || C.cols() != n)
    throw std::runtime_error("GEMM: incompatible matrix dimensions");
  blb200_gemm_desc d{};
  d.a = A.data_ptr(); d.b = B.data_ptr(); d.c = C.data_ptr();
  d.m = m; d.n = n; d.k = k; d.batch = A.batch_size();
  d.lda = A.ld(); d.ldb = B.ld(); d.ldc = C.ld();
  d.stride_a = A.stride(); d.stride_b = B.stride(); d.stride_c = C.stride();
  if constexpr (std::is_floating_point_v<T>) {
    d.alpha[0] = o.alpha; d.beta[0] = o.beta;
  } else {
    d.alpha[0] = o.alpha.real(); d.alpha[1] = o.alpha.imag();
    d.beta[0] = o.beta.real(); d.beta[1] = o.beta.imag();
  }
  d.dtype = detail::dtype_code<T>();
  d.op_a = (int)o.transA;
  d.op_b = (int)o.transB;
  std::vector<int32_t> devices;
  for (Queue& q : queues) {
    q.wait();  // the host entry runs on streams of its own: earlier work on the queues comes first
    devices.push_back((int32_t)q.device().idx);
  }
  detail::status_check(blb200_gemm_strided_batched_host_multi(&d, devices.data(), (int32_t)devices.size(), 0));
}

// ---- level-3 calls the reference builds on gemm: symm, hemm, trmm, syrk, herk ---------------------
// Same spellings as BatchLAS include/blas/functions/{symm,hemm,trmm,syrk,herk}.hh and the option
// structs of include/blas/options.hh:56-116; the expanded triangle / the full product lives in a lease
// from the queue's arena for the duration of the call.
enum class Side { Left, Right };
enum class Uplo { Upper, Lower };
enum class Diag { NonUnit, Unit };

template <typename T>
struct SymmOptions {
  T alpha = T(1);
  T beta = T(0);
  Side side = Side::Left;
  Uplo uplo = Uplo::Lower;
};
template <typename T>
struct HemmOptions {
  T alpha = T(1);
  T beta = T(0);
  Side side = Side::Left;
  Uplo uplo = Uplo::Lower;
};
template <typename T>
struct HerkOptions {
  float_t<T> alpha = float_t<T>(1);
  float_t<T> beta = float_t<T>(0);
  Uplo uplo = Uplo::Lower;
  Transpose trans = Transpose::NoTrans;
};
template <typename T>
struct SyrkOptions {
  T alpha = T(1);
  T beta = T(0);
  Uplo uplo = Uplo::Lower;
  Transpose trans = Transpose::NoTrans;
};
template <typename T>
struct TrmmOptions {
  T alpha = T(1);
  Side side = Side::Left;
  Uplo uplo = Uplo::Lower;
  Transpose trans = Transpose::NoTrans;
  Diag diag = Diag::NonUnit;
};

namespace detail {
template <typename T>
inline void set_scalar(double (&dst)[2], T v) {
  if constexpr (std::is_floating_point_v<T>) {
    dst[0] = v; dst[1] = 0.0;
  } else {
    dst[0] = v.real(); dst[1] = v.imag();
  }
}
template <typename T>
inline blb200_gemm_desc level3_desc(const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>* B,
                                    const MatrixView<T, MatrixFormat::Dense>& C) {
  blb200_gemm_desc d{};
  d.a = A.data_ptr(); d.lda = A.ld(); d.stride_a = A.stride();
  if (B) { d.b = B->data_ptr(); d.ldb = B->ld(); d.stride_b = B->stride(); } else { d.ldb = 1; }
  d.c = C.data_ptr(); d.ldc = C.ld(); d.stride_c = C.stride();
  d.batch = A.batch_size();
  d.dtype = dtype_code<T>();
  return d;
}
template <typename T>
inline Event symm_like(Queue& ctx, const char* name, bool hermitian, const MatrixView<T, MatrixFormat::Dense>& A,
                       const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C, T alpha,
                       T beta, Side side, Uplo uplo) {
  const std::string nm(name);
  if (A.rows() != A.cols()) throw std::runtime_error(nm + ": A must be square");
  if (A.batch_size() != B.batch_size() || A.batch_size() != C.batch_size())
    throw std::runtime_error(nm + ": batch size mismatch");
  const int m = C.rows(), n = C.cols(), k = side == Side::Left ? m : n;
  if (A.rows() != k || B.rows() != m || B.cols() != n) throw std::runtime_error(nm + ": incompatible matrix dimensions");
  blb200_gemm_desc d = level3_desc<T>(A, &B, C);
  d.m = m; d.n = n; d.k = k;
  set_scalar(d.alpha, alpha);
  set_scalar(d.beta, beta);
  ctx.make_current();
  WorkspaceLease ws = ctx.workspace(std::max<size_t>(blb200_level3_workspace_bytes(d.dtype, k, d.batch), 16));
  status_check(blb200_symm(&d, (int)side, (int)uplo, hermitian ? 1 : 0, ws.data(), ws.size(), ctx.native_stream()));
  return ctx.create_event_after_external_work();
}
template <typename T>
inline Event syrk_like(Queue& ctx, const char* name, bool hermitian, const MatrixView<T, MatrixFormat::Dense>& A,
                       const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Uplo uplo, Transpose transA) {
  const std::string nm(name);
  if (C.rows() != C.cols()) throw std::runtime_error(nm + ": C must be square");
  if (A.batch_size() != C.batch_size()) throw std::runtime_error(nm + ": batch size mismatch");
  const int n = C.rows();
  const int k = transA == Transpose::NoTrans ? A.cols() : A.rows();
  const int expected_n = transA == Transpose::NoTrans ? A.rows() : A.cols();
  if (expected_n != n || k <= 0) throw std::runtime_error(nm + ": incompatible matrix dimensions");
  blb200_gemm_desc d = level3_desc<T>(A, nullptr, C);
  d.m = n; d.n = n; d.k = k;
  d.op_a = (int)transA;
  set_scalar(d.alpha, alpha);
  set_scalar(d.beta, beta);
  ctx.make_current();
  WorkspaceLease ws = ctx.workspace(std::max<size_t>(blb200_level3_workspace_bytes(d.dtype, n, d.batch), 16));
  status_check(blb200_syrk(&d, (int)uplo, hermitian ? 1 : 0, ws.data(), ws.size(), ctx.native_stream()));
  return ctx.create_event_after_external_work();
}
}  // namespace detail

template <Backend Back, typename T>
inline Event symm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Side side, Uplo uplo) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  return detail::symm_like<T>(ctx, "SYMM", false, A, B, C, alpha, beta, side, uplo);
}
template <typename T>
inline Event symm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, const SymmOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return symm<Bk.value, T>(ctx, A, B, C, o.alpha, o.beta, o.side, o.uplo); });
}

// hemm exists for complex T only, as in the reference (ComplexScalar, include/blas/functions/hemm.hh).
template <Backend Back, typename T>
inline Event hemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Side side, Uplo uplo) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  static_assert(!std::is_floating_point_v<T>, "hemm needs a complex scalar; use symm for real data");
  return detail::symm_like<T>(ctx, "HEMM", true, A, B, C, alpha, beta, side, uplo);
}
template <typename T>
inline Event hemm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, const HemmOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return hemm<Bk.value, T>(ctx, A, B, C, o.alpha, o.beta, o.side, o.uplo); });
}

template <Backend Back, typename T>
inline Event syrk(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& C,
                  T alpha, T beta, Uplo uplo, Transpose transA) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  return detail::syrk_like<T>(ctx, "SYRK", false, A, C, alpha, beta, uplo, transA);
}
template <typename T>
inline Event syrk(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& C,
                  const SyrkOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return syrk<Bk.value, T>(ctx, A, C, o.alpha, o.beta, o.uplo, o.trans); });
}

template <Backend Back, typename T>
inline Event herk(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& C,
                  float_t<T> alpha, float_t<T> beta, Uplo uplo, Transpose transA) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  static_assert(!std::is_floating_point_v<T>, "herk needs a complex scalar; use syrk for real data");
  return detail::syrk_like<T>(ctx, "HERK", true, A, C, T(alpha), T(beta), uplo, transA);
}
template <typename T>
inline Event herk(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& C,
                  const HerkOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return herk<Bk.value, T>(ctx, A, C, o.alpha, o.beta, o.uplo, o.trans); });
}

template <typename T>
struct Syr2kOptions {
  T alpha = T(1);
  T beta = T(0);
  Uplo uplo = Uplo::Lower;
  Transpose trans = Transpose::NoTrans;
};
template <typename T>
struct Her2kOptions {
  T alpha = T(1);
  float_t<T> beta = float_t<T>(0);
  Uplo uplo = Uplo::Lower;
  Transpose trans = Transpose::NoTrans;
};

namespace detail {
template <typename T>
inline Event syr2k_like(Queue& ctx, const char* name, bool hermitian, const MatrixView<T, MatrixFormat::Dense>& A,
                        const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C, T alpha,
                        T beta, Uplo uplo, Transpose transA) {
  const std::string nm(name);
  if (C.rows() != C.cols()) throw std::runtime_error(nm + ": C must be square");
  if (A.batch_size() != B.batch_size() || A.batch_size() != C.batch_size())
    throw std::runtime_error(nm + ": batch size mismatch");
  if (hermitian && transA == Transpose::Trans) throw std::runtime_error(nm + ": transA must be NoTrans or ConjTrans");
  const bool no_trans = transA == Transpose::NoTrans;
  const int n = C.rows(), k = no_trans ? A.cols() : A.rows(), expected_n = no_trans ? A.rows() : A.cols();
  const int b_n = no_trans ? B.rows() : B.cols(), b_k = no_trans ? B.cols() : B.rows();
  if (expected_n != n || b_n != n || b_k != k || k <= 0) throw std::runtime_error(nm + ": incompatible matrix dimensions");
  blb200_gemm_desc d = level3_desc<T>(A, &B, C);
  d.m = n; d.n = n; d.k = k;
  d.op_a = (int)transA;
  set_scalar(d.alpha, alpha);
  set_scalar(d.beta, beta);
  ctx.make_current();
  WorkspaceLease ws = ctx.workspace(std::max<size_t>(blb200_level3_workspace_bytes(d.dtype, n, d.batch), 16));
  status_check(blb200_syr2k(&d, (int)uplo, hermitian ? 1 : 0, ws.data(), ws.size(), ctx.native_stream()));
  return ctx.create_event_after_external_work();
}
}  // namespace detail

template <Backend Back, typename T>
inline Event syr2k(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                   const MatrixView<T, MatrixFormat::Dense>& C, T alpha, T beta, Uplo uplo, Transpose transA) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  return detail::syr2k_like<T>(ctx, "SYR2K", false, A, B, C, alpha, beta, uplo, transA);
}
template <typename T>
inline Event syr2k(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                   const MatrixView<T, MatrixFormat::Dense>& C, const Syr2kOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return syr2k<Bk.value, T>(ctx, A, B, C, o.alpha, o.beta, o.uplo, o.trans); });
}
// her2k: complex alpha, real beta (include/blas/functions/her2k.hh; src/backends/cublas.cc:609-666).
template <Backend Back, typename T>
inline Event her2k(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                   const MatrixView<T, MatrixFormat::Dense>& C, T alpha, float_t<T> beta, Uplo uplo, Transpose transA) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  static_assert(!std::is_floating_point_v<T>, "her2k needs a complex scalar; use syr2k for real data");
  return detail::syr2k_like<T>(ctx, "HER2K", true, A, B, C, alpha, T(beta), uplo, transA);
}
template <typename T>
inline Event her2k(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                   const MatrixView<T, MatrixFormat::Dense>& C, const Her2kOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return her2k<Bk.value, T>(ctx, A, B, C, o.alpha, o.beta, o.uplo, o.trans); });
}

// Out of place, as the reference's trmm: C <- alpha * op(tri(A)) * B or alpha * B * op(tri(A)).
template <Backend Back, typename T>
inline Event trmm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, T alpha, Side side, Uplo uplo, Transpose transA, Diag diag) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  if (A.rows() != A.cols()) throw std::runtime_error("TRMM: A must be square");
  if (A.batch_size() != B.batch_size() || A.batch_size() != C.batch_size())
    throw std::runtime_error("TRMM: batch size mismatch");
  const int m = B.rows(), n = B.cols(), k = side == Side::Left ? m : n;
  if (A.rows() != k || C.rows() != m || C.cols() != n) throw std::runtime_error("TRMM: incompatible matrix dimensions");
  blb200_gemm_desc d = detail::level3_desc<T>(A, &B, C);
  d.m = m; d.n = n; d.k = k;
  d.op_a = (int)transA;
  detail::set_scalar(d.alpha, alpha);
  ctx.make_current();
  WorkspaceLease ws = ctx.workspace(std::max<size_t>(blb200_level3_workspace_bytes(d.dtype, k, d.batch), 16));
  detail::status_check(blb200_trmm(&d, (int)side, (int)uplo, diag == Diag::Unit ? 1 : 0, ws.data(), ws.size(),
                                   ctx.native_stream()));
  return ctx.create_event_after_external_work();
}
template <typename T>
inline Event trmm(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                  const MatrixView<T, MatrixFormat::Dense>& C, const TrmmOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return trmm<Bk.value, T>(ctx, A, B, C, o.alpha, o.side, o.uplo, o.trans, o.diag); });
}

// ---- the calls either side of gemm: gemv and the linalg:: elementwise layer -------------------------
// VectorView: `batch` vectors of `size` elements, element i of item b at data[b*stride + i*inc]
// (BatchLAS include/blas/matrix.hh:1320-1380; same constructor defaults: stride = size*inc).
template <typename T>
class VectorView {
 public:
  VectorView() = default;
  VectorView(T* data, int size, int batch_size = 1, int inc = 1, int stride = 0)
      : data_(data), size_(size), inc_(inc), stride_(stride > 0 ? stride : size * inc), batch_size_(batch_size) {}
  T* data_ptr() const { return data_; }
  int size() const { return size_; }
  int inc() const { return inc_; }
  int stride() const { return stride_; }
  int batch_size() const { return batch_size_; }
  T& at(int i, int b = 0) const { return data_[(int64_t)b * stride_ + (int64_t)i * inc_]; }

 private:
  T* data_ = nullptr;
  int size_ = 0, inc_ = 1, stride_ = 0, batch_size_ = 1;
};

template <typename T>
struct GemvOptions {
  T alpha = T(1);
  T beta = T(0);
  Transpose transA = Transpose::NoTrans;
};

// gemv<Backend::CUDA, T> (replaces gemv_vendor, BatchLAS src/backends/cublas.cc:1092-1113).
template <Backend Back, typename T>
inline Event gemv(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const VectorView<T>& X, const VectorView<T>& Y,
                  T alpha, T beta, Transpose transA) {
  static_assert(Back == Backend::CUDA, "only the CUDA backend exists in this build");
  blb200_gemv_desc d{};
  d.a = A.data_ptr(); d.x = X.data_ptr(); d.y = Y.data_ptr();
  d.m = A.rows(); d.n = A.cols(); d.batch = A.batch_size();
  d.lda = A.ld(); d.stride_a = A.stride();
  d.incx = X.inc(); d.stride_x = X.stride();
  d.incy = Y.inc(); d.stride_y = Y.stride();
  detail::set_scalar(d.alpha, alpha);
  detail::set_scalar(d.beta, beta);
  d.dtype = detail::dtype_code<T>();
  d.op_a = (int)transA;
  const int xl = transA == Transpose::NoTrans ? d.n : d.m, yl = transA == Transpose::NoTrans ? d.m : d.n;
  if (X.size() != xl || Y.size() != yl || (d.batch > 1 && (X.batch_size() != d.batch || Y.batch_size() != d.batch)))
    throw std::runtime_error("GEMV: incompatible dimensions");
  ctx.make_current();
  detail::status_check(blb200_gemv_strided_batched(&d, ctx.native_stream()));
  return ctx.create_event_after_external_work();
}
template <typename T>
inline Event gemv(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const VectorView<T>& X, const VectorView<T>& Y,
                  const GemvOptions<std::type_identity_t<T>>& o = {}) {
  return with_backend(ctx, [&](auto Bk) { return gemv<Bk.value, T>(ctx, A, X, Y, o.alpha, o.beta, o.transA); });
}

namespace linalg {
enum class BinaryOp { Add, Subtract, Multiply, Divide };

namespace detail_ew {
template <typename T>
inline blb200_ewise_desc desc(const char* where, const MatrixView<T, MatrixFormat::Dense>& A,
                              const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C) {
  auto same = [](const auto& X, const auto& Y) {
    return X.rows() == Y.rows() && X.cols() == Y.cols() && X.batch_size() == Y.batch_size();
  };
  if (!same(A, B) || !same(A, C)) throw std::invalid_argument(std::string(where) + ": operands must have the same shape");
  blb200_ewise_desc d{};
  d.a = A.data_ptr(); d.b = B.data_ptr(); d.c = C.data_ptr();
  d.rows = A.rows(); d.cols = A.cols(); d.batch = A.batch_size();
  d.lda = A.ld(); d.ldb = B.ld(); d.ldc = C.ld();
  d.stride_a = A.stride(); d.stride_b = B.stride(); d.stride_c = C.stride();
  d.dtype = batchlas::detail::dtype_code<T>();
  return d;
}
}  // namespace detail_ew

// C = op(A, B) elementwise; C may alias A or B (src/extra/elementwise.cc:42-79).
template <typename T, BinaryOp Op>
inline Event elementwise_into(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A,
                              const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C) {
  blb200_ewise_desc d = detail_ew::desc<T>("linalg::elementwise_into", A, B, C);
  ctx.make_current();
  batchlas::detail::status_check(blb200_elementwise(&d, (int)Op, ctx.native_stream()));
  return ctx.get_event();
}
// C = alpha*A + beta*B (src/extra/elementwise.cc:81-112).
template <typename T>
inline Event axpby_into(Queue& ctx, T alpha, const MatrixView<T, MatrixFormat::Dense>& A, T beta,
                        const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C) {
  blb200_ewise_desc d = detail_ew::desc<T>("linalg::axpby_into", A, B, C);
  double al[2], be[2];
  batchlas::detail::set_scalar(al, alpha);
  batchlas::detail::set_scalar(be, beta);
  ctx.make_current();
  batchlas::detail::status_check(blb200_axpby(&d, al, be, ctx.native_stream()));
  return ctx.get_event();
}
template <typename T>
inline Event scale(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, T alpha) {
  return axpby_into<T>(ctx, alpha, A, T(0), A, A);
}
template <typename T>
inline Event add_into(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                      const MatrixView<T, MatrixFormat::Dense>& C) {
  return elementwise_into<T, BinaryOp::Add>(ctx, A, B, C);
}
template <typename T>
inline Event subtract_into(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A,
                           const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C) {
  return elementwise_into<T, BinaryOp::Subtract>(ctx, A, B, C);
}
template <typename T>
inline Event multiply_into(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A,
                           const MatrixView<T, MatrixFormat::Dense>& B, const MatrixView<T, MatrixFormat::Dense>& C) {
  return elementwise_into<T, BinaryOp::Multiply>(ctx, A, B, C);
}
template <typename T>
inline Event divide_into(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                         const MatrixView<T, MatrixFormat::Dense>& C) {
  return elementwise_into<T, BinaryOp::Divide>(ctx, A, B, C);
}
// alpha * op(A) * op(B) as a new matrix; beta is forced to zero so the fresh storage is never read
// (include/blas/linalg-ops.hh:168-184).
template <typename T>
inline Matrix<T> matmul(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                        const GemmOptions<std::type_identity_t<T>>& opts = {}) {
  const bool ta = opts.transA != Transpose::NoTrans, tb = opts.transB != Transpose::NoTrans;
  Matrix<T> C(ta ? A.cols() : A.rows(), tb ? B.rows() : B.cols(), A.batch_size());
  auto o = opts;
  o.beta = T(0);
  gemm(ctx, A, B, C.view(), o);
  return C;
}
}  // namespace linalg

}  // namespace batchlas

inline batchlas::WorkspaceLease Queue::workspace(size_t bytes) {
  make_current();
  blb200_lease l{};
  batchlas::detail::status_check(blb200_arena_acquire(arena_, bytes, &l));
  return batchlas::WorkspaceLease(arena_, l);
}
