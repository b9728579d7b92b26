// C++ parity tests through the mirrored BatchLAS API (include/batchlas_b200.hh): the test bodies
// follow the reference's own (BatchLAS tests/gemm_tests.cc, backend_dispatch_tests.cc,
// options_api_tests.cc, mempool_tests.cc) with a naive host triple loop as the second
// implementation, since there is no vendor backend to compare against here.
// Build: g++ -std=c++20 -I include -I $CUDA/include tests/cpp/gemm_api_tests.cc -L batchlas_b200
//        -lbatchlas_b200 -L $CUDA/lib64 -lcudart.   `--compile-only-check` exits before touching a GPU.
#include <batchlas_b200.hh>

#include <cmath>
#include <complex>
#include <cstdio>
#include <cstring>
#include <functional>
#include <iostream>

using namespace batchlas;

static int g_failed = 0, g_run = 0;
#define CHECK(cond)                                                                   \
  do {                                                                                \
    if (!(cond)) {                                                                    \
      std::printf("  CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond);           \
      ++g_failed;                                                                     \
      return;                                                                         \
    }                                                                                 \
  } while (0)

template <typename T>
constexpr double tolerance() {  // BatchLAS tests/test_utils.hh:230-240
  using R = batchlas::float_t<T>;
  double t = std::is_same_v<R, float> ? 1e-5 : 1e-10;
  return std::is_same_v<T, R> ? t : 2 * t;
}

template <typename T>
T op_elem(const Matrix<T>& M, Transpose t, int r, int c, int b) {
  if (t == Transpose::NoTrans) return M(r, c, b);
  T v = M(c, r, b);
  if constexpr (!std::is_floating_point_v<T>) return t == Transpose::ConjTrans ? std::conj(v) : v;
  else return v;
}

// C_ref = alpha*op(A)*op(B) + beta*C0, accumulated in the widest type available.
template <typename T>
double max_abs_diff(const Matrix<T>& A, const Matrix<T>& B, const Matrix<T>& C0, const Matrix<T>& C, T alpha, T beta,
                    Transpose ta, Transpose tb, int m, int n, int k, int batch) {
  using W = std::conditional_t<std::is_floating_point_v<T>, long double, std::complex<long double>>;
  double worst = 0;
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < m; ++i) {
        W s = 0;
        for (int l = 0; l < k; ++l) s += W(op_elem(A, ta, i, l, b)) * W(op_elem(B, tb, l, j, b));
        W ref = W(alpha) * s;
        if (beta != T(0)) ref += W(beta) * W(C0(i, j, b));
        worst = std::max(worst, (double)std::abs(W(C(i, j, b)) - ref));
      }
  return worst;
}

template <typename T>
void GemmWithIdentityMatrix(Queue& ctx) {  // gemm_tests.cc:355-374
  const int rows = 10, cols = 10, ld = 10;
  auto A = Matrix<T>::Random(rows, cols);
  auto B = Matrix<T>::Identity(cols);
  auto C = Matrix<T>::Zeros(rows, cols);
  MatrixView<T, MatrixFormat::Dense> A_view(A.data_ptr(), rows, cols, ld);
  MatrixView<T, MatrixFormat::Dense> B_view(B.data_ptr(), cols, cols, ld);
  MatrixView<T, MatrixFormat::Dense> C_view(C.data_ptr(), rows, cols, ld);
  gemm(ctx, A_view, B_view, C_view, {.alpha = T(1.0), .beta = T(0.0)});
  ctx.wait();
  for (int j = 0; j < cols; ++j)
    for (int i = 0; i < rows; ++i) CHECK(std::abs(C(i, j) - A(i, j)) <= tolerance<T>());
}

template <typename T>
void BatchedGemm(Queue& ctx) {  // gemm_tests.cc:377-396
  const int n = 10, batch = 3;
  auto A = Matrix<T>::Random(n, n, false, batch);
  auto B = Matrix<T>::Identity(n, batch);
  auto C = Matrix<T>::Zeros(n, n, batch);
  gemm(ctx, A.view(), B.view(), C.view(), {.alpha = T(1.0), .beta = T(0.0)});
  ctx.wait();
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < n; ++i) CHECK(std::abs(C(i, j, b) - A(i, j, b)) <= tolerance<T>());
}

template <typename T>
void GeneralCase(Queue& ctx, int m, int n, int k, int batch, Transpose ta, Transpose tb, T alpha, T beta, double tol_mult) {
  auto A = ta == Transpose::NoTrans ? Matrix<T>::Random(m, k, false, batch) : Matrix<T>::Random(k, m, false, batch);
  auto B = tb == Transpose::NoTrans ? Matrix<T>::Random(k, n, false, batch, 43) : Matrix<T>::Random(n, k, false, batch, 43);
  auto C = Matrix<T>::Random(m, n, false, batch, 44);
  auto C0 = C.clone();
  gemm(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = beta, .transA = ta, .transB = tb});
  ctx.wait();
  double worst = max_abs_diff(A, B, C0, C, alpha, beta, ta, tb, m, n, k, batch);
  CHECK(worst <= tolerance<T>() * tol_mult);
}

template <typename T>
void ReferenceShapes(Queue& ctx) {
  GeneralCase<T>(ctx, 32, 32, 32, 4, Transpose::NoTrans, Transpose::NoTrans, T(1), T(0), 50);     // :674-739
  GeneralCase<T>(ctx, 128, 128, 128, 2, Transpose::NoTrans, Transpose::NoTrans, T(1), T(1), 100);
  GeneralCase<T>(ctx, 24, 20, 16, 3, Transpose::Trans, Transpose::Trans, T(1), T(0), 50);         // :1276-1351
  GeneralCase<T>(ctx, 96, 80, 64, 1, Transpose::Trans, Transpose::Trans, T(1), T(0), 100);
  GeneralCase<T>(ctx, 18, 14, 12, 2, Transpose::ConjTrans, Transpose::NoTrans, T(1), T(0), 50);   // :2035-2071
  GeneralCase<T>(ctx, 200, 130, 70, 3, Transpose::NoTrans, Transpose::NoTrans, T(2), T(-1), 100); // :1995-2033
}

template <typename T>
void DeducedBackendMatchesExplicit(Queue& ctx) {  // backend_dispatch_tests.cc:96-142
  const int n = 16, batch = 2;
  auto A = Matrix<T>::Random(n, n, false, batch);
  auto B = Matrix<T>::Random(n, n, false, batch, 7);
  auto C1 = Matrix<T>::Zeros(n, n, batch);
  auto C2 = Matrix<T>::Zeros(n, n, batch);
  gemm(ctx, A.view(), B.view(), C1.view(), T(1), T(0), Transpose::NoTrans, Transpose::NoTrans);
  gemm<Backend::CUDA>(ctx, A.view(), B.view(), C2.view(), T(1), T(0), Transpose::NoTrans, Transpose::NoTrans);
  ctx.wait();
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < n; ++i) CHECK(C1(i, j, b) == C2(i, j, b));
  // owning-Matrix overloads (:176-194) and defaulted ComputePrecision (:198-219)
  auto C3 = Matrix<T>::Zeros(n, n, batch);
  gemm(ctx, A, B, C3, T(1), T(0), Transpose::NoTrans, Transpose::NoTrans);
  ctx.wait();
  CHECK(C3(3, 5, 1) == C1(3, 5, 1));
}

template <typename T>
void HeterogeneousBatchedGemm(Queue& ctx) {  // gemm_tests.cc:398-586
  const int batch = 4, max_m = 40, max_n = 37, max_k = 33;
  const std::vector<int> ms = {40, 2, 0, 17}, ns = {37, 2, 4, 33}, ks = {33, 3, 3, 0};
  for (auto [ta, tb] : {std::pair{Transpose::NoTrans, Transpose::NoTrans}, std::pair{Transpose::Trans, Transpose::NoTrans},
                        std::pair{Transpose::NoTrans, Transpose::ConjTrans}}) {
    const bool an = ta == Transpose::NoTrans, bn = tb == Transpose::NoTrans;
    auto A = an ? Matrix<T>::Random(max_m, max_k, false, batch) : Matrix<T>::Random(max_k, max_m, false, batch);
    auto B = bn ? Matrix<T>::Random(max_k, max_n, false, batch, 9) : Matrix<T>::Random(max_n, max_k, false, batch, 9);
    auto C = Matrix<T>::Random(max_m, max_n, false, batch, 11);
    auto C0 = C.clone();
    A.set_active_dims(an ? ms : ks, an ? ks : ms);
    B.set_active_dims(bn ? ks : ns, bn ? ns : ks);
    C.set_active_dims(ms, ns);
    const T alpha = T(2), beta = T(0.5);
    gemm_heterogeneous(ctx, A.view(), B.view(), C.view(), alpha, beta, ta, tb);
    ctx.wait();
    // inside the active window: the per-item product (k == 0 -> C scaled by beta)
    using W = std::conditional_t<std::is_floating_point_v<T>, long double, std::complex<long double>>;
    for (int b = 0; b < batch; ++b)
      for (int j = 0; j < max_n; ++j)
        for (int i = 0; i < max_m; ++i) {
          if (i < ms[b] && j < ns[b]) {
            W s = 0;
            for (int l = 0; l < ks[b]; ++l) s += W(op_elem(A, ta, i, l, b)) * W(op_elem(B, tb, l, j, b));
            W ref = W(alpha) * s + W(beta) * W(C0(i, j, b));
            CHECK(std::abs(W(C(i, j, b)) - ref) <= tolerance<T>() * 100);
          } else {
            CHECK(C(i, j, b) == C0(i, j, b));  // outside the active window nothing is written
          }
        }
  }
  // mismatched per-item shapes are rejected like mismatched capacities
  auto A = Matrix<T>::Random(8, 8, false, 2), B = Matrix<T>::Random(8, 8, false, 2), C = Matrix<T>::Zeros(8, 8, 2);
  A.set_active_dims({8, 4}, {8, 5});
  B.set_active_dims({8, 6}, {8, 8});
  bool threw = false;
  try {
    gemm(ctx, A.view(), B.view(), C.view(), {});
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw);
}

template <typename T>
void LongKUsesSplitKFromTheArena(Queue& ctx) {
  // one small output, very long k: gemm() leases split-K scratch from the queue and gives it back
  const size_t before = ctx.workspace_capacity();
  GeneralCase<T>(ctx, 48, 40, 6000, 1, Transpose::Trans, Transpose::NoTrans, T(2), T(-1), 2000);
  CHECK(std::string(blb200_last_kernel_name()) == "splitk");
  CHECK(ctx.workspace_capacity() > before);
  const size_t cap = ctx.workspace_capacity();
  GeneralCase<T>(ctx, 48, 40, 6000, 1, Transpose::NoTrans, Transpose::NoTrans, T(1), T(0), 2000);
  CHECK(ctx.workspace_capacity() == cap);  // repeated calls do not grow the arena
  CHECK(ctx.trim_workspace());             // nothing is left leased
}

void OptionDefaultsAndErrors(Queue& ctx) {  // options_api_tests.cc:148-183
  GemmOptions<float> o;
  CHECK(o.alpha == 1.0f && o.beta == 0.0f && o.transA == Transpose::NoTrans && o.transB == Transpose::NoTrans &&
        o.precision == ComputePrecision::Default);
  auto A = Matrix<float>::Random(8, 8), B = Matrix<float>::Random(8, 8), C = Matrix<float>::Zeros(8, 8);
  auto C2 = Matrix<float>::Zeros(8, 8);
  gemm(ctx, A, B, C);  // all defaults
  gemm(ctx, A.view(), B.view(), C2.view(), {.alpha = 1.0f});
  ctx.wait();
  CHECK(C(2, 3) == C2(2, 3));
  auto Bad = Matrix<float>::Random(7, 8);
  bool threw = false;
  try {
    gemm(ctx, A.view(), Bad.view(), C.view(), {});
  } catch (const std::runtime_error& e) {
    threw = std::string(e.what()) == "GEMM: incompatible matrix dimensions";  // cublas.cc:119-121
  }
  CHECK(threw);
  threw = false;
  try {
    gemm(ctx, A.view(), B.view(), C.view(), {.precision = ComputePrecision::TF32});
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw);
  threw = false;
  try {
    ctx.set_backend(Backend::NETLIB);
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw && ctx.backend() == Backend::CUDA && Queue::backend_available(Backend::CUDA) &&
        !Queue::backend_available(Backend::ROCM));
}

void SlicedViews(Queue& ctx) {  // slices offset the base pointer: matrix.hh:855-869
  auto A = Matrix<double>::Random(40, 40, false, 2), B = Matrix<double>::Random(40, 40, false, 2, 5);
  auto C = Matrix<double>::Zeros(40, 40, 2);
  auto As = A.view()({3, 35}, {1, 20}), Bs = B.view()({0, 19}, {7, 30}), Cs = C.view()({5, 37}, {2, 25});
  CHECK(As.rows() == 32 && As.cols() == 19 && Bs.rows() == 19 && Bs.cols() == 23 && Cs.ld() == 40);
  gemm(ctx, As, Bs, Cs, {.alpha = 1.0});
  ctx.wait();
  double worst = 0;
  for (int b = 0; b < 2; ++b)
    for (int j = 0; j < 23; ++j)
      for (int i = 0; i < 32; ++i) {
        long double s = 0;
        for (int l = 0; l < 19; ++l) s += (long double)A(3 + i, 1 + l, b) * B(l, 7 + j, b);
        worst = std::max(worst, (double)std::abs(s - C(5 + i, 2 + j, b)));
      }
  CHECK(worst < 1e-12);
  CHECK(C(0, 0, 0) == 0.0 && C(39, 39, 1) == 0.0 && C(4, 2, 0) == 0.0 && C(37, 2, 0) == 0.0);  // outside the slice
}

// ---- level-3 calls through gemm: each checked against gemm on the explicitly expanded operand, the
// way the reference's tests do (symm_tests.cc:46-112, hemm_tests.cc, trmm_tests.cc:58-120,
// herk_tests.cc:337-420, syrk_tests.cc).
template <typename T>
T conj_if_complex(T v) {
  if constexpr (std::is_floating_point_v<T>) return v;
  else return std::conj(v);
}

template <typename T>
double max_diff(const Matrix<T>& X, const Matrix<T>& Y, int rows, int cols, int batch) {
  double w = 0;
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < cols; ++j)
      for (int i = 0; i < rows; ++i) w = std::max(w, (double)std::abs(X(i, j, b) - Y(i, j, b)));
  return w;
}

template <typename T>
void SymmMatchesSymmetrizedGemm(Queue& ctx) {
  const int n = 96, m = 64, batch = 3;
  const T alpha = T(1.25), beta = T(-0.5);
  const double tol = tolerance<T>() * 12 * n;
  for (bool herm : {false, true}) {
    if (herm && std::is_floating_point_v<T>) continue;
    for (auto side : {Side::Left, Side::Right})
      for (auto uplo : {Uplo::Lower, Uplo::Upper}) {
        const int rows = side == Side::Left ? n : m, cols = side == Side::Left ? m : n;
        auto A = Matrix<T>::Random(n, n, false, batch);
        auto B = Matrix<T>::Random(rows, cols, false, batch, 43);
        auto C = Matrix<T>::Random(rows, cols, false, batch, 44);
        auto C_ref = C.clone();
        auto A_ref = A.clone();
        ctx.wait();
        for (int b = 0; b < batch; ++b)
          for (int j = 0; j < n; ++j)
            for (int i = 0; i < n; ++i) {
              const bool stored = uplo == Uplo::Lower ? i >= j : i <= j;
              T v = stored ? A(i, j, b) : (herm ? conj_if_complex(A(j, i, b)) : A(j, i, b));
              if constexpr (!std::is_floating_point_v<T>) {
                if (herm && i == j) v = T(v.real(), 0);
              }
              A_ref(i, j, b) = v;
            }
        if constexpr (!std::is_floating_point_v<T>) {
          if (herm) hemm(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = beta, .side = side, .uplo = uplo});
          else symm(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = beta, .side = side, .uplo = uplo});
        } else {
          symm(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = beta, .side = side, .uplo = uplo});
        }
        if (side == Side::Left) gemm(ctx, A_ref.view(), B.view(), C_ref.view(), {.alpha = alpha, .beta = beta});
        else gemm(ctx, B.view(), A_ref.view(), C_ref.view(), {.alpha = alpha, .beta = beta});
        ctx.wait();
        CHECK(max_diff(C, C_ref, rows, cols, batch) <= tol);
      }
  }
}

template <typename T>
void TrmmAllCombinations(Queue& ctx) {
  const int n = 64, batch = 4;
  const double tol = tolerance<T>() * 12 * n;
  for (auto trans : {Transpose::NoTrans, Transpose::Trans, Transpose::ConjTrans})
    for (auto side : {Side::Right, Side::Left})
      for (auto uplo : {Uplo::Lower, Uplo::Upper})
        for (auto diag : {Diag::NonUnit, Diag::Unit}) {
          auto A = Matrix<T>::Random(n, n, false, batch);
          auto B = Matrix<T>::Random(n, n, false, batch, 43);
          auto C = Matrix<T>::Zeros(n, n, batch);
          auto C_ref = Matrix<T>::Zeros(n, n, batch);
          auto A_tri = A.clone();
          ctx.wait();
          for (int b = 0; b < batch; ++b)
            for (int j = 0; j < n; ++j)
              for (int i = 0; i < n; ++i) {
                const bool stored = uplo == Uplo::Lower ? i >= j : i <= j;
                A_tri(i, j, b) = (i == j && diag == Diag::Unit) ? T(1) : (stored ? A(i, j, b) : T(0));
              }
          trmm(ctx, A.view(), B.view(), C.view(), {.alpha = T(0.9), .side = side, .uplo = uplo, .trans = trans, .diag = diag});
          if (side == Side::Left) gemm(ctx, A_tri.view(), B.view(), C_ref.view(), {.alpha = T(0.9), .transA = trans});
          else gemm(ctx, B.view(), A_tri.view(), C_ref.view(), {.alpha = T(0.9), .transB = trans});
          ctx.wait();
          CHECK(max_diff(C, C_ref, n, n, batch) <= tol);
        }
}

template <typename T>
void SyrkHerkMatchGemm(Queue& ctx) {
  using R = batchlas::float_t<T>;
  const int n = 65, k = 40, batch = 3;
  const double tol = tolerance<T>() * 12 * k;
  constexpr bool cplx = !std::is_floating_point_v<T>;
  for (bool herm : {false, true}) {
    if (herm && !cplx) continue;
    const Transpose other = herm ? Transpose::ConjTrans : Transpose::Trans;
    for (auto trans : {Transpose::NoTrans, other})
      for (auto uplo : {Uplo::Lower, Uplo::Upper}) {
        auto A = trans == Transpose::NoTrans ? Matrix<T>::Random(n, k, false, batch) : Matrix<T>::Random(k, n, false, batch);
        auto C = Matrix<T>::Random(n, n, false, batch, 44);
        ctx.wait();
        if constexpr (cplx) {
          if (herm)  // BLAS does not reference the imaginary part of a Hermitian diagonal
            for (int b = 0; b < batch; ++b)
              for (int d = 0; d < n; ++d) C(d, d, b) = T(C(d, d, b).real(), 0);
        }
        auto C0 = C.clone();
        auto C_ref = C.clone();
        if constexpr (cplx) {
          if (herm) herk(ctx, A.view(), C.view(), {.alpha = R(0.9), .beta = R(-0.35), .uplo = uplo, .trans = trans});
          else syrk(ctx, A.view(), C.view(), {.alpha = T(0.9), .beta = T(-0.35), .uplo = uplo, .trans = trans});
        } else {
          syrk(ctx, A.view(), C.view(), {.alpha = T(0.9), .beta = T(-0.35), .uplo = uplo, .trans = trans});
        }
        gemm(ctx, A.view(), A.view(), C_ref.view(),
             {.alpha = T(0.9), .beta = T(-0.35), .transA = trans, .transB = trans == Transpose::NoTrans ? other : Transpose::NoTrans});
        ctx.wait();
        for (int b = 0; b < batch; ++b)
          for (int j = 0; j < n; ++j)
            for (int i = 0; i < n; ++i) {
              const bool referenced = uplo == Uplo::Lower ? i >= j : i <= j;
              if (!referenced) {
                CHECK(C(i, j, b) == C0(i, j, b));  // the other triangle is neither read nor written
              } else {
                CHECK(std::abs(C(i, j, b) - C_ref(i, j, b)) <= tol);
                if constexpr (cplx) {
                  if (herm && i == j) CHECK(C(i, j, b).imag() == R(0));
                }
              }
            }
      }
  }
}

template <typename T>
void Syr2kHer2kMatchTwoGemms(Queue& ctx) {  // her2k_tests.cc / syr2k_tests.cc: against gemm + gemm
  using R = batchlas::float_t<T>;
  const int n = 48, k = 20, batch = 3;
  const double tol = tolerance<T>() * 24 * k;
  constexpr bool cplx = !std::is_floating_point_v<T>;
  for (bool herm : {false, true}) {
    if (herm && !cplx) continue;
    const Transpose other = herm ? Transpose::ConjTrans : Transpose::Trans;
    for (auto trans : {Transpose::NoTrans, other})
      for (auto uplo : {Uplo::Lower, Uplo::Upper}) {
        const bool nt = trans == Transpose::NoTrans;
        auto A = nt ? Matrix<T>::Random(n, k, false, batch) : Matrix<T>::Random(k, n, false, batch);
        auto B = nt ? Matrix<T>::Random(n, k, false, batch, 43) : Matrix<T>::Random(k, n, false, batch, 43);
        auto C = Matrix<T>::Random(n, n, false, batch, 44);
        ctx.wait();
        if constexpr (cplx) {
          if (herm)
            for (int b = 0; b < batch; ++b)
              for (int d = 0; d < n; ++d) C(d, d, b) = T(C(d, d, b).real(), 0);
        }
        auto C0 = C.clone();
        auto C_ref = C.clone();
        T alpha = T(0.9), alpha2 = alpha;
        if constexpr (cplx) {
          alpha = T(0.9, -0.4);
          alpha2 = herm ? std::conj(alpha) : alpha;
        }
        if constexpr (cplx) {
          if (herm) her2k(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = R(-0.35), .uplo = uplo, .trans = trans});
          else syr2k(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = T(-0.35), .uplo = uplo, .trans = trans});
        } else {
          syr2k(ctx, A.view(), B.view(), C.view(), {.alpha = alpha, .beta = T(-0.35), .uplo = uplo, .trans = trans});
        }
        const Transpose tb = nt ? other : Transpose::NoTrans;
        gemm(ctx, A.view(), B.view(), C_ref.view(), {.alpha = alpha, .beta = T(-0.35), .transA = trans, .transB = tb});
        gemm(ctx, B.view(), A.view(), C_ref.view(), {.alpha = alpha2, .beta = T(1), .transA = trans, .transB = tb});
        ctx.wait();
        for (int b = 0; b < batch; ++b)
          for (int j = 0; j < n; ++j)
            for (int i = 0; i < n; ++i) {
              const bool referenced = uplo == Uplo::Lower ? i >= j : i <= j;
              if (!referenced) {
                CHECK(C(i, j, b) == C0(i, j, b));
              } else if (herm && i == j) {
                if constexpr (cplx) {
                  CHECK(std::abs(C(i, j, b).real() - C_ref(i, j, b).real()) <= tol && C(i, j, b).imag() == R(0));
                }
              } else {
                CHECK(std::abs(C(i, j, b) - C_ref(i, j, b)) <= tol);
              }
            }
      }
  }
}

// gemv on views (gemv_tests.cc:120-285: single / batched, N and T, alpha and beta) against the
// triple loop of its fixture.
template <typename T>
void GemvMatrixView(Queue& ctx) {
  const int rows = 10, cols = 10, batch = 3;
  auto A = Matrix<T>::Random(rows, cols, false, batch);
  auto X = Matrix<T>::Random(rows, 1, false, batch, 43);  // managed storage for the vectors
  auto Y = Matrix<T>::Random(rows, 1, false, batch, 44);
  ctx.wait();
  for (auto trans : {Transpose::NoTrans, Transpose::Trans})
    for (auto ab : {std::pair<double, double>{1.0, 0.0}, {2.5, 0.0}, {1.5, 0.8}}) {
      const T alpha = T(ab.first), beta = T(ab.second);
      auto Y0 = Y.clone();
      ctx.wait();
      VectorView<T> x(X.data_ptr(), rows, batch), y(Y.data_ptr(), rows, batch);
      gemv(ctx, A.view(), x, y, {.alpha = alpha, .beta = beta, .transA = trans});
      ctx.wait();
      for (int b = 0; b < batch; ++b)
        for (int i = 0; i < rows; ++i) {
          using W = std::conditional_t<std::is_floating_point_v<T>, long double, std::complex<long double>>;
          W s = 0;
          for (int l = 0; l < cols; ++l) s += W(trans == Transpose::NoTrans ? A(i, l, b) : A(l, i, b)) * W(X(l, 0, b));
          W ref = W(alpha) * s + W(beta) * W(Y0(i, 0, b));
          CHECK(std::abs(W(Y(i, 0, b)) - ref) <= tolerance<T>() * 20);
        }
    }
}

// linalg layer (linalg_layer_tests.cc): *_into helpers, axpby, scale, matmul.
template <typename T>
void LinalgElementwiseLayer(Queue& ctx) {
  const int rows = 7, cols = 5, batch = 3;
  auto A = Matrix<T>::Random(rows, cols, false, batch);
  auto B = Matrix<T>::Random(rows, cols, false, batch, 43);
  auto C = Matrix<T>::Zeros(rows, cols, batch);
  ctx.wait();
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < cols; ++j)
      for (int i = 0; i < rows; ++i) B(i, j, b) += T(3);  // away from zero
  const double tol = tolerance<T>() * 10;
  auto check = [&](auto&& f) {
    ctx.wait();
    double w = 0;
    for (int b = 0; b < batch; ++b)
      for (int j = 0; j < cols; ++j)
        for (int i = 0; i < rows; ++i) w = std::max(w, (double)std::abs(C(i, j, b) - f(A(i, j, b), B(i, j, b))));
    return w <= tol;
  };
  linalg::add_into(ctx, A.view(), B.view(), C.view());
  CHECK(check([](T a, T b) { return a + b; }));
  linalg::subtract_into(ctx, A.view(), B.view(), C.view());
  CHECK(check([](T a, T b) { return a - b; }));
  linalg::multiply_into(ctx, A.view(), B.view(), C.view());
  CHECK(check([](T a, T b) { return a * b; }));
  linalg::divide_into(ctx, A.view(), B.view(), C.view());
  CHECK(check([](T a, T b) { return a / b; }));
  linalg::axpby_into(ctx, T(1.5), A.view(), T(-0.25), B.view(), C.view());
  CHECK(check([](T a, T b) { return T(1.5) * a + T(-0.25) * b; }));
  auto A0 = A.clone();
  linalg::scale(ctx, A.view(), T(2));
  ctx.wait();
  for (int i = 0; i < rows; ++i) CHECK(std::abs(A(i, 1, 2) - T(2) * A0(i, 1, 2)) <= tol);
  auto P = linalg::matmul(ctx, A0.view(), B.view(), {.transB = Transpose::Trans});
  auto P_ref = Matrix<T>::Zeros(rows, rows, batch);
  gemm(ctx, A0.view(), B.view(), P_ref.view(), {.transB = Transpose::Trans});
  ctx.wait();
  CHECK(P.rows() == rows && P.cols() == rows && max_diff(P, P_ref, rows, rows, batch) == 0.0);
  bool threw = false;
  try {
    linalg::add_into(ctx, A.view(), P.view(), C.view());
  } catch (const std::invalid_argument& e) {
    threw = std::strstr(e.what(), "linalg::elementwise_into: operands must have the same shape") != nullptr;
  }
  CHECK(threw);
}

template <typename T>
void Level3ShapeErrors(Queue& ctx) {
  auto A = Matrix<T>::Zeros(8, 8, 2);
  auto R = Matrix<T>::Zeros(8, 4, 2);
  auto expect = [&](auto&& call, const char* msg) {
    bool threw = false;
    try { call(); } catch (const std::runtime_error& e) { threw = std::strstr(e.what(), msg) != nullptr; }
    return threw;
  };
  CHECK(expect([&] { symm(ctx, R.view(), R.view(), R.view()); }, "SYMM: A must be square"));
  CHECK(expect([&] { symm(ctx, A.view(), R.view(), R.view(), {.side = Side::Right}); }, "SYMM: incompatible matrix dimensions"));
  CHECK(expect([&] { trmm(ctx, A.view(), R.view(), A.view()); }, "TRMM: incompatible matrix dimensions"));
  CHECK(expect([&] { syrk(ctx, R.view(), R.view()); }, "SYRK: C must be square"));
  CHECK(expect([&] { syrk(ctx, R.view(), A.view(), {.trans = Transpose::Trans}); }, "SYRK: incompatible matrix dimensions"));
}

void WorkspaceLeases(Queue& ctx) {  // mempool_tests.cc:829-1078
  {
    auto a = ctx.workspace(1000);
    CHECK(a.data() != nullptr && a.size() == 1000 && (reinterpret_cast<uintptr_t>(a.data()) % 256) == 0);
  }
  size_t cap = ctx.workspace_capacity();
  std::byte* first = nullptr;
  for (int i = 0; i < 20; ++i) {
    auto a = ctx.workspace(1000);
    if (!first) first = a.data();
    CHECK(a.data() == first);
  }
  CHECK(ctx.workspace_capacity() == cap);  // repeated calls do not grow the arena
  {
    auto outer = ctx.workspace(4096);
    auto inner = ctx.workspace(8 << 20);
    CHECK(inner.data() + inner.size() <= outer.data() || inner.data() >= outer.data() + outer.size());
    CHECK(!ctx.trim_workspace());  // refuses while leased
    outer.release();               // early, out of order: only marked
    auto third = ctx.workspace(4096);
    CHECK(third.data() != first);
  }
  auto ws = ctx.workspace(100);
  ws = ctx.workspace(200);  // reassignment defers reclaim, never aliases
  CHECK(ws.size() == 200);
  ws.release();
  CHECK(ctx.trim_workspace() && ctx.workspace_capacity() == 0);
}

// A reference-style entry point (Backend first, a defaulted trailing argument) and its
// queue-dispatched form generated by BATCHLAS_DISPATCH_ON_QUEUE, the way the reference declares its
// own forwarders (BatchLAS include/blas/queue-dispatch.hh:103-113).
namespace batchlas {
template <Backend Back, typename T>
Event scaled_product(Queue& ctx, const MatrixView<T, MatrixFormat::Dense>& A, const MatrixView<T, MatrixFormat::Dense>& B,
                     const MatrixView<T, MatrixFormat::Dense>& C, T alpha = T(1)) {
  return gemm<Back, T>(ctx, A, B, C, alpha, T(0), Transpose::NoTrans, Transpose::NoTrans);
}
BATCHLAS_DISPATCH_ON_QUEUE(scaled_product)
}  // namespace batchlas

template <typename T>
void DispatchOnQueueMacro(Queue& ctx) {
  const int n = 24, batch = 3;
  auto A = Matrix<T>::Random(n, n, false, batch, 7), B = Matrix<T>::Random(n, n, false, batch, 8);
  Matrix<T> C1(n, n, batch), C2(n, n, batch), C3(n, n, batch);
  scaled_product(ctx, A.view(), B.view(), C1.view()).wait();                       // default alpha applies
  scaled_product<Backend::CUDA>(ctx, A.view(), B.view(), C2.view(), T(1)).wait();  // explicit backend still resolves
  scaled_product(ctx, A.view(), B.view(), C3.view(), T(2)).wait();
  ctx.wait();
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < n; ++j)
      for (int i = 0; i < n; ++i) {
        CHECK(C1(i, j, b) == C2(i, j, b));
        CHECK(std::abs(C3(i, j, b) - T(2) * C1(i, j, b)) <= 4 * tolerance<T>() * (1 + std::abs(C1(i, j, b))));
      }
}

// One call over every GPU of the box with host-resident operands (one Queue per GPU).
template <typename T>
void MultiGpuHostGemm(Queue& ctx) {
  const int m = 40, n = 24, k = 56, batch = 37;
  auto A = Matrix<T>::Random(m, k, false, batch, 11), B = Matrix<T>::Random(k, n, false, batch, 12);
  auto C0 = Matrix<T>::Random(m, n, false, batch, 13);
  ctx.wait();
  // plain host copies of the operands
  std::vector<T> hA((size_t)m * k * batch), hB((size_t)k * n * batch), hC((size_t)m * n * batch);
  for (int b = 0; b < batch; ++b) {
    for (int j = 0; j < k; ++j) for (int i = 0; i < m; ++i) hA[((size_t)b * k + j) * m + i] = A(i, j, b);
    for (int j = 0; j < n; ++j) for (int i = 0; i < k; ++i) hB[((size_t)b * n + j) * k + i] = B(i, j, b);
    for (int j = 0; j < n; ++j) for (int i = 0; i < m; ++i) hC[((size_t)b * n + j) * m + i] = C0(i, j, b);
  }
  std::vector<Queue> queues;
  for (auto& dev : Device::get_devices(DeviceType::GPU)) queues.emplace_back(dev);
  const T alpha = T(1.5), beta = T(-0.5);
  gemm_host<T>(std::span<Queue>(queues), MatrixView<T>(hA.data(), m, k, m, (int64_t)m * k, batch),
               MatrixView<T>(hB.data(), k, n, k, (int64_t)k * n, batch), MatrixView<T>(hC.data(), m, n, m, (int64_t)m * n, batch),
               {.alpha = alpha, .beta = beta});
  Matrix<T> C(m, n, batch);
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < n; ++j) for (int i = 0; i < m; ++i) C(i, j, b) = hC[((size_t)b * n + j) * m + i];
  const double worst = max_abs_diff(A, B, C0, C, alpha, beta, Transpose::NoTrans, Transpose::NoTrans, m, n, k, batch);
  CHECK(worst <= tolerance<T>() * k * 4);
  ctx.make_current();
}

int main(int argc, char** argv) {
  if (argc > 1 && std::strcmp(argv[1], "--compile-only-check") == 0) {
    std::puts("compiled: overload set resolves");
    return 0;
  }
  Queue ctx(Device::default_device());
  std::printf("device: %s\n", ctx.device().get_name().c_str());
  auto run = [&](const char* name, std::function<void()> f) {
    int before = g_failed;
    ++g_run;
    try {
      f();
    } catch (const std::exception& e) {
      std::printf("  exception: %s\n", e.what());
      ++g_failed;
    }
    std::printf("[%s] %s\n", g_failed == before ? " OK " : "FAIL", name);
  };
#define FOR_TYPES(fn)                                                       \
  run(#fn "<float>", [&] { fn<float>(ctx); });                              \
  run(#fn "<double>", [&] { fn<double>(ctx); });                            \
  run(#fn "<complex<float>>", [&] { fn<std::complex<float>>(ctx); });       \
  run(#fn "<complex<double>>", [&] { fn<std::complex<double>>(ctx); });
  FOR_TYPES(GemmWithIdentityMatrix)
  FOR_TYPES(BatchedGemm)
  FOR_TYPES(ReferenceShapes)
  FOR_TYPES(DeducedBackendMatchesExplicit)
  FOR_TYPES(DispatchOnQueueMacro)
  FOR_TYPES(MultiGpuHostGemm)
  FOR_TYPES(HeterogeneousBatchedGemm)
  FOR_TYPES(LongKUsesSplitKFromTheArena)
  FOR_TYPES(SymmMatchesSymmetrizedGemm)
  FOR_TYPES(TrmmAllCombinations)
  FOR_TYPES(SyrkHerkMatchGemm)
  FOR_TYPES(Syr2kHer2kMatchTwoGemms)
  FOR_TYPES(Level3ShapeErrors)
  FOR_TYPES(GemvMatrixView)
  FOR_TYPES(LinalgElementwiseLayer)
  run("OptionDefaultsAndErrors", [&] { OptionDefaultsAndErrors(ctx); });
  run("SlicedViews", [&] { SlicedViews(ctx); });
  run("WorkspaceLeases", [&] { WorkspaceLeases(ctx); });
  std::printf("%d test groups, %d failed\n", g_run, g_failed);
  return g_failed ? 1 : 0;
}
