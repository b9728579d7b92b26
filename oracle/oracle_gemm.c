/*
 * oracle_gemm.c — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the reference's host GEMM path, used only as the checker by tests/,
 * __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs.  Nothing in the
 * shipped library links, loads or calls this file.
 *
 * What it restates (paths inside the BatchLAS project):
 *   - src/backends/netlib_lapack.cc:108-171  gemm<Backend::NETLIB,T>: validate, then a serial
 *     loop over batch items calling column-major cblas_?gemm, with m==0||n==0 -> skip and
 *     k==0 -> C *= beta.
 *   - src/backends/gemm_variant.hh:19-44     gemm_batch_dimensions_compatible.
 *   - src/sycl/gemm_kernels.cc:366-384 + src/sycl/gemm/accessors.hh:20-32  the element rule
 *     sum_k op(A)(i,k) * op(B)(k,j) with op in {identity, transpose, conjugate transpose}.
 *
 * The arithmetic of the reference's host path lives in a third-party CBLAS that the reference
 * does not vendor and does not pin (found by CMake at configure time; OpenBLAS or distro
 * libblas).  Two providers are offered here:
 *   provider 0  built-in: the textbook column-major GEMM (j, l, i loop order: for each column
 *               of C, scale by beta, then accumulate alpha*B(l,j) times column l of op(A)),
 *               in the working precision T, no FMA contraction requested.
 *   provider 1  a CBLAS resolved at run time with dlopen (the OpenBLAS that ships inside
 *               SciPy: LP64 symbols scipy_cblas_{s,d,c,z}gemm), bound with hand-declared
 *               prototypes (102 = ColMajor, 111/112/113 = N/T/C).
 *
 * Pinning: the reference holds no golden-vector files for gemm; its known-answer tests
 * (identity products, k==0 scaling, matmul vs a naive triple loop, the configure-time
 * dgemm-vs-naive health check on sin/cos inputs) are replayed against this oracle by
 * tests/test_oracle.py, and an independent long-double accumulation (oracle_gemm_exact) is the
 * arbiter for the entrywise bound |dC| <= 4*K*eps*(|alpha|*|A|*|B| + |beta|*|C|).
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { DT_S = 0, DT_D = 1, DT_C = 2, DT_Z = 3 };
enum { OP_N = 0, OP_T = 1, OP_H = 2 };

static size_t elem_size(int dtype) {
  switch (dtype) {
    case DT_S: return 4;
    case DT_D: return 8;
    case DT_C: return 8;
    default: return 16;
  }
}

/* ---- validation: gemm_variant.hh:19-44 in strided form ---------------------------------- */
int oracle_gemm_validate(int m, int n, int k, int batch, int op_a, int op_b, int64_t lda,
                         int64_t ldb, int64_t ldc) {
  if (m < 0 || n < 0 || k < 0 || batch < 0) return 0;
  int64_t a_rows = (op_a == OP_N) ? m : k;
  int64_t b_rows = (op_b == OP_N) ? k : n;
  if (lda < (a_rows > 1 ? a_rows : 1)) return 0;
  if (ldb < (b_rows > 1 ? b_rows : 1)) return 0;
  if (ldc < (m > 1 ? m : 1)) return 0;
  return 1;
}

/* ---- provider 1: dlopen'd CBLAS ----------------------------------------------------------- */
typedef void (*sgemm_fn)(int, int, int, int, int, int, float, const float*, int, const float*, int,
                         float, float*, int);
typedef void (*dgemm_fn)(int, int, int, int, int, int, double, const double*, int, const double*,
                         int, double, double*, int);
typedef void (*cgemm_fn)(int, int, int, int, int, int, const void*, const void*, int, const void*,
                         int, const void*, void*, int);
typedef void (*set_threads_fn)(int);
typedef char* (*get_config_fn)(void);

static struct {
  void* handle;
  sgemm_fn s;
  dgemm_fn d;
  cgemm_fn c, z;
  set_threads_fn set_threads;
  get_config_fn get_config;
} g_blas;

/* Returns 1 when all four gemm symbols resolved. `prefix` is "scipy_" for SciPy's OpenBLAS,
 * "" for a system CBLAS. */
int oracle_load_cblas(const char* path, const char* prefix) {
  char name[128];
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return 0;
#define RESOLVE(field, type, sym)                       \
  do {                                                  \
    strcpy(name, prefix);                               \
    strcat(name, sym);                                  \
    g_blas.field = (type)dlsym(h, name);                \
  } while (0)
  RESOLVE(s, sgemm_fn, "cblas_sgemm");
  RESOLVE(d, dgemm_fn, "cblas_dgemm");
  RESOLVE(c, cgemm_fn, "cblas_cgemm");
  RESOLVE(z, cgemm_fn, "cblas_zgemm");
  RESOLVE(set_threads, set_threads_fn, "openblas_set_num_threads");
  RESOLVE(get_config, get_config_fn, "openblas_get_config");
#undef RESOLVE
  g_blas.handle = h;
  return g_blas.s && g_blas.d && g_blas.c && g_blas.z;
}

int oracle_cblas_loaded(void) { return g_blas.handle && g_blas.s && g_blas.d && g_blas.c && g_blas.z; }
void oracle_cblas_set_threads(int n) {
  if (g_blas.set_threads) g_blas.set_threads(n);
}
const char* oracle_cblas_config(void) { return g_blas.get_config ? g_blas.get_config() : ""; }

/* ---- provider 0: textbook column-major GEMM in the working precision --------------------- */
#define DEFINE_REAL_GEMM(NAME, T)                                                                  \
  static void NAME(int op_a, int op_b, int m, int n, int k, T alpha, const T* A, int64_t lda,      \
                   const T* B, int64_t ldb, T beta, T* C, int64_t ldc) {                           \
    for (int j = 0; j < n; ++j) {                                                                  \
      T* cj = C + (int64_t)j * ldc;                                                                \
      if (beta == (T)0) {                                                                          \
        for (int i = 0; i < m; ++i) cj[i] = (T)0;                                                  \
      } else if (beta != (T)1) {                                                                   \
        for (int i = 0; i < m; ++i) cj[i] = beta * cj[i];                                          \
      }                                                                                            \
      if (alpha == (T)0) continue;                                                                 \
      if (op_a == OP_N) {                                                                          \
        for (int l = 0; l < k; ++l) {                                                              \
          T bv = (op_b == OP_N) ? B[(int64_t)j * ldb + l] : B[(int64_t)l * ldb + j];               \
          T t = alpha * bv;                                                                        \
          const T* al = A + (int64_t)l * lda;                                                      \
          for (int i = 0; i < m; ++i) cj[i] += t * al[i];                                          \
        }                                                                                          \
      } else {                                                                                     \
        for (int i = 0; i < m; ++i) {                                                              \
          const T* ai = A + (int64_t)i * lda;                                                      \
          T acc = (T)0;                                                                            \
          for (int l = 0; l < k; ++l) {                                                            \
            T bv = (op_b == OP_N) ? B[(int64_t)j * ldb + l] : B[(int64_t)l * ldb + j];             \
            acc += ai[l] * bv;                                                                     \
          }                                                                                        \
          cj[i] += alpha * acc;                                                                    \
        }                                                                                          \
      }                                                                                            \
    }                                                                                              \
  }
DEFINE_REAL_GEMM(builtin_sgemm, float)
DEFINE_REAL_GEMM(builtin_dgemm, double)

#define DEFINE_CPLX_GEMM(NAME, T)                                                                  \
  static inline void NAME##_load(const T* M, int64_t ld, int op, int r, int c, T* re, T* im) {     \
    /* element (r,c) of op(M) */                                                                   \
    const T* p = (op == OP_N) ? M + 2 * ((int64_t)c * ld + r) : M + 2 * ((int64_t)r * ld + c);     \
    *re = p[0];                                                                                    \
    *im = (op == OP_H) ? -p[1] : p[1];                                                             \
  }                                                                                                \
  static void NAME(int op_a, int op_b, int m, int n, int k, const T* alpha, const T* A,            \
                   int64_t lda, const T* B, int64_t ldb, const T* beta, T* C, int64_t ldc) {       \
    for (int j = 0; j < n; ++j) {                                                                  \
      for (int i = 0; i < m; ++i) {                                                                \
        T sr = 0, si = 0;                                                                          \
        for (int l = 0; l < k; ++l) {                                                              \
          T ar, ai, br, bi;                                                                        \
          NAME##_load(A, lda, op_a, i, l, &ar, &ai);                                               \
          NAME##_load(B, ldb, op_b, l, j, &br, &bi);                                               \
          sr += ar * br - ai * bi;                                                                 \
          si += ar * bi + ai * br;                                                                 \
        }                                                                                          \
        T* c = C + 2 * ((int64_t)j * ldc + i);                                                     \
        T outr = alpha[0] * sr - alpha[1] * si;                                                    \
        T outi = alpha[0] * si + alpha[1] * sr;                                                    \
        if (beta[0] != (T)0 || beta[1] != (T)0) {                                                  \
          outr += beta[0] * c[0] - beta[1] * c[1];                                                 \
          outi += beta[0] * c[1] + beta[1] * c[0];                                                 \
        }                                                                                          \
        c[0] = outr;                                                                               \
        c[1] = outi;                                                                               \
      }                                                                                            \
    }                                                                                              \
  }
DEFINE_CPLX_GEMM(builtin_cgemm, float)
DEFINE_CPLX_GEMM(builtin_zgemm, double)

/* One ?gemm call, column-major, dispatching on dtype and provider. */
static void one_gemm(int provider, int dtype, int op_a, int op_b, int m, int n, int k,
                     const double* alpha, const void* A, int64_t lda, const void* B, int64_t ldb,
                     const double* beta, void* C, int64_t ldc) {
  const int CblasColMajor = 102;
  const int tr[3] = {111, 112, 113};
  if (dtype == DT_S) {
    if (provider == 1)
      g_blas.s(CblasColMajor, tr[op_a], tr[op_b], m, n, k, (float)alpha[0], (const float*)A,
               (int)lda, (const float*)B, (int)ldb, (float)beta[0], (float*)C, (int)ldc);
    else
      builtin_sgemm(op_a, op_b, m, n, k, (float)alpha[0], (const float*)A, lda, (const float*)B,
                    ldb, (float)beta[0], (float*)C, ldc);
  } else if (dtype == DT_D) {
    if (provider == 1)
      g_blas.d(CblasColMajor, tr[op_a], tr[op_b], m, n, k, alpha[0], (const double*)A, (int)lda,
               (const double*)B, (int)ldb, beta[0], (double*)C, (int)ldc);
    else
      builtin_dgemm(op_a, op_b, m, n, k, alpha[0], (const double*)A, lda, (const double*)B, ldb,
                    beta[0], (double*)C, ldc);
  } else if (dtype == DT_C) {
    float al[2] = {(float)alpha[0], (float)alpha[1]}, be[2] = {(float)beta[0], (float)beta[1]};
    if (provider == 1)
      g_blas.c(CblasColMajor, tr[op_a], tr[op_b], m, n, k, al, A, (int)lda, B, (int)ldb, be, C,
               (int)ldc);
    else
      builtin_cgemm(op_a, op_b, m, n, k, al, (const float*)A, lda, (const float*)B, ldb, be,
                    (float*)C, ldc);
  } else {
    if (provider == 1)
      g_blas.z(CblasColMajor, tr[op_a], tr[op_b], m, n, k, alpha, A, (int)lda, B, (int)ldb, beta,
               C, (int)ldc);
    else
      builtin_zgemm(op_a, op_b, m, n, k, alpha, (const double*)A, lda, (const double*)B, ldb, beta,
                    (double*)C, ldc);
  }
}

/* C_i *= beta over the m x n window (netlib_lapack.cc:151-157). */
static void scale_item(int dtype, int m, int n, const double* beta, void* C, int64_t ldc) {
  for (int col = 0; col < n; ++col)
    for (int row = 0; row < m; ++row) {
      int64_t idx = (int64_t)col * ldc + row;
      if (dtype == DT_S) {
        ((float*)C)[idx] *= (float)beta[0];
      } else if (dtype == DT_D) {
        ((double*)C)[idx] *= beta[0];
      } else if (dtype == DT_C) {
        float* c = (float*)C + 2 * idx;
        float br = (float)beta[0], bi = (float)beta[1];
        float r = c[0] * br - c[1] * bi, i = c[0] * bi + c[1] * br;
        c[0] = r;
        c[1] = i;
      } else {
        double* c = (double*)C + 2 * idx;
        double r = c[0] * beta[0] - c[1] * beta[1], i = c[0] * beta[1] + c[1] * beta[0];
        c[0] = r;
        c[1] = i;
      }
    }
}

typedef struct {
  int provider, dtype, op_a, op_b, m, n, k;
  const double *alpha, *beta;
  const char *A, *B;
  char* C;
  int64_t lda, ldb, ldc, sa, sb, sc;
  int b0, b1;
} batch_job;

static void run_items(const batch_job* j) {
  size_t es = elem_size(j->dtype);
  for (int i = j->b0; i < j->b1; ++i) {
    const void* Ai = j->A + (size_t)i * j->sa * es;
    const void* Bi = j->B + (size_t)i * j->sb * es;
    void* Ci = j->C + (size_t)i * j->sc * es;
    if (j->m == 0 || j->n == 0) continue;
    if (j->k == 0) {
      scale_item(j->dtype, j->m, j->n, j->beta, Ci, j->ldc);
      continue;
    }
    one_gemm(j->provider, j->dtype, j->op_a, j->op_b, j->m, j->n, j->k, j->alpha, Ai, j->lda, Bi,
             j->ldb, j->beta, Ci, j->ldc);
  }
}

static void* run_items_thread(void* arg) {
  run_items((const batch_job*)arg);
  return NULL;
}

/*
 * The reference host path (netlib_lapack.cc:108-171).  threads <= 1 is the path exactly as the
 * reference runs it: a serial loop over batch items on the calling thread (any threading is
 * whatever the BLAS does internally).  threads > 1 splits the batch into contiguous ranges,
 * one pthread each — the batch-parallel variant reported beside it as the fairer multi-core
 * figure; for provider 1 the caller should pin the BLAS to one thread first.
 * Returns 0, or -2 for incompatible dimensions (the reference throws
 * "GEMM: incompatible matrix dimensions").
 */
int oracle_gemm_netlib(int provider, int dtype, int op_a, int op_b, int m, int n, int k, int batch,
                       const double* alpha, const void* A, int64_t lda, int64_t stride_a,
                       const void* B, int64_t ldb, int64_t stride_b, const double* beta, void* C,
                       int64_t ldc, int64_t stride_c, int threads) {
  if (!oracle_gemm_validate(m, n, k, batch, op_a, op_b, lda, ldb, ldc)) return -2;
  if (provider == 1 && !oracle_cblas_loaded()) return -4;
  batch_job base = {provider, dtype, op_a,     op_b,     m,   n,   k,   alpha,    beta,
                    A,        B,     (char*)C, lda,      ldb, ldc, stride_a, stride_b, stride_c,
                    0,        batch};
  if (threads <= 1 || batch < 2) {
    run_items(&base);
    return 0;
  }
  if (threads > batch) threads = batch;
  pthread_t* tid = (pthread_t*)malloc(sizeof(pthread_t) * threads);
  batch_job* jobs = (batch_job*)malloc(sizeof(batch_job) * threads);
  for (int t = 0; t < threads; ++t) {
    jobs[t] = base;
    jobs[t].b0 = (int)((int64_t)batch * t / threads);
    jobs[t].b1 = (int)((int64_t)batch * (t + 1) / threads);
    pthread_create(&tid[t], NULL, run_items_thread, &jobs[t]);
  }
  for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
  free(tid);
  free(jobs);
  return 0;
}

/* ---- arbiter: long-double accumulation of S = op(A)*op(B) and P = |op(A)|*|op(B)| --------- */
static inline void load_any(int dtype, const void* M, int64_t ld, int op, int r, int c,
                            long double* re, long double* im) {
  int64_t idx = (op == OP_N) ? (int64_t)c * ld + r : (int64_t)r * ld + c;
  switch (dtype) {
    case DT_S: *re = ((const float*)M)[idx]; *im = 0; break;
    case DT_D: *re = ((const double*)M)[idx]; *im = 0; break;
    case DT_C: *re = ((const float*)M)[2 * idx]; *im = ((const float*)M)[2 * idx + 1]; break;
    default: *re = ((const double*)M)[2 * idx]; *im = ((const double*)M)[2 * idx + 1]; break;
  }
  if (op == OP_H) *im = -*im;
}

/*
 * For one batch item writes, per C entry (column-major, ld = m):
 *   expect_re/expect_im = alpha*S + beta*C0 in long double, rounded to double
 *   bound               = |alpha| * (|A|*|B|) + |beta| * |C0|       (complex moduli)
 * C0 is read only when beta != 0.
 */
void oracle_gemm_exact_item(int dtype, int op_a, int op_b, int m, int n, int k, const double* alpha,
                            const void* A, int64_t lda, const void* B, int64_t ldb,
                            const double* beta, const void* C0, int64_t ldc, double* expect_re,
                            double* expect_im, double* bound) {
  int is_cplx = (dtype >= DT_C);
  long double al_r = alpha[0], al_i = is_cplx ? alpha[1] : 0;
  long double be_r = beta[0], be_i = is_cplx ? beta[1] : 0;
  if (dtype == DT_S || dtype == DT_C) { /* scalars are rounded to T by the launcher */
    al_r = (float)alpha[0]; al_i = is_cplx ? (float)alpha[1] : 0;
    be_r = (float)beta[0]; be_i = is_cplx ? (float)beta[1] : 0;
  }
  long double abs_al = hypotl(al_r, al_i), abs_be = hypotl(be_r, be_i);
  int beta_zero = (be_r == 0 && be_i == 0);
  for (int j = 0; j < n; ++j)
    for (int i = 0; i < m; ++i) {
      long double sr = 0, si = 0, p = 0;
      for (int l = 0; l < k; ++l) {
        long double ar, ai, br, bi;
        load_any(dtype, A, lda, op_a, i, l, &ar, &ai);
        load_any(dtype, B, ldb, op_b, l, j, &br, &bi);
        sr += ar * br - ai * bi;
        si += ar * bi + ai * br;
        p += hypotl(ar, ai) * hypotl(br, bi);
      }
      long double er = al_r * sr - al_i * si, ei = al_r * si + al_i * sr;
      long double bd = abs_al * p;
      if (!beta_zero) {
        long double cr, ci;
        load_any(dtype, C0, ldc, OP_N, i, j, &cr, &ci);
        er += be_r * cr - be_i * ci;
        ei += be_r * ci + be_i * cr;
        bd += abs_be * hypotl(cr, ci);
      }
      int64_t o = (int64_t)j * m + i;
      expect_re[o] = (double)er;
      expect_im[o] = (double)ei;
      bound[o] = (double)bd;
    }
}

/*
 * Entrywise acceptance rule for one item: |got - expect| <= 4*K*eps_T*bound (+ a subnormal
 * floor).  Returns the number of violating entries and writes the largest ratio
 * |got-expect| / (4*K*eps*bound) to *worst (0 when every bound is 0 and got == expect).
 */
int64_t oracle_check_item(int dtype, int m, int n, int k, const void* got, int64_t ldc,
                          const double* expect_re, const double* expect_im, const double* bound,
                          double* worst) {
  double eps = (dtype == DT_S || dtype == DT_C) ? 5.9604644775390625e-08 * 2 /* 2^-23 */
                                                : 2.220446049250313e-16;
  double tiny = (dtype == DT_S || dtype == DT_C) ? 1e-37 : 1e-300;
  int kk = k > 1 ? k : 1;
  int64_t bad = 0;
  double w = 0;
  for (int j = 0; j < n; ++j)
    for (int i = 0; i < m; ++i) {
      long double gr, gi;
      load_any(dtype, got, ldc, OP_N, i, j, &gr, &gi);
      int64_t o = (int64_t)j * m + i;
      double err = (double)hypotl(gr - expect_re[o], gi - expect_im[o]);
      double lim = 4.0 * kk * eps * bound[o] + tiny;
      double ratio = err / lim;
      if (!(ratio <= 1.0)) ++bad; /* also catches NaN */
      if (ratio > w || ratio != ratio) w = (ratio != ratio) ? INFINITY : ratio;
    }
  *worst = w;
  return bad;
}
