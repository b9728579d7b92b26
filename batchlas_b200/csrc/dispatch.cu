// C-ABI entry points of libbatchlas_b200.so: validation, shape/dtype dispatch, diagnostics.
// The device-pointer launcher allocates nothing and never synchronises.
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

namespace blb200 {

static thread_local const char* t_last_kernel = "";
static thread_local uint64_t t_launches = 0;

void note_launch(const char* kernel_name) {
  t_last_kernel = kernel_name;
  ++t_launches;
}

// ---- environment knobs (conventions of BatchLAS include/util/env.hh) -------------------------------
// BATCHLAS_GEMM_B200_KERNEL=<generic|small32|small64|small_ring|tiled|dmma|dmma_tma|sgemm128|sgemm_tma>  forces a kernel for calls
//   that leave kernel_hint at 0 (the role BATCHLAS_GEMM_SYCL_KERNEL plays for the reference's SYCL
//   family, src/sycl/gemm_kernels.cc:270-329); a problem the forced kernel cannot run is dispatched
//   normally.
// BATCHLAS_NVTX=1  wraps every gemm call in an NVTX range "blb200.gemm <dtype> m x n x k b<batch>" and
//   marks the kernel variant chosen inside it, for timelines taken with an external profiler.
// BATCHLAS_KERNEL_TRACE=1 [BATCHLAS_KERNEL_TRACE_PATH=file]  brackets every launch with CUDA events
//   and writes a Chrome trace at exit (the reference's kernel tracer, src/util/kernel-trace.hh:46-215).
static int env_forced_kernel() {
  static const int forced = [] {
    const char* v = getenv("BATCHLAS_GEMM_B200_KERNEL");
    if (!v || !*v) return (int)BLB200_K_AUTO;
    const struct { const char* name; int id; } names[] = {
        {"generic", BLB200_K_GENERIC}, {"small32", BLB200_K_SMALL32}, {"small64", BLB200_K_SMALL64},
        {"tiled", BLB200_K_TILED},     {"dmma", BLB200_K_DMMA},       {"sgemm128", BLB200_K_SGEMM128},
        {"small_ring", BLB200_K_SMALL_RING}, {"dmma_tma", BLB200_K_DMMA_TMA}, {"sgemm_tma", BLB200_K_SGEMM_TMA}};
    for (const auto& n : names)
      if (strcmp(v, n.name) == 0) return n.id;
    return (int)BLB200_K_AUTO;
  }();
  return forced;
}

namespace {
struct TraceRecord {
  std::string name;
  cudaEvent_t start, stop;
  int device;
  long long m, n, k, batch;
};
struct Tracer {
  bool enabled = false;
  std::string path;
  std::mutex mu;
  std::vector<TraceRecord> records;
  Tracer() {
    const char* v = getenv("BATCHLAS_KERNEL_TRACE");
    enabled = v && *v && strcmp(v, "0") != 0;
    const char* pth = getenv("BATCHLAS_KERNEL_TRACE_PATH");
    path = (pth && *pth) ? pth : "batchlas_b200_trace.json";
  }
  ~Tracer() { dump(); }
  void dump() {
    std::lock_guard<std::mutex> lock(mu);
    if (!enabled || records.empty()) return;
    FILE* f = fopen(path.c_str(), "w");
    if (!f) return;
    fprintf(f, "{\"traceEvents\":[\n");
    cudaEvent_t origin = records.front().start;
    bool first = true;
    for (auto& r : records) {
      cudaSetDevice(r.device);
      if (cudaEventSynchronize(r.stop) != cudaSuccess) continue;
      float t0 = 0.f, dur = 0.f;
      if (r.device == records.front().device) cudaEventElapsedTime(&t0, origin, r.start);
      cudaEventElapsedTime(&dur, r.start, r.stop);
      fprintf(f, "%s{\"name\":\"%s\",\"ph\":\"X\",\"pid\":%d,\"tid\":0,\"ts\":%.3f,\"dur\":%.3f,"
                 "\"args\":{\"m\":%lld,\"n\":%lld,\"k\":%lld,\"batch\":%lld}}",
              first ? "" : ",\n", r.name.c_str(), r.device, t0 * 1e3, dur * 1e3, r.m, r.n, r.k, r.batch);
      first = false;
      cudaEventDestroy(r.stop);
      if (r.start != origin) cudaEventDestroy(r.start);
    }
    fprintf(f, "\n]}\n");
    fclose(f);
    records.clear();
  }
};
Tracer& tracer() {
  static Tracer t;
  return t;
}
}  // namespace

const DeviceInfo& device_info() {
  static DeviceInfo infos[64];
  static std::once_flag flags[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::call_once(flags[dev], [dev] {
    DeviceInfo& d = infos[dev];
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    d.sm_count = v > 0 ? v : 148;
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    d.smem_optin = (size_t)v;
  });
  return infos[dev];
}

static int validate(const blb200_gemm_desc* d) {
  if (!d) return BLB200_E_NULL;
  if (d->dtype < BLB200_S || d->dtype > BLB200_Z) return BLB200_E_DTYPE;
  if (d->op_a < BLB200_N || d->op_a > BLB200_H || d->op_b < BLB200_N || d->op_b > BLB200_H)
    return BLB200_E_DTYPE;
  if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0) return BLB200_E_SHAPE;
  const int64_t a_rows = d->op_a == BLB200_N ? d->m : d->k;
  const int64_t b_rows = d->op_b == BLB200_N ? d->k : d->n;
  if (d->lda < (a_rows > 1 ? a_rows : 1)) return BLB200_E_SHAPE;
  if (d->ldb < (b_rows > 1 ? b_rows : 1)) return BLB200_E_SHAPE;
  if (d->ldc < (d->m > 1 ? d->m : 1)) return BLB200_E_SHAPE;
  if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0) return BLB200_E_SHAPE;
  if (d->kernel_hint < BLB200_K_AUTO || d->kernel_hint > BLB200_K_SGEMM_TMA) return BLB200_E_UNSUPPORTED;
  const bool has_work = d->m > 0 && d->n > 0 && d->batch > 0;
  if (has_work) {
    if (!d->c) return BLB200_E_NULL;
    if (d->k > 0 && (!d->a || !d->b)) return BLB200_E_NULL;
  }
  return BLB200_OK;
}

static GemmParams to_params(const blb200_gemm_desc* d) {
  GemmParams p;
  p.a = d->a;
  p.b = d->b;
  p.c = d->c;
  p.m = d->m;
  p.n = d->n;
  p.k = d->k;
  p.batch = d->batch;
  p.lda = d->lda;
  p.ldb = d->ldb;
  p.ldc = d->ldc;
  p.sa = d->stride_a;
  p.sb = d->stride_b;
  p.sc = d->stride_c;
  const bool cplx = d->dtype >= BLB200_C;
  p.alpha[0] = d->alpha[0];
  p.alpha[1] = cplx ? d->alpha[1] : 0.0;
  p.beta[0] = d->beta[0];
  p.beta[1] = cplx ? d->beta[1] : 0.0;
  p.op_a = d->op_a;
  p.op_b = d->op_b;
  p.splits = 1;
  p.kchunk = d->k;
  p.split_a = p.split_b = 0;
  if (!cplx) {  // conjugation is the identity on real data
    if (p.op_a == BLB200_H) p.op_a = BLB200_T;
    if (p.op_b == BLB200_H) p.op_b = BLB200_T;
  }
  return p;
}

GemmParams to_params_public(const blb200_gemm_desc* d) { return to_params(d); }

static int dispatch_untraced(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream);

// The cp.async tile kernels in order of preference for this problem; the generic kernel (or
// BLB200_E_UNSUPPORTED) when none of them takes it.
static int launch_tile_kernel(const GemmParams& p, int dtype, cudaStream_t stream, bool generic_fallback = true) {
  if (dmma_tma_supported(p, dtype)) return launch_dmma_tma(p, dtype, stream);
  if (dmma_supported(p, dtype)) return launch_dmma(p, dtype, stream);
  if (sgemm128_supported(p, dtype) && sgemm128_preferred(p)) {
    // the same 128 x 128 tile in two forms: from k = 256 on the TMA-fed one is the faster (256^3: 51.0
    // against 47.4 TFLOP/s, 1024^3: 56.6 against 51.6), below that its deeper ring does not fill (128^3: 37.9 against 42.7)
    if (p.k >= 256 && sgemm_tma_supported(p, dtype)) {
      const int rc = launch_sgemm_tma(p, dtype, stream);
      if (rc != BLB200_E_INTERNAL) return rc;  // a driver that refuses the tensor map: the cp.async form takes it
    }
    return launch_sgemm128(p, dtype, stream);
  }
  // float with A transposed and long k, on the TMA-fed 128 x 128 tile: A^T B^T as the transposed product (1024^3:
  // 57.1 against 39.9 TFLOP/s on the 64 x 64 tiles; 256^3: 52.1 against 38.4), A^T B by k-pairs (1024^3: 48.3 against 39.8)
  if (dtype == BLB200_S && p.op_a != BLB200_N && p.k >= 256 && sgemm128_preferred(p) && sgemm_tma_supported(p, dtype)) {
    const int rc = launch_sgemm_tma(p, dtype, stream);
    if (rc != BLB200_E_INTERNAL) return rc;
  }
  if (tiled_supported(p, dtype)) return launch_tiled(p, dtype, stream);
  return generic_fallback ? launch_generic(p, dtype, stream) : BLB200_E_UNSUPPORTED;
}

int dispatch(const blb200_gemm_desc* d, cudaStream_t stream) { return dispatch_structured(d, nullptr, stream); }

static bool nvtx_enabled() {
  static const bool on = [] {
    const char* v = getenv("BATCHLAS_NVTX");
    return v && *v && strcmp(v, "0") != 0;
  }();
  return on;
}

static int dispatch_traced(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream);

int dispatch_structured(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream) {
  if (!nvtx_enabled() || !d) return dispatch_traced(d, hints, stream);
  char label[96];
  snprintf(label, sizeof(label), "blb200.gemm %c %dx%dx%d b%d", "sdcz"[d->dtype & 3], d->m, d->n, d->k, d->batch);
  nvtxRangePushA(label);
  const int rc = dispatch_traced(d, hints, stream);
  snprintf(label, sizeof(label), "kernel=%s rc=%d", t_last_kernel, rc);
  nvtxMarkA(label);
  nvtxRangePop();
  return rc;
}

static int dispatch_traced(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream) {
  Tracer& tr = tracer();
  if (!tr.enabled) return dispatch_untraced(d, hints, stream);
  TraceRecord rec{};
  cudaGetDevice(&rec.device);
  if (cudaEventCreate(&rec.start) != cudaSuccess || cudaEventCreate(&rec.stop) != cudaSuccess)
    return dispatch_untraced(d, hints, stream);
  cudaEventRecord(rec.start, stream);
  const int rc = dispatch_untraced(d, hints, stream);
  cudaEventRecord(rec.stop, stream);
  if (d) {
    rec.m = d->m; rec.n = d->n; rec.k = d->k; rec.batch = d->batch;
  }
  rec.name = std::string("gemm.") + t_last_kernel;
  std::lock_guard<std::mutex> lock(tr.mu);
  tr.records.push_back(rec);
  return rc;
}

static int dispatch_untraced(const blb200_gemm_desc* d, const StructureHints* hints, cudaStream_t stream) {
  int rc = validate(d);
  if (rc != BLB200_OK) return rc;
  if (d->m == 0 || d->n == 0 || d->batch == 0) return BLB200_OK;
  if (hints && (hints->tri_a | hints->tri_b | hints->out_tri)) {
    // Only the cp.async tile kernels read the hints.  An operand hint may be dropped (the zeros are
    // stored); a triangular output may not, so without such a kernel the caller has to take
    // another route.
    GemmParams hp = to_params(d);
    hp.tri_a = hints->tri_a;
    hp.tri_b = hints->tri_b;
    hp.out_tri = hints->out_tri;
    hp.out_herm = hints->out_herm;
    const int rc_tile = launch_tile_kernel(hp, d->dtype, stream, /*generic_fallback=*/false);
    if (rc_tile != BLB200_E_UNSUPPORTED || hints->out_tri) return rc_tile;
  }
  const GemmParams p = to_params(d);
  if (d->kernel_hint == BLB200_K_AUTO && env_forced_kernel() != BLB200_K_AUTO) {
    const int dt = d->dtype;
    switch (env_forced_kernel()) {
      case BLB200_K_GENERIC: return launch_generic(p, dt, stream);
      case BLB200_K_SMALL32: if (small32_supported(p, dt)) return launch_small32(p, dt, stream); break;
      case BLB200_K_SMALL64: if (small64_supported(p, dt)) return launch_small64(p, dt, stream); break;
      case BLB200_K_TILED: if (tiled_supported(p, dt)) return launch_tiled(p, dt, stream); break;
      case BLB200_K_DMMA: if (dmma_supported(p, dt)) return launch_dmma(p, dt, stream); break;
      case BLB200_K_SGEMM128: if (sgemm128_supported(p, dt)) return launch_sgemm128(p, dt, stream); break;
      case BLB200_K_SMALL_RING: if (small_ring_supported(p, dt)) return launch_small_ring(p, dt, stream); break;
      case BLB200_K_DMMA_TMA: if (dmma_tma_supported(p, dt)) return launch_dmma_tma(p, dt, stream); break;
      case BLB200_K_SGEMM_TMA: if (sgemm_tma_supported(p, dt)) return launch_sgemm_tma(p, dt, stream); break;
      default: break;
    }
  }
  switch (d->kernel_hint) {
    case BLB200_K_GENERIC: return launch_generic(p, d->dtype, stream);
    case BLB200_K_SMALL32: return launch_small32(p, d->dtype, stream);
    case BLB200_K_SMALL64: return launch_small64(p, d->dtype, stream);
    case BLB200_K_TILED: return launch_tiled(p, d->dtype, stream);
    case BLB200_K_DMMA: return launch_dmma(p, d->dtype, stream);
    case BLB200_K_SGEMM128: return launch_sgemm128(p, d->dtype, stream);
    case BLB200_K_SMALL_RING: return launch_small_ring(p, d->dtype, stream);
    case BLB200_K_DMMA_TMA: return launch_dmma_tma(p, d->dtype, stream);
    case BLB200_K_SGEMM_TMA: return launch_sgemm_tma(p, d->dtype, stream);
    default: break;
  }
  if (small32_supported(p, d->dtype)) return launch_small32(p, d->dtype, stream);
  if (small64_supported(p, d->dtype)) return launch_small64(p, d->dtype, stream);
  if (small_ring_supported(p, d->dtype)) return launch_small_ring(p, d->dtype, stream);
  return launch_tile_kernel(p, d->dtype, stream);
}

int dispatch_hetero(const blb200_gemm_desc* d, const int32_t* m_items, const int32_t* n_items,
                    const int32_t* k_items, cudaStream_t stream) {
  if (!m_items && !n_items && !k_items) return dispatch(d, stream);
  int rc = validate(d);
  if (rc != BLB200_OK) return rc;
  if (d->m == 0 || d->n == 0 || d->batch == 0) return BLB200_OK;
  GemmParams p = to_params(d);
  // The tile kernels take per-item dims when the capacity problem meets their preconditions (16-byte
  // aligned operands, more than 32 x 32); everything else goes to the generic kernel.
  if (d->kernel_hint == BLB200_K_AUTO && env_forced_kernel() == BLB200_K_AUTO) {
    GemmParams hp = p;
    hp.het_m = m_items;
    hp.het_n = n_items;
    hp.het_k = k_items;
    const int rc_tile = launch_tile_kernel(hp, d->dtype, stream, /*generic_fallback=*/false);
    if (rc_tile != BLB200_E_UNSUPPORTED) return rc_tile;
  }
  HeteroDims het{m_items, n_items, k_items, d->m, d->n, d->k};
  return launch_generic_hetero(p, het, d->dtype, stream);
}

}  // namespace blb200

extern "C" {

int blb200_gemm_heterogeneous(const blb200_gemm_desc* desc, const int32_t* m_items, const int32_t* n_items,
                              const int32_t* k_items, void* cuda_stream) {
  return blb200::dispatch_hetero(desc, m_items, n_items, k_items, (cudaStream_t)cuda_stream);
}

int blb200_gemm_validate(const blb200_gemm_desc* desc) { return blb200::validate(desc); }

int blb200_gemm_strided_batched(const blb200_gemm_desc* desc, void* cuda_stream) {
  return blb200::dispatch(desc, (cudaStream_t)cuda_stream);
}

const char* blb200_last_kernel_name(void) { return blb200::t_last_kernel; }
uint64_t blb200_launch_count(void) { return blb200::t_launches; }
const char* blb200_version(void) { return "0.1"; }

int blb200_trace_flush(void) {
  blb200::tracer().dump();
  return BLB200_OK;
}

const char* blb200_status_string(int status) {
  switch (status) {
    case BLB200_OK: return "ok";
    case BLB200_E_NULL: return "null pointer";
    case BLB200_E_SHAPE: return "GEMM: incompatible matrix dimensions";
    case BLB200_E_DTYPE: return "dtype or transpose out of range";
    case BLB200_E_UNSUPPORTED: return "requested kernel does not support this problem";
    case BLB200_E_NO_DEVICE: return "no usable CUDA device";
    case BLB200_E_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
    case BLB200_E_INTERNAL: return "internal error";
    default: break;
  }
  if (status > 0) return cudaGetErrorString((cudaError_t)status);
  return "unknown status";
}

}  // extern "C"
