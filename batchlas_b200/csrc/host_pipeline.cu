// Host-buffer entry points: the same strided-batched GEMM with A, B and C in HOST memory, on one GPU
// or sharded by contiguous batch ranges over several GPUs of the box.
//
// The reference keeps Matrix storage in host-visible shared USM (BatchLAS src/matrix.cc:150-166,
// src/util/sycl-util-impl.cc:36-46) and lets pages migrate when the GPU touches them.  Here the
// movement is explicit: the batch is cut into chunks and each chunk runs
//     H2D(A, B[, C]) -> kernel -> D2H(C)
// in order on one of three streams, so that chunk i+1's uploads and chunk i-1's download overlap
// chunk i's kernel (separate copy engines for each direction).
//
// Per-device state (three streams and a memory pool of the library's own) is created on the first
// call for a device and kept: staging is taken from that private pool with cudaMallocFromPoolAsync
// and given back to it, so repeated calls reuse the same memory, and nothing about the
// application's default pool is changed.  blb200_host_staging_trim hands the cached memory back
// to the driver.
#include <algorithm>
#include <mutex>
#include <thread>
#include <vector>

#include <sched.h>
#include <stdio.h>

#include "common.cuh"

namespace blb200 {
int dispatch(const blb200_gemm_desc* d, cudaStream_t stream);

namespace {

constexpr int kSlots = 3;

size_t elem_bytes(int dtype) {
  switch (dtype) {
    case BLB200_S: return 4;
    case BLB200_D: return 8;
    case BLB200_C: return 8;
    default: return 16;
  }
}

// Elements spanned by `items` consecutive batch items of a (rows x cols, ld, stride) operand.
size_t span_elems(int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t items) {
  if (items <= 0 || rows <= 0 || cols <= 0) return 0;
  return (size_t)((items - 1) * stride + (cols - 1) * ld + rows);
}

struct Slot {
  cudaStream_t stream = nullptr;
  char *a = nullptr, *b = nullptr, *c = nullptr;
};

// What a device keeps between calls.  One call at a time per device (the mutex is held for the
// whole call); calls for different devices run side by side.
struct DeviceCtx {
  std::mutex mu;
  bool ready = false;
  cudaStream_t streams[kSlots] = {};
  cudaMemPool_t pool = nullptr;
};

DeviceCtx* device_ctx(int device) {
  static DeviceCtx ctxs[64];
  if (device < 0 || device >= 64) return nullptr;
  return &ctxs[device];
}

// With `device` current and ctx->mu held.
int ensure_ready(DeviceCtx* ctx, int device) {
  if (ctx->ready) return BLB200_OK;
  for (int s = 0; s < kSlots; ++s) {
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->streams[s], cudaStreamNonBlocking);
    if (e != cudaSuccess) return (int)e;
  }
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;   // ordinary device memory, not migratable
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = device;
  cudaError_t e = cudaMemPoolCreate(&ctx->pool, &props);
  if (e != cudaSuccess) return (int)e;
  uint64_t keep = ~0ull;  // freed staging stays in THIS pool between calls
  e = cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep);
  if (e != cudaSuccess) return (int)e;
  ctx->ready = true;
  return BLB200_OK;
}

// Contiguous batch range of shard g of G: [floor(g*B/G), floor((g+1)*B/G)).
void shard_range(int64_t batch, int g, int G, int64_t* first, int64_t* count) {
  const int64_t b0 = batch * g / G, b1 = batch * (g + 1) / G;
  *first = b0;
  *count = b1 - b0;
}

// Best effort: run the calling thread on the cores of the NUMA node `device` hangs off, so that the
// thread feeding a GPU's copy engines sits next to them.  Silently does nothing when the topology
// cannot be read.
void bind_thread_near(int device) {
  char bdf[32] = {0};
  if (cudaDeviceGetPCIBusId(bdf, sizeof(bdf), device) != cudaSuccess) return;
  for (char* c = bdf; *c; ++c)
    if (*c >= 'A' && *c <= 'F') *c = (char)(*c - 'A' + 'a');
  char path[128];
  snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", bdf);
  FILE* f = fopen(path, "r");
  if (!f) return;
  int node = -1;
  const int got = fscanf(f, "%d", &node);
  fclose(f);
  if (got != 1 || node < 0) return;
  snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", node);
  f = fopen(path, "r");
  if (!f) return;
  cpu_set_t want, allowed, both;
  CPU_ZERO(&want);
  int lo = 0, hi = 0;
  for (;;) {
    if (fscanf(f, "%d", &lo) != 1) break;
    hi = lo;
    int ch = fgetc(f);
    if (ch == '-') {
      if (fscanf(f, "%d", &hi) != 1) break;
      ch = fgetc(f);
    }
    for (int c = lo; c <= hi && c < CPU_SETSIZE; ++c) CPU_SET(c, &want);
    if (ch != ',') break;
  }
  fclose(f);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) return;
  CPU_AND(&both, &want, &allowed);
  if (CPU_COUNT(&both) > 0) sched_setaffinity(0, sizeof(both), &both);
}

int host_gemm_on_device(const blb200_gemm_desc& d, int device, int32_t chunk_items);

}  // namespace
}  // namespace blb200

namespace blb200 {
namespace {

int host_gemm_on_device(const blb200_gemm_desc& d, int device, int32_t chunk_items) {
  int rc = BLB200_OK;
  DeviceCtx* ctx = device_ctx(device);
  if (!ctx) return BLB200_E_NO_DEVICE;
  int prev_device = 0;
  cudaGetDevice(&prev_device);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> lock(ctx->mu);
  rc = ensure_ready(ctx, device);
  if (rc != BLB200_OK) {
    cudaSetDevice(prev_device);
    return rc;
  }

  const size_t es = elem_bytes(d.dtype);
  const int64_t a_rows = d.op_a == BLB200_N ? d.m : d.k, a_cols = d.op_a == BLB200_N ? d.k : d.m;
  const int64_t b_rows = d.op_b == BLB200_N ? d.k : d.n, b_cols = d.op_b == BLB200_N ? d.n : d.k;
  const bool beta_zero = d.beta[0] == 0.0 && (d.dtype < BLB200_C || d.beta[1] == 0.0);
  const bool c_packed = d.ldc == d.m && d.stride_c == (int64_t)d.m * d.n;
  // C must be uploaded when it is read (beta != 0) or when its buffer has padding that the
  // contiguous download would otherwise overwrite with stale device bytes.
  const bool upload_c = !beta_zero || !c_packed;
  const bool a_shared = d.stride_a == 0, b_shared = d.stride_b == 0;  // one operand for every item
  const bool use_a = d.k > 0, use_b = d.k > 0;

  int64_t chunk = chunk_items;
  if (chunk <= 0) {
    const size_t per_item = (span_elems(a_rows, a_cols, d.lda, d.stride_a, 2) - span_elems(a_rows, a_cols, d.lda, d.stride_a, 1) +
                             span_elems(b_rows, b_cols, d.ldb, d.stride_b, 2) - span_elems(b_rows, b_cols, d.ldb, d.stride_b, 1) +
                             (size_t)d.stride_c) * es;
    const size_t target = (size_t)48 << 20;
    chunk = (int64_t)std::max<size_t>(1, target / std::max<size_t>(per_item, 1));
    const int64_t at_least_chunks = 2 * kSlots;
    chunk = std::min<int64_t>(chunk, std::max<int64_t>(1, (d.batch + at_least_chunks - 1) / at_least_chunks));
  }
  chunk = std::min<int64_t>(chunk, d.batch);

  const size_t a_chunk_bytes = use_a ? span_elems(a_rows, a_cols, d.lda, d.stride_a, a_shared ? 1 : chunk) * es : 0;
  const size_t b_chunk_bytes = use_b ? span_elems(b_rows, b_cols, d.ldb, d.stride_b, b_shared ? 1 : chunk) * es : 0;
  const size_t c_chunk_bytes = span_elems(d.m, d.n, d.ldc, d.stride_c, chunk) * es;

  Slot slots[kSlots];
  char *shared_a = nullptr, *shared_b = nullptr;
  cudaEvent_t shared_ready = nullptr;
  int status = BLB200_OK;
  auto fail = [&](cudaError_t err) {
    if (err != cudaSuccess && status == BLB200_OK) status = (int)err;
    return err != cudaSuccess;
  };

  const int used_slots = (int)std::min<int64_t>(kSlots, (d.batch + chunk - 1) / chunk);
  for (int s = 0; s < used_slots && status == BLB200_OK; ++s) {
    slots[s].stream = ctx->streams[s];
    if (use_a && !a_shared && fail(cudaMallocFromPoolAsync((void**)&slots[s].a, a_chunk_bytes, ctx->pool, slots[s].stream))) break;
    if (use_b && !b_shared && fail(cudaMallocFromPoolAsync((void**)&slots[s].b, b_chunk_bytes, ctx->pool, slots[s].stream))) break;
    if (fail(cudaMallocFromPoolAsync((void**)&slots[s].c, c_chunk_bytes, ctx->pool, slots[s].stream))) break;
  }
  if (status == BLB200_OK && ((use_a && a_shared) || (use_b && b_shared))) {
    cudaStream_t s0 = slots[0].stream;
    if (use_a && a_shared && !fail(cudaMallocFromPoolAsync((void**)&shared_a, a_chunk_bytes, ctx->pool, s0)))
      fail(cudaMemcpyAsync(shared_a, d.a, a_chunk_bytes, cudaMemcpyHostToDevice, s0));
    if (use_b && b_shared && !fail(cudaMallocFromPoolAsync((void**)&shared_b, b_chunk_bytes, ctx->pool, s0)))
      fail(cudaMemcpyAsync(shared_b, d.b, b_chunk_bytes, cudaMemcpyHostToDevice, s0));
    if (!fail(cudaEventCreateWithFlags(&shared_ready, cudaEventDisableTiming))) {
      fail(cudaEventRecord(shared_ready, s0));
      for (int s = 1; s < used_slots; ++s) fail(cudaStreamWaitEvent(slots[s].stream, shared_ready, 0));
    }
  }

  int64_t idx = 0;
  for (int64_t b0 = 0; b0 < d.batch && status == BLB200_OK; b0 += chunk, ++idx) {
    const int64_t nb = std::min<int64_t>(chunk, d.batch - b0);
    Slot& sl = slots[idx % used_slots];
    const char* ha = (const char*)d.a + (size_t)b0 * d.stride_a * es;
    const char* hb = (const char*)d.b + (size_t)b0 * d.stride_b * es;
    char* hc = (char*)d.c + (size_t)b0 * d.stride_c * es;
    const size_t c_bytes = span_elems(d.m, d.n, d.ldc, d.stride_c, nb) * es;
    if (use_a && !a_shared &&
        fail(cudaMemcpyAsync(sl.a, ha, span_elems(a_rows, a_cols, d.lda, d.stride_a, nb) * es,
                             cudaMemcpyHostToDevice, sl.stream)))
      break;
    if (use_b && !b_shared &&
        fail(cudaMemcpyAsync(sl.b, hb, span_elems(b_rows, b_cols, d.ldb, d.stride_b, nb) * es,
                             cudaMemcpyHostToDevice, sl.stream)))
      break;
    if (upload_c && fail(cudaMemcpyAsync(sl.c, hc, c_bytes, cudaMemcpyHostToDevice, sl.stream))) break;
    blb200_gemm_desc sub = d;
    sub.a = a_shared ? shared_a : sl.a;
    sub.b = b_shared ? shared_b : sl.b;
    sub.c = sl.c;
    sub.batch = (int32_t)nb;
    rc = dispatch(&sub, sl.stream);
    if (rc != BLB200_OK) {
      status = rc;
      break;
    }
    if (fail(cudaMemcpyAsync(hc, sl.c, c_bytes, cudaMemcpyDeviceToHost, sl.stream))) break;
  }

  for (int s = 0; s < used_slots; ++s) {
    if (!slots[s].stream) continue;
    if (slots[s].a) cudaFreeAsync(slots[s].a, slots[s].stream);
    if (slots[s].b) cudaFreeAsync(slots[s].b, slots[s].stream);
    if (slots[s].c) cudaFreeAsync(slots[s].c, slots[s].stream);
  }
  for (int s = 0; s < used_slots; ++s)
    if (slots[s].stream) fail(cudaStreamSynchronize(slots[s].stream));
  if (slots[0].stream) {
    if (shared_a) cudaFreeAsync(shared_a, slots[0].stream);
    if (shared_b) cudaFreeAsync(shared_b, slots[0].stream);
    cudaStreamSynchronize(slots[0].stream);
  }
  if (shared_ready) cudaEventDestroy(shared_ready);
  cudaSetDevice(prev_device);
  return status;
}

int check_host_desc(const blb200_gemm_desc* desc) {
  int rc = blb200_gemm_validate(desc);
  if (rc != BLB200_OK) return rc;
  const blb200_gemm_desc& d = *desc;
  if (d.batch > 1 && d.m > 0 && d.n > 0 && d.stride_c < (int64_t)(d.n - 1) * d.ldc + d.m)
    return BLB200_E_SHAPE;  // C items overlap
  return BLB200_OK;
}

}  // namespace
}  // namespace blb200

extern "C" int blb200_gemm_strided_batched_host(const blb200_gemm_desc* desc, int device, int32_t chunk_items) {
  using namespace blb200;
  const int rc = check_host_desc(desc);
  if (rc != BLB200_OK) return rc;
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  return host_gemm_on_device(*desc, device, chunk_items);
}

extern "C" void blb200_shard_range(int64_t batch, int32_t shard, int32_t shards, int64_t* first, int64_t* count) {
  int64_t f = 0, c = 0;
  if (batch > 0 && shards > 0 && shard >= 0 && shard < shards) blb200::shard_range(batch, shard, shards, &f, &c);
  if (first) *first = f;
  if (count) *count = c;
}

extern "C" int blb200_gemm_strided_batched_host_multi(const blb200_gemm_desc* desc, const int32_t* devices,
                                                      int32_t n_devices, int32_t chunk_items) {
  using namespace blb200;
  const int rc = check_host_desc(desc);
  if (rc != BLB200_OK) return rc;
  if (!devices || n_devices <= 0) return BLB200_E_NULL;
  if (n_devices > 64) return BLB200_E_TOO_LARGE;
  for (int g = 0; g < n_devices; ++g)
    for (int h = 0; h < g; ++h)
      if (devices[g] == devices[h]) return BLB200_E_UNSUPPORTED;  // one shard per GPU
  if (desc->m == 0 || desc->n == 0 || desc->batch == 0) return BLB200_OK;
  const size_t es = elem_bytes(desc->dtype);
  std::vector<int> status((size_t)n_devices, BLB200_OK);
  std::vector<std::thread> workers;
  workers.reserve((size_t)n_devices);
  for (int g = 0; g < n_devices; ++g) {
    int64_t first = 0, count = 0;
    shard_range(desc->batch, g, n_devices, &first, &count);
    if (count == 0) continue;
    blb200_gemm_desc sub = *desc;
    sub.a = (const char*)desc->a + (size_t)first * desc->stride_a * es;
    sub.b = (const char*)desc->b + (size_t)first * desc->stride_b * es;
    sub.c = (char*)desc->c + (size_t)first * desc->stride_c * es;
    sub.batch = (int32_t)count;
    const int dev = devices[g];
    workers.emplace_back([sub, dev, chunk_items, g, &status] {
      bind_thread_near(dev);
      status[(size_t)g] = host_gemm_on_device(sub, dev, chunk_items);
    });
  }
  for (auto& w : workers) w.join();
  for (int g = 0; g < n_devices; ++g)
    if (status[(size_t)g] != BLB200_OK) return status[(size_t)g];
  return BLB200_OK;
}

extern "C" int blb200_host_staging_trim(int device) {
  using namespace blb200;
  DeviceCtx* ctx = device_ctx(device);
  if (!ctx) return BLB200_E_NO_DEVICE;
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (!ctx->ready) return BLB200_OK;
  return (int)cudaMemPoolTrimTo(ctx->pool, 0);
}
