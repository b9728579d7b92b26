// Host-buffer entry point: the same strided-batched GEMM with A, B and C in HOST memory.
//
// The reference keeps Matrix storage in host-visible shared USM (BatchLAS src/matrix.cc:150-166,
// src/util/sycl-util-impl.cc:36-46) and lets pages migrate when the GPU touches them.  Here the
// movement is explicit: the batch is cut into chunks and each chunk runs
//     H2D(A, B[, C]) -> kernel -> D2H(C)
// in order on one of three streams, so that chunk i+1's uploads and chunk i-1's download overlap
// chunk i's kernel (separate copy engines for each direction).  Device staging is borrowed from
// the device's stream-ordered memory pool for the duration of the call.
#include <algorithm>
#include <mutex>

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

void keep_pool_memory(int device) {
  // Freed staging stays cached in the pool between calls instead of going back to the driver.
  static std::once_flag flags[64];
  if (device < 0 || device >= 64) return;
  std::call_once(flags[device], [device] {
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
      uint64_t keep = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
  });
}

}  // namespace
}  // namespace blb200

extern "C" int blb200_gemm_strided_batched_host(const blb200_gemm_desc* desc, int device,
                                                int32_t chunk_items) {
  using namespace blb200;
  int rc = blb200_gemm_validate(desc);
  if (rc != BLB200_OK) return rc;
  const blb200_gemm_desc& d = *desc;
  if (d.m == 0 || d.n == 0 || d.batch == 0) return BLB200_OK;
  if (d.batch > 1 && d.stride_c < (int64_t)(d.n - 1) * d.ldc + d.m) return BLB200_E_SHAPE;  // C items overlap

  int prev_device = 0;
  cudaGetDevice(&prev_device);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  keep_pool_memory(device);

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
    if (fail(cudaStreamCreateWithFlags(&slots[s].stream, cudaStreamNonBlocking))) break;
    if (use_a && !a_shared && fail(cudaMallocAsync((void**)&slots[s].a, a_chunk_bytes, slots[s].stream))) break;
    if (use_b && !b_shared && fail(cudaMallocAsync((void**)&slots[s].b, b_chunk_bytes, slots[s].stream))) break;
    if (fail(cudaMallocAsync((void**)&slots[s].c, c_chunk_bytes, slots[s].stream))) break;
  }
  if (status == BLB200_OK && ((use_a && a_shared) || (use_b && b_shared))) {
    cudaStream_t s0 = slots[0].stream;
    if (use_a && a_shared && !fail(cudaMallocAsync((void**)&shared_a, a_chunk_bytes, s0)))
      fail(cudaMemcpyAsync(shared_a, d.a, a_chunk_bytes, cudaMemcpyHostToDevice, s0));
    if (use_b && b_shared && !fail(cudaMallocAsync((void**)&shared_b, b_chunk_bytes, s0)))
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
  for (int s = 0; s < used_slots; ++s)
    if (slots[s].stream) cudaStreamDestroy(slots[s].stream);
  cudaSetDevice(prev_device);
  return status;
}
