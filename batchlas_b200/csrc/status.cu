// Aggregates the per-translation-unit device status words (set when a bounded wait gave up), and
// holds the self-test that makes one such wait run out on purpose.
#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
int small_device_status(int* out);
int gemv_ring_device_status(int* out);
int small_ring_device_status(int* out);
int dmma_tma_device_status(int* out);
int dmma_tma_device_status_clear();
int sgemm_tma_device_status(int* out);
int sgemm_tma_device_status_clear();
int small_device_status_clear();
int gemv_ring_device_status_clear();
int small_ring_device_status_clear();

namespace {
// One warp waits on a barrier that nothing ever arrives on.  The wait is the ring kernels' own
// mbar_wait with a short poll limit: it gives up, records its code and the kernel returns
// normally — no copy is in flight, nothing else shares the barrier, the context stays usable.
__global__ void wait_expiry_selftest_kernel(uint32_t max_polls, int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_limit(&bar, 0u, BLB200_WAIT_SELFTEST, max_polls);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
}
}  // namespace
}  // namespace blb200

// Synchronises the current device, then writes the first non-zero status word to *out
// (0 = no kernel ever abandoned a wait).  Returns 0 or a cudaError_t.
extern "C" int blb200_device_status(int* out) {
  if (!out) return BLB200_E_NULL;
  *out = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  int word = 0;
  int rc = blb200::small_device_status(&word);
  if (rc != 0) return rc;
  if (word == 0) {
    rc = blb200::gemv_ring_device_status(&word);
    if (rc != 0) return rc;
  }
  if (word == 0) {
    rc = blb200::small_ring_device_status(&word);
    if (rc != 0) return rc;
  }
  if (word == 0) {
    rc = blb200::dmma_tma_device_status(&word);
    if (rc != 0) return rc;
  }
  if (word == 0) {
    rc = blb200::sgemm_tma_device_status(&word);
    if (rc != 0) return rc;
  }
  if (word == 0) {
    rc = blb200::read_device_status_word(&word);
    if (rc != 0) return rc;
  }
  *out = word;
  return BLB200_OK;
}

extern "C" int blb200_device_status_reset(void) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  int rc = blb200::small_device_status_clear();
  if (rc == 0) rc = blb200::gemv_ring_device_status_clear();
  if (rc == 0) rc = blb200::small_ring_device_status_clear();
  if (rc == 0) rc = blb200::dmma_tma_device_status_clear();
  if (rc == 0) rc = blb200::sgemm_tma_device_status_clear();
  if (rc == 0) rc = blb200::clear_device_status_word();
  return rc;
}

extern "C" int blb200_selftest_wait_expiry(uint32_t max_polls, void* cuda_stream) {
  if (max_polls == 0 || max_polls > (1u << 16)) return BLB200_E_TOO_LARGE;  // at most a few milliseconds
  blb200::wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)cuda_stream>>>(max_polls, nullptr);
  return (int)cudaGetLastError();
}
