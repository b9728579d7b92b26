// Aggregates the per-translation-unit device status words (set when a bounded wait gave up).
#include "common.cuh"

namespace blb200 {
int small_device_status(int* out);
int gemv_ring_device_status(int* out);
int small_ring_device_status(int* out);
}

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
  *out = word;
  return BLB200_OK;
}
