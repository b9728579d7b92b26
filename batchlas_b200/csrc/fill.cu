// Counter-based synthetic inputs.  Element i of tensor `tensor_id` under `seed` is a pure function
// of (seed, tensor_id, first_index + i): a SplitMix64 finaliser over index * golden-ratio + key.
// The uniform path uses only integer and exactly-rounded double operations, so it is bit-identical
// to the NumPy statement of the same function used by the tests; the normal path goes through
// log/cos and agrees to rounding.
#include "common.cuh"

namespace blb200 {
namespace {

__host__ __device__ inline uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__host__ __device__ inline uint64_t make_key(uint64_t seed, uint32_t tensor_id, uint32_t lane) {
  return mix64(seed ^ ((uint64_t)tensor_id << 32) ^ ((uint64_t)lane << 56));
}

__device__ inline double unit(uint64_t idx, uint64_t key) {
  return (double)(mix64(idx * 0x9E3779B97F4A7C15ull + key) >> 11) * (1.0 / 9007199254740992.0);
}

__device__ inline double draw(uint64_t idx, uint64_t k0, uint64_t k1, int dist, double scale) {
  const double u1 = unit(idx, k0);
  if (dist == 0) return 2.0 * u1 - 1.0;
  const double u2 = unit(idx, k1);
  return sqrt(-2.0 * log(1.0 - u1)) * cos(6.283185307179586 * u2) * scale;
}

template <typename R, bool CPLX>
__global__ void fill_kernel(R* dst, uint64_t count, uint64_t first, uint64_t k0, uint64_t k1,
                            uint64_t k2, uint64_t k3, int dist, double scale) {
  const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
    const uint64_t idx = first + i;
    if (CPLX) {
      dst[2 * i] = (R)draw(idx, k0, k1, dist, scale);
      dst[2 * i + 1] = (R)draw(idx, k2, k3, dist, scale);
    } else {
      dst[i] = (R)draw(idx, k0, k1, dist, scale);
    }
  }
}

}  // namespace
}  // namespace blb200

extern "C" int blb200_fill(void* dst, int32_t dtype, uint64_t count, uint64_t first_index,
                           uint64_t seed, uint32_t tensor_id, int32_t dist, double scale,
                           void* cuda_stream) {
  using namespace blb200;
  if (count == 0) return BLB200_OK;
  if (!dst) return BLB200_E_NULL;
  if (dist < 0 || dist > 1) return BLB200_E_DTYPE;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const uint64_t k0 = make_key(seed, tensor_id, 0), k1 = make_key(seed, tensor_id, 1);
  const uint64_t k2 = make_key(seed, tensor_id, 2), k3 = make_key(seed, tensor_id, 3);
  const uint64_t want = (count + 255) / 256;
  const unsigned grid = (unsigned)(want < 148ull * 32 ? want : 148ull * 32);
  switch (dtype) {
    case BLB200_S: fill_kernel<float, false><<<grid, 256, 0, s>>>((float*)dst, count, first_index, k0, k1, k2, k3, dist, scale); break;
    case BLB200_D: fill_kernel<double, false><<<grid, 256, 0, s>>>((double*)dst, count, first_index, k0, k1, k2, k3, dist, scale); break;
    case BLB200_C: fill_kernel<float, true><<<grid, 256, 0, s>>>((float*)dst, count, first_index, k0, k1, k2, k3, dist, scale); break;
    case BLB200_Z: fill_kernel<double, true><<<grid, 256, 0, s>>>((double*)dst, count, first_index, k0, k1, k2, k3, dist, scale); break;
    default: return BLB200_E_DTYPE;
  }
  return (int)cudaGetLastError();
}
