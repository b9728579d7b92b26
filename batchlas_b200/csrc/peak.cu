// FMA issue-rate microbenchmarks: the measured FP32 / FP64 pipe peaks that the compute-bound
// configurations are judged against (the nominal figures are SMs x lanes x 2 x max clock).
// Each thread runs 16 independent dependent-chains of FMAs held in registers; nothing touches memory
// until one value is written at the end so the loop cannot be removed.
#include "common.cuh"

namespace blb200 {
namespace {

template <typename R>
__global__ void __launch_bounds__(256) fma_rate_kernel(R* sink, int iters, R a, R b) {
  R acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = (R)(threadIdx.x + i);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int rep = 0; rep < 4; ++rep)
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = acc[i] * a + b;  // contracted to one FMA
  }
  R total = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) total += acc[i];
  if (total == (R)123456789) sink[0] = total;  // practically never true; keeps the chain live
}

// FP64 tensor-core rate: mma.sync m8n8k4 (256 FMAs per warp instruction), 8 independent accumulator
// pairs per thread.
__global__ void __launch_bounds__(256) dmma_rate_kernel(double* sink, int iters, double a, double b) {
  double c[8][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) c[i][0] = c[i][1] = (double)(threadIdx.x + i);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int rep = 0; rep < 4; ++rep)
#pragma unroll
      for (int i = 0; i < 8; ++i)
        asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                     : "+d"(c[i][0]), "+d"(c[i][1])
                     : "d"(a), "d"(b));
  }
  double total = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += c[i][0] + c[i][1];
  if (total == 123456789.0) sink[0] = total;
}

// Packed FP32 FMA rate (fma.rn.f32x2: two FMAs per lane per instruction).
__global__ void __launch_bounds__(256) ffma2_rate_kernel(unsigned long long* sink, int iters, float a, float b) {
  unsigned long long acc[16], av, bv;
  asm("mov.b64 %0, {%1, %1};" : "=l"(av) : "f"(a));
  asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float f = (float)(threadIdx.x + i);
    asm("mov.b64 %0, {%1, %1};" : "=l"(acc[i]) : "f"(f));
  }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int rep = 0; rep < 4; ++rep)
#pragma unroll
      for (int i = 0; i < 16; ++i) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(av), "l"(bv));
  }
  unsigned long long total = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) total ^= acc[i];
  if (total == 0x123456789abcdefull) sink[0] = total;
}

// The same instruction in the operand pattern of an 8 x 8 register block: 32 accumulator pairs,
// 4 A pairs and 8 duplicated B values, every product a2[rp] * b2[c] (what the GEMM inner loops issue).
__global__ void __launch_bounds__(256) ffma2_outer_kernel(unsigned long long* sink, int iters, float a, float b) {
  unsigned long long acc[32], a2[4], b2[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float f = a + 0.001f * (float)(i + threadIdx.x % 3);
    asm("mov.b64 %0, {%1, %1};" : "=l"(a2[i]) : "f"(f));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float f = b + 0.001f * (float)i;
    asm("mov.b64 %0, {%1, %1};" : "=l"(b2[i]) : "f"(f));
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float f = (float)(threadIdx.x + i);
    asm("mov.b64 %0, {%1, %1};" : "=l"(acc[i]) : "f"(f));
  }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int rep = 0; rep < 2; ++rep)
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int rp = 0; rp < 4; ++rp)
          asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[rp * 8 + c]) : "l"(a2[rp]), "l"(b2[c]));
  }
  unsigned long long total = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) total ^= acc[i];
  if (total == 0x123456789abcdefull) sink[0] = total;
}

int measure_ffma2_outer(double* tflops) {
  const DeviceInfo& dev = device_info();
  unsigned long long* sink = nullptr;
  cudaError_t e = cudaMalloc(&sink, sizeof(unsigned long long));
  if (e != cudaSuccess) return (int)e;
  const int iters = 4096, blocks = dev.sm_count * 8, threads = 256;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  ffma2_outer_kernel<<<blocks, threads>>>(sink, 16, 0.999f, 0.001f);
  float best = 1e30f;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(t0);
    ffma2_outer_kernel<<<blocks, threads>>>(sink, iters, 0.999f, 0.001f);
    cudaEventRecord(t1);
    e = cudaEventSynchronize(t1);
    if (e != cudaSuccess) break;
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    if (ms < best) best = ms;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(sink);
  if (e != cudaSuccess) return (int)e;
  const double flops = 2.0 * 2.0 * 64.0 * iters * (double)blocks * threads;
  *tflops = flops / (best * 1e-3) / 1e12;
  return BLB200_OK;
}

int measure_ffma2(double* tflops) {
  const DeviceInfo& dev = device_info();
  unsigned long long* sink = nullptr;
  cudaError_t e = cudaMalloc(&sink, sizeof(unsigned long long));
  if (e != cudaSuccess) return (int)e;
  const int iters = 4096, blocks = dev.sm_count * 8, threads = 256;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  ffma2_rate_kernel<<<blocks, threads>>>(sink, 16, 0.999f, 0.001f);
  float best = 1e30f;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(t0);
    ffma2_rate_kernel<<<blocks, threads>>>(sink, iters, 0.999f, 0.001f);
    cudaEventRecord(t1);
    e = cudaEventSynchronize(t1);
    if (e != cudaSuccess) break;
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    if (ms < best) best = ms;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(sink);
  if (e != cudaSuccess) return (int)e;
  const double flops = 2.0 * 2.0 * 64.0 * iters * (double)blocks * threads;
  *tflops = flops / (best * 1e-3) / 1e12;
  return BLB200_OK;
}

int measure_dmma(double* tflops) {
  const DeviceInfo& dev = device_info();
  double* sink = nullptr;
  cudaError_t e = cudaMalloc(&sink, sizeof(double));
  if (e != cudaSuccess) return (int)e;
  const int iters = 2048, blocks = dev.sm_count * 8, threads = 256;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  dmma_rate_kernel<<<blocks, threads>>>(sink, 16, 0.999, 0.001);
  float best = 1e30f;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(t0);
    dmma_rate_kernel<<<blocks, threads>>>(sink, iters, 0.999, 0.001);
    cudaEventRecord(t1);
    e = cudaEventSynchronize(t1);
    if (e != cudaSuccess) break;
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    if (ms < best) best = ms;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(sink);
  if (e != cudaSuccess) return (int)e;
  // per warp instruction: 8*8*4 FMAs = 512 flops; 32 instructions per iteration per warp
  const double flops = 512.0 * 32.0 * iters * (double)blocks * (threads / 32);
  *tflops = flops / (best * 1e-3) / 1e12;
  return BLB200_OK;
}

template <typename R>
int measure(double* tflops, double* ms_out) {
  const DeviceInfo& dev = device_info();
  R* sink = nullptr;
  cudaError_t e = cudaMalloc(&sink, sizeof(R));
  if (e != cudaSuccess) return (int)e;
  const int iters = 4096, blocks = dev.sm_count * 8, threads = 256;
  cudaEvent_t t0, t1;
  cudaEventCreate(&t0);
  cudaEventCreate(&t1);
  fma_rate_kernel<R><<<blocks, threads>>>(sink, 64, (R)0.999, (R)0.001);  // warm-up
  float best = 1e30f;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(t0);
    fma_rate_kernel<R><<<blocks, threads>>>(sink, iters, (R)0.999, (R)0.001);
    cudaEventRecord(t1);
    e = cudaEventSynchronize(t1);
    if (e != cudaSuccess) break;
    float ms = 0;
    cudaEventElapsedTime(&ms, t0, t1);
    if (ms < best) best = ms;
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(sink);
  if (e != cudaSuccess) return (int)e;
  const double flops = 2.0 * 64.0 * iters * (double)blocks * threads;
  *tflops = flops / (best * 1e-3) / 1e12;
  if (ms_out) *ms_out = best;
  return BLB200_OK;
}

}  // namespace
}  // namespace blb200

// Measures the FMA issue rate of the current device for float (dtype S) or double (dtype D) in
// TFLOP/s (2 flops per FMA); dtype Z selects the FP64 tensor-core (DMMA m8n8k4) rate and dtype C
// the packed FP32 (fma.rn.f32x2) rate instead; 100 + BLB200_C measures fma.rn.f32x2 in the operand
// pattern of an 8 x 8 register block (32 accumulators, 4 x 8 distinct operand pairs).
// Synchronous; allocates a few bytes; a diagnostic, not a data path.
extern "C" int blb200_measure_pipe_peak(int32_t dtype, double* tflops) {
  if (!tflops) return BLB200_E_NULL;
  if (dtype == BLB200_S) return blb200::measure<float>(tflops, nullptr);
  if (dtype == BLB200_D) return blb200::measure<double>(tflops, nullptr);
  if (dtype == BLB200_Z) return blb200::measure_dmma(tflops);
  if (dtype == BLB200_C) return blb200::measure_ffma2(tflops);
  if (dtype == 100 + BLB200_C) return blb200::measure_ffma2_outer(tflops);
  return BLB200_E_DTYPE;
}
