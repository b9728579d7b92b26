// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk async copies (TMA, untiled and tiled),
// 16-byte cp.async.  Every wait is bounded: after kSpinLimit failed polls the waiter records an
// error code in a device status word and gives up, so a lost copy can never hang the GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace blb200 {

// Non-zero once a kernel of the including translation unit gave up on a wait (one word per
// translation unit; the library's blb200_device_status() reads them all).
static __device__ int g_device_status = 0;
static inline int read_device_status_word(int* out) {
  return (int)cudaMemcpyFromSymbol(out, g_device_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}
static inline int clear_device_status_word() {
  const int zero = 0;
  return (int)cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice);
}

constexpr uint32_t kSpinLimit = 1u << 22;  // polls; each poll may itself block for a short HW-defined time

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Returns false (after recording `code`) when the phase did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int code, uint32_t limit) {
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (spin > 64) __nanosleep(64);
  }
  atomicCAS(&g_device_status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
  return mbar_wait_limit(bar, parity, code, kSpinLimit);
}

// global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// shared -> global bulk copy; completion tracked by the issuing thread's bulk-group.
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy shared-memory writes visible to the async proxy (before a bulk store).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 16-byte async copy global -> shared; src_bytes < 16 zero-fills the remainder (0 = all zeros).
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem),
               "r"(src_bytes)
               : "memory");
}
// BYTES-sized (4, 8 or 16) async copy for operands that are only element-aligned; src_bytes = 0
// zero-fills.  Both addresses must be BYTES-aligned.
template <int BYTES>
__device__ __forceinline__ void cp_async_elem(void* dst_smem, const void* src_gmem, uint32_t src_bytes) {
  static_assert(BYTES == 4 || BYTES == 8 || BYTES == 16, "cp.async copies 4, 8 or 16 bytes");
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "n"(BYTES),
               "r"(src_bytes)
               : "memory");
}
// One 16-byte stage chunk from a source that is only ES-aligned (ES = 4 or 8 bytes per element,
// `valid` elements of the chunk exist, the rest is zero-filled): the widest copies the source
// address allows — one 16-byte copy when it happens to be 16-byte aligned (with an odd leading
// dimension every second column of doubles is), two 8-byte copies for floats on an 8-byte boundary
// (ld = 258: every other column), else element by element.  The destination is 16-byte aligned.
template <int ES>
__device__ __forceinline__ void cp_async_chunk_widest(unsigned char* dst, const unsigned char* src, int valid) {
  constexpr int V = 16 / ES;
  const uintptr_t a = reinterpret_cast<uintptr_t>(src);
  if (valid == V && (a & 15u) == 0) {
    cp_async_elem<16>(dst, src, 16);
  } else if (ES == 4 && valid == V && (a & 7u) == 0) {
    cp_async_elem<8>(dst, src, 8);
    cp_async_elem<8>(dst + 8, src + 8, 8);
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) cp_async_elem<ES>(dst + e * ES, e < valid ? src + e * ES : src, e < valid ? ES : 0);
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Packed FP32 FMA (Blackwell FFMA2): d.lo += a.lo*b.lo, d.hi += a.hi*b.hi, each an IEEE fused
// multiply-add.  One instruction issues two FMAs and holds the FMA pipe for two cycles.
__device__ __forceinline__ void ffma2(uint64_t& d, uint64_t a, uint64_t b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ uint64_t dup2(float f) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// Release-acquire counter bump in shared memory: the warps that share a ring slot count themselves
// off it, and the one whose old value says that all the others have left knows that they have
// finished reading the slot as well.
__device__ __forceinline__ uint32_t smem_add_acq_rel(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
  return old;
}

}  // namespace blb200
