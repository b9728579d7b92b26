// Whole-matrix-per-warp kernels for packed small float matrices: the HBM-bound end of the family.
//
// small32: m = n = k = 32, float, ld = 32 on all three operands, batch strides that are multiples
// of 4 elements, 16-byte aligned bases (BatchLAS's own fast paths are gated the same way:
// src/sycl/gemm/load_policies.hh:18-34).  Each 4 KiB matrix is one contiguous run in memory, so an
// item's operands are fetched by three untiled bulk copies (TMA, cp.async.bulk) issued by one
// producer thread into a ring of shared-memory stages guarded by full/empty mbarriers.  Consumer
// warps each own one matrix at a time: a lane keeps a 4 x 8 block of C in registers (rows
// 4*ti..4*ti+3, columns 8*tj..8*tj+7, ti = lane & 7, tj = lane >> 3) and reads operands from shared
// memory as 128-bit fragments, then writes C with 128-bit stores (8 lanes cover one 128-byte
// column).  A persistent grid of one CTA per SM walks the batch round-robin.
//
// Operand orientation only changes how fragments are read; nothing is transposed in memory:
//   M-major A (op N): float4 = 4 rows at one k.        K-major A (op T): float4 = 4 k at one row.
//   N-major B (op T): float4 = 4 cols at one k.        K-major B (op N): float4 = 4 k at one col.
// With a K-major operand, lanes walk the eight 4-wide k-chunks in a lane-dependent rotation so
// that the lanes of one shared-memory request fall into different 16-byte bank groups; the sum
// over k is the same set of products in a different order.
//
// Algorithmic traffic per item: A + B (+ C when beta != 0) read and C written, 4 KiB each.
#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads32 = 32 * (1 + kConsumerWarps);
constexpr int kMatBytes32 = 32 * 32 * 4;

enum WaitCode { kWaitFull = 101, kWaitEmpty = 102, kWaitDrain = 103 };

// acc[r][c] += sum_k opA(4ti+r, k) * opB(k, 8tj+c) for one 32x32x32 item held in shared memory.
template <bool A_KMAJOR, bool B_KMAJOR>
__device__ __forceinline__ void mma32(const float4* __restrict__ As4, const float4* __restrict__ Bs4,
                                      int ti, int tj, float (&acc)[4][8]) {
  if (!A_KMAJOR && !B_KMAJOR) {
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const float4 a = As4[k * 8 + ti];
      const float4 b0 = Bs4[k * 8 + 2 * tj];
      const float4 b1 = Bs4[k * 8 + 2 * tj + 1];
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(av[r], bv[c], acc[r][c]);
    }
  } else {
    // Rotation that keeps the more expensive operand's requests conflict-free.
    const int skew = (A_KMAJOR && B_KMAJOR) ? ti : tj;
#pragma unroll 2
    for (int s = 0; s < 8; ++s) {
      const int kc = (s + skew) & 7;
      float af[4][4];  // [row][kk]
      float bf[8][4];  // [col][kk]
      if (A_KMAJOR) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 v = As4[(4 * ti + r) * 8 + kc];
          af[r][0] = v.x; af[r][1] = v.y; af[r][2] = v.z; af[r][3] = v.w;
        }
      } else {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 v = As4[(4 * kc + kk) * 8 + ti];
          af[0][kk] = v.x; af[1][kk] = v.y; af[2][kk] = v.z; af[3][kk] = v.w;
        }
      }
      if (B_KMAJOR) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float4 v = Bs4[(8 * tj + c) * 8 + kc];
          bf[c][0] = v.x; bf[c][1] = v.y; bf[c][2] = v.z; bf[c][3] = v.w;
        }
      } else {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 v0 = Bs4[(4 * kc + kk) * 8 + 2 * tj];
          const float4 v1 = Bs4[(4 * kc + kk) * 8 + 2 * tj + 1];
          bf[0][kk] = v0.x; bf[1][kk] = v0.y; bf[2][kk] = v0.z; bf[3][kk] = v0.w;
          bf[4][kk] = v1.x; bf[5][kk] = v1.y; bf[6][kk] = v1.z; bf[7][kk] = v1.w;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(af[r][kk], bf[c][kk], acc[r][c]);
    }
  }
}

// Shared memory: `stages` x {A, B[, C]} of 4 KiB each, then full[stages], empty[stages] barriers.
template <bool A_KMAJOR, bool B_KMAJOR, bool HAS_C>
__global__ void __launch_bounds__(kThreads32, 1)
    gemm_small32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                        long long sa, long long sb, long long sc, int batch, float alpha, float beta,
                        int stages) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kStageBytes = (HAS_C ? 3 : 2) * kMatBytes32;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();

  // Items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; the j-th one uses stage j % stages
  // and consumer warp j % kConsumerWarps (stages is a multiple of kConsumerWarps).
  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < my_items; ++j) {
        const int s = j % stages;
        const uint32_t round = (uint32_t)(j / stages);
        if (!mbar_wait(&empty_bar[s], (round & 1u) ^ 1u, kWaitEmpty)) return;
        const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
        unsigned char* st = smem + (size_t)s * kStageBytes;
        mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
        bulk_g2s(st, A + item * sa, kMatBytes32, &full_bar[s]);
        bulk_g2s(st + kMatBytes32, B + item * sb, kMatBytes32, &full_bar[s]);
        if (HAS_C) bulk_g2s(st + 2 * kMatBytes32, C + item * sc, kMatBytes32, &full_bar[s]);
      }
    }
    return;
  }

  const int cw = warp - 1;
  const int ti = lane & 7, tj = lane >> 3;
  for (int j = cw; j < my_items; j += kConsumerWarps) {
    const int s = j % stages;
    const uint32_t round = (uint32_t)(j / stages);
    if (!mbar_wait(&full_bar[s], round & 1u, kWaitFull)) return;
    const unsigned char* st = smem + (size_t)s * kStageBytes;
    const float4* As4 = reinterpret_cast<const float4*>(st);
    const float4* Bs4 = reinterpret_cast<const float4*>(st + kMatBytes32);
    const float4* Cs4 = reinterpret_cast<const float4*>(st + 2 * kMatBytes32);

    float acc[4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;
    mma32<A_KMAJOR, B_KMAJOR>(As4, Bs4, ti, tj, acc);

    float4 prior[8];
    if (HAS_C) {
#pragma unroll
      for (int c = 0; c < 8; ++c) prior[c] = Cs4[(8 * tj + c) * 8 + ti];
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);  // stage may be refilled while we store

    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    float4* Cg4 = reinterpret_cast<float4*>(C + item * sc);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4 o;
      o.x = alpha * acc[0][c];
      o.y = alpha * acc[1][c];
      o.z = alpha * acc[2][c];
      o.w = alpha * acc[3][c];
      if (HAS_C) {
        o.x = fmaf(beta, prior[c].x, o.x);
        o.y = fmaf(beta, prior[c].y, o.y);
        o.z = fmaf(beta, prior[c].z, o.z);
        o.w = fmaf(beta, prior[c].w, o.w);
      }
      Cg4[(8 * tj + c) * 8 + ti] = o;
    }
  }
}

template <bool AK, bool BK, bool HC>
int launch32(const GemmParams& p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  constexpr int kStageBytes = (HC ? 3 : 2) * kMatBytes32;
  const size_t budget = dev.smem_optin > 8192 ? dev.smem_optin - 4096 : 0;
  int stages = (int)(budget / ((size_t)kStageBytes * kConsumerWarps)) * kConsumerWarps;
  if (stages > 32) stages = 32;
  if (stages < kConsumerWarps) return BLB200_E_UNSUPPORTED;
  const size_t smem = (size_t)stages * kStageBytes + (size_t)stages * 2 * sizeof(uint64_t);
  auto kern = gemm_small32_kernel<AK, BK, HC>;
  static thread_local int configured_for = -1;  // per (instantiation, thread): device last configured
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = p.batch < dev.sm_count ? p.batch : dev.sm_count;
  kern<<<grid, kThreads32, smem, stream>>>((const float*)p.a, (const float*)p.b, (float*)p.c, p.sa, p.sb,
                                           p.sc, p.batch, (float)p.alpha[0], (float)p.beta[0], stages);
  return (int)cudaGetLastError();
}


// ---- small64 ---------------------------------------------------------------------------------
// m = n = k = 64, float, packed (ld = 64).  Two consumer warps share one matrix: warp half hw owns
// columns 32*hw .. 32*hw+31 and each lane an 8 x 8 block of C (64 accumulators), which is what
// lets the FP32 pipe rather than shared memory set the pace (16 fragment floats per 64 FMAs).
//
// A K-major operand cannot be read 128 bits at a time without bank conflicts when its rows sit
// 256 bytes apart, so it is brought in row by row — 64 bulk copies of 256 bytes — into rows
// pitched 272 bytes apart, and its rows (or columns) are dealt to lanes round-robin:
//   A K-major: lane rows ti + 8r        (r = 0..7);   else rows 4ti..4ti+3 and 32+4ti..32+4ti+3
//   B K-major: lane cols 32hw + tj + 4c (c = 0..7);   else cols 32hw + 8tj + c
// With that, every fragment request of a warp touches each 16-byte bank group at most once.
constexpr int kPairs64 = 4;
constexpr int kThreads64 = 32 * (1 + 2 * kPairs64);
constexpr int kMatBytes64 = 64 * 64 * 4;
constexpr int kPitch64 = 272;                    // bytes between rows of a K-major operand
constexpr int kPadBytes64 = 64 * kPitch64;       // 17408

template <bool A_KMAJOR, bool B_KMAJOR>
__device__ __forceinline__ void mma64(const unsigned char* __restrict__ As, const unsigned char* __restrict__ Bs,
                                      int ti, int tj, int hw, float (&acc)[8][8]) {
  const float4* As4 = reinterpret_cast<const float4*>(As);
  const float4* Bs4 = reinterpret_cast<const float4*>(Bs);
#pragma unroll 2
  for (int kc = 0; kc < 16; ++kc) {
    float af[8][4], bf[8][4];  // [row or col][kk]
    if (A_KMAJOR) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 v = As4[(ti + 8 * r) * (kPitch64 / 16) + kc];
        af[r][0] = v.x; af[r][1] = v.y; af[r][2] = v.z; af[r][3] = v.w;
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 lo = As4[(4 * kc + kk) * 16 + ti];
        const float4 hi = As4[(4 * kc + kk) * 16 + 8 + ti];
        af[0][kk] = lo.x; af[1][kk] = lo.y; af[2][kk] = lo.z; af[3][kk] = lo.w;
        af[4][kk] = hi.x; af[5][kk] = hi.y; af[6][kk] = hi.z; af[7][kk] = hi.w;
      }
    }
    if (B_KMAJOR) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 v = Bs4[(32 * hw + tj + 4 * c) * (kPitch64 / 16) + kc];
        bf[c][0] = v.x; bf[c][1] = v.y; bf[c][2] = v.z; bf[c][3] = v.w;
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 v0 = Bs4[(4 * kc + kk) * 16 + 8 * hw + 2 * tj];
        const float4 v1 = Bs4[(4 * kc + kk) * 16 + 8 * hw + 2 * tj + 1];
        bf[0][kk] = v0.x; bf[1][kk] = v0.y; bf[2][kk] = v0.z; bf[3][kk] = v0.w;
        bf[4][kk] = v1.x; bf[5][kk] = v1.y; bf[6][kk] = v1.z; bf[7][kk] = v1.w;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(af[r][kk], bf[c][kk], acc[r][c]);
  }
}

template <bool A_KMAJOR, bool B_KMAJOR, bool HAS_C>
__global__ void __launch_bounds__(kThreads64, 1)
    gemm_small64_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                        long long sa, long long sb, long long sc, int batch, float alpha, float beta,
                        int stages) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kABytes = A_KMAJOR ? kPadBytes64 : kMatBytes64;
  constexpr int kBBytes = B_KMAJOR ? kPadBytes64 : kMatBytes64;
  constexpr int kStageBytes = kABytes + kBBytes + (HAS_C ? kMatBytes64 : 0);
  constexpr uint32_t kTxBytes = (uint32_t)(2 + (HAS_C ? 1 : 0)) * kMatBytes64;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 2);  // one arrival per warp of the pair
    }
    mbar_fence_init();
  }
  __syncthreads();

  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (warp == 0) {
    for (int j = 0; j < my_items; ++j) {
      const int s = j % stages;
      const uint32_t round = (uint32_t)(j / stages);
      if (!mbar_wait(&empty_bar[s], (round & 1u) ^ 1u, kWaitEmpty)) return;
      const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
      unsigned char* st = smem + (size_t)s * kStageBytes;
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], kTxBytes);
      __syncwarp();
      const float* Ai = A + item * sa;
      const float* Bi = B + item * sb;
      if (A_KMAJOR) {
        for (int r = lane; r < 64; r += 32) bulk_g2s(st + r * kPitch64, Ai + r * 64, 256, &full_bar[s]);
      } else if (lane == 0) {
        bulk_g2s(st, Ai, kMatBytes64, &full_bar[s]);
      }
      if (B_KMAJOR) {
        for (int r = lane; r < 64; r += 32) bulk_g2s(st + kABytes + r * kPitch64, Bi + r * 64, 256, &full_bar[s]);
      } else if (lane == 0) {
        bulk_g2s(st + kABytes, Bi, kMatBytes64, &full_bar[s]);
      }
      if (HAS_C && lane == 0) bulk_g2s(st + kABytes + kBBytes, C + item * sc, kMatBytes64, &full_bar[s]);
    }
    return;
  }

  const int pair = (warp - 1) >> 1, hw = (warp - 1) & 1;
  const int ti = lane & 7, tj = lane >> 3;
  for (int j = pair; j < my_items; j += kPairs64) {
    const int s = j % stages;
    const uint32_t round = (uint32_t)(j / stages);
    if (!mbar_wait(&full_bar[s], round & 1u, kWaitFull)) return;
    const unsigned char* st = smem + (size_t)s * kStageBytes;

    float acc[8][8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;
    mma64<A_KMAJOR, B_KMAJOR>(st, st + kABytes, ti, tj, hw, acc);

    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    float* Cg = C + item * sc;
    const float* Cs = reinterpret_cast<const float*>(st + kABytes + kBBytes);
    // alpha*acc (+ beta*prior from shared memory) in place, then release the stage, then store.
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int col = B_KMAJOR ? (32 * hw + tj + 4 * c) : (32 * hw + 8 * tj + c);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int row = A_KMAJOR ? (ti + 8 * r) : ((r < 4 ? 0 : 32) + 4 * ti + (r & 3));
        float o = alpha * acc[r][c];
        if (HAS_C) o = fmaf(beta, Cs[col * 64 + row], o);
        acc[r][c] = o;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int col = B_KMAJOR ? (32 * hw + tj + 4 * c) : (32 * hw + 8 * tj + c);
      if (A_KMAJOR) {
#pragma unroll
        for (int r = 0; r < 8; ++r) Cg[col * 64 + ti + 8 * r] = acc[r][c];
      } else {
        float4* dst = reinterpret_cast<float4*>(Cg + col * 64);
        dst[ti] = make_float4(acc[0][c], acc[1][c], acc[2][c], acc[3][c]);
        dst[8 + ti] = make_float4(acc[4][c], acc[5][c], acc[6][c], acc[7][c]);
      }
    }
  }
}

template <bool AK, bool BK, bool HC>
int launch64(const GemmParams& p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  constexpr int kStageBytes = (AK ? kPadBytes64 : kMatBytes64) + (BK ? kPadBytes64 : kMatBytes64) + (HC ? kMatBytes64 : 0);
  const size_t budget = dev.smem_optin > 8192 ? dev.smem_optin - 4096 : 0;
  int stages = (int)(budget / (size_t)kStageBytes);
  if (stages > 8) stages = 8;
  if (stages < 2) return BLB200_E_UNSUPPORTED;
  const size_t smem = (size_t)stages * kStageBytes + (size_t)stages * 2 * sizeof(uint64_t);
  auto kern = gemm_small64_kernel<AK, BK, HC>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = p.batch < dev.sm_count ? p.batch : dev.sm_count;
  kern<<<grid, kThreads64, smem, stream>>>((const float*)p.a, (const float*)p.b, (float*)p.c, p.sa, p.sb, p.sc,
                                           p.batch, (float)p.alpha[0], (float)p.beta[0], stages);
  return (int)cudaGetLastError();
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

}  // namespace

bool small32_supported(const GemmParams& p, int dtype) {
  if (dtype != BLB200_S) return false;
  if (p.m != 32 || p.n != 32 || p.k != 32) return false;
  if (p.lda != 32 || p.ldb != 32 || p.ldc != 32) return false;
  if ((p.sa & 3) || (p.sb & 3) || (p.sc & 3)) return false;
  if (p.batch > 1 && p.sc < 1024) return false;  // overlapping outputs: leave to the generic path
  if (!aligned16(p.a) || !aligned16(p.b) || !aligned16(p.c)) return false;
  return true;
}

int launch_small32(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!small32_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const bool ak = p.op_a != BLB200_N;  // op T stores A as k x m: k runs fastest
  const bool bk = p.op_b == BLB200_N;  // op N stores B as k x n: k runs fastest
  const bool hc = (float)p.beta[0] != 0.f;
  int rc;
#define BLB_CASE(a, b)                                                              \
  if (ak == a && bk == b) {                                                         \
    rc = hc ? launch32<a, b, true>(p, stream) : launch32<a, b, false>(p, stream);   \
  } else
  BLB_CASE(false, false) BLB_CASE(false, true) BLB_CASE(true, false) BLB_CASE(true, true) { rc = BLB200_E_INTERNAL; }
#undef BLB_CASE
  if (rc == BLB200_OK) note_launch("small32");
  return rc;
}

bool small64_supported(const GemmParams& p, int dtype) {
  if (dtype != BLB200_S) return false;
  if (p.m != 64 || p.n != 64 || p.k != 64) return false;
  if (p.lda != 64 || p.ldb != 64 || p.ldc != 64) return false;
  if ((p.sa & 3) || (p.sb & 3) || (p.sc & 3)) return false;
  if (p.batch > 1 && p.sc < 4096) return false;
  if (!aligned16(p.a) || !aligned16(p.b) || !aligned16(p.c)) return false;
  return true;
}

int launch_small64(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!small64_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const bool ak = p.op_a != BLB200_N;
  const bool bk = p.op_b == BLB200_N;
  const bool hc = (float)p.beta[0] != 0.f;
  int rc;
#define BLB_CASE(a, b)                                                              \
  if (ak == a && bk == b) {                                                         \
    rc = hc ? launch64<a, b, true>(p, stream) : launch64<a, b, false>(p, stream);   \
  } else
  BLB_CASE(false, false) BLB_CASE(false, true) BLB_CASE(true, false) BLB_CASE(true, true) { rc = BLB200_E_INTERNAL; }
#undef BLB_CASE
  if (rc == BLB200_OK) note_launch("small64");
  return rc;
}

int small_device_status(int* out) { return read_device_status_word(out); }

}  // namespace blb200
