// Whole-matrix-per-warp kernels for packed small float matrices: the HBM-bound end of the family.
//
// Shared structure.  A persistent grid of one CTA per SM walks the batch round-robin through a ring
// of shared-memory slots filled by TMA copies that complete on one "full" mbarrier per slot.  There
// is no producer warp and no "empty" barrier: a slot belongs to one warp (small32) or one warp pair
// (small64) for the whole launch, and the owner itself issues the copies of the item that uses the
// slot next, the moment it has read the slot.  (One thread issuing every copy of an SM is latency
// bound at about 4 KiB per 250 ns, well under HBM speed; a producer warp with one lane per slot
// removes that cap but its lanes wait in one diverged warp, and a lane parked in a blocking barrier
// wait delays the other slots' refills.)  Because a slot always has the same owner, a consumer
// never waits for round r of a slot before round r-1 has completed, which is what makes the one-bit
// mbarrier phase parity sufficient.
//
// small32: m = n = k = 32, ld = 32 on all three operands, 16-byte aligned bases, strides multiples
// of 4 elements (BatchLAS gates its own vector fast paths the same way:
// src/sycl/gemm/load_policies.hh:18-34).  Each 4 KiB matrix is one contiguous run, fetched by one
// untiled bulk copy per operand.  One consumer warp per matrix; a lane keeps a 4 x 8 block of C
// (rows 4ti..4ti+3, columns 8tj..8tj+7; ti = lane & 7, tj = lane >> 3), reads 128-bit fragments
// from shared memory and writes C with 128-bit stores (8 lanes cover one 128-byte column).
// Operand orientation only changes how fragments are read; nothing is transposed in memory:
//   M-major A (op N): float4 = 4 rows at one k.        K-major A (op T): float4 = 4 k at one row.
//   N-major B (op T): float4 = 4 cols at one k.        K-major B (op N): float4 = 4 k at one col.
// With a K-major operand, lanes walk the eight 4-wide k-chunks in a lane-dependent rotation so that
// the lanes of one request fall into different 16-byte bank groups; the sum over k is the same
// set of products in a different order.
//
// small64: m = n = k = 64, ld = 64, same alignment rules.  Two warps share one matrix
// (warp half hw owns columns 32hw..32hw+31, each lane an 8 x 8 block: 16 fragment floats per 64
// FMAs, so the FP32 pipe rather than shared memory sets the pace).  The ring holds half-K slots of
// 16 KiB (A half + B half); each of the 6 pairs owns 2 slots.  An M-major / N-major half is one
// contiguous 8 KiB run (untiled bulk copy).  A K-major half is 64 rows of 128 bytes, 256 bytes
// apart in memory: it is fetched by one tiled TMA copy (cp.async.bulk.tensor.3d, box 32 x 64 x 1)
// with the 128-byte swizzle, which XORs the 16-byte chunk index with (row & 7); with rows (or
// columns) dealt to lanes round-robin, every fragment request then touches each bank group once.
//
// Algorithmic traffic per item: A + B (+ C when beta != 0) read and C written.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tensor_map.cuh"

namespace blb200 {
namespace {

enum WaitCode { kWaitFull = 101 };

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// =================================================================================================
// small32
// =================================================================================================
constexpr int kMatBytes32 = 32 * 32 * 4;

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

// Shared memory: `stages` x {A, B[, C]} of 4 KiB each, then full[stages] barriers.
// `stages` is a multiple of the warp count CW; stage s belongs to warp s % CW for the whole launch.
// There is no producer warp: lane 0 of the warp that owns a stage issues the copies of the item
// that uses the stage next as soon as the warp has read its fragments, so a refill never waits for
// a hand-over that another warp has to notice.
// TRANS_OUT: the lane's 4 x 8 block is a block of C^T (used for op pair TT, which is computed as
// C^T = B_stored * A_stored with the operands swapped by the launcher, i.e. through the NN fragment
// path); the epilogue then writes row 8tj..8tj+7 of column 4ti+r as two float4.
template <int CW, bool A_KMAJOR, bool B_KMAJOR, bool HAS_C, bool TRANS_OUT = false>
__global__ void __launch_bounds__(32 * CW, 1)
    gemm_small32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                        long long sa, long long sb, long long sc, int batch, float alpha, float beta,
                        int stages) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kStageBytes = (HAS_C ? 3 : 2) * kMatBytes32;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // Items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; the j-th one uses stage j % stages.
  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  auto issue = [&](int stage, int jj) {
    unsigned char* st = smem + (size_t)stage * kStageBytes;
    const long long it = (long long)blockIdx.x + (long long)jj * gridDim.x;
    mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
    bulk_g2s(st, A + it * sa, kMatBytes32, &full_bar[stage]);
    bulk_g2s(st + kMatBytes32, B + it * sb, kMatBytes32, &full_bar[stage]);
    if (HAS_C) bulk_g2s(st + 2 * kMatBytes32, C + it * sc, kMatBytes32, &full_bar[stage]);
  };

  const int cw = warp;
  const int ti = lane & 7, tj = lane >> 3;
  if (lane == 0)
    for (int stage = cw; stage < stages && stage < my_items; stage += CW) issue(stage, stage);
  int s = cw;          // stage of this warp's current item: (cw + CW*i) % stages
  uint32_t round = 0;  // how many times this warp has been through stage `s` before
  for (int j = cw; j < my_items; j += CW) {
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
      for (int c = 0; c < 8; ++c)
        prior[c] = TRANS_OUT ? Cs4[(4 * ti + (c >> 1)) * 8 + 2 * tj + (c & 1)] : Cs4[(8 * tj + c) * 8 + ti];
    }
    __syncwarp();
    if (lane == 0 && j + stages < my_items) {  // the stage is refilled while we store
      fence_async_smem();
      issue(s, j + stages);
    }

    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    float4* Cg4 = reinterpret_cast<float4*>(C + item * sc);
    if (TRANS_OUT) {
      // acc[r][c] = C(8tj + c, 4ti + r): column 4ti+r, rows 8tj..8tj+7 -> float4 index col*8 + 2tj + half
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          float4 o;
          o.x = alpha * acc[r][4 * hf + 0];
          o.y = alpha * acc[r][4 * hf + 1];
          o.z = alpha * acc[r][4 * hf + 2];
          o.w = alpha * acc[r][4 * hf + 3];
          if (HAS_C) {
            const float4 pr = prior[2 * r + hf];
            o.x = fmaf(beta, pr.x, o.x);
            o.y = fmaf(beta, pr.y, o.y);
            o.z = fmaf(beta, pr.z, o.z);
            o.w = fmaf(beta, pr.w, o.w);
          }
          Cg4[(4 * ti + r) * 8 + 2 * tj + hf] = o;
        }
    } else
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
    s += CW;
    if (s >= stages) {
      s -= stages;
      ++round;
    }
  }
}

template <int CW, bool AK, bool BK, bool HC, bool TRANS_OUT = false>
int launch32(const GemmParams& p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  constexpr int kStageBytes = (HC ? 3 : 2) * kMatBytes32;
  constexpr int stages = CW;  // one stage per warp: 16 x 12 KiB in flight per SM
  const size_t smem = (size_t)stages * kStageBytes + (size_t)stages * sizeof(uint64_t);
  if (dev.smem_optin < smem) return BLB200_E_UNSUPPORTED;
  auto kern = gemm_small32_kernel<CW, AK, BK, HC, TRANS_OUT>;
  static thread_local int configured_for = -1;  // per (instantiation, thread): device last configured
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = p.batch < dev.sm_count ? p.batch : dev.sm_count;
  kern<<<grid, 32 * CW, smem, stream>>>((const float*)p.a, (const float*)p.b, (float*)p.c, p.sa, p.sb, p.sc, p.batch,
                                     (float)p.alpha[0], (float)p.beta[0], stages);
  return (int)cudaGetLastError();
}

// =================================================================================================
// small64
// =================================================================================================
constexpr int kSlots64 = 12;  // half-K slots; PAIRS warp pairs own kSlots64 / PAIRS of them each
constexpr int kHalfBytes64 = 32 * 64 * 4;             // one operand, half of K: 8 KiB
constexpr int kSlotBytes64 = 2 * kHalfBytes64;        // A half + B half
constexpr int kMatElems64 = 64 * 64;

// How the 64 accumulators of a lane are paired for FFMA2.  Pairs must be adjacent in the operand
// that shared memory delivers as float4 along the output dimension:
//   kRowPairs  A M-major: a float4 holds 4 consecutive rows  -> acc pairs (row 2p, 2p+1), B value duplicated
//   kColPairs  A K-major, B N-major: a float4 holds 4 consecutive columns -> pairs (col 2p, 2p+1), A duplicated
//   kScalar    both K-major: no operand is contiguous along an output dimension; plain FFMA
enum PackMode { kScalar = 0, kRowPairs = 1, kColPairs = 2 };
template <bool A_KMAJOR, bool B_KMAJOR>
__host__ __device__ constexpr PackMode pack_mode() {
  return !A_KMAJOR ? kRowPairs : (!B_KMAJOR ? kColPairs : kScalar);
}

// One half-K (32 k) of the product for this lane's 8 x 8 block.  `acc` is float[8][8] in scalar
// mode; in the packed modes the same 64 registers are addressed as uint64_t[32].
template <bool A_KMAJOR, bool B_KMAJOR>
__device__ __forceinline__ void mma64_half(const unsigned char* __restrict__ As, const unsigned char* __restrict__ Bs,
                                           int ti, int tj, int hw, float (&acc)[8][8], uint64_t (&accp)[32]) {
  constexpr PackMode PM = pack_mode<A_KMAJOR, B_KMAJOR>();
  const float4* As4 = reinterpret_cast<const float4*>(As);
  const float4* Bs4 = reinterpret_cast<const float4*>(Bs);
  const ulonglong2* As2 = reinterpret_cast<const ulonglong2*>(As);
  const ulonglong2* Bs2 = reinterpret_cast<const ulonglong2*>(Bs);
  if constexpr (PM == kRowPairs && B_KMAJOR) {
    // B fragments for a whole 4-k chunk come from 8 swizzled loads; they are fetched one chunk
    // ahead (two register buffers) so that their latency hides behind the previous chunk's FMAs.
    float bf[2][8][4];  // [buffer][col][kk]; column j = 32hw + tj + 4c
    auto load_b = [&](int kc, float (&dst)[8][4]) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int j = 32 * hw + tj + 4 * c;
        const float4 v = Bs4[j * 8 + (kc ^ (j & 7))];
        dst[c][0] = v.x; dst[c][1] = v.y; dst[c][2] = v.z; dst[c][3] = v.w;
      }
    };
    load_b(0, bf[0]);
#pragma unroll
    for (int kc = 0; kc < 8; ++kc) {
      if (kc + 1 < 8) load_b(kc + 1, bf[(kc + 1) & 1]);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const ulonglong2 lo = As2[(4 * kc + kk) * 16 + ti];
        const ulonglong2 hi = As2[(4 * kc + kk) * 16 + 8 + ti];
        const uint64_t a2[4] = {lo.x, lo.y, hi.x, hi.y};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint64_t bd = dup2(bf[kc & 1][c][kk]);
#pragma unroll
          for (int rp = 0; rp < 4; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
        }
      }
    }
    return;
  }
#pragma unroll 2
  for (int kc = 0; kc < 8; ++kc) {
    if constexpr (PM == kRowPairs) {
      float bf[8][4];  // [col][kk], k-rows of 256 bytes: columns 32hw + 8tj + c
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 v0 = Bs4[(4 * kc + kk) * 16 + 8 * hw + 2 * tj];
        const float4 v1 = Bs4[(4 * kc + kk) * 16 + 8 * hw + 2 * tj + 1];
        bf[0][kk] = v0.x; bf[1][kk] = v0.y; bf[2][kk] = v0.z; bf[3][kk] = v0.w;
        bf[4][kk] = v1.x; bf[5][kk] = v1.y; bf[6][kk] = v1.z; bf[7][kk] = v1.w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        // rows 4ti..4ti+3 and 32+4ti..32+4ti+3 as four row pairs
        const ulonglong2 lo = As2[(4 * kc + kk) * 16 + ti];
        const ulonglong2 hi = As2[(4 * kc + kk) * 16 + 8 + ti];
        const uint64_t a2[4] = {lo.x, lo.y, hi.x, hi.y};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint64_t bd = dup2(bf[c][kk]);
#pragma unroll
          for (int rp = 0; rp < 4; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
        }
      }
    } else if constexpr (PM == kColPairs) {
      float af[8][4];  // [row][kk], swizzled rows ti + 8r
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 v = As4[(ti + 8 * r) * 8 + (kc ^ ti)];
        af[r][0] = v.x; af[r][1] = v.y; af[r][2] = v.z; af[r][3] = v.w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const ulonglong2 v0 = Bs2[(4 * kc + kk) * 16 + 8 * hw + 2 * tj];
        const ulonglong2 v1 = Bs2[(4 * kc + kk) * 16 + 8 * hw + 2 * tj + 1];
        const uint64_t b2[4] = {v0.x, v0.y, v1.x, v1.y};  // column pairs (8tj+0,1) (2,3) (4,5) (6,7)
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const uint64_t ad = dup2(af[r][kk]);
#pragma unroll
          for (int cp = 0; cp < 4; ++cp) ffma2(accp[r * 4 + cp], ad, b2[cp]);
        }
      }
    } else {
      float af[8][4], bf[8][4];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 v = As4[(ti + 8 * r) * 8 + (kc ^ ti)];
        af[r][0] = v.x; af[r][1] = v.y; af[r][2] = v.z; af[r][3] = v.w;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int j = 32 * hw + tj + 4 * c;
        const float4 v = Bs4[j * 8 + (kc ^ (j & 7))];
        bf[c][0] = v.x; bf[c][1] = v.y; bf[c][2] = v.z; bf[c][3] = v.w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(af[r][kk], bf[c][kk], acc[r][c]);
    }
  }
}

// L2 prefetch hint for an untiled run (tensor_map.cuh has the one for a box of a tensor map).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// Pair p's q-th half-item lives in slot p * SPP + q % SPP (round q / SPP; SPP = slots per pair);
// half-item q is half q & 1 of the pair's (q >> 1)-th item.  There is no producer warp: the two
// warps of a pair count themselves off a slot, and the one that leaves it last issues the copies of
// the half-item that uses the slot next — the refill starts the moment the slot is free, with no
// hand-over that a third warp has to notice.
template <int PAIRS, bool A_KMAJOR, bool B_KMAJOR, bool HAS_C>
__global__ void __launch_bounds__(64 * PAIRS, 1)
    gemm_small64_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                        long long sa, long long sb, long long sc, int batch, float alpha, float beta,
                        const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b) {
  constexpr int kPairs64 = PAIRS, kSlotsPerPair64 = kSlots64 / PAIRS;
  static_assert(kSlots64 % PAIRS == 0 && kSlotsPerPair64 >= 2, "every pair owns the same number (>= 2) of slots");
  extern __shared__ unsigned char smem_raw[];
  // the 128-byte swizzle is a function of the shared-memory address: slots must be 1024-byte aligned
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kSlots64 * kSlotBytes64);
  uint32_t* left = reinterpret_cast<uint32_t*>(full_bar + kSlots64);  // per slot: warps that have left it, ever

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots64; ++s) {
      mbar_init(&full_bar[s], 1);
      left[s] = 0u;
    }
    mbar_fence_init();
  }
  __syncthreads();

  const int my_items = (batch > (int)blockIdx.x) ? (batch - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  // Programmatic dependent launch: let the next kernel in the stream place its CTAs on SMs as this
  // grid drains (its barrier set-up then overlaps our tail); no thread touches global memory
  // (operand copies, the old C, the C stores) before every earlier grid in the stream has finished.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int pair = warp >> 1, hw = warp & 1;
  const int ti = lane & 7, tj = lane >> 3;
  // items of this pair: pair, pair + PAIRS, ...
  const int pair_items = (my_items > pair) ? (my_items - 1 - pair) / kPairs64 + 1 : 0;
  const int pair_halves = 2 * pair_items;

  // While the earlier grid is still running: ask for the pair's first half-items to be brought into
  // L2.  A prefetch changes nothing that a program can observe (L2 is the point of coherence: a line
  // that the earlier grid writes afterwards is simply updated there), so it may come before the
  // dependency wait; the real copies then start from L2 instead of HBM.
  if (hw == 0 && lane == 0)
    for (int q = 0; q < kSlotsPerPair64 && q < pair_halves; ++q) {
      const int j = pair + (q >> 1) * kPairs64, half = q & 1;
      const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
      if (A_KMAJOR) tma_prefetch_3d(&map_a, 32 * half, 0, (int)item);
      else bulk_prefetch_l2(A + item * sa + half * (kMatElems64 / 2), kHalfBytes64);
      if (B_KMAJOR) tma_prefetch_3d(&map_b, 32 * half, 0, (int)item);
      else bulk_prefetch_l2(B + item * sb + half * (kMatElems64 / 2), kHalfBytes64);
    }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  auto issue = [&](int q, int slot_of_pair) {
    const int s = pair * kSlotsPerPair64 + slot_of_pair;
    unsigned char* st = smem + (size_t)s * kSlotBytes64;
    const int j = pair + (q >> 1) * kPairs64, half = q & 1;
    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    mbar_arrive_expect_tx(&full_bar[s], kSlotBytes64);
    if (A_KMAJOR) tma_load_3d(st, &map_a, 32 * half, 0, (int)item, &full_bar[s]);
    else bulk_g2s(st, A + item * sa + half * (kMatElems64 / 2), kHalfBytes64, &full_bar[s]);
    if (B_KMAJOR) tma_load_3d(st + kHalfBytes64, &map_b, 32 * half, 0, (int)item, &full_bar[s]);
    else bulk_g2s(st + kHalfBytes64, B + item * sb + half * (kMatElems64 / 2), kHalfBytes64, &full_bar[s]);
  };
  if (hw == 0 && lane == 0)
    for (int q = 0; q < kSlotsPerPair64 && q < pair_halves; ++q) issue(q, q);

  int slot_i = 0;      // q % SPP
  uint32_t round = 0;  // q / SPP
  int q = 0;
  for (int j = pair; j < my_items; j += kPairs64) {
    constexpr PackMode PM = pack_mode<A_KMAJOR, B_KMAJOR>();
    float acc[8][8];
    uint64_t accp[32];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) accp[i] = 0ull;
#pragma unroll 1
    for (int half = 0; half < 2; ++half, ++q) {
      const int s = pair * kSlotsPerPair64 + slot_i;
      if (!mbar_wait(&full_bar[s], round & 1u, kWaitFull)) return;
      const unsigned char* st = smem + (size_t)s * kSlotBytes64;
      mma64_half<A_KMAJOR, B_KMAJOR>(st, st + kHalfBytes64, ti, tj, hw, acc, accp);
      __syncwarp();
      if (lane == 0) {
        const uint32_t before = smem_add_acq_rel(&left[s], 1u);
        if ((before & 1u) && q + kSlotsPerPair64 < pair_halves) {  // the pair's other warp left earlier
          fence_async_smem();
          issue(q + kSlotsPerPair64, slot_i);
        }
      }
      if (++slot_i == kSlotsPerPair64) {
        slot_i = 0;
        ++round;
      }
    }

    if constexpr (PM != kScalar) {
      // alpha is applied to the packed accumulators (32 packed multiplies, none when alpha == 1)
      if (alpha != 1.f) {
        const uint64_t al2 = dup2(alpha);
#pragma unroll
        for (int i = 0; i < 32; ++i) asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(accp[i]) : "l"(al2));
      }
    }
    if constexpr (PM == kRowPairs) {
#pragma unroll
      for (int rp = 0; rp < 4; ++rp)
#pragma unroll
        for (int c = 0; c < 8; ++c) unpack2(accp[rp * 8 + c], acc[2 * rp][c], acc[2 * rp + 1][c]);
    } else if constexpr (PM == kColPairs) {
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) unpack2(accp[r * 4 + cp], acc[r][2 * cp], acc[r][2 * cp + 1]);
    }

    const long long item = (long long)blockIdx.x + (long long)j * gridDim.x;
    float* Cg = C + item * sc;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int col = B_KMAJOR ? (32 * hw + tj + 4 * c) : (32 * hw + 8 * tj + c);
      if (A_KMAJOR) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          float* dst = Cg + col * 64 + ti + 8 * r;
          float o = (PM == kScalar) ? alpha * acc[r][c] : acc[r][c];
          if (HAS_C) o = fmaf(beta, *dst, o);
          *dst = o;
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(Cg + col * 64);
#pragma unroll
        for (int hgh = 0; hgh < 2; ++hgh) {
          float4 o = make_float4(acc[4 * hgh][c], acc[4 * hgh + 1][c], acc[4 * hgh + 2][c], acc[4 * hgh + 3][c]);
          if (PM == kScalar) {
            o.x *= alpha; o.y *= alpha; o.z *= alpha; o.w *= alpha;
          }
          if (HAS_C) {
            const float4 pr = dst[8 * hgh + ti];
            o.x = fmaf(beta, pr.x, o.x);
            o.y = fmaf(beta, pr.y, o.y);
            o.z = fmaf(beta, pr.z, o.z);
            o.w = fmaf(beta, pr.w, o.w);
          }
          dst[8 * hgh + ti] = o;
        }
      }
    }
  }
}

// 3-D map over `batch` K-major 64 x 64 float matrices: dims (k, row, item), box 32 x 64 x 1,
// 128-byte swizzle.
int make_kmajor_map64(CUtensorMap* map, const float* base, long long stride_elems, int batch) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return BLB200_E_INTERNAL;
  const cuuint64_t dims[3] = {64, 64, (cuuint64_t)(batch > 0 ? batch : 1)};
  const cuuint64_t strides[2] = {64 * sizeof(float), (cuuint64_t)stride_elems * sizeof(float)};
  const cuuint32_t box[3] = {32, 64, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BLB200_OK : BLB200_E_INTERNAL;
}

// Tensor maps are pure functions of (base, item stride, batch): a small per-thread cache saves the
// driver call on repeated launches over the same operand (a solver loop, a benchmark).
struct MapCache64 {
  struct Entry {
    const void* base = nullptr;
    long long stride = 0;
    int batch = 0;
    bool valid = false;
    alignas(64) CUtensorMap map;
  };
  static constexpr int kEntries = 8;
  Entry e[kEntries];
  int next = 0;
  int get(CUtensorMap* out, const float* base, long long stride, int batch) {
    for (int i = 0; i < kEntries; ++i)
      if (e[i].valid && e[i].base == base && e[i].stride == stride && e[i].batch == batch) {
        memcpy(out, &e[i].map, sizeof(CUtensorMap));
        return BLB200_OK;
      }
    Entry& slot = e[next];
    next = (next + 1) % kEntries;
    slot.valid = false;
    const int rc = make_kmajor_map64(&slot.map, base, stride, batch);
    if (rc != BLB200_OK) return rc;
    slot.base = base;
    slot.stride = stride;
    slot.batch = batch;
    slot.valid = true;
    memcpy(out, &slot.map, sizeof(CUtensorMap));
    return BLB200_OK;
  }
};

template <int PAIRS, bool AK, bool BK, bool HC>
int launch64(const GemmParams& p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  const size_t smem = (size_t)kSlots64 * kSlotBytes64 + (size_t)kSlots64 * (sizeof(uint64_t) + sizeof(uint32_t)) + 1024;
  if (dev.smem_optin < smem) return BLB200_E_UNSUPPORTED;
  alignas(64) CUtensorMap map_a, map_b;
  memset(&map_a, 0, sizeof(map_a));
  memset(&map_b, 0, sizeof(map_b));
  static thread_local MapCache64 maps;
  if (AK) {
    int rc = maps.get(&map_a, (const float*)p.a, p.batch > 1 ? p.sa : kMatElems64, p.batch);
    if (rc != BLB200_OK) return rc;
  }
  if (BK) {
    int rc = maps.get(&map_b, (const float*)p.b, p.batch > 1 ? p.sb : kMatElems64, p.batch);
    if (rc != BLB200_OK) return rc;
  }
  auto kern = gemm_small64_kernel<PAIRS, AK, BK, HC>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  const int grid = p.batch < dev.sm_count ? p.batch : dev.sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(64 * PAIRS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, (const float*)p.a, (const float*)p.b, (float*)p.c, (long long)p.sa,
                                 (long long)p.sb, (long long)p.sc, p.batch, (float)p.alpha[0], (float)p.beta[0], map_a,
                                 map_b);
}

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
  if (ak && !bk) {
    // TT: C^T = B_stored * A_stored.  B (n x k, column-major) plays the M-major left operand, A (k x m)
    // the K-major right operand; the kernel writes its block transposed.
    GemmParams q = p;
    q.a = p.b; q.b = p.a;
    q.sa = p.sb; q.sb = p.sa;
    rc = hc ? launch32<16, false, true, true, true>(q, stream) : launch32<16, false, true, false, true>(q, stream);
    if (rc == BLB200_OK) note_launch("small32");
    return rc;
  }
#define BLB_CASE(a, b) \
  if (ak == a && bk == b) rc = hc ? launch32<16, a, b, true>(p, stream) : launch32<16, a, b, false>(p, stream); else
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
  if (p.batch > 1 && p.sc < kMatElems64) return false;
  // a tensor map needs a positive item stride; a broadcast operand (stride 0) takes the tiled path
  if (p.batch > 1 && (p.sa < kMatElems64 || p.sb < kMatElems64)) return false;
  if (!aligned16(p.a) || !aligned16(p.b) || !aligned16(p.c)) return false;
  return encode_tiled_fn() != nullptr;
}

int launch_small64(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!small64_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const bool ak = p.op_a != BLB200_N;
  const bool bk = p.op_b == BLB200_N;
  const bool hc = (float)p.beta[0] != 0.f;
  // Six warp pairs (three warps per scheduler) with two slots each: 52.1 TFLOP/s on 10 000 items
  // (NT 55.3) against 50.8 (51.9) for four pairs with three slots each.
  int rc;
#define BLB_CASE(a, b) \
  if (ak == a && bk == b) rc = hc ? launch64<6, a, b, true>(p, stream) : launch64<6, a, b, false>(p, stream); else
  BLB_CASE(false, false) BLB_CASE(false, true) BLB_CASE(true, false) BLB_CASE(true, true) { rc = BLB200_E_INTERNAL; }
#undef BLB_CASE
  if (rc == BLB200_OK) note_launch("small64");
  return rc;
}

int small_device_status(int* out) { return read_device_status_word(out); }
int small_device_status_clear() { return clear_device_status_word(); }

}  // namespace blb200
