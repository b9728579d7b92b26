// Large float GEMM with A not transposed (op pairs NN and NT): 128 x 128 x 32 CTA tiles, 8 warps as
// 2 (m) x 4 (n), a 64 x 32 warp tile, an 8 x 8 register block per lane accumulated with packed
// FP32 FMA (fma.rn.f32x2), fed by a 3-stage ring of 16-byte asynchronous copies.  This is the shape
// family BatchLAS tunes by hand for float (128x128x8, src/sycl/gemm/register_128x128.hh:69-300) and
// the one its published numbers are for (experiments/sycl_vs_cuda/FINDINGS.md:57-61, 124-131).
//
// Shared-memory layout per stage (32 KiB):
//   A  [32 k][128 m]    rows of 512 bytes.  A lane reads rows 4ti..4ti+3 and 32+4ti..32+4ti+3 of its
//                       warp's 64 rows as two float4 per k: already the row pairs FFMA2 wants.
//   B  op N (K-major in memory): [128 n][32 k], rows of 128 bytes, 16-byte chunk index XORed with
//                       (n & 7) by the copy's destination address; a lane owns columns tj + 4c of its
//                       warp's 32, so the four column groups of a request hit four bank groups and
//                       the eight lanes of a quarter-warp share one address.
//      op T (N-major in memory): [32 k][128 n]; a lane owns columns 8tj..8tj+7 (two float4 per k).
//   B values are duplicated into both halves of a 64-bit register for FFMA2; K-major B fragments
//   are fetched one 4-k chunk ahead.
// Preconditions as for the other tile kernels.  Operands with 16-byte aligned bases and ld, stride
// multiples of 4 elements take 16-byte copies (AL = true); operands that are only float-aligned (a
// slice with an odd offset, ld = 258) are copied one float at a time into the same stage layout and
// C is accessed by scalars (AL = false).  Edges are zero-filled on load and predicated on store;
// beta == 0 never reads C.
#include "common.cuh"
#include "ptx.cuh"

namespace blb200 {
namespace {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, THREADS = 256;
constexpr int A_STAGE = BK * BM * 4, B_STAGE = BK * BN * 4;  // 16 KiB each

// 16 bytes into a stage: one copy, or — when the source is only float-aligned — the widest copies its
// address allows (WIDEST: rows of an M- or N-major tile, where a warp copies one stored column and the
// choice is uniform) or four float copies (K-major rows, whose alignment changes from row to row
// inside a warp).  Chunk-wise measured faster than giving consecutive threads consecutive floats
// (1024^3: 41.8 against 39.7 TFLOP/s).
template <bool AL, bool WIDEST = false>
__device__ __forceinline__ void copy_chunk(unsigned char* dst, const float* src, int valid) {
  if constexpr (AL) {
    cp_async16(dst, src, valid * 4);
  } else if constexpr (WIDEST) {
    cp_async_chunk_widest<4>(dst, reinterpret_cast<const unsigned char*>(src), valid);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) cp_async_elem<4>(dst + 4 * e, e < valid ? src + e : src, e < valid ? 4 : 0);
  }
}

// A tile: 32 k-rows x 32 chunks of 4 rows.
template <bool AL>
__device__ __forceinline__ void load_a(unsigned char* dst, const float* __restrict__ A, long long lda, int m0, int M,
                                       int k0, int K, int tid) {
#pragma unroll
  for (int c = tid; c < BK * (BM / 4); c += THREADS) {
    const int kk = c >> 5, mc = c & 31;
    const int gk = k0 + kk, gm = m0 + mc * 4;
    int valid = (gk < K) ? (M - gm) : 0;
    valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
    const float* src = valid ? A + (long long)gk * lda + gm : A;
    copy_chunk<AL, true>(dst + kk * (BM * 4) + mc * 16, src, valid);
  }
}

// B tile.  KMAJOR (op N): 128 columns x 8 chunks of 4 k, swizzled; else (op T): 32 k-rows x 32 chunks of 4 columns.
template <bool KMAJOR, bool AL>
__device__ __forceinline__ void load_b(unsigned char* dst, const float* __restrict__ B, long long ldb, int n0, int N,
                                       int k0, int K, int tid) {
  if (KMAJOR) {
#pragma unroll
    for (int c = tid; c < BN * (BK / 4); c += THREADS) {
      const int j = c >> 3, kc = c & 7;
      const int gn = n0 + j, gk = k0 + kc * 4;
      int valid = (gn < N) ? (K - gk) : 0;
      valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
      const float* src = valid ? B + (long long)gn * ldb + gk : B;
      copy_chunk<AL>(dst + j * 128 + ((kc ^ (j & 7)) * 16), src, valid);
    }
  } else {
#pragma unroll
    for (int c = tid; c < BK * (BN / 4); c += THREADS) {
      const int kk = c >> 5, nc = c & 31;
      const int gk = k0 + kk, gn = n0 + nc * 4;
      int valid = (gk < K) ? (N - gn) : 0;
      valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
      const float* src = valid ? B + (long long)gk * ldb + gn : B;
      copy_chunk<AL, true>(dst + kk * (BN * 4) + nc * 16, src, valid);
    }
  }
}

// HINTS = false is the plain gemm; HINTS = true reads the structure hints of GemmParams (a separate
// instantiation, so that the plain kernel's code and register allocation stay what they were).
template <bool B_KMAJOR, bool HINTS, bool AL = true>
__global__ void __launch_bounds__(THREADS, 2) sgemm128_kernel(GemmParams p, int tiles_m, int tiles_n) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* As = smem;
  unsigned char* Bs = smem + STAGES * A_STAGE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 1, wn = warp >> 1;
  const int ti = lane & 7, tj = lane >> 3;

  const long long tiles_per_item = (long long)tiles_m * tiles_n;
  const long long tile = blockIdx.x;
  const long long vitem = tile / tiles_per_item;
  const int rem = (int)(tile - vitem * tiles_per_item);
  const SplitView sv = resolve_split(p, vitem);
  int K = sv.k;
  const int m0 = (rem % tiles_m) * BM, n0 = (rem / tiles_m) * BN;
  const float* A = (const float*)p.a + sv.item * p.sa + sv.a_off;
  const float* B = (const float*)p.b + sv.item * p.sb + sv.b_off;
  float* C = (float*)p.c + vitem * p.sc;
  if constexpr (HINTS) {  // per-item dims; triangular operand: shorter k range; triangular output: maybe nothing
    p.m = item_dim(p.het_m, sv.item, p.m);
    p.n = item_dim(p.het_n, sv.item, p.n);
    K = item_dim(p.het_k, sv.item, K);
    if (m0 >= p.m || n0 >= p.n) return;
    const TileWork w = tile_work(p, K, m0, BM, n0, BN, BK);
    if (w.skip) return;
    A += a_k_offset(p, w.k_lo);
    B += b_k_offset(p, w.k_lo);
    K = w.k_hi - w.k_lo;
  }

  uint64_t accp[32];  // [row pair rp][col c]: rows (2rp, 2rp+1) of the lane's 8, column c of its 8
#pragma unroll
  for (int i = 0; i < 32; ++i) accp[i] = 0ull;

  const int KT = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) {
      load_a<AL>(As + s * A_STAGE, A, p.lda, m0, p.m, s * BK, K, tid);
      load_b<B_KMAJOR, AL>(Bs + s * B_STAGE, B, p.ldb, n0, p.n, s * BK, K, tid);
    }
    cp_async_commit();
  }
  if (!HINTS && p.beta[0] != 0.0) {  // the epilogue reads this tile of C: ask L2 for it now (two threads per column, 128-byte lines)
    const int col = n0 + (tid >> 1), r0 = m0 + 64 * (tid & 1);
    if (col < p.n && r0 < p.m) {
      const float* pc = C + (long long)col * p.ldc + r0;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(pc));
      if (r0 + 32 < p.m) asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + 32));
    }
  }

  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = kt + STAGES - 1;
      if (nxt < KT) {
        const int s = nxt % STAGES;
        load_a<AL>(As + s * A_STAGE, A, p.lda, m0, p.m, nxt * BK, K, tid);
        load_b<B_KMAJOR, AL>(Bs + s * B_STAGE, B, p.ldb, n0, p.n, nxt * BK, K, tid);
      }
      cp_async_commit();
    }
    const ulonglong2* As2 = reinterpret_cast<const ulonglong2*>(As + (kt % STAGES) * A_STAGE) + wm * 16 + ti;
    const float4* Bs4 = reinterpret_cast<const float4*>(Bs + (kt % STAGES) * B_STAGE);

    if (B_KMAJOR) {
      float bf[2][8][4];  // [buffer][col][kk]
      auto load_bf = [&](int kc, float (&dst)[8][4]) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int j = wn * 32 + tj + 4 * c;
          const float4 v = Bs4[j * 8 + (kc ^ (j & 7))];
          dst[c][0] = v.x; dst[c][1] = v.y; dst[c][2] = v.z; dst[c][3] = v.w;
        }
      };
      load_bf(0, bf[0]);
#pragma unroll
      for (int kc = 0; kc < BK / 4; ++kc) {
        if (kc + 1 < BK / 4) load_bf(kc + 1, bf[(kc + 1) & 1]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const ulonglong2 lo = As2[(4 * kc + kk) * 32];
          const ulonglong2 hi = As2[(4 * kc + kk) * 32 + 8];
          const uint64_t a2[4] = {lo.x, lo.y, hi.x, hi.y};
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint64_t bd = dup2(bf[kc & 1][c][kk]);
#pragma unroll
            for (int rp = 0; rp < 4; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
          }
        }
      }
    } else {
#pragma unroll 8
      for (int k = 0; k < BK; ++k) {
        const ulonglong2 lo = As2[k * 32];
        const ulonglong2 hi = As2[k * 32 + 8];
        const float4 v0 = Bs4[k * 32 + wn * 8 + 2 * tj];
        const float4 v1 = Bs4[k * 32 + wn * 8 + 2 * tj + 1];
        const uint64_t a2[4] = {lo.x, lo.y, hi.x, hi.y};
        const float bv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint64_t bd = dup2(bv[c]);
#pragma unroll
          for (int rp = 0; rp < 4; ++rp) ffma2(accp[rp * 8 + c], a2[rp], bd);
        }
      }
    }
  }
  cp_async_wait<0>();

  const float alpha = (float)p.alpha[0], beta = (float)p.beta[0];
  const bool beta_zero = beta == 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int col = n0 + wn * 32 + (B_KMAJOR ? (tj + 4 * c) : (8 * tj + c));
    if (col >= p.n) continue;
    float* ccol = C + (long long)col * p.ldc;
#pragma unroll
    for (int hgh = 0; hgh < 2; ++hgh) {
      const int row = m0 + wm * 64 + 32 * hgh + 4 * ti;
      float o[4];
      unpack2(accp[(2 * hgh) * 8 + c], o[0], o[1]);
      unpack2(accp[(2 * hgh + 1) * 8 + c], o[2], o[3]);
      // with a triangular output the vector store is used only strictly inside the wanted triangle
      const bool whole = !HINTS || p.out_tri == 0 || (p.out_tri == 1 ? row >= col : row + 3 <= col);
      if (AL && row + 4 <= p.m && whole) {
        float4 out = make_float4(alpha * o[0], alpha * o[1], alpha * o[2], alpha * o[3]);
        if (!beta_zero) {
          const float4 pr = *reinterpret_cast<const float4*>(ccol + row);
          out.x = fmaf(beta, pr.x, out.x);
          out.y = fmaf(beta, pr.y, out.y);
          out.z = fmaf(beta, pr.z, out.z);
          out.w = fmaf(beta, pr.w, out.w);
        }
        *reinterpret_cast<float4*>(ccol + row) = out;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (row + e < p.m && !(HINTS && out_masked(p, row + e, col))) {
            float out = alpha * o[e];
            if (!beta_zero) out = fmaf(beta, ccol[row + e], out);
            ccol[row + e] = out;
          }
      }
    }
  }
}

template <bool B_KMAJOR, bool HINTS, bool AL = true>
int launch_one(const GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (A_STAGE + B_STAGE);
  const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
  const long long total = (long long)tiles_m * tiles_n * p.batch;
  if (total > 0x7fffffffLL) return BLB200_E_UNSUPPORTED;
  auto kern = sgemm128_kernel<B_KMAJOR, HINTS, AL>;
  static thread_local int configured_for = -1;
  int cur = 0;
  cudaGetDevice(&cur);
  if (configured_for != cur) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_for = cur;
  }
  kern<<<(unsigned)total, THREADS, smem, stream>>>(p, tiles_m, tiles_n);
  return (int)cudaGetLastError();
}

}  // namespace

bool sgemm128_supported(const GemmParams& p, int dtype) {
  if (dtype != BLB200_S || p.op_a != BLB200_N) return false;
  if (p.m < 64 || p.n < 64) return false;  // smaller outputs waste most of a 128 x 128 tile
  return tiled_supported(p, dtype);
}

// Whether the dispatcher should pick this kernel over the 64 x 64 tiles of the tiled kernel: it is
// about a quarter faster per multiply-add it performs (45 against 36 TFLOP/s on full tiles), so it
// wins as long as rounding m and n up to 128 does not add more than that in padding.
bool sgemm128_preferred(const GemmParams& p) {
  auto tiles = [](int x, int t) { return (long long)((x + t - 1) / t); };
  const long long w128 = tiles(p.m, 128) * tiles(p.n, 128) * 128 * 128, w64 = tiles(p.m, 64) * tiles(p.n, 64) * 64 * 64;
  return 4 * w128 <= 5 * w64;
}

int launch_sgemm128(const GemmParams& p, int dtype, cudaStream_t stream) {
  if (!sgemm128_supported(p, dtype)) return BLB200_E_UNSUPPORTED;
  const bool hints = has_hints(p);
  if (!operands_aligned_to(p, 4, 16)) {  // float-aligned operands (plain gemm only: tiled_supported saw to that)
    if (hints || p.splits > 1) return BLB200_E_UNSUPPORTED;
    const int rc_el = (p.op_b == BLB200_N) ? launch_one<true, false, false>(p, stream) : launch_one<false, false, false>(p, stream);
    if (rc_el == BLB200_OK) note_launch("sgemm128");
    return rc_el;
  }
  const int rc = (p.op_b == BLB200_N) ? (hints ? launch_one<true, true>(p, stream) : launch_one<true, false>(p, stream))
                                      : (hints ? launch_one<false, true>(p, stream) : launch_one<false, false>(p, stream));
  if (rc == BLB200_OK) note_launch("sgemm128");
  return rc;
}

}  // namespace blb200
