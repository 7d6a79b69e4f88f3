// Batched BF16 x rowwise-MXFP8 matrix product for the MLA absorb projections:
//   C[b] (M x N, BF16) = A[b] (M x K, BF16) @ dequant(W[b]),   1 <= M <= 32.
// W holds E4M3 codes with one UE8M0 scale per 32 elements of its contiguous axis, either
// K-major ([B, N, K], scales [B, N, K/32]) or N-major ([B, K, N], scales [B, K, N/32]); every
// tensor comes with element strides so zero-copy views of a larger allocation work. Stands in
// for the kernel behind b12x.gemm.bmm (b12x/gemm/_shared/mxfp8_bmm.py:446-1040): weights are
// dequantized to BF16 (E4M3 value times 2^(byte-127), rounded to BF16 as the BF16 multiply of
// the reference does) and multiplied with FP32 accumulation.
//
// Shape of the problem: 16 x 256 x 512 or 16 x 192 x 512 weight bytes (2 MB), at most 32 rows.
// It is bound by launch and memory latency, not by bytes or math. Two kernels: the tensor-core
// one at the end of this file (both operand blocks of a CTA resident in shared memory; taken
// whenever they fit) and the CUDA-core one that follows (any K), which is laid out to
// put every global load of a warp in flight before the first use and to finish in one pass:
//   grid = (N / columns per CTA, B), 8 warps per CTA; the warps split K (chunk c goes to warp
//   c % 8), a lane owns one (K-major) or two (N-major) output columns and all M rows of them;
//   A is staged per warp as FP32 [k][m] so one 16-byte shared load (a broadcast) feeds two
//   packed FP32x2 FMAs; the 8 partial sums per output meet in shared memory and are added in
//   warp order, so the result does not depend on timing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b12x_b200 {

struct BmmParams {
  const __nv_bfloat16* a;
  int64_t a_stride_b, a_stride_m;
  const uint8_t* w;
  int64_t w_stride_b, w_stride_r;
  const uint8_t* sf;
  int64_t sf_stride_b, sf_stride_r;
  __nv_bfloat16* c;
  int64_t c_stride_b, c_stride_m;
  int m, n, k;
};

constexpr int kBmmWarps = 8;
constexpr int kBmmThreads = kBmmWarps * 32;

template <int MAJOR, int MT>
struct BmmShape {
  static constexpr int kColsPerLane = MAJOR == 1 ? 2 : 1;
  static constexpr int kTileN = 32 * kColsPerLane;
  static constexpr int kChunk = MAJOR == 1 ? 8 : 32;      // k values per chunk
  static constexpr int kGroup = MAJOR == 1 ? 3 : 2;       // chunks whose loads fly together
  static constexpr int kParts = 32 / MT;                  // lanes sharing one row of A
  static constexpr int kLen = kChunk / kParts;            // BF16 elements of A per lane, chunk
  static constexpr int kStageFloats = kBmmWarps * kChunk * MT;
  static constexpr int kReduceFloats = kBmmWarps * MT * kTileN;
  static constexpr int kSmemBytes =
      4 * (kStageFloats > kReduceFloats ? kStageFloats : kReduceFloats);
  static_assert(kLen >= 2 && kLen % 2 == 0, "A pieces are loaded as 32-bit words");
};

__device__ __forceinline__ float bmm_ue8m0(uint32_t byte) {
  // 2^(byte - 127): byte 0 is the subnormal 2^-127, byte 255 is NaN.
  const uint32_t bits = byte == 0u ? 0x00400000u : (byte == 255u ? 0x7FC00000u : byte << 23);
  return __uint_as_float(bits);
}

__device__ __forceinline__ float bmm_round_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// Two E4M3 bytes (low byte first) to FP32.
__device__ __forceinline__ void bmm_e4m3x2(uint32_t pair, float& lo, float& hi) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)pair));
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  lo = __low2float(h);
  hi = __high2float(h);
}

__device__ __forceinline__ uint64_t bmm_dup(float x) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void bmm_fma2(uint64_t& acc, uint64_t a, uint64_t b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

__device__ __forceinline__ void bmm_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

template <int MAJOR, int MT>
__global__ void __launch_bounds__(kBmmThreads)
bmm_mxfp8_kernel(const BmmParams p) {
  using S = BmmShape<MAJOR, MT>;
  constexpr int CPL = S::kColsPerLane, KCH = S::kChunk, CG = S::kGroup, LEN = S::kLen;
  constexpr int WW = MAJOR == 1 ? KCH / 2 : KCH / 4;   // 32-bit weight words per lane, chunk
  extern __shared__ __align__(16) float bmm_smem[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y;
  const int n0 = blockIdx.x * S::kTileN;
  const int col = n0 + lane * CPL;                     // first column of this lane
  const bool col_ok = col < p.n;
  const int a_row = lane % MT, a_part = lane / MT;
  const bool row_ok = a_row < p.m;

  const uint8_t* w_b = p.w + (int64_t)b * p.w_stride_b;
  const uint8_t* sf_b = p.sf + (int64_t)b * p.sf_stride_b;
  const __nv_bfloat16* a_b = p.a + (int64_t)b * p.a_stride_b + (int64_t)a_row * p.a_stride_m;
  float* stage = bmm_smem + warp * (KCH * MT);

  uint64_t acc[CPL][MT / 2];
#pragma unroll
  for (int c = 0; c < CPL; ++c)
#pragma unroll
    for (int i = 0; i < MT / 2; ++i) acc[c][i] = 0ull;

  const int chunks = p.k / KCH;
  for (int c0 = warp; c0 < chunks; c0 += kBmmWarps * CG) {
    uint32_t wreg[CG][WW];
    uint32_t sreg[CG][MAJOR == 1 ? 2 : 1];   // N-major: 8 scale bytes; K-major: one
    uint32_t areg[CG][LEN / 2];
    // Every global load of the group first.
#pragma unroll
    for (int g = 0; g < CG; ++g) {
      const int ch = c0 + g * kBmmWarps;
      const bool live = ch < chunks;
      const int k0 = ch * KCH;
      if constexpr (MAJOR == 0) {
        if (live && col_ok) {
          const uint8_t* src = w_b + (int64_t)col * p.w_stride_r + k0;
          const uint4 lo = *reinterpret_cast<const uint4*>(src);
          const uint4 hi = *reinterpret_cast<const uint4*>(src + 16);
          wreg[g][0] = lo.x; wreg[g][1] = lo.y; wreg[g][2] = lo.z; wreg[g][3] = lo.w;
          wreg[g][4] = hi.x; wreg[g][5] = hi.y; wreg[g][6] = hi.z; wreg[g][7] = hi.w;
          sreg[g][0] = sf_b[(int64_t)col * p.sf_stride_r + ch];
        } else {
#pragma unroll
          for (int i = 0; i < WW; ++i) wreg[g][i] = 0u;
          sreg[g][0] = 127u;
        }
      } else {
        uint32_t s_lo = 0x7F7F7F7Fu, s_hi = 0x7F7F7F7Fu;
#pragma unroll
        for (int i = 0; i < WW; ++i) wreg[g][i] = 0u;
        if (live && col_ok) {
          s_lo = 0u; s_hi = 0u;
#pragma unroll
          for (int kk = 0; kk < KCH; ++kk) {
            const int64_t row = k0 + kk;
            const uint32_t two = *reinterpret_cast<const uint16_t*>(w_b + row * p.w_stride_r + col);
            wreg[g][kk >> 1] |= two << ((kk & 1) * 16);
            const uint32_t s = sf_b[row * p.sf_stride_r + (col >> 5)];
            if (kk < 4) s_lo |= s << (kk * 8); else s_hi |= s << ((kk - 4) * 8);
          }
        }
        sreg[g][0] = s_lo;
        sreg[g][1] = s_hi;
      }
      if (live && row_ok) {
        const __nv_bfloat16* src = a_b + k0 + a_part * LEN;
        if constexpr (LEN % 8 == 0) {
#pragma unroll
          for (int i = 0; i < LEN / 8; ++i) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + 8 * i);
            areg[g][4 * i + 0] = v.x; areg[g][4 * i + 1] = v.y;
            areg[g][4 * i + 2] = v.z; areg[g][4 * i + 3] = v.w;
          }
        } else if constexpr (LEN == 4) {
          const uint2 v = *reinterpret_cast<const uint2*>(src);
          areg[g][0] = v.x; areg[g][1] = v.y;
        } else {
          areg[g][0] = *reinterpret_cast<const uint32_t*>(src);
        }
      } else {
#pragma unroll
        for (int i = 0; i < LEN / 2; ++i) areg[g][i] = 0u;
      }
    }
    // Then chunk by chunk: stage A as FP32 [k][m], multiply.
#pragma unroll
    for (int g = 0; g < CG; ++g) {
      if (c0 + g * kBmmWarps >= chunks) break;   // uniform over the warp
      __syncwarp();
#pragma unroll
      for (int i = 0; i < LEN / 2; ++i) {
        const uint32_t two = areg[g][i];
        stage[(a_part * LEN + 2 * i) * MT + a_row] = __uint_as_float(two << 16);
        stage[(a_part * LEN + 2 * i + 1) * MT + a_row] = __uint_as_float(two & 0xFFFF0000u);
      }
      __syncwarp();
      float scale_k = 0.f;
      if (MAJOR == 0) scale_k = bmm_ue8m0(sreg[g][0]);
#pragma unroll
      for (int kk = 0; kk < KCH; kk += (MAJOR == 0 ? 2 : 1)) {
        float w0, w1;   // K-major: column `col` at kk and kk+1; N-major: two columns at kk
        if constexpr (MAJOR == 0) {
          bmm_e4m3x2(wreg[g][kk >> 2] >> ((kk & 2) * 8), w0, w1);
          w0 = bmm_round_bf16(w0 * scale_k);
          w1 = bmm_round_bf16(w1 * scale_k);
        } else {
          const float s = bmm_ue8m0((sreg[g][kk >> 2] >> ((kk & 3) * 8)) & 0xFFu);
          bmm_e4m3x2(wreg[g][kk >> 1] >> ((kk & 1) * 16), w0, w1);
          w0 = bmm_round_bf16(w0 * s);
          w1 = bmm_round_bf16(w1 * s);
        }
        const uint64_t w0d = bmm_dup(w0), w1d = bmm_dup(w1);
        const ulonglong2* arow0 = reinterpret_cast<const ulonglong2*>(stage + kk * MT);
        if constexpr (MAJOR == 0) {
          const ulonglong2* arow1 = reinterpret_cast<const ulonglong2*>(stage + (kk + 1) * MT);
#pragma unroll
          for (int q = 0; q < MT / 4; ++q) {
            const ulonglong2 a4 = arow0[q];
            bmm_fma2(acc[0][2 * q], a4.x, w0d);
            bmm_fma2(acc[0][2 * q + 1], a4.y, w0d);
          }
#pragma unroll
          for (int q = 0; q < MT / 4; ++q) {
            const ulonglong2 a4 = arow1[q];
            bmm_fma2(acc[0][2 * q], a4.x, w1d);
            bmm_fma2(acc[0][2 * q + 1], a4.y, w1d);
          }
        } else {
#pragma unroll
          for (int q = 0; q < MT / 4; ++q) {
            const ulonglong2 a4 = arow0[q];
            bmm_fma2(acc[0][2 * q], a4.x, w0d);
            bmm_fma2(acc[0][2 * q + 1], a4.y, w0d);
            bmm_fma2(acc[CPL - 1][2 * q], a4.x, w1d);
            bmm_fma2(acc[CPL - 1][2 * q + 1], a4.y, w1d);
          }
        }
      }
    }
  }

  // The 8 partial sums of every output meet in shared memory (which reuses the staging area)
  // and are added in warp order.
  __syncthreads();
  float* red = bmm_smem;
#pragma unroll
  for (int i = 0; i < MT / 2; ++i) {
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
      float lo, hi;
      bmm_unpack(acc[c][i], lo, hi);
      red[(warp * MT + 2 * i) * S::kTileN + lane * CPL + c] = lo;
      red[(warp * MT + 2 * i + 1) * S::kTileN + lane * CPL + c] = hi;
    }
  }
  __syncthreads();
  constexpr int kPairs = MT * S::kTileN / 2;
  __nv_bfloat16* c_b = p.c + (int64_t)b * p.c_stride_b;
  for (int pr = threadIdx.x; pr < kPairs; pr += kBmmThreads) {
    const int row = pr / (S::kTileN / 2);
    const int cc = (pr % (S::kTileN / 2)) * 2;
    if (row >= p.m || n0 + cc >= p.n) continue;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int w = 0; w < kBmmWarps; ++w) {
      const float2 v = *reinterpret_cast<const float2*>(red + (w * MT + row) * S::kTileN + cc);
      s0 += v.x;
      s1 += v.y;
    }
    __nv_bfloat16* dst = c_b + (int64_t)row * p.c_stride_m + n0 + cc;
    if (n0 + cc + 1 < p.n) {
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(s0, s1);
    } else {
      *dst = __float2bfloat16_rn(s0);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Tensor-core variant: the same product with the whole [MT x K] activation block and the whole
// dequantized [columns x K] weight tile of a CTA in shared memory as BF16 and warp-level BF16
// MMAs (m16n8k16, FP32 accumulation) over them. Used whenever the two blocks fit in shared
// memory; the CUDA-core kernel above remains for longer K. A 2 MB problem with at most 32 rows
// is far too small for the tcgen05 pipeline (its set-up alone costs more than this kernel's
// math), so the warp-level MMA is the right tool here.
//   phase 1: all 256 threads load their share of A and W (every global load of a round in
//            flight before the first use), dequantize W, store BF16 rows [row][K + 8] (the
//            8-element pad makes every fragment load conflict-free);
//   phase 2: warp w owns the 8 columns (w % blocks) of the tile and, when the tile has fewer
//            than 8 such blocks, one part of K; fragments are 32-bit shared loads;
//   phase 3: the K parts of a block are added in part order, rounded once, stored.
template <int MAJOR, int MT>
struct BmmMmaShape {
  static constexpr int kTileN = MAJOR == 1 ? 64 : 32;
  static constexpr int kBlocks = kTileN / 8;              // n8 blocks per CTA
  static constexpr int kParts = kBmmWarps / kBlocks;      // K parts per block (1 or 2)
  static constexpr int kRoundA = 8, kRoundW = 4;          // 16-byte loads per thread, round
  static __host__ __device__ int k_padded(int k) { return (k + 15) & ~15; }
  static __host__ __device__ int ld(int k) { return k_padded(k) + 8; }
  static __host__ __device__ int smem_bytes(int k) {
    return (kTileN + MT) * ld(k) * 2 + (kParts - 1) * kBlocks * (MT / 16) * 32 * 16;
  }
};

__device__ __forceinline__ void bmm_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 E4M3 codes times one scale -> 16 BF16 (as 8 packed words).
__device__ __forceinline__ void bmm_dequant16(const uint4& codes, float scale, uint32_t (&out)[8]) {
  const uint32_t w[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float lo, hi;
    bmm_e4m3x2(w[i >> 1] >> ((i & 1) * 16), lo, hi);
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo * scale, hi * scale);
    out[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
}

template <int MAJOR, int MT>
__global__ void __launch_bounds__(kBmmThreads)
bmm_mxfp8_mma_kernel(const BmmParams p) {
  using S = BmmMmaShape<MAJOR, MT>;
  constexpr int TN = S::kTileN, RA = S::kRoundA, RW = S::kRoundW;
  extern __shared__ __align__(16) float bmm_smem[];
  const int kp = S::k_padded(p.k), ld = S::ld(p.k);
  __nv_bfloat16* a_s = reinterpret_cast<__nv_bfloat16*>(bmm_smem);   // [MT][ld]
  __nv_bfloat16* w_s = a_s + MT * ld;                                // [TN][ld]
  float* red = reinterpret_cast<float*>(w_s + TN * ld);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  const int n0 = blockIdx.x * TN;
  const uint8_t* w_b = p.w + (int64_t)b * p.w_stride_b;
  const uint8_t* sf_b = p.sf + (int64_t)b * p.sf_stride_b;
  const __nv_bfloat16* a_b = p.a + (int64_t)b * p.a_stride_b;

  // ---- phase 1: weights (loads of a round first, then dequantize and store) -------------
  if constexpr (MAJOR == 0) {
    const int segs_per_row = p.k >> 4, segs = TN * segs_per_row;
    for (int base = 0; base < segs; base += kBmmThreads * RW) {
      uint4 codes[RW];
      uint32_t sbyte[RW];
#pragma unroll
      for (int j = 0; j < RW; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        const int row = idx / segs_per_row, seg = idx - row * segs_per_row;
        codes[j] = make_uint4(0u, 0u, 0u, 0u);
        sbyte[j] = 127u;
        if (idx < segs && n0 + row < p.n) {
          codes[j] = *reinterpret_cast<const uint4*>(w_b + (int64_t)(n0 + row) * p.w_stride_r + seg * 16);
          sbyte[j] = sf_b[(int64_t)(n0 + row) * p.sf_stride_r + (seg >> 1)];
        }
      }
#pragma unroll
      for (int j = 0; j < RW; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        if (idx >= segs) break;
        const int row = idx / segs_per_row, seg = idx - row * segs_per_row;
        uint32_t v[8];
        bmm_dequant16(codes[j], bmm_ue8m0(sbyte[j]), v);
        uint4* dst = reinterpret_cast<uint4*>(w_s + row * ld + seg * 16);
        dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
        dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
      }
    }
  } else {
    constexpr int kSegsPerRow = TN / 16;
    const int segs = p.k * kSegsPerRow;
    for (int base = 0; base < segs; base += kBmmThreads * RW) {
      uint4 codes[RW];
      uint32_t sbyte[RW];
#pragma unroll
      for (int j = 0; j < RW; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        const int row = idx / kSegsPerRow, col = n0 + (idx % kSegsPerRow) * 16;
        codes[j] = make_uint4(0u, 0u, 0u, 0u);
        sbyte[j] = 127u;
        if (idx < segs && col < p.n) {
          codes[j] = *reinterpret_cast<const uint4*>(w_b + (int64_t)row * p.w_stride_r + col);
          sbyte[j] = sf_b[(int64_t)row * p.sf_stride_r + (col >> 5)];
        }
      }
#pragma unroll
      for (int j = 0; j < RW; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        if (idx >= segs) break;
        const int row = idx / kSegsPerRow, c0 = (idx % kSegsPerRow) * 16;
        uint32_t v[8];
        bmm_dequant16(codes[j], bmm_ue8m0(sbyte[j]), v);
        uint16_t* dst = reinterpret_cast<uint16_t*>(w_s) + c0 * ld + row;   // transposed: [n][k]
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dst[(2 * i) * ld] = (uint16_t)(v[i] & 0xFFFFu);
          dst[(2 * i + 1) * ld] = (uint16_t)(v[i] >> 16);
        }
      }
    }
    // K rounded up to the MMA's 16: the extra weight columns are zero.
    for (int idx = tid; idx < TN * (kp - p.k); idx += kBmmThreads) {
      const int row = idx / (kp - p.k), c = p.k + idx % (kp - p.k);
      w_s[row * ld + c] = __float2bfloat16_rn(0.f);
    }
  }
  // ---- phase 1: activations (rows beyond M and columns beyond K are zero) --------------
  {
    const int segs_per_row = kp >> 3, segs = MT * segs_per_row;
    for (int base = 0; base < segs; base += kBmmThreads * RA) {
      uint4 v[RA];
#pragma unroll
      for (int j = 0; j < RA; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        const int row = idx / segs_per_row, seg = idx - row * segs_per_row;
        v[j] = make_uint4(0u, 0u, 0u, 0u);
        if (idx < segs && row < p.m && seg * 8 < p.k)
          v[j] = *reinterpret_cast<const uint4*>(a_b + (int64_t)row * p.a_stride_m + seg * 8);
      }
#pragma unroll
      for (int j = 0; j < RA; ++j) {
        const int idx = base + j * kBmmThreads + tid;
        if (idx >= segs) break;
        const int row = idx / segs_per_row, seg = idx - row * segs_per_row;
        *reinterpret_cast<uint4*>(a_s + row * ld + seg * 8) = v[j];
      }
    }
  }
  __syncthreads();

  // ---- phase 2: MMAs -------------------------------------------------------------------
  const int block = warp % S::kBlocks, part = warp / S::kBlocks;
  const int g = lane >> 2, q = lane & 3;
  const int steps = kp >> 4;
  const int s_begin = steps * part / S::kParts, s_end = steps * (part + 1) / S::kParts;
  float acc[MT / 16][4];
#pragma unroll
  for (int t = 0; t < MT / 16; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
  const uint32_t* w_words = reinterpret_cast<const uint32_t*>(w_s + (block * 8 + g) * ld) + q;
  const uint32_t* a_words = reinterpret_cast<const uint32_t*>(a_s + g * ld) + q;
  const int row_words = ld >> 1;
#pragma unroll 4
  for (int s = s_begin; s < s_end; ++s) {
    const uint32_t b0 = w_words[s * 8], b1 = w_words[s * 8 + 4];
#pragma unroll
    for (int t = 0; t < MT / 16; ++t) {
      const uint32_t* ar = a_words + t * 16 * row_words + s * 8;
      const uint32_t a[4] = {ar[0], ar[8 * row_words], ar[4], ar[8 * row_words + 4]};
      bmm_mma_bf16(acc[t], a, b0, b1);
    }
  }

  // ---- phase 3: add the K parts in order, round, store -----------------------------------
  if constexpr (S::kParts > 1) {
    float4* slot = reinterpret_cast<float4*>(red) + (block * (MT / 16)) * 32 + lane;
    if (part == 1) {
#pragma unroll
      for (int t = 0; t < MT / 16; ++t)
        slot[t * 32] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    __syncthreads();
    if (part == 1) return;
#pragma unroll
    for (int t = 0; t < MT / 16; ++t) {
      const float4 other = slot[t * 32];
      acc[t][0] += other.x; acc[t][1] += other.y; acc[t][2] += other.z; acc[t][3] += other.w;
    }
  }
  const int col = n0 + block * 8 + 2 * q;
  if (col >= p.n) return;
  __nv_bfloat16* c_b = p.c + (int64_t)b * p.c_stride_b + col;
#pragma unroll
  for (int t = 0; t < MT / 16; ++t) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = t * 16 + h * 8 + g;
      if (row >= p.m) continue;
      __nv_bfloat16* dst = c_b + (int64_t)row * p.c_stride_m;
      if (col + 1 < p.n) {
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[t][2 * h], acc[t][2 * h + 1]);
      } else {
        *dst = __float2bfloat16_rn(acc[t][2 * h]);
      }
    }
  }
}

}  // namespace b12x_b200
