// Load-time conversion of a block-scaled FP8 checkpoint weight into the MXFP8 rows the GEMM reads:
// E4M3 codes [L][M][K] with one FP32 scale per 128 x 128 block ->
//   E4M3 codes on power-of-two block scales, the UE8M0 byte of each block expanded to every row
//   and 32-column group (row-major [L][M][K/32]) and to the 512-byte scale atoms
//   ([L][ceil(M/128)][K/128], rows beyond M filled with 127 = 2^0).
//
// The arithmetic is that of pack_fp8_block_scaled_weight_mxfp8 in the reference
// (b12x/gemm/_shared/wo_mxfp8.py:873-1187), whose bytes the tests pin:
//   v = float(code) * s (one FP32 rounding), amax over the 128 x 128 block (rows beyond M count
//   as zeros), byte = 127 + clamp(ceil(log2(amax / 448)), -127, 127) (127 for an all-zero
//   block), new code = E4M3(v / 2^(byte - 127)), round to nearest even.
// When every scale is already a power of two nothing is re-derived: codes are copied and the
// byte is the scale's own exponent (requantize = 0).
//
// One CTA of 256 threads per block: thread t holds 64 consecutive codes of row t / 2.
#pragma once

#include <cuda_fp8.h>
#include <cstdint>

#include "quantize.cuh"

namespace b12x_b200 {

struct PackWeightParams {
  const uint8_t* codes;   // [L][M][K] E4M3
  const float* scale;     // [L][ceil(M/128)][K/128]
  uint8_t* out_codes;     // [L][M][K]
  uint8_t* scale_rows;    // [L][M][K/32], may be null
  uint8_t* scale_mma;     // [L][ceil(M/128)][K/128][512], may be null
  int m, k;
  int requantize;
};

__global__ void __launch_bounds__(256)
pack_block_fp8_weight_kernel(const PackWeightParams p) {
  const int kb = blockIdx.x, rt = blockIdx.y, grp = blockIdx.z;
  const int k_blocks = p.k / 128;
  const int row_tiles = (p.m + 127) / 128;
  const int t = threadIdx.x;
  const int row_in_tile = t >> 1;
  const int row = rt * 128 + row_in_tile;
  const bool live = row < p.m;
  const size_t elem0 = (static_cast<size_t>(grp) * p.m + row) * p.k + kb * 128 + (t & 1) * 64;
  const float s = p.scale[(static_cast<size_t>(grp) * row_tiles + rt) * k_blocks + kb];

  uint4 raw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    raw[i] = live ? *reinterpret_cast<const uint4*>(p.codes + elem0 + i * 16) : make_uint4(0, 0, 0, 0);

  __shared__ float warp_max[8];
  __shared__ uint32_t s_byte;
  uint32_t byte;
  if (p.requantize) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int j = 0; j < 16; ++j)
        amax = fmaxf(amax, fabsf(__fmul_rn(e4m3_to_float((w[j >> 2] >> ((j & 3) * 8)) & 0xFFu), s)));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if ((t & 31) == 0) warp_max[t >> 5] = amax;
    __syncthreads();
    if (t == 0) {
      float a = warp_max[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) a = fmaxf(a, warp_max[i]);
      s_byte = min(ue8m0_from_amax(a), 254u);
    }
    __syncthreads();
    byte = s_byte;
    // 2^(byte - 127): the divisor, subnormal for byte 0.
    const float divisor = __uint_as_float(byte == 0u ? 0x00400000u : (byte << 23));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[j] = __fdiv_rn(__fmul_rn(e4m3_to_float((w[q] >> (j * 8)) & 0xFFu), s), divisor);
        w[q] = e4m3x4(v[0], v[1], v[2], v[3]);
      }
      raw[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    // Power-of-two scale: byte = round(log2(s)) clamped to [-127, 127], plus 127, which is the
    // biased exponent field of s itself (0 for everything below 2^-126); non-positive -> 2^0.
    const uint32_t bits = __float_as_uint(s);
    byte = (s > 0.0f) ? min((bits >> 23) & 0xFFu, 254u) : 127u;
  }

  if (live) {
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(p.out_codes + elem0 + i * 16) = raw[i];
    if (p.scale_rows && (t & 1) == 0) {
      const uint32_t four = byte * 0x01010101u;
      *reinterpret_cast<uint32_t*>(p.scale_rows +
                                   (static_cast<size_t>(grp) * p.m + row) * (p.k / 32) + kb * 4) = four;
    }
  }
  if (p.scale_mma && (t & 1) == 0) {
    // Atom byte of (row r, scale column c): (r % 32) * 16 + (r / 32) * 4 + c.
    const uint32_t four = (live ? byte : 127u) * 0x01010101u;
    uint8_t* atom = p.scale_mma +
                    ((static_cast<size_t>(grp) * row_tiles + rt) * k_blocks + kb) * 512;
    *reinterpret_cast<uint32_t*>(atom + (row_in_tile & 31) * 16 + (row_in_tile >> 5) * 4) = four;
  }
}

}  // namespace b12x_b200
