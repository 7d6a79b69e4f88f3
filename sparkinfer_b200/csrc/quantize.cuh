// Row quantizers that feed the block-scaled GEMM.
//
//   quantize_mxfp8_rows : BF16/FP16 [M,K] -> E4M3 codes [M,K], one UE8M0 scale byte per 32
//                         elements, written row-major [M,K/32] and/or in 512-byte MMA atoms.
//   quantize_nvfp4_rows : BF16/FP16 [M,K] -> packed E2M1 codes [M,K/2] (low nibble = even k),
//                         one UE4M3 scale byte per 16 elements in MMA atoms, with a caller
//                         supplied FP32 global scale (device scalar, read at run time).
//
// Both are pure streaming kernels (2 bytes read, ~1.03 / ~0.56 bytes written per element):
// 16-byte loads, register amax, 8/16-byte stores. The arithmetic is IEEE round-to-nearest
// throughout (true divisions, no approximations, no contraction) so the emitted bytes are
// reproducible on a CPU.
//
// Scale atom layout (shared with the GEMM): atom index = row_tile * k_atoms + kb / 4, byte in
// atom = (r % 32) * 16 + ((r / 32) % 4) * 4 + (kb % 4), r = row % 128, kb = scale column.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace b12x_b200 {

__device__ __forceinline__ size_t sf_atom_offset(int row, int kb, int k_atoms) {
  const int r = row & 127;
  return (static_cast<size_t>(row >> 7) * k_atoms + (kb >> 2)) * 512 + (r & 31) * 16 +
         ((r >> 5) & 3) * 4 + (kb & 3);
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]);

template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& raw, float (&out)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& raw, float (&out)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 f = __half22float2(h);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// UE8M0 byte for a block with maximum magnitude `amax`:
//   127 + clamp(ceil(log2(amax / 448)), -127, 127), and 127 for an all-zero block.
// ceil(log2(v)) of a normal float is its exponent, plus one when the mantissa is non-zero.
__device__ __forceinline__ uint32_t ue8m0_from_amax(float amax) {
  if (!(amax > 0.0f)) return 127u;
  const float v = __fdiv_rn(amax, 448.0f);
  const uint32_t bits = __float_as_uint(v);
  const uint32_t exp = bits >> 23;
  if (exp == 0) return (bits > 0x00400000u) ? 1u : 0u;  // below 2^-126: 2^-127 is the split
  return exp + ((bits & 0x007FFFFFu) ? 1u : 0u);
}

// 2^(127 - byte) as a float (the exact reciprocal of the UE8M0 scale).
__device__ __forceinline__ float ue8m0_reciprocal(uint32_t byte) {
  return __uint_as_float(byte >= 254u ? (byte == 254u ? 0x00400000u : 0x00200000u)
                                      : ((254u - byte) << 23));
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One thread = 16 consecutive elements; two neighbouring lanes share one 32-element block.
// The launch covers rows_cover x (k_cover / 16) threads: rows >= m and scale columns >= k/32
// only receive the neutral scale byte 127 in the atom layout.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_mxfp8_rows_kernel(const T* __restrict__ src, int64_t ld_src, uint8_t* __restrict__ values,
                           uint8_t* __restrict__ scale_rows, uint8_t* __restrict__ scale_mma,
                           int m, int k, int rows_cover, int k_cover, int k_atoms) {
  const int units_per_row = k_cover / 16;
  const int64_t total = static_cast<int64_t>(rows_cover) * units_per_row;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool in_cover = idx < total;
  const int row = in_cover ? static_cast<int>(idx / units_per_row) : 0;
  const int unit = in_cover ? static_cast<int>(idx % units_per_row) : 0;
  const int k0 = unit * 16;
  const bool live = in_cover && row < m && k0 < k;

  float x[16];
  if (live) {
    const T* p = src + static_cast<int64_t>(row) * ld_src + k0;
    float a[8], b[8];
    unpack8<T>(ld_nc_16(p), a);
    unpack8<T>(ld_nc_16(p + 8), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { x[i] = a[i]; x[8 + i] = b[i]; }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = 0.0f;
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));

  const uint32_t byte = ue8m0_from_amax(amax);
  const float inv = ue8m0_reciprocal(byte);
  if (live) {
    float y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      y[i] = fminf(fmaxf(__fmul_rn(x[i], inv), -448.0f), 448.0f);
    uint4 out;
    out.x = e4m3x4(y[0], y[1], y[2], y[3]);
    out.y = e4m3x4(y[4], y[5], y[6], y[7]);
    out.z = e4m3x4(y[8], y[9], y[10], y[11]);
    out.w = e4m3x4(y[12], y[13], y[14], y[15]);
    *reinterpret_cast<uint4*>(values + static_cast<int64_t>(row) * k + k0) = out;
  }
  if (in_cover && (unit & 1) == 0) {
    const int kb = unit >> 1;
    if (live && scale_rows) scale_rows[static_cast<int64_t>(row) * (k / 32) + kb] = byte;
    if (scale_mma) scale_mma[sf_atom_offset(row, kb, k_atoms)] = live ? byte : 127u;
  }
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// Eight floats -> eight E2M1 nibbles (element 0 in the lowest nibble), negative zero folded
// into zero.
__device__ __forceinline__ uint32_t e2m1x8(const float* y) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t b = __nv_cvt_float2_to_fp4x2(make_float2(y[2 * i], y[2 * i + 1]), __NV_E2M1,
                                                cudaRoundNearest);
    w |= (b & 0xFFu) << (8 * i);
  }
  const uint32_t mag = w & 0x77777777u;
  const uint32_t nonzero = (mag | (mag >> 1) | (mag >> 2)) & 0x11111111u;
  return w & (0x77777777u | (nonzero << 3));
}

// One thread = one 16-element block. Rows >= m and scale columns >= k/16 inside the covered
// area receive scale byte 0 (the atom layout's padding value for NVFP4).
template <typename T>
__global__ void __launch_bounds__(256)
quantize_nvfp4_rows_kernel(const T* __restrict__ src, int64_t ld_src,
                           const float* __restrict__ global_scale, uint8_t* __restrict__ packed,
                           uint8_t* __restrict__ scale_mma, int m, int k, int rows_cover,
                           int k_cover, int k_atoms) {
  const int units_per_row = k_cover / 16;
  const int64_t total = static_cast<int64_t>(rows_cover) * units_per_row;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int row = static_cast<int>(idx / units_per_row);
  const int kb = static_cast<int>(idx % units_per_row);
  const int k0 = kb * 16;
  if (row >= m || k0 >= k) {
    scale_mma[sf_atom_offset(row, kb, k_atoms)] = 0;
    return;
  }
  const float gs = *global_scale;
  const T* p = src + static_cast<int64_t>(row) * ld_src + k0;
  float x[16];
  {
    float a[8], b[8];
    unpack8<T>(ld_nc_16(p), a);
    unpack8<T>(ld_nc_16(p + 8), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { x[i] = a[i]; x[8 + i] = b[i]; }
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));

  const float s = __fmul_rn(gs, __fdiv_rn(amax, 6.0f));
  const uint32_t s_byte =
      static_cast<uint32_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3)) & 0xFFu;
  const float s_q = e4m3_to_float(s_byte);
  const float r = (gs == 0.0f) ? 0.0f : __frcp_rn(gs);
  const float t = __fmul_rn(s_q, r);
  const float inv = (t == 0.0f) ? 0.0f : __frcp_rn(t);
  float y[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = fminf(fmaxf(__fmul_rn(x[i], inv), -6.0f), 6.0f);
  uint2 out;
  out.x = e2m1x8(y);
  out.y = e2m1x8(y + 8);
  *reinterpret_cast<uint2*>(packed + static_cast<int64_t>(row) * (k / 2) + k0 / 2) = out;
  scale_mma[sf_atom_offset(row, kb, k_atoms)] = static_cast<uint8_t>(s_byte);
}

}  // namespace b12x_b200
