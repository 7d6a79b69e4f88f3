// Row quantizers that feed the block-scaled GEMM.
//
//   quantize_mxfp8_rows : BF16/FP16 [M,K] -> E4M3 codes [M,K], one UE8M0 scale byte per 32
//                         elements, written row-major [M,K/32] and/or in 512-byte MMA atoms.
//   quantize_nvfp4_rows : BF16/FP16 [M,K] -> packed E2M1 codes [M,K/2] (low nibble = even k),
//                         one UE4M3 scale byte per 16 elements in MMA atoms, with a caller
//                         supplied FP32 global scale (device scalar, read at run time).
//
// Both are pure streaming kernels (2 bytes read, ~1.03 / ~0.56 bytes written per element):
// coalesced 16-byte loads, amax in registers and shuffles, coalesced 8/4-byte stores. The arithmetic is IEEE round-to-nearest
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

// Largest magnitude of the eight 16-bit floats in `raw`, through the packed two-lane abs / max
// instructions (exact: no rounding is involved in either).
template <typename T>
__device__ __forceinline__ float amax8(const uint4& raw);

template <>
__device__ __forceinline__ float amax8<__nv_bfloat16>(const uint4& raw) {
  const __nv_bfloat162* v = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const __nv_bfloat162 a = __hmax2(__hmax2(__habs2(v[0]), __habs2(v[1])),
                                   __hmax2(__habs2(v[2]), __habs2(v[3])));
  return fmaxf(__low2float(a), __high2float(a));
}

template <>
__device__ __forceinline__ float amax8<__half>(const uint4& raw) {
  const __half2* v = reinterpret_cast<const __half2*>(&raw);
  const __half2 a = __hmax2(__hmax2(__habs2(v[0]), __habs2(v[1])),
                            __hmax2(__habs2(v[2]), __habs2(v[3])));
  return fmaxf(__low2float(a), __high2float(a));
}

// UE8M0 byte for a block with maximum magnitude `amax`:
//   127 + clamp(ceil(log2(amax / 448)), -127, 127), and 127 for an all-zero block.
// ceil(log2(v)) of a normal float is its exponent, plus one when the mantissa is non-zero.
__device__ __forceinline__ uint32_t ue8m0_from_amax(float amax) {
  if (!(amax > 0.0f)) return 127u;
  {
    // 448 = 1.75 * 2^8, so for a quotient that stays normal the answer follows from amax's own
    // fields: exponent - 8, plus one when the mantissa exceeds that of 1.75 (the rounded
    // quotient has a non-zero mantissa exactly when the true one has, see the two neighbours of
    // 1.75). Anything near the ends of the range takes the division below.
    const uint32_t abits = __float_as_uint(amax);
    const uint32_t aexp = abits >> 23;
    if (aexp >= 10u && aexp < 255u) return aexp - 8u + (((abits & 0x007FFFFFu) > 0x00600000u) ? 1u : 0u);
  }
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

// Four floats -> four E4M3 bytes (element 0 in the lowest byte), saturating at +-448.
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  uint32_t out;
  asm("{\n"
      ".reg .b16 lo, hi;\n"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n"
      "mov.b32 %0, {lo, hi};\n"
      "}\n"
      : "=r"(out)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return out;
}

// Work decomposition shared by both quantizers: one warp owns one chunk of kChunkElems
// consecutive elements of one row and reads it with kLoadsPerLane 16-byte loads per lane, load j
// covering elements [j*256 + lane*8, +8) of the chunk. Every load instruction of a warp thus
// reads 512 contiguous bytes, all of a lane's loads are issued before the first use (64 bytes in
// flight per thread), and a scale block (16 or 32 elements) spans 2 or 4 neighbouring lanes, so
// its maximum is one or two shuffles away. A chunk that lies wholly inside the matrix (the
// common case) runs a copy of the body without any bounds predicate: the kernels are bound by
// instruction issue, not by memory, as soon as they carry per-element tests.
constexpr int kQuantLoadsPerLane = 4;
constexpr int kQuantChunkElems = kQuantLoadsPerLane * 256;

__host__ __device__ inline int64_t quant_warps(int rows_cover, int k_cover) {
  return static_cast<int64_t>(rows_cover) * ((k_cover + kQuantChunkElems - 1) / kQuantChunkElems);
}

struct QuantChunk {
  int row, chunk, lane, k_base;  // k_base = first element of this lane's load 0
};

// 32-bit on purpose (the host refuses covers with 2^31 or more warps): a 64-bit division per
// thread costs more instructions than the quantization itself. Returns false for surplus warps.
__device__ __forceinline__ bool quant_chunk_of_warp(int rows_cover, int k_cover, QuantChunk& c) {
  const uint32_t chunks_per_row =
      static_cast<uint32_t>((k_cover + kQuantChunkElems - 1) / kQuantChunkElems);
  const uint32_t warp_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= static_cast<uint32_t>(rows_cover) * chunks_per_row) return false;
  c.lane = threadIdx.x & 31;
  c.row = static_cast<int>(warp_id / chunks_per_row);
  c.chunk = static_cast<int>(warp_id - static_cast<uint32_t>(c.row) * chunks_per_row);
  c.k_base = c.chunk * kQuantChunkElems + c.lane * 8;
  return true;
}

template <typename T, bool kFull>
__device__ __forceinline__ void quantize_mxfp8_chunk(const QuantChunk& c, const T* __restrict__ src,
                                                     int64_t ld_src, uint8_t* __restrict__ values,
                                                     uint8_t* __restrict__ scale_rows,
                                                     uint8_t* __restrict__ scale_mma, int m, int k,
                                                     int k_cover, int k_atoms) {
  const bool row_live = kFull || c.row < m;
  const T* src_row = src + static_cast<int64_t>(row_live ? c.row : 0) * ld_src + c.k_base;
  uint4 raw[kQuantLoadsPerLane];
#pragma unroll
  for (int j = 0; j < kQuantLoadsPerLane; ++j) {
    const bool live = kFull || (row_live && c.k_base + j * 256 < k);
    raw[j] = live ? ld_nc_16(src_row + j * 256) : make_uint4(0, 0, 0, 0);
  }
  // Addresses for load 0; load j adds a constant (256 codes, 8 scale columns = 2 atoms).
  uint8_t* out_values = values + static_cast<int64_t>(c.row) * k + c.k_base;
  const int kb0 = c.k_base >> 5;
  uint8_t* out_rows =
      scale_rows ? scale_rows + static_cast<int64_t>(c.row) * (k >> 5) + kb0 : nullptr;
  uint8_t* out_mma = scale_mma ? scale_mma + sf_atom_offset(c.row, kb0, k_atoms) : nullptr;
  const bool scale_lane = (c.lane & 3) == 0;
#pragma unroll
  for (int j = 0; j < kQuantLoadsPerLane; ++j) {
    const int k0 = c.k_base + j * 256;
    const bool live = kFull || (row_live && k0 < k);
    float amax = amax8<T>(raw[j]);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t byte = ue8m0_from_amax(amax);
    const float inv = ue8m0_reciprocal(byte);
    if (live) {
      float x[8];
      unpack8<T>(raw[j], x);
      uint2 out;  // the conversion saturates at 448
      out.x = e4m3x4(__fmul_rn(x[0], inv), __fmul_rn(x[1], inv), __fmul_rn(x[2], inv),
                     __fmul_rn(x[3], inv));
      out.y = e4m3x4(__fmul_rn(x[4], inv), __fmul_rn(x[5], inv), __fmul_rn(x[6], inv),
                     __fmul_rn(x[7], inv));
      *reinterpret_cast<uint2*>(out_values + j * 256) = out;
    }
    if (scale_lane && (kFull || k0 < k_cover)) {
      if (live && out_rows) out_rows[j * 8] = static_cast<uint8_t>(byte);
      if (out_mma) out_mma[j * 1024] = live ? static_cast<uint8_t>(byte) : uint8_t(127);
    }
  }
}

// Both quantizers are launched with programmatic stream serialization, so in a decode step
// (GEMM, quantize, GEMM, ...) nothing waits for a whole grid to drain and a new one to start:
//   - griddepcontrol.wait: this grid may have been started while its predecessor on the stream
//     was still running; nothing is read or written before the predecessor has completed.
//   - griddepcontrol.launch_dependents, only when the quantized matrix has at most 128 rows
//     (early_release): the next kernel on the stream, if it too was launched with programmatic
//     serialization, may start now. In this library that is the decode GEMM, which streams its
//     weight operand at once and waits for this grid before it reads activations. A matrix of
//     more than 128 rows may be somebody's weight operand, so its quantization never releases
//     early (and the decode GEMM waits before streaming a weight of 128 rows or fewer).
__device__ __forceinline__ void quant_grid_prologue(int early_release) {
  if (early_release) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The launch covers rows_cover x k_cover elements: rows >= m and scale columns >= k/32 inside
// the cover only receive the neutral scale byte 127 in the atom layout.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_mxfp8_rows_kernel(const T* __restrict__ src, int64_t ld_src, uint8_t* __restrict__ values,
                           uint8_t* __restrict__ scale_rows, uint8_t* __restrict__ scale_mma,
                           int m, int k, int rows_cover, int k_cover, int k_atoms,
                           int early_release) {
  quant_grid_prologue(early_release);
  QuantChunk c;
  if (!quant_chunk_of_warp(rows_cover, k_cover, c)) return;  // whole warps leave
  if (c.row < m && (c.chunk + 1) * kQuantChunkElems <= k)
    quantize_mxfp8_chunk<T, true>(c, src, ld_src, values, scale_rows, scale_mma, m, k, k_cover,
                                  k_atoms);
  else
    quantize_mxfp8_chunk<T, false>(c, src, ld_src, values, scale_rows, scale_mma, m, k, k_cover,
                                   k_atoms);
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// Eight floats -> eight E2M1 nibbles (element 0 in the lowest nibble), saturating at +-6,
// negative zero folded into zero.
__device__ __forceinline__ uint32_t e2m1x8(const float* y) {
  uint32_t w;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}\n"
      : "=r"(w)
      : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
  const uint32_t mag = w & 0x77777777u;
  const uint32_t nonzero = (mag | (mag >> 1) | (mag >> 2)) & 0x11111111u;
  return w & (0x77777777u | (nonzero << 3));
}

template <typename T, bool kFull>
__device__ __forceinline__ void quantize_nvfp4_chunk(const QuantChunk& c, const T* __restrict__ src,
                                                     int64_t ld_src, float gs,
                                                     uint8_t* __restrict__ packed,
                                                     uint8_t* __restrict__ scale_mma, int m, int k,
                                                     int k_cover, int k_atoms) {
  const bool row_live = kFull || c.row < m;
  const T* src_row = src + static_cast<int64_t>(row_live ? c.row : 0) * ld_src + c.k_base;
  uint4 raw[kQuantLoadsPerLane];
#pragma unroll
  for (int j = 0; j < kQuantLoadsPerLane; ++j) {
    const bool live = kFull || (row_live && c.k_base + j * 256 < k);
    raw[j] = live ? ld_nc_16(src_row + j * 256) : make_uint4(0, 0, 0, 0);
  }
  const float r = (gs == 0.0f) ? 0.0f : __frcp_rn(gs);
  // Block maxima: a block is the 16 elements of two neighbouring lanes.
  float amax[kQuantLoadsPerLane];
#pragma unroll
  for (int j = 0; j < kQuantLoadsPerLane; ++j) {
    const float a = amax8<T>(raw[j]);
    amax[j] = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
  }
  // The scale arithmetic (two IEEE divisions and a round trip through E4M3) is the expensive
  // part, so the two lanes of a block split it: the even lane does loads 0 and 1, the odd lane
  // loads 2 and 3, and they swap the resulting multipliers.
  const int odd = c.lane & 1;
  const int pair_k = c.chunk * kQuantChunkElems + (c.lane >> 1) * 16;  // the pair's block of load 0
  uint8_t* out_mma = scale_mma + sf_atom_offset(c.row, pair_k >> 4, k_atoms);  // +4 atoms per load
  float inv_mine[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int j = odd * 2 + h;
    const float am = odd ? amax[2 + h] : amax[h];
    const float s = __fmul_rn(gs, __fdiv_rn(am, 6.0f));
    const uint32_t s_byte =
        static_cast<uint32_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3)) & 0xFFu;
    const float t = __fmul_rn(e4m3_to_float(s_byte), r);
    inv_mine[h] = (t == 0.0f) ? 0.0f : __frcp_rn(t);
    const int kblk = pair_k + j * 256;  // first element of the block
    if (kFull || kblk < k_cover)
      out_mma[j * 2048] = (kFull || (row_live && kblk < k)) ? static_cast<uint8_t>(s_byte) : uint8_t(0);
  }
  uint8_t* out_packed = packed + static_cast<int64_t>(c.row) * (k >> 1) + (c.k_base >> 1);
  float inv[kQuantLoadsPerLane];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float theirs = __shfl_xor_sync(0xffffffffu, inv_mine[h], 1);
    inv[h] = odd ? theirs : inv_mine[h];
    inv[2 + h] = odd ? inv_mine[h] : theirs;
  }
#pragma unroll
  for (int j = 0; j < kQuantLoadsPerLane; ++j) {
    if (kFull || (row_live && c.k_base + j * 256 < k)) {
      float x[8], y[8];
      unpack8<T>(raw[j], x);
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(x[i], inv[j]);  // the conversion saturates at 6
      *reinterpret_cast<uint32_t*>(out_packed + j * 128) = e2m1x8(y);
    }
  }
}

// Rows >= m and scale columns >= k/16 inside the covered area receive scale byte 0 (the atom
// layout's padding value for NVFP4).
template <typename T>
__global__ void __launch_bounds__(256)
quantize_nvfp4_rows_kernel(const T* __restrict__ src, int64_t ld_src,
                           const float* __restrict__ global_scale, uint8_t* __restrict__ packed,
                           uint8_t* __restrict__ scale_mma, int m, int k, int rows_cover,
                           int k_cover, int k_atoms, int early_release) {
  quant_grid_prologue(early_release);
  QuantChunk c;
  if (!quant_chunk_of_warp(rows_cover, k_cover, c)) return;  // whole warps leave
  const float gs = *global_scale;
  if (c.row < m && (c.chunk + 1) * kQuantChunkElems <= k)
    quantize_nvfp4_chunk<T, true>(c, src, ld_src, gs, packed, scale_mma, m, k, k_cover, k_atoms);
  else
    quantize_nvfp4_chunk<T, false>(c, src, ld_src, gs, packed, scale_mma, m, k, k_cover, k_atoms);
}

}  // namespace b12x_b200
