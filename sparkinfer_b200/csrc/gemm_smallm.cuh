// Weight-streaming block-scaled GEMM for decode shapes (M <= 128) on sm_100a.
//
// With a handful of activation rows the GEMM is a pure stream of the weight matrix: what
// matters is that every SM pulls an equal share of the weight bytes with enough of them in
// flight. The roles of the operands are swapped relative to the large-M kernel: 128 weight
// rows fill the M side of the tcgen05 MMA, the (padded) activation rows are its N side, so no
// shared memory or tensor-core time is spent on padding rows.
//
// Work is cut stream-K style. A unit is (weight tile of 128 rows, k-tile of 128 bytes of K);
// units are numbered tile-major and CTA c of G takes units [c*U/G, (c+1)*U/G), i.e. every
// CTA streams the same number of bytes (+-1 unit) whatever N is. A CTA range covers a run of
// segments, one per tile it touches. A segment that spans its whole tile is converted and
// stored directly. Otherwise the FP32 partial goes to scratch slot (tile, segment index) and
// a per-tile counter is bumped; the CTA that brings the counter to the segment count adds the
// slots in segment order (deterministic) and stores the tile, then resets the counter. Nobody
// waits on another CTA.
//
// Issue rate, not bandwidth, is what limits one CTA: a unit costs about a dozen tcgen05
// instructions (scale copies + MMAs) from a single thread. Two warps therefore issue, taking
// alternate units of the CTA's range into accumulators of their own; the epilogue adds the two
// (issuer 0 first, so the sum order is fixed). With 128 padded rows four accumulators do not fit
// in TMEM next to the scales and the second issuer idles.
//
// Back-to-back launches overlap. A decode step is a chain of such GEMMs, each only a few
// microseconds of streaming, and about as much again goes into fixed cost per launch: the gap
// between dependent grids, the prologue, the ~2 us until the first weight bytes arrive, the
// tail. The kernel is therefore launched with programmatic stream serialization and calls
// griddepcontrol.launch_dependents at once, so the next grid's CTAs are placed as soon as this
// grid's CTAs leave their SMs and run their prologue and first weight loads while this grid is
// still finishing. The weight producer starts streaming immediately when the weight has more
// than 128 rows: the only kernels that release their dependents early are this one (output of
// at most 128 rows) and the row quantizers (only for matrices of at most 128 rows), so such a
// weight cannot be a predecessor's output still being written. The warps that read activations
// or alpha, or write C, partials or counters, wait for the predecessor to finish
// (griddepcontrol.wait) first, and so does the weight producer for a weight of 128 rows or fewer.
// Tensor memory is addressed relative to the allocation's base column and only as many columns
// as needed are taken, so a CTA does not depend on being alone on its SM.
//
// Scratch ("workspace") layout: a 64 KiB block of per-tile int32 counters, then
// [tiles][max_segments][m_pad][128] FP32 partials. Counters must be zero before the first
// launch; every launch leaves them zero again, whatever the shape.
//
// Fused activation quantization (template parameter FUSED, M <= 16). The caller passes the
// BF16 activation rows instead of codes and scales. The activation producer brings the raw
// rows of a unit (8 or 16 rows x 256 NVFP4 / 128 MXFP8 elements) into an extra area of the
// stage with one TMA copy, in the same queue as the weights. Eight extra warps wait for the
// stage's full barrier, quantize the raw rows with exactly the arithmetic of the row
// quantizers in quantize.cuh, write codes (128-byte-swizzled, as TMA would) and scale bytes
// (atom layout) into the stage, and arrive on the stage's "ready" barrier, which is what the
// MMA issuers wait for. (Quantizer warps that loaded the rows themselves with ordinary global
// loads were measured at twice the kernel time: such a load queues behind the ~180 KiB of
// weight requests the SM has outstanding and takes microseconds.) Every CTA quantizes the K
// range it multiplies, so the rows are re-quantized once per weight tile a CTA owns: cheap
// next to the 16 KiB of weights of a unit for a handful of rows, and the reason for the
// M <= 16 limit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_blockscaled.cuh"
#include "quantize.cuh"

namespace b12x_b200 {

struct SmallMParams {
  const uint8_t* sf_w;     // weight scale atoms   [ceil(N/128)][k_atoms][512]
  const uint8_t* sf_x;     // activation scale atoms [1][k_atoms][512] (rows >= M unused)
  void* c;                 // [M, ldc]
  const float* alpha;
  int* status;
  float* partials;         // scratch, see above
  int* counters;
  int m, n, k, ldc, out_dtype;
  int m_pad;               // MMA N: 16, 32, 64 or 128
  int tiles;               // weight tiles of all groups: groups * ceil(N / 128)
  int tiles_per_group;     // ceil(N / 128)
  // Grouped GEMM: operands stacked as [groups, rows, K]; scale atoms and outputs group after
  // group (bytes / elements between groups). Group g of the quantized-C output, if any, starts
  // at column quant_col0 + g * N.
  long long sf_w_group_bytes, sf_x_group_bytes, c_group_elems;
  int k_tiles;             // ceil(K / elems per stage)
  int k_atoms_total;
  int max_segments;        // scratch slots per tile
  int num_stages;
  int stage_bytes;
  int issuers;             // MMA-issuing warps in use (2 when four accumulators fit, else 1)
  int tmem_cols;           // tensor memory to allocate: 128, 256 or 512 columns
  int sf_col0;             // first scale column (after the accumulators)
  // Fused activation quantization only: the NVFP4 global scale of the rows, and how many raw
  // BF16 rows (8 or 16) a stage holds behind the code tile.
  const float* x_gs;
  int raw_rows;
  // Fused MXFP8 quantization with the inverse rotary embedding (ROPE instantiation only): row r
  // is token r at position rope_positions[r]; in every head_dim-wide block of a group's K the
  // trailing rope_dim elements are rotated back, interleaved pairs (even, odd), with
  // cos = cache[pos * rope_dim + pair], sin = cache[pos * rope_dim + rope_dim / 2 + pair].
  const void* rope_positions;   // int32 or int64 [M]
  const void* rope_cos_sin;     // BF16 or FP32 [max_pos, rope_dim]
  int rope_pos_i64, rope_cache_f32;
  int rope_head_dim, rope_nope_dim, rope_dim;
  // Epilogue extras. bias: [N] values of the output dtype added to every row (null = none).
  // quant_*: MXFP8 re-quantization of the rounded output rows along N (null = off): E4M3 codes
  // [M, quant_ld], UE8M0 bytes row-major [M, quant_cols / 32] and/or in scale atoms, this GEMM's
  // columns starting at column quant_col0 of a quant_cols-wide matrix.
  const void* bias;
  uint8_t* quant_values;
  uint8_t* quant_scale_rows;
  uint8_t* quant_scale_mma;
  long long quant_ld;
  int quant_col0, quant_cols;
  // Non-zero: the weight stream too waits for the previous grid (weights of few rows may be a
  // predecessor's fresh output, see the header comment).
  int wait_for_weights;
  // Non-zero: whole tiles of 2-byte outputs leave through a small shared-memory staging area as
  // 16-byte stores (rows of C 16-byte aligned); zero: every lane stores its own 2-byte values.
  int packed_store;
  int smem_bytes;          // dynamic shared memory of the launch
  // Optional per-CTA time stamps (8 x uint64 per CTA, see kTimeline*); null in normal use.
  unsigned long long* timeline;
};

// Bytes after the ring: barriers and flags (first 512), then the output staging area.
constexpr int kSmallMTailBytes = 3072;
constexpr int kSmallMStagingOffset = 512;
constexpr int kSmallMStagingBytes = 2048;  // per epilogue warp: eight output rows x 32 columns x 2 bytes

// Slots of SmallMParams::timeline per CTA (global timer, nanoseconds).
enum : int {
  kTimelineEntry = 0,       // first instruction of the CTA
  kTimelineSetup = 1,       // barriers initialised, tensor memory allocated
  kTimelineDepsDone = 2,    // griddepcontrol.wait returned in the epilogue warps
  kTimelineFirstStage = 3,  // issuer 0 saw its first full stage
  kTimelineLastAcc = 4,     // epilogue saw the last accumulator of the CTA complete
  kTimelineExit = 5,        // epilogue done
  kTimelineSm = 6,          // SM id
  kTimelineDrained = 7,     // the last accumulator of the CTA has been read out of tensor memory
  kTimelineSlots = 8,
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned int sm_id() {
  unsigned int r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}

// Named barrier 3: the weight producer arrives without blocking once the stage barriers exist,
// every other warp waits for it (and for each other) before touching them.
__device__ __forceinline__ void setup_bar_arrive(uint32_t threads) {
  asm volatile("barrier.cta.arrive 3, %0;" ::"r"(threads) : "memory");
}
__device__ __forceinline__ void setup_bar_sync(uint32_t threads) {
  asm volatile("barrier.cta.sync 3, %0;" ::"r"(threads) : "memory");
}
// Named barrier 2 over the eight quantizer warps of the fused variant.
__device__ __forceinline__ void quant_bar_sync() {
  asm volatile("barrier.cta.sync 2, 256;" ::: "memory");
}

template <int KIND>
struct SmallMTile {
  static constexpr int kElemsPerMma = (KIND == kMxfp8) ? 32 : 64;
  static constexpr int kElemsPerStage = kElemsPerMma * 4;
  static constexpr int kKAtoms = (KIND == kMxfp8) ? 1 : (KIND == kNvfp4 ? 4 : 2);
  static constexpr int kWBytes = 128 * 128;
  static constexpr int kSfBytes = kKAtoms * 512;
  // Stage = weights | weight scales | activation scales | activation rows (m_pad * 128 B).
  static constexpr int kXOffset = kWBytes + 2 * kSfBytes;
  // TMEM columns: accumulator (segment parity a, issuer w) at (a * issuers + w) * m_pad, then
  // from SmallMParams::sf_col0 per issuer 16 columns of weight scales and 16 of activation scales.
  static constexpr int kSfColsPerIssuer = 32;
  static constexpr int kMaxStages = 10;
  __host__ __device__ static constexpr int stage_bytes(int m_pad) {
    return ((kXOffset + m_pad * 128 + 1023) / 1024) * 1024;
  }
};

// CTA that owns unit u when units are split as begin_c = c * U / G.
__device__ __forceinline__ int owner_of_unit(int u, int units, int ctas) {
  return static_cast<int>(((static_cast<long long>(u) + 1) * ctas - 1) / units);
}

// ----------------------------------------------------------------------------------------
// Fused activation quantization: what one quantizer warp does for one unit
// ----------------------------------------------------------------------------------------
// A "slot" is one warp-wide 16-byte-per-lane read of the raw rows in shared memory, i.e. 256
// consecutive BF16 elements: one row of an NVFP4 unit, or two rows of an MXFP8 unit (lanes
// 0..15 / 16..31). Warp q of the eight takes slot q and, for NVFP4 with more than eight rows,
// slot q + 8.
template <int KIND>
struct FusedQuant {
  static constexpr int kWarps = 8;
  static constexpr int kSlotsPerWarp = (KIND == kNvfp4) ? 2 : 1;

  __device__ static __forceinline__ int row_of(int slot, int lane) {
    return (KIND == kNvfp4) ? slot : 2 * slot + (lane >> 4);
  }
  __device__ static __forceinline__ int elem_of(int lane) {
    return (KIND == kNvfp4) ? lane * 8 : (lane & 15) * 8;
  }

  // Raw BF16 rows of a unit sit row-major behind the code tile: row r at r * kRawRowBytes.
  static constexpr int kRawRowBytes = SmallMTile<KIND>::kElemsPerStage * 2;
  __device__ static constexpr int raw_offset(int m_pad) {
    return SmallMTile<KIND>::kXOffset + m_pad * 128;
  }

  __device__ static __forceinline__ void load(const SmallMParams& p, const uint8_t* st, int wq,
                                              int lane, uint4 (&buf)[kSlotsPerWarp]) {
    const uint8_t* raw = st + raw_offset(p.m_pad);
#pragma unroll
    for (int s = 0; s < kSlotsPerWarp; ++s) {
      const int row = row_of(wq + s * kWarps, lane);
      buf[s] = (row < p.raw_rows)
                   ? *reinterpret_cast<const uint4*>(raw + row * kRawRowBytes + elem_of(lane) * 2)
                   : make_uint4(0, 0, 0, 0);
    }
  }

  // Quantize the loaded rows into the stage: codes where TMA would have put them (row r at
  // r * 128, 16-byte chunk j at position j ^ (r % 8)), scale bytes into the activation atoms.
  // Inverse rotary embedding of the lane's eight values (four interleaved pairs), in FP32
  // before anything is rounded: even' = fma(even, cos, odd * sin), odd' = fma(odd, cos,
  // -(even * sin)) (b12x/_lib/dense_gemm.py:3505-3530). `k` is the index of x[0] in the group's K.
  __device__ static __forceinline__ void inverse_rope(const SmallMParams& p, int row, int k,
                                                      float (&x)[8]) {
    const int d = k % p.rope_head_dim;
    if (d < p.rope_nope_dim || row >= p.m) return;
    const long long pos = p.rope_pos_i64
                              ? static_cast<const long long*>(p.rope_positions)[row]
                              : static_cast<long long>(static_cast<const int*>(p.rope_positions)[row]);
    const long long base = pos * p.rope_dim + ((d - p.rope_nope_dim) >> 1);
    const int half = p.rope_dim >> 1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float c, sn;
      if (p.rope_cache_f32) {
        c = static_cast<const float*>(p.rope_cos_sin)[base + j];
        sn = static_cast<const float*>(p.rope_cos_sin)[base + half + j];
      } else {
        c = __bfloat162float(static_cast<const __nv_bfloat16*>(p.rope_cos_sin)[base + j]);
        sn = __bfloat162float(static_cast<const __nv_bfloat16*>(p.rope_cos_sin)[base + half + j]);
      }
      const float e = x[2 * j], o = x[2 * j + 1];
      x[2 * j] = fmaf(e, c, __fmul_rn(o, sn));
      x[2 * j + 1] = fmaf(o, c, -__fmul_rn(e, sn));
    }
  }

  template <bool ROPE = false>
  __device__ static __forceinline__ void store(const SmallMParams& p, uint8_t* st, int wq, int lane,
                                               const uint4 (&buf)[kSlotsPerWarp], float gs,
                                               float gs_rcp, int k0 = 0) {
    using T = SmallMTile<KIND>;
    uint8_t* x_tile = st + T::kXOffset;
    uint8_t* sf_x = st + T::kWBytes + T::kSfBytes;
#pragma unroll
    for (int s = 0; s < kSlotsPerWarp; ++s) {
      const int row = row_of(wq + s * kWarps, lane);
      // Whole warps skip slots without a live row (the shuffles below stay warp-uniform).
      if (wq + s * kWarps >= ((KIND == kNvfp4) ? p.m : (p.m + 1) / 2)) continue;
      float x[8];
      unpack8<__nv_bfloat16>(buf[s], x);
      float amax;
      if constexpr (ROPE) {
        inverse_rope(p, row, k0 + elem_of(lane), x);
        amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
      } else {
        amax = amax8<__nv_bfloat16>(buf[s]);
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if (KIND == kNvfp4) {
        const float sc = __fmul_rn(gs, __fdiv_rn(amax, 6.0f));
        const uint32_t s_byte =
            static_cast<uint32_t>(__nv_cvt_float_to_fp8(sc, __NV_SATFINITE, __NV_E4M3)) & 0xFFu;
        const float t = __fmul_rn(e4m3_to_float(s_byte), gs_rcp);
        const float inv = (t == 0.0f) ? 0.0f : __frcp_rn(t);
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = __fmul_rn(x[i], inv);
        const uint32_t codes = e2m1x8(y);
        if (row < p.m) {
          const int b = lane * 4;  // byte of the row's 128
          *reinterpret_cast<uint32_t*>(x_tile + row * 128 + ((((b >> 4) ^ (row & 7))) << 4) + (b & 15)) =
              codes;
          const int kb = lane >> 1;  // 16-element block inside the unit
          if ((lane & 1) == 0) sf_x[(kb >> 2) * 512 + row * 16 + (kb & 3)] = static_cast<uint8_t>(s_byte);
        }
      } else {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t byte = ue8m0_from_amax(amax);
        const float inv = ue8m0_reciprocal(byte);
        uint2 out;
        out.x = e4m3x4(__fmul_rn(x[0], inv), __fmul_rn(x[1], inv), __fmul_rn(x[2], inv),
                       __fmul_rn(x[3], inv));
        out.y = e4m3x4(__fmul_rn(x[4], inv), __fmul_rn(x[5], inv), __fmul_rn(x[6], inv),
                       __fmul_rn(x[7], inv));
        if (row < p.m) {
          const int b = (lane & 15) * 8;
          *reinterpret_cast<uint2*>(x_tile + row * 128 + ((((b >> 4) ^ (row & 7))) << 4) + (b & 15)) = out;
          const int kb = (lane & 15) >> 2;  // 32-element block inside the unit
          if ((lane & 3) == 0) sf_x[row * 16 + kb] = static_cast<uint8_t>(byte);
        }
      }
    }
  }
};

// Final value of output element (mrow, n_global) of group `grp`: scale, round to the output
// type, store. With EPI also: add the bias and, if asked, emit the MXFP8 codes of the rounded
// row. A warp holds 32 consecutive columns of the row, which is exactly one scale block, so the
// block maximum is one warp-wide integer max of the magnitudes' bit patterns. Called by whole
// warps. Only the EPI instantiation goes through this function: the plain kernel keeps its
// store loop written out in place (routing it through here, with the predicate on n moved
// inside, cost 0.9 us at M = 16 and 2.8 us at M = 64).
template <bool EPI>
__device__ __forceinline__ void emit_output(const SmallMParams& p, float alpha, int lane, int grp,
                                            int mrow, int n_global, bool n_ok, float acc_value) {
  float v = acc_value * alpha;
  const size_t idx = static_cast<size_t>(grp) * p.c_group_elems +
                     static_cast<size_t>(mrow) * p.ldc + n_global;
  if constexpr (!EPI) {
    if (n_ok) {
      if (p.out_dtype == kOutBf16)
        static_cast<__nv_bfloat16*>(p.c)[idx] = __float2bfloat16_rn(v);
      else if (p.out_dtype == kOutFp16)
        static_cast<__half*>(p.c)[idx] = __float2half_rn(v);
      else
        static_cast<float*>(p.c)[idx] = v;
    }
    return;
  } else {
    if (p.bias != nullptr) v = add_bias_1(v, p.bias, p.out_dtype, n_global, p.n);
    float stored = v;
    if (p.out_dtype == kOutBf16) {
      const __nv_bfloat16 h = __float2bfloat16_rn(v);
      if (n_ok) static_cast<__nv_bfloat16*>(p.c)[idx] = h;
      stored = __bfloat162float(h);
    } else if (p.out_dtype == kOutFp16) {
      const __half h = __float2half_rn(v);
      if (n_ok) static_cast<__half*>(p.c)[idx] = h;
      stored = __half2float(h);
    } else if (n_ok) {
      static_cast<float*>(p.c)[idx] = v;
    }
    if (p.quant_values != nullptr) {
      const uint32_t mag = n_ok ? (__float_as_uint(stored) & 0x7FFFFFFFu) : 0u;
      const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, mag));
      const uint32_t byte = ue8m0_from_amax(amax);
      const float inv = ue8m0_reciprocal(byte);
      if (n_ok) {
        const int qcol = p.quant_col0 + grp * p.n + n_global;
        p.quant_values[static_cast<size_t>(mrow) * p.quant_ld + qcol] =
            static_cast<uint8_t>(e4m3x4(__fmul_rn(stored, inv), 0.0f, 0.0f, 0.0f) & 0xFFu);
        if (lane == 0) {
          if (p.quant_scale_rows)
            p.quant_scale_rows[static_cast<size_t>(mrow) * (p.quant_cols >> 5) + (qcol >> 5)] =
                static_cast<uint8_t>(byte);
          if (p.quant_scale_mma)
            p.quant_scale_mma[sf_atom_offset(mrow, qcol >> 5, (p.quant_cols + 127) >> 7)] =
                static_cast<uint8_t>(byte);
        }
      }
    }
  }
}

// EPI: the instantiation whose epilogue can add a bias and re-quantize the output rows; the
// plain one carries none of that code.
// Eight consecutive output rows x this warp's 32 columns, one value per row in each lane:
// turned around in the warp's 512 bytes of staging memory and stored as 16 bytes per lane (lane
// l: row l / 4, columns (l % 4) * 8 .. + 7). `vals` are final values (scaled); rows from
// `row0 + 8` on or beyond `m`, and columns beyond `n`, are not written.
__device__ __forceinline__ void store_rows8_packed(const SmallMParams& p, uint16_t* buf, int lane,
                                                   size_t c_group0, int row0, int col0,
                                                   const float (&vals)[8]) {
  __syncwarp();  // the previous eight rows have been read
#pragma unroll
  for (int r = 0; r < 8; ++r)
    buf[r * 32 + lane] = (p.out_dtype == kOutBf16) ? __bfloat16_as_ushort(__float2bfloat16_rn(vals[r]))
                                                   : __half_as_ushort(__float2half_rn(vals[r]));
  __syncwarp();
  const int r8 = lane >> 2;
  const int j4 = lane & 3;
  const int mrow = row0 + r8;
  const int col = col0 + j4 * 8;
  if (mrow < p.m && col < p.n) {
    uint16_t* dst = static_cast<uint16_t*>(p.c) + c_group0 + static_cast<size_t>(mrow) * p.ldc + col;
    if (col + 8 <= p.n) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(buf + r8 * 32 + j4 * 8);
    } else {
      for (int e = 0; col + e < p.n; ++e) dst[e] = buf[r8 * 32 + j4 * 8 + e];
    }
  }
}

template <int KIND, bool FUSED, bool EPI, bool ROPE = false>
__global__ void __launch_bounds__(FUSED ? 512 : 256, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_x, const SmallMParams p) {
  using T = SmallMTile<KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.num_stages * p.stage_bytes);
  uint64_t* empty_bar = full_bar + T::kMaxStages;
  uint64_t* ready_bar = empty_bar + T::kMaxStages;  // fused variant: codes and scales written
  uint64_t* acc_full_bar = ready_bar + T::kMaxStages;
  uint64_t* acc_empty_bar = acc_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;
  // Output staging (see packed_store); used only if it lies inside the launch's shared memory
  // (the ring's base is rounded up to 1 KiB, which may take up to 1023 bytes of the tail).
  uint8_t* staging = reinterpret_cast<uint8_t*>(full_bar) + kSmallMStagingOffset;
  const bool staging_fits = (staging + kSmallMStagingBytes) <= (smem_raw + p.smem_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* stamps =
      p.timeline ? p.timeline + static_cast<size_t>(blockIdx.x) * kTimelineSlots : nullptr;
  if (stamps && threadIdx.x == 0) {
    stamps[kTimelineEntry] = global_timer_ns();
    stamps[kTimelineSm] = sm_id();
  }

  // Let the next grid in the stream start its own prologue and weight stream now.
  grid_launch_dependents();

  // Unit arithmetic is 32-bit in the loops (the host rejects tiles * k_tiles >= 2^31); the
  // range ends use 64-bit products once.
  const int units = p.tiles * p.k_tiles;
  const int u_begin = static_cast<int>(static_cast<long long>(units) * blockIdx.x / gridDim.x);
  const int u_end = static_cast<int>(static_cast<long long>(units) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t smem_u32 = smem_addr_u32(smem);
  const uint32_t x_bytes = static_cast<uint32_t>(p.m_pad) * 128u;
  // Bytes of raw BF16 rows one stage of the fused variant receives.
  const uint32_t raw_bytes =
      FUSED ? static_cast<uint32_t>(p.raw_rows) * FusedQuant<KIND>::kRawRowBytes : 0u;

  uint32_t tmem_base = 0;
  if (warp == 0) {
    // ------------------------------ weight producer ------------------------------
    // This warp owns the stage barriers: it creates them and starts the weight stream without
    // waiting for tensor memory or for the other warps, which only need the barriers to exist
    // by the time they pass the set-up barrier below.
    if (lane == 0) {
      *abort_flag = 0;
      for (int s = 0; s < p.num_stages; ++s) {
        mbar_init(&full_bar[s], 2);  // weight producer + activation producer
        mbar_init(&empty_bar[s], 1);
        if (FUSED) mbar_init(&ready_bar[s], FusedQuant<KIND>::kWarps);
      }
      fence_mbar_init();
      fence_proxy_async_smem();
      tma_prefetch_desc(&map_w);
    }
    __syncwarp();
    setup_bar_arrive(blockDim.x);
    // A weight of more than 128 rows is never the output of a predecessor that releases its
    // dependents early (decode GEMMs write at most 128 rows, the row quantizers release early
    // only for matrices of at most 128 rows), so its stream starts at once.
    if (p.wait_for_weights) grid_dependency_wait();
    int stage = 0;
    uint32_t phase = 0;
    const int tile0 = u_begin / p.k_tiles;  // over all groups
    int kt = u_begin - tile0 * p.k_tiles;
    int grp = tile0 / p.tiles_per_group;    // group and tile inside it, kept by increments
    int local = tile0 - grp * p.tiles_per_group;
    for (int u = u_begin; u < u_end; ++u) {
      if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
        *abort_flag = 1;
        if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
        break;
      }
      if (elect_one()) {
        uint8_t* st = smem + stage * p.stage_bytes;
        uint64_t* bar = &full_bar[stage];
        const int katom0 = kt * T::kKAtoms;
        const int katoms = min(T::kKAtoms, p.k_atoms_total - katom0);
        const uint32_t sf_bytes = static_cast<uint32_t>(katoms) * 512u;
        mbar_arrive_expect_tx(bar, T::kWBytes + sf_bytes);
        tma_load_3d(st, &map_w, bar, kt * 128, local * 128, grp);
        bulk_load(st + T::kWBytes,
                  p.sf_w + grp * p.sf_w_group_bytes +
                      (static_cast<size_t>(local) * p.k_atoms_total + katom0) * 512,
                  sf_bytes, bar);
      }
      __syncwarp();
      if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
      if (++kt == p.k_tiles) {
        kt = 0;
        if (++local == p.tiles_per_group) { local = 0; ++grp; }
      }
    }
  } else {
    if (warp == 1) {
      if (lane == 0) {
        for (int a = 0; a < 2; ++a) {
          mbar_init(&acc_full_bar[a], 2);  // one arrival per issuer warp
          mbar_init(&acc_empty_bar[a], 4);
        }
        fence_mbar_init();
      }
      __syncwarp();
      tmem_alloc(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
    }
    if (warp == 6 && lane == 0) tma_prefetch_desc(&map_x);
    tc_fence_before_sync();
    setup_bar_sync(blockDim.x);
    tc_fence_after_sync();
    if (stamps && threadIdx.x == 32) stamps[kTimelineSetup] = global_timer_ns();
    // Column offset of this CTA's allocation (another CTA may hold the rest of the SM's tensor
    // memory); the lane field must be zero. Otherwise nothing is issued and everyone leaves
    // through the common tear-down (the producer sees the abort flag).
    tmem_base = *tmem_slot;
    const bool tmem_ok = (tmem_base >> 16) == 0;
    if (!tmem_ok && threadIdx.x == 32) {
      *abort_flag = 1;
      if (p.status) atomicMax(p.status, kStatusTmemLayout);
    }

    if (!tmem_ok) {
      // nothing
    } else if (warp == 6) {
      // ------------------------------ activation producer ------------------------------
      // Codes and scale atoms, or (fused variant) the raw BF16 rows the quantizer warps turn
      // into codes and scales.
      grid_dependency_wait();  // activations may come from the previous grid
      int stage = 0;
      uint32_t phase = 0;
      const int tile0 = u_begin / p.k_tiles;
      int kt = u_begin - tile0 * p.k_tiles;
      int grp = tile0 / p.tiles_per_group;
      int local = tile0 - grp * p.tiles_per_group;
      for (int u = u_begin; u < u_end; ++u) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + stage * p.stage_bytes;
          uint64_t* bar = &full_bar[stage];
          const int katom0 = kt * T::kKAtoms;
          const int katoms = min(T::kKAtoms, p.k_atoms_total - katom0);
          const uint32_t sf_bytes = static_cast<uint32_t>(katoms) * 512u;
          if (FUSED) {
            mbar_arrive_expect_tx(bar, raw_bytes);
            tma_load_3d(st + FusedQuant<KIND>::raw_offset(p.m_pad), &map_x, bar,
                        kt * T::kElemsPerStage, 0, grp);
          } else {
            mbar_arrive_expect_tx(bar, x_bytes + sf_bytes);
            tma_load_3d(st + T::kXOffset, &map_x, bar, kt * 128, 0, grp);
            bulk_load(st + T::kWBytes + T::kSfBytes,
                      p.sf_x + grp * p.sf_x_group_bytes + static_cast<size_t>(katom0) * 512,
                      sf_bytes, bar);
          }
        }
        __syncwarp();
        if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
        if (++kt == p.k_tiles) {
          kt = 0;
          if (++local == p.tiles_per_group) { local = 0; ++grp; }
        }
      }
    } else if (FUSED && warp >= 8) {
      // ------------------------------ activation quantizers ------------------------------
      using Q = FusedQuant<KIND>;
      const int wq = warp - 8;
      // Rows and scale columns nobody writes must hold finite codes and neutral scales: clear
      // the activation part of every stage once (zero codes; scale byte 0 = +0 in E4M3, 127 =
      // 2^0 in UE8M0).
      {
        const uint32_t sf_fill = (KIND == kNvfp4) ? 0u : 0x7F7F7F7Fu;
        const int t = threadIdx.x - 256;
        for (int s = 0; s < p.num_stages; ++s) {
          uint8_t* st = smem + s * p.stage_bytes;
          for (int i = t * 16; i < T::kSfBytes; i += 256 * 16)
            *reinterpret_cast<uint4*>(st + T::kWBytes + T::kSfBytes + i) =
                make_uint4(sf_fill, sf_fill, sf_fill, sf_fill);
          for (int i = t * 16; i < static_cast<int>(x_bytes); i += 256 * 16)
            *reinterpret_cast<uint4*>(st + T::kXOffset + i) = make_uint4(0, 0, 0, 0);
        }
      }
      quant_bar_sync();
      float gs = 1.0f, gs_rcp = 1.0f;
      if (KIND == kNvfp4) {
        grid_dependency_wait();  // the scale may come from the previous grid
        gs = *p.x_gs;
        gs_rcp = (gs == 0.0f) ? 0.0f : __frcp_rn(gs);
      }
      if constexpr (ROPE) grid_dependency_wait();  // positions may come from the previous grid
      int stage = 0;
      uint32_t phase = 0;
      int kt_q = u_begin % p.k_tiles;   // k-tile of the unit (used by the ROPE variant)
      for (int u = u_begin; u < u_end; ++u) {
        // Weights and raw rows of the unit have landed (which also means the tensor core is
        // done with whatever the stage held before).
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
          break;
        }
        uint8_t* st = smem + stage * p.stage_bytes;
        uint4 raw[Q::kSlotsPerWarp];
        Q::load(p, st, wq, lane, raw);
        Q::template store<ROPE>(p, st, wq, lane, raw, gs, gs_rcp, kt_q * T::kElemsPerStage);
        if (++kt_q == p.k_tiles) kt_q = 0;
        // The tensor core reads the stage through the async proxy.
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready_bar[stage]);
        if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
      }
    } else if (warp == 1 || warp == 7) {
      // ------------------------------ MMA issuers ------------------------------
      // Unit number q of the CTA's range (q = u - u_begin) belongs to issuer q % issuers. Both
      // warps walk every unit to keep the ring position; each arrives once per segment on the
      // accumulator barrier, through a commit if it issued anything there, plainly otherwise.
      const int me = (warp == 1) ? 0 : 1;
      const uint32_t idesc_base = make_idesc_block_scaled(
          128, static_cast<uint32_t>(p.m_pad), KIND == kMxfp8 ? 0u : 1u, KIND == kNvfp4 ? 0u : 1u);
      const uint32_t sfw_col = tmem_base + p.sf_col0 + me * T::kSfColsPerIssuer;
      const uint32_t sfx_col = sfw_col + 16;
      int stage = 0;
      uint32_t phase = 0;
      int seg = 0;
      bool ok = true;
      bool stamped = false;
      int u = u_begin;
      while (u < u_end && ok) {
        const int tile = u / p.k_tiles;
        const int tile_end = (tile + 1) * p.k_tiles;
        const int seg_end = tile_end < u_end ? tile_end : u_end;
        int kt = u - tile * p.k_tiles;
        const int acc = seg & 1;
        if (!mbar_wait_bounded(&acc_empty_bar[acc], ((seg >> 1) & 1) ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_taddr = tmem_base + static_cast<uint32_t>((acc * p.issuers + me) * p.m_pad);
        bool first = true;
        for (; u < seg_end; ++u, ++kt) {
          const bool mine = (p.issuers == 2) ? (((u - u_begin) & 1) == me) : (me == 0);
          if (mine) {
            // Fused variant: the stage is usable once the quantizer warps have written codes
            // and scales ("ready"); the full barrier has then long completed, and waiting on it
            // as well keeps the issuer a direct observer of the TMA writes.
            if ((FUSED && !mbar_wait_bounded(&ready_bar[stage], phase, abort_flag)) ||
                !mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
              *abort_flag = 1;
              if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (stamps && !stamped && me == 0 && lane == 0) {
              stamps[kTimelineFirstStage] = global_timer_ns();
              stamped = true;
            }
            const uint32_t st = smem_u32 + stage * p.stage_bytes;
            const int mmas =
                min(4, (p.k - kt * T::kElemsPerStage + T::kElemsPerMma - 1) / T::kElemsPerMma);
            if (elect_one()) {
              const uint64_t sf_desc = make_sf_chunk_desc(st + T::kWBytes);
#pragma unroll
              for (int ka = 0; ka < T::kKAtoms; ++ka) {
                tc_copy_sf_atom(sfw_col + ka * 4, sf_desc + ((ka * 512) >> 4));
                tc_copy_sf_atom(sfx_col + ka * 4, sf_desc + ((T::kSfBytes + ka * 512) >> 4));
              }
              const uint64_t wdesc = make_kmajor_sw128_desc(st);
              const uint64_t xdesc = make_kmajor_sw128_desc(st + T::kXOffset);
              for (int j = 0; j < mmas; ++j) {
                const uint32_t accumulate = (first && j == 0) ? 0u : 1u;
                if (KIND == kMxfp8)
                  tc_mma_mxf8(d_taddr, wdesc + 2 * j, xdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, j, j), accumulate, sfw_col, sfx_col);
                else if (KIND == kMxfp4)   // two UE8M0 bytes per MMA: bytes 0-1 or 2-3 of atom j / 2
                  tc_mma_mxf4(d_taddr, wdesc + 2 * j, xdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, (j & 1) * 2, (j & 1) * 2), accumulate,
                              sfw_col + (j >> 1) * 4, sfx_col + (j >> 1) * 4);
                else
                  tc_mma_nvf4(d_taddr, wdesc + 2 * j, xdesc + 2 * j, idesc_base, accumulate,
                              sfw_col + j * 4, sfx_col + j * 4);
              }
              tc_commit(&empty_bar[stage]);
              // Last unit of this issuer in the segment: the next one of its parity is past the end.
              if (u + p.issuers >= seg_end) tc_commit(&acc_full_bar[acc]);
            }
            __syncwarp();
            first = false;
          }
          if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
        }
        if (ok && first && lane == 0) mbar_arrive(&acc_full_bar[acc]);  // nothing issued here
        ++seg;
      }
    } else if (warp >= 2 && warp <= 5) {
      // ------------------------------ epilogue ------------------------------
      // alpha, C, the partial slots and the counters may be written or still read by the
      // previous grid.
      grid_dependency_wait();
      if (stamps && threadIdx.x == 64) stamps[kTimelineDepsDone] = global_timer_ns();
      const int quarter = warp & 3;
      const int n_local = quarter * 32 + lane;          // weight row inside the tile
      const float alpha = p.alpha ? *p.alpha : 1.0f;
      const size_t slot_floats = static_cast<size_t>(p.m_pad) * 128;
      int seg = 0;
      int u = u_begin;
      while (u < u_end) {
        const int tile = u / p.k_tiles;
        const int tile_begin = tile * p.k_tiles;
        const int tile_end = tile_begin + p.k_tiles;
        const int seg_end = tile_end < u_end ? tile_end : u_end;
        const bool whole = (u == tile_begin) && (seg_end == tile_end);
        const int acc = seg & 1;
        // The four epilogue warps meet at barriers further down, so they leave together or not
        // at all: the outcome of the wait is AND-reduced across them first.
        if (!epilogue_bar_and(mbar_wait_bounded(&acc_full_bar[acc], (seg >> 1) & 1, abort_flag))) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusEpilogueTimeout);
          break;
        }
        tc_fence_after_sync();
        if (stamps && threadIdx.x == 64 && seg_end == u_end) stamps[kTimelineLastAcc] = global_timer_ns();
        // Which issuers hold a partial of this segment: both, unless it is a single unit.
        const int first_issuer = (p.issuers == 2) ? ((u - u_begin) & 1) : 0;
        const bool both = (p.issuers == 2) && (seg_end - u >= 2);
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t taddr0 =
            lane_base + static_cast<uint32_t>((acc * p.issuers + (both ? 0 : first_issuer)) * p.m_pad);
        const uint32_t taddr1 = lane_base + static_cast<uint32_t>((acc * p.issuers + 1) * p.m_pad);
        const int grp = tile / p.tiles_per_group;
        const int n_global = (tile - grp * p.tiles_per_group) * 128 + n_local;  // inside the group
        const bool n_ok = n_global < p.n;
        const size_t c_group0 = static_cast<size_t>(grp) * p.c_group_elems;
        int first_cta = 0, segments = 1, slot = 0;
        if (!whole) {
          first_cta = owner_of_unit(tile_begin, units, gridDim.x);
          segments = owner_of_unit(tile_end - 1, units, gridDim.x) - first_cta + 1;
          slot = static_cast<int>(blockIdx.x) - first_cta;
        }
        float* my_slot = p.partials + (static_cast<size_t>(tile) * p.max_segments + slot) * slot_floats;
        if ((!EPI || p.quant_values == nullptr) && whole && p.packed_store && staging_fits) {
          // A lane holds one output column of every row, so storing from registers means one
          // 2-byte store per row and lane (64 bytes per warp instruction), and those stores
          // measured 75 ns apiece per warp: 1 us of a 16-row tile's epilogue and 4 us of a
          // 64-row one. Instead each warp turns eight rows x its 32 columns around in its own
          // 512 bytes of shared memory and stores 16 bytes per lane: one instruction per
          // eight rows, no barrier between the warps.
          const int tile_n0 = (tile - grp * p.tiles_per_group) * 128;
          uint16_t* buf = reinterpret_cast<uint16_t*>(staging) + quarter * 256;
          const int col0 = tile_n0 + quarter * 32;
          for (int c0 = 0; c0 < p.m_pad && c0 < p.m; c0 += 16) {
            uint32_t raw[16];
            tmem_load_16cols(taddr0 + c0, raw);
            if (both) {
              uint32_t other[16];
              tmem_load_16cols(taddr1 + c0, other);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                raw[i] = __float_as_uint(__fadd_rn(__uint_as_float(raw[i]), __uint_as_float(other[i])));
            } else {
              tmem_load_wait();
            }
            if (stamps && threadIdx.x == 64 && seg_end == u_end && (c0 + 16 >= p.m_pad || c0 + 16 >= p.m))
              stamps[kTimelineDrained] = global_timer_ns();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (c0 + 8 * h >= p.m) break;  // uniform: nothing but padding rows from here on
              float vals[8];
#pragma unroll
              for (int r = 0; r < 8; ++r) {
                vals[r] = __uint_as_float(raw[8 * h + r]) * alpha;
                if constexpr (EPI) {  // bias only (a quantized output keeps the per-lane path)
                  if (p.bias != nullptr) vals[r] = add_bias_1(vals[r], p.bias, p.out_dtype, n_global, p.n);
                }
              }
              store_rows8_packed(p, buf, lane, c_group0, c0 + 8 * h, col0, vals);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
          u = seg_end;
          ++seg;
          continue;
        }
        for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
          uint32_t raw[16];
          tmem_load_16cols(taddr0 + c0, raw);
          if (both) {
            uint32_t other[16];
            tmem_load_16cols(taddr1 + c0, other);
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i)
              raw[i] = __float_as_uint(__fadd_rn(__uint_as_float(raw[i]), __uint_as_float(other[i])));
          } else {
            tmem_load_wait();
          }
          if (stamps && threadIdx.x == 64 && seg_end == u_end && c0 + 16 >= p.m_pad)
            stamps[kTimelineDrained] = global_timer_ns();
          if (whole) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int mrow = c0 + i;
              if constexpr (EPI) {
                if (mrow < p.m)
                  emit_output<true>(p, alpha, lane, grp, mrow, n_global, n_ok, __uint_as_float(raw[i]));
              } else if (n_ok && mrow < p.m) {
                const float v = __uint_as_float(raw[i]) * alpha;
                const size_t idx = c_group0 + static_cast<size_t>(mrow) * p.ldc + n_global;
                if (p.out_dtype == kOutBf16)
                  static_cast<__nv_bfloat16*>(p.c)[idx] = __float2bfloat16_rn(v);
                else if (p.out_dtype == kOutFp16)
                  static_cast<__half*>(p.c)[idx] = __float2half_rn(v);
                else
                  static_cast<float*>(p.c)[idx] = v;
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              my_slot[static_cast<size_t>(c0 + i) * 128 + n_local] = __uint_as_float(raw[i]);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);

        if (!whole) {
          // Publish the partial, count the arrival, and let the last arriver finish the tile.
          __threadfence();
          epilogue_bar_sync();
          if (warp == 2 && lane == 0) {
            const int prev = atomicAdd(&p.counters[tile], 1);
            *last_flag = (prev == segments - 1) ? 1 : 0;
            if (prev == segments - 1) p.counters[tile] = 0;
          }
          epilogue_bar_sync();
          if (*last_flag) {
            __threadfence();
            const float* tile_slots = p.partials + static_cast<size_t>(tile) * p.max_segments * slot_floats;
            // Eight rows at a time so that 8 x segments loads are in flight per thread.
            for (int m0 = 0; m0 < p.m; m0 += 8) {
              float sum[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
              for (int s = 0; s < segments; ++s) {
                const float* src = tile_slots + s * slot_floats + static_cast<size_t>(m0) * 128 + n_local;
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (m0 + i < p.m) ? __ldcg(src + i * 128) : 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] += v[i];
              }
              if ((!EPI || p.quant_values == nullptr) && p.packed_store && staging_fits) {
                float vals[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  vals[i] = sum[i] * alpha;
                  if constexpr (EPI) {
                    if (p.bias != nullptr) vals[i] = add_bias_1(vals[i], p.bias, p.out_dtype, n_global, p.n);
                  }
                }
                store_rows8_packed(p, reinterpret_cast<uint16_t*>(staging) + quarter * 256, lane,
                                   c_group0, m0,
                                   (tile - grp * p.tiles_per_group) * 128 + quarter * 32, vals);
                continue;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int mrow = m0 + i;
                if constexpr (EPI) {
                  if (mrow < p.m) emit_output<true>(p, alpha, lane, grp, mrow, n_global, n_ok, sum[i]);
                } else if (n_ok && mrow < p.m) {
                  const float v = sum[i] * alpha;
                  const size_t idx = c_group0 + static_cast<size_t>(mrow) * p.ldc + n_global;
                  if (p.out_dtype == kOutBf16)
                    static_cast<__nv_bfloat16*>(p.c)[idx] = __float2bfloat16_rn(v);
                  else if (p.out_dtype == kOutFp16)
                    static_cast<__half*>(p.c)[idx] = __float2half_rn(v);
                  else
                    static_cast<float*>(p.c)[idx] = v;
                }
              }
            }
          }
          epilogue_bar_sync();
        }
        u = seg_end;
        ++seg;
      }
      if (stamps && threadIdx.x == 64) stamps[kTimelineExit] = global_timer_ns();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  drain_after_abort(abort_flag);
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(*tmem_slot, static_cast<uint32_t>(p.tmem_cols));
  }
}

}  // namespace b12x_b200
