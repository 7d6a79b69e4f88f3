// Persistent, warp-specialised block-scaled GEMM for sm_100a:
//
//     C[M,N] = cvt(alpha * sum_k (A[M,K] . SFA) (B[N,K] . SFB)^T)
//
// A and B are K-major. Two operand recipes share one kernel template:
//   kMxfp8 : E4M3 codes, one UE8M0 scale per 32 elements of K  (tcgen05 kind::mxf8f6f4)
//   kNvfp4 : packed E2M1 codes (low nibble = even k), one UE4M3 scale per 16 elements
//   kMxfp4 : packed E2M1 codes, one UE8M0 scale per 32 elements (kind::mxf4nvf4, scale_vec::2X):
//            a 512-byte scale atom covers 128 elements of K, i.e. two K = 64 instructions
//   kFp8   : E4M3 codes without block scales (tcgen05 kind::f8f6f4); alpha is the only scale.
//            No scale bytes are loaded or copied to tensor memory, and the columns they would
//            take hold a second accumulator instead.
//            (tcgen05 kind::mxf4nvf4, scale_vec::4X)
// Scale factors live in global memory as 512-byte atoms covering 128 rows x 4 scale columns,
// atom order [row_tile][k_tile], byte (r%32)*16 + ((r/32)%4)*4 + (kb%4) inside an atom. That is
// byte for byte the chunk tcgen05.cp moves from shared to tensor memory, so the atoms are
// streamed with plain bulk copies and never re-arranged.
//
// Roles inside one CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = epilogue (TMEM -> registers -> global). Accumulators sit in TMEM, double
// buffered when 2*BN plus the scale columns fit in the 512 columns, so the epilogue of tile i
// overlaps the main loop of tile i+1. One stage of the shared-memory ring holds 128 bytes of K
// for 128 rows of A and BN rows of B plus that slice's scale atoms.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace b12x_b200 {

enum OperandKind : int { kMxfp8 = 0, kNvfp4 = 1, kFp8 = 2, kMxfp4 = 3 };
enum OutDtype : int { kOutBf16 = 0, kOutFp16 = 1, kOutFp32 = 2 };

template <int KIND, int BN>
struct GemmTile {
  // Tiles start on 64-row boundaries of B: the MMA accepts a scale-factor address shifted by two
  // TMEM columns (64 rows) but faults on an odd column shift, so 32-row granularity is out.
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN must be a multiple of 64 in [64,256]");
  static constexpr int BM = 128;
  static constexpr int kRowBytes = 128;                       // bytes of K per stage and row
  static constexpr int kMmasPerStage = 4;                     // 32 bytes of K per instruction
  static constexpr bool kScaled = (KIND != kFp8);
  static constexpr int kElemsPerMma = (KIND == kNvfp4 || KIND == kMxfp4) ? 64 : 32;
  static constexpr int kElemsPerStage = kElemsPerMma * kMmasPerStage;
  static constexpr int kSfVec = (KIND == kNvfp4) ? 16 : 32;
  static constexpr int kElemsPerAtom = kSfVec * 4;            // K covered by one scale atom
  // scale atoms per stage: 1 (MXFP8), 4 (NVFP4), none (plain FP8)
  static constexpr int kKAtoms = kScaled ? kElemsPerStage / kElemsPerAtom : 0;
  // Row atoms of SFB a tile can touch: tiles that are not multiples of 128 start inside an atom.
  static constexpr int kSfbRowAtoms = (BN % 128 == 0) ? BN / 128 : (BN + 64 + 127) / 128;
  static constexpr int kABytes = BM * kRowBytes;
  static constexpr int kBBytes = BN * kRowBytes;
  static constexpr int kSfaBytes = kKAtoms * 512;
  static constexpr int kSfbBytes = kSfbRowAtoms * kKAtoms * 512;
  static constexpr int kStageBytes =
      ((kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024) * 1024;
  static constexpr int kSfaCols = kKAtoms * 4;
  static constexpr int kSfbCols = kSfbRowAtoms * kKAtoms * 4;
  static constexpr int kAccStages = (2 * BN + kSfaCols + kSfbCols <= 512) ? 2 : 1;
  static constexpr int kSfaCol0 = kAccStages * BN;
  static constexpr int kSfbCol0 = kSfaCol0 + kSfaCols;
  static_assert(kSfbCol0 + kSfbCols <= 512, "tensor memory overflow");
  static constexpr int kMaxSmem = 227 * 1024;
  static constexpr int kBarrierBytes = 1024;
  // Output staging for the TMA-store epilogue: 128 rows x 128 columns of 2-byte values, as two
  // 128-byte-swizzled sub-tiles of 64 columns; wider tiles go through it in passes.
  static constexpr int kCStageBytes = 128 * 128 * 2;
  static constexpr int kStagesRaw = (kMaxSmem - kBarrierBytes - 1024 - kCStageBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static_assert(kStages >= 2, "not enough shared memory for a pipeline");
  static constexpr int kSmemBytes = kStages * kStageBytes + kCStageBytes + kBarrierBytes + 1024;
};

struct GemmParams {
  const uint8_t* sfa;    // scale atoms of A: [ceil(M/128)][k_atoms][512]
  const uint8_t* sfb;    // scale atoms of B: [ceil(N/128)][k_atoms][512]
  void* c;               // [M, ldc] row-major
  const float* alpha;    // device scalar, may be null (= 1)
  int* status;           // device status word, may be null
  int m, n, k;           // K in elements
  int ldc;               // elements
  int out_dtype;         // OutDtype
  int tiles_m, tiles_n;
  int k_atoms_total;     // scale atoms along K in global memory
  int group_m;           // tile-order grouping along M (L2 reuse)
  int num_stages;        // shared-memory ring depth actually used (<= GemmTile::kStages)
  int use_tma_store;     // 2-byte outputs with 16-byte aligned rows: stage in smem, TMA store
  const void* bias;      // [N] values of the output dtype added to every row, or null
  // Grouped (batched) GEMM: `groups` independent problems of the same shape, operands stacked
  // as [groups, rows, K], scale atoms and outputs group after group. Tiles of all groups form
  // one list for the persistent scheduler.
  int groups;
  long long sfa_group_bytes, sfb_group_bytes;  // scale atoms of one group
  long long c_group_elems;                     // output elements between groups
};

// Tile index of the whole (grouped) problem -> group and tile inside the group.
__device__ __forceinline__ void split_group(int tile, int tiles_per_group, int& group, int& local) {
  group = tile / tiles_per_group;
  local = tile - group * tiles_per_group;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m,
                                            int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int in_group = tile - g * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Bias epilogue on 32 consecutive output columns of one row (`vals` already carry alpha). The
// result is what adding a bias tensor to the stored output gives: for 2-byte outputs the
// product is first rounded to the output type, then the sum is formed in FP32 and rounded again
// by the store (out = cvt(float(cvt(alpha * acc)) + float(bias[n]))); for FP32 outputs it is a
// plain FP32 add. Every thread of a warp asks for the same 32 bias values, so the loads
// broadcast; columns at or beyond N read as zero.
__device__ __forceinline__ void add_bias_32(float (&vals)[32], const void* bias, int out_dtype,
                                            int col0, int n) {
  if (bias == nullptr) return;
  if (out_dtype == kOutFp32) {
    const float* b = static_cast<const float*>(bias);
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < n) vals[i] = __fadd_rn(vals[i], __ldg(b + col0 + i));
    return;
  }
  const uint16_t* b = static_cast<const uint16_t*>(bias);
  uint32_t packed[16];
  if (col0 + 32 <= n && ((reinterpret_cast<uintptr_t>(b + col0) & 15) == 0)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(b + col0) + i);
      packed[4 * i] = v.x; packed[4 * i + 1] = v.y; packed[4 * i + 2] = v.z; packed[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t lo = (col0 + 2 * i < n) ? __ldg(b + col0 + 2 * i) : 0u;
      const uint32_t hi = (col0 + 2 * i + 1 < n) ? __ldg(b + col0 + 2 * i + 1) : 0u;
      packed[i] = lo | (hi << 16);
    }
  }
  if (out_dtype == kOutBf16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t y = pack_bf16x2(vals[2 * i], vals[2 * i + 1]);
      vals[2 * i] = __fadd_rn(__uint_as_float(y << 16), __uint_as_float(packed[i] << 16));
      vals[2 * i + 1] = __fadd_rn(__uint_as_float(y & 0xFFFF0000u), __uint_as_float(packed[i] & 0xFFFF0000u));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t y = pack_f16x2(vals[2 * i], vals[2 * i + 1]);
      const float2 yf = __half22float2(*reinterpret_cast<const __half2*>(&y));
      const float2 bf = __half22float2(*reinterpret_cast<const __half2*>(&packed[i]));
      vals[2 * i] = __fadd_rn(yf.x, bf.x);
      vals[2 * i + 1] = __fadd_rn(yf.y, bf.y);
    }
  }
}

// Same for a single output value (column `col`).
__device__ __forceinline__ float add_bias_1(float v, const void* bias, int out_dtype, int col, int n) {
  if (bias == nullptr || col >= n) return v;
  if (out_dtype == kOutFp32) return __fadd_rn(v, __ldg(static_cast<const float*>(bias) + col));
  const uint32_t b = __ldg(static_cast<const uint16_t*>(bias) + col);
  if (out_dtype == kOutBf16)
    return __fadd_rn(__bfloat162float(__float2bfloat16_rn(v)), __uint_as_float(b << 16));
  const __half_raw hr = {static_cast<unsigned short>(b)};
  return __fadd_rn(__half2float(__float2half_rn(v)), __half2float(__half(hr)));
}

// Writes 32 consecutive output columns of one row of group `group`. `vals` already carry alpha.
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, int group, int row, int col0,
                                                const float (&vals)[32]) {
  if (row >= p.m || col0 >= p.n) return;
  const size_t base = static_cast<size_t>(group) * p.c_group_elems +
                      static_cast<size_t>(row) * p.ldc + col0;
  const bool full = (col0 + 32 <= p.n);
  if (p.out_dtype == kOutFp32) {
    float* out = static_cast<float*>(p.c) + base;
    if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(out)[i] =
            make_float4(vals[4 * i], vals[4 * i + 1], vals[4 * i + 2], vals[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.n) out[i] = vals[i];
    }
    return;
  }
  uint16_t* out = static_cast<uint16_t*>(p.c) + base;
  uint32_t packed[16];
  if (p.out_dtype == kOutBf16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) packed[i] = pack_bf16x2(vals[2 * i], vals[2 * i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) packed[i] = pack_f16x2(vals[2 * i], vals[2 * i + 1]);
  }
  if (full && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<uint4*>(out)[i] =
          make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < p.n)
        out[i] = static_cast<uint16_t>((i & 1) ? (packed[i >> 1] >> 16) : (packed[i >> 1] & 0xFFFF));
  }
}

// BIAS: the instantiation with the bias epilogue (the plain one carries none of its code).
template <int KIND, int BN, bool BIAS>
__global__ void __launch_bounds__(192, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  using T = GemmTile<KIND, BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled operand tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* c_stage = smem + T::kStages * T::kStageBytes;
  uint8_t* bar_area = c_stage + T::kCStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_area);
  uint64_t* empty_bar = full_bar + T::kStages;
  uint64_t* acc_full_bar = empty_bar + T::kStages;
  uint64_t* acc_empty_bar = acc_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.use_tma_store) tma_prefetch_desc(&map_c);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // The CTA owns all 512 columns (one CTA per SM), so the allocation starts at column 0 and
  // every TMEM address below is a compile-time constant. Anything else is reported and the
  // CTA leaves without touching tensor memory.
  const uint32_t tmem_base = *tmem_slot;
  if (tmem_base != 0) {
    if (threadIdx.x == 0 && p.status) atomicMax(p.status, kStatusTmemLayout);
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
    return;
  }

  const int tiles_per_group = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_group * p.groups;
  const int k_tiles = (p.k + T::kElemsPerStage - 1) / T::kElemsPerStage;
  const int n_row_atoms_b = (p.n + 127) / 128;
  const uint32_t smem_u32 = smem_addr_u32(smem);

  // All lanes of the producer and MMA warps walk their loops together (waits included) and one
  // elected lane issues: the loop state stays warp-uniform, which keeps descriptor arithmetic
  // on the uniform datapath instead of costing a register shuffle per tcgen05 operand.
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn, grp, local;
      split_group(tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const int m0 = tm * T::BM;
      const int n0 = tn * BN;
      const int sfb_atom0 = n0 / 128;
      const int sfb_atoms = min((n0 % 128 + BN + 127) / 128, n_row_atoms_b - sfb_atom0);
      const uint8_t* sfa_src = p.sfa + grp * p.sfa_group_bytes + static_cast<size_t>(tm) * p.k_atoms_total * 512;
      const uint8_t* sfb_src = p.sfb + grp * p.sfb_group_bytes + static_cast<size_t>(sfb_atom0) * p.k_atoms_total * 512;
      for (int kt = 0; kt < k_tiles; ++kt) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
          ok = false;
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + stage * T::kStageBytes;
          uint64_t* bar = &full_bar[stage];
          const int katom0 = kt * T::kKAtoms;
          const int katoms = min(T::kKAtoms, p.k_atoms_total - katom0);
          const uint32_t sf_bytes = static_cast<uint32_t>(katoms) * 512u;
          mbar_arrive_expect_tx(bar, T::kABytes + T::kBBytes +
                                         (T::kScaled ? sf_bytes * (1 + sfb_atoms) : 0u));
          tma_load_3d(st, &map_a, bar, kt * T::kRowBytes, m0, grp);
          tma_load_3d(st + T::kABytes, &map_b, bar, kt * T::kRowBytes, n0, grp);
          if constexpr (T::kScaled) {
            bulk_load(st + T::kABytes + T::kBBytes, sfa_src + static_cast<size_t>(katom0) * 512,
                      sf_bytes, bar);
            for (int ra = 0; ra < sfb_atoms; ++ra)
              bulk_load(st + T::kABytes + T::kBBytes + T::kSfaBytes + ra * T::kKAtoms * 512,
                        sfb_src + (static_cast<size_t>(ra) * p.k_atoms_total + katom0) * 512,
                        sf_bytes, bar);
          }
        }
        __syncwarp();
        if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc_base =
        KIND == kFp8 ? make_idesc_f8(128, BN)
                     : make_idesc_block_scaled(128, BN, KIND == kMxfp8 ? 0u : 1u,
                                               KIND == kNvfp4 ? 0u : 1u);
    int stage = 0;
    uint32_t phase = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++iter) {
      int tm, tn, grp, local;
      split_group(tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const uint32_t sfb_col_shift = static_cast<uint32_t>(((tn * BN) % 128) / 32);
      const int acc = iter % T::kAccStages;
      const uint32_t acc_phase = (iter / T::kAccStages) & 1;
      if (!mbar_wait_bounded(&acc_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
        *abort_flag = 1;
        if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_taddr = acc * BN;
      const uint32_t sfb_taddr = T::kSfbCol0 + sfb_col_shift;
      for (int kt = 0; kt < k_tiles; ++kt) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t st = smem_u32 + stage * T::kStageBytes;
        const int mmas = min(T::kMmasPerStage,
                             (p.k - kt * T::kElemsPerStage + T::kElemsPerMma - 1) / T::kElemsPerMma);
        if (elect_one()) {
          // Scale atoms of this stage -> TMEM. Every atom slot of the stage is copied; slots the
          // producer did not fill (edge of N or K) only feed masked columns or skipped MMAs.
          if constexpr (T::kScaled) {
            const uint64_t sf_desc = make_sf_chunk_desc(st + T::kABytes + T::kBBytes);
#pragma unroll
            for (int ka = 0; ka < T::kKAtoms; ++ka) {
              tc_copy_sf_atom(T::kSfaCol0 + ka * 4, sf_desc + ((ka * 512) >> 4));
#pragma unroll
              for (int ra = 0; ra < T::kSfbRowAtoms; ++ra)
                tc_copy_sf_atom(T::kSfbCol0 + ka * T::kSfbRowAtoms * 4 + ra * 4,
                                sf_desc + ((T::kSfaBytes + (ra * T::kKAtoms + ka) * 512) >> 4));
            }
          }
          const uint64_t adesc = make_kmajor_sw128_desc(st);
          const uint64_t bdesc = make_kmajor_sw128_desc(st + T::kABytes);
          {
            // 32 bytes of K per instruction: +2 in the (address >> 4) field.
            if (mmas == T::kMmasPerStage) {
#pragma unroll
              for (int j = 0; j < T::kMmasPerStage; ++j) {
                const uint32_t accumulate = (kt > 0 || j > 0) ? 1u : 0u;
                if constexpr (KIND == kFp8)
                  tc_mma_f8(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate);
                else if (KIND == kMxfp8)
                  tc_mma_mxf8(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, j, j), accumulate, T::kSfaCol0,
                              sfb_taddr);
                else if (KIND == kMxfp4)
                  tc_mma_mxf4(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, (j & 1) * 2, (j & 1) * 2), accumulate,
                              T::kSfaCol0 + (j >> 1) * 4,
                              sfb_taddr + (j >> 1) * T::kSfbRowAtoms * 4);
                else
                  tc_mma_nvf4(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate,
                              T::kSfaCol0 + j * 4, sfb_taddr + j * T::kSfbRowAtoms * 4);
              }
            } else {
              for (int j = 0; j < mmas; ++j) {
                const uint32_t accumulate = (kt > 0 || j > 0) ? 1u : 0u;
                if constexpr (KIND == kFp8)
                  tc_mma_f8(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate);
                else if (KIND == kMxfp8)
                  tc_mma_mxf8(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, j, j), accumulate, T::kSfaCol0,
                              sfb_taddr);
                else if (KIND == kMxfp4)
                  tc_mma_mxf4(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                              idesc_with_sf_ids(idesc_base, (j & 1) * 2, (j & 1) * 2), accumulate,
                              T::kSfaCol0 + (j >> 1) * 4,
                              sfb_taddr + (j >> 1) * T::kSfbRowAtoms * 4);
                else
                  tc_mma_nvf4(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate,
                              T::kSfaCol0 + j * 4, sfb_taddr + j * T::kSfbRowAtoms * 4);
              }
            }
          }
          tc_commit(&empty_bar[stage]);
          if (kt == k_tiles - 1) tc_commit(&acc_full_bar[acc]);
        }
        __syncwarp();
        if (++stage == p.num_stages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    int iter = 0;
    bool store_pending = false;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++iter) {
      int tm, tn, grp, local;
      split_group(tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const int acc = iter % T::kAccStages;
      const uint32_t acc_phase = (iter / T::kAccStages) & 1;
      // The epilogue warps meet at barriers in the TMA-store path, so they agree on the
      // outcome of the wait before going on.
      if (!epilogue_bar_and(mbar_wait_bounded(&acc_full_bar[acc], acc_phase, abort_flag))) {
        *abort_flag = 1;
        if (p.status && lane == 0) atomicMax(p.status, kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after_sync();
      const int row_in_tile = quarter * 32 + lane;
      const int row = tm * T::BM + row_in_tile;
      const uint32_t taddr = (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (p.use_tma_store) {
        // TMEM -> registers -> swizzled smem -> TMA store, 128 columns per pass. The
        // accumulator is released as soon as its last column sits in shared memory, so the
        // global write overlaps the next tile's main loop.
        constexpr int kPasses = (BN + 127) / 128;
        const bool store_thread = (threadIdx.x == 64);
#pragma unroll 1
        for (int pass = 0; pass < kPasses; ++pass) {
          if (store_pending) {
            if (store_thread) tma_store_wait_read<0>();
            epilogue_bar_sync();
            store_pending = false;
          }
          const int chunks = min(4, BN / 32 - pass * 4);
          // The TMEM load of chunk cc+1 is in flight while chunk cc is converted and staged.
          uint32_t raw[2][32];
          tmem_load_32cols(taddr + pass * 128, raw[0]);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            if (cc < chunks) {
              tmem_load_wait();
              if (cc + 1 < chunks) tmem_load_32cols(taddr + pass * 128 + (cc + 1) * 32, raw[(cc + 1) & 1]);
              const uint32_t(&cur)[32] = raw[cc & 1];
              float vals[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) vals[i] = __uint_as_float(cur[i]) * alpha;
              if constexpr (BIAS)
                add_bias_32(vals, p.bias, p.out_dtype, tn * BN + pass * 128 + cc * 32, p.n);
              uint32_t packed[16];
              if (p.out_dtype == kOutBf16) {
#pragma unroll
                for (int i = 0; i < 16; ++i) packed[i] = pack_bf16x2(vals[2 * i], vals[2 * i + 1]);
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) packed[i] = pack_f16x2(vals[2 * i], vals[2 * i + 1]);
              }
              // Sub-tile of 64 columns = 128-byte rows; 16-byte chunk j of row r lives at
              // position j ^ (r % 8), the layout a 128-byte-swizzled TMA store expects.
              uint8_t* sub = c_stage + (cc >> 1) * (128 * 128) + row_in_tile * 128;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int j = ((cc & 1) * 4 + i) ^ (row_in_tile & 7);
                *reinterpret_cast<uint4*>(sub + j * 16) = make_uint4(
                    packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
              }
            }
          }
          if (pass == kPasses - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
          }
          fence_proxy_async_smem();
          epilogue_bar_sync();
          if (store_thread) {
            for (int sub = 0; sub < (chunks + 1) / 2; ++sub) {
              const int col = tn * BN + pass * 128 + sub * 64;
              if (col < p.n) tma_store_3d(&map_c, c_stage + sub * (128 * 128), col, tm * T::BM, grp);
            }
            tma_store_commit();
          }
          store_pending = true;
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t raw[32];
        tmem_load_32cols(taddr + c * 32, raw);
        tmem_load_wait();
        float vals[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) vals[i] = __uint_as_float(raw[i]) * alpha;
        if constexpr (BIAS) add_bias_32(vals, p.bias, p.out_dtype, tn * BN + c * 32, p.n);
        store_row_chunk(p, grp, row, tn * BN + c * 32, vals);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
    }
    if (p.use_tma_store && threadIdx.x == 64) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(0, 512);
  }
}

}  // namespace b12x_b200
