// Block-FP8 GEMM with compact FP32 scales (DeepSeek-V3 style) for sm_100a:
//
//     C[M,N] = cvt(alpha * sum_kb (A[:, kb] B[:, kb]^T) * sfa[m, kb] * sfb[n/128, kb])
//
// A [M,K] and B [N,K] are E4M3, K-major; sfa is [M, K/128] FP32 (one scale per row and 128
// columns), sfb is [N/128, K/128] FP32 (one per 128x128 block). FP32 scales cannot ride on the
// block-scaled MMA (it takes power-of-two or E4M3 scale bytes), so every 128-wide k-block is
// multiplied unscaled (tcgen05 kind::f8f6f4, four K=32 instructions) into a TMEM buffer and
// promoted into FP32 register accumulators with one FMA per element.
//
// One CTA (576 threads) owns a 128 x 256 tile: warp 0 = TMA producer, warp 1 = MMA issuer,
// warps 2..17 = promotion/epilogue (four warps per 32-lane TMEM quarter, each taking 64 of the
// 256 columns, i.e. half of one 128-column scale block). Promotion is a chain of TMEM load ->
// wait -> FMA per warp, so it is the number of warps per scheduler (four) that hides the load
// latency. The two 256-column TMEM buffers fill all 512 columns, so the MMA of k-block i+1
// overlaps the promotion of k-block i. At the end of a tile the promotion warps must get back
// to the next tile quickly (the MMA warp can only run two k-blocks ahead of them), so 2-byte
// outputs are converted into a 128-byte-swizzled staging area in shared memory and leave
// through asynchronous TMA stores, one 64-column sub-tile per group of four warps.
#pragma once

#include "gemm_blockscaled.cuh"

namespace b12x_b200 {

struct BlockFp8Tile {
  static constexpr int BM = 128;
  static constexpr int BN = 256;
  static constexpr int kABytes = BM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 3;
  static constexpr int kCStageBytes = BM * BN * 2;   // four sub-tiles of 128 rows x 64 columns
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCStageBytes + kBarrierBytes + 1024;
  static constexpr int kEpilogueWarps = 16;
  static constexpr int kColsPerWarp = BN / (kEpilogueWarps / 4);
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps);
};

struct BlockFp8Params {
  const float* sfa;   // [M, K/128]
  const float* sfb;   // [ceil(N/128), K/128]
  void* c;
  const float* alpha;
  int* status;
  int m, n, k, ldc, out_dtype;
  int tiles_m, tiles_n, group_m;
  int use_tma_store;   // 2-byte outputs with 16-byte aligned rows
  const void* bias;    // [N] values of the output dtype added to every row, or null
};

// Named barrier 1 + group over the 128 threads (four warps) that share an output sub-tile.
__device__ __forceinline__ void group_bar_sync(int group) {
  asm volatile("barrier.cta.sync %0, 128;" ::"r"(group + 1) : "memory");
}

// BIAS: the instantiation with the bias epilogue; the plain one carries none of its code (the
// promotion loop runs at the register limit, and even an untaken branch cost 45 % there).
template <bool BIAS>
__global__ void __launch_bounds__(BlockFp8Tile::kThreads, 1)
gemm_block_fp8_kernel(const __grid_constant__ CUtensorMap map_a,
                      const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_c, const BlockFp8Params p) {
  using T = BlockFp8Tile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* c_stage = smem + T::kStages * T::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(c_stage + T::kCStageBytes);
  uint64_t* empty_bar = full_bar + T::kStages;
  uint64_t* part_full_bar = empty_bar + T::kStages;
  uint64_t* part_empty_bar = part_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&part_full_bar[b], 1);
      mbar_init(&part_empty_bar[b], T::kEpilogueWarps);
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
  const uint32_t tmem_base = *tmem_slot;
  if (tmem_base != 0) {  // the CTA owns the whole TMEM, so the base is column 0
    if (threadIdx.x == 0 && p.status) atomicMax(p.status, kStatusTmemLayout);
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
    return;
  }

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = p.k / 128;
  const uint32_t smem_u32 = smem_addr_u32(smem);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
          ok = false;
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + stage * T::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], T::kStageBytes);
          tma_load_2d(st, &map_a, &full_bar[stage], kb * 128, tm * T::BM);
          tma_load_2d(st + T::kABytes, &map_b, &full_bar[stage], kb * 128, tn * T::BN);
        }
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc = make_idesc_f8(128, T::BN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1;
        // The operands are normally there long before the TMEM buffer is handed back; wait for
        // them first and have the descriptors ready, so that nothing but the issue itself
        // follows the hand-over (which is on the critical path).
        const uint32_t st = smem_u32 + stage * T::kStageBytes;
        const uint64_t adesc = make_kmajor_sw128_desc(st);
        const uint64_t bdesc = make_kmajor_sw128_desc(st + T::kABytes);
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag) ||
            !mbar_wait_bounded(&part_empty_bar[buf], ((it >> 1) & 1) ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tc_mma_f8(buf * T::BN, adesc + 2 * j, bdesc + 2 * j, idesc, j > 0 ? 1u : 0u);
          tc_commit(&part_full_bar[buf]);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------- promotion + epilogue -------------------------
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;  // which 64 of the tile's 256 columns
    constexpr int kCols = T::kColsPerWarp;
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    const int kb_total = k_blocks;
    uint32_t it = 0;
    bool ok = true;
    bool store_pending = false;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const int row = tm * T::BM + quarter * 32 + lane;
      const int col0 = tn * T::BN + group * kCols;
      const bool row_ok = row < p.m;
      const bool col_ok = col0 < p.n;
      const float* sfa_row = p.sfa + static_cast<size_t>(row_ok ? row : 0) * kb_total;
      const float* sfb_row = p.sfb + static_cast<size_t>(col_ok ? col0 / 128 : 0) * kb_total;
      float acc[kCols];
#pragma unroll
      for (int i = 0; i < kCols; ++i) acc[i] = 0.0f;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1;
        // Scales of this k-block are fetched before the wait so their latency hides behind it.
        const float scale = __fmul_rn(row_ok ? __ldg(sfa_row + kb) : 0.0f,
                                      col_ok ? __ldg(sfb_row + kb) : 0.0f);
        if (!mbar_wait_bounded(&part_full_bar[buf], (it >> 1) & 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusEpilogueTimeout);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr =
            (static_cast<uint32_t>(quarter * 32) << 16) + buf * T::BN + group * kCols;
        // Two TMEM loads in flight: chunk c+1 streams in while chunk c is promoted.
        uint32_t raw[2][16];
        tmem_load_16cols(taddr, raw[0]);
#pragma unroll
        for (int c = 0; c < kCols / 16; ++c) {
          tmem_load_wait();
          if (c + 1 < kCols / 16) {
            tmem_load_16cols(taddr + (c + 1) * 16, raw[(c + 1) & 1]);
          } else {
            // Everything of this buffer is in registers: give it back to the MMA warp before
            // the last chunk is accumulated (the hand-over is on the critical path).
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&part_empty_bar[buf]);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i)
            acc[c * 16 + i] = fmaf(__uint_as_float(raw[c & 1][i]), scale, acc[c * 16 + i]);
        }
      }
      if (!ok) break;
      if (p.use_tma_store) {
        // The four warps of a group own sub-tile `group`: rows 0..127, 64 columns = 128 bytes
        // per row; 16-byte chunk j of row r sits at position j ^ (r % 8), the layout a
        // 128-byte-swizzled TMA store expects. The sub-tile of the previous tile has long been
        // read by its store; the wait is a formality.
        const bool store_thread = (quarter == 2) && (lane == 0);  // first warp of the group
        if (store_pending) {
          if (store_thread) tma_store_wait_read<0>();
          group_bar_sync(group);
        }
        const int r = quarter * 32 + lane;
        uint8_t* sub = c_stage + group * (128 * 128) + r * 128;
        if constexpr (BIAS) {
          // acc becomes float(cvt(alpha * acc)) + bias; the packing below rounds the sum.
#pragma unroll
          for (int c = 0; c < kCols / 32; ++c) {
            float vals[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) vals[i] = acc[c * 32 + i] * alpha;
            add_bias_32(vals, p.bias, p.out_dtype, col0 + c * 32, p.n);
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[c * 32 + i] = vals[i];
          }
        }
        const float out_scale = BIAS ? 1.0f : alpha;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float lo = acc[j * 8 + 2 * h] * out_scale, hi = acc[j * 8 + 2 * h + 1] * out_scale;
            w[h] = (p.out_dtype == kOutBf16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(sub + ((j ^ (r & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
        group_bar_sync(group);
        if (store_thread) {
          const int m0 = tm * T::BM;
          if (col0 < p.n && m0 < p.m) tma_store_2d(&map_c, c_stage + group * (128 * 128), col0, m0);
          tma_store_commit();
        }
        store_pending = true;
        continue;
      }
      GemmParams gp;
      gp.c_group_elems = 0;
      gp.c = p.c;
      gp.m = p.m;
      gp.n = p.n;
      gp.ldc = p.ldc;
      gp.out_dtype = p.out_dtype;
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) {
        float vals[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) vals[i] = acc[c * 32 + i] * alpha;
        if constexpr (BIAS) add_bias_32(vals, p.bias, p.out_dtype, col0 + c * 32, p.n);
        store_row_chunk(gp, 0, row, col0 + c * 32, vals);
      }
    }
    if (p.use_tma_store && quarter == 2 && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(0, 512);
  }
}

}  // namespace b12x_b200
