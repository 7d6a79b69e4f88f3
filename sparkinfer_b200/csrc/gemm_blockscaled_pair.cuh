// CTA-pair variant of the block-scaled GEMM (tcgen05 cta_group::2) for large M.
//
// Two CTAs of a cluster own one 256 x BN output tile. Each loads its own 128 rows of A and
// only *half* of the B tile's rows; one tcgen05.mma issued by the leader multiplies the 256
// rows against all BN columns, each CTA's tensor core reading both halves of B. Per CTA and
// k-step that is 16 KiB + BN/2 * 128 B instead of 16 KiB + BN * 128 B, which is what the
// single-CTA kernel was short of: its main loop waited on operand loads with only three stages
// of 48 KiB fitting in shared memory. No load is multicast; every TMA writes the issuing CTA's
// own shared memory and signals that CTA's own barrier.
//
// Hand-shake per stage s (all waits bounded):
//   producer (each CTA)  : wait own empty[s] -> arm own full[s], issue own loads
//   relay (peer, warp 1) : wait own full[s]  -> arrive on the leader's peer_full[s]
//   issuer (leader, w 1) : wait own full[s] and peer_full[s] -> scale copies + 4 MMAs for the
//                          pair -> tcgen05.commit to empty[s] of both CTAs (two commits)
//   epilogue (each CTA)  : wait own acc_full (committed by the leader to both CTAs) -> pull own
//                          128 x 256 accumulator into registers -> arrive on the leader's
//                          acc_empty -> convert, stage in swizzled shared memory, TMA store
//
// Partial round. With T tiles on P pairs, T / P rounds keep every pair busy; the T % P tiles
// left would occupy a few pairs for a whole tile time while the rest idle (448 tiles on 74
// pairs: 4 tiles, a seventh round at 5 % occupancy). When at most half of the pairs would be
// busy, each leftover tile is instead cut along K into S = P / (T % P) segments, one per pair,
// and these segments are the FIRST thing the pairs do (while they are still in step).
// A pair multiplies its segment as usual, writes its FP32 partial tile to scratch, and counts
// itself in on the tile's counter; once all 2S CTAs of the tile have arrived (a bounded wait on
// the counter: all pairs of the grid are resident, one CTA per SM), every CTA adds up the S
// partials of its own share of the tile (one sixteenth-or-so of the columns, its own 128 rows)
// in segment order, scales, converts and stores it. The reduction is thus spread over all the
// CTAs that computed the tile and its result does not depend on timing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_blockscaled.cuh"

namespace b12x_b200 {

// CSLOTS: 16 KiB output staging slots (one 64-column sub-tile each). The ordinary kernels use
// one; the scatter kernel alternates between two.
template <int KIND, int BN, int CSLOTS = 1>
struct PairTile {
  static_assert(BN == 128 || BN == 256, "pair tiles are 128 or 256 columns wide");
  static constexpr int BM = 128;                               // rows per CTA (256 per pair)
  static constexpr int kRowBytes = 128;
  static constexpr int kMmasPerStage = 4;
  static constexpr bool kScaled = (KIND != kFp8);
  static constexpr int kElemsPerMma = (KIND == kNvfp4 || KIND == kMxfp4) ? 64 : 32;
  static constexpr int kElemsPerStage = kElemsPerMma * kMmasPerStage;
  static constexpr int kKAtoms = (KIND == kMxfp8) ? 1 : (KIND == kNvfp4 ? 4 : (KIND == kMxfp4 ? 2 : 0));
  static constexpr int kSfbRowAtoms = BN / 128;
  static constexpr int kABytes = BM * kRowBytes;
  static constexpr int kBBytes = (BN / 2) * kRowBytes;         // this CTA's half of B
  static constexpr int kSfaBytes = kKAtoms * 512;
  static constexpr int kSfbBytes = kSfbRowAtoms * kKAtoms * 512;
  static constexpr int kStageBytes =
      ((kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024) * 1024;
  static constexpr int kSfaCols = kKAtoms * 4;
  static constexpr int kSfbCols = kSfbRowAtoms * kKAtoms * 4;
  static constexpr int kAccStages = (2 * BN + kSfaCols + kSfbCols <= 512) ? 2 : 1;
  static constexpr int kSfaCol0 = kAccStages * BN;
  static constexpr int kSfbCol0 = kSfaCol0 + kSfaCols;
  static constexpr int kCSlots = CSLOTS;
  static constexpr int kCSlotBytes = 128 * 64 * 2;           // one 64-column output sub-tile
  static constexpr int kCStageBytes = CSLOTS * kCSlotBytes;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kStagesRaw =
      (227 * 1024 - kBarrierBytes - 1024 - kCStageBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCStageBytes + kBarrierBytes + 1024;
};

// One piece of work of a pair: a tile and a range of its k-tiles. segments == 1: the whole tile,
// stored by the usual epilogue; otherwise segment `seg` of leftover tile `tail_index`.
struct PairWork {
  int tile, kt_begin, kt_end, seg, segments, tail_index;
};

// it-th piece of work of `pair` (P pairs, T tiles, tail_segments = S or <= 1 for no split).
// tail_segments < -1: S = -tail_segments and the split tiles come FIRST (it = 0 of the pairs that
// have a segment), when all pairs are still in step, instead of after the whole rounds.
__device__ __forceinline__ bool pair_work(int it, int pair, int num_pairs, int num_tiles,
                                          int k_tiles, int tail_segments, PairWork& w) {
  const int rounds = num_tiles / num_pairs;
  w.kt_begin = 0;
  w.kt_end = k_tiles;
  w.seg = 0;
  w.segments = 1;
  w.tail_index = 0;
  if (tail_segments < -1) {
    const int s_count = -tail_segments;
    const int first = rounds * num_pairs;
    const int left = num_tiles - first;
    const bool has_unit = pair < left * s_count;
    if (has_unit && it == 0) {
      w.tail_index = pair / s_count;
      w.tile = first + w.tail_index;
      w.seg = pair - w.tail_index * s_count;
      w.segments = s_count;
      w.kt_begin = static_cast<int>(static_cast<long long>(k_tiles) * w.seg / s_count);
      w.kt_end = static_cast<int>(static_cast<long long>(k_tiles) * (w.seg + 1) / s_count);
      return true;
    }
    const int whole = has_unit ? it - 1 : it;
    if (whole >= rounds) return false;
    w.tile = pair + whole * num_pairs;
    return true;
  }
  if (it < rounds) {
    w.tile = pair + it * num_pairs;
    return true;
  }
  if (it > rounds) return false;
  const int first = rounds * num_pairs;
  const int left = num_tiles - first;
  if (tail_segments <= 1) {
    w.tile = first + pair;
    return pair < left;
  }
  if (pair >= left * tail_segments) return false;
  w.tail_index = pair / tail_segments;
  w.tile = first + w.tail_index;
  w.seg = pair - w.tail_index * tail_segments;
  w.segments = tail_segments;
  w.kt_begin = static_cast<int>(static_cast<long long>(k_tiles) * w.seg / tail_segments);
  w.kt_end = static_cast<int>(static_cast<long long>(k_tiles) * (w.seg + 1) / tail_segments);
  return true;
}

// Scratch of the split tail (caller-owned, inside the per-stream workspace): two int32 counters
// per leftover tile (arrived, done; zero between launches) and, per leftover tile and segment,
// two FP32 partial tiles of 128 x 256 (one per CTA of the pair) stored as [64 column quads][128
// rows][4], so that the 32 lanes of a warp write and read consecutive 16-byte pieces.
struct PairTail {
  int* counters;
  float* partials;
  int segments;  // S, or <= 1 when the tail is not split
};

// Row-parallel scatter of the output (SCATTER instantiation): the M rows are cut into `world`
// slabs of `slab_rows` (a multiple of the 256-row pair tile); a tile whose rows lie in slab s is
// stored into destination s, a [world * slab_rows][ld] buffer that may live on another GPU
// (peer-mapped), at rows rank * slab_rows + (row - s * slab_rows): slot `rank` of the owner of
// slab s, where that owner's reduction kernel expects this rank's partial.
constexpr int kMaxScatter = 8;
template <bool ON>
struct ScatterOut {};
template <>
struct ScatterOut<true> {
  void* base[kMaxScatter];       // destination s: a [world * slab_rows][ld] buffer
  int slab_rows;
  int rank;
  int world;
};

// The scheduler's consecutive tile rows alternate between the slabs (row i of the schedule is
// tile row (i % world) * tiles_m / world + i / world), so that at any moment the tiles being
// finished are spread over all destinations instead of all going to one peer: a round of 74
// pair tiles stores 9.5 MB at once, and with every tile of a round bound for the same GPU that
// burst waited for the link (two GPUs: 133 us, against 124 us once spread and 107 us for the
// plain GEMM). Dealing the rows out by twos, so that a pair's own consecutive tiles alternate
// between destinations as well, measured the same as this simple form.
__device__ __forceinline__ int scatter_tile_row(int tm, int tiles_m, int world) {
  return (tm % world) * (tiles_m / world) + tm / world;
}

constexpr int kPairPartialFloats = 128 * 256;
constexpr uint32_t kPairReducePolls = 1u << 20;

// BIAS: the instantiation with the bias epilogue (the plain one carries none of its code).
// SCATTER: the instantiation whose output tiles go to per-slab destinations (see ScatterOut).
template <int KIND, int BN, bool BIAS, bool SCATTER = false>
__global__ void __launch_bounds__(224, 1)
gemm_blockscaled_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                             const __grid_constant__ CUtensorMap map_b,
                             const __grid_constant__ CUtensorMap map_c, const GemmParams p,
                             const PairTail tail,
                             const __grid_constant__ ScatterOut<SCATTER> sc) {
  static_assert(!(BIAS && SCATTER), "the scattered output is a partial sum: no bias on it");
  using T = PairTile<KIND, BN, SCATTER ? 2 : 1>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* c_stage = smem + T::kStages * T::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(c_stage + T::kCStageBytes);
  uint64_t* peer_full_bar = full_bar + T::kStages;   // used in the leader only
  uint64_t* empty_bar = peer_full_bar + T::kStages;
  uint64_t* acc_full_bar = empty_bar + T::kStages;
  uint64_t* acc_empty_bar = acc_full_bar + 2;        // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = (rank == 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(&full_bar[s], T::kScaled ? 2 : 1);  // operand producer (+ scale producer)
      mbar_init(&peer_full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.use_tma_store) tma_prefetch_desc(&map_c);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool tmem_ok = (tmem_base == 0);
  if (!tmem_ok && threadIdx.x == 0 && p.status) atomicMax(p.status, kStatusTmemLayout);

  // tiles_m counts 256-row pair tiles here; the tiles of all groups form one list.
  const int tiles_per_group = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_group * p.groups;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int k_tiles = (p.k + T::kElemsPerStage - 1) / T::kElemsPerStage;
  const int m_row_atoms = (p.m + 127) / 128;
  const int n_row_atoms = (p.n + 127) / 128;
  const uint32_t smem_u32 = smem_addr_u32(smem);

  if (!tmem_ok) {
    // fall through to the common tear-down
  } else if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    PairWork w;
    for (int it = 0; ok && pair_work(it, pair, num_pairs, num_tiles, k_tiles, tail.segments, w); ++it) {
      int tm, tn, grp, local;
      split_group(w.tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      if constexpr (SCATTER) tm = scatter_tile_row(tm, p.tiles_m, sc.world);
      const int m0 = tm * 256 + static_cast<int>(rank) * 128;
      const int n0 = tn * BN;
      for (int kt = w.kt_begin; kt < w.kt_end; ++kt) {
        if (!mbar_wait_bounded_cluster(&empty_bar[stage], phase ^ 1, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusProducerTimeout);
          ok = false;
          break;
        }
        if (elect_one()) {
          uint8_t* st = smem + stage * T::kStageBytes;
          uint64_t* bar = &full_bar[stage];
          mbar_arrive_expect_tx(bar, T::kABytes + T::kBBytes);
          tma_load_3d(st, &map_a, bar, kt * T::kRowBytes, m0, grp);
          tma_load_3d(st + T::kABytes, &map_b, bar, kt * T::kRowBytes,
                      n0 + static_cast<int>(rank) * (BN / 2), grp);
        }
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 6 && !T::kScaled) {
    // plain FP8: there are no scale factors to bring in
  } else if (warp == 6) {
    // ------------------------- scale-factor producer (both CTAs) -------------------------
    // A second producer warp so that the five copies of a stage are issued by two warps in
    // parallel; both arrive on the stage's full barrier with their own byte counts.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    PairWork w;
    for (int it = 0; ok && pair_work(it, pair, num_pairs, num_tiles, k_tiles, tail.segments, w); ++it) {
      int tm, tn, grp, local;
      split_group(w.tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      if constexpr (SCATTER) tm = scatter_tile_row(tm, p.tiles_m, sc.world);
      const int n0 = tn * BN;
      const int sfa_atom = tm * 2 + static_cast<int>(rank);
      const bool sfa_ok = sfa_atom < m_row_atoms;
      const int sfb_atom0 = n0 / 128;
      const int sfb_atoms = min(T::kSfbRowAtoms, n_row_atoms - sfb_atom0);
      const uint8_t* sfa_src = p.sfa + grp * p.sfa_group_bytes +
                               static_cast<size_t>(sfa_ok ? sfa_atom : 0) * p.k_atoms_total * 512;
      const uint8_t* sfb_src = p.sfb + grp * p.sfb_group_bytes +
                               static_cast<size_t>(sfb_atom0) * p.k_atoms_total * 512;
      for (int kt = w.kt_begin; kt < w.kt_end; ++kt) {
        if (!mbar_wait_bounded_cluster(&empty_bar[stage], phase ^ 1, abort_flag)) {
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
          mbar_arrive_expect_tx(bar, sf_bytes * ((sfa_ok ? 1 : 0) + sfb_atoms));
          if (sfa_ok)
            bulk_load(st + T::kABytes + T::kBBytes, sfa_src + static_cast<size_t>(katom0) * 512,
                      sf_bytes, bar);
          for (int ra = 0; ra < sfb_atoms; ++ra)
            bulk_load(st + T::kABytes + T::kBBytes + T::kSfaBytes + ra * T::kKAtoms * 512,
                      sfb_src + (static_cast<size_t>(ra) * p.k_atoms_total + katom0) * 512,
                      sf_bytes, bar);
        }
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && !leader) {
    // ------------------------------ relay (peer CTA) ------------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    PairWork w;
    for (int it = 0; ok && pair_work(it, pair, num_pairs, num_tiles, k_tiles, tail.segments, w); ++it) {
      for (int kt = w.kt_begin; kt < w.kt_end; ++kt) {
        if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
          ok = false;
          break;
        }
        if (elect_one())
          mbar_arrive_cluster(map_to_cta(smem_addr_u32(&peer_full_bar[stage]), 0));
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) ------------------------------
    constexpr uint32_t idesc_base =
        KIND == kFp8 ? make_idesc_f8(256, BN)
                     : make_idesc_block_scaled(256, BN, KIND == kMxfp8 ? 0u : 1u,
                                               KIND == kNvfp4 ? 0u : 1u);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    PairWork w;
    for (int iter = 0; ok && pair_work(iter, pair, num_pairs, num_tiles, k_tiles, tail.segments, w); ++iter) {
      const int acc = iter % T::kAccStages;
      const uint32_t acc_phase = (iter / T::kAccStages) & 1;
      if (!mbar_wait_bounded_cluster(&acc_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
        *abort_flag = 1;
        if (p.status && lane == 0) atomicMax(p.status, kStatusMmaTimeout);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_taddr = acc * BN;
      for (int kt = w.kt_begin; kt < w.kt_end; ++kt) {
        const bool got_local = mbar_wait_bounded(&full_bar[stage], phase, abort_flag);
        if (!got_local ||
            !mbar_wait_bounded_cluster(&peer_full_bar[stage], phase, abort_flag)) {
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
          if constexpr (T::kScaled) {
            const uint64_t sf_desc = make_sf_chunk_desc(st + T::kABytes + T::kBBytes);
#pragma unroll
            for (int ka = 0; ka < T::kKAtoms; ++ka) {
              tc_copy_sf_atom_pair(T::kSfaCol0 + ka * 4, sf_desc + ((ka * 512) >> 4));
#pragma unroll
              for (int ra = 0; ra < T::kSfbRowAtoms; ++ra)
                tc_copy_sf_atom_pair(T::kSfbCol0 + ka * T::kSfbRowAtoms * 4 + ra * 4,
                                     sf_desc + ((T::kSfaBytes + (ra * T::kKAtoms + ka) * 512) >> 4));
            }
          }
          const uint64_t adesc = make_kmajor_sw128_desc(st);
          const uint64_t bdesc = make_kmajor_sw128_desc(st + T::kABytes);
          for (int j = 0; j < mmas; ++j) {
            const uint32_t accumulate = (kt > w.kt_begin || j > 0) ? 1u : 0u;
            if constexpr (KIND == kFp8)
              tc_mma_f8_pair(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate);
            else if (KIND == kMxfp8)
              tc_mma_mxf8_pair(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                               idesc_with_sf_ids(idesc_base, j, j), accumulate, T::kSfaCol0,
                               T::kSfbCol0);
            else if (KIND == kMxfp4)
              tc_mma_mxf4_pair(d_taddr, adesc + 2 * j, bdesc + 2 * j,
                               idesc_with_sf_ids(idesc_base, (j & 1) * 2, (j & 1) * 2), accumulate,
                               T::kSfaCol0 + (j >> 1) * 4,
                               T::kSfbCol0 + (j >> 1) * T::kSfbRowAtoms * 4);
            else
              tc_mma_nvf4_pair(d_taddr, adesc + 2 * j, bdesc + 2 * j, idesc_base, accumulate,
                               T::kSfaCol0 + j * 4, T::kSfbCol0 + j * T::kSfbRowAtoms * 4);
          }
          // Free the stage in both CTAs; publish the accumulator to both after the last step.
          const uint32_t empty_addr = smem_addr_u32(&empty_bar[stage]);
          tc_commit_pair(empty_addr);
          tc_commit_pair(map_to_cta(empty_addr, 1));
          if (kt == w.kt_end - 1) {
            const uint32_t full_addr = smem_addr_u32(&acc_full_bar[acc]);
            tc_commit_pair(full_addr);
            tc_commit_pair(map_to_cta(full_addr, 1));
          }
        }
        __syncwarp();
        if (++stage == T::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quarter = warp & 3;
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    bool store_pending = false;
    PairWork w;
    for (int iter = 0; pair_work(iter, pair, num_pairs, num_tiles, k_tiles, tail.segments, w); ++iter) {
      int tm, tn, grp, local;
      split_group(w.tile, tiles_per_group, grp, local);
      tile_coords(local, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      if constexpr (SCATTER) tm = scatter_tile_row(tm, p.tiles_m, sc.world);
      const int acc = iter % T::kAccStages;
      const uint32_t acc_phase = (iter / T::kAccStages) & 1;
      if (!epilogue_bar_and(mbar_wait_bounded_cluster(&acc_full_bar[acc], acc_phase, abort_flag))) {
        *abort_flag = 1;
        if (p.status && lane == 0) atomicMax(p.status, kStatusEpilogueTimeout);
        break;
      }
      tc_fence_after_sync();
      const int row_in_tile = quarter * 32 + lane;
      const int m0 = tm * 256 + static_cast<int>(rank) * 128;
      const int row = m0 + row_in_tile;
      const uint32_t taddr = (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const uint32_t acc_empty_leader = map_to_cta(smem_addr_u32(&acc_empty_bar[acc]), 0);
      // Where this CTA's 128 rows go: the caller's C, or (SCATTER) the slab owner's buffer.
      void* c_base = p.c;
      int dst = 0;          // destination index (SCATTER)
      int row_shift = 0;    // destination row = row + row_shift (SCATTER)
      if constexpr (SCATTER) {
        dst = m0 / sc.slab_rows;
        row_shift = (sc.rank - dst) * sc.slab_rows;
        c_base = sc.base[dst];
      }
      if (w.segments > 1) {
        // ---- segment of a leftover tile: FP32 partial to scratch, then the shared reduction ----
        const int s_count = w.segments;
        float* slots = tail.partials +
                       static_cast<size_t>(w.tail_index) * s_count * 2 * kPairPartialFloats;
        float4* mine = reinterpret_cast<float4*>(
            slots + (static_cast<size_t>(w.seg) * 2 + rank) * kPairPartialFloats);
        // Four tensor-memory loads in flight at a time (128 columns), as in the main epilogue.
#pragma unroll 1
        for (int half = 0; half < BN / 128; ++half) {
          uint32_t raw[4][32];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) tmem_load_32cols(taddr + half * 128 + cc * 32, raw[cc]);
          tmem_load_wait();
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              mine[((half * 4 + cc) * 8 + q) * 128 + row_in_tile] = make_float4(
                  __uint_as_float(raw[cc][4 * q]), __uint_as_float(raw[cc][4 * q + 1]),
                  __uint_as_float(raw[cc][4 * q + 2]), __uint_as_float(raw[cc][4 * q + 3]));
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        // Publish, count this CTA in, and wait (bounded) for the 2 * S CTAs of the tile.
        __threadfence();
        epilogue_bar_sync();
        int* arrived = tail.counters + 2 * w.tail_index;
        int* done = arrived + 1;
        bool all_in = true;
        if (threadIdx.x == 64) {
          atomicAdd(arrived, 1);
          uint32_t polls = 0;
          while (*reinterpret_cast<volatile int*>(arrived) < 2 * s_count) {
            if (++polls >= kPairReducePolls || *abort_flag != 0) {
              all_in = false;
              break;
            }
            __nanosleep(64);
          }
          __threadfence();
        }
        if (!epilogue_bar_and(all_in)) {
          *abort_flag = 1;
          if (p.status && lane == 0) atomicMax(p.status, kStatusReduceTimeout);
          break;
        }
        // This CTA's share: column quads [q_begin, q_end) of its own 128 rows, summed over the
        // segments in order.
        const int per = (BN / 4 + s_count - 1) / s_count;
        const int q_begin = w.seg * per;
        const int q_end = min(BN / 4, q_begin + per);
        const float4* base = reinterpret_cast<const float4*>(slots + static_cast<size_t>(rank) * kPairPartialFloats);
        constexpr size_t kSegStride = 2 * kPairPartialFloats / 4;  // float4 between segments
        // Eight column quads at a time, four segments per trip: up to thirty-two independent
        // 16-byte loads are in flight per thread (the loop is bound by load latency, not by
        // bytes). The adds run in segment order whatever the batching.
#pragma unroll 1
        for (int q0 = q_begin; q0 < q_end; q0 += 8) {
          float4 sum[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) sum[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 1
          for (int sg = 0; sg < s_count; sg += 4) {
            float4 v[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                v[j][i] = (sg + j < s_count && q0 + i < q_end)
                              ? __ldcg(base + static_cast<size_t>(sg + j) * kSegStride +
                                       (q0 + i) * 128 + row_in_tile)
                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              }
            }
            // Adding +0.0f for an absent segment leaves the sum unchanged bit for bit (the sum
            // is never -0.0f: it starts at +0.0f).
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                sum[i].x += v[j][i].x; sum[i].y += v[j][i].y;
                sum[i].z += v[j][i].z; sum[i].w += v[j][i].w;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int q = q0 + i;
            const int col = tn * BN + q * 4;
            if (q < q_end && row < p.m && col < p.n) {
              float o[4] = {sum[i].x * alpha, sum[i].y * alpha, sum[i].z * alpha, sum[i].w * alpha};
              if constexpr (BIAS) {
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = add_bias_1(o[j], p.bias, p.out_dtype, col + j, p.n);
              }
              const size_t idx = SCATTER ? static_cast<size_t>(row + row_shift) * p.ldc + col
                                         : static_cast<size_t>(grp) * p.c_group_elems +
                                               static_cast<size_t>(row) * p.ldc + col;
              if (p.out_dtype != kOutFp32 && col + 4 <= p.n &&
                  ((reinterpret_cast<uintptr_t>(static_cast<uint16_t*>(c_base) + idx) & 7) == 0)) {
                const bool bf = p.out_dtype == kOutBf16;
                *reinterpret_cast<uint2*>(static_cast<uint16_t*>(c_base) + idx) =
                    make_uint2(bf ? pack_bf16x2(o[0], o[1]) : pack_f16x2(o[0], o[1]),
                               bf ? pack_bf16x2(o[2], o[3]) : pack_f16x2(o[2], o[3]));
                continue;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col + j < p.n) {
                  if (p.out_dtype == kOutBf16)
                    static_cast<__nv_bfloat16*>(c_base)[idx + j] = __float2bfloat16_rn(o[j]);
                  else if (p.out_dtype == kOutFp16)
                    static_cast<__half*>(c_base)[idx + j] = __float2half_rn(o[j]);
                  else
                    static_cast<float*>(c_base)[idx + j] = o[j];
                }
              }
            }
          }
        }
        // The last CTA to finish reading clears the tile's counters for the next launch.
        epilogue_bar_sync();
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(done, 1);
          if (prev == 2 * s_count - 1) {
            *arrived = 0;
            *done = 0;
          }
        }
        continue;
      }
      if (p.use_tma_store) {
        // With one CTA per SM and 224 threads a thread may hold ~250 registers, enough for half
        // of its accumulator row raw (128 columns) plus the other half already converted. So
        // tensor memory is emptied with eight back-to-back loads in two groups and handed back
        // to the MMA warp before anything is staged or stored: the next tile's MMAs wait for
        // a few hundred cycles instead of the whole drain.
        static_assert(BN == 256, "the register-resident drain is written for 256 columns");
        const bool store_thread = (threadIdx.x == 64);
        uint32_t raw[4][32];
        uint32_t packed[64];
        // `half` = which 128 columns of the tile raw[] currently holds.
        auto convert_chunk = [&](int cc, int half) {
          if constexpr (BIAS) {
            float vals[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) vals[i] = __uint_as_float(raw[cc][i]) * alpha;
            add_bias_32(vals, p.bias, p.out_dtype, tn * BN + half * 128 + cc * 32, p.n);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              packed[cc * 16 + i] = (p.out_dtype == kOutBf16)
                                        ? pack_bf16x2(vals[2 * i], vals[2 * i + 1])
                                        : pack_f16x2(vals[2 * i], vals[2 * i + 1]);
            return;
          }
          (void)half;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float lo = __uint_as_float(raw[cc][2 * i]) * alpha;
            const float hi = __uint_as_float(raw[cc][2 * i + 1]) * alpha;
            packed[cc * 16 + i] =
                (p.out_dtype == kOutBf16) ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
          }
        };
        // Stages the 128 converted columns as two sub-tiles of 64 columns (128-byte rows; 16-byte
        // chunk j of row r at position j ^ (r % 8), the 128-byte-swizzled layout) through one
        // 16 KiB slot, one TMA store each. Tensor memory has been released by now, so the waits
        // for the previous store to have read the slot are off the critical path, and the small
        // slot leaves room for one more pipeline stage.
        auto stage_and_store = [&](int pass) {
          if constexpr (SCATTER) {
            // Scattered tiles may cross NVLink. The 128 epilogue threads stage the pass's 128
            // columns (256-byte rows; 16-byte piece q of row r at position q ^ (r % 8)) in the
            // 32 KiB slot and copy it out with ordinary 16-byte stores, two whole 256-byte rows
            // per warp instruction. Measured on 4 GPUs (4096 x 7168 x 4608 per rank, 44 MB of it
            // bound for peers): 104-107 us whichever way the tiles leave (TMA stores of 64-column
            // sub-tiles through one or four slots, ordinary stores of 128- or 256-byte row
            // pieces), against 78 us with every destination local: the kernel is bound by what
            // the links carry in a many-to-many pattern (0.45-0.5 TB/s per GPU, the rate NCCL's
            // all-reduce reaches there too), not by how the stores are issued.
            static_assert(T::kCSlots == 2, "the scatter epilogue stages 128 columns at a time");
            epilogue_bar_sync();  // everyone has finished reading the previous pass
            uint8_t* row_ptr = c_stage + row_in_tile * 256;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const int j = q ^ (row_in_tile & 7);
              *reinterpret_cast<uint4*>(row_ptr + j * 16) = make_uint4(
                  packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
            }
            epilogue_bar_sync();
            const int col0 = tn * BN + pass * 128;
            uint16_t* out_rows = static_cast<uint16_t*>(c_base) +
                                 static_cast<size_t>(m0 + row_shift) * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int idx = i * 128 + row_in_tile;   // 128 rows x 16 pieces of 16 bytes
              const int r = idx >> 4;
              const int j = idx & 15;
              const uint4 v = *reinterpret_cast<const uint4*>(c_stage + r * 256 + ((j ^ (r & 7)) * 16));
              if (m0 + r < p.m && col0 + j * 8 + 8 <= p.n)
                st_global_v4_sys(out_rows + static_cast<size_t>(r) * p.ldc + j * 8, v);
            }
            return;
          }
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            if (store_pending) {
              if (store_thread) tma_store_wait_read<0>();
              epilogue_bar_sync();
            }
            uint8_t* row_ptr = c_stage + row_in_tile * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int j = q ^ (row_in_tile & 7);
              const int w = (sub * 8 + q) * 4;
              *reinterpret_cast<uint4*>(row_ptr + j * 16) =
                  make_uint4(packed[w], packed[w + 1], packed[w + 2], packed[w + 3]);
            }
            fence_proxy_async_smem();
            epilogue_bar_sync();
            if (store_thread) {
              const int col = tn * BN + pass * 128 + sub * 64;
              if (col < p.n && m0 < p.m) tma_store_3d(&map_c, c_stage, col, m0, grp);
              tma_store_commit();
            }
            store_pending = true;
          }
        };
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_load_32cols(taddr + cc * 32, raw[cc]);
        tmem_load_wait();
        // Each chunk of the first half is converted and its registers are refilled at once with
        // the matching chunk of the second half, so those loads run under the conversion.
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          convert_chunk(cc, 0);
          tmem_load_32cols(taddr + 128 + cc * 32, raw[cc]);
        }
        tmem_load_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        stage_and_store(0);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) convert_chunk(cc, 1);
        stage_and_store(1);
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
        if constexpr (!SCATTER) store_row_chunk(p, grp, row, tn * BN + c * 32, vals);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
    }
    if (p.use_tma_store && threadIdx.x == 64) tma_store_wait_all<0>();
    // Stores that went to another GPU are fenced at system scope before the kernel ends.
    if constexpr (SCATTER) __threadfence_system();
  }

  // Neither CTA may leave (or give back tensor memory) while the pair's tensor core can still
  // read its shared memory or signal its barriers.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace b12x_b200
