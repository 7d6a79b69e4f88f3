// Thin inline-PTX layer for sm_100a: mbarriers with bounded waits, TMA (non-multicast)
// loads/stores, tensor-memory (TMEM) allocation, tcgen05 MMA / copy / load wrappers and
// the shared-memory and instruction descriptor encoders the GEMM kernels use.
//
// Every wait in this file is bounded: a wait that runs out of polls returns false, and the
// caller records a status word and leaves the kernel through its normal tear-down path.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b12x_b200 {

// ----------------------------------------------------------------------------------------
// Status words written to the caller-visible status buffer (0 = ok).
// ----------------------------------------------------------------------------------------
enum KernelStatus : int {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,   // TMA producer waited too long for a free stage
  kStatusMmaTimeout = 2,        // MMA issuer waited too long for a full stage / free accumulator
  kStatusEpilogueTimeout = 3,   // epilogue waited too long for a finished accumulator
  kStatusReduceTimeout = 4,     // split-K reduction waited too long for its peers
  kStatusTmemLayout = 5,        // tensor memory was not handed out from column 0
  kStatusPeerTimeout = 6,       // all-reduce over peer memory waited too long for another rank
};

// Polls allowed on one mbarrier phase before a wait gives up. Legitimate waits on this
// path are micro-seconds long; this limit is tens of milliseconds.
constexpr uint32_t kMaxBarrierPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Programmatic dependent launch. launch_dependents: the next grid in the stream (if it was
// launched with programmatic stream serialization) may start once every CTA of this grid has
// executed this or exited. wait: blocks until all grids this one depends on have completed and
// their memory is visible; returns at once when there is no such dependency.
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` (shared memory) lets every role leave once any role gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  for (uint32_t polls = 0; polls < kMaxBarrierPolls; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 1023u) == 1023u && *abort_flag != 0) return false;
  }
  return false;
}

// After a role gave up (abort flag set) copies of this CTA may still be in flight; give them a
// bounded time to land before shared memory and tensor memory are released.
__device__ __forceinline__ void drain_after_abort(volatile int* abort_flag) {
  if (*abort_flag == 0) return;
  const long long start = clock64();
  while (clock64() - start < 400000) {
  }
}

// Barrier 1 over the 128 epilogue threads, AND-reducing a predicate: lets the four epilogue
// warps agree on "everyone's wait succeeded" before any of them enters a barrier the others
// might never reach.
__device__ __forceinline__ bool epilogue_bar_and(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "barrier.cta.red.and.pred p, 1, 128, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

__device__ __forceinline__ void epilogue_bar_sync() {
  asm volatile("barrier.cta.sync 1, 128;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// TMA: tiled tensor loads (never multicast), plain bulk loads, tiled stores
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
      "r"(smem_addr_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Three-dimensional form: (x = bytes along K, y = row, z = group). Operands of a grouped GEMM
// are described by one map over [groups, rows, K], so a tile never reads across a group edge:
// rows at or beyond the group's row count are out of bounds and arrive as zeros.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_addr_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
      "r"(smem_addr_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map,
                                                 uint64_t* bar, int32_t x, int32_t y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_addr_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
      "r"(smem_addr_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_addr_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes),
      "r"(smem_addr_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src,
                                             int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr_u32(smem_src)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src,
                                             int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_addr_u32(smem_src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// 16-byte store that may target another GPU's memory (peer mapping).
__device__ __forceinline__ void st_global_v4_sys(void* p, const uint4& v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// ----------------------------------------------------------------------------------------
// Tensor memory
// ----------------------------------------------------------------------------------------
// Whole-warp calls. `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_addr_u32(smem_result)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_addr_u32(bar))
               : "memory");
}

// Shared memory -> tensor memory copy of one 32-row x 16-byte chunk, replicated into the four
// 32-lane quarters. This is the shape block-scale factors are staged in: one 128-row x 4-byte
// scale atom (512 bytes, row r at byte (r%32)*16 + (r/32)*4) becomes 4 TMEM columns.
__device__ __forceinline__ void tc_copy_sf_atom(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-block scale factors read from tensor memory.
// MXFP8 flavour: E4M3 operands, one UE8M0 scale per 32 elements of K, K = 32 per instruction.
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate,
                                            uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

// NVFP4 flavour: packed E2M1 operands, one UE4M3 scale per 16 elements, K = 64 per instruction.
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate,
                                            uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

// MXFP4: E2M1 codes with one UE8M0 scale per 32 elements, K = 64 per instruction (two scale
// bytes of each operand's 4-byte scale word, chosen by the scale ids in the descriptor: 0 or 2).
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate,
                                            uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

// Unscaled E4M3 x E4M3 -> FP32, K = 32 per instruction.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_load_32cols(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_16cols(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs driving one tcgen05 instruction stream, cta_group::2)
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Shared-memory address of the same variable in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// Arrive on an mbarrier that may live in the other CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // Default (CTA-scope release) semantics: the arrival only forwards the completion of
  // asynchronous copies, whose bytes the tensor core reads through the async proxy; a
  // cluster-scope release here cost ~900 cycles per arrival.
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on a barrier that the other CTA of the pair (or the pair's tensor core) signals.
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity,
                                                          volatile int* abort_flag) {
  for (uint32_t polls = 0; polls < kMaxBarrierPolls; ++polls) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((polls & 1023u) == 1023u && *abort_flag != 0) return false;
  }
  return false;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_addr_u32(smem_result)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// Completion of all prior tcgen05 work of the pair -> one arrival on the mbarrier at
// `cluster_addr` (own CTA or the peer).
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(cluster_addr)
               : "memory");
}

// Scale atom copy executed in both CTAs of the pair: each reads its own shared memory at the
// descriptor's offset and writes its own tensor memory.
__device__ __forceinline__ void tc_copy_sf_atom_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}

// 256-row MMA over the pair: rows 0..127 from the leader's A tile, 128..255 from the peer's;
// each CTA holds half of the B tile's rows; D lands in each CTA's own tensor memory.
__device__ __forceinline__ void tc_mma_mxf8_pair(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate,
                                                 uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

__device__ __forceinline__ void tc_mma_mxf4_pair(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate,
                                                 uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::2X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

// Unscaled E4M3 x E4M3 over the pair (256 rows), K = 32 per instruction.
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t d_taddr, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate,
                                                 uint32_t sfa_taddr, uint32_t sfb_taddr) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(d_taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_taddr),
      "r"(sfb_taddr)
      : "memory");
}

// ----------------------------------------------------------------------------------------
// Descriptors
// ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading-dim byte offset >> 4
//   [32,46) stride-dim byte offset >> 4   [46,48) version (1 on sm_100)
//   [49,52) base offset                [61,64) swizzle (0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B)
//
// K-major operand tile stored by TMA with 128-byte swizzle: rows are 128 bytes, eight rows form
// one 1024-byte swizzle atom, so the stride between 8-row groups is 1024 bytes. The tile base
// must be 1024-byte aligned; stepping along K inside the 128-byte row adds the byte offset to
// the start-address field.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_byte_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1024u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Unswizzled descriptor for one 32-row x 16-byte scale-factor chunk (four 8-row groups, 128
// bytes apart).
__device__ __forceinline__ uint64_t make_sf_chunk_desc(uint32_t smem_byte_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor, block-scaled kinds (32 bit):
//   [4,6) B scale id   [7,10) A format   [10,13) B format   [15] A major   [16] B major
//   [17,23) N >> 3     [23] scale format (0 = UE4M3, 1 = UE8M0)   [24,29) M >> 4
//   [29,31) A scale id [31] K size
// Formats: kind::mxf8f6f4 E4M3 = 0; kind::mxf4nvf4 E2M1 = 1.
__host__ __device__ constexpr uint32_t make_idesc_block_scaled(uint32_t m, uint32_t n,
                                                               uint32_t ab_format,
                                                               uint32_t scale_is_ue8m0) {
  return (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | (scale_is_ue8m0 << 23) |
         ((m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id,
                                                         uint32_t b_sf_id) {
  return idesc | (b_sf_id << 4) | (a_sf_id << 29);
}

// Instruction descriptor, kind::f8f6f4 with FP32 accumulation:
//   [4,6) D format (1 = F32)  [7,10) A format  [10,13) B format  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_f8(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace b12x_b200
