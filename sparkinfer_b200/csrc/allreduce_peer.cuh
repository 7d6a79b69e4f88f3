// Sum of the per-rank partial outputs of a row-parallel (K-split) linear, over peer memory.
//
// Every rank holds its partial [rows][ld] (BF16 or FP16) in a buffer that every other rank of
// the node has mapped (NVLink peer access). One kernel per rank, all ranks launching the same
// call: rank s owns the rows of slab s. It pulls that slab from every rank (its own included),
// adds the g values of an element in FP32 in rank order, rounds once, and pushes the result into
// the same place of every rank's buffer. Pull and push run in the same loop, so both directions
// of the links are busy at once; each direction carries (g - 1) / g of the matrix per rank.
// The result is the same on every rank bit for bit (each element is computed once), and for
// g = 2 equal to adding the two 2-byte partials and rounding.
//
// Ordering between ranks uses flag words in a small peer-mapped signal block per rank:
//   start: "my partial is complete" (sent by block 0 as the kernel begins; the GEMM that wrote
//          the partial precedes this kernel in the stream). Every block waits for all peers'.
//   end:   "all my pushes have been fenced" (sent by the rank's last block to finish). That block
//          waits for all peers' end flags, so that a finished kernel means the whole result is in
//          this rank's buffer and no peer will touch the buffer again.
// Flags carry a call number that only grows (kept in the signal block, advanced by the last
// block), so nothing is reset between calls and a captured graph can be replayed. Every wait is
// bounded: when it runs out the status word is raised, the data phase is skipped and the kernel
// returns.
//
// SCATTERED variant (after a GEMM that scattered its output, see ScatterOut in
// gemm_blockscaled_pair.cuh): every rank's partial of slab s already lies in rank s's own buffer,
// in slot r = rows [r * slab, (r + 1) * slab). Rank s then reads only local memory, and pushes
// the sum of its slab into a second buffer (`out`, rows [s * slab, (s + 1) * slab)) of every
// rank: the pull half of the traffic has been hidden under the GEMM's main loop.
//
// rank < 0 selects the single-GPU rehearsal used by the tests: blockIdx.y is the rank and all
// ranks run in one cooperative grid (kernels that wait on each other must not be separate
// launches on one GPU).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "gemm_blockscaled.cuh"  // pack_bf16x2 / pack_f16x2, output dtype codes
#include "sm100_ptx.cuh"

namespace b12x_b200 {

constexpr int kMaxPeers = 8;
// 32-bit words of a rank's signal block
constexpr int kSigCall = 0;       // number of completed calls
constexpr int kSigBlocksDone = 1; // blocks of the running call that have finished their share
constexpr int kSigStart = 8;      // [kSigStart + r]: rank r's partial of call n is complete
constexpr int kSigEnd = 16;       // [kSigEnd + r]: rank r has pushed and fenced its slab of call n
constexpr int kSigWords = 32;

struct PeerAllReduceParams {
  void* buf[kMaxPeers];      // rank r's [rows][ld] buffer as mapped in this process
  void* out[kMaxPeers];      // SCATTERED: rank r's [rows][ld] result buffer as mapped here
  uint32_t* sig[kMaxPeers];  // rank r's signal block as mapped in this process
  int world;
  int rank;                  // this process's rank; < 0: blockIdx.y (single-GPU rehearsal)
  long long rows, cols, ld;  // cols and ld multiples of 8 (16-byte vectors)
  int out_dtype;             // kOutBf16 or kOutFp16
  uint32_t max_polls;
  int* status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Flag store without a fence of its own: every use below follows either a kernel boundary or an
// explicit __threadfence_system(), which is what orders the data before the flag.
__device__ __forceinline__ void st_flag_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Data accesses at system scope (plain .cg accesses measured the same over NVLink).
__device__ __forceinline__ uint4 ld_peer_16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_16(uint4* p, const uint4& v) {
  asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Waits until `*flag` has reached `call` (numbers wrap, so compare the signed difference).
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t call, uint32_t max_polls) {
  for (uint32_t polls = 0; polls < max_polls; ++polls) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - call) >= 0) return true;
    __nanosleep(200);
  }
  return false;
}

template <bool BF16>
__device__ __forceinline__ void add_pairs(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
}

template <bool BF16>
__device__ __forceinline__ uint4 pack_sum(const float (&acc)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = BF16 ? pack_bf16x2(acc[2 * i], acc[2 * i + 1]) : pack_f16x2(acc[2 * i], acc[2 * i + 1]);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// G: number of ranks when known at compile time (2, 4, 8), 0 for any other count.
template <int G, bool BF16, bool SCATTERED>
__global__ void __launch_bounds__(512)
allreduce_peer_kernel(const PeerAllReduceParams p) {
  constexpr int kUnroll = (G == 2) ? 4 : 2;
  const int world = G ? G : p.world;
  const int me = p.rank >= 0 ? p.rank : static_cast<int>(blockIdx.y);
  uint32_t* mine = p.sig[me];
  __shared__ uint32_t s_call;
  __shared__ int s_last;
  // Written by this rank's previous call (an earlier kernel on this device): a plain load.
  if (threadIdx.x == 0) s_call = *reinterpret_cast<volatile uint32_t*>(mine + kSigCall) + 1;
  __syncthreads();
  const uint32_t call = s_call;

  const int t = static_cast<int>(threadIdx.x);
  // "My partial is complete": it was written (and, where it went to peers, fenced at system
  // scope) by the GEMM kernel that precedes this one in the stream, so the flag needs no fence.
  if (blockIdx.x == 0 && t < world && t != me) st_flag_sys(p.sig[t] + kSigStart + me, call);
  bool ok = true;
  if (t < world && t != me) ok = wait_flag(mine + kSigStart + t, call, p.max_polls);
  ok = __syncthreads_and(ok);
  if (!ok && t == 0 && p.status) atomicMax(p.status, kStatusPeerTimeout);

  if (ok) {
    // Slab of this rank: rows [r0, r1); vectors of 8 elements, row-major inside the slab.
    const long long r0 = p.rows * me / world;
    const long long r1 = p.rows * (me + 1) / world;
    const long long vec_per_row = p.cols / 8;
    const long long nvec = (r1 - r0) * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const bool dense = (p.ld == p.cols);
    const long long slab_elems = (p.rows / world) * p.ld;  // SCATTERED: rows % world == 0
    for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x + t; base < nvec;
         base += stride * kUnroll) {
      long long off[kUnroll];  // element offset of each vector from the start of a slab
      uint4 v[kUnroll][G ? G : kMaxPeers];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + u * stride;
        if (i < nvec) {
          off[u] = dense ? i * 8 : ((i / vec_per_row) * p.ld + (i % vec_per_row) * 8);
#pragma unroll
          for (int r = 0; r < (G ? G : kMaxPeers); ++r) {
            if (r < world) {
              // rank r's contribution: slot r of my own buffer, or my slab of rank r's buffer
              const uint16_t* src = SCATTERED
                                        ? static_cast<const uint16_t*>(p.buf[me]) + slab_elems * r
                                        : static_cast<const uint16_t*>(p.buf[r]) + r0 * p.ld;
              v[u][r] = ld_peer_16(reinterpret_cast<const uint4*>(src + off[u]));
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + u * stride;
        if (i < nvec) {
          float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int r = 0; r < (G ? G : kMaxPeers); ++r) {
            if (r < world) add_pairs<BF16>(acc, v[u][r]);
          }
          const uint4 out = pack_sum<BF16>(acc);
#pragma unroll
          for (int r = 0; r < (G ? G : kMaxPeers); ++r) {
            if (r < world) {
              uint16_t* dst = static_cast<uint16_t*>(SCATTERED ? p.out[r] : p.buf[r]) + r0 * p.ld;
              st_peer_16(reinterpret_cast<uint4*>(dst + off[u]), out);
            }
          }
        }
      }
    }
  }

  // Count this block in; the last one tells the peers, waits for theirs and closes the call.
  __threadfence_system();
  __syncthreads();
  if (t == 0) {
    const uint32_t prev = atomicAdd(mine + kSigBlocksDone, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  // Every block fenced its pushes at system scope before it was counted; this fence makes those
  // counts (and with them the pushes) precede the end flags.
  __threadfence_system();
  bool done = true;
  if (ok && t < world && t != me) {
    st_flag_sys(p.sig[t] + kSigEnd + me, call);
    done = wait_flag(mine + kSigEnd + t, call, p.max_polls);
  }
  done = __syncthreads_and(done);
  if (t == 0) {
    if (!done && p.status) atomicMax(p.status, kStatusPeerTimeout);
    // Read next by this rank's next call, a later kernel on this device.
    mine[kSigBlocksDone] = 0;
    mine[kSigCall] = call;
  }
}

}  // namespace b12x_b200
