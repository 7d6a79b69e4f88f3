// Host side of the C ABI: argument checks, TMA descriptor encoding, tile choice, launches.
#include "../../include/b12x_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "gemm_blockscaled.cuh"
#include "gemm_block_fp8.cuh"
#include "gemm_blockscaled_pair.cuh"
#include "gemm_smallm.cuh"
#include "quantize.cuh"
#include "allreduce_peer.cuh"
#include "pack_weight.cuh"
#include "bmm_mxfp8.cuh"

namespace b12x_b200 {
namespace {

thread_local char g_last_error[256] = "";

int fail_cuda(cudaError_t err, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(err));
  return B12X_B200_ERR_CUDA;
}

int fail(int code, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", what);
  return code;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime so the library carries no link-time
// dependency on libcuda (it must load on machines without a driver).
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// Checks of the optional epilogue description that do not depend on the kernel. `allow_quant`:
// whether the kernel that will run can re-quantize its output (only the decode kernel can).
int check_epilogue(const b12x_b200_epilogue_t* e, int c_dtype, int64_t n, bool allow_quant) {
  if (!e) return B12X_B200_OK;
  if (e->bias) {
    const uintptr_t align = (c_dtype == B12X_B200_FP32) ? 3 : 1;
    if (reinterpret_cast<uintptr_t>(e->bias) & align)
      return fail(B12X_B200_ERR_ALIGNMENT, "bias must be aligned to its element size");
  }
  if (e->quant_values) {
    if (!allow_quant)
      return fail(B12X_B200_ERR_UNSUPPORTED,
                  "output re-quantization is available in the decode kernel only (M <= 128)");
    if (c_dtype == B12X_B200_FP32)
      return fail(B12X_B200_ERR_UNSUPPORTED, "output re-quantization needs a BF16 or FP16 output");
    if (n % 32 != 0 || e->quant_cols % 32 != 0 || e->quant_col0 % 32 != 0 || e->quant_col0 < 0 ||
        e->quant_col0 + n > e->quant_cols || e->quant_ld < e->quant_cols ||
        e->quant_cols > INT32_MAX)
      return fail(B12X_B200_ERR_INVALID_ARGUMENT,
                  "re-quantized output: N, quant_col0 and quant_cols must be multiples of 32, "
                  "quant_col0 + N <= quant_cols <= quant_ld");
  } else if (e->quant_scale_rows || e->quant_scale_mma) {
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "quant scales given without quant_values");
  }
  return B12X_B200_OK;
}

// K-major byte matrix [rows, row_bytes] -> boxes of 128 bytes x box_rows, 128-byte swizzle.
int make_operand_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B12X_B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled failed (%d)", int(r));
    return B12X_B200_ERR_CUDA;
  }
  return B12X_B200_OK;
}

// Stack of `groups` K-major byte matrices [groups, rows, row_bytes] -> boxes of 128 bytes x
// box_rows x 1 group, 128-byte swizzle. A box never crosses into the next group: rows at or
// beyond `rows` are out of bounds and read as zeros.
int make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                     uint32_t box_rows, uint64_t groups = 1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B12X_B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[3] = {row_bytes, rows, groups};
  const cuuint64_t strides[2] = {row_bytes, rows * row_bytes};
  const cuuint32_t box[3] = {128, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled failed (%d)", int(r));
    return B12X_B200_ERR_CUDA;
  }
  return B12X_B200_OK;
}

// Row-major BF16 matrix [rows, cols] with row pitch `ld` elements -> unswizzled boxes of
// box_cols x box_rows elements (the raw activation rows of the fused-quantizer decode GEMM).
int make_raw_rows_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_cols, uint32_t box_rows, uint64_t groups = 1,
                      uint64_t group_stride = 0) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B12X_B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[3] = {cols, rows, groups};
  // Elements between the same row of consecutive groups: group-major [L][rows][ld] by default.
  const cuuint64_t strides[2] = {ld * 2, (group_stride ? group_stride : rows * ld) * 2};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box,
         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled(raw rows) failed (%d)", int(r));
    return B12X_B200_ERR_CUDA;
  }
  return B12X_B200_OK;
}

// Row-major 2-byte matrix [rows, cols] with row pitch `ld` elements -> boxes of 64 columns
// (128 bytes) x 128 rows, 128-byte swizzle; used for TMA stores of BF16/FP16 outputs.
int make_output_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B12X_B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box,
         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled(C) failed (%d)", int(r));
    return B12X_B200_ERR_CUDA;
  }
  return B12X_B200_OK;
}

// The same for a stack of `groups` outputs [groups, rows, ld] (a store never spills into the
// next group: rows at or beyond `rows` are clipped).
int make_output_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint64_t groups = 1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B12X_B200_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[3] = {cols, rows, groups};
  const cuuint64_t strides[2] = {ld * 2, rows * ld * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r =
      fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box,
         elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled(C) failed (%d)", int(r));
    return B12X_B200_ERR_CUDA;
  }
  return B12X_B200_OK;
}

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
};

int device_info(DeviceInfo* out) {
  static DeviceInfo cache[64];
  static bool have[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail_cuda(err, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 0 || dev >= 64) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "device index out of range");
  if (!have[dev]) {
    err = cudaDeviceGetAttribute(&cache[dev].sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return fail_cuda(err, "cudaDeviceGetAttribute");
    err = cudaDeviceGetAttribute(&cache[dev].cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (err != cudaSuccess) return fail_cuda(err, "cudaDeviceGetAttribute");
    have[dev] = true;
  }
  *out = cache[dev];
  return B12X_B200_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Experiment switches, read from the environment once per process (never on the launch path).
// They exist for measurements of kernel variants; none is part of the interface.
struct Switches {
  bool decode_overlap = true;   // programmatic stream serialization for decode GEMMs / quantizers
  bool pair_tail_split = true;  // split-K the last partial round of the CTA-pair kernel
  bool bmm_tensor_core = true;  // batched BF16 x MXFP8 product on warp-level MMAs when it fits
};

const Switches& switches() {
  static const Switches sw = [] {
    Switches v;
    if (const char* e = getenv("B12X_B200_DECODE_OVERLAP")) v.decode_overlap = atoi(e) != 0;
    if (const char* e = getenv("B12X_B200_PAIR_TAIL_SPLIT")) v.pair_tail_split = atoi(e) != 0;
    if (const char* e = getenv("B12X_B200_BMM_TENSOR_CORE")) v.bmm_tensor_core = atoi(e) != 0;
    return v;
  }();
  return sw;
}

// Tile width: fewest (waves x per-tile cost). The per-tile cost model is the bytes one k-step
// pulls through shared memory, (128 + BN) rows of 128 bytes, which tracks both the MMA time
// (proportional to BN) and the operand traffic.
int choose_block_n(int64_t m, int64_t n, int sms) {
  static const int candidates[] = {256, 192, 128, 64};
  const int64_t tiles_m = (m + 127) / 128;
  int best = 128;
  double best_cost = 1e300;
  for (int bn : candidates) {
    const int64_t tiles = tiles_m * ((n + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = double(waves) * (128 + bn);
    if (cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

template <int KIND, int BN, bool BIAS>
int launch_gemm_impl(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                     const GemmParams& p, int grid, cudaStream_t stream) {
  using T = GemmTile<KIND, BN>;
  // The large dynamic shared memory opt-in is per device: set it the first time each device
  // launches this instantiation.
  static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set_for[dev]) {
    const cudaError_t attr_err =
        cudaFuncSetAttribute(gemm_blockscaled_kernel<KIND, BN, BIAS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
    if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
    set_for[dev] = true;
  }
  GemmParams q = p;
  q.num_stages = (p.num_stages >= 2 && p.num_stages <= T::kStages) ? p.num_stages : T::kStages;
  gemm_blockscaled_kernel<KIND, BN, BIAS><<<grid, 192, T::kSmemBytes, stream>>>(map_a, map_b, map_c, q);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "gemm_blockscaled launch");
  return B12X_B200_OK;
}

template <int KIND, int BN>
int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                const GemmParams& p, int grid, cudaStream_t stream) {
  return p.bias ? launch_gemm_impl<KIND, BN, true>(map_a, map_b, map_c, p, grid, stream)
                : launch_gemm_impl<KIND, BN, false>(map_a, map_b, map_c, p, grid, stream);
}

// CTA-pair kernel: clusters of two CTAs, one 256 x BN tile per pair.
template <int KIND, int BN, bool BIAS, bool SCATTER = false>
int launch_gemm_pair_impl(const CUtensorMap& map_a, const CUtensorMap& map_b,
                          const CUtensorMap& map_c, const GemmParams& p, const PairTail& tail,
                          int pairs, cudaStream_t stream,
                          const ScatterOut<SCATTER>& sc = ScatterOut<SCATTER>{}) {
  using T = PairTile<KIND, BN, SCATTER ? 2 : 1>;
  static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set_for[dev]) {
    const cudaError_t attr_err =
        cudaFuncSetAttribute(gemm_blockscaled_pair_kernel<KIND, BN, BIAS, SCATTER>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
    if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
    set_for[dev] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(2 * pairs), 1, 1);
  cfg.blockDim = dim3(224, 1, 1);
  cfg.dynamicSmemBytes = T::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err =
      cudaLaunchKernelEx(&cfg, gemm_blockscaled_pair_kernel<KIND, BN, BIAS, SCATTER>, map_a, map_b,
                         map_c, p, tail, sc);
  if (err != cudaSuccess) return fail_cuda(err, "gemm_blockscaled_pair launch");
  return B12X_B200_OK;
}

template <int KIND, int BN>
int launch_gemm_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                     const GemmParams& p, const PairTail& tail, int pairs, cudaStream_t stream) {
  return p.bias ? launch_gemm_pair_impl<KIND, BN, true>(map_a, map_b, map_c, p, tail, pairs, stream)
                : launch_gemm_pair_impl<KIND, BN, false>(map_a, map_b, map_c, p, tail, pairs, stream);
}

// Rows up to which a quantized matrix is taken for an activation (its quantization releases the
// next kernel early) and a decode GEMM's weight for something a predecessor may just have
// written (its stream waits for the predecessor). One constant, so the two rules meet.
constexpr int kEarlyReleaseRows = 128;

// Launch configuration of a row quantizer: 256 threads, programmatic stream serialization.
struct QuantLaunch {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  QuantLaunch(unsigned blocks, cudaStream_t stream) {
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = switches().decode_overlap ? 1 : 0;
  }
};

template <int KIND>
int dispatch_block_n(int bn, const CUtensorMap& map_a, const CUtensorMap& map_b,
                     const CUtensorMap& map_c, const GemmParams& p, int grid,
                     cudaStream_t stream) {
  switch (bn) {
    case 64: return launch_gemm<KIND, 64>(map_a, map_b, map_c, p, grid, stream);
    case 128: return launch_gemm<KIND, 128>(map_a, map_b, map_c, p, grid, stream);
    case 192: return launch_gemm<KIND, 192>(map_a, map_b, map_c, p, grid, stream);
    case 256: return launch_gemm<KIND, 256>(map_a, map_b, map_c, p, grid, stream);
    default: return fail(B12X_B200_ERR_INVALID_ARGUMENT, "block_n must be 64, 128, 192 or 256");
  }
}

// Workspace layout shared by the kernels that need scratch (one buffer per stream serves them
// all, launches on a stream being ordered): 60 KiB of per-tile counters of the decode kernel,
// 4 KiB of counters of the CTA-pair kernel's split tail, then FP32 partial tiles from 64 KiB on.
constexpr size_t kSmallMCounterBytes = 60 * 1024;
constexpr size_t kPairCounterOffset = kSmallMCounterBytes;
constexpr size_t kPairCounterBytes = 4 * 1024;
constexpr size_t kWorkspaceHeaderBytes = kPairCounterOffset + kPairCounterBytes;

// Whether (and how) the CTA-pair kernel splits its last, partial round along K: `segments` per
// leftover tile (0 = no split) and the scratch it needs.
// Destinations of a row-parallel scatter (see ScatterOut in gemm_blockscaled_pair.cuh).
struct ScatterPlan {
  void* const* dst;
  int world;
  int rank;
};

struct PairTailPlan {
  int pairs = 0, left = 0, segments = 0;
  size_t bytes = 0;
};

PairTailPlan plan_pair_tail(int kind, int64_t m, int64_t n, int64_t k, int64_t groups, int sms) {
  PairTailPlan t;
  const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256) * groups;
  t.pairs = int(tiles < sms / 2 ? tiles : sms / 2);
  if (t.pairs < 1 || !switches().pair_tail_split) return t;
  const int64_t rounds = tiles / t.pairs;
  t.left = int(tiles - rounds * t.pairs);
  const int elems_per_stage =
      (kind == B12X_B200_KIND_NVFP4 || kind == B12X_B200_KIND_MXFP4) ? 256 : 128;
  const int64_t k_tiles = (k + elems_per_stage - 1) / elems_per_stage;
  // Split when the leftover tiles would keep at most half of the pairs busy, and never below two
  // k-tiles per segment. The split tiles are done FIRST, while all pairs are still in step: a
  // segment's epilogue waits for the other segments of its tile, and by the end of the kernel
  // the pairs have drifted apart by several microseconds. Done last, the split paid for that
  // drift (it saved nothing on 8192 x 7168 x 7168 and was restricted to a leftover of a tenth
  // of the pairs). Warm caches, split last -> split first: 4096 x 7168 x 18432 (4 tiles left on
  // 74 pairs) 179.1 -> 175.1-177.1 us; 4096 x 7168 x 9216 107.5 -> 101.2 us; 8192 x 7168 x 7168
  // (8 left, whole tiles under the old rule) 289.8 -> 285.7 us.
  if (t.left == 0 || t.left * 2 > t.pairs || size_t(t.left) * 2 * sizeof(int) > kPairCounterBytes)
    return t;
  int64_t seg = t.pairs / t.left;
  if (seg > k_tiles / 2) seg = k_tiles / 2;
  if (seg < 2) return t;
  t.segments = int(seg);
  t.bytes = kWorkspaceHeaderBytes +
            size_t(t.left) * t.segments * 2 * kPairPartialFloats * sizeof(float);
  return t;
}

}  // namespace
}  // namespace b12x_b200

using namespace b12x_b200;

extern "C" const char* b12x_b200_version(void) { return "b12x_b200 0.1.0 sm_100a"; }

extern "C" const char* b12x_b200_last_error(void) { return g_last_error; }

namespace {

int gemm_blockscaled_impl(int kind, const void* a, const void* sfa, const void* b, const void* sfb,
                          void* c, int c_dtype, const float* alpha, int64_t m, int64_t n, int64_t k,
                          int64_t ldc, int64_t groups, int block_n, int sm_count, void* workspace,
                          int64_t workspace_bytes, const b12x_b200_epilogue_t* epilogue,
                          int* status, b12x_b200_stream_t stream,
                          const ScatterPlan* scatter = nullptr) {
  if (groups < 1 || groups > 65535)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "groups must be in [1, 65535]");
  if (kind != B12X_B200_KIND_MXFP8 && kind != B12X_B200_KIND_NVFP4 && kind != B12X_B200_KIND_FP8 &&
      kind != B12X_B200_KIND_MXFP4)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "unknown operand kind");
  const bool scaled = kind != B12X_B200_KIND_FP8;
  const bool fp4 = kind == B12X_B200_KIND_NVFP4 || kind == B12X_B200_KIND_MXFP4;
  if (c_dtype < B12X_B200_BF16 || c_dtype > B12X_B200_FP32)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "unknown output dtype");
  if (m < 0 || n < 0 || k <= 0 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad problem size");
  if (block_n != 0 && block_n != B12X_B200_BLOCK_N_PAIR && block_n != 64 && block_n != 128 &&
      block_n != 192 && block_n != 256)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT,
                "block_n must be 0, 64, 128, 192, 256 or B12X_B200_BLOCK_N_PAIR");
  if (scatter) {
    if (scatter->world < 1 || scatter->world > kMaxScatter || scatter->rank < 0 ||
        scatter->rank >= scatter->world || !scatter->dst)
      return fail(B12X_B200_ERR_INVALID_ARGUMENT, "scatter: world in [1, 8], rank inside it");
    if (groups != 1 || epilogue || c_dtype == B12X_B200_FP32)
      return fail(B12X_B200_ERR_UNSUPPORTED,
                  "scatter: one group, no epilogue, BF16 or FP16 partials");
    if (m % (int64_t(scatter->world) * 256) != 0)
      return fail(B12X_B200_ERR_UNSUPPORTED, "scatter: M must be a multiple of 256 * world");
    if ((ldc * 2) % 16 != 0) return fail(B12X_B200_ERR_ALIGNMENT, "scatter: ld must be a multiple of 8");
    for (int r = 0; r < scatter->world; ++r)
      if (!scatter->dst[r] || !aligned16(scatter->dst[r]))
        return fail(B12X_B200_ERR_ALIGNMENT, "scatter: destinations must be 16-byte aligned");
    block_n = B12X_B200_BLOCK_N_PAIR;
    c = scatter->dst[scatter->rank];
  }
  if (m == 0 || n == 0) return B12X_B200_OK;
  if (!a || !b || !c || (scaled && (!sfa || !sfb)))
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (ldc < n) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "ldc < n");
  {
    const int erc = check_epilogue(epilogue, c_dtype, n, false);
    if (erc != B12X_B200_OK) return erc;
  }
  const int sf_vec = (kind == B12X_B200_KIND_NVFP4) ? 16 : 32;
  if (k % 32 != 0) return fail(B12X_B200_ERR_UNSUPPORTED, "K must be a multiple of 32");
  const int64_t row_bytes = fp4 ? k / 2 : k;
  if (row_bytes % 16 != 0) return fail(B12X_B200_ERR_ALIGNMENT, "operand rows must be 16-byte multiples");
  if (!aligned16(a) || !aligned16(b) || (scaled && (!aligned16(sfa) || !aligned16(sfb))))
    return fail(B12X_B200_ERR_ALIGNMENT, "operand and scale pointers must be 16-byte aligned");

  DeviceInfo info;
  int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  const int sms = (sm_count > 0 && sm_count < info.sm_count) ? sm_count : info.sm_count;
  if (block_n == B12X_B200_BLOCK_N_PAIR && sms < 2)
    return fail(B12X_B200_ERR_UNSUPPORTED, "the CTA-pair kernel needs two SMs");
  const int bn = block_n > 0 ? block_n : choose_block_n(m, n, sms);

  // Problems with enough 256 x 256 pair tiles go to the CTA-pair kernel unless a tile width was
  // forced. "Enough" is two thirds of the pairs: measured on 148 SMs the pair kernel wins from
  // 56 tiles up (512 x 7168, 1024 x 4096, 256 x 18432) and loses at 28-32 tiles.
  const int64_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256) * groups;
  const bool use_pair = (block_n == B12X_B200_BLOCK_N_PAIR) ||
                        ((block_n == 0) && (sms >= 2) && (pair_tiles * 3 >= sms));

  CUtensorMap map_a, map_b;
  rc = make_operand_map(&map_a, a, uint64_t(m), uint64_t(row_bytes), 128, uint64_t(groups));
  if (rc != B12X_B200_OK) return rc;
  rc = make_operand_map(&map_b, b, uint64_t(n), uint64_t(row_bytes),
                        use_pair ? 128u : uint32_t(bn), uint64_t(groups));
  if (rc != B12X_B200_OK) return rc;

  GemmParams p;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.c = c;
  p.alpha = alpha;
  p.status = status;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k);
  p.ldc = int(ldc);
  p.out_dtype = c_dtype;
  p.tiles_m = int((m + 127) / 128);
  p.tiles_n = int((n + bn - 1) / bn);
  p.k_atoms_total = scaled ? int((k + sf_vec * 4 - 1) / (sf_vec * 4)) : 0;
  p.group_m = 16;
  p.bias = epilogue ? epilogue->bias : nullptr;
  p.groups = int(groups);
  p.sfa_group_bytes = ((m + 127) / 128) * int64_t(p.k_atoms_total) * 512;
  p.sfb_group_bytes = ((n + 127) / 128) * int64_t(p.k_atoms_total) * 512;
  p.c_group_elems = m * ldc;
  p.num_stages = 0;  // filled per instantiation
  const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * groups;
  if (tiles > INT32_MAX) return fail(B12X_B200_ERR_UNSUPPORTED, "too many tiles");
  const int grid = int(tiles < sms ? tiles : sms);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Output through TMA when rows of C are 16-byte aligned 2-byte values; otherwise the
  // epilogue stores straight from registers.
  CUtensorMap map_c;
  memset(&map_c, 0, sizeof(map_c));
  p.use_tma_store = 0;
  if (c_dtype != B12X_B200_FP32 && aligned16(c) && (ldc * 2) % 16 == 0) {
    rc = make_output_map(&map_c, c, uint64_t(m), uint64_t(n), uint64_t(ldc), uint64_t(groups));
    if (rc != B12X_B200_OK) return rc;
    p.use_tma_store = 1;
  }
  if (use_pair) {
    p.tiles_m = int((m + 255) / 256);
    p.tiles_n = int((n + 255) / 256);
    // Tile rows per group of the tile order (a group walks all of N before the next group):
    // 8192 x 7168 x 7168 warm: 2 -> 289.8, 4 -> 287.7, 8 -> 285.7, 16 -> 281.6, 32 -> 291.8 us.
    p.group_m = 16;
    const int pairs = int(pair_tiles < sms / 2 ? pair_tiles : sms / 2);
    // The last partial round is split along K when the caller brought scratch for it.
    PairTail tail;
    tail.counters = nullptr;
    tail.partials = nullptr;
    tail.segments = 0;
    const PairTailPlan tp = plan_pair_tail(kind, m, n, k, groups, sms);
    if (workspace && tp.segments >= 2 && workspace_bytes >= int64_t(tp.bytes) &&
        aligned16(workspace)) {
      tail.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kPairCounterOffset);
      tail.partials =
          reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kWorkspaceHeaderBytes);
      tail.segments = -tp.segments;  // negative: the split tiles come first (see pair_work)
    }
    if (scatter) {
      ScatterOut<true> sc;
      memset(&sc, 0, sizeof(sc));
      sc.slab_rows = int(m / scatter->world);
      sc.rank = scatter->rank;
      sc.world = scatter->world;
      for (int r = 0; r < scatter->world; ++r) {
        sc.base[r] = scatter->dst[r];
      }
      if (kind == B12X_B200_KIND_MXFP8)
        return launch_gemm_pair_impl<kMxfp8, 256, false, true>(map_a, map_b, map_c, p, tail, pairs, s, sc);
      if (kind == B12X_B200_KIND_FP8)
        return launch_gemm_pair_impl<kFp8, 256, false, true>(map_a, map_b, map_c, p, tail, pairs, s, sc);
      if (kind == B12X_B200_KIND_MXFP4)
        return launch_gemm_pair_impl<kMxfp4, 256, false, true>(map_a, map_b, map_c, p, tail, pairs, s, sc);
      return launch_gemm_pair_impl<kNvfp4, 256, false, true>(map_a, map_b, map_c, p, tail, pairs, s, sc);
    }
    if (kind == B12X_B200_KIND_MXFP8)
      return launch_gemm_pair<kMxfp8, 256>(map_a, map_b, map_c, p, tail, pairs, s);
    if (kind == B12X_B200_KIND_FP8)
      return launch_gemm_pair<kFp8, 256>(map_a, map_b, map_c, p, tail, pairs, s);
    if (kind == B12X_B200_KIND_MXFP4)
      return launch_gemm_pair<kMxfp4, 256>(map_a, map_b, map_c, p, tail, pairs, s);
    return launch_gemm_pair<kNvfp4, 256>(map_a, map_b, map_c, p, tail, pairs, s);
  }
  if (kind == B12X_B200_KIND_MXFP8)
    return dispatch_block_n<kMxfp8>(bn, map_a, map_b, map_c, p, grid, s);
  if (kind == B12X_B200_KIND_FP8)
    return dispatch_block_n<kFp8>(bn, map_a, map_b, map_c, p, grid, s);
  if (kind == B12X_B200_KIND_MXFP4)
    return dispatch_block_n<kMxfp4>(bn, map_a, map_b, map_c, p, grid, s);
  return dispatch_block_n<kNvfp4>(bn, map_a, map_b, map_c, p, grid, s);
}

}  // namespace

extern "C" int b12x_b200_gemm_blockscaled(int kind, const void* a, const void* sfa, const void* b,
                                          const void* sfb, void* c, int c_dtype,
                                          const float* alpha, int64_t m, int64_t n, int64_t k,
                                          int64_t ldc, int block_n, int sm_count, int* status,
                                          b12x_b200_stream_t stream) {
  return gemm_blockscaled_impl(kind, a, sfa, b, sfb, c, c_dtype, alpha, m, n, k, ldc, 1, block_n,
                               sm_count, nullptr, 0, nullptr, status, stream);
}

extern "C" int b12x_b200_gemm_blockscaled_ex(int kind, const void* a, const void* sfa,
                                             const void* b, const void* sfb, void* c, int c_dtype,
                                             const float* alpha, int64_t m, int64_t n, int64_t k,
                                             int64_t ldc, int block_n, int sm_count,
                                             void* workspace, int64_t workspace_bytes,
                                             const b12x_b200_epilogue_t* epilogue, int* status,
                                             b12x_b200_stream_t stream) {
  return gemm_blockscaled_impl(kind, a, sfa, b, sfb, c, c_dtype, alpha, m, n, k, ldc, 1, block_n,
                               sm_count, workspace, workspace_bytes, epilogue, status, stream);
}

extern "C" int b12x_b200_gemm_blockscaled_grouped(int kind, const void* a, const void* sfa,
                                                  const void* b, const void* sfb, void* c,
                                                  int c_dtype, const float* alpha, int64_t m,
                                                  int64_t n, int64_t k, int64_t ldc,
                                                  int64_t groups, int block_n, int sm_count,
                                                  void* workspace, int64_t workspace_bytes,
                                                  const b12x_b200_epilogue_t* epilogue,
                                                  int* status, b12x_b200_stream_t stream) {
  return gemm_blockscaled_impl(kind, a, sfa, b, sfb, c, c_dtype, alpha, m, n, k, ldc, groups,
                               block_n, sm_count, workspace, workspace_bytes, epilogue, status,
                               stream);
}

namespace {

int64_t tiled_workspace_bytes(int kind, int64_t m, int64_t n, int64_t k, int64_t groups,
                              int block_n, int sm_count) {
  if (kind != B12X_B200_KIND_MXFP8 && kind != B12X_B200_KIND_NVFP4 && kind != B12X_B200_KIND_FP8 &&
      kind != B12X_B200_KIND_MXFP4)
    return -1;
  if (m <= 0 || n <= 0 || k <= 0 || groups < 1) return 0;
  DeviceInfo info;
  if (device_info(&info) != B12X_B200_OK) return -1;
  const int sms = (sm_count > 0 && sm_count < info.sm_count) ? sm_count : info.sm_count;
  const int64_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256) * groups;
  const bool use_pair = (block_n == B12X_B200_BLOCK_N_PAIR) ||
                        ((block_n == 0) && (sms >= 2) && (pair_tiles * 3 >= sms));
  if (!use_pair || sms < 2) return 0;
  const PairTailPlan tp = plan_pair_tail(kind, m, n, k, groups, sms);
  return tp.segments >= 2 ? int64_t(tp.bytes) : 0;
}

}  // namespace

extern "C" int64_t b12x_b200_gemm_blockscaled_workspace_bytes(int kind, int64_t m, int64_t n,
                                                              int64_t k, int block_n, int sm_count) {
  return tiled_workspace_bytes(kind, m, n, k, 1, block_n, sm_count);
}

extern "C" int b12x_b200_quantize_mxfp8_rows(const void* src, int src_dtype, int64_t ld_src,
                                             void* values, void* scale_rows, void* scale_mma,
                                             int64_t m, int64_t k, b12x_b200_stream_t stream) {
  if (src_dtype != B12X_B200_BF16 && src_dtype != B12X_B200_FP16)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "source must be BF16 or FP16");
  if (m < 0 || k <= 0 || m > INT32_MAX - 128 || k > INT32_MAX - 128)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad size");
  if (k % 32 != 0) return fail(B12X_B200_ERR_UNSUPPORTED, "K must be a multiple of 32");
  if (m == 0) return B12X_B200_OK;
  if (!src || !values) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (ld_src < k || ld_src % 8 != 0 || !aligned16(src) || !aligned16(values))
    return fail(B12X_B200_ERR_ALIGNMENT, "source rows and values must be 16-byte aligned");
  const int k_atoms = int((k + 127) / 128);
  const int rows_cover = scale_mma ? int((m + 127) / 128) * 128 : int(m);
  const int k_cover = scale_mma ? k_atoms * 128 : int(k);
  if (quant_warps(rows_cover, k_cover) > INT32_MAX)
    return fail(B12X_B200_ERR_UNSUPPORTED, "tensor too large");
  const int64_t blocks = (quant_warps(rows_cover, k_cover) + 7) / 8;  // 8 warps per CTA
  QuantLaunch launch(unsigned(blocks), reinterpret_cast<cudaStream_t>(stream));
  const int early = m <= kEarlyReleaseRows ? 1 : 0;
  cudaError_t err;
  if (src_dtype == B12X_B200_BF16)
    err = cudaLaunchKernelEx(&launch.cfg, quantize_mxfp8_rows_kernel<__nv_bfloat16>,
                             static_cast<const __nv_bfloat16*>(src), ld_src,
                             static_cast<uint8_t*>(values), static_cast<uint8_t*>(scale_rows),
                             static_cast<uint8_t*>(scale_mma), int(m), int(k), rows_cover, k_cover,
                             k_atoms, early);
  else
    err = cudaLaunchKernelEx(&launch.cfg, quantize_mxfp8_rows_kernel<__half>,
                             static_cast<const __half*>(src), ld_src,
                             static_cast<uint8_t*>(values), static_cast<uint8_t*>(scale_rows),
                             static_cast<uint8_t*>(scale_mma), int(m), int(k), rows_cover, k_cover,
                             k_atoms, early);
  if (err != cudaSuccess) return fail_cuda(err, "quantize_mxfp8_rows launch");
  return B12X_B200_OK;
}

extern "C" int b12x_b200_quantize_nvfp4_rows(const void* src, int src_dtype, int64_t ld_src,
                                             const float* global_scale, void* packed,
                                             void* scale_mma, int64_t m, int64_t k,
                                             b12x_b200_stream_t stream) {
  if (src_dtype != B12X_B200_BF16 && src_dtype != B12X_B200_FP16)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "source must be BF16 or FP16");
  if (m < 0 || k <= 0 || m > INT32_MAX - 128 || k > INT32_MAX - 128)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad size");
  if (k % 16 != 0) return fail(B12X_B200_ERR_UNSUPPORTED, "K must be a multiple of 16");
  if (m == 0) return B12X_B200_OK;
  if (!src || !packed || !scale_mma || !global_scale)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (ld_src < k || ld_src % 8 != 0 || !aligned16(src) || (reinterpret_cast<uintptr_t>(packed) & 7))
    return fail(B12X_B200_ERR_ALIGNMENT, "source rows must be 16-byte and packed 8-byte aligned");
  const int k_atoms = int((k + 63) / 64);
  const int rows_cover = int((m + 127) / 128) * 128;
  const int k_cover = k_atoms * 64;
  if (quant_warps(rows_cover, k_cover) > INT32_MAX)
    return fail(B12X_B200_ERR_UNSUPPORTED, "tensor too large");
  const int64_t blocks = (quant_warps(rows_cover, k_cover) + 7) / 8;  // 8 warps per CTA
  QuantLaunch launch(unsigned(blocks), reinterpret_cast<cudaStream_t>(stream));
  const int early = m <= kEarlyReleaseRows ? 1 : 0;
  cudaError_t err;
  if (src_dtype == B12X_B200_BF16)
    err = cudaLaunchKernelEx(&launch.cfg, quantize_nvfp4_rows_kernel<__nv_bfloat16>,
                             static_cast<const __nv_bfloat16*>(src), ld_src, global_scale,
                             static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scale_mma),
                             int(m), int(k), rows_cover, k_cover, k_atoms, early);
  else
    err = cudaLaunchKernelEx(&launch.cfg, quantize_nvfp4_rows_kernel<__half>,
                             static_cast<const __half*>(src), ld_src, global_scale,
                             static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scale_mma),
                             int(m), int(k), rows_cover, k_cover, k_atoms, early);
  if (err != cudaSuccess) return fail_cuda(err, "quantize_nvfp4_rows launch");
  return B12X_B200_OK;
}

namespace {

int gemm_block_fp8_impl(const void* a, const float* sfa, const void* b, const float* sfb, void* c,
                        int c_dtype, const float* alpha, int64_t m, int64_t n, int64_t k,
                        int64_t ldc, int sm_count, const b12x_b200_epilogue_t* epilogue,
                        int* status, b12x_b200_stream_t stream) {
  if (c_dtype < B12X_B200_BF16 || c_dtype > B12X_B200_FP32)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "unknown output dtype");
  if (m < 0 || n < 0 || k <= 0 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad problem size");
  if (n % 128 != 0 || k % 128 != 0)
    return fail(B12X_B200_ERR_UNSUPPORTED, "block-FP8 GEMM needs N and K divisible by 128");
  if (m == 0 || n == 0) return B12X_B200_OK;
  if (!a || !b || !sfa || !sfb || !c) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (ldc < n) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "ldc < n");
  if (!aligned16(a) || !aligned16(b) || (reinterpret_cast<uintptr_t>(sfa) & 3) ||
      (reinterpret_cast<uintptr_t>(sfb) & 3))
    return fail(B12X_B200_ERR_ALIGNMENT, "operands must be 16-byte and scales 4-byte aligned");
  {
    const int erc = check_epilogue(epilogue, c_dtype, n, false);
    if (erc != B12X_B200_OK) return erc;
  }
  DeviceInfo info;
  int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  const int sms = (sm_count > 0 && sm_count < info.sm_count) ? sm_count : info.sm_count;

  CUtensorMap map_a, map_b;
  rc = make_operand_map_2d(&map_a, a, uint64_t(m), uint64_t(k), BlockFp8Tile::BM);
  if (rc != B12X_B200_OK) return rc;
  rc = make_operand_map_2d(&map_b, b, uint64_t(n), uint64_t(k), BlockFp8Tile::BN);
  if (rc != B12X_B200_OK) return rc;

  BlockFp8Params p;
  p.sfa = sfa;
  p.sfb = sfb;
  p.c = c;
  p.alpha = alpha;
  p.status = status;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k);
  p.ldc = int(ldc);
  p.out_dtype = c_dtype;
  p.tiles_m = int((m + BlockFp8Tile::BM - 1) / BlockFp8Tile::BM);
  p.tiles_n = int((n + BlockFp8Tile::BN - 1) / BlockFp8Tile::BN);
  // Tile rows per group of the tile order: 4096 x 18432 x 7168 warm: 4 -> 525, 8 -> 508,
  // 16 -> 499, 32 (all rows of this problem) -> 496 us.
  p.group_m = 32;
  p.bias = epilogue ? epilogue->bias : nullptr;
  const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
  const int grid = int(tiles < sms ? tiles : sms);
  static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set_for[dev]) {
    cudaError_t attr_err =
        cudaFuncSetAttribute(gemm_block_fp8_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, BlockFp8Tile::kSmemBytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(gemm_block_fp8_kernel<true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      BlockFp8Tile::kSmemBytes);
    if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
    set_for[dev] = true;
  }
  // Output through TMA when rows of C are 16-byte aligned 2-byte values; otherwise the
  // epilogue stores straight from registers.
  CUtensorMap map_c;
  memset(&map_c, 0, sizeof(map_c));
  p.use_tma_store = 0;
  if (c_dtype != B12X_B200_FP32 && aligned16(c) && (ldc * 2) % 16 == 0) {
    rc = make_output_map_2d(&map_c, c, uint64_t(m), uint64_t(n), uint64_t(ldc));
    if (rc != B12X_B200_OK) return rc;
    p.use_tma_store = 1;
  }
  if (p.bias)
    gemm_block_fp8_kernel<true><<<grid, BlockFp8Tile::kThreads, BlockFp8Tile::kSmemBytes,
                                  reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, map_c, p);
  else
    gemm_block_fp8_kernel<false><<<grid, BlockFp8Tile::kThreads, BlockFp8Tile::kSmemBytes,
                                   reinterpret_cast<cudaStream_t>(stream)>>>(map_a, map_b, map_c, p);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "gemm_block_fp8 launch");
  return B12X_B200_OK;
}

}  // namespace

extern "C" int b12x_b200_gemm_block_fp8(const void* a, const float* sfa, const void* b,
                                        const float* sfb, void* c, int c_dtype,
                                        const float* alpha, int64_t m, int64_t n, int64_t k,
                                        int64_t ldc, int sm_count, int* status,
                                        b12x_b200_stream_t stream) {
  return gemm_block_fp8_impl(a, sfa, b, sfb, c, c_dtype, alpha, m, n, k, ldc, sm_count, nullptr,
                             status, stream);
}

extern "C" int b12x_b200_gemm_block_fp8_ex(const void* a, const float* sfa, const void* b,
                                           const float* sfb, void* c, int c_dtype,
                                           const float* alpha, int64_t m, int64_t n, int64_t k,
                                           int64_t ldc, int sm_count,
                                           const b12x_b200_epilogue_t* epilogue, int* status,
                                           b12x_b200_stream_t stream) {
  return gemm_block_fp8_impl(a, sfa, b, sfb, c, c_dtype, alpha, m, n, k, ldc, sm_count, epilogue,
                             status, stream);
}

namespace {

struct SmallMPlan {
  int m_pad, tiles, tiles_per_group, k_tiles, k_atoms, grid, max_segments, stages, stage_bytes;
  int issuers, sf_col0, tmem_cols, raw_rows;
  size_t partial_bytes, total_bytes;
};

// Geometry of the decode-shape kernel for (kind, m, n, k) on `sms` SMs; `fused` adds the raw
// BF16 activation rows (8 or 16 of them) to every stage. The workspace need does not depend on
// `fused`.
int plan_smallm(int kind, int64_t m, int64_t n, int64_t k, int sms, bool fused, int64_t groups,
                SmallMPlan* out) {
  if (m < 1 || m > 128) return fail(B12X_B200_ERR_UNSUPPORTED, "decode kernel needs 1 <= M <= 128");
  if (n < 1 || k < 1 || n > INT32_MAX || k > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad problem size");
  if (sms < 1) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "no SMs");
  const int sf_vec = (kind == B12X_B200_KIND_NVFP4) ? 16 : 32;
  const int elems_per_stage = (kind == B12X_B200_KIND_MXFP8) ? 128 : 256;
  SmallMPlan pl;
  pl.m_pad = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
  if (groups < 1 || groups > 65535 || ((n + 127) / 128) * groups > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "groups must be in [1, 65535]");
  pl.tiles_per_group = int((n + 127) / 128);
  pl.tiles = int(pl.tiles_per_group * groups);  // the tiles of all groups form one list
  pl.k_tiles = int((k + elems_per_stage - 1) / elems_per_stage);
  pl.k_atoms = int((k + sf_vec * 4 - 1) / (sf_vec * 4));
  const int64_t units = int64_t(pl.tiles) * pl.k_tiles;
  if (units >= (int64_t(1) << 31)) return fail(B12X_B200_ERR_UNSUPPORTED, "problem too large for the decode kernel");
  // Grid: with no more tiles than SMs, a whole number of CTAs per tile (capped by the k-tiles a
  // tile has) keeps every CTA range inside one tile, so a tile that gets a single CTA needs no
  // partial sums at all; with more tiles than SMs one CTA per SM streams an equal share.
  // (One CTA per SM regardless, which splits every tile of a 112-tile problem over two or three
  // CTAs, was measured slower: 12.6 us against 10.9 us for 16 x 14336 x 4096.)
  if (pl.tiles <= sms) {
    int per_tile = sms / pl.tiles;
    if (per_tile > pl.k_tiles) per_tile = pl.k_tiles;
    pl.grid = pl.tiles * per_tile;
  } else {
    pl.grid = int(units < sms ? units : sms);
  }
  const int64_t units_per_cta = units / pl.grid;  // >= 1
  int64_t seg = (pl.k_tiles + units_per_cta - 1) / units_per_cta + 1;
  if (seg > pl.grid) seg = pl.grid;
  pl.max_segments = int(seg);
  pl.stage_bytes = (kind == B12X_B200_KIND_MXFP8)   ? SmallMTile<kMxfp8>::stage_bytes(pl.m_pad)
                   : (kind == B12X_B200_KIND_NVFP4) ? SmallMTile<kNvfp4>::stage_bytes(pl.m_pad)
                                                    : SmallMTile<kMxfp4>::stage_bytes(pl.m_pad);
  pl.raw_rows = 0;
  if (fused) {
    pl.raw_rows = m <= 8 ? 8 : 16;
    const int x_offset = (kind == B12X_B200_KIND_MXFP8) ? SmallMTile<kMxfp8>::kXOffset
                                                        : SmallMTile<kNvfp4>::kXOffset;
    const int raw_bytes = pl.raw_rows * elems_per_stage * 2;
    pl.stage_bytes = ((x_offset + pl.m_pad * 128 + raw_bytes + 1023) / 1024) * 1024;
  }
  // Two issuing warps when four accumulators fit beside the scales (up to 64 padded rows).
  // The ring takes all of the SM's shared memory: a CTA sized for two per SM (so that the
  // next decode GEMM could run beside this one) was measured slower than a deep ring, twice:
  // with the ring capped at 4 stages the next two grids do become resident 20 us early, but a
  // chain of 16 x 14336 x 4096 GEMMs takes 11.5-11.8 us per GEMM against 10.5 (6 stages:
  // 10.8; 2 stages: 15.1): the shallow ring streams slower than the early start gains.
  pl.issuers = (pl.m_pad <= 64) ? 2 : 1;
  pl.sf_col0 = 2 * pl.issuers * pl.m_pad;
  const int cols = pl.sf_col0 + 2 * SmallMTile<kMxfp8>::kSfColsPerIssuer;
  pl.tmem_cols = cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
  const int smem_limit = 227 * 1024;
  int stages = (smem_limit - kSmallMTailBytes) / pl.stage_bytes;
  if (stages > SmallMTile<kMxfp8>::kMaxStages) stages = SmallMTile<kMxfp8>::kMaxStages;
  // With two issuing warps taking alternate units, a stage must always come back to the same
  // warp: with an odd ring a warp would skip every other phase of a stage's barrier, and a
  // parity wait cannot tell a phase from the one two before it.
  if (pl.issuers == 2) stages &= ~1;
  if (stages < 2) return fail(B12X_B200_ERR_UNSUPPORTED, "decode kernel stage does not fit");
  pl.stages = stages;
  pl.partial_bytes = size_t(pl.tiles) * pl.max_segments * pl.m_pad * 128 * sizeof(float);
  if (size_t(pl.tiles) * sizeof(int) > kSmallMCounterBytes)
    return fail(B12X_B200_ERR_UNSUPPORTED, "N too large for the decode kernel's counter block");
  pl.total_bytes = kWorkspaceHeaderBytes + pl.partial_bytes;
  *out = pl;
  return B12X_B200_OK;
}

template <int KIND, bool FUSED, bool EPI, bool ROPE = false>
int launch_smallm_impl(const CUtensorMap& map_w, const CUtensorMap& map_x, const SmallMParams& p,
                       int grid, int smem_bytes, cudaStream_t stream) {
  static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set_for[dev]) {
    const cudaError_t attr_err = cudaFuncSetAttribute(
        gemm_smallm_kernel<KIND, FUSED, EPI, ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
    // Largest shared-memory carve-out: the ring takes nearly all of it.
    const cudaError_t carve_err = cudaFuncSetAttribute(
        gemm_smallm_kernel<KIND, FUSED, EPI, ROPE>, cudaFuncAttributePreferredSharedMemoryCarveout,
        cudaSharedmemCarveoutMaxShared);
    if (carve_err != cudaSuccess) return fail_cuda(carve_err, "cudaFuncSetAttribute");
    set_for[dev] = true;
  }
  // Programmatic stream serialization: this grid may start while the previous one in the stream
  // is still running (if that one releases its dependents early, as this kernel does); the
  // kernel itself waits for the predecessor before it touches anything the predecessor may own.
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(FUSED ? 512 : 256, 1, 1);
  cfg.dynamicSmemBytes = size_t(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = switches().decode_overlap ? 1 : 0;
  const cudaError_t err =
      cudaLaunchKernelEx(&cfg, gemm_smallm_kernel<KIND, FUSED, EPI, ROPE>, map_w, map_x, p);
  if (err != cudaSuccess) return fail_cuda(err, "gemm_smallm launch");
  return B12X_B200_OK;
}

template <int KIND, bool FUSED>
int launch_smallm(const CUtensorMap& map_w, const CUtensorMap& map_x, const SmallMParams& p,
                  int grid, int smem_bytes, cudaStream_t stream) {
  return (p.bias || p.quant_values)
             ? launch_smallm_impl<KIND, FUSED, true>(map_w, map_x, p, grid, smem_bytes, stream)
             : launch_smallm_impl<KIND, FUSED, false>(map_w, map_x, p, grid, smem_bytes, stream);
}

// One decode-shape GEMM request, as every entry point of the family describes it. `x` / `sf_x`
// are codes and scale atoms; with `x_src` set instead the activation rows are BF16 and are
// quantized inside the kernel (`x_gs` = their NVFP4 global scale).
struct SmallMCall {
  int kind;
  const void* x;
  const void* sf_x;
  const void* x_src;
  int64_t ld_x;
  const float* x_gs;
  const void* w;
  const void* sf_w;
  void* c;
  int c_dtype;
  const float* alpha;
  int64_t m, n, k, ldc;
  int sm_count;
  int* status;
  unsigned long long* timeline;
  cudaStream_t stream;
  const b12x_b200_epilogue_t* epilogue = nullptr;
  int64_t groups = 1;
  int64_t x_group_stride = 0;  // fused rows: elements between groups (0: group-major rows)
  // Inverse rotary embedding in front of the fused MXFP8 quantizer (null positions: none).
  const void* rope_positions = nullptr;
  const void* rope_cos_sin = nullptr;
  int rope_pos_i64 = 0, rope_cache_f32 = 0;
  int rope_head_dim = 0, rope_nope_dim = 0, rope_dim = 0;
};

// Argument checks shared by the decode-shape entry points. On success *empty is set when there
// is nothing to compute, otherwise *plan and *sms describe the launch. Nothing is enqueued.
int check_smallm(const SmallMCall& a, SmallMPlan* plan, int* sms_out, bool* empty) {
  *empty = false;
  const bool fused = a.x_src != nullptr;
  if (a.kind == B12X_B200_KIND_MXFP4 && fused)
    return fail(B12X_B200_ERR_UNSUPPORTED, "no activation quantizer produces MXFP4");
  if (a.rope_positions || a.rope_cos_sin) {
    if (!a.rope_positions || !a.rope_cos_sin)
      return fail(B12X_B200_ERR_INVALID_ARGUMENT, "inverse-RoPE needs both positions and cos_sin_cache");
    if (!fused || a.kind != B12X_B200_KIND_MXFP8 || a.epilogue)
      return fail(B12X_B200_ERR_UNSUPPORTED,
                  "inverse-RoPE belongs to the fused MXFP8 activation quantizer without epilogue");
    if (a.rope_head_dim <= 0 || a.rope_nope_dim < 0 || a.rope_dim <= 0 ||
        a.rope_nope_dim + a.rope_dim != a.rope_head_dim || a.rope_head_dim % 32 != 0 ||
        a.rope_nope_dim % 32 != 0 || a.rope_dim % 32 != 0 || a.k % a.rope_head_dim != 0)
      return fail(B12X_B200_ERR_INVALID_ARGUMENT,
                  "inverse-RoPE requires 32-aligned head_dim = nope_dim + rope_dim dividing K");
  }
  if (a.kind != B12X_B200_KIND_MXFP8 && a.kind != B12X_B200_KIND_NVFP4 &&
      a.kind != B12X_B200_KIND_MXFP4)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "unknown operand kind");
  if (a.c_dtype < B12X_B200_BF16 || a.c_dtype > B12X_B200_FP32)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "unknown output dtype");
  if (a.m < 0 || a.n < 0 || a.k <= 0 || a.n > INT32_MAX || a.k > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad problem size");
  if (a.m == 0 || a.n == 0) {
    *empty = true;
    return B12X_B200_OK;
  }
  if (!a.w || !a.sf_w || !a.c) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (a.ldc < a.n) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "ldc < n");
  {
    const int erc = check_epilogue(a.epilogue, a.c_dtype, a.n, true);
    if (erc != B12X_B200_OK) return erc;
  }
  if (a.k % 32 != 0) return fail(B12X_B200_ERR_UNSUPPORTED, "K must be a multiple of 32");
  const int64_t row_bytes = (a.kind == B12X_B200_KIND_MXFP8) ? a.k : a.k / 2;
  if (row_bytes % 16 != 0 || !aligned16(a.w) || !aligned16(a.sf_w))
    return fail(B12X_B200_ERR_ALIGNMENT, "operands and scales must be 16-byte aligned");
  if (fused) {
    if (a.m > 16)
      return fail(B12X_B200_ERR_UNSUPPORTED, "fused activation quantization needs M <= 16");
    if (a.kind == B12X_B200_KIND_NVFP4 && !a.x_gs)
      return fail(B12X_B200_ERR_INVALID_ARGUMENT, "NVFP4 activations need a global scale");
    if (a.ld_x < a.k || a.ld_x % 8 != 0 || !aligned16(a.x_src))
      return fail(B12X_B200_ERR_ALIGNMENT, "activation rows must be 16-byte aligned");
  } else {
    if (!a.x || !a.sf_x) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
    if (!aligned16(a.x) || !aligned16(a.sf_x))
      return fail(B12X_B200_ERR_ALIGNMENT, "operands and scales must be 16-byte aligned");
  }
  DeviceInfo info;
  int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  *sms_out = (a.sm_count > 0 && a.sm_count < info.sm_count) ? a.sm_count : info.sm_count;
  return plan_smallm(a.kind, a.m, a.n, a.k, *sms_out, fused, a.groups, plan);
}

int run_smallm(const SmallMCall& a, const SmallMPlan& pl, void* workspace,
               int64_t workspace_bytes) {
  const bool fused = a.x_src != nullptr;
  if (!workspace) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (!aligned16(workspace))
    return fail(B12X_B200_ERR_ALIGNMENT, "workspace must be 16-byte aligned");
  if (workspace_bytes < int64_t(pl.total_bytes))
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "workspace smaller than b12x_b200_gemm_smallm_workspace_bytes");
  const int64_t row_bytes = (a.kind == B12X_B200_KIND_MXFP8) ? a.k : a.k / 2;
  CUtensorMap map_w, map_x;
  int rc = make_operand_map(&map_w, a.w, uint64_t(a.n), uint64_t(row_bytes), 128, uint64_t(a.groups));
  if (rc != B12X_B200_OK) return rc;
  if (fused) {
    const uint32_t elems = (a.kind == B12X_B200_KIND_MXFP8) ? 128u : 256u;
    rc = make_raw_rows_map(&map_x, a.x_src, uint64_t(a.m), uint64_t(a.k), uint64_t(a.ld_x), elems,
                           uint32_t(pl.raw_rows), uint64_t(a.groups), uint64_t(a.x_group_stride));
    if (rc != B12X_B200_OK) return rc;
  } else {
    rc = make_operand_map(&map_x, a.x, uint64_t(a.m), uint64_t(row_bytes), uint32_t(pl.m_pad),
                          uint64_t(a.groups));
    if (rc != B12X_B200_OK) return rc;
  }

  SmallMParams p;
  memset(&p, 0, sizeof(p));
  p.sf_w = static_cast<const uint8_t*>(a.sf_w);
  p.sf_x = static_cast<const uint8_t*>(a.sf_x);
  p.c = a.c;
  p.alpha = a.alpha;
  p.status = a.status;
  p.counters = static_cast<int*>(workspace);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kWorkspaceHeaderBytes);
  p.m = int(a.m);
  p.n = int(a.n);
  p.k = int(a.k);
  p.ldc = int(a.ldc);
  p.out_dtype = a.c_dtype;
  p.m_pad = pl.m_pad;
  p.tiles = pl.tiles;
  p.tiles_per_group = pl.tiles_per_group;
  p.sf_w_group_bytes = int64_t(pl.tiles_per_group) * pl.k_atoms * 512;
  p.sf_x_group_bytes = int64_t(pl.k_atoms) * 512;  // one row tile of activations per group
  p.c_group_elems = a.m * a.ldc;
  p.k_tiles = pl.k_tiles;
  p.k_atoms_total = pl.k_atoms;
  p.max_segments = pl.max_segments;
  p.num_stages = pl.stages;
  p.stage_bytes = pl.stage_bytes;
  p.issuers = pl.issuers;
  p.tmem_cols = pl.tmem_cols;
  p.sf_col0 = pl.sf_col0;
  p.x_gs = a.x_gs;
  p.raw_rows = pl.raw_rows;
  p.rope_positions = a.rope_positions;
  p.rope_cos_sin = a.rope_cos_sin;
  p.rope_pos_i64 = a.rope_pos_i64;
  p.rope_cache_f32 = a.rope_cache_f32;
  p.rope_head_dim = a.rope_head_dim;
  p.rope_nope_dim = a.rope_nope_dim;
  p.rope_dim = a.rope_dim;
  if (a.epilogue) {
    p.bias = a.epilogue->bias;
    p.quant_values = static_cast<uint8_t*>(a.epilogue->quant_values);
    p.quant_scale_rows = static_cast<uint8_t*>(a.epilogue->quant_scale_rows);
    p.quant_scale_mma = static_cast<uint8_t*>(a.epilogue->quant_scale_mma);
    p.quant_ld = a.epilogue->quant_ld;
    p.quant_col0 = int(a.epilogue->quant_col0);
    p.quant_cols = int(a.epilogue->quant_cols);
  }
  p.wait_for_weights = a.n <= kEarlyReleaseRows ? 1 : 0;
  p.timeline = a.timeline;
  p.packed_store = (a.c_dtype != B12X_B200_FP32 && aligned16(a.c) && a.ldc % 8 == 0) ? 1 : 0;
  p.smem_bytes = pl.stages * pl.stage_bytes + kSmallMTailBytes;
  const int smem_bytes = pl.stages * pl.stage_bytes + kSmallMTailBytes;
  if (a.rope_positions)   // checked: MXFP8, fused, no epilogue
    return launch_smallm_impl<kMxfp8, true, false, true>(map_w, map_x, p, pl.grid, smem_bytes, a.stream);
  if (a.kind == B12X_B200_KIND_MXFP8)
    return fused ? launch_smallm<kMxfp8, true>(map_w, map_x, p, pl.grid, smem_bytes, a.stream)
                 : launch_smallm<kMxfp8, false>(map_w, map_x, p, pl.grid, smem_bytes, a.stream);
  if (a.kind == B12X_B200_KIND_MXFP4)
    return launch_smallm<kMxfp4, false>(map_w, map_x, p, pl.grid, smem_bytes, a.stream);
  return fused ? launch_smallm<kNvfp4, true>(map_w, map_x, p, pl.grid, smem_bytes, a.stream)
               : launch_smallm<kNvfp4, false>(map_w, map_x, p, pl.grid, smem_bytes, a.stream);
}

int smallm_entry(const SmallMCall& a, void* workspace, int64_t workspace_bytes) {
  SmallMPlan pl;
  int sms = 0;
  bool empty = false;
  const int rc = check_smallm(a, &pl, &sms, &empty);
  if (rc != B12X_B200_OK || empty) return rc;
  return run_smallm(a, pl, workspace, workspace_bytes);
}

}  // namespace

extern "C" int64_t b12x_b200_gemm_smallm_workspace_bytes(int kind, int64_t m, int64_t n, int64_t k,
                                                         int sm_count) {
  if (kind != B12X_B200_KIND_MXFP8 && kind != B12X_B200_KIND_NVFP4 && kind != B12X_B200_KIND_MXFP4)
    return -1;
  if (n <= 0 || k <= 0) return -1;
  // Same SM count as the launch will use: the caller's limit, capped by the device.
  DeviceInfo info;
  if (device_info(&info) != B12X_B200_OK) return -1;
  const int sms = (sm_count > 0 && sm_count < info.sm_count) ? sm_count : info.sm_count;
  SmallMPlan pl;
  if (plan_smallm(kind, m, n, k, sms, false, 1, &pl) != B12X_B200_OK) return -1;
  return int64_t(pl.total_bytes);
}

extern "C" int b12x_b200_gemm_blockscaled_smallm(int kind, const void* x, const void* sf_x,
                                                 const void* w, const void* sf_w, void* c,
                                                 int c_dtype, const float* alpha, int64_t m,
                                                 int64_t n, int64_t k, int64_t ldc,
                                                 void* workspace, int64_t workspace_bytes,
                                                 int sm_count, int* status,
                                                 b12x_b200_stream_t stream) {
  SmallMCall a = {kind, x,     sf_x, nullptr, 0,   nullptr,  w,      sf_w,    c, c_dtype,
                  alpha, m,    n,    k,       ldc, sm_count, status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int b12x_b200_gemm_blockscaled_smallm_ex(int kind, const void* x, const void* sf_x,
                                                    const void* w, const void* sf_w, void* c,
                                                    int c_dtype, const float* alpha, int64_t m,
                                                    int64_t n, int64_t k, int64_t ldc,
                                                    void* workspace, int64_t workspace_bytes,
                                                    const b12x_b200_epilogue_t* epilogue,
                                                    int sm_count, int* status,
                                                    b12x_b200_stream_t stream) {
  SmallMCall a = {kind, x,     sf_x, nullptr, 0,   nullptr,  w,      sf_w,    c, c_dtype,
                  alpha, m,    n,    k,       ldc, sm_count, status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  a.epilogue = epilogue;
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int b12x_b200_gemm_blockscaled_smallm_grouped(
    int kind, const void* x, const void* sf_x, const void* w, const void* sf_w, void* c, int c_dtype,
    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t groups,
    void* workspace, int64_t workspace_bytes, const b12x_b200_epilogue_t* epilogue, int sm_count,
    int* status, b12x_b200_stream_t stream) {
  SmallMCall a = {kind, x,     sf_x, nullptr, 0,   nullptr,  w,      sf_w,    c, c_dtype,
                  alpha, m,    n,    k,       ldc, sm_count, status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  a.epilogue = epilogue;
  a.groups = groups;
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int64_t b12x_b200_gemm_grouped_workspace_bytes(int kind, int decode, int64_t m,
                                                          int64_t n, int64_t k, int64_t groups,
                                                          int block_n, int sm_count) {
  if (!decode) return tiled_workspace_bytes(kind, m, n, k, groups, block_n, sm_count);
  if (kind != B12X_B200_KIND_MXFP8 && kind != B12X_B200_KIND_NVFP4 && kind != B12X_B200_KIND_MXFP4)
    return -1;
  if (n <= 0 || k <= 0) return -1;
  DeviceInfo info;
  if (device_info(&info) != B12X_B200_OK) return -1;
  const int sms = (sm_count > 0 && sm_count < info.sm_count) ? sm_count : info.sm_count;
  SmallMPlan pl;
  if (plan_smallm(kind, m, n, k, sms, false, groups, &pl) != B12X_B200_OK) return -1;
  return int64_t(pl.total_bytes);
}

extern "C" int b12x_b200_gemm_smallm_fused_quant(int kind, const void* x_bf16, int64_t ld_x,
                                                 const float* x_global_scale, const void* w,
                                                 const void* sf_w, void* c, int c_dtype,
                                                 const float* alpha, int64_t m, int64_t n,
                                                 int64_t k, int64_t ldc, void* workspace,
                                                 int64_t workspace_bytes,
                                                 const b12x_b200_epilogue_t* epilogue,
                                                 int sm_count, int* status,
                                                 b12x_b200_stream_t stream) {
  if (!x_bf16) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  SmallMCall a = {kind,  nullptr, nullptr, x_bf16, ld_x, x_global_scale, w,      sf_w,    c, c_dtype,
                  alpha, m,       n,       k,      ldc,  sm_count,       status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  a.epilogue = epilogue;
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int b12x_b200_gemm_smallm_fused_quant_grouped(
    int kind, const void* x_bf16, int64_t ld_x, int64_t x_group_stride,
    const float* x_global_scale, const void* w, const void* sf_w, void* c, int c_dtype,
    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t groups,
    void* workspace, int64_t workspace_bytes, const b12x_b200_epilogue_t* epilogue, int sm_count,
    int* status, b12x_b200_stream_t stream) {
  if (!x_bf16) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (groups < 1) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "groups must be positive");
  if (groups > 1 && (x_group_stride < k || x_group_stride % 8 != 0))
    return fail(B12X_B200_ERR_ALIGNMENT, "activation groups must be 16-byte aligned and K apart at least");
  SmallMCall a = {kind,  nullptr, nullptr, x_bf16, ld_x, x_global_scale, w,      sf_w,    c, c_dtype,
                  alpha, m,       n,       k,      ldc,  sm_count,       status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  a.epilogue = epilogue;
  a.groups = groups;
  a.x_group_stride = groups > 1 ? x_group_stride : 0;
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int b12x_b200_gemm_smallm_fused_quant_grouped_inv_rope(
    const void* x_bf16, int64_t ld_x, int64_t x_group_stride, const void* positions,
    int positions_are_int64, const void* cos_sin_cache, int cache_is_fp32, int head_dim,
    int nope_dim, int rope_dim, const void* w, const void* sf_w, void* c, int c_dtype,
    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t groups,
    void* workspace, int64_t workspace_bytes, int sm_count, int* status,
    b12x_b200_stream_t stream) {
  if (!x_bf16 || !positions || !cos_sin_cache)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (groups < 1) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "groups must be positive");
  if (groups > 1 && (x_group_stride < k || x_group_stride % 8 != 0))
    return fail(B12X_B200_ERR_ALIGNMENT, "activation groups must be 16-byte aligned and K apart at least");
  SmallMCall a = {B12X_B200_KIND_MXFP8, nullptr, nullptr, x_bf16, ld_x, nullptr, w, sf_w, c, c_dtype,
                  alpha, m, n, k, ldc, sm_count, status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  a.groups = groups;
  a.x_group_stride = groups > 1 ? x_group_stride : 0;
  a.rope_positions = positions;
  a.rope_cos_sin = cos_sin_cache;
  a.rope_pos_i64 = positions_are_int64 ? 1 : 0;
  a.rope_cache_f32 = cache_is_fp32 ? 1 : 0;
  a.rope_head_dim = head_dim;
  a.rope_nope_dim = nope_dim;
  a.rope_dim = rope_dim;
  return smallm_entry(a, workspace, workspace_bytes);
}

extern "C" int b12x_b200_gemm_smallm_timeline(int kind, const void* x, const void* sf_x,
                                              const void* w, const void* sf_w, void* c,
                                              int c_dtype, const float* alpha, int64_t m,
                                              int64_t n, int64_t k, int64_t ldc, void* workspace,
                                              int64_t workspace_bytes, int sm_count,
                                              unsigned long long* stamps, int64_t stamps_len,
                                              int* status, b12x_b200_stream_t stream) {
  SmallMCall a = {kind, x,     sf_x, nullptr, 0,   nullptr,  w,      sf_w,   c, c_dtype,
                  alpha, m,    n,    k,       ldc, sm_count, status, stamps,
                  reinterpret_cast<cudaStream_t>(stream)};
  SmallMPlan pl;
  int sms = 0;
  bool empty = false;
  const int rc = check_smallm(a, &pl, &sms, &empty);
  if (rc != B12X_B200_OK || empty) return rc;
  if (!stamps || stamps_len < int64_t(pl.grid) * kTimelineSlots)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "stamp buffer needs 8 entries per SM");
  return run_smallm(a, pl, workspace, workspace_bytes);
}

// ----------------------------------------------------------------------------------------
// Decode-shape GEMM for callers that cannot allocate device memory
// ----------------------------------------------------------------------------------------
namespace {

// Scratch of the allocation-free entry point: the 64 KiB counter block plus 4 MiB of FP32
// partial tiles. It is part of the library image, so every GPU that loads the library keeps
// these bytes for the life of the process.
constexpr size_t kNoAllocScratchBytes = kWorkspaceHeaderBytes + (size_t(4) << 20);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of g_noalloc_scratch per device. In host code the array's name is only a
// handle for the runtime, not a device pointer, so the address is looked up once per device.
void* g_noalloc_scratch_ptr[64] = {};
std::mutex g_noalloc_mu;

}  // namespace

extern "C" int64_t b12x_b200_gemm_smallm_noalloc_capacity_bytes(void) {
  return int64_t(kNoAllocScratchBytes);
}

extern "C" int b12x_b200_gemm_blockscaled_smallm_noalloc(int kind, const void* x, const void* sf_x,
                                                         const void* w, const void* sf_w, void* c,
                                                         int c_dtype, const float* alpha,
                                                         int64_t m, int64_t n, int64_t k,
                                                         int64_t ldc, int sm_count, int* status,
                                                         b12x_b200_stream_t stream) {
  // Every argument check (the device's compute capability among them) comes before the symbol
  // look-up and before anything is put on the stream, so a refused call leaves no trace.
  SmallMCall a = {kind, x,     sf_x, nullptr, 0,   nullptr,  w,      sf_w,    c, c_dtype,
                  alpha, m,    n,    k,       ldc, sm_count, status, nullptr,
                  reinterpret_cast<cudaStream_t>(stream)};
  SmallMPlan pl;
  int sms = 0;
  bool empty = false;
  int rc = check_smallm(a, &pl, &sms, &empty);
  if (rc != B12X_B200_OK || empty) return rc;
  if (pl.total_bytes > kNoAllocScratchBytes) {
    snprintf(g_last_error, sizeof(g_last_error),
             "M=%lld N=%lld K=%lld needs %zu bytes of scratch; the built-in scratch of the "
             "allocation-free entry point holds %zu",
             static_cast<long long>(m), static_cast<long long>(n), static_cast<long long>(k),
             pl.total_bytes, kNoAllocScratchBytes);
    return B12X_B200_ERR_UNSUPPORTED;
  }
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail_cuda(err, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "device index out of range");
  void* scratch = nullptr;
  {
    // First call on this device: resolve the device address of the static array (the device
    // must be current, which it is: it is the one cudaGetDevice just reported).
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_scratch_ptr[dev]) {
      void* ptr = nullptr;
      err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (err != cudaSuccess) return fail_cuda(err, "cudaGetSymbolAddress(g_noalloc_scratch)");
      g_noalloc_scratch_ptr[dev] = ptr;
    }
    scratch = g_noalloc_scratch_ptr[dev];
  }
  // The array keeps whatever the previous call left. Only the per-tile counters have to start
  // at zero; partial slots are fully written before they are read.
  err = cudaMemsetAsync(scratch, 0, size_t(pl.tiles) * sizeof(int), a.stream);
  if (err != cudaSuccess) return fail_cuda(err, "cudaMemsetAsync(counters)");
  return run_smallm(a, pl, scratch, int64_t(kNoAllocScratchBytes));
}

// ----------------------------------------------------------------------------------------
// Self-test of the bounded waits
// ----------------------------------------------------------------------------------------
namespace b12x_b200 {
namespace {

// One warp waits on an mbarrier that nothing will ever complete (no copy is in flight, nobody
// arrives), with a small poll limit, and reports the time-out exactly as the GEMM kernels do:
// status word raised, normal return.
__global__ void selftest_wait_timeout_kernel(int* status, uint32_t max_polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  bool completed = false;
  for (uint32_t polls = 0; polls < max_polls && !completed; ++polls) completed = mbar_try_wait(&bar, 0);
  if (!completed && status && threadIdx.x == 0) atomicMax(status, kStatusMmaTimeout);
}

}  // namespace
}  // namespace b12x_b200

extern "C" int b12x_b200_selftest_wait_timeout(int* status, int max_polls,
                                               b12x_b200_stream_t stream) {
  if (!status) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (max_polls < 1 || max_polls > 65536)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "max_polls must be in [1, 65536]");
  DeviceInfo info;
  const int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  selftest_wait_timeout_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      status, uint32_t(max_polls));
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "selftest launch");
  return B12X_B200_OK;
}

// ------------------------------------------------------------------------------------------
// All-reduce of row-parallel partial outputs over peer memory
// ------------------------------------------------------------------------------------------
namespace b12x_b200 {
namespace {

template <int G, bool BF16, bool SCATTERED>
cudaError_t launch_allreduce_peer(const PeerAllReduceParams& p, int blocks, bool rehearsal,
                                  cudaStream_t stream) {
  if (!rehearsal) {
    allreduce_peer_kernel<G, BF16, SCATTERED><<<blocks, 512, 0, stream>>>(p);
    return cudaGetLastError();
  }
  // All ranks in one grid: its blocks wait on each other, so they must all be resident.
  PeerAllReduceParams copy = p;
  void* args[] = {&copy};
  return cudaLaunchCooperativeKernel(
      reinterpret_cast<const void*>(&allreduce_peer_kernel<G, BF16, SCATTERED>),
      dim3(blocks, p.world), dim3(512), args, 0, stream);
}

template <bool BF16, bool SCATTERED>
cudaError_t launch_allreduce_peer_any(const PeerAllReduceParams& p, int blocks, bool rehearsal,
                                      cudaStream_t stream) {
  switch (p.world) {
    case 2: return launch_allreduce_peer<2, BF16, SCATTERED>(p, blocks, rehearsal, stream);
    case 4: return launch_allreduce_peer<4, BF16, SCATTERED>(p, blocks, rehearsal, stream);
    case 8: return launch_allreduce_peer<8, BF16, SCATTERED>(p, blocks, rehearsal, stream);
    default: return launch_allreduce_peer<0, BF16, SCATTERED>(p, blocks, rehearsal, stream);
  }
}

int allreduce_peer_impl(void* const* buffers, void* const* outputs, void* const* signals, int world,
                        int rank, int dtype, int64_t rows, int64_t cols, int64_t ld, int blocks,
                        int64_t max_polls, int* status, b12x_b200_stream_t stream) {
  if (!buffers || !signals) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (world < 1 || world > kMaxPeers)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "world must be in [1, 8]");
  if (rank >= world) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "rank outside the world");
  if (dtype != B12X_B200_BF16 && dtype != B12X_B200_FP16)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "all-reduce works on BF16 or FP16 partials");
  if (rows < 0 || cols < 0 || ld < cols || cols % 8 != 0 || ld % 8 != 0)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "cols and ld must be multiples of 8 with ld >= cols");
  if (outputs && rows % world != 0)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "scattered partials: rows must be a multiple of world");
  if (max_polls < 0 || max_polls > (int64_t(1) << 31) - 1)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "max_polls outside [0, 2^31)");
  for (int r = 0; r < world; ++r) {
    if (!buffers[r] || !signals[r] || (outputs && !outputs[r]))
      return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
    if ((reinterpret_cast<uintptr_t>(buffers[r]) & 15) || (reinterpret_cast<uintptr_t>(signals[r]) & 15) ||
        (outputs && (reinterpret_cast<uintptr_t>(outputs[r]) & 15)))
      return fail(B12X_B200_ERR_INVALID_ARGUMENT, "buffers and signal blocks must be 16-byte aligned");
  }
  DeviceInfo info;
  const int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  if (rows == 0 || cols == 0) return B12X_B200_OK;
  if (world == 1 && !outputs) return B12X_B200_OK;  // one rank: the partial is the sum
  const bool rehearsal = rank < 0;
  // One block of 512 threads per SM measured best on two GPUs (74: 72 us, 148: 70, 296: 71,
  // 592: 80 for a 58.7 MB matrix).
  if (blocks <= 0) blocks = rehearsal ? std::max(1, info.sm_count / (2 * world)) : info.sm_count;
  if (rehearsal && int64_t(blocks) * world > int64_t(info.sm_count))
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "rehearsal grid would not be resident at once");
  PeerAllReduceParams p{};
  for (int r = 0; r < world; ++r) {
    p.buf[r] = buffers[r];
    p.out[r] = outputs ? outputs[r] : nullptr;
    p.sig[r] = static_cast<uint32_t*>(signals[r]);
  }
  p.world = world;
  p.rank = rank;
  p.rows = rows;
  p.cols = cols;
  p.ld = ld;
  p.out_dtype = dtype == B12X_B200_BF16 ? kOutBf16 : kOutFp16;
  // Default: 2^24 polls of a system-scope load plus a 200 ns back-off, tens of seconds. Ranks
  // of a serving process can be a second apart at the first call (host-side set-up).
  p.max_polls = max_polls ? uint32_t(max_polls) : (1u << 24);
  p.status = status;
  const cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = dtype == B12X_B200_BF16;
  cudaError_t err;
  if (outputs)
    err = bf ? launch_allreduce_peer_any<true, true>(p, blocks, rehearsal, s)
             : launch_allreduce_peer_any<false, true>(p, blocks, rehearsal, s);
  else
    err = bf ? launch_allreduce_peer_any<true, false>(p, blocks, rehearsal, s)
             : launch_allreduce_peer_any<false, false>(p, blocks, rehearsal, s);
  if (err != cudaSuccess) return fail_cuda(err, "all-reduce launch");
  return B12X_B200_OK;
}

}  // namespace
}  // namespace b12x_b200

extern "C" int64_t b12x_b200_allreduce_peer_signal_bytes(void) {
  return int64_t(b12x_b200::kSigWords) * 4;
}

extern "C" int b12x_b200_allreduce_peer(void* const* buffers, void* const* signals, int world,
                                        int rank, int dtype, int64_t rows, int64_t cols,
                                        int64_t ld, int blocks, int64_t max_polls, int* status,
                                        b12x_b200_stream_t stream) {
  return allreduce_peer_impl(buffers, nullptr, signals, world, rank, dtype, rows, cols, ld, blocks,
                             max_polls, status, stream);
}

extern "C" int b12x_b200_allreduce_peer_scattered(void* const* buffers, void* const* outputs,
                                                  void* const* signals, int world, int rank,
                                                  int dtype, int64_t rows, int64_t cols,
                                                  int64_t ld, int blocks, int64_t max_polls,
                                                  int* status, b12x_b200_stream_t stream) {
  if (!outputs) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  return allreduce_peer_impl(buffers, outputs, signals, world, rank, dtype, rows, cols, ld, blocks,
                             max_polls, status, stream);
}

extern "C" int b12x_b200_gemm_blockscaled_scatter(int kind, const void* a, const void* sfa,
                                                  const void* b, const void* sfb,
                                                  void* const* destinations, int world, int rank,
                                                  int c_dtype, const float* alpha, int64_t m,
                                                  int64_t n, int64_t k, int64_t ld, int sm_count,
                                                  void* workspace, int64_t workspace_bytes,
                                                  int* status, b12x_b200_stream_t stream) {
  ScatterPlan plan;
  plan.dst = destinations;
  plan.world = world;
  plan.rank = rank;
  return gemm_blockscaled_impl(kind, a, sfa, b, sfb, nullptr, c_dtype, alpha, m, n, k, ld, 1,
                               B12X_B200_BLOCK_N_PAIR, sm_count, workspace, workspace_bytes,
                               nullptr, status, stream, &plan);
}

// ------------------------------------------------------------------------------------------
// Load-time weight packing
// ------------------------------------------------------------------------------------------
extern "C" int b12x_b200_pack_block_fp8_weight_mxfp8(const void* codes, const float* scale,
                                                     void* out_codes, void* scale_rows,
                                                     void* scale_mma, int64_t m, int64_t k,
                                                     int64_t groups, int requantize,
                                                     b12x_b200_stream_t stream) {
  if (m <= 0 || k <= 0 || groups <= 0 || m > INT32_MAX - 128 || k > INT32_MAX || groups > 65535)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad size");
  if (k % 128 != 0) return fail(B12X_B200_ERR_UNSUPPORTED, "K must be a multiple of 128");
  if (!codes || !scale || !out_codes) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (!aligned16(codes) || !aligned16(out_codes) || (scale_rows && (uintptr_t(scale_rows) & 3)) ||
      (scale_mma && !aligned16(scale_mma)))
    return fail(B12X_B200_ERR_ALIGNMENT, "codes and atoms must be 16-byte aligned");
  const int64_t row_tiles = (m + 127) / 128;
  if (row_tiles > 65535) return fail(B12X_B200_ERR_UNSUPPORTED, "too many rows");
  DeviceInfo info;
  const int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  PackWeightParams p;
  p.codes = static_cast<const uint8_t*>(codes);
  p.scale = scale;
  p.out_codes = static_cast<uint8_t*>(out_codes);
  p.scale_rows = static_cast<uint8_t*>(scale_rows);
  p.scale_mma = static_cast<uint8_t*>(scale_mma);
  p.m = int(m);
  p.k = int(k);
  p.requantize = requantize ? 1 : 0;
  pack_block_fp8_weight_kernel<<<dim3(unsigned(k / 128), unsigned(row_tiles), unsigned(groups)), 256, 0,
                                 reinterpret_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "pack_block_fp8_weight launch");
  return B12X_B200_OK;
}

// ------------------------------------------------------------------------------------------
// Batched BF16 x rowwise-MXFP8 product (the MLA absorb projections)
// ------------------------------------------------------------------------------------------
namespace {

template <int MAJOR, int MT>
int launch_bmm(const BmmParams& p, int batch, cudaStream_t stream) {
  using S = BmmShape<MAJOR, MT>;
  if (S::kSmemBytes > 48 * 1024) {
    static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !set_for[dev]) {
      const cudaError_t attr_err =
          cudaFuncSetAttribute(bmm_mxfp8_kernel<MAJOR, MT>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
      if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
      set_for[dev] = true;
    }
  }
  const dim3 grid(unsigned((p.n + S::kTileN - 1) / S::kTileN), unsigned(batch), 1);
  bmm_mxfp8_kernel<MAJOR, MT><<<grid, kBmmThreads, S::kSmemBytes, stream>>>(p);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "bmm_mxfp8 launch");
  return B12X_B200_OK;
}

constexpr int kBmmMmaSmemLimit = 200 * 1024;

template <int MAJOR, int MT>
int launch_bmm_mma(const BmmParams& p, int batch, cudaStream_t stream) {
  using S = BmmMmaShape<MAJOR, MT>;
  static std::atomic<bool> set_for[64];  // zero-initialised; setting the attribute twice is harmless
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !set_for[dev]) {
    const cudaError_t attr_err =
        cudaFuncSetAttribute(bmm_mxfp8_mma_kernel<MAJOR, MT>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kBmmMmaSmemLimit);
    if (attr_err != cudaSuccess) return fail_cuda(attr_err, "cudaFuncSetAttribute");
    set_for[dev] = true;
  }
  const dim3 grid(unsigned((p.n + S::kTileN - 1) / S::kTileN), unsigned(batch), 1);
  bmm_mxfp8_mma_kernel<MAJOR, MT><<<grid, kBmmThreads, S::smem_bytes(p.k), stream>>>(p);
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(err, "bmm_mxfp8 launch");
  return B12X_B200_OK;
}

template <int MAJOR>
int dispatch_bmm_rows(const BmmParams& p, int batch, cudaStream_t stream) {
  // Both blocks of a CTA in shared memory: the tensor-core kernel. Longer K: the CUDA-core one.
  if (switches().bmm_tensor_core && BmmMmaShape<MAJOR, 32>::smem_bytes(p.k) <= kBmmMmaSmemLimit) {
    if (p.m <= 16) return launch_bmm_mma<MAJOR, 16>(p, batch, stream);
    return launch_bmm_mma<MAJOR, 32>(p, batch, stream);
  }
  if (p.m <= 8) return launch_bmm<MAJOR, 8>(p, batch, stream);
  if (p.m <= 16) return launch_bmm<MAJOR, 16>(p, batch, stream);
  return launch_bmm<MAJOR, 32>(p, batch, stream);
}

}  // namespace

extern "C" int b12x_b200_bmm_mxfp8(const void* a, int64_t a_stride_b, int64_t a_stride_m,
                                   const void* w_values, int64_t w_stride_b, int64_t w_stride_r,
                                   const void* w_scales, int64_t sf_stride_b, int64_t sf_stride_r,
                                   void* c, int64_t c_stride_b, int64_t c_stride_m, int n_major,
                                   int64_t batch, int64_t m, int64_t n, int64_t k,
                                   b12x_b200_stream_t stream) {
  if (batch <= 0 || batch > 65535 || m <= 0 || n <= 0 || k <= 0 || n > INT32_MAX - 64 ||
      k > INT32_MAX)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "bad size");
  if (m > 32) return fail(B12X_B200_ERR_UNSUPPORTED, "the batched product takes at most 32 rows");
  if (!a || !w_values || !w_scales || !c) return fail(B12X_B200_ERR_INVALID_ARGUMENT, "null pointer");
  if (n_major) {
    if (n % 32 != 0 || k % 8 != 0)
      return fail(B12X_B200_ERR_UNSUPPORTED, "N-major weights need N % 32 == 0 and K % 8 == 0");
  } else if (k % 32 != 0) {
    return fail(B12X_B200_ERR_UNSUPPORTED, "K-major weights need K % 32 == 0");
  }
  if (!aligned16(a) || a_stride_b % 8 != 0 || a_stride_m % 8 != 0)
    return fail(B12X_B200_ERR_ALIGNMENT, "A rows must start on 16-byte boundaries");
  if (!aligned16(w_values) || w_stride_b % 16 != 0 || w_stride_r % 16 != 0)
    return fail(B12X_B200_ERR_ALIGNMENT, "weight rows must start on 16-byte boundaries");
  if ((uintptr_t(c) & 3) || c_stride_b % 2 != 0 || c_stride_m % 2 != 0)
    return fail(B12X_B200_ERR_ALIGNMENT, "C rows must start on 4-byte boundaries");
  if (a_stride_b < 0 || a_stride_m < 0 || w_stride_b < 0 || w_stride_r < 0 || sf_stride_b < 0 ||
      sf_stride_r < 0 || c_stride_b < 0 || c_stride_m < 0)
    return fail(B12X_B200_ERR_INVALID_ARGUMENT, "negative stride");
  DeviceInfo info;
  const int rc = device_info(&info);
  if (rc != B12X_B200_OK) return rc;
  if (info.cc_major != 10) return fail(B12X_B200_ERR_NO_DEVICE_CODE, "device is not sm_100");
  BmmParams p;
  p.a = static_cast<const __nv_bfloat16*>(a);
  p.a_stride_b = a_stride_b;
  p.a_stride_m = a_stride_m;
  p.w = static_cast<const uint8_t*>(w_values);
  p.w_stride_b = w_stride_b;
  p.w_stride_r = w_stride_r;
  p.sf = static_cast<const uint8_t*>(w_scales);
  p.sf_stride_b = sf_stride_b;
  p.sf_stride_r = sf_stride_r;
  p.c = static_cast<__nv_bfloat16*>(c);
  p.c_stride_b = c_stride_b;
  p.c_stride_m = c_stride_m;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return n_major ? dispatch_bmm_rows<1>(p, int(batch), s) : dispatch_bmm_rows<0>(p, int(batch), s);
}
