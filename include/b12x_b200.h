/*
 * C ABI of the B200 (sm_100a) implementation of the b12x block-scaled GEMM hot path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches on that
 * stream, returns 0 on success or a negative B12X_B200_ERR_* code, and never allocates,
 * synchronises or throws. Pointers must be device pointers the caller has validated; the
 * functions re-check only what a wrong value would turn into a device fault (alignment,
 * divisibility, null). Tensors are row-major and dense unless a leading dimension is given.
 *
 * Scale-factor ("MMA") layout used by all entry points: 512-byte atoms that cover 128 rows x
 * 4 scale columns, atom order [row_tile][col_tile] with col_tile = ceil(scale_cols / 4) atoms
 * per row tile, byte in atom = (r % 32) * 16 + ((r / 32) % 4) * 4 + (c % 4). This is the
 * layout the reference stores (b12x/_lib/utils.py:384-407, b12x/_lib/intrinsics.py:62-93).
 *
 * Citations name the reference interface each function stands in for, as
 * path:line inside the b12x source tree.
 */
#ifndef B12X_B200_H_
#define B12X_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b12x_b200_stream_t;

enum {
  B12X_B200_OK = 0,
  B12X_B200_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad enum, bad size               */
  B12X_B200_ERR_ALIGNMENT = -2,        /* pointer / leading dimension not 16-byte aligned */
  B12X_B200_ERR_UNSUPPORTED = -3,      /* shape or option outside what the kernels cover  */
  B12X_B200_ERR_CUDA = -4,             /* a CUDA runtime / driver call failed             */
  B12X_B200_ERR_NO_DEVICE_CODE = -5    /* the device is not compute capability 10.x       */
};

/* Operand recipes. */
enum {
  B12X_B200_KIND_MXFP8 = 0, /* E4M3 codes, UE8M0 scale per 32 elements of K              */
  B12X_B200_KIND_NVFP4 = 1, /* packed E2M1 codes, UE4M3 (E4M3) scale per 16 elements     */
  /* E4M3 codes without block scales: alpha is the only scale (the reference's
   * dense_gemm(plain_fp8=True), b12x/_lib/dense_gemm.py:7096-7139, 7225-7233; MMA :268-330, per-tensor FP8 linears).
   * sfa / sfb are ignored and may be NULL. Accepted by b12x_b200_gemm_blockscaled, _ex,
   * _grouped and _scatter (tiled and CTA-pair kernels); the decode entry points refuse it. */
  B12X_B200_KIND_FP8 = 2,
  /* MXFP4: packed E2M1 codes (as NVFP4) with one UE8M0 scale per 32 elements of K, scale atoms
   * of 128 rows x 4 scale columns = 128 elements of K (the reference's float4_e2m1fn operands
   * with sf_dtype float8_e8m0fnu / sf_vec_size 32, b12x/_lib/dense_gemm.py:7225-7260). Every
   * GEMM entry point takes it except the two with fused activation quantization (no quantizer
   * produces MXFP4). */
  B12X_B200_KIND_MXFP4 = 3
};

/* Element types of dense tensors. */
enum {
  B12X_B200_BF16 = 0,
  B12X_B200_FP16 = 1,
  B12X_B200_FP32 = 2
};

/*
 * Value of `block_n` that sends b12x_b200_gemm_blockscaled to the CTA-pair kernel (two SMs per
 * 256 x 256 tile) whatever the problem size; 0 lets the library choose between the kernels.
 */
#define B12X_B200_BLOCK_N_PAIR (-256)

/*
 * Optional epilogue of the *_ex entry points (a NULL pointer, or all-zero contents, means none).
 * Stands in for the reference's bias add after its linears
 * (b12x/gemm/mxfp8_linear/_kernel.py:264-265) and for its quantized-C GEMM output
 * (dense_gemm(..., _quantized_c=...), b12x/_lib/dense_gemm.py:7497-7588, kernel :2854-3090).
 *
 *   bias   [N] values of the output dtype. Added the way a separate bias add on the stored
 *          output would: out = cvt(float(cvt(alpha * acc)) + float(bias[n])) for BF16 / FP16
 *          outputs, a plain FP32 add for FP32 outputs.
 *   quant_values  decode-shape entry points only, BF16 / FP16 output, N % 32 == 0: besides C,
 *          the rounded output rows are re-quantized to MXFP8 along N exactly as
 *          b12x_b200_quantize_mxfp8_rows would quantize C: E4M3 codes into
 *          quant_values[M, quant_ld] at columns quant_col0 .. quant_col0 + N - 1.
 *   quant_scale_rows  UE8M0 bytes, row-major [M, quant_cols / 32], or NULL.
 *   quant_scale_mma   the same bytes in scale atoms of an [M, quant_cols] operand (row tile 0..,
 *          ceil(quant_cols / 128) atoms per row tile), or NULL. Bytes of rows >= M are not
 *          written (pre-fill with 127).
 *   quant_ld, quant_col0, quant_cols  pitch of quant_values in bytes, first column and total
 *          width of the quantized matrix this GEMM writes into (several GEMMs may fill one
 *          matrix side by side, as the reference's grouped WO-A projection does).
 */
typedef struct b12x_b200_epilogue {
  const void* bias;
  void* quant_values;
  void* quant_scale_rows;
  void* quant_scale_mma;
  int64_t quant_ld;
  int64_t quant_col0;
  int64_t quant_cols;
} b12x_b200_epilogue_t;

/* Library identification: "b12x_b200 <version> sm_100a". */
const char* b12x_b200_version(void);

/* Last CUDA error text seen by this library on the calling thread ("" if none). */
const char* b12x_b200_last_error(void);

/*
 * Block-scaled GEMM  C[M,N] = cvt(alpha * (A . SFA) (B . SFB)^T).
 * Replaces dense_gemm / b12x::dense_gemm_launch for the NVFP4 and MXFP8 recipes with L = 1
 * (b12x/_lib/dense_gemm.py:7068-7098, 6335-6373; device kernel :1459-4157).
 *
 *   a      [M, K] codes (K bytes per row for MXFP8, K/2 bytes for NVFP4), K-major
 *   b      [N, K] codes, same packing
 *   sfa    scale atoms of A: ceil(M/128) x ceil(K / (4*vec)) atoms, vec = 32 / 16
 *   sfb    scale atoms of B: ceil(N/128) x the same
 *   c      [M, ldc] output of c_dtype
 *   alpha  device FP32 scalar read by the kernel at run time, or NULL for 1
 *   block_n 0 = choose, else one of 64, 128, 192, 256 (single-CTA tile width) or
 *          B12X_B200_BLOCK_N_PAIR
 *   sm_count 0 = all SMs of the current device
 *   status device int32 the kernel raises to a non-zero KernelStatus when a bounded wait
 *          ran out; may be NULL
 */
int b12x_b200_gemm_blockscaled(int kind, const void* a, const void* sfa, const void* b,
                               const void* sfb, void* c, int c_dtype, const float* alpha,
                               int64_t m, int64_t n, int64_t k, int64_t ldc, int block_n,
                               int sm_count, int* status, b12x_b200_stream_t stream);

/*
 * b12x_b200_gemm_blockscaled with caller-owned scratch and an optional epilogue (bias only;
 * see b12x_b200_epilogue_t). The CTA-pair kernel (chosen for large
 * problems, or with B12X_B200_BLOCK_N_PAIR) runs whole rounds of 256 x 256 tiles over the SM
 * pairs; when the tiles left over would occupy at most half of the pairs, it cuts them along K
 * over the pairs instead (as the first thing the pairs do) and adds the FP32 partial tiles up through this scratch
 * (in a fixed order: results do not depend on timing). Without scratch, or where no split
 * applies, the call is exactly b12x_b200_gemm_blockscaled. Plays the role of the reference's
 * split-K / stream-K policy (b12x/_lib/dense_gemm.py:387-454, 6671-6894) for large M.
 *
 *   workspace  NULL, or at least b12x_b200_gemm_blockscaled_workspace_bytes(...) bytes (0 means
 *              the shape needs none), 16-byte aligned. Same buffer and same rules as the decode
 *              GEMM's workspace: its first 64 KiB must be zero before the first launch that
 *              uses it, every launch leaves them zero, and launches that share it must not
 *              overlap on the device.
 */
int64_t b12x_b200_gemm_blockscaled_workspace_bytes(int kind, int64_t m, int64_t n, int64_t k,
                                                   int block_n, int sm_count);
int b12x_b200_gemm_blockscaled_ex(int kind, const void* a, const void* sfa, const void* b,
                                  const void* sfb, void* c, int c_dtype, const float* alpha,
                                  int64_t m, int64_t n, int64_t k, int64_t ldc, int block_n,
                                  int sm_count, void* workspace, int64_t workspace_bytes,
                                  const b12x_b200_epilogue_t* epilogue, int* status,
                                  b12x_b200_stream_t stream);

/*
 * Grouped (batched) block-scaled GEMM: `groups` independent problems of one shape in ONE launch,
 * C[g] = cvt(alpha * (A[g] . SFA[g]) (B[g] . SFB[g])^T). This is the reference's L > 1 form of
 * dense_gemm (operands [M, Kp, L] over physical [L, M, Kp], output [M, N, L] over physical
 * [L, M, N]; b12x/_lib/dense_gemm.py:7068-7098, 6469-6491), which its grouped projections use
 * (:5803-5944). The tiles (decode kernel: the weight tiles and k-tiles) of all groups form one
 * work list for the persistent scheduler, so small groups fill the machine together.
 *
 *   a, b      stacked K-major codes, group after group: [groups, M, Kbytes], [groups, N, Kbytes]
 *   sfa, sfb  each group's dense scale atoms, group after group
 *   c         [groups, M, ldc]; alpha, bias: shared by all groups
 *   epilogue  bias in both entry points; output re-quantization in the decode-shape one, where
 *             group g fills columns quant_col0 + g * N .. of the quantized matrix
 *   workspace at least b12x_b200_gemm_grouped_workspace_bytes(kind, decode, ...) bytes (decode =
 *             1 for the _smallm_grouped entry point), same rules as for the ungrouped calls
 * groups = 1 is exactly the ungrouped call.
 */
int64_t b12x_b200_gemm_grouped_workspace_bytes(int kind, int decode, int64_t m, int64_t n,
                                               int64_t k, int64_t groups, int block_n,
                                               int sm_count);
int b12x_b200_gemm_blockscaled_grouped(int kind, const void* a, const void* sfa, const void* b,
                                       const void* sfb, void* c, int c_dtype, const float* alpha,
                                       int64_t m, int64_t n, int64_t k, int64_t ldc,
                                       int64_t groups, int block_n, int sm_count, void* workspace,
                                       int64_t workspace_bytes,
                                       const b12x_b200_epilogue_t* epilogue, int* status,
                                       b12x_b200_stream_t stream);
int b12x_b200_gemm_blockscaled_smallm_grouped(int kind, const void* x, const void* sf_x,
                                              const void* w, const void* sf_w, void* c,
                                              int c_dtype, const float* alpha, int64_t m,
                                              int64_t n, int64_t k, int64_t ldc, int64_t groups,
                                              void* workspace, int64_t workspace_bytes,
                                              const b12x_b200_epilogue_t* epilogue, int sm_count,
                                              int* status, b12x_b200_stream_t stream);

/*
 * Decode-shape (1 <= M <= 128) variant of b12x_b200_gemm_blockscaled: the weight matrix is
 * streamed once, split evenly over all SMs along N and K (stream-K), and partial sums meet in
 * a caller-owned FP32 workspace. Stands in for the reference's small-M split-K policy and its
 * partial-sum reduction (b12x/_lib/dense_gemm.py:412-426, 174-206, 2685-2800), which the
 * reference has for FP8 operands only.
 *
 *   x, sf_x    activations [M, K] codes and their scale atoms (1 row tile)
 *   w, sf_w    weights [N, K] codes and their scale atoms
 *   workspace  at least b12x_b200_gemm_smallm_workspace_bytes(...) bytes, 16-byte aligned.
 *              Its first 64 KiB hold per-tile counters that must be zero before the first
 *              launch that uses the buffer (zero the buffer once); each launch leaves them
 *              zero, so one buffer serves any sequence of shapes. Launches on different
 *              streams that share a workspace must not overlap on the device.
 *
 * Ordering on one stream. The kernel is launched with programmatic stream serialization: it
 * may start while the kernel launched just before it on the same stream is still running, if
 * that kernel releases its dependents early. In this library the decode GEMMs do, and the row
 * quantizers do for matrices of at most 128 rows. The decode GEMM reads x, sf_x and alpha and
 * writes c and the workspace only after its predecessor has completed. A weight of more than
 * 128 rows is streamed at once (no kernel of this library that releases early can have written
 * it); a weight of 128 rows or fewer is streamed after the predecessor has completed, like the
 * other operands. A foreign kernel that releases its dependents early (griddepcontrol /
 * cudaTriggerProgrammaticLaunchCompletion) must not be the writer of w or sf_w.
 */
int64_t b12x_b200_gemm_smallm_workspace_bytes(int kind, int64_t m, int64_t n, int64_t k,
                                              int sm_count);
int b12x_b200_gemm_blockscaled_smallm(int kind, const void* x, const void* sf_x, const void* w,
                                      const void* sf_w, void* c, int c_dtype, const float* alpha,
                                      int64_t m, int64_t n, int64_t k, int64_t ldc,
                                      void* workspace, int64_t workspace_bytes, int sm_count,
                                      int* status, b12x_b200_stream_t stream);
/* The same with an epilogue (bias and / or MXFP8 re-quantization of the output rows). */
int b12x_b200_gemm_blockscaled_smallm_ex(int kind, const void* x, const void* sf_x,
                                         const void* w, const void* sf_w, void* c, int c_dtype,
                                         const float* alpha, int64_t m, int64_t n, int64_t k,
                                         int64_t ldc, void* workspace, int64_t workspace_bytes,
                                         const b12x_b200_epilogue_t* epilogue, int sm_count,
                                         int* status, b12x_b200_stream_t stream);

/*
 * Decode-shape GEMM with the activation quantizer fused in (1 <= M <= 16): the BF16 rows are
 * quantized inside the GEMM kernel by dedicated warps, with the arithmetic of
 * b12x_b200_quantize_mxfp8_rows / b12x_b200_quantize_nvfp4_rows, so the result equals, bit for
 * bit, quantizing the rows and calling b12x_b200_gemm_blockscaled_smallm. Replaces
 * dense_gemm_fused_quant_a (b12x/_lib/dense_gemm.py:6897-7051; producer-warp quantizer
 * :3443-3726), which the reference has for MXFP8 and M <= 8; the NVFP4 recipe is an addition.
 *
 *   x_bf16          [M, ld_x] BF16 rows, 16-byte aligned, ld_x % 8 == 0
 *   x_global_scale  NVFP4: device FP32 scalar (448 * 6 / amax), read at run time; MXFP8: NULL
 *   workspace       as for b12x_b200_gemm_blockscaled_smallm (same size query)
 *   epilogue        optional, as for b12x_b200_gemm_blockscaled_smallm_ex
 * Other arguments and stream ordering as for b12x_b200_gemm_blockscaled_smallm.
 */
int b12x_b200_gemm_smallm_fused_quant(int kind, const void* x_bf16, int64_t ld_x,
                                      const float* x_global_scale, const void* w,
                                      const void* sf_w, void* c, int c_dtype, const float* alpha,
                                      int64_t m, int64_t n, int64_t k, int64_t ldc,
                                      void* workspace, int64_t workspace_bytes,
                                      const b12x_b200_epilogue_t* epilogue, int sm_count,
                                      int* status, b12x_b200_stream_t stream);

/*
 * The same for `groups` problems of one shape in one launch: the reference's
 * dense_gemm_fused_quant_a_grouped without its inverse-RoPE option (next entry point)
 * (b12x/_lib/dense_gemm.py:5803-5944; WO-A of the MLA output projection). Row r of group g of
 * the activation starts at x + r * ld_x + g * x_group_stride elements (the reference's source
 * [M, groups, K] has ld_x = groups * K and x_group_stride = K); weights, their scale atoms and
 * the output are group-major as in b12x_b200_gemm_blockscaled_grouped.
 */
int b12x_b200_gemm_smallm_fused_quant_grouped(
    int kind, const void* x_bf16, int64_t ld_x, int64_t x_group_stride,
    const float* x_global_scale, const void* w, const void* sf_w, void* c, int c_dtype,
    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t groups,
    void* workspace, int64_t workspace_bytes, const b12x_b200_epilogue_t* epilogue, int sm_count,
    int* status, b12x_b200_stream_t stream);

/*
 * The grouped call with the reference's inverse-RoPE option (MXFP8 only,
 * b12x/_lib/dense_gemm.py:5849-5882 host contract, :3505-3530 device arithmetic): before a
 * 32-element block of an activation row is quantized, the trailing rope_dim elements of every
 * head_dim-wide slice of the group's K are rotated back in FP32. Row r is the token at
 * positions[r] (int32, or int64 when positions_are_int64); for the interleaved pair (even, odd)
 * number j of the rotary part, with cos = cache[pos * rope_dim + j] and
 * sin = cache[pos * rope_dim + rope_dim / 2 + j] (BF16, or FP32 when cache_is_fp32):
 *   even' = fma(even, cos, odd * sin),   odd' = fma(odd, cos, -(even * sin)).
 * head_dim = nope_dim + rope_dim, all multiples of 32, head_dim dividing K. positions and the
 * cache are read on the device at run time (no bounds check on positions, as in the reference).
 * No epilogue. Everything else as b12x_b200_gemm_smallm_fused_quant_grouped with kind MXFP8.
 */
int b12x_b200_gemm_smallm_fused_quant_grouped_inv_rope(
    const void* x_bf16, int64_t ld_x, int64_t x_group_stride, const void* positions,
    int positions_are_int64, const void* cos_sin_cache, int cache_is_fp32, int head_dim,
    int nope_dim, int rope_dim, const void* w, const void* sf_w, void* c, int c_dtype,
    const float* alpha, int64_t m, int64_t n, int64_t k, int64_t ldc, int64_t groups,
    void* workspace, int64_t workspace_bytes, int sm_count, int* status,
    b12x_b200_stream_t stream);

/*
 * b12x_b200_gemm_blockscaled_smallm that also records, per CTA, eight 64-bit values in
 * `stamps` (global-timer nanoseconds at entry, after set-up, after the dependency wait, at the
 * first full pipeline stage, at the last finished accumulator and at the end of the epilogue,
 * then the SM id and the time at which the last accumulator had been read out of tensor
 * memory). For the timeline summaries of the decode GEMM; it has no
 * counterpart in the reference. stamps_len (in 64-bit words) must be at least 8 x the grid
 * size, for which 8 x the SM count always suffices.
 */
int b12x_b200_gemm_smallm_timeline(int kind, const void* x, const void* sf_x, const void* w,
                                   const void* sf_w, void* c, int c_dtype, const float* alpha,
                                   int64_t m, int64_t n, int64_t k, int64_t ldc, void* workspace,
                                   int64_t workspace_bytes, int sm_count,
                                   unsigned long long* stamps, int64_t stamps_len, int* status,
                                   b12x_b200_stream_t stream);

/*
 * b12x_b200_gemm_blockscaled_smallm for callers that cannot allocate device memory. It has no
 * counterpart in the reference.
 *
 * Some callers of a decode GEMM are not in a position to call cudaMalloc (or a framework
 * allocator) for the workspace above: a serving process that gave all device memory to its own
 * pool at start-up and runs with a fixed allowance, a plugin called from a thread that is in the
 * middle of a CUDA stream capture (where an allocation fails or invalidates the capture), a
 * small C host that links this library and nothing else. For them this entry point keeps the
 * workspace inside the library: a fixed 4 MiB + 64 KiB array in device memory, present on every
 * GPU that loads the library until the process exits. The function allocates nothing and calls
 * no allocating routine; inputs and outputs are still the caller's.
 *
 *   - Shapes whose workspace need (b12x_b200_gemm_smallm_workspace_bytes) exceeds
 *     b12x_b200_gemm_smallm_noalloc_capacity_bytes() are refused with
 *     B12X_B200_ERR_UNSUPPORTED and a message naming both sizes. M <= 16 with N <= 16384 always
 *     fits; larger M fits for smaller N.
 *   - The first call on each device looks up the device address of the built-in array (with
 *     that device current). Make that first call outside any stream capture, e.g. as the
 *     warm-up call.
 *   - All calls on a device share the one array, and it keeps the previous call's contents:
 *     every call first clears the per-tile counters on the given stream. Two calls that can
 *     run on the GPU at the same time (different streams without ordering) race on it; keep
 *     them on one stream or order them with events.
 *
 * Arguments as for b12x_b200_gemm_blockscaled_smallm, minus the workspace.
 */
int64_t b12x_b200_gemm_smallm_noalloc_capacity_bytes(void);
int b12x_b200_gemm_blockscaled_smallm_noalloc(int kind, const void* x, const void* sf_x,
                                              const void* w, const void* sf_w, void* c,
                                              int c_dtype, const float* alpha, int64_t m,
                                              int64_t n, int64_t k, int64_t ldc, int sm_count,
                                              int* status, b12x_b200_stream_t stream);

/*
 * Block-FP8 GEMM with compact FP32 scales,
 *   C[M,N] = cvt(alpha * sum_kb (A[:,kb] B[:,kb]^T) * sfa[m,kb] * sfb[n/128,kb]).
 * Replaces dense_gemm(..., block_fp8=True, sf_dtype="float32", sf_vec_size=128)
 * (b12x/_lib/dense_gemm.py:7137-7139, 7190-7224, kernel :1314-1348, 2290-2348).
 *
 *   a   [M, K] E4M3, K-major      sfa [M, K/128] FP32, contiguous
 *   b   [N, K] E4M3, K-major      sfb [N/128, K/128] FP32, contiguous
 *   N and K must be multiples of 128. Other arguments as for b12x_b200_gemm_blockscaled.
 */
int b12x_b200_gemm_block_fp8(const void* a, const float* sfa, const void* b, const float* sfb,
                             void* c, int c_dtype, const float* alpha, int64_t m, int64_t n,
                             int64_t k, int64_t ldc, int sm_count, int* status,
                             b12x_b200_stream_t stream);
/* The same with an epilogue (bias only; see b12x_b200_epilogue_t). */
int b12x_b200_gemm_block_fp8_ex(const void* a, const float* sfa, const void* b, const float* sfb,
                                void* c, int c_dtype, const float* alpha, int64_t m, int64_t n,
                                int64_t k, int64_t ldc, int sm_count,
                                const b12x_b200_epilogue_t* epilogue, int* status,
                                b12x_b200_stream_t stream);

/*
 * MXFP8 row quantizer. Replaces quantize_mxfp8_rows_cute
 * (b12x/_lib/quant/mxfp8_rows.py:398-434; kernel :88-269), numerics of
 * quantize_mxfp8_rows_torch (b12x/gemm/_shared/wo_mxfp8.py:1884-1918).
 *
 *   src        [M, ld_src] BF16 or FP16, K % 32 == 0
 *   values     [M, K] E4M3 bytes
 *   scale_rows [M, K/32] UE8M0 bytes, may be NULL
 *   scale_mma  atoms for ceil(M/128) x ceil(K/128); may be NULL. Bytes of rows >= M and of
 *              scale columns >= K/32 inside those atoms are set to 127.
 */
int b12x_b200_quantize_mxfp8_rows(const void* src, int src_dtype, int64_t ld_src, void* values,
                                  void* scale_rows, void* scale_mma, int64_t m, int64_t k,
                                  b12x_b200_stream_t stream);

/*
 * NVFP4 row quantizer. Replaces Bf16ToFp4TmaKernel / compile_bf16_to_fp4_tma(...).launch
 * (b12x/quantization/nvfp4/_kernel.py:250-518, _impl.py:117-224), numerics of
 * quantize_grouped_nvfp4_torch (b12x/_lib/intrinsics.py:149-193). Unlike the reference
 * kernel M need not be a multiple of 128.
 *
 *   src          [M, ld_src] BF16 or FP16, K % 16 == 0 and K % 32 == 0 for packed rows
 *   global_scale device FP32 scalar (448 * 6 / amax of the tensor), read at run time
 *   packed       [M, K/2] bytes, low nibble = even k
 *   scale_mma    atoms for ceil(M/128) x ceil(K/64); bytes of rows >= M and of scale
 *                columns >= K/16 inside those atoms are set to 0.
 */
int b12x_b200_quantize_nvfp4_rows(const void* src, int src_dtype, int64_t ld_src,
                                  const float* global_scale, void* packed, void* scale_mma,
                                  int64_t m, int64_t k, b12x_b200_stream_t stream);

/*
 * Self-test of the bounded waits every kernel of this library uses: launches one warp that
 * waits, for at most max_polls polls (1..65536), on a barrier nothing will ever complete, and
 * then reports exactly as a GEMM kernel does when a wait runs out: *status is raised to 2 and
 * the kernel returns normally. Lets a host verify its handling of the status word without any
 * fault. It has no counterpart in the reference.
 */
int b12x_b200_selftest_wait_timeout(int* status, int max_polls, b12x_b200_stream_t stream);

/*
 * Sum of the per-rank partial outputs of a row-parallel (K-split) linear over peer memory: the
 * all-reduce that follows the GEMM when the serving stack shards K across the GPUs of a node.
 * The reference's GEMM is single-GPU and leaves this step to the caller's torch.distributed
 * all_reduce; it has no counterpart there. Every rank calls this with the same shapes, one
 * kernel per rank and call: rank s pulls the rows of slab s (rows * s / world up to
 * rows * (s + 1) / world) of every rank's partial, adds them in FP32 in rank order, rounds once
 * and pushes the result into all ranks' buffers, in place. When the call's kernel has finished
 * on a rank's stream, that rank's buffer holds the complete sum, identical on every rank.
 *
 *   buffers  host array of `world` device pointers: rank r's [rows, ld] partial as mapped in
 *            THIS process (own allocation for r == rank, peer mappings otherwise), 16-byte aligned
 *   signals  host array of `world` device pointers to each rank's signal block
 *            (b12x_b200_allreduce_peer_signal_bytes() bytes, zeroed once before the first call
 *            and before any peer can call), mapped the same way
 *   rank     this process's rank in [0, world). rank < 0 runs ALL ranks in one cooperative grid
 *            on the current device (every pointer local): a single-GPU rehearsal for tests;
 *            blocks * world must then be resident at once (<= SMs)
 *   dtype    B12X_B200_BF16 or B12X_B200_FP16; cols % 8 == 0, ld % 8 == 0
 *   blocks   thread blocks of 512 threads per rank, 0 = library default
 *   max_polls  limit of each wait for another rank's flag (one poll is a system-scope load plus
 *            a 200 ns back-off), 0 = 2^24 (tens of seconds). When a wait runs out *status is
 *            raised to 6, the data phase is skipped and the kernel returns.
 * Waits on other GPUs' kernels: the ranks must be on different devices (rank >= 0), launched
 * by their own processes or threads; never launch two ranks' calls on one device.
 */
int64_t b12x_b200_allreduce_peer_signal_bytes(void);
int b12x_b200_allreduce_peer(void* const* buffers, void* const* signals, int world, int rank,
                             int dtype, int64_t rows, int64_t cols, int64_t ld, int blocks,
                             int64_t max_polls, int* status, b12x_b200_stream_t stream);

/*
 * The two halves of the fused row-parallel step (no counterpart in the reference either).
 *
 * b12x_b200_gemm_blockscaled_scatter: the CTA-pair GEMM of b12x_b200_gemm_blockscaled whose
 * output tiles are not written to one C but scattered by row slab: M is cut into `world` slabs
 * of M / world rows (M must be a multiple of 256 * world); a tile in slab s is stored, while the
 * main loop carries on with the next tile, into destinations[s] at rows
 * rank * (M / world) + (row - s * (M / world)). destinations[s] is rank s's [M, ld] receive
 * buffer as mapped in this process (peer memory for s != rank): when all ranks' GEMMs have
 * finished, rank s holds every rank's partial of its slab, in slot order. BF16 or FP16; the
 * optional workspace is that of b12x_b200_gemm_blockscaled_ex (split leftover tiles).
 *
 * b12x_b200_allreduce_peer_scattered: the reduction that follows. Rank s adds the `world` slots
 * of its own receive buffer (buffers[s], local reads only) in FP32 in slot order, rounds once,
 * and pushes the rows of slab s into outputs[t] of every rank t ([M, ld] result buffers, peer
 * mapped). Flags, limits, status and the rehearsal mode (rank < 0) are those of
 * b12x_b200_allreduce_peer; rows % world == 0. When the kernel has finished on a rank's stream,
 * that rank's output holds the complete sum.
 */
int b12x_b200_gemm_blockscaled_scatter(int kind, const void* a, const void* sfa, const void* b,
                                       const void* sfb, void* const* destinations, int world,
                                       int rank, int c_dtype, const float* alpha, int64_t m,
                                       int64_t n, int64_t k, int64_t ld, int sm_count,
                                       void* workspace, int64_t workspace_bytes, int* status,
                                       b12x_b200_stream_t stream);
int b12x_b200_allreduce_peer_scattered(void* const* buffers, void* const* outputs,
                                       void* const* signals, int world, int rank, int dtype,
                                       int64_t rows, int64_t cols, int64_t ld, int blocks,
                                       int64_t max_polls, int* status, b12x_b200_stream_t stream);

/*
 * Load-time conversion of a block-scaled FP8 checkpoint weight (E4M3 codes [groups, M, K], one
 * FP32 scale per 128 x 128 block, [groups, ceil(M/128), K/128]) into the MXFP8 rows the GEMM
 * reads. Replaces pack_fp8_block_scaled_weight_mxfp8 and its helpers
 * (b12x/gemm/_shared/wo_mxfp8.py:873-1187), byte for byte:
 *   requantize != 0: v = code * scale in FP32, block amax, byte = 127 + clamp(ceil(log2(amax /
 *     448)), -127, 127) (127 for an all-zero block), new code = E4M3(v / 2^(byte - 127));
 *   requantize == 0 (every scale already a power of two): codes are copied, byte is the
 *     scale's exponent.
 * out_codes [groups, M, K]; scale_rows (optional) [groups, M, K/32] row-major bytes; scale_mma
 * (optional) the 512-byte atoms [groups][ceil(M/128)][K/128], rows beyond M set to 127.
 * K % 128 == 0. In place (out_codes == codes) is allowed.
 */
int b12x_b200_pack_block_fp8_weight_mxfp8(const void* codes, const float* scale, void* out_codes,
                                          void* scale_rows, void* scale_mma, int64_t m, int64_t k,
                                          int64_t groups, int requantize,
                                          b12x_b200_stream_t stream);

/*
 * Batched C[b] = A[b] @ dequant(W[b]) for b < batch: A BF16 [batch, M, K] with 1 <= M <= 32, W
 * rowwise MXFP8 (E4M3 codes and one UE8M0 byte per 32 codes of the contiguous axis), C BF16
 * [batch, M, N], FP32 accumulation. Replaces the launch of the MXFP8 backend of b12x.gemm.bmm
 * (b12x/gemm/_shared/mxfp8_bmm.py:1771-1834, kernel :446-1040; public contract
 * b12x/gemm/_bmm/api.py:41-83).
 *   n_major == 0: codes [batch, N, K], scales [batch, N, K/32]; K % 32 == 0.
 *   n_major != 0: codes [batch, K, N], scales [batch, K, N/32]; N % 32 == 0, K % 8 == 0.
 * Every tensor is given by its base and the strides (in elements) of its two outer axes; the
 * inner axis is contiguous. A rows and weight rows start on 16-byte boundaries, C rows on
 * 4-byte boundaries. A weight is dequantized as BF16(code * 2^(byte - 127)) (byte 255 is NaN).
 * No workspace, no allocation, no status word (the kernel waits on nothing); safe to capture in
 * a CUDA graph. Each output is a fixed-order sum, so repeated launches give identical bits.
 */
int b12x_b200_bmm_mxfp8(const void* a, int64_t a_stride_b, int64_t a_stride_m,
                        const void* w_values, int64_t w_stride_b, int64_t w_stride_r,
                        const void* w_scales, int64_t sf_stride_b, int64_t sf_stride_r, void* c,
                        int64_t c_stride_b, int64_t c_stride_m, int n_major, int64_t batch,
                        int64_t m, int64_t n, int64_t k, b12x_b200_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* B12X_B200_H_ */
