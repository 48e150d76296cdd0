/*
 * adangel_b200 — C ABI of the B200 (sm_100a) backend for ADAngel's O0/O1/O2 quantized GEMMs
 *
 *     Y[M,N] (fp32) = (A_int8[M,K] * A_scale[M]) @ (W_mxfp4[N,K/2] * 2^(W_scale[N,K/32]-127))^T
 *
 * This is the drop-in boundary: plain pointers and sizes, no framework types.  The reference
 * project exposes the same operations through a pybind11/torch extension module
 * (csrc/bindings.cpp:84-103, prototypes in include/adangel/kernel_api.h:13-86); each entry point
 * below names the reference interface it replaces.
 *
 * Conventions
 *   - Every function returns 0 on success and a non-zero code on failure; adg_last_error()
 *     returns the message of the calling thread's last failure.
 *   - "device" pointers are CUDA device pointers valid on the current device; work is enqueued on
 *     the given stream (a cudaStream_t passed as void*, NULL = the default stream) and the call
 *     returns without synchronising unless stated otherwise.
 *   - Tensors are dense row-major.  K must be a multiple of 64; M, N, K > 0.
 *   - E2M1 nibbles: even k in the low nibble.  UE8M0 code c means 2^(c-127); code 255 is forbidden.
 *   - There is no CPU fallback: on a machine without a B200-class GPU the compute calls fail.
 */
#ifndef ADANGEL_B200_H_
#define ADANGEL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------------------------- */

/* ABI version of this header (major * 100 + minor). */
int adg_abi_version(void);

/* Message of the calling thread's last failed call ("" if none). */
const char* adg_last_error(void);

/* Capability bits; replaces capabilities() of the reference module (csrc/bindings.cpp:11-20).
 * Bit set = the production kernel for that capability is compiled into this library. */
#define ADG_CAP_COMPILED_SM100A 0x01u
#define ADG_CAP_O0_FP16_TC 0x02u
#define ADG_CAP_O1_INT8_TC 0x04u
#define ADG_CAP_O2_MXF4_BLOCK_SCALE 0x08u
#define ADG_CAP_O2_TILED 0x10u
uint32_t adg_capabilities(void);

/* Fills name (NUL-terminated, at most name_len bytes), compute capability and SM count of the
 * current CUDA device.  Fails if no CUDA device is usable. */
int adg_device_info(char* name, int name_len, int* cc_major, int* cc_minor, int* sm_count);

/* Waits for the work enqueued on `stream`, then reads and clears the device status words written
 * by kernels whose bounded waits gave up; fails with a description if one did.  Also covers the status
 * words of asynchronous adg_o2_linear_noalloc calls (see there). */
int adg_check_status(void* stream);

/* What the planner runs for a shape: kernel, tile, pipeline depth.  Replaces the `kernel` metadata
 * dictionary the reference's benchmark functions build by hand (csrc/sm120/o0_gemm.cu:300-328,
 * o1_gemm.cu:395-429, o2_cutlass.cu:320-362).  variant: 0 = O0, 1 = O1, 2 = O2, 3 = o1x.  The rules depend on
 * the SM count: the current device's, or a B200's 148 when no device is usable. */
#define ADG_PLAN_O1_BF16 1u          /* O1 on BF16 operands (adg_gemm_o1_bf16 / adg_o1_linear) */
#define ADG_PLAN_FUSED_ACTIVATION 2u /* O0 / O2 through adg_o0_linear / adg_o2_linear */
#define ADG_PLAN_PARTIAL_DUMP 4u     /* O1 with the INT32 partial dump */
typedef struct adg_plan_desc {
  int32_t tile_m, tile_n, stages, accumulator_stages, threads, cluster;
  int32_t mma_m, mma_n, mma_k, persistent, fused_activation;
  char kernel_symbol[64];
  char mma_family[96];
} adg_plan_desc;
int adg_plan_info(int variant, int flags, int M, int N, int K, adg_plan_desc* out);

/* ---- conversion kernels (device pointers) -------------------------------------------------- */

/* O0 weight conversion: out_fp16[rows,K] = half(e2m1(nibble) * 2^(scale-127)).
 * Replaces adangel_launch_mxfp4_to_fp16 (include/adangel/kernel_api.h:21-25,
 * kernel csrc/sm120/conversion.cu:10-23). */
int adg_mxfp4_to_fp16(const void* w_mxfp4, const void* w_scale, void* out_fp16, int64_t rows, int64_t K, void* stream);

/* O0 activation conversion: out_fp16[rows,K] = half(float(a) * a_scale[row]).
 * Replaces adangel_launch_int8_to_fp16 (kernel_api.h:27-31, conversion.cu:25-37). */
int adg_int8_to_fp16(const void* a_int8, const void* a_scale, void* out_fp16, int64_t rows, int64_t K, void* stream);

/* O1 weight conversion: out_int8[rows,K] = 2 * e2m1(nibble), exact.
 * Replaces adangel_launch_mxfp4_to_int8 (kernel_api.h:33-36, conversion.cu:39-50). */
int adg_mxfp4_to_int8(const void* w_mxfp4, void* out_int8, int64_t rows, int64_t K, void* stream);

/* Operands of adg_gemm_o1_bf16 (no reference counterpart: the reference's O1 kernel takes INT8
 * operands; see adg_gemm_o1_bf16 for why these exist).
 *   out_bf16[rows,K] = bfloat16(e2m1(nibble) * 2^(scale-127)), exact (two significant bits);
 *   out_bf16[rows,K] = bfloat16(a), exact (integers of magnitude <= 128).
 * range_flag is one zero-initialised 32-bit device word shared by the two conversions and the GEMM:
 * bit 0 is set when a weight scale code lies outside [48, 208], bit 1 when an activation scale lies
 * outside [2^-46, 2^30] or is not finite -- the ranges inside which the BF16-operand kernel is
 * bit-identical to the INT8-operand kernel. */
int adg_mxfp4_to_bf16_scaled(const void* w_mxfp4, const void* w_scale, void* out_bf16, void* range_flag, int64_t rows,
                             int64_t K, void* stream);
int adg_int8_to_bf16(const void* a_int8, const void* a_scale, void* out_bf16, void* range_flag, int64_t rows, int64_t K,
                     void* stream);

/* Size in bytes of the tiled scale-factor buffer for a [rows, K/32] scale matrix (512-byte atoms
 * of 128 rows x 4 blocks, zero padded to 256 rows / 8 blocks). */
int64_t adg_o2_tiled_scale_bytes(int64_t rows, int64_t K);

/* O2 activation re-quantization, fused with the scale re-layout: per (row, K32 block) of
 * float(a)*a_scale[row]: UE8M0 scale floor(log2(amax))-2 (0 for a zero block) and E2M1
 * round-to-nearest-even codes.  Writes packed codes [M,K/2], optionally the natural scales
 * [M,K/32] (sf_natural may be NULL) and the tiled scales (sf_tiled, which the caller zero-filled
 * once so that padding is zero).  Replaces adangel_o2_quantize_activation +
 * adangel_o2_repack_scale (csrc/sm120/o2_cutlass.cu:207-274). */
int adg_o2_quantize_activation(const void* a_int8, const void* a_scale, void* a_mxfp4, void* sf_natural,
                               void* sf_tiled, int64_t M, int64_t K, void* stream);

/* O2 weight-scale re-layout: natural [rows,K/32] -> tiled buffer (padding written as zero).
 * Replaces adangel_o2_repack_scale for SFB (o2_cutlass.cu:261-274, :298-316). */
int adg_o2_tile_scales(const void* sf_natural, void* sf_tiled, int64_t rows, int64_t K, void* stream);

/* ---- sample preparation (device pointers): the step in front of the hot path ----------------- */
/* x_dtype: 0 = FP32, 1 = FP16 (widened to FP32 first, as the reference does).  Inputs must be
 * finite; the reference rejects NaN/Inf with a host-side check before quantizing and callers of
 * these entry points do the same. */

/* Symmetric per-row INT8 quantization: scale[r] = amax_r / 127 (1 for an all-zero row),
 * q = clamp(round_half_even(x / scale), -127, 127).  Replaces quantize_int8_per_row
 * (python/adangel/quantization/int8.py:6-17) as used by prepare_trace
 * (python/adangel/trace/prepare.py:113). */
int adg_quantize_int8_per_row(const void* x, int x_dtype, void* q_int8, void* scale, int64_t rows, int64_t K,
                              void* stream);

/* MXFP4 quantization of the last dimension: per (row, K32 block) the UE8M0 scale code
 * floor(log2(amax)) - 2 + 127 (127 for an all-zero block, exponent taken exactly) and packed E2M1
 * round-to-nearest-even codes [rows,K/2] (even K in the low nibble).  Replaces quantize_mxfp4
 * (python/adangel/quantization/mxfp4.py:147-180) as used by prepare_trace (prepare.py:114). */
int adg_quantize_mxfp4(const void* x, int x_dtype, void* packed, void* scale_codes, int64_t rows, int64_t K,
                       void* stream);

/* ---- GEMM kernels (device pointers) ---------------------------------------------------------- */
/* ldy is the row pitch of Y in elements (>= N); Y may be a column block of a wider matrix. */

/* O0 GEMM: Y = A_fp16 @ W_fp16^T, FP32 accumulate (tcgen05 kind::f16).
 * Replaces the cuBLASLt plan O0LtPlan::run (csrc/sm120/o0_gemm.cu:86-298). */
int adg_gemm_o0(const void* a_fp16, const void* w_fp16, float* y, int M, int N, int K, int ldy, void* stream);

/* O1 GEMM: per K32 group INT32 partial (tcgen05 kind::i8) scaled by
 * (A_scale[m] * 2^(W_scale[n,g]-127)) * 0.5 and accumulated in FP32 in ascending group order.
 * partial_dump, if not NULL, receives the INT32 partials as [M,N,K/32] (debug/parity aid).
 * Replaces adangel_o1_tma_warp_specialized (csrc/sm120/o1_gemm.cu:167-392). */
int adg_gemm_o1(const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, float* y,
                int32_t* partial_dump, int M, int N, int K, int ldy, void* stream);

/* O1 for decode-sized activations straight from the packed weights: the same recurrence and the same bits
 * as adg_gemm_o1, with W read as MXFP4 nibbles (N*K/2 bytes instead of the N*K of its INT8 image) and
 * expanded to 2*E2M1 inside the kernel.  M <= 8, or M <= 16 while N/32 does not exceed the SM count;
 * other shapes are refused with an error (use adg_mxfp4_to_int8 + adg_gemm_o1).  Half the DRAM traffic of
 * adg_gemm_o1 and no INT8 image to keep resident, for 5 - 10 % more time (every thread expands its own
 * nibbles): the form for servers that hold only the packed weights.  No reference
 * counterpart: the reference's O1 always consumes the INT8 image (csrc/sm120/o1_gemm.cu:367-392). */
int adg_gemm_o1_packed(const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_scale, float* y, int M, int N,
                       int K, int ldy, void* stream);

/* O1 GEMM on BF16 operands: the same recurrence and the same bits as adg_gemm_o1, computed with the
 * weight's power-of-two scale folded into the tensor-core operand (tcgen05 kind::f16, BF16 x BF16,
 * FP32 accumulate): each K32 partial leaves the tensor core as float(P) * 2^(W_scale-128), exact, and
 * the epilogue multiplies by A_scale[m] and adds -- no integer conversion and no per-column factor
 * in the inner loop, which is what bounds adg_gemm_o1.  a_bf16 / w_bf16 come from adg_int8_to_bf16 /
 * adg_mxfp4_to_bf16_scaled.  If *range_flag is non-zero the kernel does not compute: it records an
 * error that the next status check reports, and the caller falls back to adg_gemm_o1, which covers
 * every input.  M > 64 is the intended use (decode-sized M: adg_gemm_o1). */
int adg_gemm_o1_bf16(const void* a_bf16, const void* a_scale, const void* w_bf16, float* y, const void* range_flag, int M,
                     int N, int K, int ldy, void* stream);

/* O1 in one call, for every input and without a host synchronisation: converts A to BF16, runs
 * adg_gemm_o1_bf16, and behind it the INT8-operand kernel, which returns at once unless the first
 * one refused (operands outside its exact range).  flags points at two 32-bit device words: [0] is the
 * weight's word, zeroed by the caller and then written by adg_mxfp4_to_bf16_scaled when w_bf16 was made;
 * [1] is scratch.  a_bf16_workspace holds M*K BF16 values.  With M <= 64, or w_bf16 / the workspace NULL,
 * only the INT8-operand kernels run.  No reference counterpart. */
int adg_o1_linear(const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, const void* w_bf16,
                  void* a_bf16_workspace, void* flags, float* y, int M, int N, int K, int ldy, void* stream);

/* O2 GEMM: block-scaled MXFP4 x MXFP4 (tcgen05 kind::mxf4.block_scale), scales in tiled layout.
 * Replaces the CUTLASS block-scaled GEMM (csrc/sm120/o2_cutlass.cu:35-93, :394-472). */
int adg_gemm_o2(const void* a_mxfp4, const void* a_sf_tiled, const void* w_mxfp4, const void* w_sf_tiled, float* y,
                int M, int N, int K, int ldy, void* stream);

/* O0 / O2 steady-state pass in one call: activation conversion + GEMM, the sequence the reference runs for every
 * steady-state pass (csrc/sm120/o0_gemm.cu:432-470, o2_cutlass.cu:451-472).  With row_counters == NULL (the
 * default, and the faster path at every measured shape) the conversion kernel runs first and the GEMM behind
 * it.  With row_counters given and M > 64 the conversion runs INSIDE the GEMM kernel: a fourth warp group of
 * every CTA converts rows of A_int8 into the operand buffer (FP16, or MXFP4 codes + tiled scales) while the
 * tensor cores work, and the kernel's TMA producer waits on per-row-block counters before it loads a row
 * block; the results are bit-identical to the two-kernel sequence.  Measured on B200 the four converter
 * warps a GEMM CTA can host are not enough to stream A (O2 at 4096^3: 67 us against 50 us for the two
 * kernels; O0: 117 against 109), so the one-kernel form is kept as an option, not as the default.
 *   - a_fp16_workspace [M,K] FP16 / a_mxfp4_workspace [M,K/2] + a_sf_tiled_workspace
 *     (adg_o2_tiled_scale_bytes(M,K), zero-filled once by the caller) receive the converted operand;
 *     a_sf_natural ([M,K/32], may be NULL) the natural-layout scales.
 *   - row_counters (optional): adg_fused_workspace_bytes(M) bytes, zero-filled once by the caller; the kernel leaves
 *     them zero again.  After a call that reported a device-side error, zero them before the next call.
 *     Calls that share counters or workspaces must not overlap on the GPU. */
int64_t adg_fused_workspace_bytes(int64_t M);
int adg_o0_linear(const void* a_int8, const void* a_scale, const void* w_fp16, void* a_fp16_workspace, void* row_counters,
                  float* y, int M, int N, int K, int ldy, void* stream);
int adg_o2_linear(const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_sf_tiled, void* a_mxfp4_workspace,
                  void* a_sf_tiled_workspace, void* a_sf_natural, void* row_counters, float* y, int M, int N, int K, int ldy,
                  void* stream);

/* ---- o1x: the exact-integer variant of O1 (no reference counterpart; never selected on a caller's behalf) ----
 * The literal O1 (adg_gemm_o1, reference csrc/sm120/o1_gemm.cu:298-316) rounds twice per K32 group, which
 * keeps every INT32 partial on the FP32 pipe.  Where the scale codes of a W row differ by at most 3, the row
 * is rewritten as INT8 with one exponent, W'[n,k] = 2*e2m1 << (code[n,g] - min_g code[n,.]) (|W'| <= 96), and
 *     y[m,n] = RN(float_rn(sum_k A_int8[m,k] * W'[n,k]) * RN(A_scale[m] * 2^(mincode[n]-128)))
 * with the INT32 sum exact over all of K (tcgen05 kind::i8, accumulator in tensor memory): two roundings in
 * total.  128-column blocks of Y that contain a row with a larger spread (blocks of all-zero nibbles do not
 * count) are computed by the literal kernel instead, on a device-side list, without a host round trip.
 *   adg_o1x_prepare_weight: once per weight; writes w_int8x [N,K] INT8, col_factor [N] FP32 and `workspace`
 *     (adg_o1x_workspace_bytes(N): ineligible-row count, block flags, block list).
 *   adg_o1x_ineligible_rows: synchronises and returns the number of W rows that take the literal path.
 *   adg_gemm_o1x: the GEMM; w_int8 (adg_mxfp4_to_int8) and w_scale serve the literal path and may be NULL
 *     only if no row is ineligible. */
int64_t adg_o1x_workspace_bytes(int64_t N);
int adg_o1x_prepare_weight(const void* w_mxfp4, const void* w_scale, void* w_int8x, void* col_factor, void* workspace,
                           int64_t N, int64_t K, void* stream);
int adg_o1x_ineligible_rows(const void* workspace, void* stream, int64_t* rows);
int adg_gemm_o1x(const void* a_int8, const void* a_scale, const void* w_int8x, const void* col_factor, const void* workspace,
                 const void* w_int8, const void* w_scale, float* y, int M, int N, int K, int ldy, void* stream);

/* O2 without device allocations: Y = requantize(A) @ W^T in one call, for callers that cannot
 * allocate (a server whose memory pool already owns all of the GPU's memory, or a latency-critical
 * loop that must avoid the device-wide synchronisation of cudaMalloc/cudaFree).  The packed codes
 * and tiled scales of A and the kernels' status words live in a fixed array inside the library
 * (about 4.5 MiB held on every GPU that loads it, until the process exits); the caller passes only
 * inputs and the output.  This entry point has no counterpart in the reference.
 *   - Limits: M*K/2 <= 4 MiB of codes and adg_o2_tiled_scale_bytes(M, K) <= 512 KiB (for example
 *     1024 x 8192 or 512 x 16384); larger activations are rejected with an error.
 *   - w_sf_tiled is W's scales in tiled form (adg_o2_tile_scales, done once per weight).
 *   - The first call on a device performs one-time set-up (address look-up of the array, kernel
 *     attributes); make that first call before starting any stream capture -- and before the caller's
 *     pool takes the rest of the device's memory: the array itself comes into being when the CUDA runtime
 *     loads this library's kernels onto the device, which happens no later than that first call.
 *   - All calls share the one array: two calls that overlap on the GPU (different streams, or
 *     different host threads) race on it.  Issue them on one stream or order them yourself.
 *   - synchronize != 0: wait for the result and report a kernel wait timeout as an error;
 *     synchronize == 0: return after enqueueing; a timeout is then reported by the next
 *     adg_o2_linear_noalloc_status (or adg_check_status) call.
 * It calls no cudaMalloc/cudaFree and no allocating library routine. */
int adg_o2_linear_noalloc(const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_sf_tiled,
                          float* y, int M, int N, int K, int ldy, void* stream, int synchronize);

/* Status of earlier asynchronous adg_o2_linear_noalloc calls: waits for `stream`, reads the status words
 * that those calls' kernels keep inside the built-in array, clears them if set and fails with a
 * description.  Allocates nothing (unlike adg_check_status, whose first use on a device allocates the
 * regular path's status words).  Returns 0 when adg_o2_linear_noalloc has not been used on this device.
 * No counterpart in the reference. */
int adg_o2_linear_noalloc_status(void* stream);

/* For tests and tools: device address and size in bytes of the status words read by
 * adg_o2_linear_noalloc_status (performs the one-time set-up if needed). */
int adg_o2_linear_noalloc_status_words(void** device_address, int* bytes);

/* ---- timing harness -------------------------------------------------------------------------- */

#define ADG_MODE_CONVERSION_ONLY 0
#define ADG_MODE_COMPUTE_ONLY 1
#define ADG_MODE_COLD 2
#define ADG_MODE_STEADY_STATE 3

#define ADG_STAGE_WEIGHT 0x1u
#define ADG_STAGE_ACTIVATION 0x2u
#define ADG_STAGE_GEMM 0x4u
#define ADG_STAGE_TOTAL 0x8u

typedef struct adg_bench_args {
  int32_t variant; /* 0, 1, 2 */
  int32_t mode;    /* ADG_MODE_* */
  int32_t M, N, K;
  int32_t warmup, repeats, conversion_inner_repeats;
  /* inputs (device) */
  const void* a_int8;
  const void* a_scale;
  const void* w_mxfp4;
  const void* w_scale;
  /* caller-owned device buffers */
  float* output;        /* [M,N] */
  void* conv_weight;    /* O0: fp16 [N,K]; O1: int8 [N,K]; O2: tiled W scales */
  void* conv_act;       /* O0: fp16 [M,K]; O2: packed codes [M,K/2]; O1: unused */
  void* conv_act_sf;    /* O2: natural scales [M,K/32] */
  void* conv_act_sf_tiled; /* O2: tiled A scales, zero-filled by the caller */
  /* host result arrays, each `repeats` floats (milliseconds); filled for the stages in stages_out */
  float* t_weight;
  float* t_activation;
  float* t_gemm;
  float* t_total;
  uint32_t stages_out;
  void* stream;
  /* O1 only, optional (all three or none; ABI 101): bf16 [N,K], bf16 [M,K] and one 32-bit device word.  When
   * given, M > 64 and the operands lie inside adg_gemm_o1_bf16's exact range (decided once, before any
   * timing, by converting both and reading the word), O1 runs on BF16 operands: the activation
   * conversion stage is adg_int8_to_bf16, the weight conversion stage writes both conv_weight (INT8, the
   * tensor returned to the caller) and conv_weight_bf16, the GEMM stage is adg_gemm_o1_bf16 -- same bits. */
  void* conv_weight_bf16;
  void* conv_act_bf16;
  void* range_flag;
  /* ABI 102 */
  uint32_t flags;      /* ADG_BENCH_* */
  void* row_counters;  /* O0 / O2 with ADG_BENCH_FUSE_ACTIVATION: adg_fused_workspace_bytes(M), zero-filled */
  /* variant 3 (o1x): conv_weight is the shifted INT8 image [N,K]; plus */
  void* o1x_col_factor; /* float [N] */
  void* o1x_workspace;  /* adg_o1x_workspace_bytes(N) */
  void* o1x_w_int8;     /* int8 [N,K]: the literal path's weights */
  /* ADG_BENCH_FLUSH_L2: a device buffer larger than the L2 that is overwritten before every directly timed
   * iteration (outside its events), so that the iteration's operands come from HBM */
  void* l2_flush;
  int64_t l2_flush_bytes;
} adg_bench_args;

/* cold / steady_state of O0 and O2 run adg_o0_linear / adg_o2_linear's fused kernel: the `gemm` stage is
 * that kernel (conversion inside), `activation_conversion` is still reported from the isolated batches of the
 * stand-alone conversion kernel, and `total` is the directly timed path. */
#define ADG_BENCH_FUSE_ACTIVATION 1u
/* O1 on BF16 operands: report the INT8 -> BF16 activation conversion as a stage of its own instead of
 * inside `gemm` (the reference's O1 has no activation stage, tests/integration/test_sm120_o1.py:86-94). */
#define ADG_BENCH_O1_SPLIT_ACTIVATION 2u
/* Cold operands: overwrite l2_flush (more than the L2's size) before every directly timed iteration.  The
 * reference's protocol leaves the L2 as the previous iteration left it (docs/experiment_protocol.md:25-42),
 * which for decode-sized problems means W is served from the L2; this flag is how the weight-streaming
 * decode shapes are measured against the HBM roofline. */
#define ADG_BENCH_FLUSH_L2 4u

/* Runs the reference's timing protocol for one variant and mode (warm-up, `repeats` directly timed
 * iterations with CUDA events, conversions additionally timed as isolated batches of
 * conversion_inner_repeats launches) and leaves a valid output in args->output.  Synchronises.
 * Replaces adangel_benchmark_o0/o1/o2 (csrc/sm120/o0_gemm.cu:351-531, o1_gemm.cu:431-566,
 * o2_cutlass.cu:364-617). */
int adg_benchmark(adg_bench_args* args);

/* Known-answer probe of the block-scaled MMA's scale-factor layout: one tile, all nibbles +0.5,
 * a distinct scale per row/column/block.  Replaces adangel_verify_o2_layout_cuda
 * (csrc/sm120/o2_microkernel.cu:49-115).  Synchronises. */
int adg_verify_layout(int* passed, float* max_abs_error);

/* ---- gathering N-sharded results over NVLink ----------------------------------------------------- */
/* One process per GPU on one node, W sharded along N: rank r holds Y[:, n0_r:n1_r] as a contiguous
 * [M, width_r] FP32 buffer.  The reference is single-GPU and has no counterpart; these entry points
 * replace a library all-gather plus a local permute by ONE kernel that reads the other ranks' blocks
 * from their memory (CUDA IPC mappings, plain loads over NVLink) and writes them to their columns of a
 * contiguous [M, N] on this rank. */

#define ADG_PEER_HANDLE_BYTES 64
#define ADG_MAX_PEER_BLOCKS 16

/* Exports the allocation that contains `ptr` (device memory from cudaMalloc, e.g. a torch tensor's
 * storage): 64 opaque bytes to send to the other processes, and ptr's offset inside the allocation. */
int adg_peer_export(const void* ptr, void* handle64, uint64_t* offset);
/* Maps an allocation exported by another process of this node; *base + offset is the peer's `ptr`.
 * Enables peer access between the two devices.  One open per handle per process. */
int adg_peer_open(const void* handle64, void** base);
int adg_peer_close(void* base);

typedef struct adg_peer_blocks {
  const float* src[ADG_MAX_PEER_BLOCKS]; /* contiguous [M, width] blocks: own memory or adg_peer_open mappings */
  int col0[ADG_MAX_PEER_BLOCKS];         /* first destination column; a multiple of 4 */
  int width[ADG_MAX_PEER_BLOCKS];        /* columns; a multiple of 4 */
  int count;
} adg_peer_blocks;

/* y[row, col0_b + c] = src_b[row, c] for every block, on `stream`; y is [M, ldy] FP32, 16-byte
 * aligned, ldy a multiple of 4.  The kernel waits for nobody: order it after every rank's producer of
 * its block (a collective or barrier on the stream), and keep the blocks unchanged until every rank's
 * gather has finished.  Asynchronous. */
int adg_gather_columns_pull(const adg_peer_blocks* blocks, float* y, int M, int64_t ldy, void* stream);

/* ---- host-buffer sessions ---------------------------------------------------------------------- */
/* A session keeps one weight matrix resident on the device in the form a variant's GEMM consumes
 * (the steady-state case: weights converted once, activations arriving from the host each call). */

typedef struct adg_session adg_session;

/* Uploads W (host pointers) for `variant`, converts it and sizes activation/output buffers for up
 * to max_M rows.  Synchronises. */
int adg_session_create(adg_session** out, int variant, int max_M, int N, int K, const void* w_mxfp4_host,
                       const void* w_scale_host);

/* One end-to-end pass: host A -> device, activation conversion, GEMM, device Y -> host (y_host is
 * [M,N] fp32).  Pinned host buffers make the copies asynchronous; the call returns after the
 * result is in y_host. */
int adg_session_run(adg_session* session, const void* a_int8_host, const void* a_scale_host, int M, float* y_host);

/* The two halves of adg_session_run: submit enqueues the pass on the session's own stream and
 * returns at once (pinned host buffers; both must stay untouched until the wait), wait blocks until
 * the result is in y_host and reports device-side errors.  Several sessions submitted before their
 * waits overlap one session's copies with another's kernels.  One pass in flight per session.
 * No reference counterpart (the reference's operators are synchronous device-tensor calls). */
int adg_session_submit(adg_session* session, const void* a_int8_host, const void* a_scale_host, int M, float* y_host);
int adg_session_wait(adg_session* session);

void adg_session_destroy(adg_session* session);

#ifdef __cplusplus
}
#endif

#endif /* ADANGEL_B200_H_ */
