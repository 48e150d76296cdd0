// Host-side declarations shared by the translation units of the library: per-device context,
// tensor-map encoding, kernel launchers and GEMM plans.  Nothing here is part of the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace adg {

// ---- errors -----------------------------------------------------------------------------------
// Library calls return 0 on success; a non-zero return leaves a message for adg_last_error().
void set_error(const std::string& message);
int fail(const std::string& message);
int check_cuda(cudaError_t err, const char* what);
const char* last_error_cstr();

// ---- launches ------------------------------------------------------------------------------------
// Launch with programmatic stream serialization (and, optionally, clusters of `cluster_x` CTAs): the kernel may
// become resident while its predecessor in the stream drains; it calls pdl_wait() (common.cuh) before it
// touches global memory.  ADG_PDL=0 in the environment launches the ordinary way.
bool overlapped_launches_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                              Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (overlapped_launches_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  config.attrs = attrs;
  config.numAttrs = n;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// ---- per-device context -------------------------------------------------------------------------
struct DeviceCtx {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  uint32_t* status = nullptr;  // kStatusWords device words, zero when healthy
};
// Context of the current device (created on first use; allocates the status words once).
int device_ctx(DeviceCtx** out);
// Reads the device status words of the current device (synchronises the device's work on
// `stream` first), clears them, and returns non-zero with a message if a kernel reported an error.
int check_device_status(cudaStream_t stream);

// Status words of asynchronous adg_o2_linear_noalloc calls (noalloc.cu); a no-op when that entry point
// has not been used on the current device.
int noalloc_check_status(cudaStream_t stream, bool synchronize);

// ---- scale-factor tiled layout ---------------------------------------------------------------------
// 512-byte atoms of 128 rows x 4 K32 blocks, ordered row-block major / K-atom minor; rows are
// padded to a multiple of 256 and K32 blocks to a multiple of 8 (zero bytes).
inline long tiled_scale_rows(long rows) { return (rows + 255) / 256 * 256; }
inline long tiled_scale_katoms(long k) { return ((k / 32 + 7) / 8) * 2; }
inline long tiled_scale_bytes(long rows, long k) { return tiled_scale_rows(rows) * tiled_scale_katoms(k) * 4; }

// ---- conversion launchers (device pointers) ----------------------------------------------------------
int launch_mxfp4_to_fp16(const void* packed, const void* scales, void* out, long rows, long k, cudaStream_t stream);
int launch_int8_to_fp16(const void* in, const void* row_scale, void* out, long rows, long k, cudaStream_t stream);
int launch_mxfp4_to_int8(const void* packed, void* out, long rows, long k, cudaStream_t stream);
// Operands of the O1 kernel with BF16 operands; `range_flag` is one device word (bit 0: a weight
// scale code outside [kO1MinScaleCode, kO1MaxScaleCode]; bit 1: an activation scale outside
// [2^kO1MinAScaleExp, 2^kO1MaxAScaleExp] or not finite).
constexpr unsigned kO1MinScaleCode = 48, kO1MaxScaleCode = 208;
constexpr int kO1MinAScaleExp = -46, kO1MaxAScaleExp = 30;
int launch_mxfp4_to_bf16_scaled(const void* packed, const void* scales, void* out, void* range_flag, long rows, long k,
                                cudaStream_t stream);
int launch_int8_to_bf16(const void* in, const void* row_scale, void* out, void* range_flag, long rows, long k,
                        cudaStream_t stream);
int launch_o2_quantize(const void* a_int8, const void* row_scale, void* codes, void* sf_natural, void* sf_tiled,
                       long rows, long k, cudaStream_t stream);
int launch_o2_tile_scales(const void* natural, void* tiled, long rows, long k, cudaStream_t stream);
// sample preparation; dtype 0 = FP32, 1 = FP16
int launch_quantize_int8_rows(const void* x, int dtype, void* q, void* scale, long rows, long k, cudaStream_t stream);
int launch_quantize_mxfp4(const void* x, int dtype, void* codes, void* scale_codes, long rows, long k, cudaStream_t stream);

// ---- tensor maps ---------------------------------------------------------------------------------
// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements with a row pitch of `pitch_bytes`;
// the box is box_cols x box_rows elements; its width in bytes (64 or 128) selects the shared-memory
// swizzle of the same width.
int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t rows,
                         uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols);

// ---- GEMM plans ----------------------------------------------------------------------------------
// A plan holds the encoded tensor maps and launch geometry of one GEMM on fixed buffers; running it
// only launches the kernel.
struct GemmPlan {
  int variant = -1;  // 0 = O0 (f16), 1 = O1 (i8 + per-K32 rescale), 2 = O2 (mxf4 block-scaled), 3 = o1x (i8, exact integer)
  int M = 0, N = 0, K = 0, ldy = 0;
  int block_n = 0;
  int grid = 0;
  int use_tma_store = 0;
  CUtensorMap tm_a, tm_b, tm_y;
  CUtensorMap tm_sfa, tm_sfb;  // O2 on CTA pairs: [row block][32-bit words] views of the tiled scale arrays
  const void* a_scale = nullptr;   // O1: float [M]
  const void* w_scale = nullptr;   // O1: natural UE8M0 [N, K/32]
  const void* sfa = nullptr;       // O2: tiled A scales
  const void* sfb = nullptr;       // O2: tiled W scales
  float* y = nullptr;
  int32_t* partial_dump = nullptr;  // O1 debug: INT32 partials [M, N, K/32]
  // decode-sized O1/O2 (M <= 64): operand-swapped kernels; tm_a = A map, tm_b = W map; `grid_y`
  // is the number of 16-row slices of A (O1) or the number of CTAs that share a W row block's K extent (O2)
  int skinny = 0, grid_y = 1;
  int packed_w = 0;  // O1 decode kernel: W is the packed MXFP4 matrix itself, not its INT8 image
  int o1_bf16 = 0;                       // O1 with BF16 operands (weight scale folded into W)
  const uint32_t* range_flag = nullptr;  // O1 BF16: device word set by the operand conversions
  const uint32_t* only_if_flag = nullptr;  // O1 INT8: run only when this device word is non-zero
  int quiet_refusal = 0;                 // O1 BF16: a set flag makes the kernel return without an error status
  int pair = 0;  // O0/O2 on CTA pairs (cta_group::2): tm_b has 128-row boxes, grid = 2 x clusters
  const int32_t* n_list = nullptr;   // O1 INT8: restrict the launch to the listed column blocks ([0] = count)
  const void* col_factor = nullptr;  // o1x: float [N], 2**(emin[n]-128)
  // O0/O2 with the activation conversion done by converter warps inside the GEMM kernel: tm_a maps
  // `fused_a_out`, which those warps write from `fused_a_int8` (a_scale = the row scales); `fused_ready`
  // holds ceil(M/128) + 1 zeroed counters
  int fused = 0;
  const void* fused_a_int8 = nullptr;
  void* fused_a_out = nullptr;
  void* fused_sf_natural = nullptr;
  uint32_t* fused_ready = nullptr;
  uint32_t* status = nullptr;
};

// What a plan would run, for callers that report it (adg_plan_info).
struct PlanInfo {
  const char* symbol = "";
  const char* mma_family = "";
  int tile_m = 0, tile_n = 0, stages = 0, acc_stages = 0, threads = 0, cluster = 1;
  int mma_m = 0, mma_n = 0, mma_k = 0, persistent = 0, fused_activation = 0;
};
constexpr int kPlanO1Bf16 = 1, kPlanFusedActivation = 2, kPlanPartialDump = 4;
int plan_info(int variant, int flags, int M, int N, int K, PlanInfo* info);
void describe_gemm_acc(int variant, int block_n, bool fused, PlanInfo* info);
void describe_gemm_pair(int variant, bool fused, PlanInfo* info);
void describe_gemm_o1(PlanInfo* info);
void describe_gemm_o1_bf16(PlanInfo* info);
void describe_gemm_o1_skinny(PlanInfo* info);
void describe_gemm_o1_decode(int M, int N, int sm_count, PlanInfo* info);
void describe_gemm_o2_skinny(int M, PlanInfo* info);

int plan_o0(GemmPlan* plan, const void* a_fp16, const void* w_fp16, float* y, int M, int N, int K, int ldy);
int plan_o1(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, float* y,
            int32_t* partial_dump, int M, int N, int K, int ldy);
int plan_o2(GemmPlan* plan, const void* a_mxfp4, const void* sfa_tiled, const void* w_mxfp4, const void* sfb_tiled,
            float* y, int M, int N, int K, int ldy);
// plan_o1 without the decode-shape dispatch: always the 128 x 128-tile INT8-operand kernel
int plan_o1_tiled(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale,
                  float* y, int32_t* partial_dump, int M, int N, int K, int ldy);
int plan_o1x(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8x, const void* col_factor, float* y,
             int M, int N, int K, int ldy);
// O0 / O2 with the activation conversion inside the GEMM kernel (M > 64; `ready`: adg_fused_workspace_bytes)
int plan_o0_fused(GemmPlan* plan, const void* a_int8, const void* a_scale, void* a_fp16, const void* w_fp16, float* y,
                  void* ready, int M, int N, int K, int ldy);
int plan_o2_fused(GemmPlan* plan, const void* a_int8, const void* a_scale, void* a_mxfp4, void* sfa_tiled, void* sf_natural,
                  const void* w_mxfp4, const void* sfb_tiled, float* y, void* ready, int M, int N, int K, int ldy);
int plan_o1_bf16(GemmPlan* plan, const void* a_bf16, const void* a_scale, const void* w_bf16, float* y,
                 const void* range_flag, int M, int N, int K, int ldy);
int run_plan(const GemmPlan& plan, cudaStream_t stream);

// Kernel entry points behind run_plan (defined in gemm_acc.cu / gemm_o1.cu).
int run_gemm_acc(const GemmPlan& plan, cudaStream_t stream);
int run_gemm_o1(const GemmPlan& plan, cudaStream_t stream);
int init_gemm_acc_attributes();
int init_gemm_o1_attributes();
int o1_block_n();      // W rows per O1 tile
int o1_ctas_per_sm();  // resident O1 CTAs per SM
int init_gemm_skinny_attributes();
int init_gemm_pair_attributes();
int init_gemm_o1_bf16_attributes();
int run_gemm_o1_bf16(const GemmPlan& plan, cudaStream_t stream);
int o1_bf16_block_n();
int run_gemm_pair(const GemmPlan& plan, cudaStream_t stream);
int pair_tile_m();
int pair_tile_n();
int plan_o2_skinny(GemmPlan* plan, const void* a_mxfp4, const void* sfa_tiled, const void* w_mxfp4, const void* sfb_tiled,
                   float* y, int M, int N, int K, int ldy);
int run_gemm_o2_skinny(const GemmPlan& plan, cudaStream_t stream);
int init_gemm_o1_skinny_attributes();
int plan_o1_skinny(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale,
                   float* y, int M, int N, int K, int ldy);
int run_gemm_o1_skinny(const GemmPlan& plan, cudaStream_t stream);
int init_gemm_o1_decode_attributes();
bool o1_decode_applies(int M, int N, int sm_count);
int plan_o1_decode(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w, const void* w_scale, float* y,
                   int M, int N, int K, int ldy, bool packed_w);
int run_gemm_o1_decode(const GemmPlan& plan, cudaStream_t stream);
int plan_o1_packed(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_scale, float* y,
                   int M, int N, int K, int ldy);

}  // namespace adg
