// Host runtime of the library: error reporting, the per-device context, tensor-map encoding through
// the driver entry point (no link-time dependency on the driver library) and GEMM plan construction.
#include <cudaTypedefs.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "common.cuh"
#include "launch.h"

#include <cstdlib>

namespace adg {

namespace {
thread_local std::string g_last_error;
std::mutex g_ctx_mutex;
constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
bool g_ctx_ready[kMaxDevices] = {};
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
}  // namespace

const char* last_error_cstr() { return g_last_error.c_str(); }

bool overlapped_launches_enabled() {
  static const bool enabled = [] {
    const char* e = getenv("ADG_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return enabled;
}

void set_error(const std::string& message) { g_last_error = message; }

int fail(const std::string& message) {
  g_last_error = message;
  return 1;
}

int check_cuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return 0;
  g_last_error = std::string(what) + ": " + cudaGetErrorString(err);
  return 1;
}

int device_ctx(DeviceCtx** out) {
  int dev = -1;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= kMaxDevices) return fail("device index out of range");
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  if (!g_ctx_ready[dev]) {
    DeviceCtx ctx;
    ctx.device = dev;
    cudaDeviceProp prop;
    if (int rc = check_cuda(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties")) return rc;
    ctx.sm_count = prop.multiProcessorCount;
    ctx.cc_major = prop.major;
    ctx.cc_minor = prop.minor;
    if (prop.major != 10) {
      return fail("this library contains sm_100a kernels only; device '" + std::string(prop.name) +
                  "' has compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor));
    }
    if (int rc = check_cuda(cudaMalloc(&ctx.status, kStatusWords * sizeof(uint32_t)), "cudaMalloc(status)")) return rc;
    if (int rc = check_cuda(cudaMemset(ctx.status, 0, kStatusWords * sizeof(uint32_t)), "cudaMemset(status)")) return rc;
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      if (int rc = check_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres),
                              "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)"))
        return rc;
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail("cuTensorMapEncodeTiled is unavailable");
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    if (int rc = init_gemm_acc_attributes()) return rc;
    if (int rc = init_gemm_o1_attributes()) return rc;
    if (int rc = init_gemm_skinny_attributes()) return rc;
    if (int rc = init_gemm_pair_attributes()) return rc;
    if (int rc = init_gemm_o1_bf16_attributes()) return rc;
    if (int rc = init_gemm_o1_skinny_attributes()) return rc;
    if (int rc = init_gemm_o1_decode_attributes()) return rc;
    g_ctx[dev] = ctx;
    g_ctx_ready[dev] = true;
  }
  *out = &g_ctx[dev];
  return 0;
}

int check_device_status(cudaStream_t stream) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
  uint32_t words[kStatusWords] = {};
  if (int rc = check_cuda(cudaMemcpy(words, ctx->status, sizeof(words), cudaMemcpyDeviceToHost), "cudaMemcpy(status)"))
    return rc;
  if (words[0] == kStatusOk) return 0;
  check_cuda(cudaMemset(ctx->status, 0, sizeof(words)), "cudaMemset(status)");
  char buf[256];
  if (words[0] == kStatusOperandRange) {
    snprintf(buf, sizeof(buf),
             "O1 BF16-operand GEMM refused: operands outside its exact range (flag=0x%x: bit 0 weight scale codes, bit 1 "
             "activation scales); use the INT8-operand O1 GEMM for these inputs",
             words[1]);
    return fail(buf);
  }
  snprintf(buf, sizeof(buf), "kernel wait timeout: code=%u tag=0x%x block=%u detail=%u", words[0], words[1], words[2],
           words[3]);
  return fail(buf);
}

int encode_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base, uint64_t rows,
                         uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  if (g_encode == nullptr) return fail("tensor-map encoder not initialised");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail("tensor base address must be 16-byte aligned");
  if ((pitch_bytes & 15u) != 0) return fail("tensor row pitch must be a multiple of 16 bytes");
  const uint32_t box_bytes = box_cols * static_cast<uint32_t>(elem_bytes);
  if (box_bytes != 128u && box_bytes != 64u) return fail("box width must be 64 or 128 bytes");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult res = g_encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                CU_TENSOR_MAP_INTERLEAVE_NONE,
                                box_bytes == 128u ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(res)));
  return 0;
}

namespace {

// [rows][row_bytes] view of a byte array in 32-bit words, no swizzle: used for the tiled scale arrays,
// whose 512-byte atoms are copied as they lie.  The box is `box_rows` x `box_bytes`.
int encode_word_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                       uint32_t box_bytes) {
  if (g_encode == nullptr) return fail("tensor-map encoder not initialised");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail("tensor base address must be 16-byte aligned");
  if ((row_bytes & 15u) != 0 || box_bytes % 16u != 0 || box_bytes / 4u > 256u) return fail("unsupported word-map geometry");
  const cuuint64_t dims[2] = {row_bytes / 4u, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes / 4u, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult res = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box,
                                elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(res)));
  return 0;
}

// O0/O2 run on CTA pairs (cta_group::2, 256 x 256 tiles, bit-identical to the single-CTA kernels) where
// that was measured to pay: the shape must hold a full pair tile and pair up its 128-row blocks with
// little waste (an even number of them, or so many that the padded half block is under 3 %), and be
// large -- for O0 at least two waves of pair tiles and K >= 2048, or one wave and K >= 4096 (5 - 12 % faster from
// there: 47.9 vs 50.7 us at 2048 x 4096 x 4096, 119 vs 137 us at 2048 x 11008 x 4096; below one wave the single-CTA
// kernel wins, 27.2 vs 28.6 us at 1024 x 4096 x 4096); for O2 at least seven waves and K >= 4096, or one wave and
// K >= 8192, where a long K loop amortises the pair's hand-overs (39.6 vs 41.4 us at 2048 x 4096 x 11008); below that
// its single accumulator stage and the longer hand-overs between two CTAs cost what the halved W traffic saves
// (23.0 vs 22.7 us at 2048 x 4096 x 4096, equal at 4096^3, -17 % at K = 512).  ADG_TWO_CTA in the environment (read
// at every plan): 0 = never, 1 = whenever the shape holds a full pair tile.
bool pair_enabled(int variant, int M, int N, int K, int sm_count) {
  if (M < pair_tile_m() || N < pair_tile_n()) return false;
  const char* e = getenv("ADG_TWO_CTA");
  if (e != nullptr && e[0] == '0') return false;
  if (e != nullptr && e[0] == '1') return true;
  const int row_blocks = (M + 127) / 128;
  if (row_blocks % 2 != 0 && row_blocks < 33) return false;
  const long tiles = static_cast<long>((M + pair_tile_m() - 1) / pair_tile_m()) * ((N + pair_tile_n() - 1) / pair_tile_n());
  const long clusters = sm_count / 2;
  if (variant == 0) return (tiles >= 2 * clusters && K >= 2048) || (tiles >= clusters && K >= 4096);
  return (tiles >= 7 * clusters && K >= 4096) || (tiles >= clusters && K >= 8192);
}

int finish_pair_plan(GemmPlan* plan, int sm_count, uint32_t* status) {
  plan->pair = 1;
  plan->block_n = pair_tile_n();
  const long tiles = static_cast<long>((plan->M + pair_tile_m() - 1) / pair_tile_m()) *
                     ((plan->N + pair_tile_n() - 1) / pair_tile_n());
  const long clusters = sm_count / 2;
  plan->grid = static_cast<int>(2 * (tiles < clusters ? tiles : clusters));
  plan->status = status;
  return 0;
}

int check_shape(int M, int N, int K, int ldy) {
  if (M <= 0 || N <= 0 || K <= 0) return fail("M, N, and K must be positive");
  if (K % 64 != 0) return fail("K must be divisible by 64");
  if (ldy < N) return fail("ldy must be at least N");
  return 0;
}

// The epilogue writes Y through a TMA store when the tensor map's constraints hold, otherwise
// through predicated scalar stores.
int plan_output(GemmPlan* plan, float* y) {
  plan->y = y;
  const bool aligned = (reinterpret_cast<uintptr_t>(y) & 15u) == 0 && (static_cast<uint64_t>(plan->ldy) * 4u) % 16u == 0;
  plan->use_tma_store = aligned ? 1 : 0;
  if (aligned) {
    return encode_tensor_map_2d(&plan->tm_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, y, plan->M, plan->N,
                                static_cast<uint64_t>(plan->ldy) * 4u, 32, 16);
  }
  // a valid (unused) map keeps the kernel's prefetch harmless
  plan->tm_y = plan->tm_a;
  return 0;
}

int finish_plan(GemmPlan* plan, int block_n) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  plan->block_n = block_n;
  const long tiles = static_cast<long>((plan->M + 127) / 128) * ((plan->N + block_n - 1) / block_n);
  plan->grid = static_cast<int>(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  plan->status = ctx->status;
  return 0;
}

}  // namespace

int plan_o0(GemmPlan* plan, const void* a_fp16, const void* w_fp16, float* y, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  *plan = GemmPlan{};
  plan->variant = 0;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  const int block_n = N > 128 ? 256 : 128;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a_fp16, M, K,
                                    static_cast<uint64_t>(K) * 2, 128, 64))
    return rc;
  if (pair_enabled(0, M, N, K, ctx->sm_count)) {
    if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w_fp16, N, K,
                                      static_cast<uint64_t>(K) * 2, pair_tile_n() / 2, 64))
      return rc;
    if (int rc = plan_output(plan, y)) return rc;
    return finish_pair_plan(plan, ctx->sm_count, ctx->status);
  }
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w_fp16, N, K,
                                    static_cast<uint64_t>(K) * 2, block_n, 64))
    return rc;
  if (int rc = plan_output(plan, y)) return rc;
  return finish_plan(plan, block_n);
}

// O1 straight from the packed MXFP4 weights (no INT8 image): only the decode kernel expands nibbles itself.
int plan_o1_packed(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_scale, float* y,
                   int M, int N, int K, int ldy) {
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (!o1_decode_applies(M, N, ctx->sm_count))
    return fail("O1 on packed weights is the decode kernel's form (M <= 8, or M <= 16 while N/32 does not exceed the SM "
                "count); convert W with adg_mxfp4_to_int8 and use adg_gemm_o1 for this shape");
  return plan_o1_decode(plan, a_int8, a_scale, w_mxfp4, w_scale, y, M, N, K, ldy, true);
}

int plan_o1(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, float* y,
            int32_t* partial_dump, int M, int N, int K, int ldy) {
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (partial_dump == nullptr && o1_decode_applies(M, N, ctx->sm_count))
    return plan_o1_decode(plan, a_int8, a_scale, w_int8, w_scale, y, M, N, K, ldy, false);
  if (M <= 64 && partial_dump == nullptr) return plan_o1_skinny(plan, a_int8, a_scale, w_int8, w_scale, y, M, N, K, ldy);
  return plan_o1_tiled(plan, a_int8, a_scale, w_int8, w_scale, y, partial_dump, M, N, K, ldy);
}

int plan_o1_tiled(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale,
                  float* y, int32_t* partial_dump, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  *plan = GemmPlan{};
  plan->variant = 1;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->w_scale = w_scale;
  plan->partial_dump = partial_dump;
  plan->y = y;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_int8, M, K, K, 128, 128)) return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_int8, N, K, K, o1_block_n(), 128))
    return rc;
  plan->tm_y = plan->tm_a;
  if (int rc = finish_plan(plan, o1_block_n())) return rc;
  const long tiles = static_cast<long>((M + 127) / 128) * ((N + o1_block_n() - 1) / o1_block_n());
  const long resident = static_cast<long>(ctx->sm_count) * o1_ctas_per_sm();
  plan->grid = static_cast<int>(tiles < resident ? tiles : resident);
  return 0;
}

int plan_o1_bf16(GemmPlan* plan, const void* a_bf16, const void* a_scale, const void* w_bf16, float* y,
                 const void* range_flag, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  *plan = GemmPlan{};
  plan->variant = 1;
  plan->o1_bf16 = 1;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->range_flag = static_cast<const uint32_t*>(range_flag);
  plan->y = y;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16, M, K,
                                    static_cast<uint64_t>(K) * 2, 128, 64))
    return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_bf16, N, K,
                                    static_cast<uint64_t>(K) * 2, o1_bf16_block_n(), 64))
    return rc;
  plan->tm_y = plan->tm_a;
  return finish_plan(plan, o1_bf16_block_n());
}

int plan_o2(GemmPlan* plan, const void* a_mxfp4, const void* sfa_tiled, const void* w_mxfp4, const void* sfb_tiled,
            float* y, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  if ((reinterpret_cast<uintptr_t>(sfa_tiled) & 15u) != 0 || (reinterpret_cast<uintptr_t>(sfb_tiled) & 15u) != 0)
    return fail("tiled scale buffers must be 16-byte aligned");
  if (M <= 64) return plan_o2_skinny(plan, a_mxfp4, sfa_tiled, w_mxfp4, sfb_tiled, y, M, N, K, ldy);
  *plan = GemmPlan{};
  plan->variant = 2;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->sfa = sfa_tiled;
  plan->sfb = sfb_tiled;
  const int block_n = N > 128 ? 256 : 128;
  const uint64_t kbytes = static_cast<uint64_t>(K) / 2;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_mxfp4, M, kbytes, kbytes, 128, 128))
    return rc;
  if (pair_enabled(2, M, N, K, ctx->sm_count)) {
    if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_mxfp4, N, kbytes, kbytes,
                                      pair_tile_n() / 2, 128))
      return rc;
    // tiled scales: [row block of 128][atoms along K][512 bytes]; a 256-element K slab is two atoms
    const uint64_t row_bytes = static_cast<uint64_t>(((K / 32 + 7) / 8) * 2) * 512u;
    if (int rc = encode_word_map_2d(&plan->tm_sfa, sfa_tiled, (M + 127) / 128, row_bytes, 1, 1024)) return rc;
    if (int rc = encode_word_map_2d(&plan->tm_sfb, sfb_tiled, (N + 127) / 128, row_bytes, 2, 1024)) return rc;
    if (int rc = plan_output(plan, y)) return rc;
    return finish_pair_plan(plan, ctx->sm_count, ctx->status);
  }
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_mxfp4, N, kbytes, kbytes, block_n, 128))
    return rc;
  if (int rc = plan_output(plan, y)) return rc;
  return finish_plan(plan, block_n);
}

int plan_o1x(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8x, const void* col_factor, float* y,
             int M, int N, int K, int ldy) {
  if (int rc = check_shape(M, N, K, ldy)) return rc;
  if ((reinterpret_cast<uintptr_t>(a_scale) | reinterpret_cast<uintptr_t>(col_factor)) & 3u)
    return fail("o1x: the factor arrays must be 4-byte aligned");
  *plan = GemmPlan{};
  plan->variant = 3;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->col_factor = col_factor;
  const int block_n = N > 128 ? 256 : 128;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_int8, M, K, K, 128, 128)) return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_int8x, N, K, K, block_n, 128)) return rc;
  if (int rc = plan_output(plan, y)) return rc;
  return finish_plan(plan, block_n);
}

namespace {
int finish_fused(GemmPlan* plan, const void* a_int8, const void* a_scale, void* a_out, void* ready) {
  if (plan->skinny) return fail("the decode-shape kernels do not convert their activations themselves");
  if ((reinterpret_cast<uintptr_t>(a_int8) | reinterpret_cast<uintptr_t>(a_out)) & 15u)
    return fail("A_int8 and the operand workspace must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(a_scale) | reinterpret_cast<uintptr_t>(ready)) & 3u)
    return fail("A_scale and the row counters must be 4-byte aligned");
  if (ready == nullptr) return fail("the row counters must not be NULL");
  plan->fused = 1;
  plan->fused_a_int8 = a_int8;
  plan->a_scale = a_scale;
  plan->fused_a_out = a_out;
  plan->fused_ready = static_cast<uint32_t*>(ready);
  return 0;
}
}  // namespace

int plan_o0_fused(GemmPlan* plan, const void* a_int8, const void* a_scale, void* a_fp16, const void* w_fp16, float* y,
                  void* ready, int M, int N, int K, int ldy) {
  if (int rc = plan_o0(plan, a_fp16, w_fp16, y, M, N, K, ldy)) return rc;
  return finish_fused(plan, a_int8, a_scale, a_fp16, ready);
}

int plan_o2_fused(GemmPlan* plan, const void* a_int8, const void* a_scale, void* a_mxfp4, void* sfa_tiled, void* sf_natural,
                  const void* w_mxfp4, const void* sfb_tiled, float* y, void* ready, int M, int N, int K, int ldy) {
  if (int rc = plan_o2(plan, a_mxfp4, sfa_tiled, w_mxfp4, sfb_tiled, y, M, N, K, ldy)) return rc;
  plan->fused_sf_natural = sf_natural;
  return finish_fused(plan, a_int8, a_scale, a_mxfp4, ready);
}

// The planner's choice for a shape, without buffers: the same rules as plan_o0 / plan_o1 / plan_o2 above.
int plan_info(int variant, int flags, int M, int N, int K, PlanInfo* info) {
  if (info == nullptr) return fail("info must not be NULL");
  if (variant < 0 || variant > 3) return fail("unknown variant");
  if (int rc = check_shape(M, N, K, N)) return rc;
  // the pair rule depends on the SM count: that of the current device, or a B200's 148 without one
  int sm_count = 148;
  DeviceCtx* ctx = nullptr;
  if (device_ctx(&ctx) == 0) sm_count = ctx->sm_count;
  else set_error("");
  *info = PlanInfo{};
  const bool fused = (flags & kPlanFusedActivation) != 0 && M > 64 && (variant == 0 || variant == 2);
  const int block_n = N > 128 ? 256 : 128;
  if (variant == 1) {
    if (!(flags & kPlanPartialDump) && o1_decode_applies(M, N, sm_count)) describe_gemm_o1_decode(M, N, sm_count, info);
    else if (M <= 64 && !(flags & kPlanPartialDump)) describe_gemm_o1_skinny(info);
    else if ((flags & kPlanO1Bf16) && !(flags & kPlanPartialDump)) describe_gemm_o1_bf16(info);
    else describe_gemm_o1(info);
    return 0;
  }
  if (variant == 3) {
    describe_gemm_acc(3, block_n, false, info);
    return 0;
  }
  if (variant == 2 && M <= 64) {
    describe_gemm_o2_skinny(M, info);
    return 0;
  }
  if (pair_enabled(variant, M, N, K, sm_count)) describe_gemm_pair(variant, fused, info);
  else describe_gemm_acc(variant, block_n, fused, info);
  return 0;
}

int run_plan(const GemmPlan& plan, cudaStream_t stream) {
  if (plan.variant == 1 && plan.o1_bf16) return run_gemm_o1_bf16(plan, stream);
  if (plan.variant == 1 && plan.skinny == 2) return run_gemm_o1_decode(plan, stream);
  if (plan.variant == 1) return plan.skinny ? run_gemm_o1_skinny(plan, stream) : run_gemm_o1(plan, stream);
  if (plan.skinny) return run_gemm_o2_skinny(plan, stream);
  if (plan.variant == 3) return run_gemm_acc(plan, stream);
  if (plan.pair) return run_gemm_pair(plan, stream);
  return run_gemm_acc(plan, stream);
}

}  // namespace adg
