// extern "C" entry points declared in include/adangel_b200.h: thin wrappers over the launchers, the
// timing harness shared by all three variants, the scale-layout probe and host-buffer sessions.
#include <cmath>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "../../include/adangel_b200.h"
#include "common.cuh"
#include "launch.h"

using namespace adg;

namespace {

cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

int check_conv_dims(int64_t rows, int64_t k) {
  if (rows <= 0 || k <= 0) return fail("rows and K must be positive");
  if (k % 64 != 0) return fail("K must be divisible by 64");
  return 0;
}

// The kernels read and write these buffers with 16-byte vector accesses (4-byte for scale arrays and flag
// words): a misaligned pointer is an error here, not a fault on the device.
int check_ptr(const void* p, unsigned align, const char* name) {
  if (p == nullptr) return fail(std::string(name) + " must not be NULL");
  if ((reinterpret_cast<uintptr_t>(p) & (align - 1u)) != 0)
    return fail(std::string(name) + " must be " + std::to_string(align) + "-byte aligned");
  return 0;
}

int launched(int cuda_rc, const char* what) {
  if (cuda_rc == 0) return 0;
  return fail(std::string(what) + " launch failed: " + cudaGetErrorString(static_cast<cudaError_t>(cuda_rc)));
}

// ---- CUDA event helpers ----------------------------------------------------------------------------
struct EventList {
  std::vector<cudaEvent_t> ev;
  ~EventList() {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
  int grow(size_t n) {
    while (ev.size() < n) {
      cudaEvent_t e;
      if (int rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate")) return rc;
      ev.push_back(e);
    }
    return 0;
  }
};

using Op = std::function<int()>;

// `repeats` intervals of `inner` back-to-back launches each; returns the per-launch average of
// every interval (the reference's isolated batched conversion timing).
int measure_batched(const Op& op, int repeats, int inner, cudaStream_t stream, std::vector<float>* out) {
  EventList events;
  if (int rc = events.grow(2 * static_cast<size_t>(repeats))) return rc;
  for (int it = 0; it < repeats; ++it) {
    if (int rc = check_cuda(cudaEventRecord(events.ev[2 * it], stream), "cudaEventRecord")) return rc;
    for (int i = 0; i < inner; ++i)
      if (int rc = op()) return rc;
    if (int rc = check_cuda(cudaEventRecord(events.ev[2 * it + 1], stream), "cudaEventRecord")) return rc;
  }
  if (int rc = check_cuda(cudaEventSynchronize(events.ev.back()), "batched conversion timing synchronization"))
    return rc;
  out->resize(repeats);
  for (int it = 0; it < repeats; ++it) {
    float ms = 0.f;
    if (int rc = check_cuda(cudaEventElapsedTime(&ms, events.ev[2 * it], events.ev[2 * it + 1]), "cudaEventElapsedTime"))
      return rc;
    (*out)[it] = ms / static_cast<float>(inner);
  }
  return 0;
}

struct DeviceBuffer {
  void* p = nullptr;
  ~DeviceBuffer() {
    if (p) cudaFree(p);
  }
  int alloc(size_t bytes) { return check_cuda(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc"); }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
  }
};

}  // namespace

extern "C" {

int adg_abi_version(void) { return 104; }

const char* adg_last_error(void) { return last_error_cstr(); }

uint32_t adg_capabilities(void) {
  return ADG_CAP_COMPILED_SM100A | ADG_CAP_O0_FP16_TC | ADG_CAP_O1_INT8_TC | ADG_CAP_O2_MXF4_BLOCK_SCALE |
         ADG_CAP_O2_TILED;
}

int adg_device_info(char* name, int name_len, int* cc_major, int* cc_minor, int* sm_count) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  cudaDeviceProp prop;
  if (int rc = check_cuda(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties")) return rc;
  if (name && name_len > 0) {
    std::strncpy(name, prop.name, static_cast<size_t>(name_len) - 1);
    name[name_len - 1] = '\0';
  }
  if (cc_major) *cc_major = prop.major;
  if (cc_minor) *cc_minor = prop.minor;
  if (sm_count) *sm_count = prop.multiProcessorCount;
  return 0;
}

int adg_check_status(void* stream) {
  if (int rc = check_device_status(as_stream(stream))) return rc;
  // asynchronous calls of adg_o2_linear_noalloc keep their status words in that entry point's own array
  return noalloc_check_status(as_stream(stream), /*synchronize=*/false);
}

int adg_plan_info(int variant, int flags, int M, int N, int K, adg_plan_desc* out) {
  if (out == nullptr) return fail("out must not be NULL");
  PlanInfo info;
  if (int rc = plan_info(variant, flags, M, N, K, &info)) return rc;
  std::memset(out, 0, sizeof(*out));
  out->tile_m = info.tile_m, out->tile_n = info.tile_n, out->stages = info.stages;
  out->accumulator_stages = info.acc_stages, out->threads = info.threads, out->cluster = info.cluster;
  out->mma_m = info.mma_m, out->mma_n = info.mma_n, out->mma_k = info.mma_k;
  out->persistent = info.persistent, out->fused_activation = info.fused_activation;
  std::strncpy(out->kernel_symbol, info.symbol, sizeof(out->kernel_symbol) - 1);
  std::strncpy(out->mma_family, info.mma_family, sizeof(out->mma_family) - 1);
  return 0;
}

int adg_mxfp4_to_fp16(const void* w_mxfp4, const void* w_scale, void* out_fp16, int64_t rows, int64_t K, void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(w_mxfp4, 16, "W_mxfp4") || check_ptr(w_scale, 1, "W_scale") || check_ptr(out_fp16, 16, "out_fp16")) return 1;
  return launched(launch_mxfp4_to_fp16(w_mxfp4, w_scale, out_fp16, rows, K, as_stream(stream)), "mxfp4_to_fp16");
}

int adg_int8_to_fp16(const void* a_int8, const void* a_scale, void* out_fp16, int64_t rows, int64_t K, void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(a_int8, 16, "A_int8") || check_ptr(a_scale, 4, "A_scale") || check_ptr(out_fp16, 16, "out_fp16")) return 1;
  return launched(launch_int8_to_fp16(a_int8, a_scale, out_fp16, rows, K, as_stream(stream)), "int8_to_fp16");
}

int adg_mxfp4_to_int8(const void* w_mxfp4, void* out_int8, int64_t rows, int64_t K, void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(w_mxfp4, 16, "W_mxfp4") || check_ptr(out_int8, 16, "out_int8")) return 1;
  return launched(launch_mxfp4_to_int8(w_mxfp4, out_int8, rows, K, as_stream(stream)), "mxfp4_to_int8");
}

int adg_mxfp4_to_bf16_scaled(const void* w_mxfp4, const void* w_scale, void* out_bf16, void* range_flag, int64_t rows,
                             int64_t K, void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(w_mxfp4, 16, "W_mxfp4") || check_ptr(w_scale, 1, "W_scale") || check_ptr(out_bf16, 16, "out_bf16") ||
      check_ptr(range_flag, 4, "range_flag"))
    return 1;
  return launched(launch_mxfp4_to_bf16_scaled(w_mxfp4, w_scale, out_bf16, range_flag, rows, K, as_stream(stream)),
                  "mxfp4_to_bf16_scaled");
}

int adg_int8_to_bf16(const void* a_int8, const void* a_scale, void* out_bf16, void* range_flag, int64_t rows, int64_t K,
                     void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(a_int8, 16, "A_int8") || check_ptr(a_scale, 4, "A_scale") || check_ptr(out_bf16, 16, "out_bf16") ||
      check_ptr(range_flag, 4, "range_flag"))
    return 1;
  return launched(launch_int8_to_bf16(a_int8, a_scale, out_bf16, range_flag, rows, K, as_stream(stream)), "int8_to_bf16");
}

int64_t adg_o2_tiled_scale_bytes(int64_t rows, int64_t K) { return tiled_scale_bytes(rows, K); }

int adg_o2_quantize_activation(const void* a_int8, const void* a_scale, void* a_mxfp4, void* sf_natural,
                               void* sf_tiled, int64_t M, int64_t K, void* stream) {
  if (int rc = check_conv_dims(M, K)) return rc;
  if (check_ptr(a_int8, 16, "A_int8") || check_ptr(a_scale, 4, "A_scale") || check_ptr(a_mxfp4, 16, "A_mxfp4") ||
      check_ptr(sf_tiled, 16, "sf_tiled"))
    return 1;
  if (sf_natural != nullptr && check_ptr(sf_natural, 4, "sf_natural")) return 1;
  return launched(launch_o2_quantize(a_int8, a_scale, a_mxfp4, sf_natural, sf_tiled, M, K, as_stream(stream)), "o2_quantize");
}

int adg_o2_tile_scales(const void* sf_natural, void* sf_tiled, int64_t rows, int64_t K, void* stream) {
  if (int rc = check_conv_dims(rows, K)) return rc;
  if (check_ptr(sf_natural, 1, "sf_natural") || check_ptr(sf_tiled, 16, "sf_tiled")) return 1;
  return launched(launch_o2_tile_scales(sf_natural, sf_tiled, rows, K, as_stream(stream)), "o2_tile_scales");
}

int adg_quantize_int8_per_row(const void* x, int x_dtype, void* q_int8, void* scale, int64_t rows, int64_t K,
                              void* stream) {
  if (rows <= 0 || K <= 0) return fail("rows and K must be positive");
  if (K % 4 != 0) return fail("K must be divisible by 4");
  if (x_dtype != 0 && x_dtype != 1) return fail("x_dtype must be 0 (FP32) or 1 (FP16)");
  if (rows > 0x7fffffffL) return fail("too many rows");
  if (check_ptr(x, 16, "x") || check_ptr(q_int8, 16, "q_int8") || check_ptr(scale, 4, "scale")) return 1;
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  return launched(launch_quantize_int8_rows(x, x_dtype, q_int8, scale, rows, K, as_stream(stream)), "quantize_int8_per_row");
}

int adg_quantize_mxfp4(const void* x, int x_dtype, void* packed, void* scale_codes, int64_t rows, int64_t K,
                       void* stream) {
  if (rows <= 0 || K <= 0) return fail("rows and K must be positive");
  if (K % 32 != 0) return fail("K must be divisible by 32");
  if (x_dtype != 0 && x_dtype != 1) return fail("x_dtype must be 0 (FP32) or 1 (FP16)");
  if (check_ptr(x, 16, "x") || check_ptr(packed, 16, "packed") || check_ptr(scale_codes, 1, "scale_codes")) return 1;
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  return launched(launch_quantize_mxfp4(x, x_dtype, packed, scale_codes, rows, K, as_stream(stream)), "quantize_mxfp4");
}

int adg_gemm_o0(const void* a_fp16, const void* w_fp16, float* y, int M, int N, int K, int ldy, void* stream) {
  GemmPlan plan;
  if (int rc = plan_o0(&plan, a_fp16, w_fp16, y, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int adg_gemm_o1(const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, float* y,
                int32_t* partial_dump, int M, int N, int K, int ldy, void* stream) {
  GemmPlan plan;
  if (int rc = plan_o1(&plan, a_int8, a_scale, w_int8, w_scale, y, partial_dump, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int adg_gemm_o1_packed(const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_scale, float* y, int M, int N,
                       int K, int ldy, void* stream) {
  if (check_ptr(a_int8, 16, "A_int8") || check_ptr(a_scale, 4, "A_scale") || check_ptr(w_mxfp4, 16, "W_mxfp4") ||
      check_ptr(w_scale, 4, "W_scale") || check_ptr(y, 4, "Y"))
    return 1;
  GemmPlan plan;
  if (int rc = plan_o1_packed(&plan, a_int8, a_scale, w_mxfp4, w_scale, y, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int adg_gemm_o1_bf16(const void* a_bf16, const void* a_scale, const void* w_bf16, float* y, const void* range_flag, int M,
                     int N, int K, int ldy, void* stream) {
  GemmPlan plan;
  if (int rc = plan_o1_bf16(&plan, a_bf16, a_scale, w_bf16, y, range_flag, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int adg_o1_linear(const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale, const void* w_bf16,
                  void* a_bf16_workspace, void* flags, float* y, int M, int N, int K, int ldy, void* stream) {
  if (flags == nullptr) return fail("flags must not be NULL");
  cudaStream_t st = as_stream(stream);
  GemmPlan plan;
  if (M <= 64 || w_bf16 == nullptr || a_bf16_workspace == nullptr) {
    if (int rc = plan_o1(&plan, a_int8, a_scale, w_int8, w_scale, y, nullptr, M, N, K, ldy)) return rc;
    return run_plan(plan, st);
  }
  // flags[0]: the weight's word (set once by adg_mxfp4_to_bf16_scaled); flags[1]: this call's word =
  // the weight's bits plus the activation's.  The BF16-operand kernel computes when the call's word is
  // zero and returns at once otherwise; the INT8-operand kernel behind it does the opposite.
  uint32_t* words = static_cast<uint32_t*>(flags);
  if (int rc = check_cuda(cudaMemcpyAsync(words + 1, words, sizeof(uint32_t), cudaMemcpyDeviceToDevice, st), "flag copy")) return rc;
  if (launch_int8_to_bf16(a_int8, a_scale, a_bf16_workspace, words + 1, M, K, st)) return fail("int8_to_bf16 launch failed");
  if (int rc = plan_o1_bf16(&plan, a_bf16_workspace, a_scale, w_bf16, y, words + 1, M, N, K, ldy)) return rc;
  plan.quiet_refusal = 1;
  if (int rc = run_plan(plan, st)) return rc;
  if (int rc = plan_o1(&plan, a_int8, a_scale, w_int8, w_scale, y, nullptr, M, N, K, ldy)) return rc;
  plan.only_if_flag = words + 1;
  return run_plan(plan, st);
}

int adg_gemm_o2(const void* a_mxfp4, const void* a_sf_tiled, const void* w_mxfp4, const void* w_sf_tiled, float* y,
                int M, int N, int K, int ldy, void* stream) {
  GemmPlan plan;
  if (int rc = plan_o2(&plan, a_mxfp4, a_sf_tiled, w_mxfp4, w_sf_tiled, y, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int64_t adg_fused_workspace_bytes(int64_t M) { return 4 * ((M + 127) / 128 + 1); }

int adg_o0_linear(const void* a_int8, const void* a_scale, const void* w_fp16, void* a_fp16_workspace, void* row_counters,
                  float* y, int M, int N, int K, int ldy, void* stream) {
  GemmPlan plan;
  if (M > 64 && row_counters != nullptr) {
    if (int rc = plan_o0_fused(&plan, a_int8, a_scale, a_fp16_workspace, w_fp16, y, row_counters, M, N, K, ldy)) return rc;
    return run_plan(plan, as_stream(stream));
  }
  if (int rc = adg_int8_to_fp16(a_int8, a_scale, a_fp16_workspace, M, K, stream)) return rc;
  if (int rc = plan_o0(&plan, a_fp16_workspace, w_fp16, y, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

int adg_o2_linear(const void* a_int8, const void* a_scale, const void* w_mxfp4, const void* w_sf_tiled, void* a_mxfp4_workspace,
                  void* a_sf_tiled_workspace, void* a_sf_natural, void* row_counters, float* y, int M, int N, int K, int ldy,
                  void* stream) {
  GemmPlan plan;
  if (M > 64 && row_counters != nullptr) {
    if (a_sf_natural != nullptr && check_ptr(a_sf_natural, 4, "a_sf_natural")) return 1;
    if (int rc = plan_o2_fused(&plan, a_int8, a_scale, a_mxfp4_workspace, a_sf_tiled_workspace, a_sf_natural, w_mxfp4,
                               w_sf_tiled, y, row_counters, M, N, K, ldy))
      return rc;
    return run_plan(plan, as_stream(stream));
  }
  if (int rc = adg_o2_quantize_activation(a_int8, a_scale, a_mxfp4_workspace, a_sf_natural, a_sf_tiled_workspace, M, K, stream))
    return rc;
  if (int rc = plan_o2(&plan, a_mxfp4_workspace, a_sf_tiled_workspace, w_mxfp4, w_sf_tiled, y, M, N, K, ldy)) return rc;
  return run_plan(plan, as_stream(stream));
}

// ---- timing harness ----------------------------------------------------------------------------------
int adg_benchmark(adg_bench_args* a) {
  if (a == nullptr) return fail("args must not be NULL");
  if (a->warmup < 0) return fail("warmup must be non-negative");
  if (a->repeats <= 0) return fail("repeats must be positive");
  if (a->conversion_inner_repeats <= 1) return fail("conversion_inner_repeats must exceed one");
  if (a->variant < 0 || a->variant > 3) return fail("unknown variant");
  if (a->mode < 0 || a->mode > 3) return fail("unknown timing mode");
  const int M = a->M, N = a->N, K = a->K;
  if (M <= 0 || N <= 0 || K <= 0) return fail("M, N, and K must be positive");
  if (K % 64 != 0) return fail("K must be divisible by 64");
  cudaStream_t stream = as_stream(a->stream);

  GemmPlan plan, fused_plan;
  Op conv_w, conv_a, gemm;
  bool has_a = true;
  // O0 / O2 in the cold and steady-state modes: the activation conversion runs inside the GEMM kernel
  const bool fused = (a->flags & ADG_BENCH_FUSE_ACTIVATION) != 0 && a->row_counters != nullptr && M > 64 &&
                     (a->variant == 0 || a->variant == 2) && (a->mode == ADG_MODE_COLD || a->mode == ADG_MODE_STEADY_STATE);
  if (a->variant == 3) {
    if (a->o1x_col_factor == nullptr || a->o1x_workspace == nullptr || a->o1x_w_int8 == nullptr)
      return fail("the o1x benchmark needs o1x_col_factor, o1x_workspace and o1x_w_int8");
    conv_w = [&]() {
      if (int rc = launch_mxfp4_to_int8(a->w_mxfp4, a->o1x_w_int8, N, K, stream)) return rc;
      return adg_o1x_prepare_weight(a->w_mxfp4, a->w_scale, a->conv_weight, a->o1x_col_factor, a->o1x_workspace, N, K, stream);
    };
    conv_a = []() { return 0; };
    has_a = false;
  } else if (a->variant == 0) {
    if (int rc = plan_o0(&plan, a->conv_act, a->conv_weight, a->output, M, N, K, N)) return rc;
    if (fused)
      if (int rc = plan_o0_fused(&fused_plan, a->a_int8, a->a_scale, a->conv_act, a->conv_weight, a->output, a->row_counters,
                                 M, N, K, N))
        return rc;
    conv_w = [&]() { return launch_mxfp4_to_fp16(a->w_mxfp4, a->w_scale, a->conv_weight, N, K, stream); };
    conv_a = [&]() { return launch_int8_to_fp16(a->a_int8, a->a_scale, a->conv_act, M, K, stream); };
  } else if (a->variant == 1) {
    bool on_bf16 = a->conv_weight_bf16 != nullptr && a->conv_act_bf16 != nullptr && a->range_flag != nullptr && M > 64;
    if (on_bf16) {
      // decided once, outside every timed region: are the operands inside the BF16-operand kernel's exact range?
      uint32_t flag = 1;
      if (int rc = check_cuda(cudaMemsetAsync(a->range_flag, 0, sizeof(uint32_t), stream), "cudaMemsetAsync")) return rc;
      if (launch_mxfp4_to_bf16_scaled(a->w_mxfp4, a->w_scale, a->conv_weight_bf16, a->range_flag, N, K, stream) ||
          launch_int8_to_bf16(a->a_int8, a->a_scale, a->conv_act_bf16, a->range_flag, M, K, stream))
        return fail("O1 operand conversion launch failed");
      if (int rc = check_cuda(cudaMemcpyAsync(&flag, a->range_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream), "D2H flag"))
        return rc;
      if (int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
      on_bf16 = flag == 0;
    }
    if (on_bf16) {
      if (int rc = plan_o1_bf16(&plan, a->conv_act_bf16, a->a_scale, a->conv_weight_bf16, a->output, a->range_flag, M, N, K, N))
        return rc;
      conv_w = [&]() {
        if (int rc = launch_mxfp4_to_int8(a->w_mxfp4, a->conv_weight, N, K, stream)) return rc;
        return launch_mxfp4_to_bf16_scaled(a->w_mxfp4, a->w_scale, a->conv_weight_bf16, a->range_flag, N, K, stream);
      };
      conv_a = [&]() { return launch_int8_to_bf16(a->a_int8, a->a_scale, a->conv_act_bf16, a->range_flag, M, K, stream); };
      // the reference's O1 has no activation stage (csrc/sm120/o1_gemm.cu:431-566): by default the INT8 -> BF16
      // conversion is part of this build's GEMM stage; ADG_BENCH_O1_SPLIT_ACTIVATION reports it on its own
      has_a = (a->flags & ADG_BENCH_O1_SPLIT_ACTIVATION) != 0;
    } else {
      // (the decode kernel can also read the packed weights themselves, adg_gemm_o1_packed: half the bytes, but
      // 5 - 10 % slower because every thread expands its own nibbles; the reference's contract is the INT8 image)
      if (int rc = plan_o1(&plan, a->a_int8, a->a_scale, a->conv_weight, a->w_scale, a->output, nullptr, M, N, K, N))
        return rc;
      conv_w = [&]() { return launch_mxfp4_to_int8(a->w_mxfp4, a->conv_weight, N, K, stream); };
      conv_a = []() { return 0; };
      has_a = false;
    }
  } else {
    if (int rc = plan_o2(&plan, a->conv_act, a->conv_act_sf_tiled, a->w_mxfp4, a->conv_weight, a->output, M, N, K, N))
      return rc;
    if (fused)
      if (int rc = plan_o2_fused(&fused_plan, a->a_int8, a->a_scale, a->conv_act, a->conv_act_sf_tiled, a->conv_act_sf,
                                 a->w_mxfp4, a->conv_weight, a->output, a->row_counters, M, N, K, N))
        return rc;
    conv_w = [&]() { return launch_o2_tile_scales(a->w_scale, a->conv_weight, N, K, stream); };
    conv_a = [&]() {
      return launch_o2_quantize(a->a_int8, a->a_scale, a->conv_act, a->conv_act_sf, a->conv_act_sf_tiled, M, K, stream);
    };
  }
  const bool o1_folded = a->variant == 1 && plan.o1_bf16 && !has_a && (a->mode == ADG_MODE_COLD || a->mode == ADG_MODE_STEADY_STATE);
  if (a->variant == 3) {
    gemm = [&]() {
      return adg_gemm_o1x(a->a_int8, a->a_scale, a->conv_weight, a->o1x_col_factor, a->o1x_workspace, a->o1x_w_int8,
                          a->w_scale, a->output, M, N, K, N, stream);
    };
  } else if (o1_folded) {
    gemm = [&]() {
      if (int rc = conv_a()) return rc;
      return run_plan(plan, stream);
    };
  } else if (fused) {
    gemm = [&]() { return run_plan(fused_plan, stream); };
  } else {
    gemm = [&]() { return run_plan(plan, stream); };
  }
  const bool a_in_seq = has_a && !fused;  // a fused GEMM stage contains the activation conversion

  // which operations run inside one directly timed iteration
  std::vector<std::pair<uint32_t, Op*>> seq;
  switch (a->mode) {
    case ADG_MODE_CONVERSION_ONLY:
      seq.push_back({ADG_STAGE_WEIGHT, &conv_w});
      if (has_a) seq.push_back({ADG_STAGE_ACTIVATION, &conv_a});
      break;
    case ADG_MODE_COMPUTE_ONLY:
      if (conv_w()) return fail("weight conversion launch failed");
      if (conv_a()) return fail("activation conversion launch failed");
      seq.push_back({ADG_STAGE_GEMM, &gemm});
      break;
    case ADG_MODE_COLD:
      seq.push_back({ADG_STAGE_WEIGHT, &conv_w});
      if (a_in_seq) seq.push_back({ADG_STAGE_ACTIVATION, &conv_a});
      seq.push_back({ADG_STAGE_GEMM, &gemm});
      break;
    default:  // steady state: the weight conversion is cached
      if (conv_w()) return fail("weight conversion launch failed");
      if (a_in_seq) seq.push_back({ADG_STAGE_ACTIVATION, &conv_a});
      seq.push_back({ADG_STAGE_GEMM, &gemm});
      break;
  }

  for (int it = 0; it < a->warmup; ++it)
    for (auto& s : seq)
      if (int rc = (*s.second)()) return rc ? fail(std::string("warm-up launch failed: ") + last_error_cstr()) : 0;
  if (int rc = check_cuda(cudaStreamSynchronize(stream), "warmup synchronization")) return rc;
  if (int rc = check_device_status(stream)) return rc;

  const size_t per_iter = seq.size() + 1;
  EventList events;
  if (int rc = events.grow(per_iter * static_cast<size_t>(a->repeats))) return rc;
  const bool flush = (a->flags & ADG_BENCH_FLUSH_L2) != 0 && a->l2_flush != nullptr && a->l2_flush_bytes > 0;
  for (int it = 0; it < a->repeats; ++it) {
    cudaEvent_t* e = &events.ev[per_iter * it];
    if (flush)
      if (int rc = check_cuda(cudaMemsetAsync(a->l2_flush, it & 0xff, static_cast<size_t>(a->l2_flush_bytes), stream), "L2 flush"))
        return rc;
    if (int rc = check_cuda(cudaEventRecord(e[0], stream), "cudaEventRecord")) return rc;
    for (size_t s = 0; s < seq.size(); ++s) {
      if ((*seq[s].second)()) return fail(std::string("timed launch failed: ") + last_error_cstr());
      if (int rc = check_cuda(cudaEventRecord(e[s + 1], stream), "cudaEventRecord")) return rc;
    }
  }
  if (int rc = check_cuda(cudaEventSynchronize(events.ev.back()), "measurement synchronization")) return rc;

  // conversions are also measured as isolated batches so that event resolution and launch gaps do
  // not dominate microsecond kernels; the direct events above still give the end-to-end totals
  std::vector<float> iso_w, iso_a, iso_all;
  const bool want_w = a->mode == ADG_MODE_CONVERSION_ONLY || a->mode == ADG_MODE_COLD;
  const bool want_a = has_a && a->mode != ADG_MODE_COMPUTE_ONLY;
  if (want_w)
    if (int rc = measure_batched(conv_w, a->repeats, a->conversion_inner_repeats, stream, &iso_w)) return rc;
  if (want_a)
    if (int rc = measure_batched(conv_a, a->repeats, a->conversion_inner_repeats, stream, &iso_a)) return rc;
  if (a->mode == ADG_MODE_CONVERSION_ONLY) {
    Op all = [&]() {
      if (int rc = conv_w()) return rc;
      return has_a ? conv_a() : 0;
    };
    if (int rc = measure_batched(all, a->repeats, a->conversion_inner_repeats, stream, &iso_all)) return rc;
  }

  a->stages_out = ADG_STAGE_TOTAL;
  if (want_w) a->stages_out |= ADG_STAGE_WEIGHT;
  if (want_a) a->stages_out |= ADG_STAGE_ACTIVATION;
  if (a->mode != ADG_MODE_CONVERSION_ONLY) a->stages_out |= ADG_STAGE_GEMM;
  for (int it = 0; it < a->repeats; ++it) {
    cudaEvent_t* e = &events.ev[per_iter * it];
    if (want_w && a->t_weight) a->t_weight[it] = iso_w[it];
    if (want_a && a->t_activation) a->t_activation[it] = iso_a[it];
    if (a->mode == ADG_MODE_CONVERSION_ONLY) {
      if (a->t_total) a->t_total[it] = iso_all[it];
      continue;
    }
    float gemm_ms = 0.f, total_ms = 0.f;
    if (int rc = check_cuda(cudaEventElapsedTime(&gemm_ms, e[seq.size() - 1], e[seq.size()]), "cudaEventElapsedTime"))
      return rc;
    if (int rc = check_cuda(cudaEventElapsedTime(&total_ms, e[0], e[seq.size()]), "cudaEventElapsedTime")) return rc;
    if (a->t_gemm) a->t_gemm[it] = gemm_ms;
    if (a->t_total) a->t_total[it] = total_ms;
  }

  // conversion_only still leaves a valid output behind; this GEMM is not timed
  if (a->mode == ADG_MODE_CONVERSION_ONLY)
    if (int rc = gemm()) return rc;
  return check_device_status(stream);
}

// ---- scale-layout known-answer probe -------------------------------------------------------------------
int adg_verify_layout(int* passed, float* max_abs_error) {
  constexpr int M = 128, N = 256, K = 512;
  constexpr int G = K / 32;
  std::vector<uint8_t> a(static_cast<size_t>(M) * K / 2, 0x11), w(static_cast<size_t>(N) * K / 2, 0x11);  // +0.5
  std::vector<uint8_t> sa(static_cast<size_t>(M) * G), sb(static_cast<size_t>(N) * G);
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < G; ++g) sa[m * G + g] = static_cast<uint8_t>(124 + (m * 7 + g * 3) % 7);
  for (int n = 0; n < N; ++n)
    for (int g = 0; g < G; ++g) sb[n * G + g] = static_cast<uint8_t>(124 + (n * 5 + g) % 7);
  DeviceBuffer da, dw, dsa, dsb, dsa_t, dsb_t, dy;
  const size_t sa_t = tiled_scale_bytes(M, K), sb_t = tiled_scale_bytes(N, K);
  if (da.alloc(a.size()) || dw.alloc(w.size()) || dsa.alloc(sa.size()) || dsb.alloc(sb.size()) || dsa_t.alloc(sa_t) ||
      dsb_t.alloc(sb_t) || dy.alloc(sizeof(float) * M * N))
    return 1;
  if (int rc = check_cuda(cudaMemcpy(da.p, a.data(), a.size(), cudaMemcpyHostToDevice), "cudaMemcpy")) return rc;
  if (int rc = check_cuda(cudaMemcpy(dw.p, w.data(), w.size(), cudaMemcpyHostToDevice), "cudaMemcpy")) return rc;
  if (int rc = check_cuda(cudaMemcpy(dsa.p, sa.data(), sa.size(), cudaMemcpyHostToDevice), "cudaMemcpy")) return rc;
  if (int rc = check_cuda(cudaMemcpy(dsb.p, sb.data(), sb.size(), cudaMemcpyHostToDevice), "cudaMemcpy")) return rc;
  if (int rc = check_cuda(cudaMemset(dy.p, 0xFF, sizeof(float) * M * N), "cudaMemset")) return rc;
  if (launch_o2_tile_scales(dsa.p, dsa_t.p, M, K, nullptr)) return fail("tile_scales launch failed");
  if (launch_o2_tile_scales(dsb.p, dsb_t.p, N, K, nullptr)) return fail("tile_scales launch failed");
  if (int rc = adg_gemm_o2(da.p, dsa_t.p, dw.p, dsb_t.p, static_cast<float*>(dy.p), M, N, K, N, nullptr)) return rc;
  if (int rc = check_device_status(nullptr)) return rc;
  std::vector<float> y(static_cast<size_t>(M) * N);
  if (int rc = check_cuda(cudaMemcpy(y.data(), dy.p, sizeof(float) * M * N, cudaMemcpyDeviceToHost), "cudaMemcpy"))
    return rc;
  float worst = 0.f;
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      double want = 0.0;
      for (int g = 0; g < G; ++g) want += 8.0 * std::ldexp(1.0, sa[m * G + g] + sb[n * G + g] - 254);
      const float got = y[static_cast<size_t>(m) * N + n];
      const float err = std::isfinite(got) ? std::fabs(got - static_cast<float>(want)) : INFINITY;
      worst = std::fmax(worst, err);
    }
  }
  if (max_abs_error) *max_abs_error = worst;
  if (passed) *passed = worst <= 1e-3f ? 1 : 0;
  return 0;
}

// ---- host-buffer sessions ----------------------------------------------------------------------------------
struct adg_session {
  int variant = 0, max_M = 0, N = 0, K = 0;
  cudaStream_t stream = nullptr;
  bool in_flight = false;  // a submitted pass has not been waited for yet
  DeviceBuffer w_raw, w_scale, w_conv, a_raw, a_scale, a_conv, a_sf_tiled, y;
  // O1: the pass runs on BF16 operands (weight scale folded into W, see gemm_o1_bf16.cu) while the
  // operands stay inside that kernel's exact range, and on the INT8 operands otherwise.  The weight's
  // range is known at creation; an activation's is reported by its conversion into `flags` (device,
  // word 0 = weight, word 1 = this pass), copied to `pass_flag` (pinned) behind the GEMM.  The INT8
  // form of W is made on first need (decode-sized M, or a fallback).
  bool w_in_bf16_range = false;
  DeviceBuffer w_bf16, w_int8, flags;
  uint32_t* pass_flag = nullptr;
  bool pass_on_bf16 = false;
  int pass_M = 0;
  float* pass_y_host = nullptr;
};

namespace {

int session_w_int8(adg_session* s) {
  if (s->w_int8.p != nullptr) return 0;
  if (s->w_int8.alloc(static_cast<size_t>(s->N) * s->K)) return 1;
  return launch_mxfp4_to_int8(s->w_raw.p, s->w_int8.p, s->N, s->K, s->stream) ? fail("mxfp4_to_int8 launch failed") : 0;
}

int session_o1_int8_pass(adg_session* s, int M, float* y_host) {
  if (int rc = session_w_int8(s)) return rc;
  GemmPlan plan;
  float* y = static_cast<float*>(s->y.p);
  if (int rc = plan_o1(&plan, s->a_raw.p, s->a_scale.p, s->w_int8.p, s->w_scale.p, y, nullptr, M, s->N, s->K, s->N)) return rc;
  if (int rc = run_plan(plan, s->stream)) return rc;
  return check_cuda(cudaMemcpyAsync(y_host, y, sizeof(float) * M * static_cast<size_t>(s->N), cudaMemcpyDeviceToHost, s->stream),
                    "D2H Y");
}

}  // namespace

int adg_session_create(adg_session** out, int variant, int max_M, int N, int K, const void* w_mxfp4_host,
                       const void* w_scale_host) {
  if (out == nullptr) return fail("out must not be NULL");
  if (variant < 0 || variant > 2) return fail("unknown variant");
  if (max_M <= 0 || N <= 0 || K <= 0 || K % 64 != 0) return fail("invalid session shape");
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  adg_session* s = new adg_session();
  s->variant = variant, s->max_M = max_M, s->N = N, s->K = K;
  const size_t nk = static_cast<size_t>(N) * K, mk = static_cast<size_t>(max_M) * K;
  int rc = check_cuda(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), "cudaStreamCreate");
  rc = rc || s->w_raw.alloc(nk / 2) || s->w_scale.alloc(nk / 32) || s->a_raw.alloc(mk) ||
       s->a_scale.alloc(sizeof(float) * max_M) || s->y.alloc(sizeof(float) * max_M * static_cast<size_t>(N));
  if (!rc) rc = check_cuda(cudaMemcpyAsync(s->w_raw.p, w_mxfp4_host, nk / 2, cudaMemcpyHostToDevice, s->stream), "H2D W");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(s->w_scale.p, w_scale_host, nk / 32, cudaMemcpyHostToDevice, s->stream), "H2D W scale");
  uint32_t w_flag = 1;
  if (!rc) {
    if (variant == 0) {
      rc = s->w_conv.alloc(nk * 2) || s->a_conv.alloc(mk * 2) ||
           launch_mxfp4_to_fp16(s->w_raw.p, s->w_scale.p, s->w_conv.p, N, K, s->stream);
    } else if (variant == 1) {
      rc = s->w_bf16.alloc(nk * 2) || s->a_conv.alloc(mk * 2) || s->flags.alloc(2 * sizeof(uint32_t)) ||
           check_cuda(cudaMallocHost(reinterpret_cast<void**>(&s->pass_flag), sizeof(uint32_t)), "cudaMallocHost") ||
           check_cuda(cudaMemsetAsync(s->flags.p, 0, 2 * sizeof(uint32_t), s->stream), "cudaMemsetAsync") ||
           launch_mxfp4_to_bf16_scaled(s->w_raw.p, s->w_scale.p, s->w_bf16.p, s->flags.p, N, K, s->stream) ||
           check_cuda(cudaMemcpyAsync(&w_flag, s->flags.p, sizeof(uint32_t), cudaMemcpyDeviceToHost, s->stream), "D2H flag");
    } else {
      const size_t sfa = tiled_scale_bytes(max_M, K);
      rc = s->w_conv.alloc(tiled_scale_bytes(N, K)) || s->a_conv.alloc(mk / 2) || s->a_sf_tiled.alloc(sfa) ||
           check_cuda(cudaMemsetAsync(s->a_sf_tiled.p, 0, sfa, s->stream), "cudaMemsetAsync") ||
           launch_o2_tile_scales(s->w_scale.p, s->w_conv.p, N, K, s->stream);
    }
  }
  if (!rc) rc = check_cuda(cudaStreamSynchronize(s->stream), "session synchronization");
  if (!rc && variant == 1) {
    s->w_in_bf16_range = w_flag == 0;
    if (!s->w_in_bf16_range) {
      // this weight always takes the INT8 operands: drop the BF16 copy
      s->w_bf16.release();
      rc = session_w_int8(s) || check_cuda(cudaStreamSynchronize(s->stream), "session synchronization");
    }
  }
  if (rc) {
    adg_session_destroy(s);
    return 1;
  }
  *out = s;
  return 0;
}

int adg_session_submit(adg_session* s, const void* a_int8_host, const void* a_scale_host, int M, float* y_host) {
  if (s == nullptr) return fail("session must not be NULL");
  if (M <= 0 || M > s->max_M) return fail("M exceeds the session's max_M");
  if (s->in_flight) return fail("the session already has a pass in flight: call adg_session_wait first");
  const int N = s->N, K = s->K;
  cudaStream_t st = s->stream;
  if (int rc = check_cuda(cudaMemcpyAsync(s->a_raw.p, a_int8_host, static_cast<size_t>(M) * K, cudaMemcpyHostToDevice, st), "H2D A"))
    return rc;
  if (int rc = check_cuda(cudaMemcpyAsync(s->a_scale.p, a_scale_host, sizeof(float) * M, cudaMemcpyHostToDevice, st), "H2D A scale"))
    return rc;
  GemmPlan plan;
  float* y = static_cast<float*>(s->y.p);
  s->pass_on_bf16 = false;
  if (s->variant == 0) {
    if (launch_int8_to_fp16(s->a_raw.p, s->a_scale.p, s->a_conv.p, M, K, st)) return fail("int8_to_fp16 launch failed");
    if (int rc = plan_o0(&plan, s->a_conv.p, s->w_conv.p, y, M, N, K, N)) return rc;
  } else if (s->variant == 1) {
    if (s->w_in_bf16_range && M > 64) {
      uint32_t* pass_word = static_cast<uint32_t*>(s->flags.p) + 1;
      if (int rc = check_cuda(cudaMemsetAsync(pass_word, 0, sizeof(uint32_t), st), "cudaMemsetAsync")) return rc;
      if (launch_int8_to_bf16(s->a_raw.p, s->a_scale.p, s->a_conv.p, pass_word, M, K, st)) return fail("int8_to_bf16 launch failed");
      if (int rc = plan_o1_bf16(&plan, s->a_conv.p, s->a_scale.p, s->w_bf16.p, y, pass_word, M, N, K, N)) return rc;
      plan.quiet_refusal = 1;
      if (int rc = run_plan(plan, st)) return rc;
      if (int rc = check_cuda(cudaMemcpyAsync(s->pass_flag, pass_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, st), "D2H flag"))
        return rc;
      s->pass_on_bf16 = true;
      s->pass_M = M;
      s->pass_y_host = y_host;
    } else {
      if (int rc = session_o1_int8_pass(s, M, y_host)) return rc;
      s->in_flight = true;
      return 0;
    }
  } else {
    if (launch_o2_quantize(s->a_raw.p, s->a_scale.p, s->a_conv.p, nullptr, s->a_sf_tiled.p, M, K, st))
      return fail("o2_quantize launch failed");
    if (int rc = plan_o2(&plan, s->a_conv.p, s->a_sf_tiled.p, s->w_raw.p, s->w_conv.p, y, M, N, K, N)) return rc;
  }
  if (!s->pass_on_bf16)
    if (int rc = run_plan(plan, st)) return rc;
  if (int rc = check_cuda(cudaMemcpyAsync(y_host, y, sizeof(float) * M * static_cast<size_t>(N), cudaMemcpyDeviceToHost, st), "D2H Y"))
    return rc;
  s->in_flight = true;
  return 0;
}

int adg_session_wait(adg_session* s) {
  if (s == nullptr) return fail("session must not be NULL");
  s->in_flight = false;
  if (int rc = check_device_status(s->stream)) return rc;
  if (s->pass_on_bf16 && *s->pass_flag != 0u) {
    // an activation scale outside the BF16-operand kernel's exact range: that kernel did not
    // compute; run the pass on the INT8 operands (A is still on the device)
    s->pass_on_bf16 = false;
    if (int rc = session_o1_int8_pass(s, s->pass_M, s->pass_y_host)) return rc;
    return check_device_status(s->stream);
  }
  return 0;
}

int adg_session_run(adg_session* s, const void* a_int8_host, const void* a_scale_host, int M, float* y_host) {
  if (int rc = adg_session_submit(s, a_int8_host, a_scale_host, M, y_host)) return rc;
  return adg_session_wait(s);
}

void adg_session_destroy(adg_session* s) {
  if (s == nullptr) return;
  if (s->stream) cudaStreamDestroy(s->stream);
  if (s->pass_flag) cudaFreeHost(s->pass_flag);
  delete s;
}

}  // extern "C"
