// adg_o2_linear_noalloc: the O2 activation path (re-quantize A to MXFP4, then the block-scaled
// GEMM) for callers that must not allocate device memory.
//
// Who needs this: a serving process that has handed all of the GPU's memory to its own arena (a
// KV-cache or tensor pool) has nothing left for cudaMalloc to return, and a latency-critical decode
// loop cannot afford cudaMalloc/cudaFree because they synchronise the whole device.  Such callers
// can still run O2 through this entry point: the intermediate buffers that the regular path takes
// from the caller or allocates (packed E2M1 codes of A, A's UE8M0 scales in the tensor core's tiled
// layout, and the kernels' status words) live in one fixed array that is part of the library image.
//
// The array is a file-scope __device__ symbol.  Host code cannot use the symbol's name as an
// address; the device address is looked up with cudaGetSymbolAddress once per device, with that
// device current, and that pointer is what the kernels and tensor maps receive.
#include <cudaTypedefs.h>

#include <mutex>
#include <string>

#include "../../include/adangel_b200.h"
#include "common.cuh"
#include "launch.h"

using namespace adg;

namespace {

constexpr size_t kCodesBytes = size_t(4) << 20;    // packed codes of A: M*K/2 bytes
constexpr size_t kScalesBytes = size_t(512) << 10;  // tiled scales of A
constexpr size_t kStatusBytes = 256;                // kernel status words
constexpr size_t kScratchBytes = kCodesBytes + kScalesBytes + kStatusBytes;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct Setup {
  bool ready = false;
  unsigned char* base = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
Setup g_setup[kMaxDevices];
std::mutex g_mutex;
PFN_cuTensorMapEncodeTiled_v12000 g_encode_fn = nullptr;

// Once per device, with that device current.  Looks up addresses and sets function attributes;
// allocates nothing.
int setup_current_device(Setup** out) {
  int dev = -1;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= kMaxDevices) return fail("device index out of range");
  std::lock_guard<std::mutex> lock(g_mutex);
  Setup& s = g_setup[dev];
  if (!s.ready) {
    int major = 0;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "cudaDeviceGetAttribute"))
      return rc;
    if (major != 10) return fail("adg_o2_linear_noalloc: this library contains sm_100a kernels only");
    if (int rc = check_cuda(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))
      return rc;
    void* ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)")) return rc;
    if (ptr == nullptr) return fail("cudaGetSymbolAddress returned a null scratch address");
    s.base = static_cast<unsigned char*>(ptr);
    if (g_encode_fn == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      if (int rc = check_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres),
                              "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)"))
        return rc;
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail("cuTensorMapEncodeTiled is unavailable");
      g_encode_fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    if (int rc = init_gemm_acc_attributes()) return rc;
    if (int rc = check_cuda(cudaMemset(s.base + kCodesBytes + kScalesBytes, 0, kStatusBytes), "cudaMemset(status)")) return rc;
    s.ready = true;
  }
  *out = &s;
  return 0;
}

int encode_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t rows, uint64_t cols,
               uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail("tensor base address must be 16-byte aligned");
  if ((pitch_bytes & 15u) != 0) return fail("tensor row pitch must be a multiple of 16 bytes");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult res = g_encode_fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   box_cols * (dtype == CU_TENSOR_MAP_DATA_TYPE_FLOAT32 ? 4u : 1u) == 128u ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(res)));
  return 0;
}

// Reads (and, if set, clears) the status words that this entry point's kernels keep in the scratch array.
int read_status(Setup* s, const char* who) {
  uint32_t* status = reinterpret_cast<uint32_t*>(s->base + kCodesBytes + kScalesBytes);
  uint32_t words[4] = {};
  if (int rc = check_cuda(cudaMemcpy(words, status, sizeof(words), cudaMemcpyDeviceToHost), "cudaMemcpy(status)")) return rc;
  if (words[0] == kStatusOk) return 0;
  check_cuda(cudaMemset(status, 0, kStatusBytes), "cudaMemset(status)");
  return fail(std::string(who) + ": kernel wait timeout: code=" + std::to_string(words[0]) + " tag=" + std::to_string(words[1]) +
              " block=" + std::to_string(words[2]));
}

}  // namespace

namespace adg {
// Status of asynchronous adg_o2_linear_noalloc calls on the current device; does nothing (and sets
// nothing up) when the entry point has not been used on this device.
int noalloc_check_status(cudaStream_t stream, bool synchronize) {
  int dev = -1;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= kMaxDevices) return 0;
  Setup* s = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_setup[dev].ready) return 0;
    s = &g_setup[dev];
  }
  if (synchronize)
    if (int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
  return read_status(s, "adg_o2_linear_noalloc");
}
}  // namespace adg

extern "C" int adg_o2_linear_noalloc_status(void* stream) {
  return noalloc_check_status(static_cast<cudaStream_t>(stream), /*synchronize=*/true);
}

extern "C" int adg_o2_linear_noalloc_status_words(void** device_address, int* bytes) {
  Setup* s = nullptr;
  if (int rc = setup_current_device(&s)) return rc;
  if (device_address) *device_address = s->base + kCodesBytes + kScalesBytes;
  if (bytes) *bytes = static_cast<int>(kStatusBytes);
  return 0;
}

extern "C" int adg_o2_linear_noalloc(const void* a_int8, const void* a_scale, const void* w_mxfp4,
                                     const void* w_sf_tiled, float* y, int M, int N, int K, int ldy, void* stream_v,
                                     int synchronize) {
  if (M <= 0 || N <= 0 || K <= 0) return fail("M, N, and K must be positive");
  if (K % 64 != 0) return fail("K must be divisible by 64");
  if (ldy < N) return fail("ldy must be at least N");
  const size_t codes_bytes = static_cast<size_t>(M) * K / 2;
  const size_t scales_bytes = static_cast<size_t>(tiled_scale_bytes(M, K));
  if (codes_bytes > kCodesBytes || scales_bytes > kScalesBytes) {
    return fail("adg_o2_linear_noalloc: activation too large for the built-in scratch (needs " +
                std::to_string(codes_bytes) + " B of codes, limit " + std::to_string(kCodesBytes) + "; " +
                std::to_string(scales_bytes) + " B of tiled scales, limit " + std::to_string(kScalesBytes) +
                "); use adg_o2_quantize_activation + adg_gemm_o2 with caller-provided buffers");
  }
  if ((reinterpret_cast<uintptr_t>(w_sf_tiled) & 15u) != 0) return fail("tiled scale buffers must be 16-byte aligned");
  if (a_int8 == nullptr || a_scale == nullptr || w_mxfp4 == nullptr || y == nullptr) return fail("adg_o2_linear_noalloc: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(a_int8) & 15u) != 0) return fail("A_int8 must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(a_scale) & 3u) != 0) return fail("A_scale must be 4-byte aligned");
  Setup* s = nullptr;
  if (int rc = setup_current_device(&s)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  unsigned char* codes = s->base;
  unsigned char* scales = s->base + kCodesBytes;
  uint32_t* status = reinterpret_cast<uint32_t*>(s->base + kCodesBytes + kScalesBytes);

  // the array keeps whatever the previous call left: the padding of the tiled scales must be zero
  if (int rc = check_cuda(cudaMemsetAsync(scales, 0, scales_bytes, stream), "cudaMemsetAsync(scales)")) return rc;
  if (launch_o2_quantize(a_int8, a_scale, codes, nullptr, scales, M, K, stream)) return fail("o2_quantize launch failed");

  GemmPlan plan;
  plan.variant = 2;
  plan.M = M, plan.N = N, plan.K = K, plan.ldy = ldy;
  plan.sfa = scales;
  plan.sfb = w_sf_tiled;
  plan.y = y;
  plan.status = status;
  plan.block_n = N > 128 ? 256 : 128;
  const uint64_t kbytes = static_cast<uint64_t>(K) / 2;
  if (int rc = encode_map(&plan.tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, codes, M, kbytes, kbytes, 128, 128)) return rc;
  if (int rc = encode_map(&plan.tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, w_mxfp4, N, kbytes, kbytes, plan.block_n, 128))
    return rc;
  const bool aligned = (reinterpret_cast<uintptr_t>(y) & 15u) == 0 && (static_cast<uint64_t>(ldy) * 4u) % 16u == 0;
  plan.use_tma_store = aligned ? 1 : 0;
  if (aligned) {
    if (int rc = encode_map(&plan.tm_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, y, M, N, static_cast<uint64_t>(ldy) * 4u, 32, 16))
      return rc;
  } else {
    plan.tm_y = plan.tm_a;
  }
  const long tiles = static_cast<long>((M + 127) / 128) * ((N + plan.block_n - 1) / plan.block_n);
  plan.grid = static_cast<int>(tiles < s->sm_count ? tiles : s->sm_count);
  if (int rc = run_gemm_acc(plan, stream)) return rc;
  if (!synchronize) return 0;

  if (int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
  return read_status(s, "adg_o2_linear_noalloc");
}
