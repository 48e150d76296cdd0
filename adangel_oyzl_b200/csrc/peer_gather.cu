// Gathering the ranks' column blocks of Y by reading the peers' memory over NVLink.
//
// The N-sharded GEMM leaves rank r with Y[:, n0_r:n1_r] as a contiguous [M, width_r] buffer.  A
// contiguous [M, N] on every rank is then (world - 1) / world of the matrix per GPU over the links.
// Through a library all-gather that is one collective into a [world, M, width] buffer plus a local
// permute of the whole matrix; here every rank maps the other ranks' blocks into its address space
// (CUDA IPC: one process per GPU on one node) and ONE kernel of its own copies them, row by row, straight
// to their columns of the destination -- plain 16-byte loads from peer memory, no staging buffer, no
// second pass.  The kernel waits for nobody: the caller orders it after every rank's GEMM (a collective
// or a host barrier on the stream) and keeps the blocks unchanged until every rank has finished reading.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <string>

#include "../../include/adangel_b200.h"
#include "convert_device.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kGatherThreads = 256;
constexpr int kGatherUnroll = 4;
constexpr int kGatherCtasPerSm = 8;

struct GatherBlocks {
  const float4* src[ADG_MAX_PEER_BLOCKS];
  uint32_t col4[ADG_MAX_PEER_BLOCKS];    // first destination column / 4
  uint32_t width4[ADG_MAX_PEER_BLOCKS];  // columns / 4
  uint32_t magic[ADG_MAX_PEER_BLOCKS];   // multiply-high reciprocal of width4
  int count;
};

// Block b is a contiguous [M, width] array; element (row, c) goes to y[row * ldy + col + c].
__global__ void __launch_bounds__(kGatherThreads) gather_columns_kernel(const GatherBlocks blocks, float4* __restrict__ y,
                                                                        uint32_t M, uint32_t ldy4) {
  // blockIdx.y = block: all blocks are copied at the same time, so that the local copy of the rank's own block
  // and the loads over the links overlap
  const uint32_t stride = gridDim.x * kGatherThreads;
  const int b = blockIdx.y;
  const float4* __restrict__ src = blocks.src[b];
  const uint32_t w4 = blocks.width4[b], magic = blocks.magic[b];
  const uint32_t total = M * w4;
  float4* dst = y + blocks.col4[b];
  for (uint32_t base = blockIdx.x * kGatherThreads + threadIdx.x; base < total; base += stride * kGatherUnroll) {
    float4 v[kGatherUnroll];
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const uint32_t i = base + u * stride;
      if (i < total) v[u] = __ldcs(src + i);  // read once, over the link: do not keep it in the caches
    }
#pragma unroll
    for (int u = 0; u < kGatherUnroll; ++u) {
      const uint32_t i = base + u * stride;
      if (i < total) {
        const uint32_t row = fast_div(i, w4, magic);
        dst[static_cast<size_t>(row) * ldy4 + (i - row * w4)] = v[u];
      }
    }
  }
}

}  // namespace

}  // namespace adg

using namespace adg;

extern "C" {

int adg_peer_export(const void* ptr, void* handle64, uint64_t* offset) {
  if (ptr == nullptr || handle64 == nullptr || offset == nullptr) return fail("adg_peer_export: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == ADG_PEER_HANDLE_BYTES, "handle size");
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  cudaPointerAttributes attr{};
  if (int rc = check_cuda(cudaPointerGetAttributes(&attr, ptr), "cudaPointerGetAttributes")) return rc;
  if (attr.type != cudaMemoryTypeDevice) return fail("adg_peer_export: not a device pointer");
  // the handle names the whole allocation: find its base
  CUdeviceptr base = 0;
  size_t size = 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (int rc = check_cuda(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres),
                          "cudaGetDriverEntryPoint(cuMemGetAddressRange)"))
    return rc;
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail("adg_peer_export: cuMemGetAddressRange is unavailable");
  if (reinterpret_cast<PFN_cuMemGetAddressRange_v3020>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
    return fail("adg_peer_export: cuMemGetAddressRange failed");
  cudaIpcMemHandle_t handle;
  if (int rc = check_cuda(cudaIpcGetMemHandle(&handle, reinterpret_cast<void*>(base)), "cudaIpcGetMemHandle")) return rc;
  std::memcpy(handle64, &handle, sizeof(handle));
  *offset = static_cast<uint64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return 0;
}

int adg_peer_open(const void* handle64, void** base) {
  if (handle64 == nullptr || base == nullptr) return fail("adg_peer_open: NULL argument");
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle64, sizeof(handle));
  return check_cuda(cudaIpcOpenMemHandle(base, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int adg_peer_close(void* base) {
  if (base == nullptr) return 0;
  return check_cuda(cudaIpcCloseMemHandle(base), "cudaIpcCloseMemHandle");
}

int adg_gather_columns_pull(const adg_peer_blocks* blocks, float* y, int M, int64_t ldy, void* stream) {
  if (blocks == nullptr || y == nullptr) return fail("adg_gather_columns_pull: NULL argument");
  if (blocks->count <= 0 || blocks->count > ADG_MAX_PEER_BLOCKS) return fail("adg_gather_columns_pull: bad block count");
  if (M <= 0 || ldy <= 0 || (ldy & 3) != 0 || (reinterpret_cast<uintptr_t>(y) & 15u) != 0)
    return fail("adg_gather_columns_pull: y must be 16-byte aligned with ldy a multiple of 4");
  GatherBlocks g{};
  g.count = blocks->count;
  uint64_t most = 0;
  for (int b = 0; b < blocks->count; ++b) {
    const int col = blocks->col0[b], width = blocks->width[b];
    if (blocks->src[b] == nullptr || (reinterpret_cast<uintptr_t>(blocks->src[b]) & 15u) != 0)
      return fail("adg_gather_columns_pull: block pointers must be non-NULL and 16-byte aligned");
    if (col < 0 || width <= 0 || (col & 3) != 0 || (width & 3) != 0 || static_cast<int64_t>(col) + width > ldy)
      return fail("adg_gather_columns_pull: block columns must be multiples of 4 inside the row");
    const uint64_t total = static_cast<uint64_t>(M) * static_cast<uint64_t>(width / 4);
    if (total >= (1ull << 31)) return fail("adg_gather_columns_pull: block too large for 32-bit indexing");
    g.src[b] = reinterpret_cast<const float4*>(blocks->src[b]);
    g.col4[b] = static_cast<uint32_t>(col / 4);
    g.width4[b] = static_cast<uint32_t>(width / 4);
    g.magic[b] = width == 4 ? 0xFFFFFFFFu : fast_div_magic(static_cast<uint32_t>(width / 4));
    most = total > most ? total : most;
  }
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  const uint64_t per_wave = static_cast<uint64_t>(kGatherThreads) * kGatherUnroll;
  uint64_t grid = (most + per_wave - 1) / per_wave;
  uint64_t cap = static_cast<uint64_t>(ctx->sm_count) * kGatherCtasPerSm / static_cast<uint64_t>(blocks->count);
  if (cap == 0) cap = 1;
  if (grid > cap) grid = cap;
  gather_columns_kernel<<<dim3(static_cast<unsigned>(grid), static_cast<unsigned>(blocks->count)), kGatherThreads, 0,
                          static_cast<cudaStream_t>(stream)>>>(
      g, reinterpret_cast<float4*>(y), static_cast<uint32_t>(M), static_cast<uint32_t>(ldy / 4));
  return check_cuda(cudaGetLastError(), "gather_columns_kernel launch");
}

}  // extern "C"
