// does a tcgen05.commit between groups of MMAs open a bubble in the tensor pipe?
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
template <int N>
__global__ void __launch_bounds__(128, 1) bench(int groups, int per_group, int commit_mode, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_end, bar_sink[8];
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar_end, 1); for (int i = 0; i < 8; ++i) mbar_init(&bar_sink[i], 1000000); fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t adesc = make_desc_sw128(smem_u32(smem));
    const uint64_t bdesc = make_desc_sw128(smem_u32(smem) + 128 * 128);
    constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, 128, N);
    umma_f16(tmem, adesc, bdesc, idesc, 0);
    umma_commit(&bar_end);
    { int spin = 0; while (!mbar_test_wait(&bar_end, 0) && ++spin < 2000000) {} }
    long long t0 = clock64();
    for (int g = 0; g < groups; ++g) {
#pragma unroll 4
      for (int i = 0; i < per_group; ++i) umma_f16(tmem, adesc + (i & 3) * 2, bdesc + (i & 3) * 2, idesc, 1u);
      if (commit_mode == 1) umma_commit(&bar_sink[g & 7]);
      if (commit_mode == 2 && (g & 1)) umma_commit(&bar_sink[g & 7]);
    }
    long long t_issue = clock64();
    umma_commit(&bar_end);
    { int spin = 0; while (!mbar_test_wait(&bar_end, 1) && ++spin < 4000000) {} }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t_issue - t0; out[1] = t1 - t0; }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  cudaFuncSetAttribute(bench<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int mode = 0; mode < 3; ++mode)
    for (int pg : {2, 4, 8}) {
      const int groups = 256 / pg;
      bench<256><<<148, 128, 64 * 1024>>>(groups, pg, mode, out);
      if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return 1; }
      long long h[2]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
      printf("N=256 f16, %d MMAs per group, commit mode %d (0 none, 1 every group, 2 every other): issue %.1f total %.1f cycles per MMA\n",
             pg, mode, (double)h[0] / 256, (double)h[1] / 256);
    }
  return 0;
}
