// cost of tcgen05.cp (scale-factor copies) next to block-scaled MMAs: per "stage" 4 MMAs (N=256) and ncp copies,
// issued by one thread or by two (copies from a second thread)
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
__global__ void __launch_bounds__(128, 1) bench(int stages, int ncp, int two_threads, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar, bar2;
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4 + 4096 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&bar2, 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sf_s = sbase + (128 + 256) * 128;
  if (threadIdx.x == 0) {
    const uint64_t adesc = make_desc_sw128(sbase);
    const uint64_t bdesc = make_desc_sw128(sbase + 128 * 128);
    for (int c = 0; c < 8; ++c) tmem_cp_32x128b_warpx4(tmem + 256 + c * 4, make_desc_sf(sf_s + (c & 3) * 512));
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, 0) && ++spin < 2000000) {} }
    long long t0 = clock64();
    for (int s = 0; s < stages; ++s) {
      if (!two_threads) {
#pragma unroll 1
        for (int c = 0; c < ncp; ++c) tmem_cp_32x128b_warpx4(tmem + 256 + 32 + ((s & 1) * 6 + c) * 4, make_desc_sf(sf_s + (c & 3) * 512));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t sf_id = (i & 1) * 2;
        const uint32_t idesc = make_idesc_mxf4(128, 256, sf_id, sf_id);
        umma_mxf4(tmem, adesc + i * 2, bdesc + i * 2, idesc, 1u, tmem + 256 + (i >> 1) * 4, tmem + 256 + 8 + (i >> 1) * 8);
      }
    }
    long long t_issue = clock64();
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, 1) && ++spin < 8000000) {} }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t_issue - t0; out[1] = t1 - t0; }
  } else if (threadIdx.x == 32 && two_threads) {
    for (int s = 0; s < stages; ++s) {
#pragma unroll 1
      for (int c = 0; c < ncp; ++c) tmem_cp_32x128b_warpx4(tmem + 256 + 32 + ((s & 1) * 6 + c) * 4, make_desc_sf(sf_s + (c & 3) * 512));
    }
    umma_commit(&bar2);
    { int spin = 0; while (!mbar_test_wait(&bar2, 0) && ++spin < 8000000) {} }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int two : {0, 1})
    for (int ncp : {0, 2, 6}) {
      bench<<<148, 128, 64 * 1024>>>(64, ncp, two, out);
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) { printf("ERR %s\n", cudaGetErrorString(e)); return 1; }
      long long h[2]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
      printf("copies per stage %d, issued by %s: issue %.0f total %.0f cycles per stage of 4 MMAs (N=256)\n", ncp, two ? "a second thread" : "the MMA thread", (double)h[0] / 64, (double)h[1] / 64);
    }
  return 0;
}
