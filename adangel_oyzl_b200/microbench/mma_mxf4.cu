// cycles per back-to-back tcgen05.mma kind::mxf4.block_scale (M=128, K=64) for N = 128 and 256, one issuing thread;
// operands and scale factors are zero (shared memory / tensor memory cleared)
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
template <int N>
__global__ void __launch_bounds__(128, 1) bench(int count, int vary_sf, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4 + 2048 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t sbase = smem_u32(smem);
    const uint64_t adesc = make_desc_sw128(sbase);
    const uint64_t bdesc = make_desc_sw128(sbase + 128 * 128);
    // zero scale bytes into tensor-memory columns 256.. (scale code 0 = 2^-127; products are zero anyway)
    for (int c = 0; c < 8; ++c) tmem_cp_32x128b_warpx4(tmem + 256 + c * 4, make_desc_sf(sbase + (128 + 256) * 128 + (c & 3) * 512));
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, 0) && ++spin < 2000000) {} }
    long long t0 = clock64();
#pragma unroll 4
    for (int i = 0; i < count; ++i) {
      const uint32_t sf_id = (i & 1) * 2;
      const uint32_t idesc = make_idesc_mxf4(128, N, sf_id, sf_id);
      const uint32_t sfa = tmem + 256 + (vary_sf ? ((i >> 1) & 1) * 4 : 0);
      const uint32_t sfb = tmem + 256 + 8 + (vary_sf ? ((i >> 1) & 1) * 8 : 0);
      umma_mxf4(tmem, adesc + (i & 3) * 2, bdesc + (i & 3) * 2, idesc, 1u, sfa, sfb);
    }
    long long t_issue = clock64();
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, 1) && ++spin < 4000000) {} }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t_issue - t0; out[1] = t1 - t0; }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}
template <int N> void run(long long* out) {
  cudaFuncSetAttribute(bench<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int vary : {0, 1})
    for (int c : {16, 256}) {
      bench<N><<<148, 128, 64 * 1024>>>(c, vary, out);
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) { printf("ERR %s\n", cudaGetErrorString(e)); return; }
      long long h[2]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
      printf("mxf4.block_scale N=%d vary_sf=%d n=%d: issue %.1f total %.1f cycles per MMA\n", N, vary, c, (double)h[0] / c, (double)h[1] / c);
    }
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  run<128>(out); run<256>(out);
  return 0;
}
