// Sustained tensor-pipe rate on all SMs: cycles per back-to-back tcgen05.mma (M=128, N=256; kind::f16 and
// kind::mxf4.block_scale) over 8 K and 262 K MMAs per CTA, operands all zero or pseudo-random, on 1 and 148
// CTAs, with the wall time from %globaltimer: separates the pipe's cycle count (constant) from the SM clock the
// power management settles at (which drops with random operands on a full grid).
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
template <int KIND>
__global__ void __launch_bounds__(128, 1) bench(int count, int zero, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int words = (128 + 256) * 128 / 4;
  uint32_t seed = 0x9E3779B9u * (blockIdx.x * 131 + threadIdx.x + 1);
  for (int i = threadIdx.x; i < words; i += blockDim.x) {
    seed = seed * 1664525u + 1013904223u;
    uint32_t v = seed ^ (seed >> 13);
    if (KIND == 0) v &= 0x3BFF3BFFu;  // halves below 1.0 in magnitude: no overflow to inf
    reinterpret_cast<uint32_t*>(smem)[i] = zero ? 0u : v;
  }
  for (int i = threadIdx.x; i < 2048 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[words + i] = zero ? 0u : 0x70717273u + (i & 3) * 0x01010101u;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t sbase = smem_u32(smem);
    const uint64_t adesc = make_desc_sw128(sbase);
    const uint64_t bdesc = make_desc_sw128(sbase + 128 * 128);
    if (KIND == 2) for (int c = 0; c < 8; ++c) tmem_cp_32x128b_warpx4(tmem + 256 + c * 4, make_desc_sf(sbase + (128 + 256) * 128 + (c & 3) * 512));
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, 0) && ++spin < 2000000) {} }
    unsigned long long g0 = gtime();
    long long t0 = clock64();
    uint32_t ph = 1;
    for (int i = 0; i < count; i += 64) {
#pragma unroll 4
      for (int j = 0; j < 64; ++j) {
        // a fresh accumulation every 64 MMAs keeps the values finite
        if (KIND == 2) {
          const uint32_t sf_id = (j & 1) * 2;
          const uint32_t idesc = make_idesc_mxf4(128, 256, sf_id, sf_id);
          umma_mxf4(tmem, adesc + (j & 3) * 2, bdesc + (j & 3) * 2, idesc, j != 0, tmem + 256 + ((j >> 1) & 1) * 4, tmem + 256 + 8 + ((j >> 1) & 1) * 8);
        } else {
          constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, 128, 256);
          umma_f16(tmem, adesc + (j & 3) * 2, bdesc + (j & 3) * 2, idesc, j != 0);
        }
      }
      // keep at most ~128 MMAs in flight
      if ((i & 64) != 0) {
        umma_commit(&bar);
        int spin = 0; while (!mbar_test_wait(&bar, ph) && ++spin < 4000000) {}
        ph ^= 1;
      }
    }
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, ph) && ++spin < 4000000) {} }
    long long t1 = clock64();
    unsigned long long g1 = gtime();
    out[blockIdx.x * 2] = t1 - t0; out[blockIdx.x * 2 + 1] = (long long)(g1 - g0);
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}
template <int KIND> void run(int grid, int count, int zero) {
  long long* out; cudaMalloc(&out, 148 * 16); cudaMemset(out, 0, 148 * 16);
  cudaFuncSetAttribute(bench<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int rep = 0; rep < 2; ++rep) {
    bench<KIND><<<grid, 128, 64 * 1024>>>(count, zero, out);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("ERR %s\n", cudaGetErrorString(e)); return; }
  }
  long long h[296]; cudaMemcpy(h, out, grid * 16, cudaMemcpyDeviceToHost);
  double cyc = 0, ns = 0; for (int b = 0; b < grid; ++b) { cyc += h[2 * b]; ns += h[2 * b + 1]; }
  cyc /= grid; ns /= grid;
  const double flop = (KIND == 2 ? 2.0 * 128 * 256 * 64 : 2.0 * 128 * 256 * 16) * count * grid;
  printf("kind %s grid %d count %d zero %d: %.1f cycles/MMA, %.3f ms, clock %.0f MHz, %.0f TFLOP/s\n", KIND == 2 ? "mxf4" : "f16", grid, count, zero,
         cyc / count, ns * 1e-6, cyc / ns * 1e3, flop / ns * 1e-3);
  cudaFree(out);
}
int main() {
  for (int zero = 1; zero >= 0; --zero)
    for (int grid : {1, 148}) {
      run<0>(grid, 8192, zero); run<0>(grid, 262144, zero);
      run<2>(grid, 8192, zero); run<2>(grid, 262144, zero);
    }
  return 0;
}
