// does a warp that only needs a slot now and then (tcgen05.ld + wait) get starved by warps issuing long
// runs of independent arithmetic on the same scheduler?
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
__global__ void __launch_bounds__(512, 1) bench(int math_warps_per_sched, int run_len, int count, long long* out, float* sink) {
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int done;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) done = 0;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const int sched = warp & 3, slot = warp >> 2;   // 4 warps per scheduler: slot 0 loads, slots 1.. do math
  if (slot == 0) {
    const uint32_t base = tmem + (static_cast<uint32_t>(sched * 32) << 16);
    uint32_t r[32]; uint32_t acc = 0;
    long long t0 = clock64();
    for (int i = 0; i < count; ++i) {
      tmem_ld_32x32(base + (i & 3) * 32, r);
      tmem_wait_ld_for(r);
#pragma unroll
      for (int j = 0; j < 32; ++j) acc ^= r[j];
    }
    long long t1 = clock64();
    if ((threadIdx.x & 31) == 0 && blockIdx.x == 0) { out[sched] = (t1 - t0) / count; out[8 + sched] = acc; }
    __syncwarp();
    if (threadIdx.x == 0) done = 1;
  } else if (slot <= math_warps_per_sched) {
    float a[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = threadIdx.x * 0.001f + j;
    int it = 0;
    while (!done && ++it < 2000000) {
      for (int r = 0; r < run_len; ++r) {
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = __fmaf_rn(a[j], 1.0001f, 0.5f);
      }
    }
    float s = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) s += a[j];
    sink[blockIdx.x * 512 + threadIdx.x] = s;
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; float* sink; cudaMalloc(&out, 256); cudaMalloc(&sink, 148 * 512 * 4);
  for (int mw : {0, 1, 3})
    for (int run : {1, 4}) {
      bench<<<148, 512>>>(mw, run, 512, out, sink);
      if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return 1; }
      long long h[4]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
      printf("math warps per scheduler %d, independent-FMA run %3d instr: tcgen05.ld x32 + wait + 32 xor = %lld cycles per iteration\n", mw, run * 32, h[0]);
      if (mw == 0) break;
    }
  return 0;
}
