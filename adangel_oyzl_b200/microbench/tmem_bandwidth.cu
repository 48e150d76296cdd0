// tcgen05.ld latency and bandwidth
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
__global__ void __launch_bounds__(512, 1) bench(int nwarps, int count, int x16, long long* out) {
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  uint32_t acc = 0;
  long long t0 = 0, t1 = 0;
  if (warp < nwarps) {
    const uint32_t base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + (warp >> 2) * 32;
    uint32_t r[32]; uint32_t r16[16];
    t0 = clock64();
    if (x16) {
      for (int i = 0; i < count; ++i) { tmem_ld_32x16(base + (i & 3) * 128, r16); if ((i & 3) == 3) { tmem_wait_ld_for(r16); acc += r16[i & 15]; } }
      tmem_wait_ld_for(r16); acc += r16[0];
    } else {
      for (int i = 0; i < count; ++i) { tmem_ld_32x32(base + (i & 3) * 128, r); if ((i & 3) == 3) { tmem_wait_ld_for(r); acc += r[i & 31]; } }
      tmem_wait_ld_for(r); acc += r[0];
    }
    t1 = clock64();
  }
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && warp < nwarps) { out[warp * 2] = t1 - t0; out[warp * 2 + 1] = acc; }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; cudaMalloc(&out, 1024);
  for (int x16 = 0; x16 < 2; ++x16)
    for (int nw : {1, 4, 8, 16})
      for (int count : {1, 4, 64, 256}) {
        bench<<<148, 512>>>(nw, count, x16, out);
        if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return 1; }
        long long h[32]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
        long long mx = 0; for (int w = 0; w < nw; ++w) if (h[2 * w] > mx) mx = h[2 * w];
        const double bytes = (double)nw * count * 32 * (x16 ? 16 : 32) * 4;
        printf("x%d warps=%2d count=%3d : %6lld cycles  (%.1f cycles/ld/warp, %.1f B/clk/SM)\n", x16 ? 16 : 32, nw, count, mx, (double)mx / count, bytes / mx);
        fflush(stdout);
      }
  return 0;
}
