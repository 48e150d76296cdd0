// bandwidth of tcgen05.ld: shapes 32x32b.x32 vs two 16x256b.x4 (same 32 lanes x 32 columns),
// 1, 2 or 4 blocks requested before each wait; results consumed with static register indices
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
template <int SHAPE, int DEPTH>
__global__ void __launch_bounds__(512, 1) bench(int nwarps, int count, long long* out) {
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  uint32_t acc = 0;
  long long t0 = 0, t1 = 0;
  if (warp < nwarps) {
    const uint32_t base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + (warp >> 2) * 32;
    uint32_t r[DEPTH][32];
    t0 = clock64();
    for (int i = 0; i < count; i += DEPTH) {
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        if (SHAPE == 0) {
          tmem_ld_32x32(base + d * 128, r[d]);
        } else {
          uint32_t (&lo)[16] = *reinterpret_cast<uint32_t (*)[16]>(&r[d][0]);
          uint32_t (&hi)[16] = *reinterpret_cast<uint32_t (*)[16]>(&r[d][16]);
          tmem_ld_16x256b_x4(base + d * 128, lo);
          tmem_ld_16x256b_x4(base + (16u << 16) + d * 128, hi);
        }
      }
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        tmem_wait_ld_for(r[d]);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc ^= r[d][j];
      }
    }
    t1 = clock64();
  }
  if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && warp < nwarps) { out[warp * 2] = t1 - t0; out[warp * 2 + 1] = acc; }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
template <int SHAPE, int DEPTH> void run(long long* out) {
  for (int nw : {1, 4, 8, 16}) {
    const int count = 256;
    bench<SHAPE, DEPTH><<<148, 512>>>(nw, count, out);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return; }
    long long h[32]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    long long mx = 0; for (int w = 0; w < nw; ++w) if (h[2 * w] > mx) mx = h[2 * w];
    printf("%s depth=%d warps=%2d: %.1f cycles per 32x32 block per warp, %.1f B/clk/SM\n", SHAPE ? "2 x 16x256b.x4" : "32x32b.x32    ", DEPTH, nw, (double)mx / count, (double)nw * count * 4096 / mx);
  }
}
int main() {
  long long* out; cudaMalloc(&out, 1024);
  run<0, 1>(out); run<0, 2>(out); run<0, 4>(out);
  run<1, 1>(out); run<1, 2>(out);
  return 0;
}
