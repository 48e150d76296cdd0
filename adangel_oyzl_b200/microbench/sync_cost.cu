// cost of synchronisation primitives for one warp (optionally with other warps spinning)
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
#define REP16(x) x x x x x x x x x x x x x x x x
__global__ void __launch_bounds__(256, 1) bench(long long* out) {
  __shared__ uint64_t bar_done, bar_big;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { mbar_init(&bar_done, 1); mbar_init(&bar_big, 100000); fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x == 0) mbar_arrive(&bar_done);   // phase 0 of bar_done completes
  __syncthreads();
  const uint32_t tmem = tmem_slot;
  if (warp == 1) {
    const uint32_t bd = smem_u32(&bar_done), bb = smem_u32(&bar_big);
    uint32_t acc = 0;
    uint32_t r[32];
    long long t[12];
    t[0] = clock64();
    REP16(acc += mbar_test_wait_a(bd, 0) ? 1u : 0u;)
    t[1] = clock64();
    REP16(if (lane == 0) mbar_arrive_a(bb);)
    t[2] = clock64();
    REP16(tc_fence_before();)
    t[3] = clock64();
    REP16(tc_fence_after();)
    t[4] = clock64();
    REP16(__syncwarp();)
    t[5] = clock64();
    const uint32_t ta = tmem + ((1u * 32) << 16);
    tmem_ld_32x32(ta, r); tmem_wait_ld_for(r); acc += r[3];
    t[6] = clock64();
    // load issue followed by fence_before + arrive: does the fence wait for the load?
    tmem_ld_32x32(ta, r);
    long long a0 = clock64();
    tc_fence_before();
    if (lane == 0) mbar_arrive_a(bb);
    long long a1 = clock64();
    tmem_wait_ld_for(r); acc += r[5];
    t[7] = clock64();
    // the epilogue's hand-over sequence, 16 times: wait::ld, probe, fence, ld issue, fence, arrive
    tmem_ld_32x32(ta, r);
    t[8] = clock64();
    REP16(tmem_wait_ld_for(r); acc += r[7]; acc += mbar_test_wait_a(bd, 0) ? 1u : 0u; tc_fence_after(); tmem_ld_32x32(ta, r); tc_fence_before(); if (lane == 0) mbar_arrive_a(bb);)
    t[9] = clock64();
    tmem_wait_ld_for(r); acc += r[9];
    if (lane == 0) {
      for (int i = 0; i < 9; ++i) out[i] = t[i + 1] - t[i];
      out[9] = a1 - a0; out[10] = acc;
    }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; cudaMalloc(&out, 256);
  for (int rep = 0; rep < 2; ++rep) {
    bench<<<1, 256>>>(out);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return 1; }
  }
  long long h[11]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  printf("16x test_wait(ready)      : %lld (%.0f each)\n", h[0], h[0] / 16.0);
  printf("16x arrive (lane 0)       : %lld (%.0f each)\n", h[1], h[1] / 16.0);
  printf("16x tcgen05.fence::before : %lld (%.0f each)\n", h[2], h[2] / 16.0);
  printf("16x tcgen05.fence::after  : %lld (%.0f each)\n", h[3], h[3] / 16.0);
  printf("16x __syncwarp            : %lld (%.0f each)\n", h[4], h[4] / 16.0);
  printf("ld x32 + wait::ld         : %lld\n", h[5]);
  printf("ld issue; [fence_before+arrive = %lld]; wait::ld : total %lld\n", h[9], h[6]);
  printf("16x hand-over sequence    : %lld (%.0f each)\n", h[8], h[8] / 16.0);
  return 0;
}
