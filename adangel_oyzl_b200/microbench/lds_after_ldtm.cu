// is a shared-memory load issued after a tcgen05.ld delayed until the tensor-memory load returns?
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;
__global__ void __launch_bounds__(512, 1) bench(long long* out, int nwarps_loading) {
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) float table[1024];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) table[i] = i * 0.5f;
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t ta = tmem + ((static_cast<uint32_t>(warp & 3) * 32) << 16) + (warp >> 2) * 32;
  uint32_t r[32];
  float acc = 0.f;
  long long t_lds_alone = 0, t_lds_after = 0, t_ld_total = 0;
  const uint32_t tb = smem_u32(table);
  if (warp < nwarps_loading) {
    // warm
    tmem_ld_32x32(ta, r); tmem_wait_ld_for(r); acc += __uint_as_float(r[1]);
    for (int rep = 0; rep < 8; ++rep) {
      __syncwarp();
      long long t0 = clock64();
      float4 s;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w) : "r"(tb + rep * 16));
      acc += s.x + s.y + s.z + s.w;
      asm volatile("" :: "f"(acc));
      long long t1 = clock64();
      // four loads in flight, then the shared-memory load
      tmem_ld_32x32(ta, r);
      long long t2 = clock64();
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w) : "r"(tb + 512 + rep * 16));
      acc += s.x + s.y + s.z + s.w;
      asm volatile("" :: "f"(acc));
      long long t3 = clock64();
      tmem_wait_ld_for(r); acc += __uint_as_float(r[rep]);
      asm volatile("" :: "f"(acc));
      long long t4 = clock64();
      t_lds_alone += t1 - t0; t_lds_after += t3 - t2; t_ld_total += t4 - t2;
    }
    if (lane == 0 && warp == 0 && blockIdx.x == 0) { out[0] = t_lds_alone / 8; out[1] = t_lds_after / 8; out[2] = t_ld_total / 8; out[3] = (long long)acc; }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  for (int nw : {1, 4, 16}) {
    bench<<<148, 512>>>(out, nw);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("ERR\n"); return 1; }
    long long h[4]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    printf("%2d warps: ld.shared alone %lld cycles; ld.shared issued right after a tcgen05.ld %lld cycles; tcgen05.ld issue -> wait::ld done %lld cycles\n", nw, h[0], h[1], h[2]);
  }
  return 0;
}
