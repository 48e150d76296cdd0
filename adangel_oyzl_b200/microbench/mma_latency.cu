// latency/throughput of tcgen05.mma patterns (single CTA per SM, zero-filled operands)
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;

// mode 0: same D, accumulate=1; mode 1: rotating D (4 x 128 cols), accumulate=0; mode 2: rotating D, accumulate=1
// kind 0: f16 (K=16) ; kind 1: i8 (K=32)
template <int KIND, int N>
__global__ void __launch_bounds__(640, 1) bench(int count, int mode, int commit_each, long long* out, int poll_mode) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint64_t bar2;
  __shared__ volatile int done_flag;
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&bar2, 1); done_flag = 0; fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t adesc = make_desc_sw128(smem_u32(smem));
    const uint64_t bdesc = make_desc_sw128(smem_u32(smem) + 128 * 128);
    constexpr uint32_t idesc = KIND == 0 ? make_idesc(1, kFmtF16, kFmtF16, 128, N) : make_idesc(2, kFmtS8, kFmtS8, 128, N);
    uint32_t parity = 0;
    // warm
    if (KIND == 0) umma_f16(tmem, adesc, bdesc, idesc, 0); else umma_i8(tmem, adesc, bdesc, idesc, 0);
    umma_commit(&bar);
    { int spin = 0; while (!mbar_test_wait(&bar, parity) && ++spin < 2000000) {} }
    parity ^= 1;
    long long t0 = clock64();
    for (int i = 0; i < count; ++i) {
      const uint32_t d = tmem + (mode == 0 ? 0 : (i % (512 / N)) * N);
      const uint32_t accum = mode == 1 ? 0u : 1u;
      if (KIND == 0) umma_f16(d, adesc + (i & 3) * 2, bdesc + (i & 3) * 2, idesc, accum);
      else umma_i8(d, adesc + (i & 3) * 2, bdesc + (i & 3) * 2, idesc, accum);
      if (commit_each == 2) {
        umma_commit(&bar);
        { int spin = 0; while (!mbar_test_wait(&bar, parity) && ++spin < 2000000) {} } parity ^= 1;
      }
    }
    long long t_issue = clock64();
    if (commit_each == 0) umma_commit(&bar);
    if (commit_each == 0) { { int spin = 0; while (!mbar_test_wait(&bar, parity) && ++spin < 2000000) {} } parity ^= 1; }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t_issue - t0; out[1] = t1 - t0; }
    done_flag = 1;
  } else if (threadIdx.x >= 128 && poll_mode != 0) {
    // background pollers: warps 4..19 poll a barrier that never completes
    int it = 0;
    while (!done_flag && ++it < 4000000) {
      if (poll_mode == 1) { if (mbar_test_wait(&bar2, 0)) break; }
      else if (poll_mode == 2) { if (mbar_try_wait(&bar2, 0)) break; }
      else if (poll_mode == 3) { if ((threadIdx.x & 31) == 0) { if (mbar_test_wait(&bar2, 0)) break; } __syncwarp(); }
    }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

template <int KIND, int N> void run(const char* name, long long* out, int poll_mode) {
  cudaFuncSetAttribute(bench<KIND, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int counts[] = {1, 2, 4, 8, 32, 128};
  for (int mode = 1; mode < 2; ++mode)
    for (int ce = 0; ce < 3; ce += 2) {
      printf("%s poll=%d mode=%d commit=%d :", name, poll_mode, mode, ce);
      for (int c : counts) {
        bench<KIND, N><<<148, 640, 64 * 1024>>>(c, mode, ce, out, poll_mode);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf(" ERR %s\n", cudaGetErrorString(e)); return; }
        long long h[2]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
        printf("  n=%d total %lld (issue %lld, %.0f/mma)", c, h[1], h[0], (double)h[1] / c);
      }
      printf("\n"); fflush(stdout);
    }
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  for (int pm = 0; pm < 4; ++pm) run<1, 128>("i8  N=128", out, pm);
  return 0;
}
