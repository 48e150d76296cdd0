// issue/throughput of back-to-back tcgen05.mma of various N from 1 or 2 issuing threads
#include <cstdio>
#include <cstdint>
#include "../csrc/common.cuh"
using namespace adg;

// issuers: threads 0 and 32 (if nthr==2). Each issues `count` MMAs to its own TMEM half (256 cols), rotating D.
template <int KIND, int N>
__global__ void __launch_bounds__(128, 1) bench(int count, int nthr, int accum_mode, int same_desc, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_slot;
  for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(&bar[0], 1); mbar_init(&bar[1], 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && w < nthr) {
    const uint64_t adesc = make_desc_sw128(smem_u32(smem));
    const uint64_t bdesc = make_desc_sw128(smem_u32(smem) + 128 * 128);
    constexpr uint32_t idesc = KIND == 0 ? make_idesc(1, kFmtF16, kFmtF16, 128, N) : make_idesc(2, kFmtS8, kFmtS8, 128, N);
    const uint32_t base = tmem + w * 256;
    if (KIND == 0) umma_f16(base, adesc, bdesc, idesc, 0); else umma_i8(base, adesc, bdesc, idesc, 0);
    umma_commit(&bar[w]);
    { int spin = 0; while (!mbar_test_wait(&bar[w], 0) && ++spin < 2000000) {} }
    long long t0 = clock64();
#pragma unroll 4
    for (int i = 0; i < count; ++i) {
      const uint32_t d = base + (i % (256 / N)) * N;
      const uint32_t accum = accum_mode;
      const int ko = same_desc ? 0 : (i & 3) * 2;
      if (KIND == 0) umma_f16(d, adesc + ko, bdesc + ko, idesc, accum);
      else umma_i8(d, adesc + ko, bdesc + ko, idesc, accum);
    }
    long long t_issue = clock64();
    umma_commit(&bar[w]);
    { int spin = 0; while (!mbar_test_wait(&bar[w], 1) && ++spin < 2000000) {} }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[2 * w] = t_issue - t0; out[2 * w + 1] = t1 - t0; }
  }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

template <int KIND, int N> void run(const char* name, long long* out) {
  cudaFuncSetAttribute(bench<KIND, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  for (int nthr = 1; nthr <= 2; ++nthr)
    for (int accum = 0; accum < 2; ++accum) {
      printf("%s N=%d issuers=%d accum=%d :", name, N, nthr, accum);
      for (int c : {4, 16, 64, 256}) {
        bench<KIND, N><<<148, 128, 64 * 1024>>>(c, nthr, accum, 0, out);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf(" ERR %s\n", cudaGetErrorString(e)); return; }
        long long h[4]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
        printf("  n=%d issue %.0f total %.0f /mma", c, (double)h[0] / c, (double)h[1] / c);
        if (nthr == 2) printf(" [t1: %.0f %.0f]", (double)h[2] / c, (double)h[3] / c);
      }
      printf("\n"); fflush(stdout);
    }
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  run<1, 16>("i8 ", out); run<1, 32>("i8 ", out); run<1, 64>("i8 ", out); run<1, 128>("i8 ", out); run<1, 256>("i8 ", out);
  run<0, 16>("f16", out); run<0, 64>("f16", out); run<0, 128>("f16", out); run<0, 256>("f16", out);
  return 0;
}
