// isolated cost of the O1 epilogue arithmetic for one warp (per 32 partials per thread)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ float ue8m0_half_to_float(uint32_t code) {
  return __uint_as_float(code >= 2 ? ((code - 1) << 23) : (code == 1 ? 0x00400000u : 0x00200000u));
}
// variant 0: fused per element; 1: three passes scalar; 2: three passes packed (f32x2)
template <int V>
__global__ void bench(const uint32_t* __restrict__ in, float* out, long long* cyc, int iters, uint32_t codes) {
  uint32_t p[32];
  float acc[32];
  const float a_m = 0.37f + threadIdx.x * 1e-3f;
  for (int j = 0; j < 32; ++j) acc[j] = 0.f;
  long long total = 0;
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int j = 0; j < 32; ++j) p[j] = in[(it * 32 + j) * 32 + (threadIdx.x & 31)];
    // make sure loads are done before timing
    uint32_t chk = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) chk ^= p[j];
    if (chk == 0xdeadbeef) out[0] = 1.f;
    __syncwarp();
    long long t0 = clock64();
    const float s = ue8m0_half_to_float((codes >> (8 * (it & 3))) & 0xFFu);
    if (V == 0) {
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = __fmaf_rn(__fmul_rn(__int2float_rn((int)p[j]), a_m), s, acc[j]);
    } else if (V == 1) {
#pragma unroll
      for (int j = 0; j < 32; ++j) p[j] = __float_as_uint(__int2float_rn((int)p[j]));
#pragma unroll
      for (int j = 0; j < 32; ++j) p[j] = __float_as_uint(__fmul_rn(__uint_as_float(p[j]), a_m));
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = __fmaf_rn(__uint_as_float(p[j]), s, acc[j]);
    } else {
      const float2 a2 = make_float2(a_m, a_m), s2 = make_float2(s, s);
#pragma unroll
      for (int j = 0; j < 32; ++j) p[j] = __float_as_uint(__int2float_rn((int)p[j]));
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float2 u = __fmul2_rn(make_float2(__uint_as_float(p[2 * j]), __uint_as_float(p[2 * j + 1])), a2);
        p[2 * j] = __float_as_uint(u.x); p[2 * j + 1] = __float_as_uint(u.y);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float2 r = __ffma2_rn(make_float2(__uint_as_float(p[2 * j]), __uint_as_float(p[2 * j + 1])), s2, make_float2(acc[2 * j], acc[2 * j + 1]));
        acc[2 * j] = r.x; acc[2 * j + 1] = r.y;
      }
    }
    // consume
    float sink = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) sink += acc[j];
    if (sink == 123.456f) out[1] = sink;
    long long t1 = clock64();
    total += t1 - t0;
  }
  float sum = 0.f;
  for (int j = 0; j < 32; ++j) sum += acc[j];
  out[threadIdx.x + blockIdx.x * blockDim.x] = sum;
  if (threadIdx.x == 0 && blockIdx.x == 0) cyc[0] = total / iters;
}
int main() {
  const int iters = 64;
  uint32_t* in; float* out; long long* cyc;
  cudaMalloc(&in, iters * 32 * 32 * 4); cudaMemset(in, 1, iters * 32 * 32 * 4);
  cudaMalloc(&out, 148 * 1024 * 4); cudaMalloc(&cyc, 8);
  for (int threads : {32, 128, 256, 512}) {
    long long h;
    bench<0><<<148, threads>>>(in, out, cyc, iters, 0x7f807e81u); cudaDeviceSynchronize(); cudaMemcpy(&h, cyc, 8, cudaMemcpyDeviceToHost);
    printf("threads/SM %3d: fused per element %lld", threads, h);
    bench<1><<<148, threads>>>(in, out, cyc, iters, 0x7f807e81u); cudaDeviceSynchronize(); cudaMemcpy(&h, cyc, 8, cudaMemcpyDeviceToHost);
    printf("   three passes scalar %lld", h);
    bench<2><<<148, threads>>>(in, out, cyc, iters, 0x7f807e81u); cudaDeviceSynchronize(); cudaMemcpy(&h, cyc, 8, cudaMemcpyDeviceToHost);
    printf("   three passes packed %lld   cycles per 32 partials per thread (incl. 32-add sink)\n", h);
  }
  return 0;
}
