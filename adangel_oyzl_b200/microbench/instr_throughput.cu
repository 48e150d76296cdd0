// micro-benchmark: per-SM throughput of candidate instructions on sm_100a
#include <cstdio>
#include <cuda_runtime.h>
#include <cstdint>
#define ITERS 2048
#define CHAINS 8
template <int OP> __device__ __forceinline__ void op(uint32_t& r, uint32_t c) {
  if (OP == 0) { asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 1) { asm volatile("cvt.rn.f32.s32 %0, %0;" : "+r"(r)); }
  if (OP == 2) { asm volatile("{.reg .b16 lo, hi; .reg .b8 b0,b1; mov.b32 {lo,hi}, %0; cvt.rn.f32.s16 %0, lo;}" : "+r"(r)); }
  if (OP == 3) { asm volatile("cvt.rn.f16x2.f32 %0, %0, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 4) { asm volatile("{.reg .b8 t; .reg .b16 h; cvt.rn.satfinite.e2m1x2.f32 t, %0, %1; mov.b16 h, {t, t}; mov.b32 %0, {h, h};}" : "+r"(r) : "r"(c)); }
  if (OP == 5) { asm volatile("{.reg .b8 lo, hi; .reg .b16 a, b; mov.b32 {a, b}, %0; mov.b16 {lo, hi}, a; cvt.rn.f16x2.e2m1x2 %0, lo;}" : "+r"(r)); }
  if (OP == 6) { asm volatile("prmt.b32 %0, %0, %1, 0x3120;" : "+r"(r) : "r"(c)); }
  if (OP == 8) { asm volatile("{.reg .b16 a, b; mov.b32 {a, b}, %0; cvt.f32.f16 %0, a;}" : "+r"(r)); }
  if (OP == 9) { asm volatile("mul.rn.f16x2 %0, %0, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 10) { asm volatile("add.s32 %0, %0, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 11) { asm volatile("max.f32 %0, %0, %1, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 12) { asm volatile("add.rn.f32 %0, %0, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 13) { asm volatile("{.reg .b16 lo, hi; mov.b32 {lo,hi}, %0; cvt.rn.f32.s8 %0, lo;}" : "+r"(r)); }
  if (OP == 14) { asm volatile("max.f32 %0, %0, %1;" : "+r"(r) : "r"(c)); }
  if (OP == 15) { asm volatile("lop3.b32 %0, %0, %1, %1, 0x96;" : "+r"(r) : "r"(c)); }
}
template <int OP> __global__ void bench(uint32_t* out, uint32_t c) {
  uint32_t r[CHAINS];
  for (int i = 0; i < CHAINS; ++i) r[i] = threadIdx.x * 7 + i + c;
  if (OP == 7) {
    uint64_t q[CHAINS]; uint64_t cc = ((uint64_t)c << 32) | c;
    for (int i = 0; i < CHAINS; ++i) q[i] = ((uint64_t)r[i] << 32) | r[i];
    for (int it = 0; it < ITERS; ++it)
#pragma unroll
      for (int i = 0; i < CHAINS; ++i) asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(q[i]) : "l"(cc));
    for (int i = 0; i < CHAINS; ++i) r[i] = (uint32_t)q[i] ^ (uint32_t)(q[i] >> 32);
  } else {
    for (int it = 0; it < ITERS; ++it)
#pragma unroll
      for (int i = 0; i < CHAINS; ++i) op<OP>(r[i], c);
  }
  uint32_t s = 0;
  for (int i = 0; i < CHAINS; ++i) s ^= r[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}
template <int OP> void run(const char* name, uint32_t* out, double per_op) {
  cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
  const int blocks = 148 * 8, threads = 256;
  bench<OP><<<blocks, threads>>>(out, 0x3f800001u); cudaDeviceSynchronize();
  cudaEventRecord(a); bench<OP><<<blocks, threads>>>(out, 0x3f800001u); cudaEventRecord(b); cudaEventSynchronize(b);
  float ms; cudaEventElapsedTime(&ms, a, b);
  double ops = (double)blocks * threads * ITERS * CHAINS * per_op;
  printf("%-28s %8.3f ms  %8.1f Gop/s  = %6.1f lanes/clk/SM @1.965GHz\n", name, ms, ops / ms / 1e6, ops / (ms * 1e-3) / 148 / 1.965e9);
}
int main() {
  uint32_t* out; cudaMalloc(&out, 148 * 8 * 256 * 4);
  run<0>("fma.f32", out, 1); run<12>("add.f32", out, 1); run<7>("fma.f32x2 (per elem)", out, 2);
  run<10>("add.s32", out, 1); run<15>("lop3", out, 1); run<6>("prmt", out, 1);
  run<1>("cvt.f32.s32", out, 1); run<2>("cvt.f32.s16", out, 1); run<13>("cvt.f32.s8", out, 1);
  run<3>("cvt.f16x2.f32 (per instr)", out, 1); run<4>("cvt.e2m1x2.f32 (per instr)", out, 1);
  run<5>("cvt.f16x2.e2m1x2 (per instr)", out, 1); run<8>("cvt.f32.f16", out, 1);
  run<9>("mul.f16x2 (per instr)", out, 1); run<14>("max.f32", out, 1); run<11>("max.f32 3-input", out, 1);
  return 0;
}
