// Quantizers of the step in front of the hot path: turning a floating-point activation / weight
// matrix into the prepared sample the GEMM variants consume.  The reference does this on the CPU
// with torch ops (python/adangel/trace/prepare.py:113-114); at the larger benchmark shapes that
// takes minutes and gigabytes of temporaries, so the two quantizers are HBM-bound kernels here.
//
//   quantize_int8_rows   symmetric per-row INT8 (reference python/adangel/quantization/int8.py:6-17):
//                        scale = amax/127 (1 for an all-zero row), q = clamp(rint(x / scale), +-127)
//   quantize_mxfp4       MXFP4 E2M1 codes + one UE8M0 scale per K32 block
//                        (reference python/adangel/quantization/mxfp4.py:147-180): exponent
//                        floor(log2(amax)) - 2 taken exactly from the FP32 bits (what the
//                        reference's scalar helper and CUDA kernel do), x / 2**e (exact),
//                        round-to-nearest-even onto the E2M1 grid, sign bit = (x / 2**e < 0)
//
// Inputs are FP32 or FP16 (the reference's raw traces are FP16 and are widened to FP32 first).
// Both results are bit-identical to the CPU functions for finite inputs; rejecting NaN/Inf is the
// caller's job, as in the reference, where that check is a host-side torch call.
#include <cuda_fp16.h>

#include "codecs.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kRowThreads = 256;
constexpr int kBlockThreads = 256;

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// One CTA per row: pass 1 finds the row's amax, pass 2 (the row is still in L1/L2) quantizes.
// K is a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) quantize_int8_rows_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                                                         float* __restrict__ scale, long k) {
  __shared__ float warp_max[kRowThreads / 32];
  __shared__ float row_scale;
  const long row = blockIdx.x;
  const T* xr = x + row * k;
  float amax = 0.0f;
  for (long i = static_cast<long>(threadIdx.x) * 4; i < k; i += kRowThreads * 4) {
    const float4 v = load4<T>(xr + i);
    amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = warp_max[0];
#pragma unroll
    for (int w = 1; w < kRowThreads / 32; ++w) m = fmaxf(m, warp_max[w]);
    const float s = m == 0.0f ? 1.0f : __fdiv_rn(m, 127.0f);
    row_scale = s;
    scale[row] = s;
  }
  __syncthreads();
  const float s = row_scale;
  uint32_t* qr = reinterpret_cast<uint32_t*>(q + row * k);
  for (long i = static_cast<long>(threadIdx.x) * 4; i < k; i += kRowThreads * 4) {
    const float4 v = load4<T>(xr + i);
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float r = fminf(fmaxf(rintf(__fdiv_rn(f[b], s)), -127.0f), 127.0f);
      word |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xFFu) << (8 * b);
    }
    qr[i >> 2] = word;
  }
}

// One K32 block per thread: 32 values in, 16 bytes of codes and one scale byte out.
template <typename T>
__global__ void __launch_bounds__(kBlockThreads) quantize_mxfp4_kernel(const T* __restrict__ x, uint4* __restrict__ codes,
                                                                       uint8_t* __restrict__ scale_codes, long blocks) {
  const long gid = static_cast<long>(blockIdx.x) * kBlockThreads + threadIdx.x;
  const bool valid = gid < blocks;
  const T* xb = x + (valid ? gid : 0) * 32;
  float v[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 t = load4<T>(xb + 4 * i);
    v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  // exact floor(log2(amax)) - 2 clamped to +-127 (a subnormal amax clamps to -127 either way);
  // an all-zero block uses exponent 0
  int e = 0;
  if (amax != 0.0f) {
    e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 2;
    e = e < -127 ? -127 : e;  // e <= 125 for every finite FP32 amax
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2**-e, exact
  uint32_t o[4];
#pragma unroll
  for (int qd = 0; qd < 4; ++qd) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = qd * 8 + b * 2;
      // the fused add of +0 turns a quotient of -0 into +0, which must encode as code 0
      const float x0 = __fmaf_rn(v[i], inv, 0.0f);
      const float x1 = __fmaf_rn(v[i + 1], inv, 0.0f);
      word |= float2_to_e2m1x2(x0, x1) << (8 * b);
    }
    o[qd] = word;
  }
  if (valid) {
    codes[gid] = make_uint4(o[0], o[1], o[2], o[3]);
    scale_codes[gid] = static_cast<uint8_t>(e + 127);
  }
}

inline unsigned grid_for(long items, int per_block) {
  return static_cast<unsigned>((items + per_block - 1) / per_block);
}

}  // namespace

// dtype: 0 = FP32, 1 = FP16
int launch_quantize_int8_rows(const void* x, int dtype, void* q, void* scale, long rows, long k, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (dtype == 0) {
    quantize_int8_rows_kernel<float><<<static_cast<unsigned>(rows), kRowThreads, 0, stream>>>(
        static_cast<const float*>(x), static_cast<int8_t*>(q), static_cast<float*>(scale), k);
  } else {
    quantize_int8_rows_kernel<__half><<<static_cast<unsigned>(rows), kRowThreads, 0, stream>>>(
        static_cast<const __half*>(x), static_cast<int8_t*>(q), static_cast<float*>(scale), k);
  }
  return static_cast<int>(cudaGetLastError());
}

int launch_quantize_mxfp4(const void* x, int dtype, void* codes, void* scale_codes, long rows, long k,
                          cudaStream_t stream) {
  const long blocks = rows * (k / 32);
  if (blocks == 0) return 0;
  if (dtype == 0) {
    quantize_mxfp4_kernel<float><<<grid_for(blocks, kBlockThreads), kBlockThreads, 0, stream>>>(
        static_cast<const float*>(x), static_cast<uint4*>(codes), static_cast<uint8_t*>(scale_codes), blocks);
  } else {
    quantize_mxfp4_kernel<__half><<<grid_for(blocks, kBlockThreads), kBlockThreads, 0, stream>>>(
        static_cast<const __half*>(x), static_cast<uint4*>(codes), static_cast<uint8_t*>(scale_codes), blocks);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace adg
