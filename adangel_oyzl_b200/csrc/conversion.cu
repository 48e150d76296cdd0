// HBM-bound conversion kernels of the O0/O1/O2 path, written for sm_100a.
//
// Each kernel streams its input once with coalesced vector loads and writes its output once with
// coalesced 16-byte stores; several independent loads per thread are kept in flight.
//
//   mxfp4_to_fp16      O0 weight conversion    (reference csrc/sm120/conversion.cu:10-23)
//   int8_to_fp16       O0 activation conversion (reference csrc/sm120/conversion.cu:25-37)
//   mxfp4_to_int8      O1 weight conversion    (reference csrc/sm120/conversion.cu:39-50)
//   mxfp4_to_bf16_scaled / int8_to_bf16   operands of the O1 kernel that takes the weight scale through the
//                      tensor core (gemm_o1_bf16.cu); no reference counterpart
//   o2_quantize        O2 activation re-quantization fused with the scale-factor re-layout
//                      (reference csrc/sm120/o2_cutlass.cu:207-259 and :261-274)
//   o2_tile_scales     O2 weight-scale re-layout (reference csrc/sm120/o2_cutlass.cu:261-274)
#include <cuda_bf16.h>

#include "codecs.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// ---- O0 weight: packed E2M1 + UE8M0 -> FP16 -------------------------------------------------
// One 32-bit word (8 elements) per thread per step; `words` = rows*K/8.  The scale of word i is
// scales[i / 4] because both tensors are contiguous and K is a multiple of 32.
__global__ void __launch_bounds__(kThreads) mxfp4_to_fp16_kernel(const uint32_t* __restrict__ packed,
                                                                 const uint8_t* __restrict__ scales,
                                                                 uint4* __restrict__ out, long words) {
  const long base = (static_cast<long>(blockIdx.x) * kUnroll) * kThreads + threadIdx.x;
  uint32_t w[kUnroll];
  uint32_t sc[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i < words) {
      w[u] = __ldg(packed + i);
      sc[u] = __ldg(scales + (i >> 2));
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i >= words) continue;
    const int k = static_cast<int>(sc[u]) - 127;
    __half2 h[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) h[b] = e2m1x2_to_half2((w[u] >> (8 * b)) & 0xFFu);
    if (k >= -23 && k <= 13) {
      // every product is exactly representable in FP16, so one FP16 multiply equals
      // round_to_half(fp32 product)
      const __half2 s2 = __half2half2(__ushort_as_half(
          k >= -14 ? static_cast<unsigned short>((k + 15) << 10) : static_cast<unsigned short>(1u << (k + 24))));
#pragma unroll
      for (int b = 0; b < 4; ++b) h[b] = __hmul2(h[b], s2);
    } else {
      const float s = ue8m0_to_float(sc[u]);
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float2 f = __half22float2(h[b]);
        h[b] = __floats2half2_rn(f.x * s, f.y * s);
      }
    }
    uint4 v;
    v.x = *reinterpret_cast<uint32_t*>(&h[0]);
    v.y = *reinterpret_cast<uint32_t*>(&h[1]);
    v.z = *reinterpret_cast<uint32_t*>(&h[2]);
    v.w = *reinterpret_cast<uint32_t*>(&h[3]);
    out[i] = v;
  }
}

// ---- O0 activation: INT8 * row scale -> FP16 --------------------------------------------------
// Eight elements (one 64-bit load, one 128-bit store) per thread per step; `oct` = rows*K/8.
__global__ void __launch_bounds__(kThreads) int8_to_fp16_kernel(const uint2* __restrict__ in,
                                                                const float* __restrict__ row_scale,
                                                                uint4* __restrict__ out, long octs, int octs_per_row) {
  const long base = (static_cast<long>(blockIdx.x) * kUnroll) * kThreads + threadIdx.x;
  uint2 v[kUnroll];
  float s[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i < octs) {
      v[u] = __ldg(in + i);
      s[u] = __ldg(row_scale + i / octs_per_row);
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i >= octs) continue;
    uint32_t o[4];
    float lo[4], hi[4];
    int8x4_to_float4(v[u].x, lo);
    int8x4_to_float4(v[u].y, hi);
    const __half2 h0 = __floats2half2_rn(lo[0] * s[u], lo[1] * s[u]);
    const __half2 h1 = __floats2half2_rn(lo[2] * s[u], lo[3] * s[u]);
    const __half2 h2 = __floats2half2_rn(hi[0] * s[u], hi[1] * s[u]);
    const __half2 h3 = __floats2half2_rn(hi[2] * s[u], hi[3] * s[u]);
    o[0] = *reinterpret_cast<const uint32_t*>(&h0);
    o[1] = *reinterpret_cast<const uint32_t*>(&h1);
    o[2] = *reinterpret_cast<const uint32_t*>(&h2);
    o[3] = *reinterpret_cast<const uint32_t*>(&h3);
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- O1 (BF16 operands) weight: packed E2M1 + UE8M0 -> BF16 of e2m1 * 2^(scale-127) ------------
// Exact: the value has two significant bits.  One 32-bit word (8 elements) per thread per step.
// A scale code outside [kO1MinScaleCode, kO1MaxScaleCode] sets bit 0 of *range_flag.
__global__ void __launch_bounds__(kThreads) mxfp4_to_bf16_scaled_kernel(const uint32_t* __restrict__ packed,
                                                                        const uint8_t* __restrict__ scales,
                                                                        uint4* __restrict__ out, long words,
                                                                        uint32_t* __restrict__ range_flag) {
  const long base = (static_cast<long>(blockIdx.x) * kUnroll) * kThreads + threadIdx.x;
  bool bad = false;
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i >= words) continue;
    const uint32_t w = __ldg(packed + i);
    const uint32_t code = __ldg(scales + (i >> 2));
    bad |= code < kO1MinScaleCode || code > kO1MaxScaleCode;
    const float s = __uint_as_float((code == 0u ? 1u : code) << 23);  // 2^(code-127); unused when out of range
    uint32_t o[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float2 f = __half22float2(e2m1x2_to_half2((w >> (8 * b)) & 0xFFu));
      const __nv_bfloat162 v = __floats2bfloat162_rn(f.x * s, f.y * s);
      o[b] = *reinterpret_cast<const uint32_t*>(&v);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(range_flag, 1u);
}

// ---- O1 (BF16 operands) activation: INT8 -> BF16 of the integer itself, exact ------------------
// Eight elements per thread per step.  The first `rows` threads of the grid also check the row
// scales: one outside [2^kO1MinAScaleExp, 2^kO1MaxAScaleExp] (or not finite) sets bit 1 of *range_flag.
__global__ void __launch_bounds__(kThreads) int8_to_bf16_kernel(const uint2* __restrict__ in,
                                                                const float* __restrict__ row_scale,
                                                                uint4* __restrict__ out, long octs, long rows,
                                                                uint32_t* __restrict__ range_flag) {
  const long base = (static_cast<long>(blockIdx.x) * kUnroll) * kThreads + threadIdx.x;
  uint2 v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i < octs) v[u] = __ldg(in + i);
  }
  bool bad = false;
  const long gid = static_cast<long>(blockIdx.x) * kThreads + threadIdx.x;
  if (gid < rows) {
    const float s = __ldg(row_scale + gid);
    bad = !(s >= exp2f(static_cast<float>(kO1MinAScaleExp)) && s <= exp2f(static_cast<float>(kO1MaxAScaleExp)));
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i >= octs) continue;
    float lo[4], hi[4];
    int8x4_to_float4(v[u].x, lo);
    int8x4_to_float4(v[u].y, hi);
    const __nv_bfloat162 b0 = __floats2bfloat162_rn(lo[0], lo[1]);
    const __nv_bfloat162 b1 = __floats2bfloat162_rn(lo[2], lo[3]);
    const __nv_bfloat162 b2 = __floats2bfloat162_rn(hi[0], hi[1]);
    const __nv_bfloat162 b3 = __floats2bfloat162_rn(hi[2], hi[3]);
    out[i] = make_uint4(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1),
                        *reinterpret_cast<const uint32_t*>(&b2), *reinterpret_cast<const uint32_t*>(&b3));
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(range_flag, 2u);
}

// ---- O1 weight: packed E2M1 -> INT8 (2*E2M1) ---------------------------------------------------
// Sixteen elements (64-bit load, 128-bit store) per thread per step; `pairs` = rows*K/16.
__global__ void __launch_bounds__(kThreads) mxfp4_to_int8_kernel(const uint2* __restrict__ packed,
                                                                 uint4* __restrict__ out, long pairs) {
  const long base = (static_cast<long>(blockIdx.x) * kUnroll) * kThreads + threadIdx.x;
  uint2 v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i < pairs) v[u] = __ldg(packed + i);
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const long i = base + static_cast<long>(u) * kThreads;
    if (i >= pairs) continue;
    uint4 o;
    e2m1x8_to_int8x8(v[u].x, o.x, o.y);
    e2m1x8_to_int8x8(v[u].y, o.z, o.w);
    out[i] = o;
  }
}

// ---- O2 activation: INT8 * row scale -> MXFP4 codes + UE8M0 scales -------------------------------
// One K32 block per thread: 32 bytes in, 16 bytes of packed codes out, one scale byte written to
// the natural [M, K/32] array (optional) and to the 512-byte-atom layout the tensor core reads.
__device__ __forceinline__ long tiled_sf_offset(int row, int g, int katoms) {
  return (static_cast<long>(row >> 7) * katoms + (g >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (g & 3);
}

__global__ void __launch_bounds__(kThreads) o2_quantize_kernel(const uint4* __restrict__ in,
                                                               const float* __restrict__ row_scale,
                                                               uint4* __restrict__ codes, uint8_t* __restrict__ sf_natural,
                                                               uint8_t* __restrict__ sf_tiled, long blocks, int groups,
                                                               int katoms) {
  const long gid = static_cast<long>(blockIdx.x) * kThreads + threadIdx.x;
  const bool valid = gid < blocks;
  const long g_safe = valid ? gid : 0;
  const int row = static_cast<int>(g_safe / groups);
  const int g = static_cast<int>(g_safe - static_cast<long>(row) * groups);
  const uint4 lo = __ldg(in + 2 * g_safe);
  const uint4 hi = __ldg(in + 2 * g_safe + 1);
  const float s = __ldg(row_scale + row);
  const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  float v[32];
  float amax = 0.0f;
#pragma unroll
  for (int wi = 0; wi < 8; ++wi) {
    float f[4];
    int8x4_to_float4(words[wi], f);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      v[wi * 4 + b] = f[b] * s;
      amax = fmaxf(amax, fabsf(v[wi * 4 + b]));
    }
  }
  // exact floor(log2(amax)) - 2, clamped; an all-zero block uses exponent 0
  int e = 0;
  if (amax != 0.0f) {
    e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 2;
    e = e < -127 ? -127 : (e > 127 ? 127 : e);
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2**-e, exact
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = q * 8 + b * 2;
      // the fused add of +0 turns a product of -0 into +0, which must encode as code 0
      const float x0 = __fmaf_rn(v[i], inv, 0.0f);
      const float x1 = __fmaf_rn(v[i + 1], inv, 0.0f);
      word |= float2_to_e2m1x2(x0, x1) << (8 * b);
    }
    o[q] = word;
  }
  if (valid) codes[gid] = make_uint4(o[0], o[1], o[2], o[3]);
  const uint32_t code = static_cast<uint32_t>(e + 127);
  if ((groups & 3) == 0) {
    // four consecutive lanes hold the four blocks of one tiled-layout word: gather and store once
    uint32_t packed = code | (__shfl_down_sync(0xffffffffu, code, 1) << 8);
    packed |= __shfl_down_sync(0xffffffffu, packed, 2) << 16;
    if (valid && (threadIdx.x & 3) == 0) {
      if (sf_natural != nullptr) *reinterpret_cast<uint32_t*>(sf_natural + gid) = packed;
      *reinterpret_cast<uint32_t*>(sf_tiled + tiled_sf_offset(row, g, katoms)) = packed;
    }
  } else if (valid) {
    if (sf_natural != nullptr) sf_natural[gid] = static_cast<uint8_t>(code);
    sf_tiled[tiled_sf_offset(row, g, katoms)] = static_cast<uint8_t>(code);
  }
}

// ---- O2 weight scales: natural [rows, K/32] -> 512-byte atoms, zero padding included -----------
// One thread per (padded row, K-atom of 4 blocks).
__global__ void __launch_bounds__(kThreads) o2_tile_scales_kernel(const uint8_t* __restrict__ natural,
                                                                  uint32_t* __restrict__ tiled, int rows, int groups,
                                                                  int padded_rows, int katoms) {
  const long idx = static_cast<long>(blockIdx.x) * kThreads + threadIdx.x;
  if (idx >= static_cast<long>(padded_rows) * katoms) return;
  const int row = static_cast<int>(idx / katoms);
  const int ka = static_cast<int>(idx - static_cast<long>(row) * katoms);
  uint32_t word = 0;
  if (row < rows) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int g = ka * 4 + b;
      if (g < groups) word |= static_cast<uint32_t>(__ldg(natural + static_cast<long>(row) * groups + g)) << (8 * b);
    }
  }
  tiled[tiled_sf_offset(row, ka * 4, katoms) >> 2] = word;
}

inline unsigned grid_for(long items, int per_block) {
  return static_cast<unsigned>((items + per_block - 1) / per_block);
}

}  // namespace

int launch_mxfp4_to_fp16(const void* packed, const void* scales, void* out, long rows, long k, cudaStream_t stream) {
  const long words = rows * k / 8;
  if (words == 0) return 0;
  mxfp4_to_fp16_kernel<<<grid_for(words, kThreads * kUnroll), kThreads, 0, stream>>>(
      static_cast<const uint32_t*>(packed), static_cast<const uint8_t*>(scales), static_cast<uint4*>(out), words);
  return static_cast<int>(cudaGetLastError());
}

int launch_int8_to_fp16(const void* in, const void* row_scale, void* out, long rows, long k, cudaStream_t stream) {
  const long octs = rows * k / 8;
  if (octs == 0) return 0;
  int8_to_fp16_kernel<<<grid_for(octs, kThreads * kUnroll), kThreads, 0, stream>>>(
      static_cast<const uint2*>(in), static_cast<const float*>(row_scale), static_cast<uint4*>(out), octs,
      static_cast<int>(k / 8));
  return static_cast<int>(cudaGetLastError());
}

int launch_mxfp4_to_bf16_scaled(const void* packed, const void* scales, void* out, void* range_flag, long rows, long k,
                                cudaStream_t stream) {
  const long words = rows * k / 8;
  if (words == 0) return 0;
  mxfp4_to_bf16_scaled_kernel<<<grid_for(words, kThreads * kUnroll), kThreads, 0, stream>>>(
      static_cast<const uint32_t*>(packed), static_cast<const uint8_t*>(scales), static_cast<uint4*>(out), words,
      static_cast<uint32_t*>(range_flag));
  return static_cast<int>(cudaGetLastError());
}

int launch_int8_to_bf16(const void* in, const void* row_scale, void* out, void* range_flag, long rows, long k,
                        cudaStream_t stream) {
  const long octs = rows * k / 8;
  if (octs == 0) return 0;
  // K >= 32, so the grid has at least `rows` threads for the row-scale check
  int8_to_bf16_kernel<<<grid_for(octs, kThreads * kUnroll), kThreads, 0, stream>>>(
      static_cast<const uint2*>(in), static_cast<const float*>(row_scale), static_cast<uint4*>(out), octs, rows,
      static_cast<uint32_t*>(range_flag));
  return static_cast<int>(cudaGetLastError());
}

int launch_mxfp4_to_int8(const void* packed, void* out, long rows, long k, cudaStream_t stream) {
  const long pairs = rows * k / 16;
  if (pairs == 0) return 0;
  mxfp4_to_int8_kernel<<<grid_for(pairs, kThreads * kUnroll), kThreads, 0, stream>>>(
      static_cast<const uint2*>(packed), static_cast<uint4*>(out), pairs);
  return static_cast<int>(cudaGetLastError());
}

int launch_o2_quantize(const void* a_int8, const void* row_scale, void* codes, void* sf_natural, void* sf_tiled,
                       long rows, long k, cudaStream_t stream) {
  const long blocks = rows * (k / 32);
  if (blocks == 0) return 0;
  o2_quantize_kernel<<<grid_for(blocks, kThreads), kThreads, 0, stream>>>(
      static_cast<const uint4*>(a_int8), static_cast<const float*>(row_scale), static_cast<uint4*>(codes),
      static_cast<uint8_t*>(sf_natural), static_cast<uint8_t*>(sf_tiled), blocks, static_cast<int>(k / 32),
      static_cast<int>(tiled_scale_katoms(k)));
  return static_cast<int>(cudaGetLastError());
}

int launch_o2_tile_scales(const void* natural, void* tiled, long rows, long k, cudaStream_t stream) {
  const long padded_rows = tiled_scale_rows(rows);
  const long katoms = tiled_scale_katoms(k);
  const long items = padded_rows * katoms;
  o2_tile_scales_kernel<<<grid_for(items, kThreads), kThreads, 0, stream>>>(
      static_cast<const uint8_t*>(natural), static_cast<uint32_t*>(tiled), static_cast<int>(rows),
      static_cast<int>(k / 32), static_cast<int>(padded_rows), static_cast<int>(katoms));
  return static_cast<int>(cudaGetLastError());
}

}  // namespace adg
