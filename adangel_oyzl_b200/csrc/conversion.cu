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

#include "common.cuh"
#include "convert_device.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kChunk = kThreads * kUnroll;  // items one CTA handles per loop trip

// Every kernel below handles chunks of kChunk items; each thread keeps kUnroll independent vector loads in
// flight per chunk.  The launchers start one CTA per chunk (the loops then run once): with a fixed number of
// resident CTAs striding over the chunks the same kernels were measured 15 - 20 % slower at 16384 x 8192 and no
// faster at 4096 x 4096 -- the hardware's CTA scheduler balances the tail better.  Item counts are below 2**31
// (checked by the launchers), so all index arithmetic is 32-bit; the row of an item comes from a
// multiply-high instead of the 64-bit division that held int8_to_fp16 at 0.79 of the HBM rate (now 0.97).
constexpr int kCtasPerSm = 8;
constexpr int kQuantCtasPerSm = 4;  // the re-quantizer needs up to 64 registers per thread

// ---- O0 weight: packed E2M1 + UE8M0 -> FP16 -------------------------------------------------
// One 32-bit word (8 elements) per item; the scale of word i is scales[i / 4] because both tensors
// are contiguous and K is a multiple of 32.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) mxfp4_to_fp16_kernel(const uint32_t* __restrict__ packed,
                                                                 const uint8_t* __restrict__ scales,
                                                                 uint4* __restrict__ out, uint32_t words) {
  pdl_launch_dependents();
  pdl_wait();
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < words; base += gridDim.x * kChunk) {
    uint32_t w[kUnroll];
    uint32_t sc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < words) {
        w[u] = __ldg(packed + i);
        sc[u] = __ldg(scales + (i >> 2));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
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
}

// ---- O0 activation: INT8 * row scale -> FP16 --------------------------------------------------
// Eight elements (one 64-bit load, one 128-bit store) per item; `octs` = rows*K/8.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) int8_to_fp16_kernel(const uint2* __restrict__ in,
                                                                const float* __restrict__ row_scale,
                                                                uint4* __restrict__ out, uint32_t octs,
                                                                uint32_t octs_per_row, uint32_t magic) {
  pdl_launch_dependents();
  pdl_wait();
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < octs; base += gridDim.x * kChunk) {
    uint2 v[kUnroll];
    float s[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < octs) {
        v[u] = __ldg(in + i);
        s[u] = __ldg(row_scale + fast_div(i, octs_per_row, magic));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < octs) out[i] = int8x8_to_half8(v[u], s[u]);
    }
  }
}

// ---- O1 (BF16 operands) weight: packed E2M1 + UE8M0 -> BF16 of e2m1 * 2^(scale-127) ------------
// Exact: the value has two significant bits.  One 32-bit word (8 elements) per item.
// A scale code outside [kO1MinScaleCode, kO1MaxScaleCode] sets bit 0 of *range_flag.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) mxfp4_to_bf16_scaled_kernel(const uint32_t* __restrict__ packed,
                                                                        const uint8_t* __restrict__ scales,
                                                                        uint4* __restrict__ out, uint32_t words,
                                                                        uint32_t* __restrict__ range_flag) {
  pdl_launch_dependents();
  pdl_wait();
  bool bad = false;
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < words; base += gridDim.x * kChunk) {
    uint32_t w[kUnroll];
    uint32_t sc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < words) {
        w[u] = __ldg(packed + i);
        sc[u] = __ldg(scales + (i >> 2));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i >= words) continue;
      const uint32_t code = sc[u];
      bad |= code < kO1MinScaleCode || code > kO1MaxScaleCode;
      const float s = __uint_as_float((code == 0u ? 1u : code) << 23);  // 2^(code-127); unused when out of range
      uint32_t o[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const float2 f = __half22float2(e2m1x2_to_half2((w[u] >> (8 * b)) & 0xFFu));
        const __nv_bfloat162 v = __floats2bfloat162_rn(f.x * s, f.y * s);
        o[b] = *reinterpret_cast<const uint32_t*>(&v);
      }
      out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(range_flag, 1u);
}

// ---- O1 (BF16 operands) activation: INT8 -> BF16 of the integer itself, exact ------------------
// Eight elements per item.  The grid's threads also check the row scales (grid-stride): one outside
// [2^kO1MinAScaleExp, 2^kO1MaxAScaleExp] (or not finite) sets bit 1 of *range_flag.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) int8_to_bf16_kernel(const uint2* __restrict__ in,
                                                                const float* __restrict__ row_scale,
                                                                uint4* __restrict__ out, uint32_t octs, uint32_t rows,
                                                                uint32_t* __restrict__ range_flag) {
  pdl_launch_dependents();
  pdl_wait();
  bool bad = false;
  for (uint32_t r = blockIdx.x * kThreads + threadIdx.x; r < rows; r += gridDim.x * kThreads) {
    const float s = __ldg(row_scale + r);
    bad |= !(s >= exp2f(static_cast<float>(kO1MinAScaleExp)) && s <= exp2f(static_cast<float>(kO1MaxAScaleExp)));
  }
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < octs; base += gridDim.x * kChunk) {
    uint2 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < octs) v[u] = __ldg(in + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
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
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(range_flag, 2u);
}

// ---- O1 weight: packed E2M1 -> INT8 (2*E2M1) ---------------------------------------------------
// Sixteen elements (64-bit load, 128-bit store) per item; `pairs` = rows*K/16.
__global__ void __launch_bounds__(kThreads, kCtasPerSm) mxfp4_to_int8_kernel(const uint2* __restrict__ packed,
                                                                 uint4* __restrict__ out, uint32_t pairs) {
  pdl_launch_dependents();
  pdl_wait();
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < pairs; base += gridDim.x * kChunk) {
    uint2 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i < pairs) v[u] = __ldg(packed + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      if (i >= pairs) continue;
      uint4 o;
      e2m1x8_to_int8x8(v[u].x, o.x, o.y);
      e2m1x8_to_int8x8(v[u].y, o.z, o.w);
      out[i] = o;
    }
  }
}

// ---- O2 activation: INT8 * row scale -> MXFP4 codes + UE8M0 scales -------------------------------
// Half a K32 block per item: 16 bytes in (a warp's load covers 512 contiguous bytes), 8 bytes of packed
// codes out; lane pairs share a block (one shuffle for its maximum), and the eight lanes that hold four
// consecutive blocks of a row gather their scale bytes into one 32-bit word of the natural [M, K/32]
// array (optional) and of the 512-byte-atom layout the tensor core reads.  `halves` = rows*K/16,
// `halves_per_row` = K/16 (a multiple of 4, so a block never straddles two warps or two rows).
__global__ void __launch_bounds__(kThreads, kQuantCtasPerSm) o2_quantize_kernel(const uint4* __restrict__ in,
                                                               const float* __restrict__ row_scale,
                                                               uint2* __restrict__ codes, uint8_t* __restrict__ sf_natural,
                                                               uint8_t* __restrict__ sf_tiled, uint32_t halves,
                                                               uint32_t halves_per_row, uint32_t magic, int katoms) {
  pdl_launch_dependents();
  pdl_wait();
  const bool words_ok = (halves_per_row & 7u) == 0;  // K/32 a multiple of 4: whole scale words per row
  for (uint32_t base = blockIdx.x * kChunk + threadIdx.x; base - threadIdx.x < halves; base += gridDim.x * kChunk) {
    uint4 v[kUnroll];
    float s[kUnroll];
    uint32_t row[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      const uint32_t i_safe = i < halves ? i : 0u;
      row[u] = fast_div(i_safe, halves_per_row, magic);
      v[u] = __ldg(in + i_safe);
      s[u] = __ldg(row_scale + row[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * kThreads;
      const bool valid = i < halves;
      uint32_t code;
      const uint2 c = o2_quantize_half_block(v[u], s[u], code);  // all lanes: shuffles inside
      if (valid) codes[i] = c;
      const int g = static_cast<int>((valid ? i : 0u) - row[u] * halves_per_row) >> 1;
      if (words_ok) {
        // lanes 0,2,4,6 of each group of eight hold the four blocks of one scale word
        uint32_t word = code | (__shfl_down_sync(0xffffffffu, code, 2) << 8);
        word |= __shfl_down_sync(0xffffffffu, word, 4) << 16;
        if (valid && (threadIdx.x & 7) == 0) {
          if (sf_natural != nullptr) *reinterpret_cast<uint32_t*>(sf_natural + (i >> 1)) = word;
          *reinterpret_cast<uint32_t*>(sf_tiled + tiled_sf_offset(static_cast<int>(row[u]), g, katoms)) = word;
        }
      } else if (valid && (threadIdx.x & 1) == 0) {
        if (sf_natural != nullptr) sf_natural[i >> 1] = static_cast<uint8_t>(code);
        sf_tiled[tiled_sf_offset(static_cast<int>(row[u]), g, katoms)] = static_cast<uint8_t>(code);
      }
    }
  }
}

// ---- O2 weight scales: natural [rows, K/32] -> 512-byte atoms, zero padding included -----------
// One thread per (padded row, K-atom of 4 blocks).
__global__ void __launch_bounds__(kThreads) o2_tile_scales_kernel(const uint8_t* __restrict__ natural,
                                                                  uint32_t* __restrict__ tiled, int rows, int groups,
                                                                  int padded_rows, int katoms) {
  pdl_launch_dependents();
  pdl_wait();
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

constexpr long kMaxItems = 0x7fffffffL - 2 * kChunk;
int too_large() { return static_cast<int>(cudaErrorInvalidValue); }

}  // namespace

int launch_mxfp4_to_fp16(const void* packed, const void* scales, void* out, long rows, long k, cudaStream_t stream) {
  const long words = rows * k / 8;
  if (words == 0) return 0;
  if (words > kMaxItems) return too_large();
  const cudaError_t err = launch_overlapped(mxfp4_to_fp16_kernel, dim3(grid_for(words, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint32_t*>(packed), static_cast<const uint8_t*>(scales), static_cast<uint4*>(out),
      static_cast<uint32_t>(words));
  return static_cast<int>(err);
}

int launch_int8_to_fp16(const void* in, const void* row_scale, void* out, long rows, long k, cudaStream_t stream) {
  const long octs = rows * k / 8;
  if (octs == 0) return 0;
  if (octs > kMaxItems) return too_large();
  const uint32_t per_row = static_cast<uint32_t>(k / 8);
  const cudaError_t err = launch_overlapped(int8_to_fp16_kernel, dim3(grid_for(octs, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint2*>(in), static_cast<const float*>(row_scale), static_cast<uint4*>(out),
      static_cast<uint32_t>(octs), per_row, fast_div_magic(per_row));
  return static_cast<int>(err);
}

int launch_mxfp4_to_bf16_scaled(const void* packed, const void* scales, void* out, void* range_flag, long rows, long k,
                                cudaStream_t stream) {
  const long words = rows * k / 8;
  if (words == 0) return 0;
  if (words > kMaxItems) return too_large();
  const cudaError_t err = launch_overlapped(mxfp4_to_bf16_scaled_kernel, dim3(grid_for(words, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint32_t*>(packed), static_cast<const uint8_t*>(scales), static_cast<uint4*>(out),
      static_cast<uint32_t>(words), static_cast<uint32_t*>(range_flag));
  return static_cast<int>(err);
}

int launch_int8_to_bf16(const void* in, const void* row_scale, void* out, void* range_flag, long rows, long k,
                        cudaStream_t stream) {
  const long octs = rows * k / 8;
  if (octs == 0) return 0;
  if (octs > kMaxItems) return too_large();
  const cudaError_t err = launch_overlapped(int8_to_bf16_kernel, dim3(grid_for(octs, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint2*>(in), static_cast<const float*>(row_scale), static_cast<uint4*>(out),
      static_cast<uint32_t>(octs), static_cast<uint32_t>(rows), static_cast<uint32_t*>(range_flag));
  return static_cast<int>(err);
}

int launch_mxfp4_to_int8(const void* packed, void* out, long rows, long k, cudaStream_t stream) {
  const long pairs = rows * k / 16;
  if (pairs == 0) return 0;
  if (pairs > kMaxItems) return too_large();
  const cudaError_t err = launch_overlapped(mxfp4_to_int8_kernel, dim3(grid_for(pairs, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint2*>(packed), static_cast<uint4*>(out), static_cast<uint32_t>(pairs));
  return static_cast<int>(err);
}

int launch_o2_quantize(const void* a_int8, const void* row_scale, void* codes, void* sf_natural, void* sf_tiled,
                       long rows, long k, cudaStream_t stream) {
  const long halves = rows * (k / 16);
  if (halves == 0) return 0;
  if (halves > kMaxItems) return too_large();
  const uint32_t per_row = static_cast<uint32_t>(k / 16);
  const cudaError_t err = launch_overlapped(o2_quantize_kernel, dim3(grid_for(halves, kChunk)), dim3(kThreads), 0, stream, 1,
      static_cast<const uint4*>(a_int8), static_cast<const float*>(row_scale), static_cast<uint2*>(codes),
      static_cast<uint8_t*>(sf_natural), static_cast<uint8_t*>(sf_tiled), static_cast<uint32_t>(halves), per_row,
      fast_div_magic(per_row), static_cast<int>(tiled_scale_katoms(k)));
  return static_cast<int>(err);
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
