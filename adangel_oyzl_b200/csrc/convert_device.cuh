// Per-thread bodies of the activation-side conversions, shared by the stand-alone conversion kernels
// (conversion.cu) and by the GEMM kernels that convert A themselves while their tensor cores run
// (the converter warps of gemm_acc.cu / gemm_acc2.cu).
//
//   int8x8_to_half8      O0: eight INT8 values * row scale -> eight FP16 (reference
//                        csrc/sm120/conversion.cu:25-37)
//   o2_quantize_block    O2: one K32 block of INT8 * row scale -> 16 bytes of packed E2M1 codes and
//                        the block's UE8M0 scale code (reference csrc/sm120/o2_cutlass.cu:207-259)
//   tiled_sf_offset      byte offset of (row, K32 block) in the 512-byte-atom scale layout the
//                        block-scaled MMA reads (reference csrc/sm120/o2_cutlass.cu:261-274)
#pragma once

#include "codecs.cuh"

namespace adg {

__device__ __forceinline__ uint4 int8x8_to_half8(uint2 v, float s) {
  float lo[4], hi[4];
  int8x4_to_float4(v.x, lo);
  int8x4_to_float4(v.y, hi);
  const __half2 h0 = __floats2half2_rn(lo[0] * s, lo[1] * s);
  const __half2 h1 = __floats2half2_rn(lo[2] * s, lo[3] * s);
  const __half2 h2 = __floats2half2_rn(hi[0] * s, hi[1] * s);
  const __half2 h3 = __floats2half2_rn(hi[2] * s, hi[3] * s);
  return make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                    *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
}

__device__ __forceinline__ long tiled_sf_offset(int row, int g, int katoms) {
  return (static_cast<long>(row >> 7) * katoms + (g >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (g & 3);
}

// `lo`, `hi`: the block's 32 INT8 values; `s`: the row scale.  Returns the packed codes (even k in the
// low nibble); `code` receives the UE8M0 scale code: exact floor(log2(amax)) - 2 + 127, clamped, 127
// for an all-zero block.
__device__ __forceinline__ uint4 o2_quantize_block(const uint4 lo, const uint4 hi, const float s, uint32_t& code) {
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
      // the scaling multiply is a fused add of +0: a product of -0 becomes +0, which must encode as
      // code 0 (the reference's sign bit is `value < 0`)
      const float x0 = __fmaf_rn(v[i], inv, 0.0f);
      const float x1 = __fmaf_rn(v[i + 1], inv, 0.0f);
      word |= float2_to_e2m1x2(x0, x1) << (8 * b);
    }
    o[q] = word;
  }
  code = static_cast<uint32_t>(e + 127);
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Half of a K32 block per lane: `in` holds 16 INT8 values, the partner lane (lane ^ 1) holds the other
// half of the same block, so one shuffle completes the block maximum.  Every lane of the warp must call
// this together.  Returns the lane's 8 bytes of packed codes; `code` as in o2_quantize_block (both lanes
// of a pair receive it).
__device__ __forceinline__ uint2 o2_quantize_half_block(const uint4 in, const float s, uint32_t& code) {
  const uint32_t words[4] = {in.x, in.y, in.z, in.w};
  float v[16];
  float amax = 0.0f;
#pragma unroll
  for (int wi = 0; wi < 4; ++wi) {
    float f[4];
    int8x4_to_float4(words[wi], f);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      v[wi * 4 + b] = f[b] * s;
      amax = fmaxf(amax, fabsf(v[wi * 4 + b]));
    }
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  int e = 0;
  if (amax != 0.0f) {
    e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 2;
    e = e < -127 ? -127 : (e > 127 ? 127 : e);
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2**-e, exact
  uint32_t o[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = q * 8 + b * 2;
      const float x0 = __fmaf_rn(v[i], inv, 0.0f);  // -0 -> +0, see o2_quantize_block
      const float x1 = __fmaf_rn(v[i + 1], inv, 0.0f);
      word |= float2_to_e2m1x2(x0, x1) << (8 * b);
    }
    o[q] = word;
  }
  code = static_cast<uint32_t>(e + 127);
  return make_uint2(o[0], o[1]);
}

__device__ __forceinline__ void int8x16_to_half16(const uint4 in, const float s, uint4& o0, uint4& o1) {
  o0 = int8x8_to_half8(make_uint2(in.x, in.y), s);
  o1 = int8x8_to_half8(make_uint2(in.z, in.w), s);
}

// ---- activation conversion as a role inside a GEMM kernel ------------------------------------------
// The converter warps of every CTA walk the rows of A (row = cta, cta + num_ctas, ...: ascending, the order
// in which the GEMM's tiles need them), convert one row at a time and then count the row into
// ready[row / 128].  The GEMM's TMA producer waits until a row block's counter has reached the number of
// rows in the block before it loads the block's tiles.  The writes are made by ordinary stores and read
// by the copy engine, hence the proxy fences on both sides of the counter.
struct FusedConvert {
  const uint4* a_int8;     // [M, K] INT8, rows of K bytes
  const float* a_scale;    // [M]
  void* a_out;             // O0: FP16 [M, K]; O2: packed E2M1 codes [M, K/2]
  uint8_t* sf_natural;     // O2, optional: [M, K/32]
  uint8_t* sf_tiled;       // O2: tiled scales (padding zero-filled by the caller once)
  uint32_t* ready;         // [ceil(M/128) + 1] zero before the first launch; the kernel re-zeroes it at its end
};

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

constexpr int kConvThreads = 128;  // one warp group
constexpr int kConvBatch = 4;      // 16-byte items per thread and batch: 4 * 128 * 16 = 8192 elements

// KIND 0: INT8 * row scale -> FP16; KIND 2: -> MXFP4 codes + scales.  `tid` in [0, kConvThreads); all
// threads of the warp group call this together (named barrier `bar_id`, shuffles inside).
template <int KIND>
__device__ __forceinline__ void convert_rows_role(const FusedConvert& c, const int M, const int K, const int tid,
                                                  const int cta, const int num_ctas, const int bar_id) {
  const int hpr = K >> 4;  // 16-byte items per row
  const int katoms = ((K / 32 + 7) / 8) * 2;
  const bool words_ok = (hpr & 7) == 0;
  struct Unit {
    int row, h0;
  };
  auto load = [&](const Unit& u, uint4 (&buf)[kConvBatch], float& s) {
    const uint4* src = c.a_int8 + static_cast<long>(u.row) * hpr;
    s = __ldg(c.a_scale + u.row);
#pragma unroll
    for (int j = 0; j < kConvBatch; ++j) {
      const int h = u.h0 + j * kConvThreads + tid;
      buf[j] = h < hpr ? __ldg(src + h) : make_uint4(0, 0, 0, 0);
    }
  };
  auto compute = [&](const Unit& u, const uint4 (&buf)[kConvBatch], const float s) {
#pragma unroll
    for (int j = 0; j < kConvBatch; ++j) {
      const int h = u.h0 + j * kConvThreads + tid;
      if (u.h0 + j * kConvThreads >= hpr) break;  // uniform across the warp group
      const bool valid = h < hpr;
      if constexpr (KIND == 0) {
        uint4 o0, o1;
        int8x16_to_half16(buf[j], s, o0, o1);
        if (valid) {
          uint4* dst = static_cast<uint4*>(c.a_out) + (static_cast<long>(u.row) * hpr + h) * 2;
          dst[0] = o0;
          dst[1] = o1;
        }
      } else {
        uint32_t code;
        const uint2 packed = o2_quantize_half_block(buf[j], s, code);
        if (valid) static_cast<uint2*>(c.a_out)[static_cast<long>(u.row) * hpr + h] = packed;
        const int g = (valid ? h : 0) >> 1;
        if (words_ok) {
          uint32_t word = code | (__shfl_down_sync(0xffffffffu, code, 2) << 8);
          word |= __shfl_down_sync(0xffffffffu, word, 4) << 16;
          if (valid && (tid & 7) == 0) {
            if (c.sf_natural != nullptr)
              *reinterpret_cast<uint32_t*>(c.sf_natural + static_cast<long>(u.row) * (hpr >> 1) + g) = word;
            *reinterpret_cast<uint32_t*>(c.sf_tiled + tiled_sf_offset(u.row, g, katoms)) = word;
          }
        } else if (valid && (tid & 1) == 0) {
          if (c.sf_natural != nullptr) c.sf_natural[static_cast<long>(u.row) * (hpr >> 1) + g] = static_cast<uint8_t>(code);
          c.sf_tiled[tiled_sf_offset(u.row, g, katoms)] = static_cast<uint8_t>(code);
        }
      }
    }
  };
  auto advance = [&](const Unit& u) {
    Unit n = u;
    n.h0 += kConvBatch * kConvThreads;
    if (n.h0 >= hpr) {
      n.h0 = 0;
      n.row += num_ctas;
    }
    return n;
  };
  // the row is complete: publish it
  auto publish = [&](const int row) {
    __threadfence();
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kConvThreads) : "memory");
    if (tid == 0) {
      fence_proxy_async_all();
      red_release_gpu_add(c.ready + (row >> 7), 1u);
    }
  };
  Unit cur{cta, 0};
  if (cur.row >= M) return;
  uint4 buf_a[kConvBatch], buf_b[kConvBatch];
  float s_a, s_b;
  load(cur, buf_a, s_a);
  while (true) {
    Unit nxt = advance(cur);
    if (nxt.row < M) load(nxt, buf_b, s_b);
    compute(cur, buf_a, s_a);
    if (nxt.row != cur.row) publish(cur.row);
    if (nxt.row >= M) break;
    cur = nxt;
    nxt = advance(cur);
    if (nxt.row < M) load(nxt, buf_a, s_a);
    compute(cur, buf_b, s_b);
    if (nxt.row != cur.row) publish(cur.row);
    if (nxt.row >= M) break;
    cur = nxt;
  }
}

// Quotient of a 32-bit index by an invariant divisor without the integer-division sequence:
// `magic` = floor(2**32 / d) (host side: fast_div_magic); the estimate is at most one too small.
__host__ __device__ inline uint32_t fast_div_magic(uint32_t d) { return static_cast<uint32_t>((1ull << 32) / d); }
__device__ __forceinline__ uint32_t fast_div(uint32_t i, uint32_t d, uint32_t magic) {
  uint32_t q = __umulhi(i, magic);
  if (i - q * d >= d) ++q;
  return q;
}

}  // namespace adg
