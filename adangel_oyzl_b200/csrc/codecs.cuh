// Scalar/packed E2M1, UE8M0 and INT8 codecs used by the conversion kernels.
//
// Semantics follow the reference's scalar codecs (include/adangel/data_types.cuh:12-43 in the
// reference project): E2M1 magnitudes {0,.5,1,1.5,2,3,4,6} with bit 3 as sign; the O1 image of a
// nibble is 2*E2M1 as INT8; E2M1 encoding is round-to-nearest-even with saturation and keeps the
// sign of a negative value that rounds to zero; a UE8M0 code c means 2**(c-127).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace adg {

constexpr int kGroup = 32;  // elements sharing one UE8M0 scale

// 2**(code-127) as FP32 bits; code 0 is the subnormal 2**-127.
__device__ __forceinline__ float ue8m0_to_float(uint32_t code) {
  return __uint_as_float(code == 0 ? 0x00400000u : (code << 23));
}
// 2**(code-128) as FP32 (the O1 per-group weight factor 2**(code-127) * 0.5).
__device__ __forceinline__ float ue8m0_half_to_float(uint32_t code) {
  return __uint_as_float(code >= 2 ? ((code - 1) << 23) : (code == 1 ? 0x00400000u : 0x00200000u));
}

// Two packed E2M1 nibbles (low nibble = first element) -> half2 (x = first element).
__device__ __forceinline__ __half2 e2m1x2_to_half2(uint32_t byte) {
  uint32_t out;
  const uint16_t b = static_cast<uint16_t>(byte & 0xFFu);
  asm("{\n"
      ".reg .b8 lo, hi;\n"
      "mov.b16 {lo, hi}, %1;\n"
      "cvt.rn.f16x2.e2m1x2 %0, lo;\n"
      "}\n"
      : "=r"(out)
      : "h"(b));
  return *reinterpret_cast<__half2*>(&out);
}

// Two FP32 values -> one byte of packed E2M1 (first -> low nibble), round-to-nearest-even,
// saturating to +-6.
__device__ __forceinline__ uint32_t float2_to_e2m1x2(float first, float second) {
  uint16_t out;
  asm("{\n"
      ".reg .b8 t;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n"
      "mov.b16 %0, {t, 0};\n"
      "}\n"
      : "=h"(out)
      : "f"(first), "f"(second));
  return out;
}

// Eight FP32 values -> one 32-bit word of packed E2M1 (x[0] in the lowest nibble), round-to-nearest-even,
// saturating to +-6: four conversions and one byte merge.
__device__ __forceinline__ uint32_t float8_to_e2m1x8(const float (&x)[8]) {
  uint32_t out;
  asm("{\n"
      ".reg .b8 t0, t1, t2, t3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n"
      "mov.b32 %0, {t0, t1, t2, t3};\n"
      "}\n"
      : "=r"(out)
      : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
  return out;
}

// prmt.b32 in its default mode: selector nibble bits [2:0] pick one of the eight source bytes
// {b:a}; bit 3 replaces the picked byte by eight copies of its most significant bit.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

// Four packed INT8 values -> four FP32 values without the (slow) integer-to-float conversion unit:
// each byte, biased by 128, is spliced into the mantissa of 2**23, and 2**23 + 128 is subtracted.
// Exact for every INT8 value.
__device__ __forceinline__ void int8x4_to_float4(uint32_t w, float (&f)[4]) {
  const uint32_t biased = w ^ 0x80808080u;
  const float bias = 8388736.0f;  // 2**23 + 128
  f[0] = __uint_as_float(prmt(biased, 0x4B000000u, 0x7540u)) - bias;
  f[1] = __uint_as_float(prmt(biased, 0x4B000000u, 0x7541u)) - bias;
  f[2] = __uint_as_float(prmt(biased, 0x4B000000u, 0x7542u)) - bias;
  f[3] = __uint_as_float(prmt(biased, 0x4B000000u, 0x7543u)) - bias;
}

// Eight E2M1 nibbles of one 32-bit word -> eight INT8 values 2*E2M1 (two 32-bit words).
// Magnitudes come from a byte-permute lookup, signs from a sign-replicating byte permute.
__device__ __forceinline__ void e2m1x8_to_int8x8(uint32_t w, uint32_t& lo4, uint32_t& hi4) {
  const uint32_t pos_lo = 0x03020100u, pos_hi = 0x0C080604u;  // 0,1,2,3 | 4,6,8,12
  const uint32_t neg_lo = 0xFDFEFF00u, neg_hi = 0xF4F8FAFCu;  // 0,-1,-2,-3 | -4,-6,-8,-12
  const uint32_t sel0 = w & 0x7777u;
  const uint32_t sel1 = (w >> 16) & 0x7777u;
  const uint32_t ws = w << 4;  // bit 3 of every even nibble becomes the MSB of its byte
  // elements 0..3 live in bytes 0,1 of w; elements 4..7 in bytes 2,3
  const uint32_t m0 = prmt(ws, w, 0xD9C8u);
  const uint32_t m1 = prmt(ws, w, 0xFBEAu);
  const uint32_t p0 = prmt(pos_lo, pos_hi, sel0);
  const uint32_t p1 = prmt(pos_lo, pos_hi, sel1);
  const uint32_t n0 = prmt(neg_lo, neg_hi, sel0);
  const uint32_t n1 = prmt(neg_lo, neg_hi, sel1);
  lo4 = (p0 & ~m0) | (n0 & m0);
  hi4 = (p1 & ~m1) | (n1 & m1);
}

}  // namespace adg
