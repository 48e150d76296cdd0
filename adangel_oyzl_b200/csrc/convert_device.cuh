// Per-thread bodies of the activation-side conversions, shared by the stand-alone conversion kernels
// (conversion.cu) and by the GEMM kernels that convert A themselves while their tensor cores run
// (the converter warps of gemm_acc.cu / gemm_acc2.cu).
//
//   int8x8_to_half8      O0: eight INT8 values * row scale -> eight FP16 (reference
//                        csrc/sm120/conversion.cu:25-37)
//   o2_quantize_half_block  O2: half a K32 block of INT8 * row scale per lane -> 8 bytes of packed E2M1 codes and
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

// ---- O2 activation re-quantization ---------------------------------------------------------------------
// Per K32 block of v[k] = RN(float(a[k]) * s):  amax = max |v|;  e = floor(log2 amax) - 2 (0 for a zero block,
// clamped to [-127, 127]);  code[k] = E2M1_rne(v[k] / 2**e) with sign bit `v < 0`;  scale code = e + 127.
//
// Fast path (row scale a normal number with 2**-111 <= |s| < 2**112; always taken for real activations):
//   * RN and |.| are monotone, so amax = RN(max|a| * |s|): the maximum is taken over the integers, one
//     multiply per block instead of one per element;
//   * scaling by a power of two commutes with rounding inside the normal range, so
//     v / 2**e = RN(a * s) * 2**-e = RN(a * (s * 2**-e)): ONE fused multiply-add per element (its +0 addend turns
//     a product of -0 into +0, which must encode as code 0) instead of a multiply and a scaling.  In that range
//     nothing is subnormal: 1/32 <= |s * 2**-e| <= 8 whenever the block holds a non-zero element.
// Outside that range (tiny, huge, zero, negative-zero, NaN/Inf scales) the two roundings are done literally.
// Both paths give the bits of the reference's kernel (csrc/sm120/o2_cutlass.cu:207-259).
__device__ __forceinline__ bool o2_scale_is_plain(float s) {
  const uint32_t ex = (__float_as_uint(s) >> 23) & 0xFFu;
  return ex >= 16u && ex < 239u;
}
__device__ __forceinline__ int o2_block_exponent(float amax) {
  if (amax == 0.0f) return 0;
  const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 2;
  return e < -127 ? -127 : (e > 127 ? 127 : e);
}

// Half of a K32 block per lane: `in` holds 16 INT8 values, the partner lane (lane ^ 1) holds the other
// half of the same block, so one shuffle completes the block maximum.  Every lane of the warp must call
// this together.  Returns the lane's 8 bytes of packed codes (even k in the low nibble); `code` receives the
// block's UE8M0 scale code (both lanes of a pair).
__device__ __forceinline__ uint2 o2_quantize_half_block(const uint4 in, const float s, uint32_t& code) {
  float f[16];
  {
    float t[4];
    int8x4_to_float4(in.x, t), f[0] = t[0], f[1] = t[1], f[2] = t[2], f[3] = t[3];
    int8x4_to_float4(in.y, t), f[4] = t[0], f[5] = t[1], f[6] = t[2], f[7] = t[3];
    int8x4_to_float4(in.z, t), f[8] = t[0], f[9] = t[1], f[10] = t[2], f[11] = t[3];
    int8x4_to_float4(in.w, t), f[12] = t[0], f[13] = t[1], f[14] = t[2], f[15] = t[3];
  }
  // whether the whole warp can take the fast path: the shuffles below need every lane in the same branch
  const bool plain = __all_sync(0xffffffffu, o2_scale_is_plain(s));
  float x[16];
  int e;
  if (plain) {
    float m[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      m[i] = fmaxf(fmaxf(fabsf(f[4 * i]), fabsf(f[4 * i + 1])), fmaxf(fabsf(f[4 * i + 2]), fabsf(f[4 * i + 3])));
    float imax = fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
    imax = fmaxf(imax, __shfl_xor_sync(0xffffffffu, imax, 1));
    e = o2_block_exponent(imax * fabsf(s));
    // s * 2**-e: exponent arithmetic on the bits (exact; the result is a normal number, see above)
    const float s_e = __uint_as_float(__float_as_uint(s) - (static_cast<uint32_t>(e) << 23));
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = __fmaf_rn(f[i], s_e, 0.0f);
  } else {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      f[i] = f[i] * s;
      amax = fmaxf(amax, fabsf(f[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    e = o2_block_exponent(amax);
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2**-e, exact
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = __fmaf_rn(f[i], inv, 0.0f);
  }
  code = static_cast<uint32_t>(e + 127);
  const float(&lo)[8] = *reinterpret_cast<const float(*)[8]>(&x[0]);
  const float(&hi)[8] = *reinterpret_cast<const float(*)[8]>(&x[8]);
  return make_uint2(float8_to_e2m1x8(lo), float8_to_e2m1x8(hi));
}

__device__ __forceinline__ void int8x16_to_half16(const uint4 in, const float s, uint4& o0, uint4& o1) {
  o0 = int8x8_to_half8(make_uint2(in.x, in.y), s);
  o1 = int8x8_to_half8(make_uint2(in.z, in.w), s);
}

// ---- activation conversion as a role inside a GEMM kernel ------------------------------------------
// The converter warps of every CTA walk the rows of A (row = cta, cta + num_ctas, ...: ascending, the order
// in which the GEMM's tiles need them) and convert one row at a time; after each row they bump a counter in
// shared memory and go on.  A publisher thread (another warp of the CTA) watches that counter, makes the
// finished rows visible device-wide with ONE fence per batch of rows -- the fence waits for the stores to be
// acknowledged, most of a microsecond that the converters must not spend per row -- and then counts each
// row into ready[row / 128].  The GEMM's TMA producer waits until a row block's counter has reached the
// number of rows in the block before it loads the block's tiles.  The rows are written by ordinary stores and
// read by the copy engine, hence the proxy fences on both sides of the counters.
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
__device__ __forceinline__ uint32_t ld_acquire_cta_shared(uint32_t smem_addr) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(uint32_t smem_addr, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr), "r"(v) : "memory");
}

constexpr int kConvThreads = 128;  // one warp group
constexpr int kConvSlots = 8;      // 16-byte items a thread keeps in flight per unit of work

// KIND 0: INT8 * row scale -> FP16; KIND 2: -> MXFP4 codes + scales.  `tid` in [0, kConvThreads); all
// threads of the warp group call this together (named barrier `bar_id`, shuffles inside).
// `done_slot`: shared-memory address of the CTA's count of finished rows (zero at kernel start).
//
// A unit of work is kConvSlots items per thread: several whole rows when a row needs few items per thread
// (K = 4096: two items, four rows per unit), or a part of one row when it needs more than kConvSlots.  The
// loads of unit u+1 are issued before unit u is converted, so that about two units of reads are in flight
// per CTA (with one row in flight the role ran at the latency of a single load per row).
template <int KIND>
__device__ __forceinline__ void convert_rows_role(const FusedConvert& c, const int M, const int K, const int tid,
                                                  const int cta, const int num_ctas, const int bar_id,
                                                  const uint32_t done_slot) {
  const int hpr = K >> 4;  // 16-byte items per row
  const int katoms = ((K / 32 + 7) / 8) * 2;
  const bool words_ok = (hpr & 7) == 0;
  const int ipr = (hpr + kConvThreads - 1) / kConvThreads;           // items per thread and row
  const int rows_per_unit = ipr >= kConvSlots ? 1 : kConvSlots / ipr;  // whole rows in a unit
  const int parts_per_row = ipr > kConvSlots ? (ipr + kConvSlots - 1) / kConvSlots : 1;
  const int my_rows = cta < M ? (M - cta + num_ctas - 1) / num_ctas : 0;
  if (my_rows == 0) return;
  // unit u covers local rows [first, first + rows_per_unit) (part = 0), or part `part` of local row `first`
  struct Unit {
    int first, part;
  };
  // slot -> (local row, item index within the row) of a unit; item < 0 when the slot is unused
  auto slot_row = [&](const Unit& u, int slot) { return ipr >= kConvSlots ? u.first : u.first + slot / ipr; };
  auto slot_item = [&](const Unit& u, int slot) {
    const int it = ipr >= kConvSlots ? u.part * kConvSlots + slot : (slot / ipr < rows_per_unit ? slot % ipr : -1);
    return it < ipr ? it : -1;
  };
  auto load = [&](const Unit& u, uint4 (&buf)[kConvSlots], float (&sc)[kConvSlots]) {
#pragma unroll
    for (int slot = 0; slot < kConvSlots; ++slot) {
      const int lr = slot_row(u, slot);
      const int it = slot_item(u, slot);
      const int h = it * kConvThreads + tid;
      const bool valid = it >= 0 && lr < my_rows && h < hpr;
      const long row = cta + static_cast<long>(lr) * num_ctas;
      buf[slot] = valid ? __ldg(c.a_int8 + row * hpr + h) : make_uint4(0, 0, 0, 0);
      sc[slot] = (it >= 0 && lr < my_rows) ? __ldg(c.a_scale + row) : 0.0f;
    }
  };
  auto compute = [&](const Unit& u, const uint4 (&buf)[kConvSlots], const float (&sc)[kConvSlots]) {
#pragma unroll
    for (int slot = 0; slot < kConvSlots; ++slot) {
      const int lr = slot_row(u, slot);
      const int it = slot_item(u, slot);
      if (it < 0 || lr >= my_rows) continue;  // uniform across the warp group
      const int h = it * kConvThreads + tid;
      const bool valid = h < hpr;
      const int row = cta + lr * num_ctas;
      if constexpr (KIND == 0) {
        uint4 o0, o1;
        int8x16_to_half16(buf[slot], sc[slot], o0, o1);
        if (valid) {
          uint4* dst = static_cast<uint4*>(c.a_out) + (static_cast<long>(row) * hpr + h) * 2;
          dst[0] = o0;
          dst[1] = o1;
        }
      } else {
        uint32_t code;
        const uint2 packed = o2_quantize_half_block(buf[slot], sc[slot], code);
        if (valid) static_cast<uint2*>(c.a_out)[static_cast<long>(row) * hpr + h] = packed;
        const int g = (valid ? h : 0) >> 1;
        if (words_ok) {
          uint32_t word = code | (__shfl_down_sync(0xffffffffu, code, 2) << 8);
          word |= __shfl_down_sync(0xffffffffu, word, 4) << 16;
          if (valid && (tid & 7) == 0) {
            if (c.sf_natural != nullptr)
              *reinterpret_cast<uint32_t*>(c.sf_natural + static_cast<long>(row) * (hpr >> 1) + g) = word;
            *reinterpret_cast<uint32_t*>(c.sf_tiled + tiled_sf_offset(row, g, katoms)) = word;
          }
        } else if (valid && (tid & 1) == 0) {
          if (c.sf_natural != nullptr) c.sf_natural[static_cast<long>(row) * (hpr >> 1) + g] = static_cast<uint8_t>(code);
          c.sf_tiled[tiled_sf_offset(row, g, katoms)] = static_cast<uint8_t>(code);
        }
      }
    }
  };
  auto advance = [&](const Unit& u) {
    Unit n = u;
    if (++n.part >= parts_per_row) {
      n.part = 0;
      n.first += rows_per_unit;
    }
    return n;
  };
  // rows [u.first, ...) of a finished unit are complete when its last part is done: tell the publisher
  // (the barrier orders every converter's stores before the count)
  uint32_t rows_done = 0;
  auto finish = [&](const Unit& u) {
    if (u.part + 1 < parts_per_row) return;
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kConvThreads) : "memory");
    rows_done += static_cast<uint32_t>(min(rows_per_unit, my_rows - u.first));
    if (tid == 0) st_release_cta_shared(done_slot, rows_done);
  };
  Unit cur{0, 0};
  uint4 buf_a[kConvSlots], buf_b[kConvSlots];
  float sc_a[kConvSlots], sc_b[kConvSlots];
  load(cur, buf_a, sc_a);
  while (true) {
    Unit nxt = advance(cur);
    if (nxt.first < my_rows) load(nxt, buf_b, sc_b);
    compute(cur, buf_a, sc_a);
    finish(cur);
    if (nxt.first >= my_rows) break;
    cur = nxt;
    nxt = advance(cur);
    if (nxt.first < my_rows) load(nxt, buf_a, sc_a);
    compute(cur, buf_b, sc_b);
    finish(cur);
    if (nxt.first >= my_rows) break;
    cur = nxt;
  }
}

// The publisher: one thread per CTA.  `abort_flag` is the CTA's abort word; gives up after `timeout_ns`.
// Returns false if it gave up (the caller records the status).
__device__ __forceinline__ bool publish_rows_role(const FusedConvert& c, const int M, const int cta, const int num_ctas,
                                                  const uint32_t done_slot, volatile uint32_t* abort_flag,
                                                  const unsigned long long timeout_ns) {
  if (cta >= M) return true;
  const uint32_t total = static_cast<uint32_t>((M - cta + num_ctas - 1) / num_ctas);
  uint32_t published = 0;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (published < total) {
    const uint32_t done = ld_acquire_cta_shared(done_slot);
    if (done > published) {
      __threadfence();          // cumulative: the converters' stores of rows [published, done) are visible device-wide
      fence_proxy_async_all();  // ... also to the copy engine
      for (uint32_t i = published; i < done; ++i) red_release_gpu_add(c.ready + ((cta + static_cast<int>(i) * num_ctas) >> 7), 1u);
      published = done;
      spins = 0;
      t0 = 0;
      continue;
    }
    if ((++spins & 0x3FFu) == 0) {
      if (*abort_flag) return true;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) return false;
    }
  }
  return true;
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
