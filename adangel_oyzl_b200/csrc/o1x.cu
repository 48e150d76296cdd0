// "o1x": the exact-integer variant of O1.  It is NOT the O1 recurrence and is never chosen on a caller's
// behalf; callers ask for it by name.
//
// The literal O1 (reference python/adangel/reference/o1.py:16-20, csrc/sm120/o1_gemm.cu:298-316) rounds once per
// K32 group and operation:  acc = RN(acc + RN(float(P_g) * s_g)),  s_g = A_scale[m] * 2**(e[n,g]-128).  That
// forces every INT32 partial out of the tensor core and through the FP32 pipe, which bounds the kernel far
// below the INT8 tensor rate.  When the scale codes of one W row differ by at most 3, the row can be
// rewritten exactly as integers with ONE exponent:
//     W'[n,k] = 2*e2m1(W[n,k]) << (e[n,g] - emin[n])      |W'| <= 12 * 8 = 96, still INT8
// so that  sum_g P_g * 2**(e[n,g]-128) = (sum_k A[m,k] * W'[n,k]) * 2**(emin[n]-128)  with the integer sum
// exact in INT32 (K * 127 * 96 < 2**31 for K < 176000).  o1x computes
//     S = sum_k A_int8[m,k] * W'[n,k]           exact, kind::i8 MMAs accumulating over all of K in tensor memory
//     y = RN(float_rn(S) * RN(A_scale[m] * 2**(emin[n]-128)))
// i.e. two roundings in total instead of two per K32 group; it differs from the literal O1 by the latter's
// accumulated rounding (relative 1e-6 .. 1e-5 at K = 4096, see tests/test_gpu_o1x.py).
//
// Rows whose code spread exceeds 3 are "ineligible" (blocks whose nibbles are all zero do not count: they
// contribute nothing whatever their code).  Every 128-column block of Y that contains an ineligible row is
// computed by the literal INT8-operand kernel instead, launched behind the integer GEMM on a device-side list
// of those blocks (no host round trip); the fraction of such rows is reported to the caller.
#include "../../include/adangel_b200.h"
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kPrepThreads = 256;
constexpr int kMaxSpread = 3;

// One CTA per W row: min / max scale code over the row's non-zero blocks, then the shifted INT8 image.
//   info[0] += 1 per ineligible row; n_list[0] = number of listed column blocks (filled by the finish kernel)
//   block_bad[n / 128] = 1 when row n is ineligible
__global__ void __launch_bounds__(kPrepThreads)
o1x_prepare_kernel(const uint4* __restrict__ packed, const uint8_t* __restrict__ scales, uint4* __restrict__ out,
                   float* __restrict__ col_factor, uint32_t* __restrict__ block_bad, uint32_t* __restrict__ info,
                   int groups) {
  __shared__ uint32_t s_min, s_max;
  const int n = blockIdx.x;
  if (threadIdx.x == 0) {
    s_min = 255u;
    s_max = 0u;
  }
  __syncthreads();
  const uint4* src = packed + static_cast<long>(n) * groups;  // 16 bytes = one K32 block
  const uint8_t* sc = scales + static_cast<long>(n) * groups;
  uint32_t lo = 255u, hi = 0u;
  for (int g = threadIdx.x; g < groups; g += kPrepThreads) {
    const uint4 w = __ldg(src + g);
    if (((w.x | w.y | w.z | w.w) & 0x77777777u) != 0u) {
      const uint32_t c = __ldg(sc + g);
      lo = min(lo, c);
      hi = max(hi, c);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&s_min, lo);
    atomicMax(&s_max, hi);
  }
  __syncthreads();
  uint32_t emin = s_min;
  const uint32_t emax = s_max;
  if (emax < emin) emin = 127u;  // an all-zero row: any exponent serves
  const bool eligible = emax < emin || emax - emin <= static_cast<uint32_t>(kMaxSpread);
  if (threadIdx.x == 0) {
    col_factor[n] = eligible ? ue8m0_half_to_float(emin) : 0.0f;
    if (!eligible) {
      atomicAdd(info, 1u);
      block_bad[n >> 7] = 1u;
    }
  }
  uint4* dst = out + static_cast<long>(n) * groups * 2;  // 32 INT8 per block
  for (int g = threadIdx.x; g < groups; g += kPrepThreads) {
    uint4 o0 = make_uint4(0, 0, 0, 0), o1 = o0;
    if (eligible) {
      const uint4 w = __ldg(src + g);
      const int shift = min(max(static_cast<int>(__ldg(sc + g)) - static_cast<int>(emin), 0), kMaxSpread);
      uint32_t b[8];
      e2m1x8_to_int8x8(w.x, b[0], b[1]);
      e2m1x8_to_int8x8(w.y, b[2], b[3]);
      e2m1x8_to_int8x8(w.z, b[4], b[5]);
      e2m1x8_to_int8x8(w.w, b[6], b[7]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // per-byte arithmetic shift left: magnitudes are at most 12, so 12 << 3 = 96 stays inside a byte;
        // shifting the whole word and masking off what crossed a byte boundary keeps the sign bits right
        // because a negative byte's high bits are ones and the bits shifted in from below are masked
        const uint32_t keep = 0x01010101u * (0xFFu & (0xFFu << shift));
        b[i] = (b[i] << shift) & keep;
      }
      o0 = make_uint4(b[0], b[1], b[2], b[3]);
      o1 = make_uint4(b[4], b[5], b[6], b[7]);
    }
    dst[2 * g] = o0;
    dst[2 * g + 1] = o1;
  }
}

// n_list[0] = number of column blocks with an ineligible row, n_list[1..] their indices (ascending).
__global__ void o1x_finish_kernel(const uint32_t* __restrict__ block_bad, int32_t* __restrict__ n_list, int num_blocks) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int count = 0;
  for (int b = 0; b < num_blocks; ++b)
    if (block_bad[b] != 0u) n_list[1 + count++] = b;
  n_list[0] = count;
}

}  // namespace

}  // namespace adg

using namespace adg;

extern "C" {

int64_t adg_o1x_workspace_bytes(int64_t N) {
  const int64_t blocks = (N + 127) / 128;
  // info word + padding, per-block flags, the block list (count + indices)
  return 16 + 4 * blocks + 4 * (blocks + 1);
}

int adg_o1x_prepare_weight(const void* w_mxfp4, const void* w_scale, void* w_int8x, void* col_factor, void* workspace,
                           int64_t N, int64_t K, void* stream_v) {
  if (N <= 0 || K <= 0) return fail("rows and K must be positive");
  if (K % 64 != 0) return fail("K must be divisible by 64");
  if (K > 170000) return fail("o1x: K too large for exact INT32 accumulation");
  if (w_mxfp4 == nullptr || w_scale == nullptr || w_int8x == nullptr || col_factor == nullptr || workspace == nullptr)
    return fail("o1x: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(w_mxfp4) | reinterpret_cast<uintptr_t>(w_int8x) | reinterpret_cast<uintptr_t>(workspace)) & 15u)
    return fail("o1x: W_mxfp4, the INT8 image and the workspace must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(col_factor) & 3u) return fail("o1x: col_factor must be 4-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int blocks = static_cast<int>((N + 127) / 128);
  uint32_t* info = static_cast<uint32_t*>(workspace);
  uint32_t* block_bad = info + 4;
  int32_t* n_list = reinterpret_cast<int32_t*>(block_bad + blocks);
  if (int rc = check_cuda(cudaMemsetAsync(workspace, 0, static_cast<size_t>(adg_o1x_workspace_bytes(N)), stream), "cudaMemsetAsync"))
    return rc;
  o1x_prepare_kernel<<<static_cast<unsigned>(N), kPrepThreads, 0, stream>>>(
      static_cast<const uint4*>(w_mxfp4), static_cast<const uint8_t*>(w_scale), static_cast<uint4*>(w_int8x),
      static_cast<float*>(col_factor), block_bad, info, static_cast<int>(K / 32));
  if (int rc = check_cuda(cudaGetLastError(), "o1x_prepare_kernel launch")) return rc;
  o1x_finish_kernel<<<1, 32, 0, stream>>>(block_bad, n_list, blocks);
  return check_cuda(cudaGetLastError(), "o1x_finish_kernel launch");
}

int adg_o1x_ineligible_rows(const void* workspace, void* stream_v, int64_t* rows) {
  if (workspace == nullptr || rows == nullptr) return fail("o1x: NULL argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  uint32_t count = 0;
  if (int rc = check_cuda(cudaMemcpyAsync(&count, workspace, sizeof(count), cudaMemcpyDeviceToHost, stream), "D2H o1x info")) return rc;
  if (int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize")) return rc;
  *rows = count;
  return 0;
}

int adg_gemm_o1x(const void* a_int8, const void* a_scale, const void* w_int8x, const void* col_factor, const void* workspace,
                 const void* w_int8, const void* w_scale, float* y, int M, int N, int K, int ldy, void* stream_v) {
  if (workspace == nullptr) return fail("o1x: workspace must not be NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  GemmPlan plan;
  if (int rc = plan_o1x(&plan, a_int8, a_scale, w_int8x, col_factor, y, M, N, K, ldy)) return rc;
  if (int rc = run_plan(plan, stream)) return rc;
  // the literal kernel on the column blocks that hold an ineligible row: it returns at once when the list is empty
  if (w_int8 == nullptr || w_scale == nullptr) return 0;
  const int blocks = (N + 127) / 128;
  const uint32_t* info = static_cast<const uint32_t*>(workspace);
  const int32_t* n_list = reinterpret_cast<const int32_t*>(info + 4 + blocks);
  if (int rc = plan_o1_tiled(&plan, a_int8, a_scale, w_int8, w_scale, y, nullptr, M, N, K, ldy)) return rc;
  plan.n_list = n_list;
  return run_plan(plan, stream);
}

}  // extern "C"
