// O1 for decode-sized activations (M <= 64): warp-level INT8 MMAs with the per-K32 FP32 rescale in
// registers, on 32-row blocks of W so that the whole GPU streams the weights.
//
// Semantics are those of gemm_o1_kernel (reference/o1.py:16-20, csrc/sm120/o1_gemm.cu:167-333):
// for every output element and every K32 group g, in ascending g,
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                        (INT32, exact)
//     acc = fma(RN(float(P) * A_scale[m]), 2**(W_scale[n,g]-128), acc)   (FP32)
// which equals the reference's acc + float(P) * ((A_scale*2**(W_scale-127))*0.5) bit for bit: P is
// exact in any order, and the FP32 steps are the same operations in the same order.
//
// One K32 group of 16 rows of W against 8 activation rows is exactly one mma.sync m16n8k32 (s8 x s8 ->
// s32) with the rows of W as the MMA's M dimension; its four results per thread are rescaled and added
// to accumulators that stay in registers over all of K.  Nothing passes through tensor memory, so a
// group costs one shared-memory fragment load, one MMA and twelve FP32 instructions instead of the
// issue / commit / tensor-memory-load / hand-over chain of the tcgen05 formulation, whose fixed costs
// dominate when there are only a few activation rows.  A CTA owns 32 rows of W (N = 4096 gives 128
// CTAs) and all activation rows; two producer warps (even and odd stages) feed a ring of shared-memory
// stages by TMA, each stage one 128-byte K slab of W (32 rows) and of A (128-byte swizzle, so that
// the fragment loads are conflict-free).
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kRowsD = 32;              // W rows per CTA: two 16-row MMA tiles
constexpr int kTileWD = kRowsD * 128;   // bytes of W per stage
constexpr int kMaxStagesD = 12;
constexpr int kRingBytesD = 72 * 1024;  // three CTAs per SM
constexpr int kProducerWarps = 2;
constexpr int kMaxComputeWarps = 8;
constexpr int kMaxThreadsD = (kProducerWarps + kMaxComputeWarps) * 32;
constexpr int kSmemBytesD = kRingBytesD + 1024 + 256;

enum : uint32_t { kTagEmptyD = 0x3500, kTagFullD = 0x3600 };

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
// D (16 x 8, s32) = A (16 x 32, s8, row-major) * B (32 x 8, s8, column-major)
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

int stages_for(int stage_bytes) {
  int s = kRingBytesD / stage_bytes;
  s = s > kMaxStagesD ? kMaxStagesD : s;
  return s & ~1;  // even: the two producer warps alternate
}

// NT = 8-row activation tiles per compute warp.  a_rows = rows of the A box (a multiple of 8 * NT).
template <int NT>
__global__ void __launch_bounds__(kMaxThreadsD)
gemm_o1_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                      const float* __restrict__ a_scale, const uint8_t* __restrict__ w_scale, float* __restrict__ y,
                      int M, int N, int K, int ldy, int a_rows, int stages, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = kTileWD + a_rows * 128;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kRingBytesD);
  uint64_t* empty_bar = full_bar + kMaxStagesD;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(empty_bar + kMaxStagesD);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int compute_warps = static_cast<int>(blockDim.x >> 5) - kProducerWarps;
  const WaitEnv env{status, abort_flag};
  const int nb = blockIdx.x;
  const int groups = K / 32;
  const int num_kb = (groups + 3) / 4;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], static_cast<uint32_t>(compute_warps));
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_a);
  }
  __syncthreads();
  const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);

  if (warp < kProducerWarps) {
    // producers: warp p takes the stages of parity p; the warp stays converged and one elected lane
    // issues each copy
    int stage = warp;
    uint32_t phase = 0;
    for (int kb = warp; kb < num_kb; kb += kProducerWarps) {
      if (!mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, env, kTagEmptyD | stage)) break;
      const uint32_t st = smem0 + stage * stage_bytes;
      const uint32_t bar = full0 + stage * 8;
      mbar_expect_tx_elect(bar, static_cast<uint32_t>(stage_bytes));
      tma_load_2d_elect(st, &tm_w, bar, kb * 128, nb * kRowsD);
      tma_load_2d_elect(st + kTileWD, &tm_a, bar, kb * 128, 0);
      stage += kProducerWarps;
      if (stage >= stages) {
        stage -= stages;
        phase ^= 1u;
      }
    }
    return;
  }

  // ------------------------------- compute warps ------------------------------------------------
  const int cw = warp - kProducerWarps;
  const int rt = cw & 1;          // which 16 of the CTA's 32 rows of W
  const int t0 = (cw >> 1) * NT;  // first of this warp's 8-row activation tiles
  const int lrow = lane >> 2, lcol = (lane & 3) * 2;
  // this thread's results: rows n_lo and n_lo + 8 of W, activation rows m, m + 1 of each tile
  const int n_lo = nb * kRowsD + rt * 16 + lrow;
  const int n_hi = n_lo + 8;
  const uint8_t* sc_lo = w_scale + static_cast<long>(n_lo < N ? n_lo : 0) * groups;
  const uint8_t* sc_hi = w_scale + static_cast<long>(n_hi < N ? n_hi : 0) * groups;
  const bool vec16 = (groups & 15) == 0;

  float asc[NT][2], acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int m = (t0 + t) * 8 + lcol + c;
      asc[t][c] = m < M ? __ldg(a_scale + m) : 0.0f;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[t][c] = 0.0f;
  }
  // the 16 UE8M0 codes of stages 4*sb .. 4*sb+3 of one row; absent groups read as 0 and are never used
  auto load_codes = [&](const uint8_t* row, int sb) -> uint4 {
    const int g0 = sb * 16;
    if (g0 >= groups) return make_uint4(0u, 0u, 0u, 0u);
    if (vec16) return __ldg(reinterpret_cast<const uint4*>(row + g0));
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (g0 + i < groups) w[i >> 2] |= static_cast<uint32_t>(__ldg(row + g0 + i)) << (8 * (i & 3));
    return make_uint4(w[0], w[1], w[2], w[3]);
  };

  // fragment-load addresses inside a stage: lane -> (8 x 8 matrix, row r of it); the 16-byte chunk index is
  // XORed with the row's position in its 8-row swizzle atom
  const int mat = lane >> 3, r = lane & 7;
  const uint32_t w_base = static_cast<uint32_t>((rt * 16 + (mat & 1) * 8 + r) * 128);
  const uint32_t w_chunk = static_cast<uint32_t>(mat >> 1);
  // A: x4 covers two tiles (matrices: tile 0 chunk 0, tile 0 chunk 1, tile 1 chunk 0, tile 1 chunk 1);
  // x2 uses the addresses of lanes 0-15 only
  const uint32_t a_base = static_cast<uint32_t>(kTileWD + ((t0 + (NT == 2 ? (mat >> 1) : 0)) * 8 + r) * 128);
  const uint32_t a_chunk = static_cast<uint32_t>(mat & 1);
  const uint32_t rx = static_cast<uint32_t>(r);

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  // Fragment loads and MMAs of stage kb (partials of its up to four K32 groups into `p`), then the
  // stage is handed back: its bytes are in registers once the MMAs have been issued.
  auto issue = [&](int kb, int (&p)[4][NT][4]) {
    ok = mbar_wait_warp(full0 + stage * 8, phase, env, kTagFullD | stage);
    if (!ok) return;
    const uint32_t st = smem0 + static_cast<uint32_t>(stage * stage_bytes);
    const int ng = min(4, groups - kb * 4);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g < ng) {
        uint32_t wf[4];
        ldsm_x4(st + w_base + (((static_cast<uint32_t>(2 * g) + w_chunk) ^ rx) << 4), wf);
        if constexpr (NT == 2) {
          uint32_t af[4];
          ldsm_x4(st + a_base + (((static_cast<uint32_t>(2 * g) + a_chunk) ^ rx) << 4), af);
          mma_s8(p[g][0], wf, af[0], af[1]);
          mma_s8(p[g][1], wf, af[2], af[3]);
        } else {
          uint32_t af[2];
          ldsm_x2(st + a_base + (((static_cast<uint32_t>(2 * g) + a_chunk) ^ rx) << 4), af);
          mma_s8(p[g][0], wf, af[0], af[1]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive_a(empty0 + stage * 8);
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
  };
  auto accumulate = [&](int kb, const int (&p)[4][NT][4], uint32_t c_lo, uint32_t c_hi) {
    const int ng = min(4, groups - kb * 4);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g < ng) {
        const float s_lo = ue8m0_half_to_float((c_lo >> (8 * g)) & 0xFFu);
        const float s_hi = ue8m0_half_to_float((c_hi >> (8 * g)) & 0xFFu);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          acc[t][0] = __fmaf_rn(__fmul_rn(__int2float_rn(p[g][t][0]), asc[t][0]), s_lo, acc[t][0]);
          acc[t][1] = __fmaf_rn(__fmul_rn(__int2float_rn(p[g][t][1]), asc[t][1]), s_lo, acc[t][1]);
          acc[t][2] = __fmaf_rn(__fmul_rn(__int2float_rn(p[g][t][2]), asc[t][0]), s_hi, acc[t][2]);
          acc[t][3] = __fmaf_rn(__fmul_rn(__int2float_rn(p[g][t][3]), asc[t][1]), s_hi, acc[t][3]);
        }
      }
    }
  };

  // software pipeline: the MMAs of stage kb + 1 are in flight while stage kb is rescaled and added
  int pa[4][NT][4], pb[4][NT][4];
  uint4 next_lo = load_codes(sc_lo, 0), next_hi = load_codes(sc_hi, 0);
  if (num_kb > 0) issue(0, pa);
  for (int sb = 0; ok && sb * 4 < num_kb; ++sb) {
    const uint32_t code_lo[4] = {next_lo.x, next_lo.y, next_lo.z, next_lo.w};
    const uint32_t code_hi[4] = {next_hi.x, next_hi.y, next_hi.z, next_hi.w};
    next_lo = load_codes(sc_lo, sb + 1);
    next_hi = load_codes(sc_hi, sb + 1);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int kb = sb * 4 + b;
      if (kb >= num_kb) break;
      if (kb + 1 < num_kb) {
        if (b & 1) issue(kb + 1, pa);
        else issue(kb + 1, pb);
        if (!ok) break;
      }
      if (b & 1) accumulate(kb, pb, code_lo[b], code_hi[b]);
      else accumulate(kb, pa, code_lo[b], code_hi[b]);
    }
  }
  if (ok) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int m = (t0 + t) * 8 + lcol + (c & 1);
        const int n = (c & 2) ? n_hi : n_lo;
        if (m < M && n < N) y[static_cast<long>(m) * ldy + n] = acc[t][c];
      }
    }
  }
}

template <int NT>
int launch_decode(const GemmPlan& p, cudaStream_t stream) {
  const int a_rows = p.block_n;
  const int warps = 2 * (a_rows / (8 * NT));
  gemm_o1_decode_kernel<NT><<<p.grid, (kProducerWarps + warps) * 32, kSmemBytesD, stream>>>(
      p.tm_b, p.tm_a, static_cast<const float*>(p.a_scale), static_cast<const uint8_t*>(p.w_scale), p.y, p.M, p.N, p.K,
      p.ldy, a_rows, stages_for(kTileWD + a_rows * 128), p.status);
  return check_cuda(cudaGetLastError(), "gemm_o1_decode_kernel launch");
}

// 8-row activation tiles per warp: one up to 16 rows (two or four compute warps), two above.
int tiles_per_warp(int M) { return M <= 16 ? 1 : 2; }
int a_box_rows(int M) {
  const int unit = 8 * tiles_per_warp(M);
  return (M + unit - 1) / unit * unit;
}

}  // namespace

int init_gemm_o1_decode_attributes() {
  if (int rc = check_cuda(cudaFuncSetAttribute(gemm_o1_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               kSmemBytesD),
                          "cudaFuncSetAttribute(gemm_o1_decode_kernel<1>)"))
    return rc;
  return check_cuda(
      cudaFuncSetAttribute(gemm_o1_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesD),
      "cudaFuncSetAttribute(gemm_o1_decode_kernel<2>)");
}

// Plan for the decode-shape O1 GEMM: tm_b = W map (32-row boxes), tm_a = A map (all activation rows,
// rounded up to whole tiles; rows past M read as zero).
int plan_o1_decode(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale,
                   float* y, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (M <= 0 || M > 64) return fail("plan_o1_decode: M must be in [1, 64]");
  *plan = GemmPlan{};
  plan->variant = 1;
  plan->skinny = 2;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->w_scale = w_scale;
  plan->y = y;
  plan->status = ctx->status;
  plan->block_n = a_box_rows(M);
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_int8, N, K, K, kRowsD, 128)) return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_int8, M, K, K, plan->block_n, 128))
    return rc;
  plan->tm_y = plan->tm_a;
  plan->grid = (N + kRowsD - 1) / kRowsD;
  plan->grid_y = 1;
  return 0;
}

int run_gemm_o1_decode(const GemmPlan& p, cudaStream_t stream) {
  return tiles_per_warp(p.M) == 1 ? launch_decode<1>(p, stream) : launch_decode<2>(p, stream);
}

void describe_gemm_o1_decode(int M, PlanInfo* info) {
  const int nt = tiles_per_warp(M);
  const int a_rows = a_box_rows(M);
  info->symbol = nt == 1 ? "gemm_o1_decode_kernel<1>" : "gemm_o1_decode_kernel<2>";
  info->mma_family = "mma.sync.m16n8k32.s8";
  info->tile_m = a_rows, info->tile_n = kRowsD, info->stages = stages_for(kTileWD + a_rows * 128), info->acc_stages = 0;
  info->threads = (kProducerWarps + 2 * (a_rows / (8 * nt))) * 32, info->cluster = 1;
  info->mma_m = 16, info->mma_n = 8, info->mma_k = 32;
  info->persistent = 0;
}

}  // namespace adg
