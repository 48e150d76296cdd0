// O1 for decode-sized activations (M <= 64): the INT8 tensor-core GEMM with per-K32 FP32 rescale,
// with the operands swapped so that the weight rows fill the tensor core's 128 rows.
//
// Semantics are those of gemm_o1_kernel (reference/o1.py:16-20, csrc/sm120/o1_gemm.cu:167-333):
// for every output element and every K32 group g, in ascending g,
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                        (INT32, exact)
//     acc = fma(RN(float(P) * A_scale[m]), 2**(W_scale[n,g]-128), acc)   (FP32)
// which equals the reference's acc + float(P) * ((A_scale*2**(W_scale-127))*0.5) bit for bit.
//
// A CTA owns 128 rows of W and 16 rows of A: one tcgen05.mma kind::i8 (128 x 16 x 32) produces the
// partials P^T[n, m] of one K32 group, four groups (one 128-byte K slab) form a batch that lands in
// 64 tensor-memory columns, and four such batches can be in flight.  The grid is
// (N/128) x ceil(M/16); each CTA walks all of K in order, so the accumulation order per element is
// the reference's and the result does not depend on the grid.  An epilogue thread owns one row n of
// W and 8 of the CTA's 16 activation rows: its weight scale is per thread, the activation scales
// are per register.  While one batch is scaled and accumulated, the tensor-memory load of the next
// is in flight.  A thread needs 100+ cycles to issue one MMA whatever its size, so two warps issue
// (even and odd batches; every batch has its own tensor-memory slot, so they need no ordering).
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kRows = 128;   // W rows per CTA (MMA M)
constexpr int kCols = 16;    // A rows per CTA (MMA N)
constexpr int kStages = 8;
constexpr int kTileW = kRows * 128;
constexpr int kTileA = kCols * 128;
constexpr int kStageBytes = kTileW + kTileA;
constexpr int kSlots = 4;                 // batches of partials in tensor memory
constexpr int kSlotCols = 4 * kCols;      // four K32 groups x 16 columns
constexpr int kTmemCols = kSlots * kSlotCols;
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kColsPerWarp = kCols / (kEpiWarps / 4);  // 8
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;  // warp 0 producer, warps 1-2 MMA, warps 4-11 epilogue
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;

enum : uint32_t { kTagEmpty = 0x3100, kTagFull = 0x3200, kTagSlotEmpty = 0x3300, kTagSlotFull = 0x3400 };

__global__ void __launch_bounds__(kThreads, 1)
gemm_o1_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                      const float* __restrict__ a_scale, const uint8_t* __restrict__ w_scale, float* __restrict__ y,
                      int M, int N, int K, int ldy, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* slot_full_bar = empty_bar + kStages;
  uint64_t* slot_empty_bar = slot_full_bar + kSlots;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(slot_empty_bar + kSlots);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};
  const int nb = blockIdx.x;         // 128-row block of W
  const int m0 = blockIdx.y * kCols;  // first activation row of this CTA
  const int groups = K / 32;
  const int num_kb = (groups + 3) / 4;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&slot_full_bar[s], 1);
      mbar_init(&slot_empty_bar[s], kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_a);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, env, kTagEmpty | stage)) break;
        uint8_t* st = smem + stage * kStageBytes;
        mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
        tma_load_2d(st, &tm_w, &full_bar[stage], kb * 128, nb * kRows);
        tma_load_2d(st + kTileW, &tm_a, &full_bar[stage], kb * 128, m0);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(2, kFmtS8, kFmtS8, kRows, kCols);
      for (int kb = warp - 1; kb < num_kb; kb += 2) {
        const int stage = kb % kStages;
        const uint32_t phase = static_cast<uint32_t>(kb / kStages) & 1u;
        const int slot = kb % kSlots;
        const uint32_t slot_phase = static_cast<uint32_t>(kb / kSlots) & 1u;
        if (!mbar_wait(&full_bar[stage], phase, env, kTagFull | stage)) break;
        if (!mbar_wait(&slot_empty_bar[slot], slot_phase ^ 1u, env, kTagSlotEmpty | slot)) break;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + stage * kStageBytes);
        const uint64_t wdesc = make_desc_sw128(st);
        const uint64_t adesc = make_desc_sw128(st + kTileW);
        const uint32_t d = tmem_base + static_cast<uint32_t>(slot * kSlotCols);
        const int ng = min(4, groups - kb * 4);
        for (int g = 0; g < ng; ++g) umma_i8(d + g * kCols, wdesc + g * 2, adesc + g * 2, idesc, 0u);
        umma_commit(&slot_full_bar[slot]);
        umma_commit(&empty_bar[stage]);
      }
    }
  } else if (warp >= kFirstEpiWarp) {
    // ------------------------------- epilogue ---------------------------------------------------
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const int n = nb * kRows + q * 32 + lane;
    const bool n_ok = n < N;
    const int ch = (warp - kFirstEpiWarp) >> 2;  // which 8 of the CTA's 16 activation rows
    const int mc = m0 + ch * kColsPerWarp;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(ch * kColsPerWarp);
    const uint8_t* sc_row = w_scale + static_cast<long>(n_ok ? n : 0) * groups;
    const bool vec = (groups & 3) == 0;

    float asc[kColsPerWarp], acc[kColsPerWarp];
#pragma unroll
    for (int j = 0; j < kColsPerWarp; ++j) {
      asc[j] = (mc + j < M) ? __ldg(a_scale + mc + j) : 0.0f;
      acc[j] = 0.0f;
    }

    // the four UE8M0 codes of batch kb for this thread's row (absent groups read as code 0 and are
    // never used)
    auto load_codes = [&](int kb) -> uint32_t {
      if (!n_ok || kb >= num_kb) return 0u;
      if (vec) return __ldg(reinterpret_cast<const uint32_t*>(sc_row + kb * 4));
      uint32_t c = 0;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        if (kb * 4 + g < groups) c |= static_cast<uint32_t>(__ldg(sc_row + kb * 4 + g)) << (8 * g);
      return c;
    };
    auto load_batch = [&](int slot, uint32_t (&p)[4][kColsPerWarp]) {
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld_32x8(t_lane + static_cast<uint32_t>(slot * kSlotCols + g * kCols), p[g]);
    };
    auto wait_batch = [&](uint32_t (&p)[4][kColsPerWarp]) {
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_wait_ld_for(p[g]);
    };
    // convert, multiply and accumulate as separate in-place passes: runs of independent instructions
    auto accumulate = [&](uint32_t (&p)[4][kColsPerWarp], uint32_t codes, int ng) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int j = 0; j < kColsPerWarp; ++j) p[g][j] = __float_as_uint(__int2float_rn(static_cast<int>(p[g][j])));
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int j = 0; j < kColsPerWarp; ++j) p[g][j] = __float_as_uint(__fmul_rn(__uint_as_float(p[g][j]), asc[j]));
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (g < ng) {
          const float s = ue8m0_half_to_float((codes >> (8 * g)) & 0xFFu);
#pragma unroll
          for (int j = 0; j < kColsPerWarp; ++j) acc[j] = __fmaf_rn(__uint_as_float(p[g][j]), s, acc[j]);
        }
      }
    };
    auto release = [&](int slot) {
      tc_fence_before();  // tcgen05.wait::ld is warp-collective: every lane's loads have landed
      if (lane == 0) mbar_arrive(&slot_empty_bar[slot]);
    };

    uint32_t pa[4][kColsPerWarp], pb[4][kColsPerWarp];
    int slot = 0;
    uint32_t slot_phase = 0;
    auto next_slot = [&]() {
      if (++slot == kSlots) {
        slot = 0;
        slot_phase ^= 1u;
      }
    };
    bool ok = num_kb > 0 ? mbar_wait(&slot_full_bar[0], 0, env, kTagSlotFull) : false;
    uint32_t codes_a = load_codes(0), codes_b = 0;
    if (ok) {
      tc_fence_after();
      load_batch(0, pa);
    }
    for (int kb = 0; ok && kb < num_kb; kb += 2) {
      // ---- even batch (in pa): wait for it, free its slot, start loading the odd batch, compute
      wait_batch(pa);
      release(slot);
      next_slot();
      const bool has_b = kb + 1 < num_kb;
      if (has_b) {
        ok = mbar_wait(&slot_full_bar[slot], slot_phase, env, kTagSlotFull | slot);
        if (!ok) break;
        tc_fence_after();
        load_batch(slot, pb);
        codes_b = load_codes(kb + 1);
      }
      accumulate(pa, codes_a, min(4, groups - kb * 4));
      if (!has_b) break;
      // ---- odd batch (in pb)
      wait_batch(pb);
      release(slot);
      next_slot();
      if (kb + 2 < num_kb) {
        ok = mbar_wait(&slot_full_bar[slot], slot_phase, env, kTagSlotFull | slot);
        if (!ok) break;
        tc_fence_after();
        load_batch(slot, pa);
        codes_a = load_codes(kb + 2);
      }
      accumulate(pb, codes_b, min(4, groups - (kb + 1) * 4));
    }
    if (ok && n_ok) {
#pragma unroll
      for (int j = 0; j < kColsPerWarp; ++j)
        if (mc + j < M) y[static_cast<long>(mc + j) * ldy + n] = acc[j];
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int init_gemm_o1_skinny_attributes() {
  return check_cuda(
      cudaFuncSetAttribute(gemm_o1_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
      "cudaFuncSetAttribute(gemm_o1_skinny_kernel)");
}

// Plan for the O1 GEMM with M <= 64: tm_b = W map (128-row boxes), tm_a = A map (16-row boxes).
int plan_o1_skinny(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w_int8, const void* w_scale,
                   float* y, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (M <= 0 || M > 64) return fail("plan_o1_skinny: M must be in [1, 64]");
  *plan = GemmPlan{};
  plan->variant = 1;
  plan->skinny = 1;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->w_scale = w_scale;
  plan->y = y;
  plan->status = ctx->status;
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_int8, N, K, K, kRows, 128)) return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_int8, M, K, K, kCols, 128)) return rc;
  plan->tm_y = plan->tm_a;
  plan->grid = (N + kRows - 1) / kRows;
  plan->grid_y = (M + kCols - 1) / kCols;  // 16-row slices of A
  return 0;
}

int run_gemm_o1_skinny(const GemmPlan& p, cudaStream_t stream) {
  gemm_o1_skinny_kernel<<<dim3(p.grid, p.grid_y), kThreads, kSmemBytes, stream>>>(
      p.tm_b, p.tm_a, static_cast<const float*>(p.a_scale), static_cast<const uint8_t*>(p.w_scale), p.y, p.M, p.N, p.K,
      p.ldy, p.status);
  return check_cuda(cudaGetLastError(), "gemm_o1_skinny_kernel launch");
}

void describe_gemm_o1_skinny(PlanInfo* info) {
  info->symbol = "gemm_o1_skinny_kernel";
  info->mma_family = "tcgen05.mma.cta_group::1.kind::i8";
  info->tile_m = kCols, info->tile_n = kRows, info->stages = kStages, info->acc_stages = kSlots;
  info->threads = kThreads, info->cluster = 1, info->mma_m = kRows, info->mma_n = kCols, info->mma_k = 32;
  info->persistent = 0;
}

}  // namespace adg
