// O1 with the weight scale folded into the tensor-core operand: the K32 partials leave the tensor
// core already multiplied by 2**(W_scale-128), as FP32, and exact.
//
// The O1 recurrence (reference reference/o1.py:16-20, kernel csrc/sm120/o1_gemm.cu:167-333), for every
// output element and every K32 group g in ascending order:
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                         (exact integer, |P| <= 48768)
//     acc = acc + float(P) * ((A_scale[m] * 2**(W_scale[n,g]-127)) * 0.5)   (FP32, rounded each step)
// Because the weight's factor is a power of two, RN(float(P) * A_scale * 2**x) = RN(float(P) * 2**x *
// A_scale) as long as nothing under- or overflows, and float(P) * 2**x is exactly representable.  So
// the operands are handed to the tensor core as BF16 -- A as the integers themselves (8 significant
// bits), W as e2m1 * 2**(W_scale-127) (2 significant bits, BF16's 8-bit exponent) -- and one K32
// group is two kind::f16 MMAs (K = 16 each) with FP32 accumulation: all products and all their partial
// sums are integer multiples of 2**(W_scale-128) below 2**24 of them, hence exact.  The epilogue is
// left with one multiply by A_scale[m] and one add per partial and element: no integer-to-float
// conversion, no per-column factor, no scale ring in shared memory, no scale warp.  Measured at
// 4096^3: 323 us against 414 us for the INT8-operand kernel, bit-identical; converting A to BF16
// costs another 12 us per call, and W takes two bytes per element instead of one.
//
// Preconditions (checked on the device by the conversion kernels, which set bits in `range_flag`):
// W scale codes in [48, 208] and A scales in [2**-46, 2**30], so that no intermediate leaves the
// normal FP32/BF16 range.  When the flag is set this kernel records an error status and returns
// without computing; the INT8 kernel (gemm_o1.cu) covers every input.
//
// Roles (640 threads): warp 0 TMA producer; warps 1 and 2 MMA issuers (warp 1 owns tensor memory);
// warps 4-19 epilogue (4 per tensor-memory lane quarter, 32 columns each); warp 3 only completes the
// first warp group, which hands its registers to the epilogue.  One 128-byte K slab (64 BF16 = two
// K32 groups) per pipeline stage.  Tensor memory holds four 128-column buffers, one K32 partial
// each, handed over one by one: issuer 0 fills buffers 0 and 2 with the even groups, issuer 1
// buffers 1 and 3 with the odd groups (the two MMAs of a group must come from one thread, in order;
// different groups are independent), and an epilogue warp gives a buffer back as soon as its 32
// columns are in registers -- in the middle of the previous partial's arithmetic -- and asks for the
// next partial before its arithmetic if that partial is already there.  The epilogue arithmetic is packed (two
// elements per instruction), which frees issue slots for the hand-over instructions.  Measured at 4096^3: 375 us with two-group buffers and
// one issuer, 365 us with per-group buffers, 342 us with the second issuer, 335 us with the early
// request, 326 us with the next buffer released in the middle of the arithmetic, 323 us with the
// one-thread roles waiting suspended, 283 us with packed arithmetic, 274 us with the role warps converged
// and one elected lane per copy / MMA instruction; the kernel (before packing)
// without the arithmetic takes 199 us, so the hand-over chain
// (MMA -> commit -> load -> release, about a thousand cycles, over four buffers) and the arithmetic
// (137 us, near the FP32 pipe's rate) add up instead of overlapping.
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kStages = 6;      // A 128 x 128 B + W 128 x 128 B each: two K32 groups
constexpr int kBufs = 4;         // 128-column tensor-memory buffers, one K32 partial each
constexpr int kFirstEpiWarp = 4;
// Geometry of the epilogue by the number of tensor-memory columns one epilogue warp owns (CW): 32 -> 16 warps
// (four per scheduler), 64 -> 8 warps (two per scheduler, twice as much arithmetic between two hand-overs;
// measured 293 us against 283 us at 4096^3, same bits, so 32 is what is built).
// Registers: the first warp group keeps kRoleRegs per thread and hands the rest to the epilogue warps.
constexpr int kColsPerEpiWarp = 32;
template <int CW>
struct EpiCfg {
  static constexpr int kEpiWarps = 4 * (kBlockN / CW);
  static constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
  static constexpr int kLaunchRegs = (65536 / kThreads) / 8 * 8;  // registers per thread at launch
  static constexpr int kRoleRegs = 32;
  static constexpr int kEpiRegs = kLaunchRegs + (kLaunchRegs - kRoleRegs) * 4 / kEpiWarps / 8 * 8;
  static_assert(128 * kRoleRegs + kEpiWarps * 32 * kEpiRegs <= 65536, "register budget");
  static_assert(kEpiRegs <= 248, "register budget");
};
constexpr int kTile = kBlockM * 128;
constexpr int kStageBytes = kTile + kBlockN * 128;
constexpr int kTmemCols = kBufs * kBlockN;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
constexpr int kGroupM = 8;
constexpr uint32_t kFmtBF16 = 1;  // kind::f16 operand format: bfloat16
static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");

enum : uint32_t {
  kTagEmpty = 0x5100,
  kTagFull = 0x5200,
  kTagTmemEmpty = 0x5300,
  kTagTmemFull = 0x5400,
};

// The one-thread roles wait suspended by the hardware: their probe loops would take issue slots from
// the four arithmetic warps of their scheduler (-1 % measured).
// (suspending the epilogue warps' waits as well changes nothing).
#define ADG_ROLE_WAIT mbar_wait_suspended_a

struct TileCoord {
  int m_blk, n_blk;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n) {
  const int per_group = kGroupM * num_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(num_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  TileCoord t;
  t.m_blk = first_m + in_group % gsize;
  t.n_blk = in_group / gsize;
  return t;
}

template <int CW>
__global__ void __launch_bounds__(EpiCfg<CW>::kThreads, 1)
gemm_o1_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const float* __restrict__ a_scale, float* __restrict__ y, const uint32_t* __restrict__ range_flag,
                    int quiet_refusal, int M, int N, int K, int ldy, uint32_t* status) {
  pdl_launch_dependents();
  pdl_wait();  // the range flag below is written by the conversion kernel in front of this one
  // operands outside the exact range: refuse, before any barrier or tensor memory exists -- loudly (an
  // error status for the next check) unless the caller watches the flag itself and falls back
  if (range_flag != nullptr) {
    const uint32_t flag = *range_flag;
    if (flag != 0u) {
      if (!quiet_refusal && threadIdx.x == 0 && atomicCAS(status, 0u, static_cast<uint32_t>(kStatusOperandRange)) == 0u) {
        status[1] = flag;
        status[2] = blockIdx.x;
        status[3] = 0;
      }
      return;
    }
  }
  constexpr int kEpiWarps = EpiCfg<CW>::kEpiWarps;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + kBufs;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + kBufs);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t abort_a = smem_u32(const_cast<uint32_t*>(abort_flag));
  const uint32_t tmem_full_a = smem_u32(tmem_full_bar), tmem_empty_a = smem_u32(tmem_empty_bar);
  const uint32_t full_a = smem_u32(full_bar), empty_a = smem_u32(empty_bar);

  const int num_m = (M + kBlockM - 1) / kBlockM;
  const int num_n = (N + kBlockN - 1) / kBlockN;
  const int num_tiles = num_m * num_n;
  const int num_pairs = K / 64;  // K is a multiple of 64: K32 groups come in pairs, one pair per stage

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 2);  // both issuers commit the MMAs that read the stage
    }
    for (int s = 0; s < kBufs; ++s) {
      mbar_init(&tmem_full_bar[s], 1);
      mbar_init(&tmem_empty_bar[s], kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp < kFirstEpiWarp) {
    reg_dealloc<EpiCfg<CW>::kRoleRegs>();  // what this warp group returns is what the epilogue warps gain below
    // The one-instruction roles run as converged warps with one elected lane per instruction: a lone thread
    // inside a divergent branch needs 100 - 160 cycles per copy or MMA instruction.  All lanes wait
    // suspended on the same barrier and see the same outcome; a vote per probe would cost the arithmetic
    // warps of the scheduler more issue slots than the elected issue saves (308 us instead of 274 us).
    if (warp == 0) {
      // ------------------------------- TMA producer -------------------------------------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        for (int kb = 0; kb < num_pairs; ++kb) {
          ok = mbar_wait_suspended_a(empty_a + stage * 8, phase ^ 1u, status, abort_a, kTagEmpty | stage);
          if (!ok) break;
          const uint32_t st = smem0 + stage * kStageBytes;
          const uint32_t bar = full_a + stage * 8;
          mbar_expect_tx_elect(bar, kStageBytes);
          tma_load_2d_elect(st, &tm_a, bar, kb * 64, tc.m_blk * kBlockM);
          tma_load_2d_elect(st + kTile, &tm_b, bar, kb * 64, tc.n_blk * kBlockN);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else if (warp == 1 || warp == 2) {
      // ------------------------------- two MMA issuers: warp 1 takes the even K32 groups, warp 2 the odd
      const int id = warp - 1;
      int stage = 0, buf = id;
      uint32_t phase = 0, buf_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(1, kFmtBF16, kFmtBF16, kBlockM, kBlockN);
      const uint32_t smem0 = smem_u32(smem);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; ok && kb < num_pairs; ++kb) {
          ok = mbar_wait_suspended_a(full_a + stage * 8, phase, status, abort_a, kTagFull | stage);
          if (!ok) break;
          ok = mbar_wait_suspended_a(tmem_empty_a + buf * 8, buf_phase ^ 1u, status, abort_a, kTagTmemEmpty | buf);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem0 + stage * kStageBytes;
          const uint64_t adesc = make_desc_sw128(st) + id * 4;
          const uint64_t bdesc = make_desc_sw128(st + kTile) + id * 4;
          const uint32_t d = tmem_base + static_cast<uint32_t>(buf * kBlockN);
          // one K32 group: two K16 MMAs into a fresh buffer
          umma_f16_elect(d, adesc, bdesc, idesc, 0u);
          umma_f16_elect(d, adesc + 2, bdesc + 2, idesc, 1u);
          umma_commit_elect(tmem_full_a + buf * 8);
          umma_commit_elect(empty_a + stage * 8);
          buf ^= 2;
          if (buf == id) buf_phase ^= 1u;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    reg_alloc<EpiCfg<CW>::kEpiRegs>();
    // ------------------------------- epilogue ---------------------------------------------------
    // Each warp owns 32 columns of one lane quarter and alternates between two register buffers:
    // while one partial is scaled and accumulated, the load of the next is in flight.
    const int q = warp & 3;                     // tensor-memory lane quarter
    const int cs = (warp - kFirstEpiWarp) >> 2;  // CW-column slice of the 128-column partial
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(cs * CW);
    int pair = 0;  // tensor-memory buffer of the next partial
    uint32_t pair_phase = 0;
    bool ok = true;

    // The arithmetic (accumulate_part below) is two passes, each a run of independent instructions:
    // u = RN(partial * A_scale), acc = RN(acc + u), two elements per instruction (mul.rn.f32x2, add.rn.f32x2).
    // The FP32 pipe needs two cycles for a packed instruction, which leaves every other issue slot of the
    // scheduler to the other warps' hand-over instructions: 283 us against 326 us with scalar arithmetic at
    // 4096^3, same bits.  This translation unit is compiled with -fmad=false: left to itself the assembler
    // contracts the packed multiply and add into one fused multiply-add -- a single rounding where the
    // recurrence has two, which changes 30 % of the results by an ulp.

    // elements of a partial handled before the next buffer is released (8, 16 and 24 measure alike)
    constexpr int kSplit = CW / 2;
    // elements [lo, hi) of a partial (both even)
    auto accumulate_part = [&](uint32_t (&p)[CW], float2 (&acc)[CW / 2], const float a, const int lo, const int hi) {
      // two elements per instruction: the FP32 pipe needs two cycles for each, which leaves every other
      // issue slot of the scheduler to the other warps' hand-over instructions.  This translation unit is
      // compiled with -fmad=false so that the multiply and the add stay two roundings.
      uint64_t a2;
      asm("mov.b64 %0, {%1, %1};" : "=l"(a2) : "r"(__float_as_uint(a)));
#pragma unroll
      for (int j = 0; j < CW / 2; ++j) {
        if (2 * j >= lo && 2 * j < hi) {
          uint64_t v;
          asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(p[2 * j]), "r"(p[2 * j + 1]));
          asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(v), "l"(a2));
          asm("mov.b64 {%0, %1}, %2;" : "=r"(p[2 * j]), "=r"(p[2 * j + 1]) : "l"(v));
        }
      }
#pragma unroll
      for (int j = 0; j < CW / 2; ++j) {
        if (2 * j >= lo && 2 * j < hi) {
          uint64_t v, c;
          asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(p[2 * j]), "r"(p[2 * j + 1]));
          asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "r"(__float_as_uint(acc[j].x)), "r"(__float_as_uint(acc[j].y)));
          asm("add.rn.f32x2 %0, %1, %2;" : "=l"(c) : "l"(c), "l"(v));
          uint32_t x, y2;
          asm("mov.b64 {%0, %1}, %2;" : "=r"(x), "=r"(y2) : "l"(c));
          acc[j] = make_float2(__uint_as_float(x), __uint_as_float(y2));
        }
      }
    };

    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const int row = tc.m_blk * kBlockM + q * 32 + lane;
      const int col0 = tc.n_blk * kBlockN + cs * CW;
      const float a_m = row < M ? __ldg(a_scale + row) : 0.0f;
      float2 acc[CW / 2];
#pragma unroll
      for (int j = 0; j < CW / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);
      uint32_t pa[CW], pb[CW];
      // CW columns of this warp's lane quarter -> registers (one or two 32-column loads)
      auto load_partial = [&](uint32_t taddr, uint32_t (&dst)[CW]) {
#pragma unroll
        for (int i = 0; i < CW / 32; ++i) tmem_ld_32x32(taddr + i * 32, *reinterpret_cast<uint32_t(*)[32]>(&dst[i * 32]));
      };
      auto wait_partial = [&](uint32_t (&dst)[CW]) {
        if constexpr (CW == 32) {
          tmem_wait_ld_for(dst);
        } else {
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < CW; ++i) asm volatile("" : "+r"(dst[i]));  // no use of the registers ahead of the wait
        }
      };
      // Per-partial hand-over: a buffer goes back to the MMA thread as soon as its 32 columns are in
      // registers; the load of partial i+1 is in flight while partial i is scaled and accumulated.
      auto next_buf = [&]() {
        if (++pair == kBufs) {
          pair = 0;
          pair_phase ^= 1u;
        }
      };
      // The partial in `cur` has landed and its buffer is released.  The next partial is requested
      // first (if it is there), and its buffer is released in the MIDDLE of the current partial's
      // arithmetic, as soon as its load can have landed -- not after the arithmetic.
      auto release_buf = [&]() {
        tc_fence_before();
        if (lane == 0) mbar_arrive_a(tmem_empty_a + pair * 8);
        next_buf();
      };
      ok = mbar_wait_a(tmem_full_a + pair * 8, pair_phase, status, abort_a, kTagTmemFull | pair);
      if (!ok) break;
      tc_fence_after();
      load_partial(t_lane + pair * kBlockN, pa);
      wait_partial(pa);
      release_buf();
#define ADG_STEP(cur, nxt, more)                                                                              \
  {                                                                                                           \
    bool issued = false;                                                                                      \
    if ((more) && mbar_test_wait_a(tmem_full_a + pair * 8, pair_phase)) {                                     \
      tc_fence_after();                                                                                       \
      load_partial(t_lane + pair * kBlockN, nxt);                                                             \
      issued = true;                                                                                          \
    }                                                                                                         \
    accumulate_part(cur, acc, a_m, 0, kSplit);                                                                \
    if (issued) {                                                                                             \
      wait_partial(nxt);                                                                                      \
      release_buf();                                                                                          \
    }                                                                                                         \
    accumulate_part(cur, acc, a_m, kSplit, CW);                                                               \
    if ((more) && !issued) {                                                                                  \
      ok = mbar_wait_a(tmem_full_a + pair * 8, pair_phase, status, abort_a, kTagTmemFull | pair);             \
      if (!ok) break;                                                                                         \
      tc_fence_after();                                                                                       \
      load_partial(t_lane + pair * kBlockN, nxt);                                                             \
      wait_partial(nxt);                                                                                      \
      release_buf();                                                                                          \
    }                                                                                                         \
  }
      for (int kb = 0; ok && kb < num_pairs; ++kb) {
        ADG_STEP(pa, pb, true)
        ADG_STEP(pb, pa, kb + 1 < num_pairs)
      }
#undef ADG_STEP
      if (ok && row < M) {
        float* dst = y + static_cast<long>(row) * ldy + col0;
        if (col0 + CW <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
          for (int j4 = 0; j4 < CW / 4; ++j4) {
            reinterpret_cast<float4*>(dst)[j4] = make_float4(acc[2 * j4].x, acc[2 * j4].y, acc[2 * j4 + 1].x, acc[2 * j4 + 1].y);
          }
        } else {
#pragma unroll
          for (int j = 0; j < CW / 2; ++j) {
            if (col0 + 2 * j < N) dst[2 * j] = acc[j].x;
            if (col0 + 2 * j + 1 < N) dst[2 * j + 1] = acc[j].y;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int init_gemm_o1_bf16_attributes() {
  return check_cuda(cudaFuncSetAttribute(gemm_o1_bf16_kernel<kColsPerEpiWarp>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                    "cudaFuncSetAttribute(gemm_o1_bf16_kernel)");
}

int o1_bf16_block_n() { return kBlockN; }

int run_gemm_o1_bf16(const GemmPlan& p, cudaStream_t stream) {
  if (p.variant != 1 || !p.o1_bf16) return fail("run_gemm_o1_bf16: plan is not an O1 BF16-operand plan");
  return check_cuda(launch_overlapped(gemm_o1_bf16_kernel<kColsPerEpiWarp>, dim3(p.grid), dim3(EpiCfg<kColsPerEpiWarp>::kThreads),
                                      kSmemBytes, stream, 1, p.tm_a, p.tm_b, static_cast<const float*>(p.a_scale), p.y, p.range_flag,
                                      p.quiet_refusal, p.M, p.N, p.K, p.ldy, p.status),
                    "gemm_o1_bf16_kernel launch");
}

void describe_gemm_o1_bf16(PlanInfo* info) {
  info->symbol = "gemm_o1_bf16_kernel";
  info->mma_family = "tcgen05.mma.cta_group::1.kind::f16 (bf16 operands; exact integer partials)";
  info->tile_m = kBlockM, info->tile_n = kBlockN, info->stages = kStages, info->acc_stages = kBufs;
  info->threads = EpiCfg<kColsPerEpiWarp>::kThreads, info->cluster = 1, info->mma_m = kBlockM, info->mma_n = kBlockN, info->mma_k = 16;
  info->persistent = 1;
}

}  // namespace adg
