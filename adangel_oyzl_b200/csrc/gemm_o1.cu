// O1: INT8 tensor-core GEMM whose every K32 partial is rescaled and accumulated in FP32.
// Replaces the reference kernel adangel_o1_tma_warp_specialized (csrc/sm120/o1_gemm.cu:167-333).
//
// For every output element and every K32 group g, in ascending g (reference/o1.py:16-20):
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                      (INT32, exact)
//     acc = acc + float(P) * ((A_scale[m] * 2**(W_scale[n,g]-127)) * 0.5)  (FP32, round-to-nearest each step)
// One tcgen05.mma kind::i8 instruction has K = 32, i.e. it computes exactly one group's partial
// for a 128x128 tile.  Partials are produced two at a time (two MMAs, one commit) into one of two
// 256-column halves of tensor memory, because an MMA into a fresh accumulator followed by its own
// commit costs about a thousand cycles of latency that only back-to-back MMAs amortise.  The
// epilogue warps drain the partials and keep the FP32 accumulators in registers for the whole K
// loop:  u = RN(float(P) * A_scale[m]);  acc = fma(u, 2**(W_scale-128), acc).  The factor
// 2**(W_scale-128) is a power of two, so u * 2**(W_scale-128) is exact and the fused form rounds
// exactly where the reference's multiply-then-add does (barring FP32 underflow of the scale).
//
// Roles (640 threads): warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warp 2 turns
// the tile's UE8M0 weight scales into FP32 factors in a shared-memory ring, warps 4-19 epilogue
// (4 per tensor-memory lane quarter, 32 columns each).  The first warp group hands registers to the
// epilogue warp groups so that each epilogue warp can keep the next partial's tensor-memory load in
// flight while it scales and accumulates the current one (a tensor-memory load takes several
// hundred cycles to return).
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kCtasPerSm = 128 / kBlockN;
constexpr int kStages = kBlockN == 128 ? 6 : 4;  // A 128x128 B + W kBlockN x 128 B (4 groups) each
constexpr int kScStages = 8;    // 4 groups x kBlockN FP32 factors each
constexpr int kPairs = 2;       // tensor-memory halves, each holding the partials of two K32 groups
constexpr int kEpiWarps = 4 * (kBlockN / 32);
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr int kTile = kBlockM * 128;
constexpr int kStageBytes = kTile + kBlockN * 128;
constexpr int kScBytes = 4 * kBlockN * 4;
constexpr int kTmemCols = kPairs * 2 * kBlockN;
constexpr int kEpiRegs = kBlockN == 128 ? 112 : 104;
constexpr int kSmemBytes = kStages * kStageBytes + kScStages * kScBytes + 1024 + 1024;
constexpr int kGroupM = 8;

enum : uint32_t {
  kTagEmpty = 0x1100,
  kTagFull = 0x1200,
  kTagTmemEmpty = 0x1300,
  kTagTmemFull = 0x1400,
  kTagScEmpty = 0x1500,
  kTagScFull = 0x1600,
};

struct TileCoord {
  int m_blk, n_blk;
};
// `n_list`, if given, restricts the launch to some column blocks: n_list[0] of them, listed from n_list[1]
// (the exact-integer O1 variant sends only the column blocks that hold an ineligible W row through here).
template <bool kListed>
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, const int32_t* __restrict__ n_list) {
  const int per_group = kGroupM * num_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(num_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  TileCoord t;
  t.m_blk = first_m + in_group % gsize;
  t.n_blk = in_group / gsize;
  if constexpr (kListed) t.n_blk = __ldg(n_list + 1 + t.n_blk);
  return t;
}

// kDump = true adds the debug store of every INT32 partial, kListed = true the restriction to listed column
// blocks (separate instantiations so that the production kernel carries none of their register pressure:
// its epilogue has no register to spare).
template <bool kDump, bool kListed>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
gemm_o1_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const float* __restrict__ a_scale, const uint8_t* __restrict__ w_scale, float* __restrict__ y,
               int32_t* __restrict__ partial_dump, int M, int N, int K, int ldy, uint32_t* status,
               const uint32_t* __restrict__ only_if_flag, const int32_t* __restrict__ n_list) {
  // second half of a sync-free fallback: run only when the BF16-operand kernel in front refused
  if (only_if_flag != nullptr && *only_if_flag == 0u) return;
  if constexpr (kListed) {
    if (__ldg(n_list) <= 0) return;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kScStages * kScBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + kPairs;
  uint64_t* sc_full_bar = tmem_empty_bar + kPairs;
  uint64_t* sc_empty_bar = sc_full_bar + kScStages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sc_empty_bar + kScStages);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t abort_a = smem_u32(const_cast<uint32_t*>(abort_flag));
  const uint32_t tmem_full_a = smem_u32(tmem_full_bar), tmem_empty_a = smem_u32(tmem_empty_bar);
  const uint32_t sc_full_a = smem_u32(sc_full_bar), sc_empty_a = smem_u32(sc_empty_bar);
  const uint32_t full_a = smem_u32(full_bar), empty_a = smem_u32(empty_bar);

  const int num_m = (M + kBlockM - 1) / kBlockM;
  const int num_n = kListed ? __ldg(n_list) : (N + kBlockN - 1) / kBlockN;
  const int num_tiles = num_m * num_n;
  const int groups = K / 32;
  const int num_kb = (groups + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kPairs; ++s) {
      mbar_init(&tmem_full_bar[s], 1);
      mbar_init(&tmem_empty_bar[s], kEpiWarps);
    }
    for (int s = 0; s < kScStages; ++s) {
      mbar_init(&sc_full_bar[s], 32);
      mbar_init(&sc_empty_bar[s], kEpiWarps);
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
  reg_dealloc<32>();  // 128 threads x 64 registers returned = 512 threads x 16 registers gained below
  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord<kListed>(tile, num_m, num_n, n_list);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_a(empty_a + stage * 8, phase ^ 1u, status, abort_a, kTagEmpty | stage);
          if (!ok) break;
          uint8_t* st = smem + stage * kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(st, &tm_a, &full_bar[stage], kb * 128, tc.m_blk * kBlockM);
          tma_load_2d(st + kTile, &tm_b, &full_bar[stage], kb * 128, tc.n_blk * kBlockN);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    if (lane == 0) {
      int stage = 0, pair = 0;
      uint32_t phase = 0, pair_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(2, kFmtS8, kFmtS8, kBlockM, kBlockN);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; ok && kb < num_kb; ++kb) {
          ok = mbar_wait_a(full_a + stage * 8, phase, status, abort_a, kTagFull | stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_desc_sw128(st);
          const uint64_t bdesc = make_desc_sw128(st + kTile);
          const int ng = min(4, groups - kb * 4);  // K is a multiple of 64, so ng is 2 or 4
          for (int g = 0; g < ng; g += 2) {
            ok = mbar_wait_a(tmem_empty_a + pair * 8, pair_phase ^ 1u, status, abort_a, kTagTmemEmpty | pair);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d = tmem_base + static_cast<uint32_t>(pair * 2 * kBlockN);
            umma_i8(d, adesc + g * 2, bdesc + g * 2, idesc, 0u);
            umma_i8(d + kBlockN, adesc + (g + 1) * 2, bdesc + (g + 1) * 2, idesc, 0u);
            umma_commit_a(tmem_full_a + pair * 8);
            if (++pair == kPairs) {
              pair = 0;
              pair_phase ^= 1u;
            }
          }
          if (ok) umma_commit_a(empty_a + stage * 8);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------- weight-scale factors ---------------------------------------
    // Lane l converts rows l, l+32, ... of the tile's W rows.  The codes of the next K slab are
    // requested before the current slab is converted, so that the global-load latency (these
    // strided 4-byte reads mostly miss the small L1) never sits between two ring slots.
    int scs = 0;
    uint32_t sc_phase = 0;
    bool ok = true;
    const bool vec = (groups & 3) == 0;
    constexpr int kRowsPerLane = kBlockN / 32;
    auto load_codes = [&](int n_blk, int kb, uint32_t (&codes)[kRowsPerLane]) {
#pragma unroll
      for (int i = 0; i < kRowsPerLane; ++i) {
        const int n = n_blk * kBlockN + lane + 32 * i;
        codes[i] = 0;
        if (n < N) {
          const uint8_t* src = w_scale + static_cast<long>(n) * groups + kb * 4;
          if (vec) {
            codes[i] = __ldg(reinterpret_cast<const uint32_t*>(src));
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (kb * 4 + g < groups) codes[i] |= static_cast<uint32_t>(__ldg(src + g)) << (8 * g);
          }
        }
      }
    };
    uint32_t next_codes[kRowsPerLane];
    int tile = blockIdx.x;
    if (tile < num_tiles) load_codes(tile_coord<kListed>(tile, num_m, num_n, n_list).n_blk, 0, next_codes);
    for (; ok && tile < num_tiles; tile += gridDim.x) {
      const int n_blk = tile_coord<kListed>(tile, num_m, num_n, n_list).n_blk;
      for (int kb = 0; kb < num_kb; ++kb) {
        uint32_t codes[kRowsPerLane];
#pragma unroll
        for (int i = 0; i < kRowsPerLane; ++i) codes[i] = next_codes[i];
        if (kb + 1 < num_kb) {
          load_codes(n_blk, kb + 1, next_codes);
        } else if (tile + static_cast<int>(gridDim.x) < num_tiles) {
          load_codes(tile_coord<kListed>(tile + gridDim.x, num_m, num_n, n_list).n_blk, 0, next_codes);
        }
        ok = mbar_wait_a(sc_empty_a + scs * 8, sc_phase ^ 1u, status, abort_a, kTagScEmpty | scs);
        if (!ok) break;
        float* dst = sc_ring + scs * (kScBytes / 4);
#pragma unroll
        for (int i = 0; i < kRowsPerLane; ++i) {
          const int n_local = lane + 32 * i;
          const bool row_ok = n_blk * kBlockN + n_local < N;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const bool valid = row_ok && kb * 4 + g < groups;
            dst[g * kBlockN + n_local] = valid ? ue8m0_half_to_float((codes[i] >> (8 * g)) & 0xFFu) : 0.0f;
          }
        }
        mbar_arrive_a(sc_full_a + scs * 8);
        if (++scs == kScStages) {
          scs = 0;
          sc_phase ^= 1u;
        }
      }
    }
  }
  } else {
    reg_alloc<kEpiRegs>();
    // ------------------------------- epilogue ---------------------------------------------------
    // Each warp owns 32 columns of one lane quarter.  The two partials of a pair go to two register
    // buffers: while one partial is scaled and accumulated, the load of the next is in flight.
    const int q = warp & 3;                     // tensor-memory lane quarter
    const int cs = (warp - kFirstEpiWarp) >> 2;  // 32-column slice of the 128-column partial
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(cs * 32);
    const uint32_t sc_base = smem_u32(sc_ring) + static_cast<uint32_t>(cs * 32 * 4);
    int pair = 0, scs = 0;
    uint32_t pair_phase = 0, sc_phase = 0;
    bool ok = true;

    // Three passes over the partial (in place), each a run of independent instructions, so that
    // the chain convert -> multiply -> fma of one element never stalls the warp.
    auto accumulate = [&](uint32_t (&p)[32], float2 (&acc)[16], const float2 a2, const uint32_t sc) {
#pragma unroll
      for (int j = 0; j < 32; ++j) p[j] = __float_as_uint(__int2float_rn(static_cast<int>(p[j])));
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 u = __fmul2_rn(make_float2(__uint_as_float(p[2 * j]), __uint_as_float(p[2 * j + 1])), a2);
        p[2 * j] = __float_as_uint(u.x);
        p[2 * j + 1] = __float_as_uint(u.y);
      }
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        float4 s;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w) : "r"(sc + j4 * 16));
        acc[2 * j4] = __ffma2_rn(make_float2(__uint_as_float(p[4 * j4]), __uint_as_float(p[4 * j4 + 1])), make_float2(s.x, s.y), acc[2 * j4]);
        acc[2 * j4 + 1] = __ffma2_rn(make_float2(__uint_as_float(p[4 * j4 + 2]), __uint_as_float(p[4 * j4 + 3])), make_float2(s.z, s.w), acc[2 * j4 + 1]);
      }
    };

    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const TileCoord tc = tile_coord<kListed>(tile, num_m, num_n, n_list);
      const int row = tc.m_blk * kBlockM + q * 32 + lane;
      const int col0 = tc.n_blk * kBlockN + cs * 32;
      const float a_m = row < M ? __ldg(a_scale + row) : 0.0f;
      const float2 a2 = make_float2(a_m, a_m);
      float2 acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.0f, 0.0f);
      uint32_t pa[32], pb[32];
      // prologue: the first partial of the tile's first pair
      ok = mbar_wait_a(tmem_full_a + pair * 8, pair_phase, status, abort_a, kTagTmemFull | pair);
      if (!ok) break;
      tc_fence_after();
      tmem_ld_32x32(t_lane + pair * 2 * kBlockN, pa);
      for (int g = 0; ok && g < groups; g += 2) {  // K is a multiple of 64: groups come in pairs
        if ((g & 3) == 0) {
          ok = mbar_wait_a(sc_full_a + scs * 8, sc_phase, status, abort_a, kTagScFull | scs);
          if (!ok) break;
        }
        const uint32_t sc = sc_base + static_cast<uint32_t>(scs * kScBytes + ((g & 3) * kBlockN) * 4);
        // ---- first partial of the pair: wait for it, start loading the second, compute
        tmem_wait_ld_for(pa);
        tmem_ld_32x32(t_lane + (pair * 2 + 1) * kBlockN, pb);
        if constexpr (kDump) {
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) partial_dump[(static_cast<long>(row) * N + col0 + j) * groups + g] = static_cast<int>(pa[j]);
          }
        }
        accumulate(pa, acc, a2, sc);
        // ---- second partial: wait for it, hand the pair back, start loading the next pair's first
        tmem_wait_ld_for(pb);
        // the next pair's first load goes out before this pair is handed back, so that the warp
        // has no load in flight only for the length of one barrier probe
        const int done_pair = pair;
        if (++pair == kPairs) {
          pair = 0;
          pair_phase ^= 1u;
        }
        const bool more = g + 2 < groups;
        if (more) {
          ok = mbar_wait_a(tmem_full_a + pair * 8, pair_phase, status, abort_a, kTagTmemFull | pair);
          if (!ok) break;
          tc_fence_after();
          tmem_ld_32x32(t_lane + pair * 2 * kBlockN, pa);
        }
        tc_fence_before();  // tcgen05.wait::ld is warp-collective: every lane's loads have landed
        if (lane == 0) mbar_arrive_a(tmem_empty_a + done_pair * 8);
        if constexpr (kDump) {
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) partial_dump[(static_cast<long>(row) * N + col0 + j) * groups + g + 1] = static_cast<int>(pb[j]);
          }
        }
        accumulate(pb, acc, a2, sc + kBlockN * 4);
        if ((g & 3) == 2 || !more) {
          __syncwarp();
          if (lane == 0) mbar_arrive_a(sc_empty_a + scs * 8);
          if (++scs == kScStages) {
            scs = 0;
            sc_phase ^= 1u;
          }
        }
      }
      if (ok && row < M) {
        float* dst = y + static_cast<long>(row) * ldy + col0;
        if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            reinterpret_cast<float4*>(dst)[j4] = make_float4(acc[2 * j4].x, acc[2 * j4].y, acc[2 * j4 + 1].x, acc[2 * j4 + 1].y);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
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

int init_gemm_o1_attributes() {
  if (int rc = check_cuda(cudaFuncSetAttribute(gemm_o1_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                          "cudaFuncSetAttribute(gemm_o1_kernel)"))
    return rc;
  if (int rc = check_cuda(cudaFuncSetAttribute(gemm_o1_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                          "cudaFuncSetAttribute(gemm_o1_kernel<listed>)"))
    return rc;
  return check_cuda(cudaFuncSetAttribute(gemm_o1_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                    "cudaFuncSetAttribute(gemm_o1_kernel<dump>)");
}

int o1_block_n() { return kBlockN; }
int o1_ctas_per_sm() { return kCtasPerSm; }

int run_gemm_o1(const GemmPlan& p, cudaStream_t stream) {
  if (p.variant != 1) return fail("run_gemm_o1: plan is not an O1 plan");
  const float* a_scale = static_cast<const float*>(p.a_scale);
  const uint8_t* w_scale = static_cast<const uint8_t*>(p.w_scale);
  if (p.partial_dump != nullptr) {
    if (p.n_list != nullptr) return fail("run_gemm_o1: the partial dump and a column-block list exclude one another");
    gemm_o1_kernel<true, false><<<p.grid, kThreads, kSmemBytes, stream>>>(p.tm_a, p.tm_b, a_scale, w_scale, p.y, p.partial_dump, p.M,
                                                                         p.N, p.K, p.ldy, p.status, p.only_if_flag, nullptr);
  } else if (p.n_list != nullptr) {
    gemm_o1_kernel<false, true><<<p.grid, kThreads, kSmemBytes, stream>>>(p.tm_a, p.tm_b, a_scale, w_scale, p.y, nullptr, p.M, p.N,
                                                                         p.K, p.ldy, p.status, p.only_if_flag, p.n_list);
  } else {
    gemm_o1_kernel<false, false><<<p.grid, kThreads, kSmemBytes, stream>>>(p.tm_a, p.tm_b, a_scale, w_scale, p.y, nullptr, p.M, p.N,
                                                                          p.K, p.ldy, p.status, p.only_if_flag, nullptr);
  }
  return check_cuda(cudaGetLastError(), "gemm_o1_kernel launch");
}

void describe_gemm_o1(PlanInfo* info) {
  info->symbol = "gemm_o1_kernel";
  info->mma_family = "tcgen05.mma.cta_group::1.kind::i8";
  info->tile_m = kBlockM, info->tile_n = kBlockN, info->stages = kStages, info->acc_stages = kPairs;
  info->threads = kThreads, info->cluster = 1, info->mma_m = kBlockM, info->mma_n = kBlockN, info->mma_k = 32;
  info->persistent = 1;
}

}  // namespace adg
