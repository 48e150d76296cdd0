// O1: INT8 tensor-core GEMM whose every K32 partial is rescaled and accumulated in FP32.
// Replaces the reference kernel adangel_o1_tma_warp_specialized (csrc/sm120/o1_gemm.cu:167-333).
//
// For every output element and every K32 group g, in ascending g (reference/o1.py:16-20):
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                      (INT32, exact)
//     acc = acc + float(P) * ((A_scale[m] * 2**(W_scale[n,g]-127)) * 0.5)  (FP32, round-to-nearest each step)
// One tcgen05.mma kind::i8 instruction has K = 32, i.e. it computes exactly one group's partial
// for a 128x128 tile.  The partial is written to one of four 128-column tensor-memory slots and
// drained by the epilogue warps, which keep the FP32 accumulators in registers for the whole K
// loop:  u = RN(float(P) * A_scale[m]);  acc = fma(u, 2**(W_scale-128), acc).  The factor
// 2**(W_scale-128) is a power of two, so u * 2**(W_scale-128) is exact and the fused form rounds
// exactly where the reference's multiply-then-add does (barring FP32 underflow of the scale).
//
// Roles (640 threads): warp 0 TMA producer, warp 1 MMA issuer + tensor-memory owner, warp 2 turns
// the tile's UE8M0 weight scales into FP32 factors in a shared-memory ring, warps 4-19 epilogue
// (4 per tensor-memory lane quarter, 32 columns each).
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kStages = 6;      // 32 KB each: A 128x128 B + W 128x128 B (4 groups)
constexpr int kScStages = 8;    // 2 KB each: 4 groups x 128 FP32 factors
constexpr int kSlots = 4;       // tensor-memory partial slots of 128 columns
constexpr int kEpiWarps = 16;
constexpr int kFirstEpiWarp = 4;
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr int kTile = kBlockM * 128;
constexpr int kStageBytes = 2 * kTile;
constexpr int kScBytes = 4 * kBlockN * 4;
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

__global__ void __launch_bounds__(kThreads, 1)
gemm_o1_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const float* __restrict__ a_scale, const uint8_t* __restrict__ w_scale, float* __restrict__ y,
               int32_t* __restrict__ partial_dump, int M, int N, int K, int ldy, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sc_ring = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kScStages * kScBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + kSlots;
  uint64_t* sc_full_bar = tmem_empty_bar + kSlots;
  uint64_t* sc_empty_bar = sc_full_bar + kScStages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sc_empty_bar + kScStages);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};

  const int num_m = (M + kBlockM - 1) / kBlockM;
  const int num_n = (N + kBlockN - 1) / kBlockN;
  const int num_tiles = num_m * num_n;
  const int groups = K / 32;
  const int num_kb = (groups + 3) / 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kSlots; ++s) {
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
    tmem_alloc(tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, env, kTagEmpty | stage);
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
      int stage = 0, slot = 0;
      uint32_t phase = 0, slot_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(2, kFmtS8, kFmtS8, kBlockM, kBlockN);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; ok && kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, env, kTagFull | stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_desc_sw128(st);
          const uint64_t bdesc = make_desc_sw128(st + kTile);
          const int ng = min(4, groups - kb * 4);
          for (int g = 0; g < ng; ++g) {
            ok = mbar_wait(&tmem_empty_bar[slot], slot_phase ^ 1u, env, kTagTmemEmpty | slot);
            if (!ok) break;
            tc_fence_after();
            umma_i8(tmem_base + static_cast<uint32_t>(slot * kBlockN), adesc + g * 2, bdesc + g * 2, idesc, 0u);
            umma_commit(&tmem_full_bar[slot]);
            if (++slot == kSlots) {
              slot = 0;
              slot_phase ^= 1u;
            }
          }
          if (ok) umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------- weight-scale factors ---------------------------------------
    int scs = 0;
    uint32_t sc_phase = 0;
    bool ok = true;
    const bool vec = (groups & 3) == 0;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(&sc_empty_bar[scs], sc_phase ^ 1u, env, kTagScEmpty | scs);
        if (!ok) break;
        float* dst = sc_ring + scs * (kScBytes / 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n_local = lane + 32 * i;
          const int n = tc.n_blk * kBlockN + n_local;
          uint32_t codes = 0;
          uint32_t valid = 0;
          if (n < N) {
            const uint8_t* src = w_scale + static_cast<long>(n) * groups + kb * 4;
            if (vec) {
              codes = __ldg(reinterpret_cast<const uint32_t*>(src));
              valid = 0xF;
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (kb * 4 + g < groups) {
                  codes |= static_cast<uint32_t>(__ldg(src + g)) << (8 * g);
                  valid |= 1u << g;
                }
              }
            }
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            dst[g * kBlockN + n_local] = ((valid >> g) & 1u) ? ue8m0_half_to_float((codes >> (8 * g)) & 0xFFu) : 0.0f;
          }
        }
        mbar_arrive(&sc_full_bar[scs]);
        if (++scs == kScStages) {
          scs = 0;
          sc_phase ^= 1u;
        }
      }
    }
  } else if (warp >= kFirstEpiWarp) {
    // ------------------------------- epilogue ---------------------------------------------------
    // Each warp owns 32 columns of one lane quarter.  A partial is fetched in two 16-column halves
    // into two register buffers so that the tensor-memory load of the next half is in flight while
    // the current half is scaled and accumulated.
    const int q = warp & 3;                     // tensor-memory lane quarter
    const int cs = (warp - kFirstEpiWarp) >> 2;  // 32-column slice of the 128-column partial
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(cs * 32);
    int slot = 0, scs = 0;
    uint32_t slot_phase = 0, sc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const int row = tc.m_blk * kBlockM + q * 32 + lane;
      const int col0 = tc.n_blk * kBlockN + cs * 32;
      const float a_m = row < M ? __ldg(a_scale + row) : 0.0f;
      const float2 a2 = make_float2(a_m, a_m);
      float2 acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.0f, 0.0f);
      uint32_t lo[16], hi[16];
      // prologue: both halves of the tile's first partial
      ok = mbar_wait(&tmem_full_bar[slot], slot_phase, env, kTagTmemFull | slot);
      if (!ok) break;
      tc_fence_after();
      tmem_ld_32x16(t_lane + slot * kBlockN, lo);
      tmem_ld_32x16(t_lane + slot * kBlockN + 16, hi);
      tmem_wait_ld_for(lo);
      for (int g = 0; ok && g < groups; ++g) {
        if ((g & 3) == 0) {
          ok = mbar_wait(&sc_full_bar[scs], sc_phase, env, kTagScFull | scs);
          if (!ok) break;
        }
        const float4* sc = reinterpret_cast<const float4*>(sc_ring + scs * (kScBytes / 4) + (g & 3) * kBlockN + cs * 32);
        if (partial_dump != nullptr) {  // warp-uniform: the wait below is a warp-wide instruction
          tmem_wait_ld_for(hi);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (row >= M) break;
            if (col0 + j < N) partial_dump[(static_cast<long>(row) * N + col0 + j) * groups + g] = static_cast<int>(lo[j]);
            if (col0 + 16 + j < N)
              partial_dump[(static_cast<long>(row) * N + col0 + 16 + j) * groups + g] = static_cast<int>(hi[j]);
          }
        }
        // ---- first half: columns 0..15 of this warp's slice
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 s = sc[j4];
          const float2 f0 = make_float2(__int2float_rn(static_cast<int>(lo[4 * j4])), __int2float_rn(static_cast<int>(lo[4 * j4 + 1])));
          const float2 f1 = make_float2(__int2float_rn(static_cast<int>(lo[4 * j4 + 2])), __int2float_rn(static_cast<int>(lo[4 * j4 + 3])));
          acc[2 * j4] = __ffma2_rn(__fmul2_rn(f0, a2), make_float2(s.x, s.y), acc[2 * j4]);
          acc[2 * j4 + 1] = __ffma2_rn(__fmul2_rn(f1, a2), make_float2(s.z, s.w), acc[2 * j4 + 1]);
        }
        // the second half has arrived: the slot is fully read and can take a new partial
        tmem_wait_ld_for(hi);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[slot]);
        if (++slot == kSlots) {
          slot = 0;
          slot_phase ^= 1u;
        }
        const bool more = g + 1 < groups;
        if (more) {
          ok = mbar_wait(&tmem_full_bar[slot], slot_phase, env, kTagTmemFull | slot);
          if (!ok) break;
          tc_fence_after();
          tmem_ld_32x16(t_lane + slot * kBlockN, lo);  // in flight during the second half's arithmetic
        }
        // ---- second half: columns 16..31
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 s = sc[4 + j4];
          const float2 f0 = make_float2(__int2float_rn(static_cast<int>(hi[4 * j4])), __int2float_rn(static_cast<int>(hi[4 * j4 + 1])));
          const float2 f1 = make_float2(__int2float_rn(static_cast<int>(hi[4 * j4 + 2])), __int2float_rn(static_cast<int>(hi[4 * j4 + 3])));
          acc[8 + 2 * j4] = __ffma2_rn(__fmul2_rn(f0, a2), make_float2(s.x, s.y), acc[8 + 2 * j4]);
          acc[8 + 2 * j4 + 1] = __ffma2_rn(__fmul2_rn(f1, a2), make_float2(s.z, s.w), acc[8 + 2 * j4 + 1]);
        }
        if (more) {
          tmem_wait_ld_for(lo);
          tmem_ld_32x16(t_lane + slot * kBlockN + 16, hi);  // in flight during the next first half
        }
        if ((g & 3) == 3 || !more) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&sc_empty_bar[scs]);
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
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace

int init_gemm_o1_attributes() {
  return check_cuda(
      cudaFuncSetAttribute(gemm_o1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
      "cudaFuncSetAttribute(gemm_o1_kernel)");
}

int run_gemm_o1(const GemmPlan& p, cudaStream_t stream) {
  if (p.variant != 1) return fail("run_gemm_o1: plan is not an O1 plan");
  gemm_o1_kernel<<<p.grid, kThreads, kSmemBytes, stream>>>(
      p.tm_a, p.tm_b, static_cast<const float*>(p.a_scale), static_cast<const uint8_t*>(p.w_scale), p.y,
      p.partial_dump, p.M, p.N, p.K, p.ldy, p.status);
  return check_cuda(cudaGetLastError(), "gemm_o1_kernel launch");
}

}  // namespace adg
