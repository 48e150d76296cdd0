// Persistent, warp-specialised tcgen05 GEMMs that accumulate over the whole K extent in tensor
// memory: the O0 FP16 GEMM (kind::f16) and the O2 block-scaled MXFP4 GEMM (kind::mxf4.block_scale).
// They replace the reference's cuBLASLt plan (csrc/sm120/o0_gemm.cu:86-298) and its CUTLASS
// block-scaled GEMM (csrc/sm120/o2_cutlass.cu:35-93, :394-472).
//
//   Y[M,N] (f32) = A[M,K] . W[N,K]^T        both operands K-major, W is used as stored
//
// A third kind, kind::i8 with INT32 accumulation over the whole K extent and one scaling at the end, serves
// the exact-integer O1 variant ("o1x": W pre-shifted per row so that one factor per output column remains).
//
// One CTA per SM walks output tiles of 128 x BLOCK_N.  Roles:
//   warp 0      TMA producer: A/W tiles (128-byte-wide K slabs, 128-byte swizzle) and, for O2, the
//               scale-factor atoms, into a multi-stage shared-memory ring guarded by mbarriers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma and commits completion to the
//               mbarriers
//   warp 2      (O2) one lane copies each stage's scale-factor atoms from shared to tensor memory
//               (tcgen05.cp) and commits to a per-stage mbarrier, so that the MMA lane, whose
//               instruction issue is the scarce resource, issues nothing but MMAs
//   warps 4-11  epilogue: two warps per 32-lane quarter of tensor memory, each draining half of the
//               accumulator's columns into registers in one go (so the accumulator is released
//               after a few hundred cycles), then writing 32x16 blocks through swizzled
//               shared-memory staging with TMA stores while the next tile's MMAs already run
//   warps 12-15 (FUSED kernels only) activation converters: they turn A_int8 into the operand the MMAs
//               read (FP16 for O0, MXFP4 codes + tiled scales for O2) row by row while the tensor cores
//               work, and publish per-row-block counters that the TMA producer waits on before it loads
//               a row block's tiles -- the conversion that the reference runs as a kernel of its own in
//               front of every GEMM (csrc/sm120/o0_gemm.cu:351-531, o2_cutlass.cu:207-259 then :451-472)
//               leaves the critical path.  Registers are re-balanced between the warp groups
//               (setmaxnreg) so that the 512-thread CTA keeps the epilogue's 128-register drain.
// All waits are bounded (see common.cuh); on a timeout the kernel records an error and returns.
#include "common.cuh"
#include "convert_device.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;
constexpr int kEpiWarps = 8;
constexpr int kSfWarp = 2;
constexpr int kPublishWarp = 3;   // FUSED kernels: publishes the converter warps' finished rows        // copies scale factors into tensor memory (O2 only)
constexpr int kFirstEpiWarp = 4;  // the epilogue is warp groups 1 and 2
constexpr int kFirstConvWarp = kFirstEpiWarp + kEpiWarps;  // warp group 3 (FUSED kernels)
constexpr int kAccThreads = kFirstConvWarp * 32;
constexpr int kFusedThreads = kAccThreads + kConvThreads;
// Register budget of a FUSED CTA (512 threads, 128 registers each at launch = the whole file): the
// one-thread roles give back 64, the converters 16, and the two epilogue warp groups take 40 each.
constexpr int kFusedRegsRoles = 64, kFusedRegsConv = 112, kFusedRegsEpi = 168;
static_assert(128 * (kFusedRegsRoles + kFusedRegsConv + 2 * kFusedRegsEpi) == 65536, "register budget");
constexpr int kConvBarrier = 1;  // named barrier of the converter warp group
constexpr int kStagingPerWarp = 2048;  // one 32-row x 16-column FP32 block
constexpr int kGroupM = 8;  // tile rasterisation: sweep 8 row-blocks before moving to the next column-block

enum : uint32_t {  // wait tags reported on timeout
  kTagEmpty = 0x100,
  kTagFull = 0x200,
  kTagTmemEmpty = 0x300,
  kTagTmemFull = 0x400,
  kTagSfFull = 0x500,
  kTagRowsReady = 0x600,
};

// Waits of the roles that have nothing else to do.  In a FUSED kernel the waiting warps share their
// schedulers with the converter warps: they wait suspended by the hardware (mbarrier.try_wait with a time
// hint) instead of probing in a loop, so that their probes do not take the converters' issue slots.
template <bool FUSED>
__device__ __forceinline__ bool role_wait(uint64_t* bar, uint32_t parity, const WaitEnv& env, uint32_t tag) {
  if constexpr (FUSED) {
    return mbar_wait_suspended_a(smem_u32(bar), parity, env.status, smem_u32(const_cast<uint32_t*>(env.abort)), tag);
  } else {
    return mbar_wait(bar, parity, env, tag);
  }
}

// Bounded wait until `*counter` has reached `need` (rows of a row block converted by the converter
// warps of all CTAs).  Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_rows_ready(const uint32_t* counter, uint32_t need, const WaitEnv& env, uint32_t tag) {
  if (ld_acquire_gpu(counter) >= need) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu(counter) < need) {
    __nanosleep(200);
    if ((++spins & 0xFFu) == 0) {
      if (*env.abort) return false;
      if (global_timer_ns() - t0 > kWaitTimeoutNs) {
        *env.abort = 1;
        if (atomicCAS(env.status, 0u, static_cast<uint32_t>(kStatusWaitTimeout)) == 0u) {
          env.status[1] = tag;
          env.status[2] = blockIdx.x;
          env.status[3] = need;
        }
        return false;
      }
    }
  }
  return true;
}

template <int KIND, int BLOCK_N>
struct AccCfg {
  static constexpr bool kScaled = KIND == 2;
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kElemsPerStage = KIND == 2 ? 256 : (KIND == 1 ? 128 : 64);  // K elements covered by 128 bytes
  static constexpr int kTileA = kBlockM * 128;
  static constexpr int kTileB = BLOCK_N * 128;
  static constexpr int kSfa = kScaled ? 1024 : 0;                    // two 512-byte atoms (8 K32 blocks)
  static constexpr int kSfb = kScaled ? (BLOCK_N / 128) * 1024 : 0;  // per 128 rows: two atoms
  static constexpr int kStageBytes = kTileA + kTileB + kSfa + kSfb;
  static constexpr int kAccStages = (kScaled && BLOCK_N == 256) ? 1 : 2;
  static constexpr int kStagingBytes = kEpiWarps * kStagingPerWarp;
  static constexpr int kColsPerWarp = BLOCK_N / 2;  // accumulator columns drained by one epilogue warp
  static constexpr int kSfColsPerStage = kScaled ? 8 + 2 * (BLOCK_N / 32) : 0;
  static constexpr int kSfColBase = kAccStages * BLOCK_N;
  static constexpr int kTmemCols = 512;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
  static_assert(kSfColBase + kStages * kSfColsPerStage <= kTmemCols, "tensor memory over-subscribed");
  static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");
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

template <int KIND, int BLOCK_N, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kAccThreads, 1)
gemm_acc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_y, const uint8_t* __restrict__ sfa,
                const uint8_t* __restrict__ sfb, float* __restrict__ y, int M, int N, int K, int ldy,
                int use_tma_store, uint32_t* status, const FusedConvert conv, const float* __restrict__ row_factor,
                const float* __restrict__ col_factor) {
  using Cfg = AccCfg<KIND, BLOCK_N>;
  // Without the in-kernel converters warp 3 is free: it issues the scale-factor copies of the O2 stages,
  // so that neither producer warp has more than two or three copies to start per stage.
  constexpr bool kSplitProducer = Cfg::kScaled && !FUSED;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* tmem_full_bar = bars + 2 * Cfg::kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + Cfg::kAccStages;
  uint64_t* sf_full_bar = tmem_empty_bar + Cfg::kAccStages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(sf_full_bar + Cfg::kStages);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  uint32_t* conv_done_slot = tmem_base_slot + 2;  // FUSED: rows finished by this CTA's converter warps

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};

  const int num_m = (M + kBlockM - 1) / kBlockM;
  const int num_n = (N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + Cfg::kElemsPerStage - 1) / Cfg::kElemsPerStage;
  const int katoms = static_cast<int>(((K / 32 + 7) / 8) * 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], kSplitProducer ? 2 : 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_full_bar[s], 1);
    }
    for (int a = 0; a < Cfg::kAccStages; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], kEpiWarps);
    }
    *abort_flag = 0;
    *conv_done_slot = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();  // barriers, tensor memory and descriptors are set up: now wait for the kernel in front of this one

  // Warp group 0: the one-thread roles.  (FUSED: each warp group starts its branch with the register
  // re-balancing, all four warps of the group at the same instruction.)
  if (warp < kFirstEpiWarp) {
    if constexpr (FUSED) reg_dealloc<kFusedRegsRoles>();
  }
  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if constexpr (!FUSED) {
      // the whole warp walks the loop converged and one elected lane issues each copy
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, env, kTagEmpty | stage);
          if (!ok) break;
          const uint32_t st = smem0 + stage * Cfg::kStageBytes;
          const uint32_t bar = full0 + stage * 8;
          mbar_expect_tx_elect(bar, kSplitProducer ? Cfg::kTileA + Cfg::kTileB : Cfg::kStageBytes);
          const int x = kb * (KIND == 0 ? 64 : 128);  // tensor-map elements: halves or bytes
          tma_load_2d_elect(st, &tm_a, bar, x, tc.m_blk * kBlockM);
          tma_load_2d_elect(st + Cfg::kTileA, &tm_b, bar, x, tc.n_blk * BLOCK_N);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        uint32_t seen_rows = 0;  // FUSED: the counter of this tile's row block as read one tile earlier
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          const TileCoord tc = tile_coord(tile, num_m, num_n);
          if constexpr (FUSED) {
            // the row block's operand is being written by the converter warps of all CTAs; its counter was
            // requested while the previous tile's loads were issued, so a finished block costs no round trip
            const uint32_t need = static_cast<uint32_t>(min(kBlockM, M - tc.m_blk * kBlockM));
            if (seen_rows < need) {
              ok = wait_rows_ready(conv.ready + tc.m_blk, need, env, kTagRowsReady);
              if (!ok) break;
            }
            fence_proxy_async_all();
            const int next_tile = tile + static_cast<int>(gridDim.x);
            if (next_tile < num_tiles) seen_rows = ld_acquire_gpu(conv.ready + tile_coord(next_tile, num_m, num_n).m_blk);
          }
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = role_wait<FUSED>(&empty_bar[stage], phase ^ 1u, env, kTagEmpty | stage);
            if (!ok) break;
            uint8_t* st = smem + stage * Cfg::kStageBytes;
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
            const int x = kb * (KIND == 0 ? 64 : 128);  // tensor-map elements: halves or bytes
            tma_load_2d(st, &tm_a, &full_bar[stage], x, tc.m_blk * kBlockM);
            tma_load_2d(st + Cfg::kTileA, &tm_b, &full_bar[stage], x, tc.n_blk * BLOCK_N);
            if constexpr (Cfg::kScaled) {
              uint8_t* sfa_s = st + Cfg::kTileA + Cfg::kTileB;
              uint8_t* sfb_s = sfa_s + Cfg::kSfa;
              bulk_load(sfa_s, sfa + (static_cast<long>(tc.m_blk) * katoms + kb * 2) * 512, 1024, &full_bar[stage]);
#pragma unroll
              for (int rb = 0; rb < BLOCK_N / 128; ++rb) {
                const long row_blk = static_cast<long>(tc.n_blk) * (BLOCK_N / 128) + rb;
                bulk_load(sfb_s + rb * 1024, sfb + (row_blk * katoms + kb * 2) * 512, 1024, &full_bar[stage]);
              }
            }
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    if constexpr (!FUSED) {
      // converged warp, one elected lane per instruction
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint32_t sf_full0 = smem_u32(sf_full_bar), tfull0 = smem_u32(tmem_full_bar), tempty0 = smem_u32(tmem_empty_bar);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile % Cfg::kAccStages;
        const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
        ok = mbar_wait_warp(tempty0 + acc * 8, acc_phase ^ 1u, env, kTagTmemEmpty | acc);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_warp(full0 + stage * 8, phase, env, kTagFull | stage);
          if (!ok) break;
          const uint32_t st = smem0 + stage * Cfg::kStageBytes;
          const uint64_t adesc = make_desc_sw128(st);
          const uint64_t bdesc = make_desc_sw128(st + Cfg::kTileA);
          if constexpr (Cfg::kScaled) {
            ok = mbar_wait_warp(sf_full0 + stage * 8, phase, env, kTagSfFull | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
            const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint32_t sf_id = (ks & 1) * 2;
              const uint32_t idesc = make_idesc_mxf4(kBlockM, BLOCK_N, sf_id, sf_id);
              umma_mxf4_elect(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u,
                              sfa_t + (ks >> 1) * 4, sfb_t + (ks >> 1) * (BLOCK_N / 32));
            }
          } else {
            tc_fence_after();
            if constexpr (KIND == 1) {
              constexpr uint32_t idesc = make_idesc(2, kFmtS8, kFmtS8, kBlockM, BLOCK_N);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) umma_i8_elect(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
            } else {
              constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, kBlockM, BLOCK_N);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) umma_f16_elect(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
            }
          }
          umma_commit_elect(empty0 + stage * 8);  // the stage may be refilled once these MMAs have read it
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit_elect(tfull0 + acc * 8);
      }
    } else {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        int local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
          const int acc = local_tile % Cfg::kAccStages;
          const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
          ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, env, kTagTmemEmpty | acc);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait(&full_bar[stage], phase, env, kTagFull | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint64_t adesc = make_desc_sw128(st);
            const uint64_t bdesc = make_desc_sw128(st + Cfg::kTileA);
            if constexpr (Cfg::kScaled) {
              ok = mbar_wait(&sf_full_bar[stage], phase, env, kTagSfFull | stage);
              if (!ok) break;
              tc_fence_after();
              const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
              const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                const uint32_t sf_id = (ks & 1) * 2;
                const uint32_t idesc = make_idesc_mxf4(kBlockM, BLOCK_N, sf_id, sf_id);
                umma_mxf4(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u,
                          sfa_t + (ks >> 1) * 4, sfb_t + (ks >> 1) * (BLOCK_N / 32));
              }
            } else {
              if constexpr (KIND == 1) {
                constexpr uint32_t idesc = make_idesc(2, kFmtS8, kFmtS8, kBlockM, BLOCK_N);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  umma_i8(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
                }
              } else {
                constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, kBlockM, BLOCK_N);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  umma_f16(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
                }
              }
            }
            umma_commit(&empty_bar[stage]);  // the stage may be refilled once these MMAs have read it
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) umma_commit(&tmem_full_bar[acc]);
        }
      }
    }
  } else if (warp == kSfWarp) {
    // ------------------------------- scale-factor copier (O2) -----------------------------------
    if constexpr (Cfg::kScaled && !FUSED) {
      // converged warp, one elected lane per instruction
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), sf_full0 = smem_u32(sf_full_bar);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          // the stage's data has landed; its tensor-memory scale columns were last read by MMAs
          // that completed before the stage was handed back to the producer
          ok = mbar_wait_warp(full0 + stage * 8, phase, env, kTagFull | 0x80 | stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sfa_s = smem0 + stage * Cfg::kStageBytes + Cfg::kTileA + Cfg::kTileB;
          const uint32_t sfb_s = sfa_s + Cfg::kSfa;
          const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
          const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
          for (int ka = 0; ka < 2; ++ka) {
            tmem_cp_32x128b_warpx4_elect(sfa_t + ka * 4, make_desc_sf(sfa_s + ka * 512));
#pragma unroll
            for (int rb = 0; rb < BLOCK_N / 128; ++rb) {
              tmem_cp_32x128b_warpx4_elect(sfb_t + ka * (BLOCK_N / 32) + rb * 4, make_desc_sf(sfb_s + rb * 1024 + ka * 512));
            }
          }
          umma_commit_elect(sf_full0 + stage * 8);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    if constexpr (Cfg::kScaled && FUSED) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
          for (int kb = 0; kb < num_kb; ++kb) {
            // the stage's data has landed; its tensor-memory scale columns were last read by MMAs
            // that completed before the stage was handed back to the producer
            ok = role_wait<FUSED>(&full_bar[stage], phase, env, kTagFull | 0x80 | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint32_t sfa_s = st + Cfg::kTileA + Cfg::kTileB;
            const uint32_t sfb_s = sfa_s + Cfg::kSfa;
            const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
            const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
            for (int ka = 0; ka < 2; ++ka) {
              tmem_cp_32x128b_warpx4(sfa_t + ka * 4, make_desc_sf(sfa_s + ka * 512));
#pragma unroll
              for (int rb = 0; rb < BLOCK_N / 128; ++rb) {
                tmem_cp_32x128b_warpx4(sfb_t + ka * (BLOCK_N / 32) + rb * 4, make_desc_sf(sfb_s + rb * 1024 + ka * 512));
              }
            }
            umma_commit(&sf_full_bar[stage]);
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == kPublishWarp) {
    if constexpr (kSplitProducer) {
      // ------------------------------- scale-factor producer (O2) -------------------------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, env, kTagEmpty | 0x40 | stage);
          if (!ok) break;
          const uint32_t sfa_s = smem0 + stage * Cfg::kStageBytes + Cfg::kTileA + Cfg::kTileB;
          const uint32_t bar = full0 + stage * 8;
          mbar_expect_tx_elect(bar, Cfg::kSfa + Cfg::kSfb);
          bulk_load_elect(sfa_s, sfa + (static_cast<long>(tc.m_blk) * katoms + kb * 2) * 512, 1024, bar);
#pragma unroll
          for (int rb = 0; rb < BLOCK_N / 128; ++rb) {
            const long row_blk = static_cast<long>(tc.n_blk) * (BLOCK_N / 128) + rb;
            bulk_load_elect(sfa_s + Cfg::kSfa + rb * 1024, sfb + (row_blk * katoms + kb * 2) * 512, 1024, bar);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    // ------------------------------- row publisher (FUSED) -------------------------------------
    if constexpr (FUSED) {
      if (lane == 0 && !publish_rows_role(conv, M, blockIdx.x, gridDim.x, smem_u32(conv_done_slot), abort_flag, kWaitTimeoutNs)) {
        *abort_flag = 1;
        if (atomicCAS(status, 0u, static_cast<uint32_t>(kStatusWaitTimeout)) == 0u) {
          status[1] = kTagRowsReady | 0x80u;
          status[2] = blockIdx.x;
          status[3] = 0;
        }
      }
    }
  } else if (warp >= kFirstEpiWarp && warp < kFirstConvWarp) {
    if constexpr (FUSED) reg_alloc<kFusedRegsEpi>();
    // ------------------------------- epilogue ---------------------------------------------------
    const int q = warp & 3;                     // the 32-lane quarter of tensor memory this warp can read
    const int h = (warp - kFirstEpiWarp) >> 2;  // which half of the accumulator's columns this warp drains
    constexpr int CW = Cfg::kColsPerWarp;
    uint8_t* buf = staging + (warp - kFirstEpiWarp) * kStagingPerWarp;
    const uint32_t buf_row = smem_u32(buf) + lane * 64;
    const uint32_t swz = static_cast<uint32_t>((lane >> 1) & 3);
    const uint64_t store_policy = l2_policy_evict_first();
    int local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const int acc = local_tile % Cfg::kAccStages;
      const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
      ok = role_wait<FUSED>(&tmem_full_bar[acc], acc_phase, env, kTagTmemFull | acc);
      if (!ok) break;
      tc_fence_after();
      const int row0 = tc.m_blk * kBlockM + q * 32;
      const int col0 = tc.n_blk * BLOCK_N + h * CW;
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N + h * CW);
      uint32_t r[CW / 32][32];
#pragma unroll
      for (int i = 0; i < CW / 32; ++i) tmem_ld_32x32(t_addr + i * 32, r[i]);
      tmem_wait_ld();
      // this warp's share of the accumulator is in registers: hand the columns back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      if constexpr (KIND == 1) {
        // exact-integer O1: y = RN(float(S) * RN(A_scale[m] * c[n])), S the INT32 sum over all of K
        const float a_m = row0 + lane < M ? __ldg(row_factor + row0 + lane) : 0.0f;
#pragma unroll
        for (int i = 0; i < CW / 32; ++i) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + i * 32 + j;
            const float c_n = col < N ? __ldg(col_factor + col) : 0.0f;
            r[i][j] = __float_as_uint(__fmul_rn(__int2float_rn(static_cast<int>(r[i][j])), __fmul_rn(a_m, c_n)));
          }
        }
      }
      if (use_tma_store) {
#pragma unroll
        for (int c = 0; c < CW / 16; ++c) {
          if (lane == 0) bulk_wait_group_read<0>();  // the previous block has left the staging buffer
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = (c & 1) * 16 + 4 * j;
            const uint32_t addr = buf_row + ((static_cast<uint32_t>(j) ^ swz) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[c >> 1][e]),
                         "r"(r[c >> 1][e + 1]), "r"(r[c >> 1][e + 2]), "r"(r[c >> 1][e + 3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col = col0 + c * 16;
            // Y is written once and never re-read here: marked evict-first so that it does not
            // push the operand tiles, which every CTA re-reads, out of the L2
            if (row0 < M && col < N) tma_store_2d_hint(&tm_y, buf, col, row0, store_policy);
            bulk_commit_group();
          }
        }
      } else {
        const int row = row0 + lane;
        if (row < M) {
          float* dst = y + static_cast<long>(row) * ldy + col0;
#pragma unroll
          for (int j = 0; j < CW; ++j) {
            if (col0 + j < N) dst[j] = __uint_as_float(r[j >> 5][j & 31]);
          }
        }
      }
    }
    if (lane == 0) bulk_wait_group<0>();
  } else if (warp >= kFirstConvWarp) {
    // ------------------------------- activation converters (FUSED) ------------------------------
    if constexpr (FUSED) {
      reg_dealloc<kFusedRegsConv>();
      convert_rows_role<KIND>(conv, M, K, static_cast<int>(threadIdx.x) - kAccThreads, blockIdx.x, gridDim.x, kConvBarrier,
                              smem_u32(conv_done_slot));
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
  if constexpr (FUSED) {
    // the last CTA to get here puts the counters back to zero for the next launch: by then every CTA
    // has finished waiting on them
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(conv.ready + num_m, 1u) == gridDim.x - 1) {
        for (int i = 0; i <= num_m; ++i) conv.ready[i] = 0u;
        __threadfence();
      }
    }
  }
}

template <int KIND, int BLOCK_N, bool FUSED>
int set_attr() {
  using Cfg = AccCfg<KIND, BLOCK_N>;
  return check_cuda(cudaFuncSetAttribute(gemm_acc_kernel<KIND, BLOCK_N, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm_acc_kernel)");
}

template <int KIND, int BLOCK_N, bool FUSED>
int launch(const GemmPlan& p, cudaStream_t stream) {
  using Cfg = AccCfg<KIND, BLOCK_N>;
  FusedConvert conv{};
  if constexpr (FUSED) {
    conv.a_int8 = static_cast<const uint4*>(p.fused_a_int8);
    conv.a_scale = static_cast<const float*>(p.a_scale);
    conv.a_out = p.fused_a_out;
    conv.sf_natural = static_cast<uint8_t*>(p.fused_sf_natural);
    conv.sf_tiled = static_cast<uint8_t*>(const_cast<void*>(p.sfa));
    conv.ready = p.fused_ready;
  }
  return check_cuda(launch_overlapped(gemm_acc_kernel<KIND, BLOCK_N, FUSED>, dim3(p.grid), dim3(FUSED ? kFusedThreads : kAccThreads),
                                      Cfg::kSmemBytes, stream, 1, p.tm_a, p.tm_b, p.tm_y, static_cast<const uint8_t*>(p.sfa),
                                      static_cast<const uint8_t*>(p.sfb), p.y, p.M, p.N, p.K, p.ldy, p.use_tma_store, p.status, conv,
                                      static_cast<const float*>(p.a_scale), static_cast<const float*>(p.col_factor)),
                    "gemm_acc_kernel launch");
}

template <int KIND, bool FUSED>
int launch_n(const GemmPlan& p, cudaStream_t stream) {
  return p.block_n == 256 ? launch<KIND, 256, FUSED>(p, stream) : launch<KIND, 128, FUSED>(p, stream);
}

}  // namespace

int init_gemm_acc_attributes() {
  if (int rc = set_attr<0, 256, false>()) return rc;
  if (int rc = set_attr<0, 128, false>()) return rc;
  if (int rc = set_attr<1, 256, false>()) return rc;
  if (int rc = set_attr<1, 128, false>()) return rc;
  if (int rc = set_attr<2, 256, false>()) return rc;
  if (int rc = set_attr<2, 128, false>()) return rc;
  if (int rc = set_attr<0, 256, true>()) return rc;
  if (int rc = set_attr<0, 128, true>()) return rc;
  if (int rc = set_attr<2, 256, true>()) return rc;
  if (int rc = set_attr<2, 128, true>()) return rc;
  return 0;
}

int run_gemm_acc(const GemmPlan& p, cudaStream_t stream) {
  if (p.fused) {
    if (p.fused_ready == nullptr || p.fused_a_int8 == nullptr || p.fused_a_out == nullptr)
      return fail("run_gemm_acc: a fused plan needs A_int8, the operand buffer and the row counters");
    if (p.variant == 0) return launch_n<0, true>(p, stream);
    if (p.variant == 2) return launch_n<2, true>(p, stream);
    return fail("run_gemm_acc: only O0 and O2 convert their activations inside the GEMM");
  }
  if (p.variant == 0) return launch_n<0, false>(p, stream);
  if (p.variant == 2) return launch_n<2, false>(p, stream);
  if (p.variant == 3) {
    if (p.a_scale == nullptr || p.col_factor == nullptr) return fail("run_gemm_acc: the o1x plan lacks its factors");
    return launch_n<1, false>(p, stream);
  }
  return fail("run_gemm_acc: plan is not an O0/O2/o1x plan");
}

void describe_gemm_acc(int variant, int block_n, bool fused, PlanInfo* info) {
  info->tile_m = kBlockM;
  info->tile_n = block_n;
  info->threads = fused ? kFusedThreads : kAccThreads;
  info->cluster = 1;
  info->persistent = 1;
  info->fused_activation = fused ? 1 : 0;
  info->mma_m = kBlockM;
  info->mma_n = block_n;
  if (variant == 0) {
    info->stages = block_n == 256 ? AccCfg<0, 256>::kStages : AccCfg<0, 128>::kStages;
    info->acc_stages = 2;
    info->mma_k = 16;
    info->symbol = fused ? "gemm_acc_kernel<0,fused>" : "gemm_acc_kernel<0>";
    info->mma_family = "tcgen05.mma.cta_group::1.kind::f16";
  } else if (variant == 2) {
    info->stages = block_n == 256 ? AccCfg<2, 256>::kStages : AccCfg<2, 128>::kStages;
    info->acc_stages = block_n == 256 ? AccCfg<2, 256>::kAccStages : AccCfg<2, 128>::kAccStages;
    info->mma_k = 64;
    info->symbol = fused ? "gemm_acc_kernel<2,fused>" : "gemm_acc_kernel<2>";
    info->mma_family = "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32";
  } else {
    info->stages = block_n == 256 ? AccCfg<1, 256>::kStages : AccCfg<1, 128>::kStages;
    info->acc_stages = 2;
    info->mma_k = 32;
    info->symbol = "gemm_acc_kernel<1>";
    info->mma_family = "tcgen05.mma.cta_group::1.kind::i8";
  }
}

}  // namespace adg
