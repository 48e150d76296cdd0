// O0 (kind::f16) and O2 (kind::mxf4.block_scale) GEMMs on CTA pairs: tcgen05.mma.cta_group::2 over a
// 256 x 256 output tile.
//
// Two CTAs of a cluster (ranks 0 and 1, on neighbouring SMs) share one tile: each owns 128 rows of A
// and of Y and the 128 x 256 FP32 accumulator for them in its own tensor memory, and each loads only
// HALF of the W tile (128 of its 256 rows) into its shared memory; the pair's tensor cores read both
// halves.  Per 128-byte K slab a CTA therefore brings in 32 KB instead of 48 KB, which buys six
// pipeline stages instead of four and two thirds of the L2 traffic.  One thread of the even CTA (the
// leader) issues every MMA for the pair.  For O2 every CTA also loads the scale factors of its own 128
// rows of A and of all 256 rows of the W tile (through 2-D tensor maps over the tiled scale arrays, so
// that these loads, too, can signal the leader's barrier), and one more thread of the leader issues the
// shared -> tensor-memory copies, which run in both CTAs, each from its own shared memory.
//
// Protocol (all mbarriers live in each CTA's shared memory at the same offsets):
//   full[s]        the LEADER's barrier collects the bytes of all four TMA loads of a stage: the
//                  leader's producer announces 64 KB, both CTAs' loads name the leader's barrier
//   empty[s]       every CTA's producer waits on its own; the leader's MMA thread commits to both
//   tmem_full[a]   every CTA's epilogue waits on its own; the leader commits to both
//   tmem_empty[a]  the LEADER's barrier counts the epilogue warps of both CTAs (the follower's warps
//                  arrive remotely)
//   sf_full[s]     (O2) the leader's copier thread commits the stage's scale-factor copies to it
// FUSED kernels add a fourth warp group to every CTA that converts A_int8 into the operand (FP16 for O0, MXFP4
// codes + tiled scales for O2) while the tensor cores run; each producer waits for the row counters of its
// own 128 rows before loading them (see gemm_acc.cu for the role and the register re-balancing).
// All waits are bounded (see common.cuh); the two cluster-wide barriers at start and end are reached
// by every thread after its bounded loops.
#include "common.cuh"
#include "convert_device.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;     // rows per CTA
constexpr int kBlockN = 256;     // columns of the pair's tile
constexpr int kHalfN = kBlockN / 2;
constexpr int kTileA = kBlockM * 128;
constexpr int kTileB = kHalfN * 128;
constexpr int kEpiWarps = 8;
constexpr int kSfWarp = 2;
constexpr int kPublishWarp = 3;   // FUSED kernels: publishes the converter warps' finished rows
constexpr int kFirstEpiWarp = 4;  // the epilogue is warp groups 1 and 2
constexpr int kFirstConvWarp = kFirstEpiWarp + kEpiWarps;  // warp group 3 (FUSED kernels)
constexpr int kThreads = kFirstConvWarp * 32;
constexpr int kFusedThreads = kThreads + kConvThreads;
constexpr int kFusedRegsRoles = 64, kFusedRegsConv = 112, kFusedRegsEpi = 168;  // see gemm_acc.cu
static_assert(128 * (kFusedRegsRoles + kFusedRegsConv + 2 * kFusedRegsEpi) == 65536, "register budget");
constexpr int kConvBarrier = 1;
constexpr int kStagingPerWarp = 2048;
constexpr int kStagingBytes = kEpiWarps * kStagingPerWarp;
constexpr int kGroupM = 4;  // tile rasterisation: sweep 4 row-pairs before moving to the next column block

template <int KIND>
struct PairCfg {
  static constexpr bool kScaled = KIND == 2;
  static constexpr int kStages = kScaled ? 5 : 6;
  static constexpr int kElemsPerStage = kScaled ? 256 : 64;  // K elements covered by 128 bytes
  static constexpr int kSfa = kScaled ? 1024 : 0;            // own 128 rows: two 512-byte atoms (8 K32 blocks)
  static constexpr int kSfb = kScaled ? 2048 : 0;            // all 256 rows of the W tile
  static constexpr int kStageBytes = kTileA + kTileB + kSfa + kSfb;
  static constexpr int kAccStages = kScaled ? 1 : 2;
  static constexpr int kSfColsPerStage = kScaled ? 8 + 2 * (kBlockN / 32) : 0;
  static constexpr int kSfColBase = kAccStages * kBlockN;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 1024;
  static_assert(kStageBytes % 1024 == 0, "stages keep the 1024-byte alignment of the swizzled tiles");
  static_assert(kSfColBase + kStages * kSfColsPerStage <= 512, "tensor memory over-subscribed");
  static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");
};

enum : uint32_t { kTagEmpty = 0x4100, kTagFull = 0x4200, kTagTmemEmpty = 0x4300, kTagTmemFull = 0x4400, kTagSfFull = 0x4500,
                  kTagRowsReady = 0x4600 };

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

// Bounded wait until `*counter` has reached `need` (see gemm_acc.cu).
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

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of the pair protocol: the bytes are counted on the barrier of the even CTA
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxf4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// In both CTAs: 32 rows x 16 bytes of the CTA's own shared memory into 4 columns of its own tensor
// memory, replicated into the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_pair_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// arrive on `cluster_addr` (any CTA of the cluster) when the pair's MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

// ---- the same instructions issued by a converged warp (all 32 lanes call, one elected lane issues): a lone
// thread inside a divergent branch needs 100 - 160 cycles per copy or MMA instruction
__device__ __forceinline__ void tma_load_2d_pair_elect(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "@P cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      "}\n" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                    uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, P;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "@P tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_mxf4_pair_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p, P;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "@P tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_pair_32x128b_warpx4_elect(uint32_t taddr, uint64_t sdesc) {
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "@P tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n"
      "}\n" ::"r"(taddr), "l"(sdesc)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_elect(uint32_t cluster_addr) {
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "@P tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n" ::"r"(cluster_addr)
      : "memory");
}

struct TileCoord {
  int m_pair, n_blk;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_mp, int num_n) {
  const int per_group = kGroupM * num_n;
  const int group = tile / per_group;
  const int first = group * kGroupM;
  const int gsize = min(num_mp - first, kGroupM);
  const int in_group = tile - group * per_group;
  TileCoord t;
  t.m_pair = first + in_group % gsize;
  t.n_blk = in_group / gsize;
  return t;
}

template <int KIND, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_y, const __grid_constant__ CUtensorMap tm_sfa,
                 const __grid_constant__ CUtensorMap tm_sfb, float* __restrict__ y, int M, int N, int K, int ldy,
                 int use_tma_store, uint32_t* status, const FusedConvert conv) {
  using Cfg = PairCfg<KIND>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kStages;
  uint64_t* sf_full_bar = bars + 2 * Cfg::kStages;  // (O2) the stage's scale factors are in tensor memory
  uint64_t* tmem_full_bar = bars + 3 * Cfg::kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + Cfg::kAccStages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + Cfg::kAccStages);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  uint32_t* conv_done_slot = tmem_base_slot + 2;  // FUSED: rows finished by this CTA's converter warps

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  const int num_mp = (M + 2 * kBlockM - 1) / (2 * kBlockM);
  const int num_n = (N + kBlockN - 1) / kBlockN;
  const int num_tiles = num_mp * num_n;
  const int num_kb = (K + Cfg::kElemsPerStage - 1) / Cfg::kElemsPerStage;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_full_bar[s], 1);
    }
    for (int a = 0; a < Cfg::kAccStages; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * kEpiWarps);
    }
    *abort_flag = 0;
    *conv_done_slot = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_y);
    if constexpr (Cfg::kScaled) {
      tma_prefetch_desc(&tm_sfa);
      tma_prefetch_desc(&tm_sfb);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, 512);
    tmem_relinquish_pair();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything of ours reaches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();  // set-up done: now wait for the kernel in front of this one in the stream

  // Warp group 0: the one-thread roles.  (FUSED: each warp group starts its branch with the register
  // re-balancing, all four warps of the group at the same instruction.)
  if (warp < kFirstEpiWarp) {
    if constexpr (FUSED) reg_dealloc<kFusedRegsRoles>();
  }
  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------------
    if constexpr (!FUSED) {
      // converged warp, one elected lane per instruction
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem), full_own = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint32_t full_leader = map_to_cta(full_own, 0);
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        const TileCoord tc = tile_coord(tile, num_mp, num_n);
        const int m_blk = tc.m_pair * 2 + static_cast<int>(rank);
        const int row0 = m_blk * kBlockM;
        const int wrow0 = tc.n_blk * kBlockN + static_cast<int>(rank) * kHalfN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, env, kTagEmpty | stage);
          if (!ok) break;
          const uint32_t st = smem0 + stage * Cfg::kStageBytes;
          if (rank == 0) mbar_expect_tx_elect(full_own + stage * 8, 2 * Cfg::kStageBytes);
          const uint32_t bar = full_leader + stage * 8;
          const int x = kb * (KIND == 0 ? 64 : 128);  // tensor-map elements: halves or bytes
          tma_load_2d_pair_elect(st, &tm_a, bar, x, row0);
          tma_load_2d_pair_elect(st + kTileA, &tm_b, bar, x, wrow0);
          if constexpr (Cfg::kScaled) {
            // the scale maps are [row block][32-bit words of the block's atoms]: 256 words = the two
            // atoms of this 256-element K slab
            tma_load_2d_pair_elect(st + kTileA + kTileB, &tm_sfa, bar, kb * 256, m_blk);
            tma_load_2d_pair_elect(st + kTileA + kTileB + Cfg::kSfa, &tm_sfb, bar, kb * 256, tc.n_blk * 2);
          }
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
        const uint32_t full_leader = map_to_cta(smem_u32(full_bar), 0);
        uint32_t seen_rows = 0;  // FUSED: the counter of this tile's row block as read one tile earlier
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
          const TileCoord tc = tile_coord(tile, num_mp, num_n);
          const int m_blk = tc.m_pair * 2 + static_cast<int>(rank);
          const int row0 = m_blk * kBlockM;
          const int wrow0 = tc.n_blk * kBlockN + static_cast<int>(rank) * kHalfN;
          if constexpr (FUSED) {
            // this CTA's 128 rows of the operand are being written by the converter warps of all CTAs
            // (a pair's second row block may lie wholly beyond M: nothing to wait for, the loads read zeros)
            const int rows_left = M - row0;
            if (rows_left > 0 && seen_rows < static_cast<uint32_t>(min(kBlockM, rows_left))) {
              ok = wait_rows_ready(conv.ready + m_blk, static_cast<uint32_t>(min(kBlockM, rows_left)), env, kTagRowsReady);
              if (!ok) break;
            }
            fence_proxy_async_all();
            // request the next tile's counter now: it arrives while this tile's loads are issued
            const int next_tile = tile + num_clusters;
            seen_rows = 0;
            if (next_tile < num_tiles) {
              const int next_blk = tile_coord(next_tile, num_mp, num_n).m_pair * 2 + static_cast<int>(rank);
              if (next_blk * kBlockM < M) seen_rows = ld_acquire_gpu(conv.ready + next_blk);
            }
          }
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = role_wait<FUSED>(&empty_bar[stage], phase ^ 1u, env, kTagEmpty | stage);
            if (!ok) break;
            uint8_t* st = smem + stage * Cfg::kStageBytes;
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * Cfg::kStageBytes);
            const uint32_t bar = full_leader + stage * 8;
            const int x = kb * (KIND == 0 ? 64 : 128);  // tensor-map elements: halves or bytes
            tma_load_2d_pair(st, &tm_a, bar, x, row0);
            tma_load_2d_pair(st + kTileA, &tm_b, bar, x, wrow0);
            if constexpr (Cfg::kScaled) {
              // the scale maps are [row block][32-bit words of the block's atoms]: 256 words = the two
              // atoms of this 256-element K slab
              tma_load_2d_pair(st + kTileA + kTileB, &tm_sfa, bar, kb * 256, m_blk);
              tma_load_2d_pair(st + kTileA + kTileB + Cfg::kSfa, &tm_sfb, bar, kb * 256, tc.n_blk * 2);
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
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if constexpr (!FUSED) {
      if (rank == 0) {
        // converged warp, one elected lane per instruction
        int stage = 0;
        uint32_t phase = 0;
        int local_tile = 0;
        bool ok = true;
        const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), sf_full0 = smem_u32(sf_full_bar);
        const uint32_t tempty0 = smem_u32(tmem_empty_bar);
        const uint32_t empty_own = smem_u32(empty_bar), empty_peer = map_to_cta(empty_own, peer);
        const uint32_t tfull_own = smem_u32(tmem_full_bar), tfull_peer = map_to_cta(tfull_own, peer);
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++local_tile) {
          const int acc = local_tile % Cfg::kAccStages;
          const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
          ok = mbar_wait_warp(tempty0 + acc * 8, acc_phase ^ 1u, env, kTagTmemEmpty | acc);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBlockN);
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait_warp(full0 + stage * 8, phase, env, kTagFull | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem0 + stage * Cfg::kStageBytes;
            const uint64_t adesc = make_desc_sw128(st);
            const uint64_t bdesc = make_desc_sw128(st + kTileA);
            if constexpr (Cfg::kScaled) {
              ok = mbar_wait_warp(sf_full0 + stage * 8, phase, env, kTagSfFull | stage);
              if (!ok) break;
              tc_fence_after();
              const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
              const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                const uint32_t sf_id = (ks & 1) * 2;
                const uint32_t idesc = make_idesc_mxf4(2 * kBlockM, kBlockN, sf_id, sf_id);
                umma_mxf4_pair_elect(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u,
                                     sfa_t + (ks >> 1) * 4, sfb_t + (ks >> 1) * (kBlockN / 32));
              }
            } else {
              constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, 2 * kBlockM, kBlockN);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                umma_f16_pair_elect(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
            }
            // both CTAs' copies of the stage may be refilled once these MMAs have read them
            umma_commit_pair_elect(empty_own + stage * 8);
            umma_commit_pair_elect(empty_peer + stage * 8);
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) {
            umma_commit_pair_elect(tfull_own + acc * 8);
            umma_commit_pair_elect(tfull_peer + acc * 8);
          }
        }
      }
    } else {
      if (lane == 0 && rank == 0) {
        int stage = 0;
        uint32_t phase = 0;
        int local_tile = 0;
        bool ok = true;
        const uint32_t empty_own = smem_u32(empty_bar), empty_peer = map_to_cta(empty_own, peer);
        const uint32_t tfull_own = smem_u32(tmem_full_bar), tfull_peer = map_to_cta(tfull_own, peer);
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++local_tile) {
          const int acc = local_tile % Cfg::kAccStages;
          const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
          ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, env, kTagTmemEmpty | acc);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBlockN);
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait(&full_bar[stage], phase, env, kTagFull | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint64_t adesc = make_desc_sw128(st);
            const uint64_t bdesc = make_desc_sw128(st + kTileA);
            if constexpr (Cfg::kScaled) {
              ok = mbar_wait(&sf_full_bar[stage], phase, env, kTagSfFull | stage);
              if (!ok) break;
              tc_fence_after();
              const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
              const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                const uint32_t sf_id = (ks & 1) * 2;
                const uint32_t idesc = make_idesc_mxf4(2 * kBlockM, kBlockN, sf_id, sf_id);
                umma_mxf4_pair(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u,
                               sfa_t + (ks >> 1) * 4, sfb_t + (ks >> 1) * (kBlockN / 32));
              }
            } else {
              constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, 2 * kBlockM, kBlockN);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) umma_f16_pair(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
            }
            // both CTAs' copies of the stage may be refilled once these MMAs have read them
            umma_commit_pair(empty_own + stage * 8);
            umma_commit_pair(empty_peer + stage * 8);
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) {
            umma_commit_pair(tfull_own + acc * 8);
            umma_commit_pair(tfull_peer + acc * 8);
          }
        }
      }
    }
  } else if (warp == kSfWarp) {
    // ------------------------------- scale-factor copier (O2, leader CTA only) ----------------
    if constexpr (Cfg::kScaled && !FUSED) {
      if (rank == 0) {
        // converged warp, one elected lane per instruction
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), sf_full_own = smem_u32(sf_full_bar);
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
          for (int kb = 0; kb < num_kb; ++kb) {
            // both CTAs' scale factors of the stage have landed; the stage's tensor-memory scale
            // columns were last read by MMAs that completed before the stage was handed back
            ok = mbar_wait_warp(full0 + stage * 8, phase, env, kTagFull | 0x80 | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem0 + stage * Cfg::kStageBytes;
            const uint32_t sfa_s = st + kTileA + kTileB;
            const uint32_t sfb_s = sfa_s + Cfg::kSfa;
            const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
            const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
            for (int ka = 0; ka < 2; ++ka) {
              tmem_cp_pair_32x128b_warpx4_elect(sfa_t + ka * 4, make_desc_sf(sfa_s + ka * 512));
#pragma unroll
              for (int rb = 0; rb < kBlockN / 128; ++rb) {
                tmem_cp_pair_32x128b_warpx4_elect(sfb_t + ka * (kBlockN / 32) + rb * 4,
                                                  make_desc_sf(sfb_s + rb * 1024 + ka * 512));
              }
            }
            umma_commit_pair_elect(sf_full_own + stage * 8);
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    if constexpr (Cfg::kScaled && FUSED) {
      if (lane == 0 && rank == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const uint32_t sf_full_own = smem_u32(sf_full_bar);
        for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
          for (int kb = 0; kb < num_kb; ++kb) {
            // both CTAs' scale factors of the stage have landed; the stage's tensor-memory scale
            // columns were last read by MMAs that completed before the stage was handed back
            ok = role_wait<FUSED>(&full_bar[stage], phase, env, kTagFull | 0x80 | stage);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem_u32(smem + stage * Cfg::kStageBytes);
            const uint32_t sfa_s = st + kTileA + kTileB;
            const uint32_t sfb_s = sfa_s + Cfg::kSfa;
            const uint32_t sfa_t = tmem_base + Cfg::kSfColBase + stage * Cfg::kSfColsPerStage;
            const uint32_t sfb_t = sfa_t + 8;
#pragma unroll
            for (int ka = 0; ka < 2; ++ka) {
              tmem_cp_pair_32x128b_warpx4(sfa_t + ka * 4, make_desc_sf(sfa_s + ka * 512));
#pragma unroll
              for (int rb = 0; rb < kBlockN / 128; ++rb) {
                tmem_cp_pair_32x128b_warpx4(sfb_t + ka * (kBlockN / 32) + rb * 4, make_desc_sf(sfb_s + rb * 1024 + ka * 512));
              }
            }
            umma_commit_pair(sf_full_own + stage * 8);
            if (++stage == Cfg::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == kPublishWarp) {
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
    // ------------------------------- epilogue (both CTAs) -------------------------------------
    const int q = warp & 3;
    const int h = (warp - kFirstEpiWarp) >> 2;
    constexpr int CW = kBlockN / 2;
    uint8_t* buf = staging + (warp - kFirstEpiWarp) * kStagingPerWarp;
    const uint32_t buf_row = smem_u32(buf) + lane * 64;
    const uint32_t swz = static_cast<uint32_t>((lane >> 1) & 3);
    const uint64_t store_policy = l2_policy_evict_first();
    const uint32_t tempty_leader = map_to_cta(smem_u32(tmem_empty_bar), 0);
    int local_tile = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++local_tile) {
      const TileCoord tc = tile_coord(tile, num_mp, num_n);
      const int acc = local_tile % Cfg::kAccStages;
      const uint32_t acc_phase = static_cast<uint32_t>(local_tile / Cfg::kAccStages) & 1u;
      ok = role_wait<FUSED>(&tmem_full_bar[acc], acc_phase, env, kTagTmemFull | acc);
      if (!ok) break;
      tc_fence_after();
      const int row0 = (tc.m_pair * 2 + static_cast<int>(rank)) * kBlockM + q * 32;
      const int col0 = tc.n_blk * kBlockN + h * CW;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * kBlockN + h * CW);
      uint32_t r[CW / 32][32];
#pragma unroll
      for (int i = 0; i < CW / 32; ++i) tmem_ld_32x32(t_addr + i * 32, r[i]);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + acc * 8);
      if (use_tma_store) {
#pragma unroll
        for (int c = 0; c < CW / 16; ++c) {
          if (lane == 0) bulk_wait_group_read<0>();
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
    // ------------------------------- activation converters (FUSED, both CTAs) ------------------
    if constexpr (FUSED) {
      reg_dealloc<kFusedRegsConv>();
      convert_rows_role<KIND>(conv, M, K, static_cast<int>(threadIdx.x) - kThreads, blockIdx.x, gridDim.x, kConvBarrier,
                              smem_u32(conv_done_slot));
    }
  }

  // neither CTA may leave (or release tensor memory) while the other can still read its shared
  // memory, signal its barriers or run MMAs into its tensor memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
  if constexpr (FUSED) {
    // the last CTA to get here zeroes the row counters for the next launch (see gemm_acc.cu)
    if (threadIdx.x == 0) {
      const int num_m = (M + kBlockM - 1) / kBlockM;
      __threadfence();
      if (atomicAdd(conv.ready + num_m, 1u) == gridDim.x - 1) {
        for (int i = 0; i <= num_m; ++i) conv.ready[i] = 0u;
        __threadfence();
      }
    }
  }
}

template <int KIND, bool FUSED>
int launch_pair(const GemmPlan& p, cudaStream_t stream) {
  FusedConvert conv{};
  if constexpr (FUSED) {
    conv.a_int8 = static_cast<const uint4*>(p.fused_a_int8);
    conv.a_scale = static_cast<const float*>(p.a_scale);
    conv.a_out = p.fused_a_out;
    conv.sf_natural = static_cast<uint8_t*>(p.fused_sf_natural);
    conv.sf_tiled = static_cast<uint8_t*>(const_cast<void*>(p.sfa));
    conv.ready = p.fused_ready;
  }
  return check_cuda(launch_overlapped(gemm_pair_kernel<KIND, FUSED>, dim3(static_cast<unsigned>(p.grid)),
                                      dim3(FUSED ? kFusedThreads : kThreads), PairCfg<KIND>::kSmemBytes, stream, 2, p.tm_a, p.tm_b,
                                      p.tm_y, p.tm_sfa, p.tm_sfb, p.y, p.M, p.N, p.K, p.ldy, p.use_tma_store, p.status, conv),
                    "gemm_pair_kernel launch");
}

template <int KIND, bool FUSED>
int set_pair_attr() {
  return check_cuda(cudaFuncSetAttribute(gemm_pair_kernel<KIND, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PairCfg<KIND>::kSmemBytes),
                    "cudaFuncSetAttribute(gemm_pair_kernel)");
}

}  // namespace

int init_gemm_pair_attributes() {
  if (int rc = set_pair_attr<0, false>()) return rc;
  if (int rc = set_pair_attr<2, false>()) return rc;
  if (int rc = set_pair_attr<0, true>()) return rc;
  return set_pair_attr<2, true>();
}

// The plan's tm_b must have 128-row boxes (one CTA's half of the W tile); grid = 2 x clusters; an O2
// plan also carries the tensor maps of the two tiled scale arrays.
int run_gemm_pair(const GemmPlan& p, cudaStream_t stream) {
  if (p.fused) {
    if (p.fused_ready == nullptr || p.fused_a_int8 == nullptr || p.fused_a_out == nullptr)
      return fail("run_gemm_pair: a fused plan needs A_int8, the operand buffer and the row counters");
    if (p.variant == 0) return launch_pair<0, true>(p, stream);
    if (p.variant == 2) return launch_pair<2, true>(p, stream);
  } else {
    if (p.variant == 0) return launch_pair<0, false>(p, stream);
    if (p.variant == 2) return launch_pair<2, false>(p, stream);
  }
  return fail("run_gemm_pair: plan is not an O0/O2 plan");
}

int pair_tile_m() { return 2 * kBlockM; }
int pair_tile_n() { return kBlockN; }

void describe_gemm_pair(int variant, bool fused, PlanInfo* info) {
  info->tile_m = 2 * kBlockM;
  info->tile_n = kBlockN;
  info->threads = fused ? kFusedThreads : kThreads;
  info->cluster = 2;
  info->persistent = 1;
  info->fused_activation = fused ? 1 : 0;
  info->mma_m = 2 * kBlockM;
  info->mma_n = kBlockN;
  if (variant == 0) {
    info->stages = PairCfg<0>::kStages;
    info->acc_stages = PairCfg<0>::kAccStages;
    info->mma_k = 16;
    info->symbol = fused ? "gemm_pair_kernel<0,fused>" : "gemm_pair_kernel<0>";
    info->mma_family = "tcgen05.mma.cta_group::2.kind::f16";
  } else {
    info->stages = PairCfg<2>::kStages;
    info->acc_stages = PairCfg<2>::kAccStages;
    info->mma_k = 64;
    info->symbol = fused ? "gemm_pair_kernel<2,fused>" : "gemm_pair_kernel<2>";
    info->mma_family = "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32";
  }
}

}  // namespace adg
