// O0 GEMM on CTA pairs: tcgen05.mma.cta_group::2 over a 256 x 256 output tile.
//
// Two CTAs of a cluster (ranks 0 and 1, on neighbouring SMs) share one tile: each owns 128 rows of A
// and of Y and the 128 x 256 FP32 accumulator for them in its own tensor memory, and each loads only
// HALF of the W tile (128 of its 256 rows) into its shared memory; the pair's tensor cores read both
// halves.  Per 128-byte K slab a CTA therefore brings in 32 KB instead of 48 KB, which buys six
// pipeline stages instead of four and two thirds of the L2 traffic.  One thread of the even CTA (the
// leader) issues every MMA for the pair.
//
// Protocol (all mbarriers live in each CTA's shared memory at the same offsets):
//   full[s]        the LEADER's barrier collects the bytes of all four TMA loads of a stage: the
//                  leader's producer announces 64 KB, both CTAs' loads name the leader's barrier
//   empty[s]       every CTA's producer waits on its own; the leader's MMA thread commits to both
//   tmem_full[a]   every CTA's epilogue waits on its own; the leader commits to both
//   tmem_empty[a]  the LEADER's barrier counts the epilogue warps of both CTAs (the follower's warps
//                  arrive remotely)
// Opt-in (environment variable read by the planner); the single-CTA kernel stays the default.
// All waits are bounded (see common.cuh); the two cluster-wide barriers at start and end are reached
// by every thread after its bounded loops.
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kBlockM = 128;     // rows per CTA
constexpr int kBlockN = 256;     // columns of the pair's tile
constexpr int kHalfN = kBlockN / 2;
constexpr int kStages = 6;
constexpr int kTileA = kBlockM * 128;
constexpr int kTileB = kHalfN * 128;
constexpr int kStageBytes = kTileA + kTileB;
constexpr int kAccStages = 2;
constexpr int kEpiWarps = 8;
constexpr int kThreads = (2 + kEpiWarps + 2) * 32;
constexpr int kStagingPerWarp = 2048;
constexpr int kStagingBytes = kEpiWarps * kStagingPerWarp;
constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 1024;
constexpr int kGroupM = 4;  // tile rasterisation: sweep 4 row-pairs before moving to the next column block
static_assert(kSmemBytes <= 232448, "shared memory over-subscribed");

enum : uint32_t { kTagEmpty = 0x4100, kTagFull = 0x4200, kTagTmemEmpty = 0x4300, kTagTmemFull = 0x4400 };

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
// arrive on `cluster_addr` (any CTA of the cluster) when the pair's MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
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

__global__ void __launch_bounds__(kThreads, 1)
gemm_o0_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_y, float* __restrict__ y, int M, int N, int K, int ldy,
                    int use_tma_store, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + kAccStages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + kAccStages);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

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
  const int num_kb = (K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything of ours reaches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ---------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t full_leader = map_to_cta(smem_u32(full_bar), 0);
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters) {
        const TileCoord tc = tile_coord(tile, num_mp, num_n);
        const int row0 = (tc.m_pair * 2 + static_cast<int>(rank)) * kBlockM;
        const int wrow0 = tc.n_blk * kBlockN + static_cast<int>(rank) * kHalfN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, env, kTagEmpty | stage);
          if (!ok) break;
          uint8_t* st = smem + stage * kStageBytes;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);
          tma_load_2d_pair(st, &tm_a, full_leader + stage * 8, kb * 64, row0);
          tma_load_2d_pair(st + kTileA, &tm_b, full_leader + stage * 8, kb * 64, wrow0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -----------------------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      constexpr uint32_t idesc = make_idesc(1, kFmtF16, kFmtF16, 2 * kBlockM, kBlockN);
      const uint32_t empty_own = smem_u32(empty_bar), empty_peer = map_to_cta(empty_own, peer);
      const uint32_t tfull_own = smem_u32(tmem_full_bar), tfull_peer = map_to_cta(tfull_own, peer);
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++local_tile) {
        const int acc = local_tile % kAccStages;
        const uint32_t acc_phase = static_cast<uint32_t>(local_tile / kAccStages) & 1u;
        ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, env, kTagTmemEmpty | acc);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kBlockN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, env, kTagFull | stage);
          if (!ok) break;
          tc_fence_after();
          const uint32_t st = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_desc_sw128(st);
          const uint64_t bdesc = make_desc_sw128(st + kTileA);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) umma_f16_pair(d_tmem, adesc + ks * 2, bdesc + ks * 2, idesc, (kb | ks) != 0 ? 1u : 0u);
          // both CTAs' copies of the stage may be refilled once these MMAs have read them
          umma_commit_pair(empty_own + stage * 8);
          umma_commit_pair(empty_peer + stage * 8);
          if (++stage == kStages) {
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
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ------------------------------- epilogue (both CTAs) -------------------------------------
    const int q = warp & 3;
    const int h = (warp - 2) >> 2;
    constexpr int CW = kBlockN / 2;
    uint8_t* buf = staging + (warp - 2) * kStagingPerWarp;
    const uint32_t buf_row = smem_u32(buf) + lane * 64;
    const uint32_t swz = static_cast<uint32_t>((lane >> 1) & 3);
    const uint64_t store_policy = l2_policy_evict_first();
    const uint32_t tempty_leader = map_to_cta(smem_u32(tmem_empty_bar), 0);
    int local_tile = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++local_tile) {
      const TileCoord tc = tile_coord(tile, num_mp, num_n);
      const int acc = local_tile % kAccStages;
      const uint32_t acc_phase = static_cast<uint32_t>(local_tile / kAccStages) & 1u;
      ok = mbar_wait(&tmem_full_bar[acc], acc_phase, env, kTagTmemFull | acc);
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
  }

  // neither CTA may leave (or release tensor memory) while the other can still read its shared
  // memory, signal its barriers or run MMAs into its tensor memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

}  // namespace

int init_gemm_pair_attributes() {
  return check_cuda(cudaFuncSetAttribute(gemm_o0_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                    "cudaFuncSetAttribute(gemm_o0_pair_kernel)");
}

// The plan's tm_b must have 128-row boxes (one CTA's half of the W tile); grid = 2 x clusters.
int run_gemm_o0_pair(const GemmPlan& p, cudaStream_t stream) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(p.grid));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&config, gemm_o0_pair_kernel, p.tm_a, p.tm_b, p.tm_y, p.y, p.M, p.N, p.K, p.ldy,
                                       p.use_tma_store, p.status),
                    "gemm_o0_pair_kernel launch");
}

int o0_pair_tile_m() { return 2 * kBlockM; }
int o0_pair_tile_n() { return kBlockN; }

}  // namespace adg
