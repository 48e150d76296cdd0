// O2 for decode-sized activations (M <= 64): a weight-streaming block-scaled MXFP4 GEMM.
//
// With so few activation rows the 128-row tile of the regular kernel would be almost empty and only
// N/256 CTAs would stream W, so the operands are swapped: the tensor core computes
// Y^T[n, m] = W[n, :] . A[m, :]^T with the 128 MMA rows taken from W and the MMA N extent equal to M
// rounded up to 16.  A 128-row block of W is handled by a cluster of S CTAs (S = 1, 2 or 4, chosen so
// that the grid covers the GPU once): each walks 1/S of K, accumulates in its tensor memory, and the
// partial sums meet in the first CTA's shared memory (distributed shared memory: st.async, whose bytes are
// counted on the first CTA's barrier as they land), which adds them in rank order -- deterministic -- and
// writes the block of Y.  Up to 16 activation rows the partials land in the part of the stage buffers that
// no copy ever writes (the TMA box of A is 16 rows of the 64-row tile); above that they land in the stage
// buffers proper, once the first CTA has told the senders that its MMAs are done.  For O2 the accumulation
// order is free, so the split changes results only within the rounding of the FP32 sums.  (Of a CTA's
// 7600 cycles at M = 1, N = K = 4096 about 900 are set-up, 1400 the first DRAM round trip, 2500 the four
// K slabs and the rest the hand-over of the partial sums and the store; two cluster-wide meetings instead
// of the st.async hand-over cost 1600 cycles more, an earlier split over independent CTAs with a
// last-arriver reduction through global memory more than it saved.)
//
// Scale factors: W's tiled scales are the MMA's A-side scales (128-row atoms as stored), A's tiled
// scales are the B-side scales (row block 0 of A's tiled buffer).
#include <type_traits>

#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kRows = 128;      // W rows per CTA
constexpr int kMaxM = 64;       // activation rows covered by one MMA
constexpr int kStages = 4;
constexpr int kTileW = kRows * 128;
constexpr int kTileA = kMaxM * 128;
constexpr int kSf = 1024;       // two 512-byte atoms (8 K32 blocks) for each side
constexpr int kStageBytes = kTileW + kTileA + 2 * kSf;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
constexpr int kThreads = 256;   // warps 0 and 7 producers (W side, A side), warp 1 MMA, warps 2-5 epilogue, warp 6 scale-factor copier
constexpr int kAccCols = 64;
constexpr int kSfColBase = kAccCols;
constexpr int kSfColsPerStage = 16;  // per K-atom: 4 (W side) + 4 (A side); two K-atoms per stage
constexpr int kTmemCols = 128;

enum : uint32_t { kTagEmpty = 0x2100, kTagFull = 0x2200, kTagAcc = 0x2300, kTagSfFull = 0x2400 };
constexpr int kMaxSplit = 4;
static_assert((kMaxSplit - 1) * kRows * kMaxM * 4 <= kStages * kStageBytes, "the partial sums of the other ranks fit the stage buffers");

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__global__ void __launch_bounds__(kThreads, 2)
gemm_o2_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                      const uint8_t* __restrict__ sf_w, const uint8_t* __restrict__ sf_a, float* __restrict__ y,
                      int M, int N, int K, int ldy, int a_box, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* acc_bar = bars + 2 * kStages;
  uint64_t* sf_full_bar = acc_bar + 1;
  uint64_t* reduce_bar = sf_full_bar + kStages;  // first CTA of a cluster: the other ranks' partial sums have landed
  uint64_t* go_bar = reduce_bar + 1;      // ranks 1..: the first CTA's stage buffers may be written
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(go_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};
  const int split = static_cast<int>(cluster_size());
  const int rank = static_cast<int>(cluster_rank());
  const int nb = blockIdx.x / split;  // 128-row block of W
  const int num_kb_total = (K + 255) / 256;
  const int per_rank = (num_kb_total + split - 1) / split;
  const int kb0 = min(rank * per_rank, num_kb_total), kb1 = min(kb0 + per_rank, num_kb_total);
  const int katoms = static_cast<int>(((K / 32 + 7) / 8) * 2);
  const uint32_t m_pad = static_cast<uint32_t>((M + 15) / 16 * 16);

  // one barrier per thread of the last warp (the barriers are contiguous: full, empty, accumulator, scale copies,
  // reduce, go): a single thread initialising all fifteen one after the other costs several hundred cycles.
  // Arrival counts: full = one per producer warp; reduce = the first CTA's own expect_tx arrival (the senders'
  // bytes complete the phase); all others one.
  if (warp == 7 && lane < 3 * kStages + 3) {
    mbar_init(&bars[lane], lane < kStages ? 2u : 1u);
    fence_mbar_init();
  }
  if (threadIdx.x == 0) *abort_flag = 0;
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
  // every CTA's barriers exist before another CTA of the cluster signals one: arrive now, wait where the first
  // remote access is made (long after, so the wait costs nothing)
  if (split > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  // The one-instruction-at-a-time roles run as converged warps with one elected lane per instruction:
  // a lone thread inside a divergent branch needs 100 - 160 cycles per copy or MMA instruction, which
  // made the producer (four copies per stage) the slowest link of the chain.  The copies of a stage
  // are split over two warps for the same reason.
  const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
  const uint32_t sf_full0 = smem_u32(sf_full_bar);
  if (warp == 0 || warp == 7) {
    int stage = 0;
    uint32_t phase = 0;
    for (int kb = kb0; kb < kb1; ++kb) {
      if (!mbar_wait_warp(empty0 + stage * 8, phase ^ 1u, env, kTagEmpty | stage)) break;
      const uint32_t st = smem0 + stage * kStageBytes;
      const uint32_t bar = full0 + stage * 8;
      if (warp == 0) {
        mbar_expect_tx_elect(bar, kTileW + kSf);
        tma_load_2d_elect(st, &tm_w, bar, kb * 128, nb * kRows);
        bulk_load_elect(st + kTileW + kTileA, sf_w + (static_cast<long>(nb) * katoms + kb * 2) * 512, kSf, bar);
      } else {
        mbar_expect_tx_elect(bar, static_cast<uint32_t>(a_box * 128 + kSf));
        tma_load_2d_elect(st + kTileW, &tm_a, bar, kb * 128, 0);
        bulk_load_elect(st + kTileW + kTileA + kSf, sf_a + static_cast<long>(kb * 2) * 512, kSf, bar);
      }
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = kb0; kb < kb1; ++kb) {
      // the scale-factor warp has copied this stage's scales into tensor memory (which also
      // means the stage's operand tiles have landed)
      ok = mbar_wait_warp(sf_full0 + stage * 8, phase, env, kTagSfFull | stage);
      if (!ok) break;
      tc_fence_after();
      const uint32_t st = smem0 + stage * kStageBytes;
      const uint64_t wdesc = make_desc_sw128(st);
      const uint64_t adesc = make_desc_sw128(st + kTileW);
      const uint32_t sfw_t = tmem_base + kSfColBase + stage * kSfColsPerStage;  // MMA A-side scales (W)
      const uint32_t sfa_t = sfw_t + 8;                                          // MMA B-side scales (A)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t sf_id = (ks & 1) * 2;
        const uint32_t idesc = make_idesc_mxf4(kRows, m_pad, sf_id, sf_id);
        umma_mxf4_elect(tmem_base, wdesc + ks * 2, adesc + ks * 2, idesc, (kb != kb0 || ks != 0) ? 1u : 0u,
                        sfw_t + (ks >> 1) * 4, sfa_t + (ks >> 1) * 4);
      }
      umma_commit_elect(empty0 + stage * 8);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (ok) umma_commit_elect(smem_u32(acc_bar));
  } else if (warp == 6) {
    // scale-factor copier: the four copies per stage are kept off the MMA warp
    int stage = 0;
    uint32_t phase = 0;
    for (int kb = kb0; kb < kb1; ++kb) {
      // the stage's tensor-memory scale columns were last read by MMAs that completed before the
      // stage was handed back to the producers
      if (!mbar_wait_warp(full0 + stage * 8, phase, env, kTagFull | 0x80 | stage)) break;
      tc_fence_after();
      const uint32_t st = smem0 + stage * kStageBytes;
      const uint32_t sfw_t = tmem_base + kSfColBase + stage * kSfColsPerStage;
      const uint32_t sfa_t = sfw_t + 8;
#pragma unroll
      for (int ka = 0; ka < 2; ++ka) {
        tmem_cp_32x128b_warpx4_elect(sfw_t + ka * 4, make_desc_sf(st + kTileW + kTileA + ka * 512));
        tmem_cp_32x128b_warpx4_elect(sfa_t + ka * 4, make_desc_sf(st + kTileW + kTileA + kSf + ka * 512));
      }
      umma_commit_elect(sf_full0 + stage * 8);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  }

  // ---- every thread: the partial sums of a cluster meet in its first CTA (a cluster of one passes straight through)
  // epilogue warps 2-5: lane = one row n of W, registers = the M outputs of that row
  const bool epi = warp >= 2 && warp < 6;
  uint32_t r[2][32];
  bool have = false;
  const int q = warp & 3;
  if (epi) {
    have = kb1 > kb0 ? mbar_wait(acc_bar, 0, env, kTagAcc) : true;
    if (have) {
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      if (kb1 > kb0) {
        tmem_ld_32x32(t_addr, r[0]);
        tmem_ld_32x32(t_addr + 32, r[1]);
        tmem_wait_ld_for(r[0]);
        tmem_wait_ld_for(r[1]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[0][j] = r[1][j] = 0u;
      }
    }
  }
  // The partial sums of ranks 1.. travel to the first CTA with st.async, whose bytes are counted on its barrier as
  // they land: no cluster-wide meeting after the K loop and no release fence in the senders (two meetings cost 2000
  // cycles of a 9000-cycle CTA, a release-arrive per sender 1200).  A unit = 128 rows x 4 floats of one (rank, group
  // of four activation rows) = 2 KB.
  //  * Up to 16 activation rows the TMA box of A covers 16 rows, so rows 16..63 of every stage's A tile (6 KB per
  //    stage) are never written by a copy: stage g receives the units of row group g, one per sender, at any time.
  //  * Above that the units land in the stage buffers proper ([sender][group][row][4 floats]), which the first CTA's
  //    MMAs must have finished reading: it tells every sender so (one remote arrival each) once its accumulator is
  //    complete, and the senders wait for that.
  const bool direct = a_box <= 16;
  if (split > 1) {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // the peers' barriers exist (see the prologue)
    const int row = q * 32 + lane;
    const uint32_t m_groups = (static_cast<uint32_t>(M) + 3u) / 4u;
    auto unit_offset = [&](int sender, int g) -> uint32_t {
      return direct ? static_cast<uint32_t>(g * kStageBytes + kTileW + 16 * 128 + (sender - 1) * 2048)
                    : static_cast<uint32_t>((sender - 1) * (kRows * kMaxM * 4) + g * (kRows * 16));
    };
    if (rank == 0 && threadIdx.x == 64) {  // one thread of the first epilogue warp
      mbar_arrive_expect_tx(reduce_bar, static_cast<uint32_t>(split - 1) * 128u * m_groups * 16u);
      if (!direct && have) {
        for (int p = 1; p < split; ++p) mbar_arrive_cluster(map_to_rank(smem_u32(go_bar), static_cast<uint32_t>(p)));
      }
    }
    auto send = [&](auto gmax) {
      const uint32_t remote_bar = map_to_rank(smem_u32(reduce_bar), 0u);
      const uint32_t remote_base = map_to_rank(smem_u32(smem), 0u);
#pragma unroll
      for (int g = 0; g < decltype(gmax)::value; ++g) {
        if (static_cast<uint32_t>(g) < m_groups) {
          asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                       ::"r"(remote_base + unit_offset(rank, g) + static_cast<uint32_t>(row) * 16u), "r"(r[g >> 3][(g & 7) * 4]),
                       "r"(r[g >> 3][(g & 7) * 4 + 1]), "r"(r[g >> 3][(g & 7) * 4 + 2]), "r"(r[g >> 3][(g & 7) * 4 + 3]),
                       "r"(remote_bar)
                       : "memory");
        }
      }
    };
    auto add = [&](auto gmax) {
#pragma unroll
      for (int other = 1; other < kMaxSplit; ++other) {
        if (other < split) {
#pragma unroll
          for (int g = 0; g < decltype(gmax)::value; ++g) {
            if (static_cast<uint32_t>(g) < m_groups) {
              const float4 p = *reinterpret_cast<const float4*>(smem + unit_offset(other, g) + row * 16);
              uint32_t* dst = &r[g >> 3][(g & 7) * 4];
              dst[0] = __float_as_uint(__uint_as_float(dst[0]) + p.x);
              dst[1] = __float_as_uint(__uint_as_float(dst[1]) + p.y);
              dst[2] = __float_as_uint(__uint_as_float(dst[2]) + p.z);
              dst[3] = __float_as_uint(__uint_as_float(dst[3]) + p.w);
            }
          }
        }
      }
    };
    if (epi && rank != 0) {
      if (direct) {
        send(std::integral_constant<int, 4>{});
      } else if (mbar_wait(go_bar, 0, env, kTagAcc | 0x40u)) {
        send(std::integral_constant<int, kMaxM / 4>{});
      }
    }
    if (epi && rank == 0 && have) {
      // bounded wait for the senders' bytes
      if (!mbar_wait(reduce_bar, 0, env, kTagAcc | 0x80u)) have = false;
      if (have) {
        if (direct) add(std::integral_constant<int, 4>{});
        else add(std::integral_constant<int, kMaxM / 4>{});
      }
    }
  }
  if (epi && have && rank == 0) {
    const int n = nb * kRows + q * 32 + lane;
    if (n < N) {
      // guards in blocks of eight rows: a lone warp pays a few cycles for every instruction it issues
#pragma unroll
      for (int blk = 0; blk < kMaxM / 8; ++blk) {
        if (blk * 8 < M) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int m = blk * 8 + j;
            if (m < M) y[static_cast<long>(m) * ldy + n] = __uint_as_float(r[m >> 5][m & 31]);
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

int init_gemm_skinny_attributes() {
  return check_cuda(
      cudaFuncSetAttribute(gemm_o2_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
      "cudaFuncSetAttribute(gemm_o2_skinny_kernel)");
}

// Plan for Y[M,N] = A_mxfp4 . W_mxfp4^T with M <= 64.
int plan_o2_skinny(GemmPlan* plan, const void* a_mxfp4, const void* sfa_tiled, const void* w_mxfp4, const void* sfb_tiled,
                   float* y, int M, int N, int K, int ldy) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (M <= 0 || M > kMaxM) return fail("plan_o2_skinny: M must be in [1, 64]");
  *plan = GemmPlan{};
  plan->variant = 2;
  plan->skinny = 1;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->sfa = sfa_tiled;
  plan->sfb = sfb_tiled;
  plan->y = y;
  plan->status = ctx->status;
  const uint64_t kbytes = static_cast<uint64_t>(K) / 2;
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_mxfp4, N, kbytes, kbytes, kRows, 128))
    return rc;
  // up to 16 activation rows: a 16-row box, which leaves the rest of every stage's A tile to the partial sums
  plan->block_n = M <= 16 ? 16 : kMaxM;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_mxfp4, M, kbytes, kbytes, plan->block_n, 128))
    return rc;
  plan->tm_y = plan->tm_a;
  // split K over a cluster of 1, 2 or 4 CTAs: as many as keep the grid within what the GPU holds at once (two
  // CTAs per SM fit) and leave every rank at least two K slabs
  const int blocks = (N + kRows - 1) / kRows;
  const int slabs = (K + 255) / 256;
  int split = 1;
  while (split < kMaxSplit && blocks * split * 2 <= 2 * ctx->sm_count && slabs / (split * 2) >= 2) split *= 2;
  plan->grid = blocks * split;
  plan->grid_y = split;  // cluster size
  return 0;
}

int run_gemm_o2_skinny(const GemmPlan& p, cudaStream_t stream) {
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(p.grid));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(p.grid_y);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&config, gemm_o2_skinny_kernel, p.tm_b, p.tm_a, static_cast<const uint8_t*>(p.sfb),
                                       static_cast<const uint8_t*>(p.sfa), p.y, p.M, p.N, p.K, p.ldy, p.block_n, p.status),
                    "gemm_o2_skinny_kernel launch");
}

void describe_gemm_o2_skinny(int M, PlanInfo* info) {
  const int m_pad = (M + 15) / 16 * 16;
  info->symbol = "gemm_o2_skinny_kernel";
  info->mma_family = "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32";
  info->tile_m = m_pad, info->tile_n = kRows, info->stages = kStages, info->acc_stages = 1;
  info->threads = kThreads, info->cluster = 1, info->mma_m = kRows, info->mma_n = m_pad, info->mma_k = 64;
  info->persistent = 0;
}

}  // namespace adg
