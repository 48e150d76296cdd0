// O1 for the smallest activations (decode, M <= 16): the integer dot products on dp4a, the FP32
// rescale chain handed round a ring of warps, on 32-row blocks of W so that the whole GPU streams
// the weights.
//
// Semantics are those of gemm_o1_kernel (reference/o1.py:16-20, csrc/sm120/o1_gemm.cu:167-333):
// for every output element and every K32 group g, in ascending g,
//     P   = sum_{k in g} A_int8[m,k] * W_int8[n,k]                        (INT32, exact)
//     t   = RN(float(P) * A_scale[m])
//     acc = fma(t, 2**(W_scale[n,g]-128), acc)                            (FP32)
// which equals the reference's acc + float(P) * ((A_scale*2**(W_scale-127))*0.5) bit for bit: P is
// exact in any order, and the FP32 steps are the same operations in the same order.
//
// Only the last line is a chain; P and t of different groups are independent.  With a handful of
// activation rows the tensor-core formulation spends its time on fixed costs per K slab (issue, commit,
// tensor-memory load, hand-over between warps: about 1100 cycles per 128-byte slab whatever M is), and a
// single warp that does everything for its rows needs 650 cycles per slab because a lone warp issues
// one dependent instruction every few cycles.  Here a CTA owns 32 rows of W (lane = row, N = 4096 gives
// 128 CTAs) and its eight warps take the K slabs in turn: warp w computes P and t of slabs w, w + 8, ...
// ahead of time, then waits for the accumulators from the warp of the previous slab, applies its four
// fma per output and passes them on through shared memory.  The chain costs one hand-over and 4 fma
// per slab instead of the whole slab's arithmetic.
//
// Loads: every warp refills the shared-memory slot it has just read with the slab 16 further on (TMA,
// 128-byte swizzle so that the 32 rows of a warp fall into different banks; the slot count is a multiple
// of the ring, so a slot always belongs to the same warp and needs no "empty" barrier).
#include "codecs.cuh"
#include "common.cuh"
#include "launch.h"

namespace adg {

namespace {

constexpr int kRowsD = 32;             // W rows per CTA: one per lane
// bytes of W per slab (128 K elements): INT8 image, or the packed MXFP4 nibbles themselves
__host__ __device__ constexpr int tile_w_bytes(bool packed) { return kRowsD * (packed ? 64 : 128); }

enum : uint32_t { kTagFullD = 0x3600, kTagTokenD = 0x3700 };

// MT activation rows per thread, T slabs per turn, RING warps.  Every warp owns T shared-memory slots.
__host__ __device__ constexpr int a_rows_for(int mt) { return mt < 8 ? 8 : mt; }  // whole 8-row swizzle atoms
__host__ __device__ constexpr int slot_bytes_for(int mt, bool packed) { return tile_w_bytes(packed) + a_rows_for(mt) * 128; }
__host__ __device__ constexpr int smem_bytes_for(int mt, int t, int ring, bool packed) {
  return t * ring * slot_bytes_for(mt, packed) + ring * mt * 32 * 4 + 1024 + 512;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ int dot32(const uint4& w0, const uint4& w1, const uint4& a0, const uint4& a1) {
  int p = __dp4a(static_cast<int>(w0.x), static_cast<int>(a0.x), 0);
  p = __dp4a(static_cast<int>(w0.y), static_cast<int>(a0.y), p);
  p = __dp4a(static_cast<int>(w0.z), static_cast<int>(a0.z), p);
  p = __dp4a(static_cast<int>(w0.w), static_cast<int>(a0.w), p);
  p = __dp4a(static_cast<int>(w1.x), static_cast<int>(a1.x), p);
  p = __dp4a(static_cast<int>(w1.y), static_cast<int>(a1.y), p);
  p = __dp4a(static_cast<int>(w1.z), static_cast<int>(a1.z), p);
  p = __dp4a(static_cast<int>(w1.w), static_cast<int>(a1.w), p);
  return p;
}

// Wait for the accumulators of the previous turn.  Every lane probes by itself (no vote per probe: the
// hand-over is the chain's critical path) and the warp agrees on the outcome once at the end.  Bounded
// by a probe count instead of the timer.
__device__ __forceinline__ bool token_wait(uint32_t bar, uint32_t parity, const WaitEnv& env, uint32_t tag) {
  bool ok = true;
  uint32_t spins = 0;
  while (!mbar_test_wait_a(bar, parity)) {
    if ((++spins & 0xFFFu) == 0) {
      if (*env.abort) {
        ok = false;
        break;
      }
      if (spins >= (1u << 25)) {  // seconds: nothing is coming
        *env.abort = 1;
        if (atomicCAS(env.status, 0u, static_cast<uint32_t>(kStatusWaitTimeout)) == 0u) {
          env.status[1] = tag;
          env.status[2] = blockIdx.x;
          env.status[3] = parity;
        }
        ok = false;
        break;
      }
    }
  }
  return __all_sync(0xFFFFFFFFu, ok);
}

// MT = activation rows held per thread (M <= MT; rows past M are read as zero and never stored);
// T = K slabs per turn of a warp; RING = warps.  Turn u covers slabs u*T .. u*T + T - 1 and belongs to
// warp u % RING, which keeps those slabs in its own T shared-memory slots.
template <int MT, int T, int RING, bool PACKED>
__global__ void __launch_bounds__(RING * 32, RING == 4 ? 3 : (MT <= 4 ? 2 : 1))
gemm_o1_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                      const float* __restrict__ a_scale, const uint8_t* __restrict__ w_scale, float* __restrict__ y,
                      int M, int N, int K, int ldy, uint32_t* status) {
  constexpr int kSlotBytes = slot_bytes_for(MT, PACKED);
  constexpr int kTileWD = tile_w_bytes(PACKED);
  constexpr int kSlots = T * RING;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* handoff = reinterpret_cast<float*>(smem + kSlots * kSlotBytes);  // [RING][MT][32]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(handoff + RING * MT * 32);
  uint64_t* token_bar = full_bar + kSlots;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(token_bar + RING);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitEnv env{status, abort_flag};
  const int nb = blockIdx.x;
  const int groups = K / 32;
  const int num_kb = (groups + 3) / 4;
  const int num_turns = (num_kb + T - 1) / T;
  // one barrier per thread (full barriers and token barriers are contiguous): a single thread initialising all
  // of them one after the other costs several hundred cycles of a kernel that lasts a few thousand
  if (threadIdx.x < kSlots + RING) {
    mbar_init(&full_bar[threadIdx.x], 1);
    fence_mbar_init();
  }
  if (threadIdx.x == 32) {
    *abort_flag = 0;
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_a);
  }
  __syncthreads();
  const uint32_t smem0 = smem_u32(smem), full0 = smem_u32(full_bar), token0 = smem_u32(token_bar);

  // slab kb into slot `slot` of this warp (converged warp, one elected lane issues)
  auto load_slab = [&](int kb, int slot) {
    const uint32_t st = smem0 + slot * kSlotBytes;
    const uint32_t bar = full0 + slot * 8;
    mbar_expect_tx_elect(bar, kSlotBytes);
    tma_load_2d_elect(st, &tm_w, bar, kb * (PACKED ? 64 : 128), nb * kRowsD);
    tma_load_2d_elect(st + kTileWD, &tm_a, bar, kb * 128, 0);
  };
#pragma unroll
  for (int i = 0; i < T; ++i)
    if (warp * T + i < num_kb) load_slab(warp * T + i, warp * T + i);

  const int n = nb * kRowsD + lane;
  const bool n_ok = n < N;
  const uint8_t* sc_row = w_scale + static_cast<long>(n_ok ? n : 0) * groups;
  const bool vec4 = (groups & 3) == 0;
  // the four UE8M0 codes of slab kb for this thread's row (absent groups read as 0 and are never used)
  auto load_codes = [&](int kb) -> uint32_t {
    if (kb >= num_kb) return 0u;
    if (vec4) return __ldg(reinterpret_cast<const uint32_t*>(sc_row + kb * 4));
    uint32_t c = 0;
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (kb * 4 + g < groups) c |= static_cast<uint32_t>(__ldg(sc_row + kb * 4 + g)) << (8 * g);
    return c;
  };
  float asc[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) asc[j] = j < M ? __ldg(a_scale + j) : 0.0f;

  // INT8 rows: 128 bytes, 128-byte swizzle (chunk ^ row % 8); packed rows: 64 bytes, 64-byte swizzle (chunk ^ (row / 2) % 4)
  const uint32_t w_off = static_cast<uint32_t>(lane * (PACKED ? 64 : 128));
  const uint32_t w_xor = static_cast<uint32_t>(PACKED ? (lane >> 1) & 3 : lane & 7);
  const int prev = (warp + RING - 1) % RING;
  float* my_handoff = handoff + (warp * MT) * 32 + lane;
  const float* prev_handoff = handoff + (prev * MT) * 32 + lane;

  uint32_t codes[T];
#pragma unroll
  for (int i = 0; i < T; ++i) codes[i] = load_codes(warp * T + i);
  int it = 0;
  for (int u = warp; u < num_turns; u += RING, ++it) {
    uint32_t codes_next[T];
#pragma unroll
    for (int i = 0; i < T; ++i) codes_next[i] = load_codes((u + RING) * T + i);
    // ---- ahead of the chain: P and t of this turn's groups
    float t[T][4][MT], sc[T][4];
    bool ok = true;
#pragma unroll
    for (int i = 0; i < T; ++i) {
      const int kb = u * T + i;
      if (kb < num_kb) {
        const int slot = warp * T + i;
        ok = mbar_wait_warp(full0 + slot * 8, static_cast<uint32_t>(it) & 1u, env, kTagFullD | slot);
        if (!ok) break;
        const uint32_t st = smem0 + slot * kSlotBytes;
        const int ng = min(4, groups - kb * 4);
#pragma unroll
        for (int g = 0; g < 4; ++g) sc[i][g] = ue8m0_half_to_float((codes[i] >> (8 * g)) & 0xFFu);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (g < ng) {
            uint4 w0, w1;
            if constexpr (PACKED) {
              // 32 nibbles of this row's group -> their INT8 images 2 * E2M1, in K order
              const uint4 c = lds128(st + w_off + ((static_cast<uint32_t>(g) ^ w_xor) << 4));
              e2m1x8_to_int8x8(c.x, w0.x, w0.y);
              e2m1x8_to_int8x8(c.y, w0.z, w0.w);
              e2m1x8_to_int8x8(c.z, w1.x, w1.y);
              e2m1x8_to_int8x8(c.w, w1.z, w1.w);
            } else {
              w0 = lds128(st + w_off + ((static_cast<uint32_t>(2 * g) ^ w_xor) << 4));
              w1 = lds128(st + w_off + ((static_cast<uint32_t>(2 * g + 1) ^ w_xor) << 4));
            }
#pragma unroll
            for (int j = 0; j < MT; ++j) {
              const uint32_t a_row = st + kTileWD + j * 128;
              const uint4 a0 = lds128(a_row + ((static_cast<uint32_t>(2 * g) ^ static_cast<uint32_t>(j & 7)) << 4));
              const uint4 a1 = lds128(a_row + ((static_cast<uint32_t>(2 * g + 1) ^ static_cast<uint32_t>(j & 7)) << 4));
              t[i][g][j] = __fmul_rn(__int2float_rn(dot32(w0, w1, a0, a1)), asc[j]);
            }
          }
        }
        // the slot's bytes are in registers: refill it with the slab of this warp's next turn
        __syncwarp();
        if ((u + RING) * T + i < num_kb) {
          fence_proxy_async_smem();
          load_slab((u + RING) * T + i, slot);
        }
      }
    }
    if (!ok) break;
    // ---- the chain: accumulators from the warp of the previous turn, four fma per group, pass them on
    float acc[MT];
    if (u > 0) {
      const uint32_t parity = static_cast<uint32_t>(warp == 0 ? it - 1 : it) & 1u;
      if (!token_wait(token0 + prev * 8, parity, env, kTagTokenD | prev)) break;
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[j] = prev_handoff[j * 32];
    } else {
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[j] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < T; ++i) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if ((u * T + i) * 4 + g < groups) {
#pragma unroll
          for (int j = 0; j < MT; ++j) acc[j] = __fmaf_rn(t[i][g][j], sc[i][g], acc[j]);
        }
      }
    }
    if (u == num_turns - 1) {
      if (n_ok) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
          if (j < M) y[static_cast<long>(j) * ldy + n] = acc[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < MT; ++j) my_handoff[j * 32] = acc[j];
      __syncwarp();
      if (lane == 0) mbar_arrive_a(token0 + warp * 8);
    }
#pragma unroll
    for (int i = 0; i < T; ++i) codes[i] = codes_next[i];
  }
}

// Configurations.  Two slabs per turn halve the hand-overs where the registers allow it (MT <= 8).
// A ring of eight keeps 16 slabs in flight per CTA (80 KB; two CTAs per SM up to MT = 4, one above);
// grids too large for that run rings of four (8 slabs, 40 KB, three CTAs per SM), so that all CTAs
// are resident at once.
struct DecodeCfg {
  int mt, t, ring;
};
DecodeCfg choose_cfg(int M, int N, int sm_count) {
  const int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  if (mt == 16) return {16, 1, 8};
  const int ctas = (N + kRowsD - 1) / kRowsD;
  return {mt, 2, ctas <= (mt <= 4 ? 2 : 1) * sm_count ? 8 : 4};
}

template <int MT, int T, int RING, bool PACKED>
int launch_decode(const GemmPlan& p, cudaStream_t stream) {
  gemm_o1_decode_kernel<MT, T, RING, PACKED><<<p.grid, RING * 32, smem_bytes_for(MT, T, RING, PACKED), stream>>>(
      p.tm_b, p.tm_a, static_cast<const float*>(p.a_scale), static_cast<const uint8_t*>(p.w_scale), p.y, p.M, p.N, p.K,
      p.ldy, p.status);
  return check_cuda(cudaGetLastError(), "gemm_o1_decode_kernel launch");
}
template <int MT, int T, int RING>
int set_smem_attribute() {
  if (int rc = check_cuda(cudaFuncSetAttribute(gemm_o1_decode_kernel<MT, T, RING, false>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_for(MT, T, RING, false)),
                          "cudaFuncSetAttribute(gemm_o1_decode_kernel)"))
    return rc;
  return check_cuda(cudaFuncSetAttribute(gemm_o1_decode_kernel<MT, T, RING, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes_for(MT, T, RING, true)),
                    "cudaFuncSetAttribute(gemm_o1_decode_kernel, packed W)");
}
template <int MT>
int set_smem_attributes() {
  if (int rc = set_smem_attribute<MT, 2, 8>()) return rc;
  return set_smem_attribute<MT, 2, 4>();
}
template <int MT, int T, int RING>
int launch_either(const GemmPlan& p, cudaStream_t stream) {
  return p.packed_w ? launch_decode<MT, T, RING, true>(p, stream) : launch_decode<MT, T, RING, false>(p, stream);
}
template <int MT>
int launch_for_ring(const GemmPlan& p, int ring, cudaStream_t stream) {
  return ring == 8 ? launch_either<MT, 2, 8>(p, stream) : launch_either<MT, 2, 4>(p, stream);
}

}  // namespace

// Up to 8 activation rows always; 9 - 16 rows (one CTA per SM) while the 32-row blocks of W fit the GPU once.
bool o1_decode_applies(int M, int N, int sm_count) {
  return M <= 8 || (M <= 16 && (N + kRowsD - 1) / kRowsD <= sm_count);
}

int init_gemm_o1_decode_attributes() {
  if (int rc = set_smem_attributes<1>()) return rc;
  if (int rc = set_smem_attributes<2>()) return rc;
  if (int rc = set_smem_attributes<4>()) return rc;
  if (int rc = set_smem_attributes<8>()) return rc;
  return set_smem_attribute<16, 1, 8>();
}

// Plan for the decode-shape O1 GEMM: tm_b = W map (32-row boxes; the INT8 image or, packed_w, the MXFP4 nibbles), tm_a = A map (all activation rows in one
// box, rounded up to whole 8-row swizzle atoms; rows past M read as zero).
int plan_o1_decode(GemmPlan* plan, const void* a_int8, const void* a_scale, const void* w, const void* w_scale, float* y,
                   int M, int N, int K, int ldy, bool packed_w) {
  DeviceCtx* ctx = nullptr;
  if (int rc = device_ctx(&ctx)) return rc;
  if (M <= 0 || M > 16) return fail("plan_o1_decode: M must be in [1, 16]");
  if ((reinterpret_cast<uintptr_t>(w_scale) & 3u) != 0 || (reinterpret_cast<uintptr_t>(a_scale) & 3u) != 0)
    return fail("W_scale and A_scale must be 4-byte aligned");
  *plan = GemmPlan{};
  plan->variant = 1;
  plan->skinny = 2;
  plan->M = M, plan->N = N, plan->K = K, plan->ldy = ldy;
  plan->a_scale = a_scale;
  plan->w_scale = w_scale;
  plan->y = y;
  plan->status = ctx->status;
  const DecodeCfg cfg = choose_cfg(M, N, ctx->sm_count);
  plan->block_n = cfg.mt;
  plan->packed_w = packed_w ? 1 : 0;
  // W: [N, K] INT8 in 128-byte boxes, or [N, K/2] packed nibbles in 64-byte boxes (64-byte swizzle)
  const uint64_t w_pitch = packed_w ? static_cast<uint64_t>(K) / 2 : static_cast<uint64_t>(K);
  if (int rc = encode_tensor_map_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, N, w_pitch, w_pitch, kRowsD, packed_w ? 64 : 128))
    return rc;
  if (int rc = encode_tensor_map_2d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_int8, M, K, K,
                                    a_rows_for(plan->block_n), 128))
    return rc;
  plan->tm_y = plan->tm_a;
  plan->grid = (N + kRowsD - 1) / kRowsD;
  plan->grid_y = cfg.ring;  // the ring size travels in grid_y; the grid is one-dimensional
  return 0;
}

int run_gemm_o1_decode(const GemmPlan& p, cudaStream_t stream) {
  switch (p.block_n) {
    case 1: return launch_for_ring<1>(p, p.grid_y, stream);
    case 2: return launch_for_ring<2>(p, p.grid_y, stream);
    case 4: return launch_for_ring<4>(p, p.grid_y, stream);
    case 8: return launch_for_ring<8>(p, p.grid_y, stream);
    default: return launch_either<16, 1, 8>(p, stream);
  }
}

void describe_gemm_o1_decode(int M, int N, int sm_count, PlanInfo* info) {
  const DecodeCfg cfg = choose_cfg(M, N, sm_count);
  info->symbol = "gemm_o1_decode_kernel";
  info->mma_family = "dp4a";
  info->tile_m = cfg.mt, info->tile_n = kRowsD, info->stages = cfg.t * cfg.ring, info->acc_stages = 0;
  info->threads = cfg.ring * 32, info->cluster = 1;
  info->mma_m = 1, info->mma_n = 1, info->mma_k = 4;
  info->persistent = 0;
}

}  // namespace adg
