// gemm_tcgen05_pair.cuh — the fp32 GEMM on CTA pairs (tcgen05 cta_group::2).
//
// Same operator, operand panels and epilogue as gemm_tcgen05.cuh; what changes
// is the tile: two thread blocks on neighbouring SMs form a cluster and compute
// one 256x256 tile of D together.  Each block owns 128 rows of the tile (its
// own 128x32 A tile and its own 128x256 fp32 accumulator in tensor memory) and
// loads only half of the B tile (128 of its 256 N-rows); the MMA unit reads the
// other half from the peer's shared memory.  Per block and k-block that is
// 32 KiB of TMA traffic instead of 48 KiB for the same 512 MMA cycles, so the
// shared-memory ring holds 6 stages instead of 4 (TF32 mode; 3 instead of 2 in
// 3xTF32 mode): less L2 bandwidth and 5/6 of 192 KiB in flight per SM.
//
// Roles per block: warp 0 lane 0 loads this block's A tile and B half with TMA
// (completion counted on the leader's `full` barrier); warp 1 lane 0 of the
// leader block (cluster rank 0) issues the 256x256x8 MMAs for both blocks and
// commits to the `empty` and `tmem_full` barriers of both; warps 2-5 of both
// blocks run the epilogue on their own accumulator rows and hand the
// accumulator back by arriving on the leader's `tmem_empty` barrier.
// Every TMA load is issued by the block that consumes it (plain per-block loads).
#pragma once
#include "gemm_tcgen05.cuh"

namespace sb200 {

constexpr int PAIR_BM = 256;        // tile rows (128 per block)
constexpr int PAIR_BN = 256;        // tile columns of the large tile; 128 and 64 serve problems with few tiles
constexpr int PAIR_GROUP_M = 8;     // rasterisation: bands of 8 row tiles
constexpr uint32_t PAIR_A_BYTES = 128 * GEMM_BK * 4;  // this block's A rows: 16 KiB

// BN = tile columns (256, 128 or 64).  Each block loads BN/2 columns of B.  The narrower tiles need more
// shared-memory bandwidth per MMA cycle and exist for problems that would otherwise fill only a
// fraction of the SMs with 256x256 tiles; results do not depend on BN.
template <int MODE, int BN = PAIR_BN>
struct PairCfg {
  static_assert(BN == 256 || BN == 128 || BN == 64, "tile columns");
  static constexpr int kOperands = (MODE == 3 || MODE == 4 || MODE == 5) ? 2 : 1;  // high parts (+ low parts)
  static constexpr uint32_t kBBytes = (BN / 2) * GEMM_BK * 4;  // this block's half of B: 16, 8 or 4 KiB (rows of 128 bytes)
  static constexpr uint32_t kStageBytes = kOperands * (PAIR_A_BYTES + kBBytes);
  static constexpr int kStagesFit = (192 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;  // 6 / 8 / 8 (TF32), 3 / 4 / 4 (3xTF32)
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + GEMM_EPI_BUF_BYTES + GEMM_CTRL_BYTES + 1024;
};

constexpr int PAIR_EPOCH_RING = 64;    // epoch counters (a pair far ahead wraps onto an old counter: harmless, a hint)

// Count this pair into epoch e and wait, for wait_ns at most, until all `pairs` pairs of the launch have reached it.
__device__ __forceinline__ void pair_soft_epoch(unsigned int* ctr, unsigned int e, unsigned int pairs, uint64_t wait_ns) {
  unsigned int* slot = ctr + (e % PAIR_EPOCH_RING);
  const unsigned int target = pairs * (e / PAIR_EPOCH_RING + 1);
  atomicAdd(slot, 1u);
  const uint64_t t0 = global_timer_ns();
  while (*reinterpret_cast<volatile unsigned int*>(slot) < target && global_timer_ns() - t0 < wait_ns) {
  }
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int band_tiles = group_m * tiles_n;
  const int band = tile / band_tiles;
  const int within = tile - band * band_tiles;
  const int first_m = band * group_m;
  const int band_m = min(group_m, tiles_m - first_m);
  tm = first_m + within % band_m;
  tn = within / band_m;
}

// DIRECT: map_a_hi is a TFLOAT32 tensor map over the caller's row-major A (TMA rounds to TF32 on the
// way in) and map_b_hi one over the caller's row-major B, loaded as four [32 k][32 n] slabs per stage
// (swizzle 128B with 32-byte atoms) and consumed through an MN-major descriptor.  TF32 mode then needs
// no panels at all; 3xTF32 mode needs only the low parts: map_a_lo over an [M x Kp] panel, map_b_lo
// over a row-major [K x Np] panel read as slabs like B itself.
//
// MODE 5 (mixed; always DIRECT): map_a_hi / map_b_hi are those TFLOAT32 maps over the caller's matrices, map_a_lo /
// map_b_lo lie over the fp16 panels of the high parts and map_a_x / map_b_x over those of the low parts (all K-major,
// [rows x Kp], Kp a multiple of 64).  A tile is computed in three runs of stages, every stage the same 4 x 16 KiB:
// K/64 cross stages (the four fp16 tiles of 64 k: lo*hi + hi*lo, eight fp16 MMAs), then the rescale stages (tiles from
// beyond the end of K, which TMA fills with zeros: one MMA each whose only effect is the scaling of the
// accumulator by 2^-15), then K/64 main stages (A and B of two consecutive k-blocks of 32 where the other modes keep
// high and low parts: eight TF32 MMAs, the first of which scales the accumulator by 2^-first_scale).
template <int MODE, bool DIRECT = false, int BN = PAIR_BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_b_hi,
                 const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
                 const __grid_constant__ CUtensorMap map_a_x, const __grid_constant__ CUtensorMap map_b_x,
                 const GemmParams p) {
  using Cfg = PairCfg<MODE, BN>;
  constexpr bool MIXED = MODE == 5;
  static_assert(!MIXED || DIRECT, "the mixed mode reads the main term's operands where they lie");
  // MODE 1: TF32, one MMA per k-step.  MODE 3: 3xTF32, lo*hi + hi*lo + hi*hi.  MODE 4: the same three-term split on
  // fp16 panels (kind::f16): a 128-byte operand row holds 64 halves instead of 32 floats, so a k-block spans 64 k
  // and a k-step 16, in the same bytes, descriptors and cycles as the TF32 forms.  MODE 2: fp16 panels, one MMA.
  constexpr bool THREE = MODE == 3 || MODE == 4;
  constexpr bool F16 = MODE == 4 || MODE == 2;  // MODE 2: one fp16 MMA per k-step on the high parts alone
  constexpr int BK_ELEMS = F16 ? 2 * GEMM_BK : GEMM_BK;  // elements of K per k-block
  static_assert(!(F16 && DIRECT), "fp16 panels are always prepared");
  constexpr int STAGES = Cfg::kStages;
  constexpr uint32_t B_BYTES = Cfg::kBBytes;
  constexpr int HALF_N = BN / 2;        // columns of B this block loads
  constexpr int SLABS = HALF_N / 32;    // [32 k][32 n] slabs per stage in the direct layout
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* epi_buf = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes + GEMM_EPI_BUF_BYTES);
  uint64_t* full_bar = bars;                        // used in the leader only
  uint64_t* empty_bar = bars + STAGES;              // one set per block
  uint64_t* tmem_full_bar = bars + 2 * STAGES;      // one set per block
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2; // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 8);  // four epilogue warps in each of the two blocks
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a_hi);
    tma_prefetch_desc(&map_b_hi);
    if (THREE || MIXED) {
      tma_prefetch_desc(&map_a_lo);
      tma_prefetch_desc(&map_b_lo);
    }
    if (MIXED) {
      tma_prefetch_desc(&map_a_x);
      tma_prefetch_desc(&map_b_x);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), GEMM_TMEM_COLS);
    tmem_relinquish_pair();
    tc_fence_before_sync();
  }
  __syncthreads();
  // both blocks' barriers exist before any signal crosses between them
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched no global memory, so it may overlap the tail of the kernel before this one in
  // the stream (the preparation of the low-part panels); from here on its results are needed.
  grid_dependency_wait();
  // a gated kernel whose gate is closed has no tiles: every role falls through to the common exit
  const bool gate_open = !p.gate || *p.gate == p.gate_value;
  const int num_tiles = gate_open ? p.tiles_m * p.tiles_n : 0;
  int mix_rescale = 0, mix_first = 0;
  if (MIXED && gate_open) {
    const MixCtl* ctl = reinterpret_cast<const MixCtl*>(p.mix_ctl);
    mix_rescale = ctl->rescale_stages;
    mix_first = ctl->first_scale;
  }
  // stages per tile: the k-blocks; in mixed mode the cross stages, the rescale stages, the main stages
  const int stages_per_tile = MIXED ? 2 * p.num_k_blocks + mix_rescale : p.num_k_blocks;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = l2_policy(p.l2_policy & 3), pol_b = l2_policy((p.l2_policy >> 2) & 3);
      const bool lockstep = p.epoch_ctr != nullptr && rank == 0;
      const int epoch_stages = p.epoch_stages > 0 ? p.epoch_stages : 64;
      const int epochs_per_tile = (stages_per_tile + epoch_stages - 1) / epoch_stages;
      int my_tiles = 0;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++my_tiles) {
        int tm, tn;
        pair_tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        const int m0 = tm * PAIR_BM + static_cast<int>(rank) * 128;  // this block's rows of A
        const int n0 = tn * BN + static_cast<int>(rank) * HALF_N;    // this block's half of B's N-rows
        for (int it = 0; it < stages_per_tile; ++it) {
          const int kb = MIXED ? (it < p.num_k_blocks + mix_rescale ? it : it - p.num_k_blocks - mix_rescale) : it;
          if (lockstep && (it % epoch_stages) == 0)
            pair_soft_epoch(p.epoch_ctr, static_cast<unsigned int>(my_tiles * epochs_per_tile + it / epoch_stages),
                            static_cast<unsigned int>(num_pairs), static_cast<uint64_t>(p.epoch_wait_ns));
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            atomicCAS(p.status, 0, 0x1100 | (rank << 4) | stage);
            ok = false;
            break;
          }
          // the leader arms its barrier with the bytes of both blocks
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * Cfg::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          uint8_t* sp = stage_base + stage * Cfg::kStageBytes;
          if (MIXED) {
            if (it < p.num_k_blocks + mix_rescale) {
              // cross stage: 64 k of the four fp16 panels; a rescale stage asks for k-blocks past the end: zeros
              tma_load_2d_pair_hint(smem_u32(sp), &map_a_lo, bar, kb * 64, m0, pol_a);
              tma_load_2d_pair_hint(smem_u32(sp + PAIR_A_BYTES), &map_b_lo, bar, kb * 64, n0, pol_b);
              tma_load_2d_pair_hint(smem_u32(sp + PAIR_A_BYTES + B_BYTES), &map_a_x, bar, kb * 64, m0, pol_a);
              tma_load_2d_pair_hint(smem_u32(sp + 2 * PAIR_A_BYTES + B_BYTES), &map_b_x, bar, kb * 64, n0, pol_b);
            } else {
              // main stage: two consecutive k-blocks of 32 of the caller's A and B
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint8_t* hp = sp + h * (PAIR_A_BYTES + B_BYTES);
                tma_load_2d_pair_hint(smem_u32(hp), &map_a_hi, bar, kb * 64 + 32 * h, m0, pol_a);
#pragma unroll
                for (int sl = 0; sl < SLABS; ++sl)
                  tma_load_2d_pair_hint(smem_u32(hp + PAIR_A_BYTES + sl * 4096), &map_b_hi, bar, n0 + 32 * sl, kb * 64 + 32 * h, pol_b);
              }
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          tma_load_2d_pair_hint(smem_u32(sp), &map_a_hi, bar, kb * BK_ELEMS, m0, pol_a);
          if (DIRECT) {
            // B is K x N row-major: x = column, y = k; slabs of 32 columns cover this block's half
#pragma unroll
            for (int sl = 0; sl < SLABS; ++sl)
              tma_load_2d_pair_hint(smem_u32(sp + PAIR_A_BYTES + sl * 4096), &map_b_hi, bar, n0 + 32 * sl, kb * BK_ELEMS, pol_b);
          } else {
            tma_load_2d_pair_hint(smem_u32(sp + PAIR_A_BYTES), &map_b_hi, bar, kb * BK_ELEMS, n0, pol_b);
          }
          if (THREE) {
            tma_load_2d_pair_hint(smem_u32(sp + PAIR_A_BYTES + B_BYTES), &map_a_lo, bar, kb * BK_ELEMS, m0, pol_a);
            if (DIRECT) {
#pragma unroll
              for (int sl = 0; sl < SLABS; ++sl)
                tma_load_2d_pair_hint(smem_u32(sp + 2 * PAIR_A_BYTES + B_BYTES + sl * 4096), &map_b_lo, bar, n0 + 32 * sl,
                                 kb * BK_ELEMS, pol_b);
            } else {
              tma_load_2d_pair_hint(smem_u32(sp + 2 * PAIR_A_BYTES + B_BYTES), &map_b_lo, bar, kb * BK_ELEMS, n0, pol_b);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (lockstep) {
        // a pair with fewer tiles than the others counts itself into the epochs it will not reach
        const int most_tiles = (num_tiles + num_pairs - 1) / num_pairs;
        for (int e = my_tiles * epochs_per_tile; e < most_tiles * epochs_per_tile; ++e)
          atomicAdd(p.epoch_ctr + (e % PAIR_EPOCH_RING), 1u);
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader block)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = F16 ? umma_idesc_f16(PAIR_BM, BN) : umma_idesc_tf32(PAIR_BM, BN, DIRECT);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, 0x1200 | acc);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < stages_per_tile; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, abort_flag)) {
            atomicCAS(p.status, 0, 0x1300 | stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa_hi = smem_u32(stage_base + stage * Cfg::kStageBytes);
          const uint32_t sb_hi = sa_hi + PAIR_A_BYTES;
          const uint32_t sa_lo = sb_hi + B_BYTES;
          const uint32_t sb_lo = sa_lo + PAIR_A_BYTES;
          if (MIXED) {
            constexpr uint32_t idesc16 = umma_idesc_f16(PAIR_BM, BN);
            constexpr uint32_t idesc32 = umma_idesc_tf32(PAIR_BM, BN, true);
            if (kb < p.num_k_blocks) {
              // cross terms of 64 k: lo(a)*hi(b) + hi(a)*lo(b), four k-steps of 16
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t koff = k * 32;
                umma_f16_pair(tmem_d, umma_desc_k_sw128(sa_lo + koff), umma_desc_k_sw128(sb_hi + koff), idesc16, (kb | k) ? 1u : 0u);
                umma_f16_pair(tmem_d, umma_desc_k_sw128(sa_hi + koff), umma_desc_k_sw128(sb_lo + koff), idesc16, 1u);
              }
            } else if (kb < p.num_k_blocks + mix_rescale) {
              // zero tiles: the product adds nothing, the accumulator is scaled by 2^-15
              umma_f16_pair_scaled(tmem_d, umma_desc_k_sw128(sa_hi), umma_desc_k_sw128(sb_hi), idesc16, 15);
            } else {
              const bool first = kb == p.num_k_blocks + mix_rescale;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t sa = h ? sa_lo : sa_hi, sb = h ? sb_lo : sb_hi;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint64_t da = umma_desc_k_sw128(sa + k * 32);
                  const uint64_t db = umma_desc_mn_sw128_32b(sb + k * 1024, 4096);
                  if (first && h == 0 && k == 0)
                    umma_tf32_pair_scaled(tmem_d, da, db, idesc32, mix_first);
                  else
                    umma_tf32_pair(tmem_d, da, db, idesc32, 1u);
                }
              }
            }
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint32_t koff = k * GEMM_UMMA_K * 4;
            const uint64_t da_hi = umma_desc_k_sw128(sa_hi + koff);
            // MN-major B: k-step k is the k-th 8-row group (1024 bytes) of every slab
            const uint64_t db_hi = DIRECT ? umma_desc_mn_sw128_32b(sb_hi + k * 1024, 4096) : umma_desc_k_sw128(sb_hi + koff);
            const uint32_t accumulate = (kb | k) ? 1u : 0u;
            if (F16 && !THREE) {
              umma_f16_pair(tmem_d, da_hi, db_hi, idesc, accumulate);
            } else if (F16) {
              const uint64_t da_lo = umma_desc_k_sw128(sa_lo + koff);
              const uint64_t db_lo = umma_desc_k_sw128(sb_lo + koff);
              umma_f16_pair(tmem_d, da_lo, db_hi, idesc, accumulate);
              umma_f16_pair(tmem_d, da_hi, db_lo, idesc, 1u);
              umma_f16_pair(tmem_d, da_hi, db_hi, idesc, 1u);
            } else if (MODE == 3) {
              const uint64_t da_lo = umma_desc_k_sw128(sa_lo + koff);
              const uint64_t db_lo = DIRECT ? umma_desc_mn_sw128_32b(sb_lo + k * 1024, 4096) : umma_desc_k_sw128(sb_lo + koff);
              umma_tf32_pair(tmem_d, da_lo, db_hi, idesc, accumulate);
              umma_tf32_pair(tmem_d, da_hi, db_lo, idesc, 1u);
              umma_tf32_pair(tmem_d, da_hi, db_hi, idesc, 1u);
            } else {
              umma_tf32_pair(tmem_d, da_hi, db_hi, idesc, accumulate);
            }
          }
          // the stage is free in both blocks once these MMAs retire
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          umma_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc]), 1));
        }
      }
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    float* tbuf = epi_buf + (warp - 2) * (32 * GEMM_EPI_LD);
    int local_tile = 0;
    bool ok = true;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      int tm, tn;
      pair_tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const int row0 = tm * PAIR_BM + static_cast<int>(rank) * 128 + quarter * 32;
      const int n0 = tn * BN;
      const bool landed = mbar_wait_bounded(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0) atomicCAS(p.status, 0, 0x1400 | (rank << 4) | acc);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      epilogue_rows<BN>(p, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN, tbuf, lane, row0, n0);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
    }
    __syncwarp();
  }

  // Neither block may retire, or free tensor memory, while its peer can still
  // signal its barriers, read its shared memory or write its accumulators.
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, GEMM_TMEM_COLS);
  }
  (void)peer;
}

}  // namespace sb200
