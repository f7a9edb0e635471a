// gemm_tcgen05.cuh — fp32 GEMM for sm_100a on tcgen05 tensor cores.
//
//   D[M x N] = act(alpha * A[M x K] . B[K x N] + beta * C + bias[col])
//
// replaces the matrix_mul and matrix_mul_tiled kernels of the reference
// (benchmarks/bench_matrix_mul.ml:55-73, benchmarks/bench_matrix_mul_tiled.ml:55-94),
// with the epilogue fused into the accumulator read-out so the product never
// makes a round trip through HBM.
//
// Two stages:
//  1. operand preparation (prep_a_kernel / prep_b_kernel): A and B are split
//     into TF32-exact panels  hi = rn_tf32(x),  lo = rn_tf32(x - hi)  (lo only
//     in 3xTF32 mode).  B is transposed on the way so both panels are K-major,
//     and K is zero-padded to a multiple of 32 so every TMA box starts on a
//     128-byte boundary whatever K is.
//  2. gemm_tf32_kernel: a persistent, warp-specialised kernel, one block per
//     SM.  Warp 0 streams 128x32 (A) and 256x32 (B) fp32 tiles into a ring of
//     shared-memory stages with TMA (128-byte swizzle, no cluster forms);
//     warp 1 issues tcgen05.mma kind::tf32 128x256x8 into one of two 256-column
//     fp32 accumulators in tensor memory; warps 2-5 read the finished
//     accumulator back with tcgen05.ld, apply the epilogue and store D while
//     the MMA warp already works on the next tile.
//     3xTF32 mode issues  lo*hi + hi*lo + hi*hi  per k-step into the same
//     accumulator (the lo*lo term, ~2^-22 relative, is dropped).
//
// Work per launch: 2*M*N*K useful flops (3x that in MMA flops in 3xTF32
// mode); the bound is the tensor pipe.
#pragma once
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace sb200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BN = 256;
constexpr int GEMM_BK = 32;      // floats per k-block = one 128-byte swizzle row
constexpr int GEMM_UMMA_K = 8;   // floats per tcgen05.mma kind::tf32 (32 bytes)
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 16;  // tile rasterisation: bands of 16 row tiles
constexpr uint32_t GEMM_A_BYTES = GEMM_BM * GEMM_BK * 4;  // 16 KiB
constexpr uint32_t GEMM_B_BYTES = GEMM_BN * GEMM_BK * 4;  // 32 KiB
constexpr uint32_t GEMM_TMEM_COLS = 512;                  // two 256-column accumulators
constexpr int GEMM_EPI_LD = 36;                           // row stride (floats) of a warp's staging tile: 144 B, 16-byte aligned, conflict-free
constexpr uint32_t GEMM_EPI_BUF_BYTES = 4 * 32 * GEMM_EPI_LD * 4;  // per-warp 32-row staging tiles
constexpr uint32_t GEMM_CTRL_BYTES = 256;

template <int MODE>
struct GemmCfg {
  static constexpr int kOperands = (MODE == 3) ? 2 : 1;  // hi (+ lo)
  static constexpr int kStages = (MODE == 3) ? 2 : 4;
  static constexpr uint32_t kStageBytes = kOperands * (GEMM_A_BYTES + GEMM_B_BYTES);
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + GEMM_EPI_BUF_BYTES + GEMM_CTRL_BYTES + 1024;
};

struct GemmParams {
  int M, N;
  int num_k_blocks;  // padded K / 32
  int tiles_m, tiles_n;
  float* D;
  long long ldd;
  const float* C;  // may be null
  long long ldc;
  const float* bias;  // may be null
  float alpha, beta;
  int act;      // 0 none, 1 relu
  int* status;  // device word, set non-zero when a bounded wait expired
  int group_m;  // CTA-pair kernel: row tiles per rasterisation band
  // Gathered result: when n_replicas > 0 every output element is also stored to the same position of
  // these further copies of D (this GPU's own or peers' memory mapped into this process), so that a
  // row-sharded product leaves the whole matrix on every GPU without a separate all-gather.
  int n_replicas;
  float* replicas[7];
  // Set by the host when D, C, bias and every replica are 16-byte aligned with leading dimensions and N that
  // are multiples of 4: the epilogue then moves 128-bit vectors (four rows of 128 bytes per warp instruction).
  int vec_epilogue;
  // L2 eviction policies, 2 bits each (0 normal, 1 evict first, 2 evict last): bits 0-1 loads of A (hi and lo),
  // bits 2-3 loads of B, bits 4-5 the epilogue's reads of C and writes of D.
  int l2_policy;
  // fp16 modes: row i of the A panel holds A[i,:] * 2^ea(i) and row j of the B panel holds B[:,j] * 2^eb(j); the
  // preparation kernels leave 2^-ea(i) in row_scale[i] and 2^-eb(j) in col_scale[j], and the epilogue multiplies
  // each accumulator by both (exact: powers of two) before anything else.  Null in the TF32 modes.
  const float* row_scale;
  const float* col_scale;
  // A kernel with a gate runs only when *gate == gate_value (a word an earlier kernel of the stream wrote): the
  // mixed mode launches its own kernel and, behind it, the plain 3xTF32 pair for operands it cannot take; exactly one
  // of the two does the work.  Null: always run.
  const int* gate;
  int gate_value;
  // Mixed mode: the control words its preparation wrote (MixCtl below).
  const int* mix_ctl;
  // Soft lockstep for long k-loops (CTA-pair kernel; null: off): 64 epoch counters in global memory, zero before the
  // launch.  Every 64 stages the TMA lane of each pair's leader counts itself into its epoch's counter and waits a few
  // microseconds at most for the other pairs, so that the pairs of a wave, which share rows of A and columns of B
  // through L2, stay within L2's reach of one another.  A hint: nothing depends on the wait.
  unsigned int* epoch_ctr;
  int epoch_stages;   // stages between two epochs (64 unless SAREK_B200_LOCKSTEP_STAGES says otherwise)
  int epoch_wait_ns;  // longest wait at an epoch (4000)
};

// Control words of the mixed mode, in device memory: the preparation kernels fill them, the GEMM reads them.
struct MixCtl {
  unsigned int max_a, max_b;  // largest magnitudes of A and B as float bits (atomicMax; zero before)
  int ok;                     // 1: the mixed kernel runs; 0: the plain 3xTF32 kernels behind it run instead
  int rescale_stages;         // stages of zero tiles between the cross terms and the main term, each scaling by 2^-15
  int first_scale;            // the first main-term MMA scales the accumulated cross terms by 2^-first_scale (0..15)
  int shift_a, shift_b;       // the fp16 panels hold A * 2^shift_a and B * 2^shift_b (low parts 2^11 times that)
};

__device__ __forceinline__ void store_replicas(const GemmParams& p, long long offset, float x) {
#pragma unroll 1
  for (int r = 0; r < p.n_replicas; ++r) p.replicas[r][offset] = x;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band_tiles = GEMM_GROUP_M * tiles_n;
  const int band = tile / band_tiles;
  const int within = tile - band * band_tiles;
  const int first_m = band * GEMM_GROUP_M;
  const int band_m = min(GEMM_GROUP_M, tiles_m - first_m);
  tm = first_m + within % band_m;
  tn = within / band_m;
}

// Epilogue of one warp for its 32 rows x BN columns of a finished accumulator: tensor memory -> registers
// (lane = row) -> the warp's staging tile in shared memory -> D = act(alpha*acc + beta*C + bias), and the same
// values to every replica of D.  `taddr` addresses the warp's 32 tensor-memory lanes at the accumulator's
// first column.  Both GEMM kernels use it; every element goes through the same operations in the same order
// on either path, so the vector and scalar paths give the same bits.
template <int BN>
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, uint32_t taddr, float* tbuf, int lane, int row0, int n0) {
  const int rows_here = min(32, p.M - row0);  // may be <= 0 for a ragged last tile
  if (p.vec_epilogue) {
    const int sub = lane >> 3;       // this lane's row within each group of four rows
    const int cq = (lane & 7) * 4;   // first column of this lane's quad within a 32-column chunk
    const uint64_t pol = l2_policy((p.l2_policy >> 4) & 3);
#pragma unroll 1
    for (int chunk = 0; chunk < BN / 32; ++chunk) {
      if (n0 + chunk * 32 >= p.N) break;  // warp-uniform
      uint32_t v[32];
      tmem_ld_32x32b_x32(taddr + chunk * 32, v);
      tmem_ld_wait();
      float4* trow = reinterpret_cast<float4*>(tbuf + lane * GEMM_EPI_LD);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        trow[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                              __uint_as_float(v[4 * j + 3]));
      __syncwarp();
      const int col = n0 + chunk * 32 + cq;
      if (col < p.N) {  // N is a multiple of 4 on this path: the whole quad is inside
        const float4 bv = p.bias ? *reinterpret_cast<const float4*>(p.bias + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 cs = p.col_scale ? *reinterpret_cast<const float4*>(p.col_scale + col) : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 cv[8];
        if (p.C) {
          // all loads of C before the first use, so that their latencies overlap
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = sub + 4 * i;
            if (r < rows_here) cv[i] = ld_global_v4_hint(p.C + static_cast<long long>(row0 + r) * p.ldc + col, pol);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = sub + 4 * i;
          if (r < rows_here) {
            const float4 a = *reinterpret_cast<const float4*>(tbuf + r * GEMM_EPI_LD + cq);
            const float rs = p.row_scale ? p.row_scale[row0 + r] : 1.0f;
            float4 x = make_float4(p.alpha * ((a.x * rs) * cs.x), p.alpha * ((a.y * rs) * cs.y), p.alpha * ((a.z * rs) * cs.z),
                                   p.alpha * ((a.w * rs) * cs.w));
            if (p.C) {
              x.x = fmaf(p.beta, cv[i].x, x.x);
              x.y = fmaf(p.beta, cv[i].y, x.y);
              x.z = fmaf(p.beta, cv[i].z, x.z);
              x.w = fmaf(p.beta, cv[i].w, x.w);
            }
            x.x += bv.x;
            x.y += bv.y;
            x.z += bv.z;
            x.w += bv.w;
            if (p.act == 1) {
              x.x = (x.x > 0.0f) ? x.x : 0.0f;
              x.y = (x.y > 0.0f) ? x.y : 0.0f;
              x.z = (x.z > 0.0f) ? x.z : 0.0f;
              x.w = (x.w > 0.0f) ? x.w : 0.0f;
            }
            const long long off = static_cast<long long>(row0 + r) * p.ldd + col;
            st_global_v4_hint(p.D + off, x, pol);
            cv[i] = x;  // kept for the replicas
          }
        }
        // gathered result: the same four rows x 128 bytes per instruction to every other copy of D
#pragma unroll 1
        for (int rep = 0; rep < p.n_replicas; ++rep) {
          float* base = p.replicas[rep];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = sub + 4 * i;
            if (r < rows_here) *reinterpret_cast<float4*>(base + static_cast<long long>(row0 + r) * p.ldd + col) = cv[i];
          }
        }
      }
      __syncwarp();
    }
    return;
  }
  // general path: any alignment, any N; the tile is staged transposed so that lane = column
#pragma unroll 1
  for (int chunk = 0; chunk < BN / 32; ++chunk) {
    const int col = n0 + chunk * 32 + lane;
    if (n0 + chunk * 32 >= p.N) break;  // warp-uniform
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + chunk * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) tbuf[lane * 33 + j] = __uint_as_float(v[j]);
    __syncwarp();
    if (col < p.N) {
      const float bias_v = p.bias ? p.bias[col] : 0.0f;
      const float cs = p.col_scale ? p.col_scale[col] : 1.0f;
      if (rows_here >= 32) {
        // full 32-row slab: issue all 32 loads of C before the first use so that
        // their latencies overlap instead of adding up
        float cv[32];
        if (p.C) {
          const float* cp = p.C + static_cast<long long>(row0) * p.ldc + col;
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) cv[rr] = cp[rr * p.ldc];
        }
        float* dp = p.D + static_cast<long long>(row0) * p.ldd + col;
#pragma unroll
        for (int rr = 0; rr < 32; ++rr) {
          const float rs = p.row_scale ? p.row_scale[row0 + rr] : 1.0f;
          float x = p.alpha * ((tbuf[rr * 33 + lane] * rs) * cs);
          if (p.C) x = fmaf(p.beta, cv[rr], x);
          x += bias_v;
          if (p.act == 1) x = (x > 0.0f) ? x : 0.0f;
          dp[rr * p.ldd] = x;
          if (p.n_replicas) store_replicas(p, static_cast<long long>(row0 + rr) * p.ldd + col, x);
        }
      } else {
        for (int rr = 0; rr < rows_here; ++rr) {
          const long long row = row0 + rr;
          const float rs = p.row_scale ? p.row_scale[row] : 1.0f;
          float x = p.alpha * ((tbuf[rr * 33 + lane] * rs) * cs);
          if (p.C) x = fmaf(p.beta, p.C[row * p.ldc + col], x);
          x += bias_v;
          if (p.act == 1) x = (x > 0.0f) ? x : 0.0f;
          p.D[row * p.ldd + col] = x;
          if (p.n_replicas) store_replicas(p, row * p.ldd + col, x);
        }
      }
    }
    __syncwarp();
  }
}

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_b_hi,
                 const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
                 const GemmParams p) {
  using Cfg = GemmCfg<MODE>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern is anchored to
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  float* epi_buf = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes + GEMM_EPI_BUF_BYTES);
  // bars[0..STAGES) full, [STAGES..2*STAGES) empty, then tmem_full[2], tmem_empty[2]
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a_hi);
    tma_prefetch_desc(&map_b_hi);
    if (MODE == 3) {
      tma_prefetch_desc(&map_a_lo);
      tma_prefetch_desc(&map_b_lo);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), GEMM_TMEM_COLS);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * GEMM_BM, n0 = tn * GEMM_BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            atomicCAS(p.status, 0, 0x100 | stage);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[stage]);
          uint8_t* sp = stage_base + stage * Cfg::kStageBytes;
          mbar_arrive_expect_tx(bar, Cfg::kStageBytes);
          tma_load_2d(smem_u32(sp), &map_a_hi, bar, kb * GEMM_BK, m0);
          tma_load_2d(smem_u32(sp + GEMM_A_BYTES), &map_b_hi, bar, kb * GEMM_BK, n0);
          if (MODE == 3) {
            tma_load_2d(smem_u32(sp + GEMM_A_BYTES + GEMM_B_BYTES), &map_a_lo, bar, kb * GEMM_BK, m0);
            tma_load_2d(smem_u32(sp + 2 * GEMM_A_BYTES + GEMM_B_BYTES), &map_b_lo, bar, kb * GEMM_BK, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Give loads that are still in flight a bounded chance to land before
        // the block retires: a stage whose load was issued completes its
        // full barrier regardless of the consumer.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(GEMM_BM, GEMM_BN);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, 0x200 | acc);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * GEMM_BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, abort_flag)) {
            atomicCAS(p.status, 0, 0x300 | stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa_hi = smem_u32(stage_base + stage * Cfg::kStageBytes);
          const uint32_t sb_hi = sa_hi + GEMM_A_BYTES;
          const uint32_t sa_lo = sb_hi + GEMM_B_BYTES;
          const uint32_t sb_lo = sa_lo + GEMM_A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; ++k) {
            const uint32_t koff = k * GEMM_UMMA_K * 4;  // 32 bytes along K inside the swizzle row
            const uint64_t da_hi = umma_desc_k_sw128(sa_hi + koff);
            const uint64_t db_hi = umma_desc_k_sw128(sb_hi + koff);
            const uint32_t first = (kb | k) ? 1u : 0u;
            if (MODE == 3) {
              const uint64_t da_lo = umma_desc_k_sw128(sa_lo + koff);
              const uint64_t db_lo = umma_desc_k_sw128(sb_lo + koff);
              umma_tf32(tmem_d, da_lo, db_hi, idesc, first);
              umma_tf32(tmem_d, da_hi, db_lo, idesc, 1u);
              umma_tf32(tmem_d, da_hi, db_hi, idesc, 1u);
            } else {
              umma_tf32(tmem_d, da_hi, db_hi, idesc, first);
            }
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // stage is free once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));
      }
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, 32*quarter+32)
    float* tbuf = epi_buf + (warp - 2) * (32 * GEMM_EPI_LD);
    int local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * GEMM_BM + quarter * 32;
      const int n0 = tn * GEMM_BN;
      // every lane waits; the warp then agrees on the outcome so that the
      // warp-collective tensor-memory loads below are never partly skipped
      const bool landed = mbar_wait_bounded(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0) atomicCAS(p.status, 0, 0x400 | acc);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      epilogue_rows<GEMM_BN>(p, tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * GEMM_BN, tbuf, lane, row0, n0);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
  }
}

// ------------------------------------------------------------------------
// Operand preparation
// ------------------------------------------------------------------------

// Low part of the 3xTF32 split: rn_tf32(x - hi).  When hi is not finite (x is an infinity or a NaN, or a
// finite x so close to FLT_MAX that rounding to TF32 overflows) x - hi would be Inf - Inf; the low part is
// then zero.  Non-finite operands still do not follow fp32 exactly in 3xTF32 mode: the cross term
// hi(a) * lo(b) is Inf * 0 = NaN whenever the other operand is exactly representable in TF32, so an element
// whose row of A or column of B holds an infinity comes out non-finite (Inf or NaN) where fp32 gives Inf.
// Elements that no non-finite operand reaches are unaffected; TF32 mode keeps fp32's Inf/NaN semantics.
__device__ __forceinline__ float tf32_lo(float x, float hi) {
  return (fabsf(hi) <= 3.402823466e+38f) ? tf32_round(x - hi) : 0.0f;
}

// A[M x K] (row stride lda) -> hi[M x Kp] (and lo[M x Kp]), Kp = K rounded up
// to 32, columns K..Kp zero.  One thread per 4 consecutive k.
// LO_ONLY: store just the low parts (the high parts are then taken from the source matrix itself by a
// TFLOAT32 tensor map, which applies the same rounding).
template <int MODE, bool LO_ONLY = false>
__global__ void prep_a_kernel(const float* __restrict__ A, long long lda, float* __restrict__ hi,
                              float* __restrict__ lo, int M, int K, int Kp, int vec_ok) {
  const long long quads_per_row = Kp >> 2;
  const long long total = static_cast<long long>(M) * quads_per_row;
  for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < total;
       q += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = q / quads_per_row;
    const int k = static_cast<int>(q - row * quads_per_row) << 2;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* src = A + row * lda + k;
    if (vec_ok && k + 3 < K) {
      x = *reinterpret_cast<const float4*>(src);
    } else {
      if (k < K) x.x = src[0];
      if (k + 1 < K) x.y = src[1];
      if (k + 2 < K) x.z = src[2];
      if (k + 3 < K) x.w = src[3];
    }
    float4 h = make_float4(tf32_round(x.x), tf32_round(x.y), tf32_round(x.z), tf32_round(x.w));
    if (!LO_ONLY) *reinterpret_cast<float4*>(hi + row * Kp + k) = h;
    if (MODE == 3) {
      float4 l = make_float4(tf32_lo(x.x, h.x), tf32_lo(x.y, h.y), tf32_lo(x.z, h.z), tf32_lo(x.w, h.w));
      *reinterpret_cast<float4*>(lo + row * Kp + k) = l;
    }
  }
}

// The low parts of two row-major matrices in one launch (A and B of a 3xTF32 product whose high parts TMA
// takes from the caller's matrices): lo[r][c] = rn_tf32(x - rn_tf32(x)), row length padded to colsp with
// zeros.  Blocks [0, blocks_a) work on job a, the rest on job b.
struct PrepLoJob {
  const float* src;
  long long ld;
  float* lo;
  int rows, cols, colsp;
};

__device__ __forceinline__ void prep_lo_rows(const PrepLoJob& j, long long block, long long nblocks) {
  const long long quads_per_row = j.colsp >> 2;
  const long long total = static_cast<long long>(j.rows) * quads_per_row;
  for (long long q = block * blockDim.x + threadIdx.x; q < total; q += nblocks * blockDim.x) {
    const long long row = q / quads_per_row;
    const int k = static_cast<int>(q - row * quads_per_row) << 2;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* src = j.src + row * j.ld + k;   // callers guarantee 16-byte aligned rows
    if (k + 3 < j.cols) {
      x = *reinterpret_cast<const float4*>(src);
    } else {
      if (k < j.cols) x.x = src[0];
      if (k + 1 < j.cols) x.y = src[1];
      if (k + 2 < j.cols) x.z = src[2];
    }
    const float4 l = make_float4(tf32_lo(x.x, tf32_round(x.x)), tf32_lo(x.y, tf32_round(x.y)),
                                 tf32_lo(x.z, tf32_round(x.z)), tf32_lo(x.w, tf32_round(x.w)));
    *reinterpret_cast<float4*>(j.lo + row * j.colsp + k) = l;
  }
}

// gate: when not null the kernel works only if *gate == 0 (the mixed mode declined the operands).
__global__ void prep_lo_two_kernel(const PrepLoJob a, const PrepLoJob b, int blocks_a, const int* gate = nullptr) {
  grid_launch_dependents();  // the GEMM behind this launch may set itself up now; it waits before reading
  if (gate && *gate != 0) return;
  if (static_cast<int>(blockIdx.x) < blocks_a)
    prep_lo_rows(a, blockIdx.x, blocks_a);
  else
    prep_lo_rows(b, blockIdx.x - blocks_a, gridDim.x - blocks_a);
}

// B[K x N] (row stride ldb) -> hi[N x Kp] (and lo[N x Kp]): 32x32 tiles
// transposed through shared memory; block (32, 8); 1-D grid over
// (Kp/32) * ceil(N/32) tiles.
template <int MODE>
__global__ void prep_b_kernel(const float* __restrict__ B, long long ldb, float* __restrict__ hi,
                              float* __restrict__ lo, int K, int N, int Kp) {
  __shared__ float tile[32][33];
  const long long k_tiles = Kp >> 5;
  const long long n_tiles = (N + 31) >> 5;
  const long long total = k_tiles * n_tiles;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    // n varies fastest so consecutive blocks read consecutive 128-byte runs of a B row
    const long long kt = t / n_tiles;
    const int n0 = static_cast<int>(t - kt * n_tiles) << 5;
    const int k0 = static_cast<int>(kt) << 5;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int k = k0 + threadIdx.y + j, n = n0 + threadIdx.x;
      tile[threadIdx.y + j][threadIdx.x] = (k < K && n < N) ? B[static_cast<long long>(k) * ldb + n] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int n = n0 + threadIdx.y + j, k = k0 + threadIdx.x;
      if (n < N) {
        const float x = tile[threadIdx.x][threadIdx.y + j];
        const float h = tf32_round(x);
        hi[static_cast<long long>(n) * Kp + k] = h;
        if (MODE == 3) lo[static_cast<long long>(n) * Kp + k] = tf32_lo(x, h);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------
// Operand preparation for the fp16 modes
// ------------------------------------------------------------------------
// fp16 has the mantissa of TF32 (11 significant bits) but a 5-bit exponent, so every row of A and every column of
// B is first scaled by a power of two of its own that brings its largest magnitude into [2^14, 2^15) — exact — and
// then split as
//   hi = rn_f16(x * s),   lo = rn_f16(x * s - hi)        (the difference is exact in fp32).
// The epilogue undoes the scales (row_scale[i] * col_scale[j], exact).  Elements more than 2^16 below the largest
// of their row (column) lose low bits of `lo` to fp16's subnormal spacing: an absolute error below 2^-39 of that
// largest element.

// The power of two that maps a largest magnitude (given as float bits) into [2^14, 2^15); 1 for an all-zero row or
// one that holds a NaN or an infinity (its products are non-finite whatever the scale).
__device__ __forceinline__ float f16_panel_scale(unsigned int maxbits) {
  const int e = static_cast<int>(maxbits >> 23);           // biased exponent of the maximum
  if (maxbits == 0 || e == 255) return 1.0f;
  int shift = (14 + 127) - (e == 0 ? 1 : e);              // subnormal maxima count as exponent 1
  if (shift > 127) shift = 127;                            // the scale itself must be a normal float
  if (shift < -126) shift = -126;
  return __uint_as_float(static_cast<unsigned int>(shift + 127) << 23);
}

__device__ __forceinline__ void f16_split(float x, float s, __half& hi, __half& lo) {
  const float xs = x * s;
  hi = __float2half_rn(xs);
  const float h = __half2float(hi);
  lo = (fabsf(h) <= 65504.0f) ? __float2half_rn(xs - h) : __float2half_rn(0.0f);
}

__device__ __forceinline__ unsigned int abs_bits(float x) { return __float_as_uint(x) & 0x7fffffffu; }

// A[M x K] -> hi, lo [M x Kp] halves (lo may be null: single-pass mode), Kp = K rounded up to 64, padding zero, and
// row_scale[M].  One warp per row: a first sweep finds the row's largest magnitude (non-negative floats order like
// unsigned integers), a second — the row comes from cache — scales, splits and stores 8 elements per lane and step
// (two 128-bit loads when the rows allow it, one 128-bit store per panel).
__global__ void prep_a_f16_kernel(const float* __restrict__ A, long long lda, __half* __restrict__ hi, __half* __restrict__ lo,
                                  float* __restrict__ row_scale, int M, int K, int Kp, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (long long row = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); row < M;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const float* src = A + row * lda;
    unsigned int m = 0;
    if (vec_ok) {
      const float4* v = reinterpret_cast<const float4*>(src);
      const int nq = K >> 2;
      int q = lane;
      for (; q + 96 < nq; q += 128) {  // four independent 128-bit loads in flight per lane
        const float4 x0 = v[q], x1 = v[q + 32], x2 = v[q + 64], x3 = v[q + 96];
        m = max(max(m, abs_bits(x0.x)), max(abs_bits(x0.y), max(abs_bits(x0.z), abs_bits(x0.w))));
        m = max(max(m, abs_bits(x1.x)), max(abs_bits(x1.y), max(abs_bits(x1.z), abs_bits(x1.w))));
        m = max(max(m, abs_bits(x2.x)), max(abs_bits(x2.y), max(abs_bits(x2.z), abs_bits(x2.w))));
        m = max(max(m, abs_bits(x3.x)), max(abs_bits(x3.y), max(abs_bits(x3.z), abs_bits(x3.w))));
      }
      for (; q < nq; q += 32) {
        const float4 x = v[q];
        m = max(max(m, abs_bits(x.x)), max(abs_bits(x.y), max(abs_bits(x.z), abs_bits(x.w))));
      }
      for (int k = (K & ~3) + lane; k < K; k += 32) m = max(m, abs_bits(src[k]));
    } else {
      for (int k = lane; k < K; k += 32) m = max(m, abs_bits(src[k]));
    }
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float s = f16_panel_scale(m);
    if (lane == 0) row_scale[row] = 1.0f / s;  // exact: s is a power of two
    for (int k = lane * 8; k < Kp; k += 256) {
      float x[8];
      if (vec_ok && k + 7 < K) {
        const float4 u = *reinterpret_cast<const float4*>(src + k), w = *reinterpret_cast<const float4*>(src + k + 4);
        x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
        x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = (k + j < K) ? src[k + j] : 0.0f;
      }
      __align__(16) __half h[8];
      __align__(16) __half l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f16_split(x[j], s, h[j], l[j]);
      *reinterpret_cast<uint4*>(hi + row * Kp + k) = *reinterpret_cast<const uint4*>(h);
      if (lo) *reinterpret_cast<uint4*>(lo + row * Kp + k) = *reinterpret_cast<const uint4*>(l);
    }
  }
}

// Largest magnitude of every column of B[K x N] as float bits in col_bits[N] (zero before the launch).  Block
// (x, y) scans rows [rows_per_block * y, ...) of a band of columns.  VEC: four columns per thread with 128-bit loads
// (B 16-byte aligned, ldb and N multiples of 4), 1024 columns per block; else one column per thread, 256 per block.
template <bool VEC>
__global__ void colmax_kernel(const float* __restrict__ B, long long ldb, int K, int N, int rows_per_block,
                              unsigned int* __restrict__ col_bits) {
  const int k0 = blockIdx.y * rows_per_block, k1 = min(K, k0 + rows_per_block);
  if (VEC) {
    const int n = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (n >= N) return;
    unsigned int m0 = 0, m1 = 0, m2 = 0, m3 = 0;
    for (int k = k0; k < k1; ++k) {
      const float4 x = *reinterpret_cast<const float4*>(B + static_cast<long long>(k) * ldb + n);
      m0 = max(m0, abs_bits(x.x));
      m1 = max(m1, abs_bits(x.y));
      m2 = max(m2, abs_bits(x.z));
      m3 = max(m3, abs_bits(x.w));
    }
    if (m0) atomicMax(col_bits + n, m0);
    if (m1) atomicMax(col_bits + n + 1, m1);
    if (m2) atomicMax(col_bits + n + 2, m2);
    if (m3) atomicMax(col_bits + n + 3, m3);
  } else {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    unsigned int m = 0;
    for (int k = k0; k < k1; ++k) m = max(m, abs_bits(B[static_cast<long long>(k) * ldb + n]));
    if (m) atomicMax(col_bits + n, m);
  }
}

// B[K x N] -> hi, lo [N x Kp] halves and col_scale[N], transposed through shared memory in tiles of 64 k x 32 n so
// that every warp store writes one 128-byte run of a panel row (64 halves of k); block (32, 8); Kp is a multiple
// of 64; column j is scaled by the power of two its largest magnitude (col_bits) asks for.
__global__ void prep_b_f16_kernel(const float* __restrict__ B, long long ldb, __half* __restrict__ hi, __half* __restrict__ lo,
                                  float* __restrict__ col_scale, const unsigned int* __restrict__ col_bits, int K, int N, int Kp) {
  __shared__ float tile[64][33];
  const long long k_tiles = Kp >> 6;
  const long long n_tiles = (N + 31) >> 5;
  const long long total = k_tiles * n_tiles;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    // n varies fastest so consecutive blocks read consecutive 128-byte runs of a B row
    const long long kt = t / n_tiles;
    const int n0 = static_cast<int>(t - kt * n_tiles) << 5;
    const int k0 = static_cast<int>(kt) << 6;
#pragma unroll
    for (int j = 0; j < 64; j += 8) {
      const int k = k0 + threadIdx.y + j, n = n0 + threadIdx.x;
      tile[threadIdx.y + j][threadIdx.x] = (k < K && n < N) ? B[static_cast<long long>(k) * ldb + n] : 0.0f;
    }
    __syncthreads();
    // lane l of a warp takes k = k0 + 2l and 2l + 1 of panel row n: one 4-byte store per lane, 128 bytes per warp
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int nl = threadIdx.y + j, n = n0 + nl;
      if (n < N) {
        const float s = f16_panel_scale(col_bits[n]);
        if (kt == 0 && threadIdx.x == 0) col_scale[n] = 1.0f / s;
        __half h0, l0, h1, l1;
        f16_split(tile[2 * threadIdx.x][nl], s, h0, l0);
        f16_split(tile[2 * threadIdx.x + 1][nl], s, h1, l1);
        const long long off = static_cast<long long>(n) * Kp + k0 + 2 * threadIdx.x;
        *reinterpret_cast<__half2*>(hi + off) = __halves2half2(h0, h1);
        if (lo) *reinterpret_cast<__half2*>(lo + off) = __halves2half2(l0, l1);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------
// Operand preparation for the mixed mode (SB200_MODE_3XMIXED)
// ------------------------------------------------------------------------
// The three-term split  a*b ~ hi(a)*hi(b) + hi(a)*lo(b) + lo(a)*hi(b)  with hi = rn_tf32, lo = x - hi, as in 3xTF32 mode,
// but only the main term runs on the TF32 pipe (from the caller's fp32 matrices, any magnitudes).  The two cross
// terms are 2^-11 of the main term, need 11-bit factors only, and run on the fp16 pipe at twice the rate: panels
//   hi16 = f16(hi * 2^sa),  lo16 = f16(lo * 2^(sa+11))        (hi has 11 significant bits: exact when normal)
// with ONE power of two per matrix, chosen from its largest magnitude so that the panels peak in [2^14, 2^15) when
// that is possible.  The cross terms are accumulated first, in units of 2^-(sa+sb+11); the accumulator is then scaled by
// that power of two exactly — tcgen05.mma's scale-input-d, at most 2^-15 per instruction: `rescale_stages` MMAs on
// zero tiles and the first MMA of the main term — and the main term is accumulated on top in true units.
// An element more than 2^29 below its matrix's largest loses bits of its cross terms to fp16's subnormal spacing;
// in the worst case (flushed to zero) its products keep TF32 accuracy, 2^-11 relative.  Every other product carries
// the error of 3xTF32 mode.  Magnitudes for which no such scaling exists (product of the two maxima above 2^39 or
// below 2^-60, non-finite values) clear `ok`, and the plain 3xTF32 kernels that follow do the work.
__host__ __device__ __forceinline__ MixCtl mix_plan(unsigned int max_a, unsigned int max_b) {
  MixCtl c;
  c.max_a = max_a;
  c.max_b = max_b;
  c.ok = 0;
  c.rescale_stages = 0;
  c.first_scale = 0;
  c.shift_a = c.shift_b = 0;
  const int ea = static_cast<int>(max_a >> 23), eb = static_cast<int>(max_b >> 23);
  if (ea == 255 || eb == 255) return c;  // an infinity or a NaN somewhere
  if (max_a == 0 || max_b == 0) {        // a zero matrix: the cross terms vanish whatever the scales
    c.ok = 1;
    return c;
  }
  // largest magnitudes lie in [2^alpha, 2^(alpha+1)); subnormal maxima count as exponent -126
  const int alpha = (ea == 0 ? 1 : ea) - 127, beta = (eb == 0 ? 1 : eb) - 127;
  // panels peak below 2^ta and 2^tb; the total rescaling is T = 11 + shift_a + shift_b = 9 + ta + tb - alpha - beta
  int T = 39 - alpha - beta;              // ta = tb = 15
  if (T < 0) return c;                    // magnitudes too large for fp16 panels even unscaled
  if (T > 75) T = 75;                     // at most four rescale stages; smaller panels' peaks instead
  const int tsum = T - 9 + alpha + beta;  // ta + tb
  if (tsum < 8) return c;                 // less than 2^18 of range per matrix: not worth it
  const int ta = tsum - tsum / 2, tb = tsum / 2;
  c.shift_a = ta - alpha - 1;
  c.shift_b = tb - beta - 1;
  if (c.shift_a + 11 > 126 || c.shift_b + 11 > 126 || c.shift_a < -126 || c.shift_b < -126) return c;
  c.rescale_stages = T > 15 ? (T - 1) / 15 : 0;
  c.first_scale = T - 15 * c.rescale_stages;
  c.ok = 1;
  return c;
}

__device__ __forceinline__ float pow2f(int e) { return __uint_as_float(static_cast<unsigned int>(e + 127) << 23); }

__device__ __forceinline__ void mix_split(float x, float s_hi, float s_lo, __half& hi, __half& lo) {
  const float h = tf32_round(x);
  hi = __float2half_rn(h * s_hi);
  lo = __float2half_rn((x - h) * s_lo);
}

struct AbsMaxJob {
  const float* src;
  long long ld;
  int rows, cols, vec_ok;
};

__device__ __forceinline__ void absmax_rows(const AbsMaxJob& j, unsigned int block, unsigned int blocks, unsigned int* out) {
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  unsigned int m = 0;
  for (long long row = static_cast<long long>(block) * warps + (threadIdx.x >> 5); row < j.rows;
       row += static_cast<long long>(blocks) * warps) {
    const float* src = j.src + row * j.ld;
    if (j.vec_ok) {
      const float4* v = reinterpret_cast<const float4*>(src);
      const int nq = j.cols >> 2;
      int q = lane;
      for (; q + 96 < nq; q += 128) {
        const float4 x0 = v[q], x1 = v[q + 32], x2 = v[q + 64], x3 = v[q + 96];
        m = max(max(m, abs_bits(x0.x)), max(abs_bits(x0.y), max(abs_bits(x0.z), abs_bits(x0.w))));
        m = max(max(m, abs_bits(x1.x)), max(abs_bits(x1.y), max(abs_bits(x1.z), abs_bits(x1.w))));
        m = max(max(m, abs_bits(x2.x)), max(abs_bits(x2.y), max(abs_bits(x2.z), abs_bits(x2.w))));
        m = max(max(m, abs_bits(x3.x)), max(abs_bits(x3.y), max(abs_bits(x3.z), abs_bits(x3.w))));
      }
      for (; q < nq; q += 32) {
        const float4 x = v[q];
        m = max(max(m, abs_bits(x.x)), max(abs_bits(x.y), max(abs_bits(x.z), abs_bits(x.w))));
      }
      for (int k = (j.cols & ~3) + lane; k < j.cols; k += 32) m = max(m, abs_bits(src[k]));
    } else {
      for (int k = lane; k < j.cols; k += 32) m = max(m, abs_bits(src[k]));
    }
  }
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0 && m) atomicMax(out, m);
}

// Largest magnitudes of A and of B into ctl->max_a and ctl->max_b (zero before the launch).
__global__ void absmax_two_kernel(const AbsMaxJob a, const AbsMaxJob b, int blocks_a, MixCtl* ctl) {
  if (static_cast<int>(blockIdx.x) < blocks_a)
    absmax_rows(a, blockIdx.x, blocks_a, &ctl->max_a);
  else
    absmax_rows(b, blockIdx.x - blocks_a, gridDim.x - blocks_a, &ctl->max_b);
}

// A[M x K] -> hi16, lo16 [M x Kp] halves, Kp = K rounded up to 64, padding zero; 8 elements per thread and step.
// Block 0 also publishes the plan (ok, rescale stages, scales) for the kernels behind it.
__global__ void prep_mix_a_kernel(const float* __restrict__ A, long long lda, __half* __restrict__ hi, __half* __restrict__ lo,
                                  int M, int K, int Kp, int vec_ok, MixCtl* ctl) {
  const MixCtl plan = mix_plan(ctl->max_a, ctl->max_b);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    ctl->ok = plan.ok;
    ctl->rescale_stages = plan.rescale_stages;
    ctl->first_scale = plan.first_scale;
    ctl->shift_a = plan.shift_a;
    ctl->shift_b = plan.shift_b;
  }
  if (!plan.ok) return;
  const float s_hi = pow2f(plan.shift_a), s_lo = pow2f(plan.shift_a + 11);
  const long long octs_per_row = Kp >> 3;
  const long long total = static_cast<long long>(M) * octs_per_row;
  for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < total;
       q += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = q / octs_per_row;
    const int k = static_cast<int>(q - row * octs_per_row) << 3;
    const float* src = A + row * lda + k;
    float x[8];
    if (vec_ok && k + 7 < K) {
      const float4 u = *reinterpret_cast<const float4*>(src), w = *reinterpret_cast<const float4*>(src + 4);
      x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
      x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (k + j < K) ? src[j] : 0.0f;
    }
    __align__(16) __half h[8];
    __align__(16) __half l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) mix_split(x[j], s_hi, s_lo, h[j], l[j]);
    *reinterpret_cast<uint4*>(hi + row * Kp + k) = *reinterpret_cast<const uint4*>(h);
    *reinterpret_cast<uint4*>(lo + row * Kp + k) = *reinterpret_cast<const uint4*>(l);
  }
}

// B[K x N] -> hi16, lo16 [N x Kp] halves, transposed through shared memory in tiles of 64 k x 32 n as in
// prep_b_f16_kernel; block (32, 8).
__global__ void prep_mix_b_kernel(const float* __restrict__ B, long long ldb, __half* __restrict__ hi, __half* __restrict__ lo,
                                  int K, int N, int Kp, const MixCtl* ctl) {
  grid_launch_dependents();  // the GEMM behind this launch may set itself up now; it waits before reading
  const MixCtl plan = mix_plan(ctl->max_a, ctl->max_b);
  if (!plan.ok) return;
  const float s_hi = pow2f(plan.shift_b), s_lo = pow2f(plan.shift_b + 11);
  __shared__ float tile[64][33];
  const long long k_tiles = Kp >> 6;
  const long long n_tiles = (N + 31) >> 5;
  const long long total = k_tiles * n_tiles;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long kt = t / n_tiles;
    const int n0 = static_cast<int>(t - kt * n_tiles) << 5;
    const int k0 = static_cast<int>(kt) << 6;
#pragma unroll
    for (int j = 0; j < 64; j += 8) {
      const int k = k0 + threadIdx.y + j, n = n0 + threadIdx.x;
      tile[threadIdx.y + j][threadIdx.x] = (k < K && n < N) ? B[static_cast<long long>(k) * ldb + n] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int nl = threadIdx.y + j, n = n0 + nl;
      if (n < N) {
        __half h0, l0, h1, l1;
        mix_split(tile[2 * threadIdx.x][nl], s_hi, s_lo, h0, l0);
        mix_split(tile[2 * threadIdx.x + 1][nl], s_hi, s_lo, h1, l1);
        const long long off = static_cast<long long>(n) * Kp + k0 + 2 * threadIdx.x;
        *reinterpret_cast<__half2*>(hi + off) = __halves2half2(h0, h1);
        *reinterpret_cast<__half2*>(lo + off) = __halves2half2(l0, l1);
      }
    }
    __syncthreads();
  }
}

// Exercises the bounded-wait path without any fault: one thread waits on an mbarrier that nothing ever
// arrives on, for at most limit_ns, then records the give-up in the status word exactly as the GEMM
// roles do, and the block returns normally.
__global__ void wait_timeout_probe_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    mbar_fence_init();
    if (!mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, limit_ns)) atomicCAS(status, 0, 0x900);
  }
}

// Degenerate product (K == 0): D = act(beta*C + bias).
__global__ void gemm_k0_kernel(GemmParams p) {
  const long long total = static_cast<long long>(p.M) * p.N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / p.N;
    const int col = static_cast<int>(i - row * p.N);
    float x = 0.0f;
    if (p.C) x = fmaf(p.beta, p.C[row * p.ldc + col], x);
    if (p.bias) x += p.bias[col];
    if (p.act == 1) x = (x > 0.0f) ? x : 0.0f;
    p.D[row * p.ldd + col] = x;
    if (p.n_replicas) store_replicas(p, row * p.ldd + col, x);
  }
}

}  // namespace sb200
