// ptx_sm100.cuh — thin inline-PTX wrappers for the sm_100a features the GEMM
// kernel uses: mbarrier, bulk-tensor (TMA) loads, tcgen05 tensor-memory
// allocation / MMA / load.  Every wait is bounded; see mbar_wait_bounded.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Wait for the phase with the given parity to complete, for at most
// `limit_ns` of wall time.  Returns false when the wait gave up (either it
// ran out of time or another role of the block already raised the abort
// flag); the caller then leaves its loop and joins the block's teardown.
// The abort flag lives in shared memory so every role sees it quickly.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s, far above any legitimate wait

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// -------------------------------------------------------------------- TMA
// 2-D tiled bulk-tensor load global -> this block's shared memory, completing
// `bytes` on the mbarrier.  x is the innermost coordinate (elements) and must
// make x * 4 a multiple of 16 bytes; callers pass multiples of 32.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// --------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the mbarrier once every tcgen05 operation issued so far by this
// thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// columns [col, col+32) of tensor-memory lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------- CTA pairs (cta_group::2)
// Helpers for kernels launched as clusters of two blocks that drive one
// 256-row MMA together.  Block rank 0 of the pair (the leader) issues the
// MMAs; both blocks load operands and run epilogues.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may
// start while the kernel before it in the stream still runs; grid_dependency_wait() returns once that kernel
// has completed and its writes are visible (at once when there is no such kernel).  A kernel lets its
// successor start early with grid_launch_dependents().
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in block `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// arrive on an mbarrier that may live in the peer block (address from map_to_cta)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are counted on an mbarrier of either block
// of the pair (`bar` is a shared::cluster address); data lands in this block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// The same load carrying an L2 eviction policy (from l2_policy below) for the lines it brings in.
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                      int32_t x, int32_t y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// L2 eviction policies for cache-hinted accesses: 0 normal, 1 evict first (streamed once), 2 evict last (kept
// for the re-reads that follow).  A policy is a 64-bit value that travels with the instruction; it changes
// no setting of the device.
__device__ __forceinline__ uint64_t l2_policy(int kind) {
  uint64_t pol;
  if (kind == 1)
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  else if (kind == 2)
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  else
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ float4 ld_global_v4_hint(const float* p, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ void st_global_v4_hint(float* p, float4 v, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w),
               "l"(policy)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One MMA over both blocks: rows [0,128) of A and D belong to the leader, rows
// [128,256) to its peer; each block's shared memory holds half of B's N rows.
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same MMA on half-precision (fp16) operands with fp32 accumulation: 256 x N x 16 per instruction,
// twice the arithmetic of the TF32 form in the same number of operand bytes and cycles.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same instructions with scale-input-d: D = A*B + D * 2^-scale, scale in 0..15 (an immediate of the instruction,
// hence the switch).  The accumulator is always an input here.
#define SB200_UMMA_SCALED_CASE(KIND, N)                                                                      \
  case N:                                                                                                    \
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 1, 0;\ntcgen05.mma.cta_group::2.kind::" KIND               \
                 " [%0], %1, %2, %3, p, " #N ";\n}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc)       \
                 : "memory");                                                                                \
    break;
#define SB200_UMMA_SCALED_BODY(KIND)                                                                       \
  switch (scale) {                                                                                         \
    SB200_UMMA_SCALED_CASE(KIND, 0) SB200_UMMA_SCALED_CASE(KIND, 1) SB200_UMMA_SCALED_CASE(KIND, 2)        \
    SB200_UMMA_SCALED_CASE(KIND, 3) SB200_UMMA_SCALED_CASE(KIND, 4) SB200_UMMA_SCALED_CASE(KIND, 5)        \
    SB200_UMMA_SCALED_CASE(KIND, 6) SB200_UMMA_SCALED_CASE(KIND, 7) SB200_UMMA_SCALED_CASE(KIND, 8)        \
    SB200_UMMA_SCALED_CASE(KIND, 9) SB200_UMMA_SCALED_CASE(KIND, 10) SB200_UMMA_SCALED_CASE(KIND, 11)      \
    SB200_UMMA_SCALED_CASE(KIND, 12) SB200_UMMA_SCALED_CASE(KIND, 13) SB200_UMMA_SCALED_CASE(KIND, 14)     \
    default:                                                                                               \
      asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 1, 0;\ntcgen05.mma.cta_group::2.kind::" KIND           \
                   " [%0], %1, %2, %3, p, 15;\n}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc)       \
                   : "memory");                                                                            \
      break;                                                                                               \
  }
__device__ __forceinline__ void umma_tf32_pair_scaled(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int scale) {
  SB200_UMMA_SCALED_BODY("tf32")
}
__device__ __forceinline__ void umma_f16_pair_scaled(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int scale) {
  SB200_UMMA_SCALED_BODY("f16")
}
// Arrive on one mbarrier (a shared::cluster address: this block's or the
// peer's) once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// 128 bytes (32 floats) long, stored with the 128-byte swizzle the TMA load
// applies: 8-row groups of 1024 bytes.  Fields (64 bits): start address >> 4
// in [0,14); leading byte offset >> 4 in [16,30) (unused for this layout, 1);
// stride byte offset >> 4 in [32,46) = 1024 >> 4; descriptor version 1 in
// [46,48); layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate, both operands
// K-major, no negation, dense: c_format=1 at bit 4, a_format=2 at bit 7,
// b_format=2 at bit 10, B MN-major flag at bit 16, N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(uint32_t m, uint32_t n, bool b_mn_major = false) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor for kind::f16 with fp16 operands (a_format = b_format = 0), fp32 accumulate, both
// operands K-major: same fields as above.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Round to TF32 (10 explicit mantissa bits), nearest-even: the same rounding a
// tensor map of type TFLOAT32 applies when TMA loads float32 data, so operands
// rounded here and operands rounded by TMA are bit-identical.
__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Shared-memory matrix descriptor for an MN-major TF32 operand (rows of the tile run along N, as in a
// row-major K x N matrix).  32-bit MN-major operands have one legal swizzled layout: 128-byte rows whose
// 32-byte pieces are permuted by (row mod 4), layout type 1, which is what a tensor map with swizzle mode
// 128B_ATOM_32B writes.  The tile is held as slabs of [k rows][32 floats]: four k-rows (512 bytes) form
// one swizzle atom, an MMA k-step of 8 spans two atoms 512 bytes apart (the stride byte offset), and
// consecutive 32-column slabs are `slab_bytes` apart (the leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128_32b(uint32_t smem_addr, uint32_t slab_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((slab_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(1) << 61;
  return d;
}

}  // namespace sb200
