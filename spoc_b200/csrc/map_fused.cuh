// map_fused.cuh — HBM-bound fused element-wise map kernels for sm_100a.
//
// Replaces the scalar one-element-per-thread kernels the reference generates
// for vector_add (benchmarks/bench_vector_add.ml:47-55), stream_triad
// (benchmarks/bench_stream_triad.ml:22-31) and the chains its fusion pass
// builds from them (sarek/sarek/Sarek_fusion.ml:459-547).
//
// One skeleton, instantiated per expression functor: every thread moves
// kUnroll 128-bit vectors per input per iteration (all loads issued before
// the first use, so 2 inputs x 4 x 16 B are in flight per thread), evaluates
// the expression in registers with explicit FMAs, and writes 128-bit vectors
// with a streaming hint.  Nothing is re-read, so the traffic is the
// algorithmic 4 bytes per element per operand.  The ragged ends (up to 3 elements
// before the first aligned vector and up to 3 after the last) are handled inside
// the same launch; operands with differing misalignment take a scalar kernel.
// Either way a map is exactly one launch.
//
// Arithmetic contract (what the parity tests check against the Native
// backend's double-then-round result, <= 1 ulp): one fmaf per multiply-add,
// never left to compiler contraction.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

constexpr int MAP_THREADS = 256;
constexpr int MAP_UNROLL = 4;

__device__ __forceinline__ float4 ld_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.L2::256B.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(float4* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ---- expression functors: out(s) = f(in0, in1, scalar) --------------------
struct VecAddOp {  // c = a + b
  static constexpr int kOutputs = 1;
  __device__ __forceinline__ static void apply(float x0, float x1, float, float& y0, float&) { y0 = x0 + x1; }
};
struct TriadOp {  // a = b + c*s
  static constexpr int kOutputs = 1;
  __device__ __forceinline__ static void apply(float b, float c, float s, float& y0, float&) { y0 = fmaf(c, s, b); }
};
struct ChainOp {  // a = b + c*s ; d = a*a + b   (d only)
  static constexpr int kOutputs = 1;
  __device__ __forceinline__ static void apply(float b, float c, float s, float& y0, float&) {
    const float a = fmaf(c, s, b);
    y0 = fmaf(a, a, b);
  }
};
struct ChainKeepOp {  // same, the intermediate a is also written (y1)
  static constexpr int kOutputs = 2;
  __device__ __forceinline__ static void apply(float b, float c, float s, float& y0, float& y1) {
    const float a = fmaf(c, s, b);
    y0 = fmaf(a, a, b);
    y1 = a;
  }
};

template <class Op>
__device__ __forceinline__ void apply4(const float4& x0, const float4& x1, float s, float4& y0, float4& y1) {
  Op::apply(x0.x, x1.x, s, y0.x, y1.x);
  Op::apply(x0.y, x1.y, s, y0.y, y1.y);
  Op::apply(x0.z, x1.z, s, y0.z, y1.z);
  Op::apply(x0.w, x1.w, s, y0.w, y1.w);
}

// Vector body with ragged ends, one launch: the operands share one 16-byte misalignment, so after
// `head` (0..3) leading elements all four pointers are 16-byte aligned and `nvec` whole vectors follow;
// the up to 3 elements after them and the head are single elements handled by the first threads of
// block 0 (a branch only the first warp of that block diverges on).  Each block owns contiguous chunks
// of MAP_THREADS*MAP_UNROLL vectors so a warp's accesses are 512-byte runs.
template <class Op>
__global__ void __launch_bounds__(MAP_THREADS)
map2_vec_kernel(const float* __restrict__ sin0, const float* __restrict__ sin1, float* __restrict__ sout0,
                float* __restrict__ sout1, float s, int head, long long nvec, long long n) {
  if (blockIdx.x == 0) {
    const long long body_end = head + nvec * 4;
    const int ragged = head + static_cast<int>(n - body_end);  // at most 6
    if (static_cast<int>(threadIdx.x) < ragged) {
      const long long i = static_cast<int>(threadIdx.x) < head ? threadIdx.x : body_end + (threadIdx.x - head);
      float y0, y1;
      Op::apply(sin0[i], sin1[i], s, y0, y1);
      sout0[i] = y0;
      if (Op::kOutputs == 2) sout1[i] = y1;
    }
  }
  const float4* __restrict__ in0 = reinterpret_cast<const float4*>(sin0 + head);
  const float4* __restrict__ in1 = reinterpret_cast<const float4*>(sin1 + head);
  float4* __restrict__ out0 = reinterpret_cast<float4*>(sout0 + head);
  float4* __restrict__ out1 = Op::kOutputs == 2 ? reinterpret_cast<float4*>(sout1 + head) : nullptr;
  constexpr long long kChunk = static_cast<long long>(MAP_THREADS) * MAP_UNROLL;
  const long long nchunks = (nvec + kChunk - 1) / kChunk;
  for (long long c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const long long base = c * kChunk + threadIdx.x;
    float4 x0[MAP_UNROLL], x1[MAP_UNROLL];
    if (base + (MAP_UNROLL - 1) * MAP_THREADS < nvec) {
#pragma unroll
      for (int u = 0; u < MAP_UNROLL; ++u) x0[u] = ld_stream(in0 + base + u * MAP_THREADS);
#pragma unroll
      for (int u = 0; u < MAP_UNROLL; ++u) x1[u] = ld_stream(in1 + base + u * MAP_THREADS);
#pragma unroll
      for (int u = 0; u < MAP_UNROLL; ++u) {
        float4 y0, y1;
        apply4<Op>(x0[u], x1[u], s, y0, y1);
        st_stream(out0 + base + u * MAP_THREADS, y0);
        if (Op::kOutputs == 2) st_stream(out1 + base + u * MAP_THREADS, y1);
      }
    } else {
#pragma unroll
      for (int u = 0; u < MAP_UNROLL; ++u) {
        const long long i = base + u * MAP_THREADS;
        if (i < nvec) {
          float4 y0, y1;
          apply4<Op>(ld_stream(in0 + i), ld_stream(in1 + i), s, y0, y1);
          st_stream(out0 + i, y0);
          if (Op::kOutputs == 2) st_stream(out1 + i, y1);
        }
      }
    }
  }
}

// Scalar path: elements [first, n).  Used for vectors shorter than one 128-bit vector after the head
// and for operands whose addresses differ in their 16-byte misalignment (4-byte accesses stay coalesced).
template <class Op>
__global__ void __launch_bounds__(MAP_THREADS)
map2_scalar_kernel(const float* __restrict__ in0, const float* __restrict__ in1, float* __restrict__ out0,
                   float* __restrict__ out1, float s, long long first, long long n) {
  for (long long i = first + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float y0, y1;
    Op::apply(in0[i], in1[i], s, y0, y1);
    out0[i] = y0;
    if (Op::kOutputs == 2) out1[i] = y1;
  }
}

// ---- seeded synthetic data (counter-based, splitmix64) ----------------------
__device__ __forceinline__ uint64_t splitmix64_dev(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void fill_kernel(float* __restrict__ dst, long long n, uint64_t seed, uint64_t stream_id, int kind,
                            double sigma, long long first) {
  const uint64_t key = seed ^ (stream_id * 0x9E3779B97F4A7C15ull);
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint64_t r = splitmix64_dev(key ^ static_cast<uint64_t>(first + j));
    float v;
    if (kind == 2) {
      const double u1 = static_cast<double>((r >> 40) + 1) * (1.0 / 16777216.0);
      const double u2 = static_cast<double>((r >> 16) & 0xFFFFFF) * (1.0 / 16777216.0);
      v = static_cast<float>(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2) * sigma);
    } else {
      v = static_cast<float>(static_cast<double>(r >> 40) * (1.0 / 8388608.0) - 1.0);
      if (kind == 1) v = __fmul_rn(v, 0.1f);
    }
    dst[j] = v;
  }
}

}  // namespace sb200
