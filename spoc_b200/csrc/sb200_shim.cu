// sb200_shim.cu — the C ABI of libsarek_b200.so (see include/sb200.h).
//
// Host side of the B200 backend: device/memory/stream/event plumbing in the
// shape of sarek-cuda/Cuda_api.ml, kernel "compilation" (IR recognition) and
// launch in the shape of sarek-cuda/Cuda_plugin.ml:174-210, and the direct
// GEMM / map operators the recognised kernels dispatch to.  There is no CPU
// execution path in this library: every operator launches CUDA kernels or
// returns an error.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <thread>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/sb200.h"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_pair.cuh"
#include "internal.hpp"
#include "ir.hpp"
#include "map_fused.cuh"
#include "map_jit.hpp"
#include "transfer.hpp"

using namespace sb200;

namespace {

constexpr int kMaxDevices = 16;
constexpr int kVersion = 100;

thread_local std::string g_err;
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_mode{0};  // 0 = not yet read from the environment

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  // clear the sticky-less error state so the next call starts clean
  cudaGetLastError();
  return fail(static_cast<int>(e), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

#define CU_TRY(call)                                      \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

bool debug_kernel() {
  static int v = -1;
  if (v < 0) {
    const char* s = getenv("SAREK_DEBUG");
    v = (s && (strstr(s, "kernel") || strstr(s, "all"))) ? 1 : 0;
  }
  return v == 1;
}

struct DeviceState {
  std::mutex mu;
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  // the scratch is shared by every stream of the device: a call on another stream than the last user's waits for it
  cudaEvent_t ws_event = nullptr;
  cudaStream_t ws_last_stream = nullptr;
  bool ws_in_use = false;
  // held by a call from the moment it sizes the scratch until its launches are enqueued and its event recorded, so
  // that another host thread cannot free and regrow the scratch under launches that already point into it
  std::mutex scratch_mu;
  int* status = nullptr;  // device word written by kernels whose bounded waits expire
  MixCtl* mix_ctl = nullptr;  // control words of the mixed mode (largest magnitudes, plan), ordered like the scratch
  unsigned int* epoch_rings = nullptr;  // eight rings of epoch counters for the soft lockstep of long k-loops
  std::atomic<unsigned int> epoch_seq{0};
  // set by every launch of a kernel that has bounded waits; while it is clear a synchronise has nothing to read
  // back, which keeps the launch-plus-synchronise latency of the map kernels free of a device-to-host copy
  std::atomic<bool> status_armed{false};
  std::map<uint64_t, uint64_t> allocs;  // base address -> bytes of every buffer sb200_mem_alloc handed out (ordered: range lookups)
  // kernel profiling (enable_profiling): event triples recorded around the GEMM stages
  struct ProfRec {
    cudaEvent_t e0, e1, e2;
  };
  std::vector<ProfRec> prof;
  // host-operand GEMM (sb200_gemm_f32_host): device mirrors of the operands and three streams
  void* host_stage = nullptr;
  size_t host_stage_bytes = 0;
  cudaStream_t pipe_in = nullptr, pipe_compute = nullptr, pipe_out = nullptr;
  std::mutex host_call_mu;  // one host-operand call per device at a time: they share the mirrors and the three streams
};
DeviceState g_dev[kMaxDevices];
std::atomic<int> g_profiling{0};
std::atomic<int> g_gemm_variant{-1};  // -1 = not yet read from the environment; 0 auto, 1 single-CTA tiles, 2 CTA pairs

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
std::once_flag g_encode_once;

int device_ready(int dev, DeviceState** out) {
  if (dev < 0 || dev >= kMaxDevices) return fail(SB200_ERR_INVALID_VALUE, "device index %d out of range", dev);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(SB200_ERR_NO_DEVICE, "no CUDA device available (%s)", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
  }
  if (dev >= count) return fail(SB200_ERR_INVALID_VALUE, "device index %d but only %d device(s)", dev, count);
  DeviceState& d = g_dev[dev];
  CU_TRY(cudaSetDevice(dev));
  std::lock_guard<std::mutex> lock(d.mu);
  if (!d.ready) {
    cudaDeviceProp prop;
    CU_TRY(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return fail(SB200_ERR_NO_DEVICE, "device %d is sm_%d%d; this library carries sm_100a code only", dev, prop.major,
                  prop.minor);
    d.sm_count = prop.multiProcessorCount;
    d.cc_major = prop.major;
    CU_TRY(cudaMalloc(&d.status, sizeof(int)));
    CU_TRY(cudaMemset(d.status, 0, sizeof(int)));
    d.ready = true;
  }
  *out = &d;
  return SB200_OK;
}

// device_wide: the caller has just synchronised the whole device, so nothing that could still raise the word is in
// flight and the check is disarmed until the next such launch; after a stream synchronise it stays armed.
int check_status_word(DeviceState& d, bool device_wide = false) {
  if (!d.status_armed.load()) return SB200_OK;
  if (device_wide) d.status_armed.store(false);
  int h = 0;
  CU_TRY(cudaMemcpy(&h, d.status, sizeof(int), cudaMemcpyDeviceToHost));
  if (h != 0) {
    cudaMemset(d.status, 0, sizeof(int));
    return fail(SB200_ERR_TIMEOUT, "a bounded device-side wait expired in the GEMM pipeline (site 0x%x)", h);
  }
  return SB200_OK;
}

// An operand that lies inside a buffer this library allocated must end inside it too; operands in memory from
// elsewhere (another allocator's) are taken at the caller's word.  Turns a wrong size into an error instead of a fault.
int check_extent(DeviceState& d, uint64_t ptr, uint64_t bytes, const char* what) {
  if (!ptr || bytes == 0) return SB200_OK;
  std::lock_guard<std::mutex> lock(d.mu);
  auto it = d.allocs.upper_bound(ptr);
  if (it == d.allocs.begin()) return SB200_OK;
  --it;
  if (ptr >= it->first + it->second) return SB200_OK;  // not inside one of ours
  if (ptr + bytes > it->first + it->second)
    return fail(SB200_ERR_BOUNDS, "%s needs %llu bytes from its address but the buffer it lies in ends after %llu", what,
                static_cast<unsigned long long>(bytes), static_cast<unsigned long long>(it->first + it->second - ptr));
  return SB200_OK;
}

inline cudaStream_t as_stream(uint64_t s) { return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(s)); }
inline cudaEvent_t as_event(uint64_t e) { return reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(e)); }
template <class T>
inline T* as_ptr(uint64_t p) {
  return reinterpret_cast<T*>(static_cast<uintptr_t>(p));
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, what);
  count_launch();
  return SB200_OK;
}

int current_mode() {
  int m = g_mode.load();
  if (m == 0) {
    const char* s = getenv("SAREK_B200_MODE");
    m = (s && (!strcmp(s, "tf32") || !strcmp(s, "TF32"))) ? SB200_MODE_TF32
        : (s && (!strcmp(s, "3xf16") || !strcmp(s, "3xF16"))) ? SB200_MODE_3XF16
        : (s && (!strcmp(s, "f16") || !strcmp(s, "F16"))) ? SB200_MODE_F16
        : (s && (!strcmp(s, "3xmixed") || !strcmp(s, "mixed"))) ? SB200_MODE_3XMIXED : SB200_MODE_3XTF32;
    g_mode.store(m);
  }
  return m;
}

// --------------------------------------------------------------- map host
template <class Op>
int launch_map2(DeviceState& d, cudaStream_t st, const float* in0, const float* in1, float* out0, float* out1, float s,
                long long n) {
  if (n <= 0) return SB200_OK;
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(in0), a1 = reinterpret_cast<uintptr_t>(in1),
                  a2 = reinterpret_cast<uintptr_t>(out0),
                  a3 = Op::kOutputs == 2 ? reinterpret_cast<uintptr_t>(out1) : a2;
  const uintptr_t mis = a0 & 15;
  const bool same = (a1 & 15) == mis && (a2 & 15) == mis && (a3 & 15) == mis && (mis & 3) == 0;
  long long head = 0, nvec = 0;
  if (same) {
    head = mis ? static_cast<long long>((16 - mis) >> 2) : 0;
    if (head > n) head = n;
    nvec = (n - head) >> 2;
  }
  if (nvec > 0) {
    // one launch: vector body, with the ragged ends taken by the first threads of block 0
    const long long chunk = static_cast<long long>(MAP_THREADS) * MAP_UNROLL;
    const long long nchunks = (nvec + chunk - 1) / chunk;
    long long grid = nchunks;
    const long long cap = static_cast<long long>(d.sm_count) * 32;
    if (grid > cap) grid = cap;
    map2_vec_kernel<Op><<<static_cast<unsigned>(grid), MAP_THREADS, 0, st>>>(in0, in1, out0, Op::kOutputs == 2 ? out1 : nullptr, s,
                                                                             static_cast<int>(head), nvec, n);
    return launch_check("map body");
  }
  {
    long long grid = (n + MAP_THREADS - 1) / MAP_THREADS;
    const long long cap = static_cast<long long>(d.sm_count) * 16;
    if (grid > cap) grid = cap;
    map2_scalar_kernel<Op><<<static_cast<unsigned>(grid), MAP_THREADS, 0, st>>>(in0, in1, out0, out1, s, 0, n);
    int rc = launch_check("map scalar");
    if (rc) return rc;
  }
  return SB200_OK;
}

int run_map(DeviceState& d, cudaStream_t st, int op, uint64_t out0, uint64_t out1, uint64_t in0, uint64_t in1, float s,
            long long n) {
  if (n < 0) return fail(SB200_ERR_INVALID_VALUE, "negative element count %lld", n);
  if (n == 0) return SB200_OK;
  if (!out0 || !in0 || !in1) return fail(SB200_ERR_INVALID_VALUE, "null device pointer passed to a map operator");
  if ((out0 | out1 | in0 | in1) & 3) return fail(SB200_ERR_ALIGNMENT, "float32 vectors must be 4-byte aligned");
  for (uint64_t p : {out0, out1, in0, in1}) {
    int rc = check_extent(d, p, static_cast<uint64_t>(n) * 4, "map operand");
    if (rc) return rc;
  }
  const float* p0 = as_ptr<const float>(in0);
  const float* p1 = as_ptr<const float>(in1);
  float* q0 = as_ptr<float>(out0);
  float* q1 = as_ptr<float>(out1);
  switch (op) {
    case OP_VECADD: return launch_map2<VecAddOp>(d, st, p0, p1, q0, nullptr, s, n);
    case OP_TRIAD: return launch_map2<TriadOp>(d, st, p0, p1, q0, nullptr, s, n);
    case OP_CHAIN: return launch_map2<ChainOp>(d, st, p0, p1, q0, nullptr, s, n);
    case OP_CHAIN_KEEP:
      if (!out1) return fail(SB200_ERR_INVALID_VALUE, "null intermediate vector");
      return launch_map2<ChainKeepOp>(d, st, p0, p1, q0, q1, s, n);
  }
  return fail(SB200_ERR_INVALID_VALUE, "unknown map operator %d", op);
}

// -------------------------------------------------------------- GEMM host
inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

int ensure_workspace(DeviceState& d, size_t bytes) {
  if (bytes <= d.workspace_bytes) return SB200_OK;
  if (d.workspace) {
    CU_TRY(cudaDeviceSynchronize());
    CU_TRY(cudaFree(d.workspace));
    d.workspace = nullptr;
    d.workspace_bytes = 0;
  }
  CU_TRY(cudaMalloc(&d.workspace, bytes));
  d.workspace_bytes = bytes;
  return SB200_OK;
}

int encode_map_2d(CUtensorMap* map, const float* base, long long inner, long long rows, long long row_stride_elems, int box_inner,
                  int box_rows, bool round_tf32, bool atom32 = false);

int resolve_encode_tiled() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    cudaGetLastError();
  });
  if (!g_encode_tiled) return fail(SB200_ERR_NO_DEVICE, "driver does not export cuTensorMapEncodeTiled");
  return SB200_OK;
}

int encode_panel_map(CUtensorMap* map, const float* base, long long kp, long long rows, int box_rows) {
  return encode_map_2d(map, base, kp, rows, kp, GEMM_BK, box_rows, false);
}

// 2-D float32 tensor map with the 128-byte swizzle.  round_tf32 selects the TFLOAT32 element type:
// TMA then rounds each value to TF32 (nearest-even) while loading.
// atom32 selects the 128-byte swizzle with 32-byte atoms, the layout an MN-major TF32 operand needs.
int encode_map_2d(CUtensorMap* map, const float* base, long long inner, long long rows, long long row_stride_elems, int box_inner,
                  int box_rows, bool round_tf32, bool atom32) {
  const long long kp = inner;
  if (int rc = resolve_encode_tiled()) return rc;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(kp), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride_elems) * 4};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode_tiled(map, round_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SB200_ERR_INVALID_VALUE, "cuTensorMapEncodeTiled failed with CUresult %d (kp=%lld rows=%lld)", (int)r, kp,
                rows);
  return SB200_OK;
}

std::atomic<int> g_l2_policy{-1};  // -1 = not yet read from the environment

// Eviction-policy bits the GEMM kernels attach to their loads and stores (GemmParams::l2_policy);
// SAREK_B200_L2_POLICY overrides the default for experiments.
int l2_policy_setting() {
  int v = g_l2_policy.load();
  if (v < 0) {
    const char* e = getenv("SAREK_B200_L2_POLICY");
    v = e ? (atoi(e) & 63) : 0;
    g_l2_policy.store(v);
  }
  return v;
}

// Fields of GemmParams that follow from the others: whether the epilogue may move 128-bit vectors, and the
// eviction policies.
int env_int(const char* name, int fallback, int lo, int hi) {
  const char* e = getenv(name);
  const int v = e ? atoi(e) : fallback;
  return v >= lo && v <= hi ? v : fallback;
}

void derive_params(GemmParams* gp) {
  static const int epoch_stages = env_int("SAREK_B200_LOCKSTEP_STAGES", 64, 4, 4096);
  static const int epoch_wait_ns = env_int("SAREK_B200_LOCKSTEP_WAIT_NS", 4000, 0, 1000000);
  gp->epoch_stages = epoch_stages;
  gp->epoch_wait_ns = epoch_wait_ns;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  bool vec = (gp->N & 3) == 0 && al16(gp->D) && (gp->ldd & 3) == 0 && (!gp->C || (al16(gp->C) && (gp->ldc & 3) == 0)) &&
             (!gp->bias || al16(gp->bias));
  for (int r = 0; r < gp->n_replicas; ++r) vec = vec && al16(gp->replicas[r]);
  gp->vec_epilogue = vec ? 1 : 0;
  gp->l2_policy = l2_policy_setting();
}

// The epoch counters for one launch of the CTA-pair kernel, zeroed on `st` — or null when the lockstep is off: k-loops
// below 128 stages (K < 4096: two epochs at most, nothing to hold together), SAREK_B200_LOCKSTEP=0, or no memory for the
// rings.  Measured in the sustained loop at 8192^3: 245 against 221-227 TFLOP/s in alternating runs on one box, the SM
// clock under the power cap 1400 against 1267-1305 MHz, because the pairs that stay together re-read less from DRAM.  Eight rings are handed out in turn so that launches in flight on several streams rarely share one
// (sharing only blunts the hint).
std::atomic<int> g_lockstep{-2};  // -2 = not yet read from the environment; -1 by k-loop length, 0 off, 1 always

unsigned int* next_epoch_ring(DeviceState& d, cudaStream_t st, long long stages_per_tile, bool by_default = true) {
  int setting = g_lockstep.load();
  if (setting == -2) {
    const char* e = getenv("SAREK_B200_LOCKSTEP");
    setting = e ? (atoi(e) != 0 ? 1 : 0) : -1;
    g_lockstep.store(setting);
  }
  // by_default = false: TF32 mode.  Its stages are a third as long as 3xTF32's, so an epoch's wait weighs three times as
  // much, and alternating runs gave 474-476 TFLOP/s with the lockstep against 593-606 without on one box (573 against 535
  // on another): off unless forced.
  if (setting == 0 || (setting < 0 && (stages_per_tile < 128 || !by_default))) return nullptr;
  constexpr int kRings = 8, kRingWords = 64;
  if (!d.epoch_rings) {
    // never allocate while the stream is being captured into a graph (it would invalidate the capture): such a
    // launch simply runs without the hint
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return nullptr;
    }
    std::lock_guard<std::mutex> lock(d.mu);
    if (!d.epoch_rings && cudaMalloc(&d.epoch_rings, kRings * kRingWords * sizeof(unsigned int)) != cudaSuccess) {
      cudaGetLastError();
      d.epoch_rings = nullptr;
      return nullptr;
    }
  }
  unsigned int* ring = d.epoch_rings + (d.epoch_seq.fetch_add(1) % kRings) * kRingWords;
  if (cudaMemsetAsync(ring, 0, kRingWords * sizeof(unsigned int), st) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return ring;
}

size_t gemm_workspace_need(int mode, long long M, long long N, long long K) {
  const long long kp = round_up(K, GEMM_BK);
  const size_t ops = mode == SB200_MODE_3XTF32 ? 2 : 1;
  const size_t a = round_up(M * kp * 4, 1024), b = round_up(N * kp * 4, 1024);
  return ops * (a + b);
}

std::atomic<int> g_tile_n{-1};  // -1 = not yet read from the environment; 0 automatic, else 64 / 128 / 256

// Tile columns for the CTA-pair kernel.  256x256 tiles have the best ratio of tensor-core work to
// shared-memory and L2 traffic, so they serve every problem that fills the GPU with them.  A problem
// with fewer tiles than CTA pairs takes a narrower tile, which puts more SMs to work and shortens
// the epilogue that nothing overlaps when a pair computes a single tile.  The estimate is in
// MMA-cycle units per pair: waves * (k-blocks * cycles per k-block + fill and epilogue).
int choose_tile_n(long long M, long long N, long long kblocks, int clusters, int mode) {
  int forced = g_tile_n.load();
  if (forced < 0) {
    const char* e = getenv("SAREK_B200_TILE_N");
    forced = e ? atoi(e) : 0;
    if (forced != 64 && forced != 128 && forced != 256) forced = 0;
    g_tile_n.store(forced);
  }
  if (forced) return forced;
  const long long tiles_m = (M + PAIR_BM - 1) / PAIR_BM;
  const double mmas = mode == 3 ? 3.0 : 1.0;
  auto cost = [&](int bn) {
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    const long long waves = (tiles + clusters - 1) / clusters;
    // cycles per k-block: 4 MMAs of bn/2 cycles each (x3 in 3xTF32 mode), or the time to fetch the stage at
    // about 60 bytes per cycle and SM, whichever is longer.  That rate is the 192 KiB ring divided by the
    // loaded TMA latency (measured); narrow tiles need more bytes per MMA cycle because A is re-read once
    // per column of tiles, so they are fetch-bound where 256-column tiles are tensor-bound
    const double mma_cycles = 4.0 * (bn / 2.0) * mmas;
    const double fetch_cycles = (mode == 3 ? 2.0 : 1.0) * (16384.0 + bn * 64.0) / 60.0;
    const double per_kblock = (mma_cycles > fetch_cycles ? mma_cycles : fetch_cycles) * (bn == 256 ? 1.0 : 1.1);
    const double fixed = 6000.0 + 1000.0 * (bn / 32.0);
    return static_cast<double>(waves) * (static_cast<double>(kblocks) * per_kblock + fixed);
  };
  int best = 256;
  double best_cost = cost(256);
  for (int bn : {128, 64}) {
    const double c = cost(bn);
    if (c < 0.97 * best_cost) {  // a narrower tile must win clearly
      best = bn;
      best_cost = c;
    }
  }
  return best;
}

// One instantiation of the CTA-pair kernel: shared-memory attribute and resident-cluster count are
// looked up once per device, then the launch.
template <int MODE, bool DIRECT, int BN>
int launch_pair(DeviceState& d, int dev_index, cudaStream_t st, const CUtensorMap& ma_hi, const CUtensorMap& mb_hi,
                const CUtensorMap& ma_lo, const CUtensorMap& mb_lo, GemmParams gp, long long M, long long N,
                const CUtensorMap* ma_x = nullptr, const CUtensorMap* mb_x = nullptr) {
  using PCfg = PairCfg<MODE, BN>;
  static std::atomic<int> resident[kMaxDevices];  // 0 = not yet asked
  int max_clusters = resident[dev_index].load();
  if (max_clusters == 0) {
    CU_TRY(cudaFuncSetAttribute(gemm_pair_kernel<MODE, DIRECT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(PCfg::kSmemBytes)));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(static_cast<unsigned>(d.sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PCfg::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, gemm_pair_kernel<MODE, DIRECT, BN>, &cfg) != cudaSuccess ||
        max_clusters <= 0) {
      cudaGetLastError();
      max_clusters = d.sm_count / 2;
    }
    resident[dev_index].store(max_clusters);
  }
  gp.tiles_m = static_cast<int>((M + PAIR_BM - 1) / PAIR_BM);
  gp.tiles_n = static_cast<int>((N + BN - 1) / BN);
  gp.group_m = PAIR_GROUP_M;  // 8 measured best at 8192^3 against 2, 4, 16, 32 (both modes)
  const long long tiles = static_cast<long long>(gp.tiles_m) * gp.tiles_n;
  const long long pairs = tiles < max_clusters ? tiles : max_clusters;
  // programmatic dependent launch: the kernel's set-up may overlap the preparation launch in front of it
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = PCfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  CU_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE, DIRECT, BN>, ma_hi, mb_hi, ma_lo, mb_lo, ma_x ? *ma_x : ma_lo,
                            mb_x ? *mb_x : mb_lo, gp));
  return launch_check("gemm_pair_kernel");
}

template <int MODE, bool DIRECT>
int launch_pair_bn(int bn, DeviceState& d, int dev_index, cudaStream_t st, const CUtensorMap& ma_hi, const CUtensorMap& mb_hi,
                   const CUtensorMap& ma_lo, const CUtensorMap& mb_lo, const GemmParams& gp, long long M, long long N,
                   const CUtensorMap* ma_x = nullptr, const CUtensorMap* mb_x = nullptr) {
  if (bn == 64) return launch_pair<MODE, DIRECT, 64>(d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N, ma_x, mb_x);
  if (bn == 128) return launch_pair<MODE, DIRECT, 128>(d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N, ma_x, mb_x);
  return launch_pair<MODE, DIRECT, 256>(d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N, ma_x, mb_x);
}

// How sb200_gemm_f32 will run a product: which kernel, which tile, how much scratch.  One function decides, the
// launch path and sb200_gemm_describe both ask it.
struct GemmRoute {
  bool pair = false;    // CTA-pair kernel (else the single-CTA kernel)
  bool direct = false;  // operands read where they lie (else from prepared panels)
  int tile_n = GEMM_BN;
  int stages = 0;
  long long tiles = 0, waves = 0;
  size_t workspace = 0;  // bytes of library scratch
};

int gemm_variant_setting() {
  int variant = g_gemm_variant.load();
  if (variant < 0) {
    const char* e = getenv("SAREK_B200_GEMM");
    variant = (e && !strcmp(e, "single")) ? 1 : (e && !strcmp(e, "pair")) ? 2 : (e && !strcmp(e, "pair-panels")) ? 3 : 0;
    g_gemm_variant.store(variant);
  }
  return variant;
}

GemmRoute route_gemm(int mode, long long M, long long N, long long K, bool addressable, int sm_count, long long panel_rows_a) {
  GemmRoute r;
  const int variant = gemm_variant_setting();
  // CTA pairs work on 256-row tiles.  With at most 128 rows the second block of a pair computes nothing, and
  // the pair kernel still wins when it can read the operands directly (measured 2x at 64..128 rows: no
  // transposing pass over B); from prepared panels the single-CTA kernel serves such problems.
  r.pair = variant >= 2 || (variant == 0 && (M > GEMM_BM || addressable));
  // CTA pairs read the caller's matrices directly when TMA can address them: 16-byte aligned bases and
  // row strides.  TMA rounds A and B to TF32 while loading and B is consumed N-major, so TF32 mode needs
  // neither preparation kernels nor panel scratch, and 3xTF32 mode prepares only the low parts.
  r.direct = r.pair && variant != 3 && addressable;
  const long long kp = round_up(K, GEMM_BK);
  const int clusters = sm_count / 2 > 0 ? sm_count / 2 : 1;
  r.tile_n = r.pair ? choose_tile_n(M, N, kp / GEMM_BK, clusters, mode == SB200_MODE_3XTF32 ? 3 : 1) : GEMM_BN;
  if (r.pair) {
    const bool three = mode == SB200_MODE_3XTF32;
    r.stages = r.tile_n == 256 ? (three ? PairCfg<3, 256>::kStages : PairCfg<1, 256>::kStages)
             : r.tile_n == 128 ? (three ? PairCfg<3, 128>::kStages : PairCfg<1, 128>::kStages)
                               : (three ? PairCfg<3, 64>::kStages : PairCfg<1, 64>::kStages);
    r.tiles = ((M + PAIR_BM - 1) / PAIR_BM) * ((N + r.tile_n - 1) / r.tile_n);
    r.waves = (r.tiles + clusters - 1) / clusters;
  } else {
    r.stages = mode == SB200_MODE_3XTF32 ? GemmCfg<3>::kStages : GemmCfg<1>::kStages;
    r.tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
    r.waves = (r.tiles + sm_count - 1) / (sm_count > 0 ? sm_count : 1);
  }
  if (panel_rows_a < M) panel_rows_a = M;
  if (!r.direct) {
    r.workspace = gemm_workspace_need(mode, panel_rows_a, N, K);
  } else if (mode == SB200_MODE_3XTF32) {
    r.workspace = round_up(K * round_up(N, 32) * 4, 1024) + round_up(panel_rows_a * kp * 4, 1024);
  }
  return r;
}

template <int MODE>
int launch_gemm_mode(DeviceState& d, cudaStream_t st, long long M, long long N, long long K, const float* A,
                     long long lda, const float* B, long long ldb, const GemmParams& gp_in, long long panel_rows_a = 0,
                     bool b_panels_ready = false) {
  // panel_rows_a: rows the A panels are laid out for (>= M); callers that run several row blocks
  // against one prepared B pass the largest block so that the B panels keep their place.
  if (panel_rows_a < M) panel_rows_a = M;
  using Cfg = GemmCfg<MODE>;

  const bool addressable = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 3) == 0 &&
                           (reinterpret_cast<uintptr_t>(B) & 15) == 0 && (ldb & 3) == 0;
  const GemmRoute route = route_gemm(MODE == 3 ? SB200_MODE_3XTF32 : SB200_MODE_TF32, M, N, K, addressable, d.sm_count, panel_rows_a);
  const bool pair = route.pair, direct = route.direct;
  const int tile_n = route.tile_n;

  const long long kp = round_up(K, GEMM_BK);
  const size_t a_bytes = round_up(panel_rows_a * kp * 4, 1024), b_bytes = round_up(N * kp * 4, 1024);
  int rc = SB200_OK;
  const long long np = round_up(N, 32);  // row length of the low-part panel of B in the direct layout
  const size_t blo_bytes = round_up(K * np * 4, 1024);
  // Calls that use the device's scratch are ordered across streams: two streams would otherwise write their
  // operand panels into the same memory at once.  Not while the stream is being captured into a graph (an
  // event of the capture cannot order work outside it): a captured sequence is ordered by its own stream.
  bool track_scratch = false;
  std::unique_lock<std::mutex> scratch_lock(d.scratch_mu, std::defer_lock);
  if (route.workspace) {
    scratch_lock.lock();
    rc = ensure_workspace(d, route.workspace);
    if (rc) return rc;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
      cudaGetLastError();
      cap = cudaStreamCaptureStatusActive;
    }
    track_scratch = cap == cudaStreamCaptureStatusNone;
    if (track_scratch) {
      std::lock_guard<std::mutex> lock(d.mu);
      if (d.ws_in_use && d.ws_last_stream != st) CU_TRY(cudaStreamWaitEvent(st, d.ws_event, 0));
    }
  }
  unsigned int* epoch_ring = pair ? next_epoch_ring(d, st, kp / GEMM_BK, MODE == 3) : nullptr;  // zeroed ahead of the preparation launch
  const bool prof = g_profiling.load() != 0;
  DeviceState::ProfRec rec{nullptr, nullptr, nullptr};
  if (prof) {
    CU_TRY(cudaEventCreate(&rec.e0));
    CU_TRY(cudaEventCreate(&rec.e1));
    CU_TRY(cudaEventCreate(&rec.e2));
    CU_TRY(cudaEventRecord(rec.e0, st));
  }
  CUtensorMap ma_hi, mb_hi, ma_lo, mb_lo;
  if (direct) {
    if ((rc = encode_map_2d(&ma_hi, A, K, M, lda, GEMM_BK, GEMM_BM, true))) return rc;
    if ((rc = encode_map_2d(&mb_hi, B, N, K, ldb, 32, GEMM_BK, true, true))) return rc;
    ma_lo = ma_hi;
    mb_lo = mb_hi;
    if constexpr (MODE == 3) {
      // low parts only: B's first (K x np, row-major like B), then A's (rows x kp)
      uint8_t* ws = static_cast<uint8_t*>(d.workspace);
      float* b_lo = reinterpret_cast<float*>(ws);
      float* a_lo = reinterpret_cast<float*>(ws + blo_bytes);
      const long long cap = static_cast<long long>(d.sm_count) * 16;
      long long grid_a = (M * (kp >> 2) + 255) / 256;
      if (grid_a > cap) grid_a = cap;
      if (b_panels_ready) {
        prep_a_kernel<3, true><<<static_cast<unsigned>(grid_a), 256, 0, st>>>(A, lda, nullptr, a_lo, static_cast<int>(M),
                                                                               static_cast<int>(K), static_cast<int>(kp), 1);
        if ((rc = launch_check("prep_a_kernel(lo)"))) return rc;
      } else {
        // both low-part panels in one launch
        long long grid_b = (K * (np >> 2) + 255) / 256;
        if (grid_b > cap) grid_b = cap;
        const PrepLoJob ja{A, lda, a_lo, static_cast<int>(M), static_cast<int>(K), static_cast<int>(kp)};
        const PrepLoJob jb{B, ldb, b_lo, static_cast<int>(K), static_cast<int>(N), static_cast<int>(np)};
        prep_lo_two_kernel<<<static_cast<unsigned>(grid_a + grid_b), 256, 0, st>>>(ja, jb, static_cast<int>(grid_a));
        if ((rc = launch_check("prep_lo_two_kernel"))) return rc;
      }
      if ((rc = encode_map_2d(&ma_lo, a_lo, kp, M, kp, GEMM_BK, GEMM_BM, false))) return rc;
      if ((rc = encode_map_2d(&mb_lo, b_lo, N, K, np, 32, GEMM_BK, false, true))) return rc;
    }
  } else {
    // workspace layout: B panels first (their size does not depend on M), then the A panels
    uint8_t* ws = static_cast<uint8_t*>(d.workspace);
    constexpr size_t kOps = MODE == 3 ? 2 : 1;
    float* b_hi = reinterpret_cast<float*>(ws);
    float* b_lo = MODE == 3 ? reinterpret_cast<float*>(ws + b_bytes) : b_hi;
    float* a_hi = reinterpret_cast<float*>(ws + kOps * b_bytes);
    float* a_lo = MODE == 3 ? reinterpret_cast<float*>(ws + kOps * b_bytes + a_bytes) : a_hi;
    {
      const long long quads = M * (kp >> 2);
      long long grid = (quads + 255) / 256;
      const long long cap = static_cast<long long>(d.sm_count) * 16;
      if (grid > cap) grid = cap;
      const int vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 3) == 0) ? 1 : 0;
      prep_a_kernel<MODE><<<static_cast<unsigned>(grid), 256, 0, st>>>(A, lda, a_hi, a_lo, static_cast<int>(M),
                                                                        static_cast<int>(K), static_cast<int>(kp), vec_ok);
      rc = launch_check("prep_a_kernel");
      if (rc) return rc;
    }
    if (!b_panels_ready) {
      const long long tiles = (kp >> 5) * ((N + 31) >> 5);
      long long grid = tiles;
      const long long cap = static_cast<long long>(d.sm_count) * 32;
      if (grid > cap) grid = cap;
      prep_b_kernel<MODE><<<static_cast<unsigned>(grid), dim3(32, 8), 0, st>>>(B, ldb, b_hi, b_lo, static_cast<int>(K),
                                                                                 static_cast<int>(N), static_cast<int>(kp));
      rc = launch_check("prep_b_kernel");
      if (rc) return rc;
    }
    const int b_box_rows = pair ? tile_n / 2 : GEMM_BN;
    if ((rc = encode_panel_map(&ma_hi, a_hi, kp, M, GEMM_BM))) return rc;
    if ((rc = encode_panel_map(&mb_hi, b_hi, kp, N, b_box_rows))) return rc;
    if ((rc = encode_panel_map(&ma_lo, a_lo, kp, M, GEMM_BM))) return rc;
    if ((rc = encode_panel_map(&mb_lo, b_lo, kp, N, b_box_rows))) return rc;
  }

  GemmParams gp = gp_in;
  gp.num_k_blocks = static_cast<int>(kp / GEMM_BK);
  gp.status = d.status;
  d.status_armed.store(true);
  gp.epoch_ctr = epoch_ring;
  derive_params(&gp);
  if (prof) CU_TRY(cudaEventRecord(rec.e1, st));
  if (pair) {
    const int dev_index = static_cast<int>(&d - g_dev);
    rc = direct ? launch_pair_bn<MODE, true>(tile_n, d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N)
                : launch_pair_bn<MODE, false>(tile_n, d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N);
  } else {
    gp.tiles_m = static_cast<int>((M + GEMM_BM - 1) / GEMM_BM);
    gp.tiles_n = static_cast<int>((N + GEMM_BN - 1) / GEMM_BN);
    const long long tiles = static_cast<long long>(gp.tiles_m) * gp.tiles_n;
    const unsigned grid = static_cast<unsigned>(tiles < d.sm_count ? tiles : d.sm_count);
    static std::atomic<int> attr_set[kMaxDevices];  // the shared-memory attribute is per device: set once on each
    const int dev_index = static_cast<int>(&d - g_dev);
    if (!attr_set[dev_index].load()) {
      CU_TRY(cudaFuncSetAttribute(gemm_tf32_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(Cfg::kSmemBytes)));
      attr_set[dev_index].store(1);
    }
    gemm_tf32_kernel<MODE><<<grid, GEMM_THREADS, Cfg::kSmemBytes, st>>>(ma_hi, mb_hi, ma_lo, mb_lo, gp);
    rc = launch_check("gemm_tf32_kernel");
  }
  if (prof) {
    CU_TRY(cudaEventRecord(rec.e2, st));
    std::lock_guard<std::mutex> lock(d.mu);
    d.prof.push_back(rec);
  }
  if (track_scratch && rc == SB200_OK) {
    std::lock_guard<std::mutex> lock(d.mu);
    if (!d.ws_event) CU_TRY(cudaEventCreateWithFlags(&d.ws_event, cudaEventDisableTiming));
    CU_TRY(cudaEventRecord(d.ws_event, st));
    d.ws_last_stream = st;
    d.ws_in_use = true;
  }
  return rc;
}

// ---- mode 4: the three-term split on fp16 panels -------------------------------------------------------
int encode_map_f16(CUtensorMap* map, const __half* base, long long kp, long long rows, int box_rows) {
  if (int rc = resolve_encode_tiled()) return rc;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(kp), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(kp) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SB200_ERR_INVALID_VALUE, "cuTensorMapEncodeTiled (fp16 panel) failed with CUresult %d (kp=%lld rows=%lld)", (int)r, kp, rows);
  return SB200_OK;
}

size_t gemm_f16_workspace_need(long long M, long long N, long long K, bool three) {
  const long long kp = round_up(K, 64);
  return 2 * round_up(N * 4, 1024) + round_up(M * 4, 1024) +
         (three ? 2 : 1) * (round_up(M * kp * 2, 1024) + round_up(N * kp * 2, 1024));
}

// THREE: hi and lo panels, three MMAs per k-step (SB200_MODE_3XF16); else hi panels only, one MMA (SB200_MODE_F16).
template <bool THREE>
int launch_gemm_f16(DeviceState& d, cudaStream_t st, long long M, long long N, long long K, const float* A, long long lda,
                    const float* B, long long ldb, const GemmParams& gp_in) {
  const long long kp = round_up(K, 64);
  const size_t a_bytes = round_up(M * kp * 2, 1024), b_bytes = round_up(N * kp * 2, 1024);
  const size_t need = gemm_f16_workspace_need(M, N, K, THREE);
  std::unique_lock<std::mutex> scratch_lock(d.scratch_mu);
  int rc = ensure_workspace(d, need);
  if (rc) return rc;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
    cudaGetLastError();
    cap = cudaStreamCaptureStatusActive;
  }
  const bool track_scratch = cap == cudaStreamCaptureStatusNone;
  if (track_scratch) {
    std::lock_guard<std::mutex> lock(d.mu);
    if (d.ws_in_use && d.ws_last_stream != st) CU_TRY(cudaStreamWaitEvent(st, d.ws_event, 0));
  }
  unsigned int* epoch_ring = next_epoch_ring(d, st, kp / 64);
  const bool prof = g_profiling.load() != 0;
  DeviceState::ProfRec rec{nullptr, nullptr, nullptr};
  if (prof) {
    CU_TRY(cudaEventCreate(&rec.e0));
    CU_TRY(cudaEventCreate(&rec.e1));
    CU_TRY(cudaEventCreate(&rec.e2));
    CU_TRY(cudaEventRecord(rec.e0, st));
  }
  // scratch: [column maxima of B, N words][1/scale per column, N floats][1/scale per row of A, M floats]
  //          [A_hi][B_hi]([A_lo][B_lo]), every part rounded up to 1 KiB
  uint8_t* ws = static_cast<uint8_t*>(d.workspace);
  const size_t col_bytes = round_up(N * 4, 1024), row_bytes = round_up(M * 4, 1024);
  unsigned int* col_bits = reinterpret_cast<unsigned int*>(ws);
  float* col_scale = reinterpret_cast<float*>(ws + col_bytes);
  float* row_scale = reinterpret_cast<float*>(ws + 2 * col_bytes);
  uint8_t* panels = ws + 2 * col_bytes + row_bytes;
  __half* a_hi = reinterpret_cast<__half*>(panels);
  __half* b_hi = reinterpret_cast<__half*>(panels + a_bytes);
  __half* a_lo = THREE ? reinterpret_cast<__half*>(panels + a_bytes + b_bytes) : nullptr;
  __half* b_lo = THREE ? reinterpret_cast<__half*>(panels + 2 * a_bytes + b_bytes) : nullptr;
  CU_TRY(cudaMemsetAsync(col_bits, 0, static_cast<size_t>(N) * 4, st));
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  {
    // A: one warp per row finds the row's scale and writes its panels
    long long grid = (M + 7) / 8;
    const long long cap = static_cast<long long>(d.sm_count) * 8;  // fewer rows in flight (to keep them in L2) measured slower
    if (grid > cap) grid = cap;
    const int vec_ok = (al16(A) && (lda & 3) == 0) ? 1 : 0;
    prep_a_f16_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(A, lda, a_hi, a_lo, row_scale, static_cast<int>(M),
                                                                    static_cast<int>(K), static_cast<int>(kp), vec_ok);
    if ((rc = launch_check("prep_a_f16_kernel"))) return rc;
    // B: column maxima, then the transposing split
    const int rows_per_block = 64;
    const bool vec_b = al16(B) && (ldb & 3) == 0 && (N & 3) == 0;
    const long long cols_per_block = vec_b ? 1024 : 256;
    const dim3 cgrid(static_cast<unsigned>((N + cols_per_block - 1) / cols_per_block),
                     static_cast<unsigned>((K + rows_per_block - 1) / rows_per_block));
    if (cgrid.y > 65535u) return fail(SB200_ERR_TOO_LARGE, "K beyond the fp16 modes' column scan (K=%lld)", K);
    if (vec_b)
      colmax_kernel<true><<<cgrid, 256, 0, st>>>(B, ldb, static_cast<int>(K), static_cast<int>(N), rows_per_block, col_bits);
    else
      colmax_kernel<false><<<cgrid, 256, 0, st>>>(B, ldb, static_cast<int>(K), static_cast<int>(N), rows_per_block, col_bits);
    if ((rc = launch_check("colmax_kernel"))) return rc;
    long long tiles = (kp >> 6) * ((N + 31) >> 5);
    const long long cap32 = static_cast<long long>(d.sm_count) * 32;
    if (tiles > cap32) tiles = cap32;
    prep_b_f16_kernel<<<static_cast<unsigned>(tiles), dim3(32, 8), 0, st>>>(B, ldb, b_hi, b_lo, col_scale, col_bits,
                                                                             static_cast<int>(K), static_cast<int>(N),
                                                                             static_cast<int>(kp));
    if ((rc = launch_check("prep_b_f16_kernel"))) return rc;
  }
  const int clusters = d.sm_count / 2 > 0 ? d.sm_count / 2 : 1;
  const int tile_n = choose_tile_n(M, N, kp / 64, clusters, THREE ? 3 : 1);
  CUtensorMap ma_hi, mb_hi, ma_lo, mb_lo;
  if ((rc = encode_map_f16(&ma_hi, a_hi, kp, M, GEMM_BM))) return rc;
  if ((rc = encode_map_f16(&mb_hi, b_hi, kp, N, tile_n / 2))) return rc;
  ma_lo = ma_hi;
  mb_lo = mb_hi;
  if (THREE) {
    if ((rc = encode_map_f16(&ma_lo, a_lo, kp, M, GEMM_BM))) return rc;
    if ((rc = encode_map_f16(&mb_lo, b_lo, kp, N, tile_n / 2))) return rc;
  }
  GemmParams gp = gp_in;
  gp.num_k_blocks = static_cast<int>(kp / 64);
  gp.status = d.status;
  d.status_armed.store(true);
  gp.epoch_ctr = epoch_ring;
  derive_params(&gp);
  gp.row_scale = row_scale;
  gp.col_scale = col_scale;
  if (prof) CU_TRY(cudaEventRecord(rec.e1, st));
  const int dev_index = static_cast<int>(&d - g_dev);
  rc = THREE ? launch_pair_bn<4, false>(tile_n, d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N)
             : launch_pair_bn<2, false>(tile_n, d, dev_index, st, ma_hi, mb_hi, ma_lo, mb_lo, gp, M, N);
  if (prof) {
    CU_TRY(cudaEventRecord(rec.e2, st));
    std::lock_guard<std::mutex> lock(d.mu);
    d.prof.push_back(rec);
  }
  if (track_scratch && rc == SB200_OK) {
    std::lock_guard<std::mutex> lock(d.mu);
    if (!d.ws_event) CU_TRY(cudaEventCreateWithFlags(&d.ws_event, cudaEventDisableTiming));
    CU_TRY(cudaEventRecord(d.ws_event, st));
    d.ws_last_stream = st;
    d.ws_in_use = true;
  }
  return rc;
}

// ---- mode 5: main term on the TF32 pipe, cross terms on the fp16 pipe ---------------------------------------
// Products below this many multiply-adds, operands TMA cannot address, and problems the pair kernel does not serve
// go to plain 3xTF32: the mixed mode costs five more launches (magnitudes, two panel passes, two gated fallbacks).
constexpr long long kMixMinMacs = 1ll << 34;  // measured: 1.12x at 4096^3 (2^36), 0.96x at 2048^3 (2^33)
std::atomic<long long> g_mix_min_macs{0};    // 0 = the default above

bool operands_addressable(const float* A, long long lda, const float* B, long long ldb) {
  return (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 3) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0 && (ldb & 3) == 0;
}

bool gemm_mix_applies(long long M, long long N, long long K, bool addressable) {
  const long long set = g_mix_min_macs.load(), least = set > 0 ? set : kMixMinMacs;
  return addressable && M > GEMM_BM && K >= 64 && M * N * K >= least && gemm_variant_setting() == 0;
}

size_t gemm_mix_workspace_need(long long M, long long N, long long K) {
  const long long kp64 = round_up(K, 64), kp32 = round_up(K, GEMM_BK);
  const size_t mixed = 2 * (round_up(M * kp64 * 2, 1024) + round_up(N * kp64 * 2, 1024));
  const size_t plain = round_up(K * round_up(N, 32) * 4, 1024) + round_up(M * kp32 * 4, 1024);
  return mixed > plain ? mixed : plain;  // one or the other runs: the two layouts share the scratch
}

int launch_gemm_mix(DeviceState& d, cudaStream_t st, long long M, long long N, long long K, const float* A, long long lda,
                    const float* B, long long ldb, const GemmParams& gp_in) {
  const long long kp = round_up(K, 64), kp32 = round_up(K, GEMM_BK), np = round_up(N, 32);
  const size_t a_bytes = round_up(M * kp * 2, 1024), b_bytes = round_up(N * kp * 2, 1024);
  std::unique_lock<std::mutex> scratch_lock(d.scratch_mu);
  int rc = ensure_workspace(d, gemm_mix_workspace_need(M, N, K));
  if (rc) return rc;
  if (!d.mix_ctl) CU_TRY(cudaMalloc(&d.mix_ctl, sizeof(MixCtl)));
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
    cudaGetLastError();
    cap = cudaStreamCaptureStatusActive;
  }
  const bool track_scratch = cap == cudaStreamCaptureStatusNone;
  if (track_scratch) {
    std::lock_guard<std::mutex> lock(d.mu);
    if (d.ws_in_use && d.ws_last_stream != st) CU_TRY(cudaStreamWaitEvent(st, d.ws_event, 0));
  }
  unsigned int* epoch_ring = next_epoch_ring(d, st, 2 * (kp / 64) + 4);
  const bool prof = g_profiling.load() != 0;
  DeviceState::ProfRec rec{nullptr, nullptr, nullptr};
  if (prof) {
    CU_TRY(cudaEventCreate(&rec.e0));
    CU_TRY(cudaEventCreate(&rec.e1));
    CU_TRY(cudaEventCreate(&rec.e2));
    CU_TRY(cudaEventRecord(rec.e0, st));
  }
  uint8_t* ws = static_cast<uint8_t*>(d.workspace);
  __half* a_hi = reinterpret_cast<__half*>(ws);
  __half* b_hi = reinterpret_cast<__half*>(ws + a_bytes);
  __half* a_lo = reinterpret_cast<__half*>(ws + a_bytes + b_bytes);
  __half* b_lo = reinterpret_cast<__half*>(ws + 2 * a_bytes + b_bytes);
  CU_TRY(cudaMemsetAsync(d.mix_ctl, 0, sizeof(MixCtl), st));
  const long long cap16 = static_cast<long long>(d.sm_count) * 16;
  {
    // largest magnitudes of both matrices, one launch: a warp per row
    long long grid_a = (M + 7) / 8, grid_b = (K + 7) / 8;
    const long long cap8 = static_cast<long long>(d.sm_count) * 8;
    if (grid_a > cap8) grid_a = cap8;
    if (grid_b > cap8) grid_b = cap8;
    const AbsMaxJob ja{A, lda, static_cast<int>(M), static_cast<int>(K), 1};
    const AbsMaxJob jb{B, ldb, static_cast<int>(K), static_cast<int>(N), 1};
    absmax_two_kernel<<<static_cast<unsigned>(grid_a + grid_b), 256, 0, st>>>(ja, jb, static_cast<int>(grid_a), d.mix_ctl);
    if ((rc = launch_check("absmax_two_kernel"))) return rc;
    long long grid = (M * (kp >> 3) + 255) / 256;
    if (grid > cap16) grid = cap16;
    prep_mix_a_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(A, lda, a_hi, a_lo, static_cast<int>(M), static_cast<int>(K),
                                                                    static_cast<int>(kp), 1, d.mix_ctl);
    if ((rc = launch_check("prep_mix_a_kernel"))) return rc;
    long long tiles = (kp >> 6) * ((N + 31) >> 5);
    const long long cap32 = static_cast<long long>(d.sm_count) * 32;
    if (tiles > cap32) tiles = cap32;
    prep_mix_b_kernel<<<static_cast<unsigned>(tiles), dim3(32, 8), 0, st>>>(B, ldb, b_hi, b_lo, static_cast<int>(K),
                                                                             static_cast<int>(N), static_cast<int>(kp), d.mix_ctl);
    if ((rc = launch_check("prep_mix_b_kernel"))) return rc;
  }
  const int clusters = d.sm_count / 2 > 0 ? d.sm_count / 2 : 1;
  const int tile_n = choose_tile_n(M, N, kp32 / GEMM_BK, clusters, 3);
  CUtensorMap ma, mb, ma_hi16, mb_hi16, ma_lo16, mb_lo16;
  if ((rc = encode_map_2d(&ma, A, K, M, lda, GEMM_BK, GEMM_BM, true))) return rc;
  if ((rc = encode_map_2d(&mb, B, N, K, ldb, 32, GEMM_BK, true, true))) return rc;
  if ((rc = encode_map_f16(&ma_hi16, a_hi, kp, M, GEMM_BM))) return rc;
  if ((rc = encode_map_f16(&mb_hi16, b_hi, kp, N, tile_n / 2))) return rc;
  if ((rc = encode_map_f16(&ma_lo16, a_lo, kp, M, GEMM_BM))) return rc;
  if ((rc = encode_map_f16(&mb_lo16, b_lo, kp, N, tile_n / 2))) return rc;
  GemmParams gp = gp_in;
  gp.status = d.status;
  d.status_armed.store(true);
  gp.epoch_ctr = epoch_ring;
  derive_params(&gp);
  gp.mix_ctl = reinterpret_cast<const int*>(d.mix_ctl);
  gp.gate = &d.mix_ctl->ok;
  if (prof) CU_TRY(cudaEventRecord(rec.e1, st));
  const int dev_index = static_cast<int>(&d - g_dev);
  gp.num_k_blocks = static_cast<int>(kp / 64);
  gp.gate_value = 1;
  rc = launch_pair_bn<5, true>(tile_n, d, dev_index, st, ma, mb, ma_hi16, mb_hi16, gp, M, N, &ma_lo16, &mb_lo16);
  if (rc == SB200_OK) {
    // behind it, gated the other way: plain 3xTF32 on the same operands, its low-part panels in the same scratch
    float* pb_lo = reinterpret_cast<float*>(ws);
    float* pa_lo = reinterpret_cast<float*>(ws + round_up(K * np * 4, 1024));
    long long grid_a = (M * (kp32 >> 2) + 255) / 256, grid_b = (K * (np >> 2) + 255) / 256;
    if (grid_a > cap16) grid_a = cap16;
    if (grid_b > cap16) grid_b = cap16;
    const PrepLoJob ja{A, lda, pa_lo, static_cast<int>(M), static_cast<int>(K), static_cast<int>(kp32)};
    const PrepLoJob jb{B, ldb, pb_lo, static_cast<int>(K), static_cast<int>(N), static_cast<int>(np)};
    prep_lo_two_kernel<<<static_cast<unsigned>(grid_a + grid_b), 256, 0, st>>>(ja, jb, static_cast<int>(grid_a), gp.gate);
    if ((rc = launch_check("prep_lo_two_kernel(gated)"))) return rc;
    CUtensorMap pma_lo, pmb_lo;
    if ((rc = encode_map_2d(&pma_lo, pa_lo, kp32, M, kp32, GEMM_BK, GEMM_BM, false))) return rc;
    if ((rc = encode_map_2d(&pmb_lo, pb_lo, N, K, np, 32, GEMM_BK, false, true))) return rc;
    gp.num_k_blocks = static_cast<int>(kp32 / GEMM_BK);
    gp.gate_value = 0;
    gp.epoch_ctr = nullptr;  // the ring belongs to the launch in front
    rc = launch_pair_bn<3, true>(tile_n, d, dev_index, st, ma, mb, pma_lo, pmb_lo, gp, M, N);
  }
  if (prof) {
    CU_TRY(cudaEventRecord(rec.e2, st));
    std::lock_guard<std::mutex> lock(d.mu);
    d.prof.push_back(rec);
  }
  if (track_scratch && rc == SB200_OK) {
    std::lock_guard<std::mutex> lock(d.mu);
    if (!d.ws_event) CU_TRY(cudaEventCreateWithFlags(&d.ws_event, cudaEventDisableTiming));
    CU_TRY(cudaEventRecord(d.ws_event, st));
    d.ws_last_stream = st;
    d.ws_in_use = true;
  }
  return rc;
}

int run_gemm(DeviceState& d, cudaStream_t st, int mode, long long M, long long N, long long K, uint64_t A, long long lda,
             uint64_t B, long long ldb, uint64_t D, long long ldd, float alpha, uint64_t C, long long ldc, float beta,
             uint64_t bias, int act, const uint64_t* replicas = nullptr, int n_replicas = 0) {
  if (!sb200::valid_mode(mode))
    return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (M < 0 || N < 0 || K < 0) return fail(SB200_ERR_INVALID_VALUE, "negative GEMM dimension (M=%lld N=%lld K=%lld)", M, N, K);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL - 64)
    return fail(SB200_ERR_TOO_LARGE, "GEMM dimension beyond 2^31-1 (M=%lld N=%lld K=%lld)", M, N, K);
  if (act != SB200_ACT_NONE && act != SB200_ACT_RELU) return fail(SB200_ERR_INVALID_VALUE, "unknown activation %d", act);
  if (M == 0 || N == 0) return SB200_OK;
  if (!D || (K > 0 && (!A || !B))) return fail(SB200_ERR_INVALID_VALUE, "null device pointer passed to GEMM");
  if ((K > 0 && lda < K) || (K > 0 && ldb < N) || ldd < N || (C && ldc < N))
    return fail(SB200_ERR_INVALID_VALUE, "leading dimension smaller than the row length (lda=%lld ldb=%lld ldc=%lld ldd=%lld)",
                lda, ldb, ldc, ldd);
  if ((A | B | C | D | bias) & 3) return fail(SB200_ERR_ALIGNMENT, "float32 matrices must be 4-byte aligned");
  {
    auto extent = [](long long rows, long long cols, long long ld) {
      return static_cast<uint64_t>((rows - 1) * ld + cols) * 4;
    };
    int rc = SB200_OK;
    if (K > 0 && ((rc = check_extent(d, A, extent(M, K, lda), "GEMM operand A")) || (rc = check_extent(d, B, extent(K, N, ldb), "GEMM operand B"))))
      return rc;
    if ((rc = check_extent(d, D, extent(M, N, ldd), "GEMM result D")) || (rc = check_extent(d, C, extent(M, N, ldc), "GEMM operand C")) ||
        (rc = check_extent(d, bias, static_cast<uint64_t>(N) * 4, "GEMM bias")))
      return rc;
    for (int r = 0; r < n_replicas; ++r)
      if ((rc = check_extent(d, replicas[r], 0, "replica"))) return rc;
  }
  GemmParams gp;
  memset(&gp, 0, sizeof gp);
  gp.M = static_cast<int>(M);
  gp.N = static_cast<int>(N);
  gp.D = as_ptr<float>(D);
  gp.ldd = ldd;
  gp.C = as_ptr<const float>(C);
  gp.ldc = ldc;
  gp.bias = as_ptr<const float>(bias);
  gp.alpha = alpha;
  gp.beta = beta;
  gp.act = act;
  gp.n_replicas = n_replicas;
  for (int r = 0; r < n_replicas; ++r) gp.replicas[r] = as_ptr<float>(replicas[r]);
  if (K == 0) {
    const long long total = M * N;
    long long grid = (total + 255) / 256;
    const long long cap = static_cast<long long>(d.sm_count) * 16;
    if (grid > cap) grid = cap;
    gemm_k0_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(gp);
    return launch_check("gemm_k0_kernel");
  }
  if (mode == SB200_MODE_3XF16)
    return launch_gemm_f16<true>(d, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  if (mode == SB200_MODE_F16)
    return launch_gemm_f16<false>(d, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  if (mode == SB200_MODE_3XMIXED && gemm_mix_applies(M, N, K, operands_addressable(as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb)))
    return launch_gemm_mix(d, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  if (mode == SB200_MODE_3XTF32 || mode == SB200_MODE_3XMIXED)
    return launch_gemm_mode<3>(d, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  return launch_gemm_mode<1>(d, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
}

// ---------------------------------------------------------- kernel objects
struct KernelObj {
  int dev;
  KernelPlan plan;
  std::string cubin;          // generic maps: compiled at sb200_kernel_compile (needs no GPU)
  JitModule jit[kMaxDevices]; // loaded on first launch per device
  std::mutex mu;
};
std::mutex g_kernels_mu;
std::unordered_set<KernelObj*> g_kernels;

KernelObj* find_kernel(uint64_t h) {
  KernelObj* k = reinterpret_cast<KernelObj*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lock(g_kernels_mu);
  return g_kernels.count(k) ? k : nullptr;
}

struct Slot {
  bool is_vec = false;
  uint64_t ptr = 0;
  const void* host = nullptr;  // launch-from-host: the device buffer is to be filled from here first
  void* host_out = nullptr;    // launch-from-host: where the caller keeps the host copy (result brought back behind the kernel)
  int arg = -1;                // position of the buffer in the caller's argument list
  long long len = 0;
  double f = 0.0;
  long long i = 0;
};

int bind_args(const KernelPlan& plan, const sb200_arg* args, int nargs, std::vector<Slot>* slots,
              const void* const* host_ptrs = nullptr, void* const* host_out = nullptr) {
  slots->assign(plan.params.size(), Slot());
  int a = 0;
  for (size_t p = 0; p < plan.params.size(); ++p) {
    const ParamInfo& pi = plan.params[p];
    Slot& s = (*slots)[p];
    if (pi.is_vec) {
      if (a + 1 >= nargs || args[a].tag != SB200_ARG_BUFFER || args[a + 1].tag != SB200_ARG_I32)
        return fail(SB200_ERR_ARGS, "kernel '%s': parameter %zu (%s) expects a buffer followed by its int32 length",
                    plan.name.c_str(), p, pi.name.c_str());
      s.is_vec = true;
      s.ptr = args[a].v.buffer;
      s.host = host_ptrs ? host_ptrs[a] : nullptr;
      s.host_out = host_out ? host_out[a] : nullptr;
      s.arg = a;
      s.len = args[a + 1].v.i32;
      if (s.len < 0) return fail(SB200_ERR_ARGS, "kernel '%s': negative length for vector %s", plan.name.c_str(), pi.name.c_str());
      a += 2;
    } else {
      if (a >= nargs) return fail(SB200_ERR_ARGS, "kernel '%s': too few arguments (%d)", plan.name.c_str(), nargs);
      const sb200_arg& x = args[a++];
      const bool is_float = pi.elt == "f32" || pi.elt == "f64";
      switch (x.tag) {
        case SB200_ARG_I32: s.i = x.v.i32; s.f = static_cast<double>(x.v.i32); break;
        case SB200_ARG_I64: s.i = x.v.i64; s.f = static_cast<double>(x.v.i64); break;
        case SB200_ARG_F32: s.f = x.v.f32; s.i = static_cast<long long>(x.v.f32); break;
        case SB200_ARG_F64: s.f = x.v.f64; s.i = static_cast<long long>(x.v.f64); break;
        default:
          return fail(SB200_ERR_ARGS, "kernel '%s': scalar parameter %s received a buffer", plan.name.c_str(), pi.name.c_str());
      }
      if (is_float != (x.tag == SB200_ARG_F32 || x.tag == SB200_ARG_F64))
        return fail(SB200_ERR_ARGS, "kernel '%s': scalar parameter %s has type %s but the argument tag is %d", plan.name.c_str(),
                    pi.name.c_str(), pi.elt.c_str(), x.tag);
    }
  }
  if (a != nargs) return fail(SB200_ERR_ARGS, "kernel '%s': %d arguments passed, %d consumed", plan.name.c_str(), nargs, a);
  return SB200_OK;
}

float coef_value(const Coef& c, const std::vector<Slot>& slots) {
  return static_cast<float>(c.param >= 0 ? slots[c.param].f : c.value);
}

int launch_generic_map(DeviceState& d, KernelObj& k, const std::vector<Slot>& s, long long n, cudaStream_t st) {
  const GenericMap& gm = k.plan.generic;
  JitModule* jm = &k.jit[k.dev];
  {
    std::lock_guard<std::mutex> lock(k.mu);
    if (!jm->module) {
      std::string err;
      int rc = jit_load(k.cubin, false, jm, &err);
      if (rc) return fail(rc, "kernel '%s': %s", k.plan.name.c_str(), err.c_str());
    }
  }
  if (n <= 0) return SB200_OK;
  const size_t ni = gm.inputs.size(), no = gm.outputs.size(), ns = gm.scalars.size();
  std::vector<uint64_t> ptrs;
  for (int p : gm.inputs) ptrs.push_back(s[p].ptr);
  for (int p : gm.outputs) ptrs.push_back(s[p].ptr);
  uintptr_t mis = ptrs[0] & 15;
  bool same = (mis & 3) == 0;
  for (uint64_t p : ptrs) {
    if (!p) return fail(SB200_ERR_INVALID_VALUE, "kernel '%s': null device pointer", k.plan.name.c_str());
    if (p & 3) return fail(SB200_ERR_ALIGNMENT, "float32 vectors must be 4-byte aligned");
    if ((p & 15) != mis) same = false;
  }
  long long head = 0, nvec = 0;
  if (same) {
    head = mis ? static_cast<long long>((16 - mis) >> 2) : 0;
    if (head > n) head = n;
    nvec = (n - head) >> 2;
  }
  std::vector<double> sd(ns);
  std::vector<long long> si(ns);
  auto scalar_arg = [&](size_t i) -> void* {
    const std::string& elt = k.plan.params[gm.scalars[i]].elt;
    if (elt == "f32" || elt == "f64") {
      sd[i] = s[gm.scalars[i]].f;
      return &sd[i];
    }
    si[i] = s[gm.scalars[i]].i;
    return &si[i];
  };
  std::string err;
  auto run_scalar = [&](long long first, long long last) -> int {
    std::vector<void*> args;
    for (size_t i = 0; i < ni + no; ++i) args.push_back(&ptrs[i]);
    for (size_t i = 0; i < ns; ++i) args.push_back(scalar_arg(i));
    args.push_back(&first);
    args.push_back(&last);
    long long grid = (last - first + 255) / 256;
    const long long cap = static_cast<long long>(d.sm_count) * 16;
    if (grid > cap) grid = cap;
    int rc = jit_launch(jm->scalar_fn, static_cast<unsigned>(grid), 256, st, args.data(), &err);
    if (rc) return fail(rc, "kernel '%s': %s", k.plan.name.c_str(), err.c_str());
    count_launch();
    return SB200_OK;
  };
  if (nvec > 0) {
    // one launch: the vector kernel takes the ragged ends in block 0
    int head_i = static_cast<int>(head);
    std::vector<void*> args;
    for (size_t i = 0; i < ni + no; ++i) args.push_back(&ptrs[i]);
    for (size_t i = 0; i < ns; ++i) args.push_back(scalar_arg(i));
    args.push_back(&head_i);
    args.push_back(&nvec);
    args.push_back(&n);
    long long grid = (nvec + 255) / 256;
    const long long cap = static_cast<long long>(d.sm_count) * 8;
    if (grid > cap) grid = cap;
    int rc = jit_launch(jm->vec_fn, static_cast<unsigned>(grid), 256, st, args.data(), &err);
    if (rc) return fail(rc, "kernel '%s': %s", k.plan.name.c_str(), err.c_str());
    count_launch();
    return SB200_OK;
  }
  return run_scalar(0, n);
}

// out[b] = sum of f(inputs[gid]) over block b's elements, for the b < grid.x blocks of the reference launch
int launch_block_reduce(DeviceState& d, KernelObj& k, const std::vector<Slot>& s, const uint32_t grid[3], const uint32_t block[3],
                        cudaStream_t st) {
  const KernelPlan& plan = k.plan;
  const GenericMap& gm = plan.generic;
  if (static_cast<int>(block[0]) != plan.reduce.block || block[1] != 1 || block[2] != 1)
    return fail(SB200_ERR_ARGS, "kernel '%s': block is %ux%ux%u but the kernel reduces blocks of %d threads", plan.name.c_str(),
                block[0], block[1], block[2], plan.reduce.block);
  long long n = s[plan.reduce.n_param].i;
  if (n < 0) n = 0;
  long long nseg = grid[0];
  const long long covered = std::min<long long>(n, nseg * plan.reduce.block);
  for (int p : gm.inputs)
    if (s[p].len < covered)
      return fail(SB200_ERR_BOUNDS, "kernel '%s': launch reads %lld elements but vector %s holds %lld", plan.name.c_str(), covered,
                  plan.params[p].name.c_str(), s[p].len);
  const int out = gm.outputs[0];
  if (s[out].len < nseg)
    return fail(SB200_ERR_BOUNDS, "kernel '%s': %lld blocks but vector %s holds %lld", plan.name.c_str(), nseg,
                plan.params[out].name.c_str(), s[out].len);
  JitModule* jm = &k.jit[k.dev];
  {
    std::lock_guard<std::mutex> lock(k.mu);
    if (!jm->module) {
      std::string err;
      int rc = jit_load(k.cubin, true, jm, &err);
      if (rc) return fail(rc, "kernel '%s': %s", plan.name.c_str(), err.c_str());
    }
  }
  std::vector<uint64_t> ptrs;
  for (int p : gm.inputs) ptrs.push_back(s[p].ptr);
  ptrs.push_back(s[out].ptr);
  for (uint64_t p : ptrs)
    if (!p || (p & 3)) return fail(SB200_ERR_INVALID_VALUE, "kernel '%s': null or misaligned device pointer", plan.name.c_str());
  const size_t ns = gm.scalars.size();
  std::vector<double> sd(ns);
  std::vector<long long> si(ns);
  std::vector<void*> args;
  for (auto& p : ptrs) args.push_back(&p);
  for (size_t i = 0; i < ns; ++i) {
    const std::string& elt = plan.params[gm.scalars[i]].elt;
    if (elt == "f32" || elt == "f64") {
      sd[i] = s[gm.scalars[i]].f;
      args.push_back(&sd[i]);
    } else {
      si[i] = s[gm.scalars[i]].i;
      args.push_back(&si[i]);
    }
  }
  args.push_back(&n);
  args.push_back(&nseg);
  // one warp per segment, 8 warps per block
  long long blocks = (nseg + 7) / 8;
  const long long cap = static_cast<long long>(d.sm_count) * 16;
  if (blocks > cap) blocks = cap;
  std::string err;
  int rc = jit_launch(jm->reduce_fn, static_cast<unsigned>(blocks), 256, st, args.data(), &err);
  if (rc) return fail(rc, "kernel '%s': %s", plan.name.c_str(), err.c_str());
  count_launch();
  return SB200_OK;
}

int launch_map_kernel(DeviceState& d, KernelObj& kobj, const std::vector<Slot>& s, const uint32_t grid[3],
                      const uint32_t block[3], cudaStream_t st) {
  const KernelPlan& plan = kobj.plan;
  const MapPlan& m = plan.map;
  // which element indices the reference launch would touch
  long long covered = m.index_kind == IDX_GLOBAL ? static_cast<long long>(grid[0]) * block[0] : block[0];
  long long n = covered;
  if (m.n_param >= 0) {
    if (s[m.n_param].i < n) n = s[m.n_param].i;
    if (n < 0) n = 0;
  }
  std::vector<int> vecs = {m.out0, m.out1, m.in0, m.in1};
  if (m.op == OP_GENERIC) {
    vecs = plan.generic.inputs;
    vecs.insert(vecs.end(), plan.generic.outputs.begin(), plan.generic.outputs.end());
  }
  for (int v : vecs)
    if (v >= 0 && s[v].len < n)
      return fail(SB200_ERR_BOUNDS, "kernel '%s': launch covers %lld elements but vector %s holds %lld", plan.name.c_str(), n,
                  plan.params[v].name.c_str(), s[v].len);
  if (m.op == OP_GENERIC) return launch_generic_map(d, kobj, s, n, st);
  return run_map(d, st, m.op, s[m.out0].ptr, m.out1 >= 0 ? s[m.out1].ptr : 0, s[m.in0].ptr, s[m.in1].ptr,
                 coef_value(m.scalar, s), n);
}

int gemm_upload_pipeline(DeviceState& d, cudaStream_t st, int mode, long long M, long long N, long long K, const Slot& a,
                         const Slot& b, const Slot* c, const Slot* bias, const Slot& dd, float alpha, float beta, int act, void* d_host);

int ensure_pipe_streams(DeviceState& d) {
  std::lock_guard<std::mutex> lock(d.mu);  // callers on several host threads may get here at once
  if (!d.pipe_out) {
    if (!d.pipe_in) CU_TRY(cudaStreamCreateWithFlags(&d.pipe_in, cudaStreamNonBlocking));
    if (!d.pipe_compute) CU_TRY(cudaStreamCreateWithFlags(&d.pipe_compute, cudaStreamNonBlocking));
    CU_TRY(cudaStreamCreateWithFlags(&d.pipe_out, cudaStreamNonBlocking));  // last: its presence says all three exist
  }
  return SB200_OK;
}

// Copies `bytes` from the device to page-locked host memory on the outbound stream, behind what `st` holds so far.
int download_behind(DeviceState& d, cudaStream_t st, void* host, uint64_t dev_ptr, size_t bytes) {
  int rc = ensure_pipe_streams(d);
  if (rc) return rc;
  cudaEvent_t e = nullptr;
  CU_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  cudaError_t ce = cudaEventRecord(e, st);
  if (ce == cudaSuccess) ce = cudaStreamWaitEvent(d.pipe_out, e, 0);
  if (ce == cudaSuccess && bytes) ce = cudaMemcpyAsync(host, as_ptr<void>(dev_ptr), bytes, cudaMemcpyDeviceToHost, d.pipe_out);
  cudaEventDestroy(e);
  return ce == cudaSuccess ? SB200_OK : cuda_fail(ce, "download of a result behind its kernel");
}

// The element-wise operators by chunks: the inputs of a chunk come over on the inbound stream, the kernel of the chunk
// follows them on `st`, and the outputs of the chunk go back on the outbound stream to the page-locked arrays the caller
// named for them (out_host[0], out_host[1]; null: stay on the device).  Every element depends on its own index only, so
// the chunks compute what the one launch computes.  Vectors longer than the launch covers travel whole, as after
// Transfer.to_device.  Returns when every upload has completed.
int map_upload_pipeline(DeviceState& d, cudaStream_t st, const KernelPlan& plan, const std::vector<Slot>& s, long long n,
                        void* const out_host[2]) {
  std::lock_guard<std::mutex> host_call_lock(d.host_call_mu);
  int rc = ensure_pipe_streams(d);
  if (rc) return rc;
  const MapPlan& m = plan.map;
  std::vector<cudaEvent_t> events;
  auto done = [&](int r) {
    cudaStreamSynchronize(d.pipe_in);
    for (auto e : events) cudaEventDestroy(e);
    cudaGetLastError();
    return r;
  };
  auto order = [&](cudaStream_t from, cudaStream_t to) -> int {  // `to` continues behind what `from` holds so far
    cudaEvent_t e = nullptr;
    cudaError_t ce = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    if (ce == cudaSuccess) {
      events.push_back(e);
      ce = cudaEventRecord(e, from);
    }
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(to, e, 0);
    return ce == cudaSuccess ? SB200_OK : cuda_fail(ce, "ordering a chunk behind its upload");
  };
  if ((rc = order(st, d.pipe_in))) return done(rc);  // not before work that still uses these buffers on `st`
  const int vecs[4] = {m.in0, m.in1, m.out0, m.out1};
  auto seen_before = [&](int idx) {  // the same buffer bound to several parameters moves once
    for (int j = 0; j < idx; ++j)
      if (vecs[j] >= 0 && vecs[idx] >= 0 && s[vecs[j]].ptr == s[vecs[idx]].ptr) return true;
    return false;
  };
  auto upload = [&](const Slot& v, long long first, long long count) -> bool {
    if (!v.host || count <= 0) return true;
    return cudaMemcpyAsync(as_ptr<float>(v.ptr) + first, static_cast<const float*>(v.host) + first, static_cast<size_t>(count) * 4,
                           cudaMemcpyHostToDevice, d.pipe_in) == cudaSuccess;
  };
  // beyond the launch: whole tails of every vector; of the outputs also nothing below n (the kernel writes all of it)
  for (int j = 0; j < 4; ++j)
    if (vecs[j] >= 0 && !seen_before(j) && !upload(s[vecs[j]], n, s[vecs[j]].len - n))
      return done(cuda_fail(cudaGetLastError(), "upload of a vector's tail"));
  long long chunk = (n + 15) / 16;
  chunk = (chunk + 1023) / 1024 * 1024;  // keeps every chunk 16-byte aligned for the vector loads
  for (long long e0 = 0; e0 < n && !rc; e0 += chunk) {
    const long long cnt = std::min(chunk, n - e0);
    for (int j = 0; j < 2; ++j)  // inputs (an output that is also an input is one of them)
      if (vecs[j] >= 0 && !seen_before(j) && !upload(s[vecs[j]], e0, cnt))
        return done(cuda_fail(cudaGetLastError(), "upload of a chunk"));
    if ((rc = order(d.pipe_in, st))) break;
    const uint64_t off = static_cast<uint64_t>(e0) * 4;
    rc = run_map(d, st, m.op, s[m.out0].ptr + off, m.out1 >= 0 ? s[m.out1].ptr + off : 0, s[m.in0].ptr + off, s[m.in1].ptr + off,
                 coef_value(m.scalar, s), cnt);
    if (!rc && out_host[0]) rc = download_behind(d, st, static_cast<float*>(out_host[0]) + e0, s[m.out0].ptr + off, static_cast<size_t>(cnt) * 4);
    if (!rc && out_host[1] && m.out1 >= 0)
      rc = download_behind(d, st, static_cast<float*>(out_host[1]) + e0, s[m.out1].ptr + off, static_cast<size_t>(cnt) * 4);
  }
  for (int j = 0; j < 2 && !rc; ++j) {  // the outputs' tails complete the host copies
    const int v = j == 0 ? m.out0 : m.out1;
    if (v >= 0 && out_host[j] && s[v].len > n)
      rc = download_behind(d, st, static_cast<float*>(out_host[j]) + n, s[v].ptr + static_cast<uint64_t>(n) * 4,
                           static_cast<size_t>(s[v].len - n) * 4);
  }
  return done(rc);
}

// pipeline_uploads: some operands are still in (pinned) host memory; when the launch covers the whole product they are
// moved by row blocks with the GEMM of each block behind its rows.  *pipelined tells the caller whether that happened.
// d_host: page-locked host memory the result is to be brought back to behind the kernel (null: leave it on the device).
int launch_gemm_kernel(DeviceState& d, const KernelPlan& plan, const std::vector<Slot>& s, const uint32_t grid[3],
                       const uint32_t block[3], cudaStream_t st, bool pipeline_uploads = false, bool* pipelined = nullptr,
                       void* d_host = nullptr) {
  const GemmPlan& g = plan.gemm;
  const long long M = s[g.m].i, N = s[g.n].i, K = s[g.k].i;
  if (M < 0 || N < 0 || K < 0) return fail(SB200_ERR_ARGS, "kernel '%s': negative m, n or k", plan.name.c_str());
  auto need = [&](int v, long long elems) -> int {
    if (v >= 0 && s[v].len < elems)
      return fail(SB200_ERR_BOUNDS, "kernel '%s': vector %s holds %lld elements, the launch needs %lld", plan.name.c_str(),
                  plan.params[v].name.c_str(), s[v].len, elems);
    return SB200_OK;
  };
  int rc;
  if ((rc = need(g.a, M * K)) || (rc = need(g.b, K * N)) || (rc = need(g.d, M * N)) || (rc = need(g.c, M * N)) ||
      (rc = need(g.bias, N)))
    return rc;
  const float alpha = coef_value(g.alpha, s), beta = g.c >= 0 ? coef_value(g.beta, s) : 0.0f;
  const uint64_t A = s[g.a].ptr, B = s[g.b].ptr, D = s[g.d].ptr, C = g.c >= 0 ? s[g.c].ptr : 0,
                 bias = g.bias >= 0 ? s[g.bias].ptr : 0;
  const int mode = current_mode();
  if (plan.kind == KIND_GEMM_TILED) {
    if (static_cast<long long>(block[0]) != g.tile || static_cast<long long>(block[1]) != g.tile)
      return fail(SB200_ERR_ARGS, "kernel '%s': block is %ux%u but the kernel's tiles are %dx%d", plan.name.c_str(), block[0],
                  block[1], g.tile, g.tile);
    // the reference launch computes rows < gy*by and columns < gx*bx only
    long long Me = static_cast<long long>(grid[1]) * block[1], Ne = static_cast<long long>(grid[0]) * block[0];
    if (Me > M) Me = M;
    if (Ne > N) Ne = N;
    if (pipeline_uploads && Me == M && Ne == N && M > 0 && N > 0) {
      *pipelined = true;
      return gemm_upload_pipeline(d, st, mode, M, N, K, s[g.a], s[g.b], g.c >= 0 ? &s[g.c] : nullptr, g.bias >= 0 ? &s[g.bias] : nullptr,
                                  s[g.d], alpha, beta, g.act, d_host);
    }
    if (pipeline_uploads) return SB200_OK;  // partial launch: the caller uploads whole vectors and launches again
    rc = run_gemm(d, st, mode, Me, Ne, K, A, K, B, N, D, N, alpha, C, N, beta, bias, g.act);
    if (!rc && d_host) rc = download_behind(d, st, d_host, D, static_cast<size_t>(s[g.d].len) * 4);
    return rc;
  }
  // naive shape: thread tid computes element tid of the row-major result
  long long covered = static_cast<long long>(grid[0]) * block[0];
  if (covered > M * N) covered = M * N;
  if (N == 0) return d_host && !pipeline_uploads ? download_behind(d, st, d_host, D, static_cast<size_t>(s[g.d].len) * 4) : SB200_OK;
  if (pipeline_uploads && covered == M * N && M > 0) {
    *pipelined = true;
    return gemm_upload_pipeline(d, st, mode, M, N, K, s[g.a], s[g.b], g.c >= 0 ? &s[g.c] : nullptr, g.bias >= 0 ? &s[g.bias] : nullptr,
                                s[g.d], alpha, beta, g.act, d_host);
  }
  if (pipeline_uploads) return SB200_OK;  // partial launch: as above
  const long long full_rows = covered / N, rest = covered - full_rows * N;
  rc = run_gemm(d, st, mode, full_rows, N, K, A, K, B, N, D, N, alpha, C, N, beta, bias, g.act);
  if (!rc && rest != 0) {
    const uint64_t off_a = static_cast<uint64_t>(full_rows) * K * 4, off_d = static_cast<uint64_t>(full_rows) * N * 4;
    rc = run_gemm(d, st, mode, 1, rest, K, A + off_a, K, B, N, D + off_d, N, alpha, C ? C + off_d : 0, N, beta, bias, g.act);
  }
  if (!rc && d_host) rc = download_behind(d, st, d_host, D, static_cast<size_t>(s[g.d].len) * 4);
  return rc;
}

// Operands that still sit in pinned host memory are brought over by row blocks on the device's inbound stream while
// the GEMM of the blocks that have arrived runs on `st`: B and the bias first, then A and C in about eight row blocks
// (multiples of 256 rows so that block edges are tile edges).  Returns once every upload has completed — the caller's
// host arrays may then be changed — while the last GEMMs may still be running on `st`.  With d_host, each block of
// D follows its GEMM back to the host on the outbound stream (the caller waits for that stream before reading it).
int gemm_upload_pipeline(DeviceState& d, cudaStream_t st, int mode, long long M, long long N, long long K, const Slot& a,
                         const Slot& b, const Slot* c, const Slot* bias, const Slot& dd, float alpha, float beta, int act, void* d_host) {
  std::lock_guard<std::mutex> host_call_lock(d.host_call_mu);  // the inbound stream is shared with the host-operand calls
  int src = ensure_pipe_streams(d);
  if (src) return src;
  static const int nblocks = [] {  // row blocks per product (SAREK_B200_PIPE_BLOCKS, 2..64)
    const char* e = getenv("SAREK_B200_PIPE_BLOCKS");
    const int v = e ? atoi(e) : 0;
    return v >= 2 && v <= 64 ? v : 8;
  }();
  long long block_rows = (M + nblocks - 1) / nblocks;
  block_rows = (block_rows + 255) / 256 * 256;
  if (block_rows > M) block_rows = M;
  std::vector<cudaEvent_t> events;
  auto done = [&](int rc) {
    cudaStreamSynchronize(d.pipe_in);  // every upload has landed (or failed) before the host arrays are given back
    for (auto e : events) cudaEventDestroy(e);
    cudaGetLastError();
    return rc;
  };
  auto mark = [&]() -> int {  // `st` continues only after what the inbound stream has been given so far
    cudaEvent_t e = nullptr;
    cudaError_t ce = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    if (ce == cudaSuccess) {
      events.push_back(e);
      ce = cudaEventRecord(e, d.pipe_in);
    }
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(st, e, 0);
    return ce == cudaSuccess ? SB200_OK : cuda_fail(ce, "ordering a row block behind its upload");
  };
  // the inbound stream must not overtake work that still reads or writes these buffers on `st`
  {
    cudaEvent_t e = nullptr;
    CU_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    events.push_back(e);
    CU_TRY(cudaEventRecord(e, st));
    CU_TRY(cudaStreamWaitEvent(d.pipe_in, e, 0));
  }
  int rc = SB200_OK;
  const uint64_t D = dd.ptr;
  // what lies beyond the operands proper (vectors longer than the product needs) and the old contents of D's vector
  // travel too, so that every device buffer ends up equal to its host array as after Transfer.to_device; the kernel
  // overwrites the first M*N elements of D, which therefore need not be sent
  auto upload_from = [&](const Slot* v, long long first) -> bool {
    if (!v || !v->host || v->len <= first) return true;
    return cudaMemcpyAsync(as_ptr<float>(v->ptr) + first, static_cast<const float*>(v->host) + first,
                           static_cast<size_t>(v->len - first) * 4, cudaMemcpyHostToDevice, d.pipe_in) == cudaSuccess;
  };
  if (!upload_from(&a, M * K) || !upload_from(&b, K * N) || !upload_from(c, M * N) || !upload_from(bias, N) ||
      !upload_from(&dd, c && c->ptr == dd.ptr ? dd.len : M * N))
    return done(cuda_fail(cudaGetLastError(), "upload of a vector's tail"));
  if (b.host && K > 0)
    if (cudaMemcpyAsync(as_ptr<void>(b.ptr), b.host, static_cast<size_t>(K) * N * 4, cudaMemcpyHostToDevice, d.pipe_in) != cudaSuccess)
      return done(cuda_fail(cudaGetLastError(), "upload of B"));
  if (bias && bias->host)
    if (cudaMemcpyAsync(as_ptr<void>(bias->ptr), bias->host, static_cast<size_t>(N) * 4, cudaMemcpyHostToDevice, d.pipe_in) != cudaSuccess)
      return done(cuda_fail(cudaGetLastError(), "upload of the bias"));
  if ((rc = mark())) return done(rc);
  // The last block's GEMM and download cannot hide behind any upload, so the final stretch is cut finer: whole blocks
  // while more than one block remains, then half of what is left, a quarter, a quarter (multiples of 256 rows).
  std::vector<long long> cuts;  // first row of every block, then M
  {
    long long r = 0;
    while (M - r > block_rows) {
      cuts.push_back(r);
      r += block_rows;
    }
    static const bool taper = [] {
      const char* e = getenv("SAREK_B200_PIPE_TAPER");
      return !(e && e[0] == '0');
    }();
    for (int split = 0; split < 2 && taper && M - r >= 512; ++split) {
      cuts.push_back(r);
      r += ((M - r) / 2 + 255) / 256 * 256;
    }
    if (r < M) cuts.push_back(r);
    cuts.push_back(M);
  }
  for (size_t bi = 0; bi + 1 < cuts.size() && !rc; ++bi) {
    const long long r0 = cuts[bi], rows = cuts[bi + 1] - r0;
    if (a.host && K > 0 &&
        cudaMemcpyAsync(as_ptr<float>(a.ptr) + r0 * K, static_cast<const float*>(a.host) + r0 * K, static_cast<size_t>(rows) * K * 4,
                        cudaMemcpyHostToDevice, d.pipe_in) != cudaSuccess)
      return done(cuda_fail(cudaGetLastError(), "upload of a block of A"));
    if (c && c->host &&
        cudaMemcpyAsync(as_ptr<float>(c->ptr) + r0 * N, static_cast<const float*>(c->host) + r0 * N, static_cast<size_t>(rows) * N * 4,
                        cudaMemcpyHostToDevice, d.pipe_in) != cudaSuccess)
      return done(cuda_fail(cudaGetLastError(), "upload of a block of C"));
    if ((rc = mark())) break;
    rc = run_gemm(d, st, mode, rows, N, K, a.ptr + static_cast<uint64_t>(r0) * K * 4, K, b.ptr, N, D + static_cast<uint64_t>(r0) * N * 4, N,
                  alpha, c ? c->ptr + static_cast<uint64_t>(r0) * N * 4 : 0, N, beta, bias ? bias->ptr : 0, act);
    if (!rc && d_host)
      rc = download_behind(d, st, static_cast<float*>(d_host) + r0 * N, D + static_cast<uint64_t>(r0) * N * 4, static_cast<size_t>(rows) * N * 4);
  }
  // what D's vector holds beyond the product goes back too: the caller is told that the whole host copy is current
  if (!rc && d_host && dd.len > M * N)
    rc = download_behind(d, st, static_cast<float*>(d_host) + M * N, D + static_cast<uint64_t>(M) * N * 4, static_cast<size_t>(dd.len - M * N) * 4);
  return done(rc);
}

}  // namespace

namespace sb200 {
int set_error(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}
}  // namespace sb200

// =========================================================================
// C ABI
// =========================================================================
extern "C" {

int sb200_init(void) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(SB200_ERR_NO_DEVICE, "CUDA is not available: %s", cudaGetErrorString(e));
  }
  if (count == 0) return fail(SB200_ERR_NO_DEVICE, "no CUDA device");
  return SB200_OK;
}

int sb200_version(void) { return kVersion; }

const char* sb200_last_error_string(void) { return g_err.c_str(); }

int sb200_device_count(int* count) {
  if (!count) return fail(SB200_ERR_INVALID_VALUE, "null count pointer");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    return SB200_OK;  // no driver / no device: zero devices, like Cuda_api.is_available () = false
  }
  int usable = 0;
  for (int i = 0; i < n && i < kMaxDevices; ++i) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) usable = i + 1;
  }
  *count = usable;
  return SB200_OK;
}

int sb200_device_get_info(int dev, sb200_device_info* out) {
  if (!out) return fail(SB200_ERR_INVALID_VALUE, "null info pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  cudaDeviceProp p;
  CU_TRY(cudaGetDeviceProperties(&p, dev));
  memset(out, 0, sizeof *out);
  snprintf(out->name, sizeof out->name, "%s", p.name);
  out->total_mem = p.totalGlobalMem;
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->sm_count = p.multiProcessorCount;
  out->max_threads_per_block = p.maxThreadsPerBlock;
  out->max_shared_per_block = static_cast<int32_t>(p.sharedMemPerBlockOptin);
  out->warp_size = p.warpSize;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
  out->clock_khz = khz;
  out->l2_bytes = p.l2CacheSize;
  return SB200_OK;
}

int sb200_device_set_current(int dev) {
  DeviceState* d;
  return device_ready(dev, &d);
}

int sb200_device_synchronize(int dev) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  CU_TRY(cudaDeviceSynchronize());
  return check_status_word(*d, true);
}

int sb200_mem_alloc(int dev, uint64_t bytes, uint64_t* dptr) {
  if (!dptr) return fail(SB200_ERR_INVALID_VALUE, "null dptr pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  void* p = nullptr;
  CU_TRY(cudaMalloc(&p, bytes ? bytes : 1));
  *dptr = reinterpret_cast<uintptr_t>(p);
  std::lock_guard<std::mutex> lock(d->mu);
  d->allocs[*dptr] = bytes;
  return SB200_OK;
}

int sb200_mem_free(int dev, uint64_t dptr) {
  if (!dptr) return SB200_OK;
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  {
    std::lock_guard<std::mutex> lock(d->mu);
    auto it = d->allocs.find(dptr);
    if (it == d->allocs.end()) return SB200_OK;  // already freed (or never ours): idempotent
    d->allocs.erase(it);
  }
  CU_TRY(cudaFree(as_ptr<void>(dptr)));  // cudaFree waits for work that may still use the buffer
  return SB200_OK;
}

int sb200_mem_size(int dev, uint64_t dptr, uint64_t* bytes) {
  if (!bytes) return fail(SB200_ERR_INVALID_VALUE, "null bytes pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(d->mu);
  auto it = d->allocs.find(dptr);
  if (it == d->allocs.end()) return fail(SB200_ERR_INVALID_HANDLE, "unknown device buffer");
  *bytes = it->second;
  return SB200_OK;
}

int sb200_memset32(int dev, uint64_t dptr, uint32_t value, uint64_t count, uint64_t stream) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (count == 0) return SB200_OK;
  if (!dptr || (dptr & 3)) return fail(SB200_ERR_INVALID_VALUE, "memset32 needs a 4-byte aligned device pointer");
  if ((rc = check_extent(*d, dptr, count * 4, "memset32 destination"))) return rc;
  if (value == 0) {
    CU_TRY(cudaMemsetAsync(as_ptr<void>(dptr), 0, count * 4, as_stream(stream)));
    return SB200_OK;
  }
  // cuMemsetD32 equivalent through the runtime's 2-D memset is byte-wise only; use the driver entry
  typedef CUresult (*MemsetFn)(CUdeviceptr, unsigned int, size_t, CUstream);
  static MemsetFn fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemsetD32Async", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<MemsetFn>(f);
  }
  if (!fn) return fail(SB200_ERR_NO_DEVICE, "driver does not export cuMemsetD32Async");
  CUresult r = fn(static_cast<CUdeviceptr>(dptr), value, count, reinterpret_cast<CUstream>(as_stream(stream)));
  if (r != CUDA_SUCCESS) return fail(static_cast<int>(r), "cuMemsetD32Async failed with CUresult %d", (int)r);
  return SB200_OK;
}

int sb200_memcpy_htod(int dev, uint64_t dst, const void* src, uint64_t bytes) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (bytes == 0) return SB200_OK;
  if (!dst || !src) return fail(SB200_ERR_INVALID_VALUE, "null pointer passed to memcpy_htod");
  if ((rc = check_extent(*d, dst, bytes, "copy destination"))) return rc;
  if (bytes >= kStagedCopyMinBytes && staged_copy_enabled() && host_memory_is_pageable(src)) {
    const int e = staged_copy_to_device(dev, as_ptr<void>(dst), src, bytes);
    if (e) return cuda_fail(static_cast<cudaError_t>(e), "staged host-to-device copy");
    return SB200_OK;
  }
  CU_TRY(cudaMemcpy(as_ptr<void>(dst), src, bytes, cudaMemcpyHostToDevice));
  return SB200_OK;
}

int sb200_memcpy_dtoh(int dev, void* dst, uint64_t src, uint64_t bytes) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (bytes == 0) return SB200_OK;
  if (!dst || !src) return fail(SB200_ERR_INVALID_VALUE, "null pointer passed to memcpy_dtoh");
  if ((rc = check_extent(*d, src, bytes, "copy source"))) return rc;
  if (bytes >= kStagedCopyMinBytes && staged_copy_enabled() && host_memory_is_pageable(dst)) {
    const int e = staged_copy_to_host(dev, dst, as_ptr<void>(src), bytes);
    if (e) return cuda_fail(static_cast<cudaError_t>(e), "staged device-to-host copy");
    return check_status_word(*d);
  }
  CU_TRY(cudaMemcpy(dst, as_ptr<void>(src), bytes, cudaMemcpyDeviceToHost));
  return check_status_word(*d);
}

int sb200_memcpy_dtod(int dev, uint64_t dst, uint64_t src, uint64_t bytes) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (bytes == 0) return SB200_OK;
  if (!dst || !src) return fail(SB200_ERR_INVALID_VALUE, "null pointer passed to memcpy_dtod");
  if ((rc = check_extent(*d, dst, bytes, "copy destination")) || (rc = check_extent(*d, src, bytes, "copy source"))) return rc;
  CU_TRY(cudaMemcpy(as_ptr<void>(dst), as_ptr<void>(src), bytes, cudaMemcpyDeviceToDevice));
  return SB200_OK;
}

int sb200_memcpy_htod_async(int dev, uint64_t dst, const void* src, uint64_t bytes, uint64_t stream) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (bytes == 0) return SB200_OK;
  if (!dst || !src) return fail(SB200_ERR_INVALID_VALUE, "null pointer passed to memcpy_htod_async");
  if ((rc = check_extent(*d, dst, bytes, "copy destination"))) return rc;
  CU_TRY(cudaMemcpyAsync(as_ptr<void>(dst), src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return SB200_OK;
}

int sb200_memcpy_dtoh_async(int dev, void* dst, uint64_t src, uint64_t bytes, uint64_t stream) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (bytes == 0) return SB200_OK;
  if (!dst || !src) return fail(SB200_ERR_INVALID_VALUE, "null pointer passed to memcpy_dtoh_async");
  if ((rc = check_extent(*d, src, bytes, "copy source"))) return rc;
  CU_TRY(cudaMemcpyAsync(dst, as_ptr<void>(src), bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return SB200_OK;
}

int sb200_host_alloc(uint64_t bytes, void** ptr) {
  if (!ptr) return fail(SB200_ERR_INVALID_VALUE, "null ptr pointer");
  CU_TRY(cudaMallocHost(ptr, bytes ? bytes : 1));
  return SB200_OK;
}

int sb200_host_free(void* ptr) {
  if (!ptr) return SB200_OK;
  CU_TRY(cudaFreeHost(ptr));
  return SB200_OK;
}

int sb200_host_register(void* ptr, uint64_t bytes) {
  if (!ptr || bytes == 0) return fail(SB200_ERR_INVALID_VALUE, "null pointer or empty range");
  cudaError_t e = cudaHostRegister(ptr, bytes, cudaHostRegisterPortable);
  if (e == cudaErrorHostMemoryAlreadyRegistered) {
    cudaGetLastError();
    return SB200_OK;
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaHostRegister");
  return SB200_OK;
}

int sb200_host_unregister(void* ptr) {
  if (!ptr) return SB200_OK;
  cudaError_t e = cudaHostUnregister(ptr);
  if (e == cudaErrorHostMemoryNotRegistered) {
    cudaGetLastError();
    return SB200_OK;
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaHostUnregister");
  return SB200_OK;
}

int sb200_stream_create(int dev, uint64_t* stream) {
  if (!stream) return fail(SB200_ERR_INVALID_VALUE, "null stream pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  cudaStream_t s;
  CU_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = reinterpret_cast<uintptr_t>(s);
  return SB200_OK;
}

int sb200_stream_destroy(int dev, uint64_t stream) {
  if (!stream) return SB200_OK;
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  CU_TRY(cudaStreamDestroy(as_stream(stream)));
  return SB200_OK;
}

int sb200_stream_synchronize(int dev, uint64_t stream) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  CU_TRY(cudaStreamSynchronize(as_stream(stream)));
  return check_status_word(*d);
}

int sb200_stream_wrap(int dev, uint64_t native_stream, uint64_t* stream) {
  if (!stream) return fail(SB200_ERR_INVALID_VALUE, "null stream pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  *stream = native_stream;
  return SB200_OK;
}

int sb200_event_create(int dev, uint64_t* event) {
  if (!event) return fail(SB200_ERR_INVALID_VALUE, "null event pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  cudaEvent_t e;
  CU_TRY(cudaEventCreate(&e));
  *event = reinterpret_cast<uintptr_t>(e);
  return SB200_OK;
}

int sb200_event_destroy(int dev, uint64_t event) {
  if (!event) return SB200_OK;
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  CU_TRY(cudaEventDestroy(as_event(event)));
  return SB200_OK;
}

int sb200_event_record(int dev, uint64_t event, uint64_t stream) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!event) return fail(SB200_ERR_INVALID_HANDLE, "null event");
  CU_TRY(cudaEventRecord(as_event(event), as_stream(stream)));
  return SB200_OK;
}

int sb200_event_synchronize(int dev, uint64_t event) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!event) return fail(SB200_ERR_INVALID_HANDLE, "null event");
  CU_TRY(cudaEventSynchronize(as_event(event)));
  return SB200_OK;
}

int sb200_event_elapsed_ms(int dev, uint64_t start, uint64_t stop, float* ms) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!start || !stop || !ms) return fail(SB200_ERR_INVALID_HANDLE, "null event or result pointer");
  CU_TRY(cudaEventElapsedTime(ms, as_event(start), as_event(stop)));
  return SB200_OK;
}

int sb200_kernel_compile(int dev, const char* ir_text, const char* name, uint64_t* kernel) {
  if (!ir_text || !kernel) return fail(SB200_ERR_INVALID_VALUE, "null IR text or kernel pointer");
  if (dev < 0 || dev >= kMaxDevices) return fail(SB200_ERR_INVALID_VALUE, "device index %d out of range", dev);
  KernelObj* k = new KernelObj;
  k->dev = dev;
  std::string err;
  int rc = ir_compile(ir_text, &k->plan, &err);
  if (rc) {
    delete k;
    return fail(rc, "%s", err.c_str());
  }
  if ((k->plan.kind == KIND_MAP && k->plan.map.op == OP_GENERIC) || k->plan.kind == KIND_BLOCK_REDUCE) {
    rc = jit_compile_cubin(k->plan.generic.source, k->plan.name, &k->cubin, &err);
    if (rc) {
      delete k;
      return fail(rc, "%s", err.c_str());
    }
  }
  if (name && *name && k->plan.name != name && debug_kernel())
    fprintf(stderr, "[sarek-b200] kernel name '%s' requested, IR names it '%s'\n", name, k->plan.name.c_str());
  if (debug_kernel()) fprintf(stderr, "[sarek-b200] compiled %s -> %s\n", k->plan.name.c_str(), k->plan.description.c_str());
  {
    std::lock_guard<std::mutex> lock(g_kernels_mu);
    g_kernels.insert(k);
  }
  *kernel = reinterpret_cast<uintptr_t>(k);
  return SB200_OK;
}

int sb200_kernel_destroy(uint64_t kernel) {
  KernelObj* k = reinterpret_cast<KernelObj*>(static_cast<uintptr_t>(kernel));
  {
    std::lock_guard<std::mutex> lock(g_kernels_mu);
    if (!g_kernels.erase(k)) return SB200_OK;
  }
  for (int i = 0; i < kMaxDevices; ++i)
    if (k->jit[i].module && cudaSetDevice(i) == cudaSuccess) jit_unload(&k->jit[i]);
  delete k;
  return SB200_OK;
}

int sb200_kernel_kind(uint64_t kernel, int* kind) {
  KernelObj* k = find_kernel(kernel);
  if (!k || !kind) return fail(SB200_ERR_INVALID_HANDLE, "unknown kernel handle");
  *kind = k->plan.kind;
  return SB200_OK;
}

int sb200_kernel_describe(uint64_t kernel, char* buf, int buflen) {
  KernelObj* k = find_kernel(kernel);
  if (!k || !buf || buflen <= 0) return fail(SB200_ERR_INVALID_HANDLE, "unknown kernel handle");
  snprintf(buf, static_cast<size_t>(buflen), "%s", k->plan.description.c_str());
  return SB200_OK;
}

static int kernel_launch_impl(uint64_t kernel, const sb200_arg* args, int nargs, const void* const* host_ptrs, void* const* host_out,
                              int32_t* prefetched, const uint32_t grid[3], const uint32_t block[3], uint64_t stream) {
  KernelObj* k = find_kernel(kernel);
  if (!k) return fail(SB200_ERR_INVALID_HANDLE, "unknown kernel handle");
  if ((!args && nargs > 0) || nargs < 0 || !grid || !block) return fail(SB200_ERR_INVALID_VALUE, "null argument list or dims");
  for (int i = 0; i < 3; ++i)
    if (grid[i] == 0 || block[i] == 0) return fail(SB200_ERR_INVALID_VALUE, "grid and block dimensions must be positive");
  std::vector<Slot> slots;
  int rc = bind_args(k->plan, args, nargs, &slots, host_ptrs, host_out);
  if (rc) return rc;
  if (prefetched)
    for (int i = 0; i < nargs; ++i) prefetched[i] = 0;
  DeviceState* d;
  rc = device_ready(k->dev, &d);
  if (rc) return rc;
  // a vector that lies in a buffer of this library cannot be longer than what is left of that buffer,
  // whatever length the caller passes with it
  for (size_t p = 0; p < slots.size(); ++p) {
    if (!slots[p].is_vec) continue;
    const std::string what = "kernel '" + k->plan.name + "': vector " + k->plan.params[p].name + " of stated length " +
                             std::to_string(slots[p].len);
    if ((rc = check_extent(*d, slots[p].ptr, static_cast<uint64_t>(slots[p].len) * 4, what.c_str()))) return rc;
  }
  if (debug_kernel())
    fprintf(stderr, "[sarek-b200] launch %s grid=(%u,%u,%u) block=(%u,%u,%u)\n", k->plan.description.c_str(), grid[0], grid[1],
            grid[2], block[0], block[1], block[2]);
  cudaStream_t st = as_stream(stream);
  // launch-from-host: which vectors still have to be brought over, and whether all of them can be copied asynchronously
  bool any_host = false, all_pinned = true;  // all_pinned: every large host array is page-locked
  for (const Slot& sl : slots)
    if (sl.is_vec && sl.host && sl.len > 0) {
      any_host = true;
      // small pageable arrays (a bias) go through the driver's own staging and do not stand in the way of the pipeline
      if (static_cast<size_t>(sl.len) * 4 >= kStagedCopyMinBytes && host_memory_is_pageable(sl.host)) all_pinned = false;
    }
  // the result of a matmul follows its kernel back to the host when the caller names a page-locked array for it
  const bool is_gemm = k->plan.kind != KIND_MAP && k->plan.kind != KIND_BLOCK_REDUCE;
  void* d_host = nullptr;
  int d_arg = -1;
  if (is_gemm && prefetched) {
    const Slot& out = slots[k->plan.gemm.d];
    if (out.host_out && out.len > 0 && !host_memory_is_pageable(out.host_out)) {
      d_host = out.host_out;
      d_arg = out.arg;
    }
  }
  // the element-wise operators by chunks, when the vectors are large and the launch indexes by the global thread id
  if (k->plan.kind == KIND_MAP && k->plan.map.op != OP_GENERIC && k->plan.map.index_kind == IDX_GLOBAL && all_pinned) {
    const MapPlan& m = k->plan.map;
    long long n = static_cast<long long>(grid[0]) * block[0];
    if (m.n_param >= 0 && slots[m.n_param].i < n) n = slots[m.n_param].i;
    void* out_host[2] = {nullptr, nullptr};
    int out_arg[2] = {-1, -1};
    for (int j = 0; j < 2 && prefetched; ++j) {
      const int v = j == 0 ? m.out0 : m.out1;
      if (v >= 0 && slots[v].host_out && slots[v].len > 0 && !host_memory_is_pageable(slots[v].host_out)) {
        out_host[j] = slots[v].host_out;
        out_arg[j] = slots[v].arg;
      }
    }
    bool fits = n > 0;
    for (int v : {m.out0, m.out1, m.in0, m.in1})
      if (v >= 0 && slots[v].len < n) fits = false;  // the plain launch reports it
    if (fits && static_cast<size_t>(n) * 4 >= kStagedCopyMinBytes && (any_host || out_host[0] || out_host[1])) {
      rc = map_upload_pipeline(*d, st, k->plan, slots, n, out_host);
      for (int j = 0; j < 2 && !rc; ++j)
        if (out_arg[j] >= 0) prefetched[out_arg[j]] = 1;
      return rc;
    }
  }
  if (any_host) {
    if (is_gemm && all_pinned) {
      bool pipelined = false;
      rc = launch_gemm_kernel(*d, k->plan, slots, grid, block, st, true, &pipelined, d_host);
      if (pipelined) {
        if (!rc && d_host) prefetched[d_arg] = 1;
        return rc;
      }
      if (rc) return rc;
    }
    // no pipelining for this launch: whole vectors first (staged when pageable and large), ordered before the kernel
    CU_TRY(cudaStreamSynchronize(st));
    for (const Slot& sl : slots) {
      if (!sl.is_vec || !sl.host || sl.len <= 0) continue;
      const size_t bytes = static_cast<size_t>(sl.len) * 4;
      if (staged_copy_enabled() && bytes >= kStagedCopyMinBytes && host_memory_is_pageable(sl.host)) {
        const int e = staged_copy_to_device(k->dev, as_ptr<void>(sl.ptr), sl.host, bytes, true);
        if (e) return cuda_fail(static_cast<cudaError_t>(e), "staged copy of a kernel argument");
      } else {
        CU_TRY(cudaMemcpy(as_ptr<void>(sl.ptr), sl.host, bytes, cudaMemcpyHostToDevice));
      }
    }
    CU_TRY(cudaStreamSynchronize(0));
  }
  if (k->plan.kind == KIND_MAP) return launch_map_kernel(*d, *k, slots, grid, block, st);
  if (k->plan.kind == KIND_BLOCK_REDUCE) return launch_block_reduce(*d, *k, slots, grid, block, st);
  rc = launch_gemm_kernel(*d, k->plan, slots, grid, block, st, false, nullptr, d_host);
  if (!rc && d_host) prefetched[d_arg] = 1;
  return rc;
}

int sb200_kernel_launch(uint64_t kernel, const sb200_arg* args, int nargs, const uint32_t grid[3], const uint32_t block[3],
                        uint32_t shared_mem, uint64_t stream) {
  (void)shared_mem;  // forwarded by the caller even when arrays are static; our kernels size their own
  return kernel_launch_impl(kernel, args, nargs, nullptr, nullptr, nullptr, grid, block, stream);
}

int sb200_kernel_launch_from_host(uint64_t kernel, const sb200_arg* args, int nargs, const void* const* host_ptrs,
                                  void* const* host_out, int32_t* prefetched, const uint32_t grid[3], const uint32_t block[3],
                                  uint32_t shared_mem, uint64_t stream) {
  (void)shared_mem;
  if (!host_ptrs && nargs > 0) return fail(SB200_ERR_INVALID_VALUE, "null host pointer table");
  if ((host_out == nullptr) != (prefetched == nullptr))
    return fail(SB200_ERR_INVALID_VALUE, "host_out and prefetched go together: both tables or neither");
  return kernel_launch_impl(kernel, args, nargs, host_ptrs, host_out, prefetched, grid, block, stream);
}

int sb200_prefetch_wait(int dev) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (d->pipe_out) CU_TRY(cudaStreamSynchronize(d->pipe_out));
  return check_status_word(*d, false);
}

static int copy_out(const std::string& s, char* out, int outlen) {
  if (!out || outlen <= 0) return fail(SB200_ERR_INVALID_VALUE, "null output buffer");
  if (static_cast<int>(s.size()) + 1 > outlen)
    return fail(SB200_ERR_TOO_LARGE, "output buffer of %d bytes is too small for %zu bytes", outlen, s.size() + 1);
  memcpy(out, s.c_str(), s.size() + 1);
  return SB200_OK;
}

int sb200_ir_can_fuse(const char* producer, const char* consumer, const char* intermediate, int* result) {
  if (!producer || !consumer || !intermediate || !result) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  bool ok = false;
  std::string err;
  int rc = ir_can_fuse(producer, consumer, intermediate, &ok, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  *result = ok ? 1 : 0;
  return SB200_OK;
}

int sb200_ir_fuse(const char* producer, const char* consumer, const char* intermediate, char* out, int outlen) {
  if (!producer || !consumer || !intermediate) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  std::string text, err;
  int rc = ir_fuse(producer, consumer, intermediate, &text, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  return copy_out(text, out, outlen);
}

int sb200_ir_fuse_pipeline(const char* const* kernels, int count, char* out, int outlen, char* eliminated, int elimlen) {
  if (!kernels || count <= 0) return fail(SB200_ERR_INVALID_VALUE, "empty kernel list");
  std::vector<std::string> ks;
  for (int i = 0; i < count; ++i) {
    if (!kernels[i]) return fail(SB200_ERR_INVALID_VALUE, "null kernel text");
    ks.push_back(kernels[i]);
  }
  std::string text, err;
  std::vector<std::string> elim;
  int rc = ir_fuse_pipeline(ks, &text, &elim, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  std::string joined;
  for (size_t i = 0; i < elim.size(); ++i) joined += (i ? "," : "") + elim[i];
  if (eliminated && elimlen > 0 && (rc = copy_out(joined, eliminated, elimlen))) return rc;
  return copy_out(text, out, outlen);
}

int sb200_ir_fuse_pipeline_as(const char* const* kernels, int count, int kind, char* out, int outlen, char* eliminated,
                              int elimlen) {
  if (!kernels || count <= 0) return fail(SB200_ERR_INVALID_VALUE, "empty kernel list");
  std::vector<std::string> ks;
  for (int i = 0; i < count; ++i) {
    if (!kernels[i]) return fail(SB200_ERR_INVALID_VALUE, "null kernel text");
    ks.push_back(kernels[i]);
  }
  std::string text, err;
  std::vector<std::string> elim;
  int rc = ir_fuse_pipeline_as(ks, kind, &text, &elim, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  std::string joined;
  for (size_t i = 0; i < elim.size(); ++i) joined += (i ? "," : "") + elim[i];
  if (eliminated && elimlen > 0 && (rc = copy_out(joined, eliminated, elimlen))) return rc;
  return copy_out(text, out, outlen);
}

int sb200_ir_should_fuse(const char* producer, const char* consumer, const char* intermediate, char* decision, int declen,
                         char* reason, int reasonlen) {
  if (!producer || !consumer || !intermediate) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  std::string d, r, err;
  int rc = ir_should_fuse(producer, consumer, intermediate, &d, &r, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  if ((rc = copy_out(d, decision, declen))) return rc;
  return copy_out(r, reason, reasonlen);
}

int sb200_ir_auto_fuse_pipeline(const char* const* kernels, int count, char* out, int outlen, char* eliminated, int elimlen,
                                char* skipped, int skiplen) {
  if (!kernels || count <= 0) return fail(SB200_ERR_INVALID_VALUE, "empty kernel list");
  std::vector<std::string> ks;
  for (int i = 0; i < count; ++i) {
    if (!kernels[i]) return fail(SB200_ERR_INVALID_VALUE, "null kernel text");
    ks.push_back(kernels[i]);
  }
  std::string text, err;
  std::vector<std::string> elim, skip;
  int rc = ir_auto_fuse_pipeline(ks, &text, &elim, &skip, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  std::string je, js;
  for (size_t i = 0; i < elim.size(); ++i) je += (i ? "," : "") + elim[i];
  for (size_t i = 0; i < skip.size(); ++i) js += (i ? "\n" : "") + skip[i];
  if (eliminated && elimlen > 0 && (rc = copy_out(je, eliminated, elimlen))) return rc;
  if (skipped && skiplen > 0 && (rc = copy_out(js, skipped, skiplen))) return rc;
  return copy_out(text, out, outlen);
}

int sb200_ir_can_fuse_as(const char* producer, const char* consumer, const char* intermediate, int kind, int* result) {
  if (!producer || !consumer || !intermediate || !result) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  bool ok = false;
  std::string err;
  int rc = ir_can_fuse_as(producer, consumer, intermediate, kind, &ok, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  if (!ok && !err.empty()) fail(SB200_OK, "%s", err.c_str());  // the reason, for sb200_last_error_string
  *result = ok ? 1 : 0;
  return SB200_OK;
}

int sb200_ir_fuse_as(const char* producer, const char* consumer, const char* intermediate, int kind, char* out, int outlen,
                     int* fused) {
  if (!producer || !consumer || !intermediate || !fused) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  std::string text, err;
  bool f = false;
  int rc = ir_fuse_as(producer, consumer, intermediate, kind, &text, &f, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  if (!f && !err.empty()) fail(SB200_OK, "%s", err.c_str());  // the reason, for sb200_last_error_string
  *fused = f ? 1 : 0;
  return copy_out(text, out, outlen);
}

int sb200_ir_analyze(const char* kernel, char* out, int outlen) {
  if (!kernel) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  std::string rep, err;
  int rc = ir_analyze(kernel, &rep, &err);
  if (rc) return fail(rc, "%s", err.c_str());
  return copy_out(rep, out, outlen);
}

int sb200_gemm_f32(int dev, uint64_t stream, int mode, int64_t M, int64_t N, int64_t K, uint64_t A, int64_t lda, uint64_t B,
                   int64_t ldb, uint64_t D, int64_t ldd, float alpha, uint64_t C, int64_t ldc, float beta, uint64_t bias,
                   int act) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  return run_gemm(*d, as_stream(stream), mode, M, N, K, A, lda, B, ldb, D, ldd, alpha, C, ldc, beta, bias, act);
}

int sb200_gemm_f32_gather(int dev, uint64_t stream, int mode, int64_t M_local, int64_t N, int64_t K, uint64_t A, int64_t lda,
                          uint64_t B, int64_t ldb, const uint64_t* d_copies, int n_copies, int64_t row_offset, int64_t ldd,
                          float alpha, uint64_t C, int64_t ldc, float beta, uint64_t bias, int act) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!d_copies || n_copies < 1 || n_copies > 8) return fail(SB200_ERR_INVALID_VALUE, "between 1 and 8 copies of D are supported");
  if (row_offset < 0 || ldd < N) return fail(SB200_ERR_INVALID_VALUE, "bad row offset or leading dimension");
  uint64_t shifted[8];
  for (int r = 0; r < n_copies; ++r) {
    if (!d_copies[r] || (d_copies[r] & 3)) return fail(SB200_ERR_INVALID_VALUE, "null or misaligned copy of D (%d)", r);
    shifted[r] = d_copies[r] + static_cast<uint64_t>(row_offset) * static_cast<uint64_t>(ldd) * 4;
  }
  // copy 0 is the kernel's primary output (and what C may alias); the others are the replicas
  return run_gemm(*d, as_stream(stream), mode, M_local, N, K, A, lda, B, ldb, shifted[0], ldd, alpha, C, ldc, beta, bias, act,
                  shifted + 1, n_copies - 1);
}

int sb200_ipc_export(int dev, uint64_t dptr, void* handle64) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!dptr || !handle64) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  cudaIpcMemHandle_t h;
  CU_TRY(cudaIpcGetMemHandle(&h, as_ptr<void>(dptr)));
  memcpy(handle64, &h, 64);
  return SB200_OK;
}

int sb200_ipc_open(int dev, const void* handle64, uint64_t* dptr) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!handle64 || !dptr) return fail(SB200_ERR_INVALID_VALUE, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  CU_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *dptr = reinterpret_cast<uintptr_t>(p);
  return SB200_OK;
}

int sb200_ipc_close(int dev, uint64_t dptr) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (!dptr) return SB200_OK;
  CU_TRY(cudaIpcCloseMemHandle(as_ptr<void>(dptr)));
  return SB200_OK;
}

int sb200_gemm_workspace_bytes(int mode, int64_t M, int64_t N, int64_t K, uint64_t* bytes) {
  if (!bytes || M < 0 || N < 0 || K < 0) return fail(SB200_ERR_INVALID_VALUE, "bad argument");
  if (!sb200::valid_mode(mode))
    return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (mode == SB200_MODE_3XF16 || mode == SB200_MODE_F16) {
    *bytes = (M == 0 || N == 0 || K == 0) ? 0 : gemm_f16_workspace_need(M, N, K, mode == SB200_MODE_3XF16);
    return SB200_OK;
  }
  if (mode == SB200_MODE_3XMIXED) {  // upper bound: which of the two routes runs depends on the operands' addresses
    const size_t plain = gemm_workspace_need(SB200_MODE_3XTF32, M, N, K), mixed = gemm_mix_workspace_need(M, N, K);
    *bytes = (M == 0 || N == 0 || K == 0) ? 0 : (plain > mixed ? plain : mixed);
    return SB200_OK;
  }
  *bytes = (M == 0 || N == 0 || K == 0) ? 0 : gemm_workspace_need(mode, M, N, K);
  return SB200_OK;
}

int sb200_gemm_describe(int mode, int64_t M, int64_t N, int64_t K, int addressable, int sm_count, char* out, int outlen) {
  if (M < 0 || N < 0 || K < 0 || sm_count <= 0) return fail(SB200_ERR_INVALID_VALUE, "bad argument");
  if (!sb200::valid_mode(mode))
    return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (M == 0 || N == 0) return copy_out("nothing to do", out, outlen);
  if (K == 0) return copy_out("gemm_k0_kernel (epilogue only)", out, outlen);
  if (mode == SB200_MODE_3XF16 || mode == SB200_MODE_F16) {
    const bool three = mode == SB200_MODE_3XF16;
    const long long kp = round_up(K, 64);
    const int clusters = sm_count / 2 > 0 ? sm_count / 2 : 1;
    const int tn = choose_tile_n(M, N, kp / 64, clusters, three ? 3 : 1);
    const long long tiles = ((M + PAIR_BM - 1) / PAIR_BM) * ((N + tn - 1) / tn);
    const int stages = tn == 256 ? (three ? PairCfg<4, 256>::kStages : PairCfg<2, 256>::kStages)
                     : tn == 128 ? (three ? PairCfg<4, 128>::kStages : PairCfg<2, 128>::kStages)
                                 : (three ? PairCfg<4, 64>::kStages : PairCfg<2, 64>::kStages);
    char fb[256];
    snprintf(fb, sizeof fb, "pair fp16-panels tile=%dx%d stages=%d tiles=%lld waves=%lld workspace=%zu launches=4", PAIR_BM, tn, stages,
             tiles, (tiles + clusters - 1) / clusters, gemm_f16_workspace_need(M, N, K, three));
    return copy_out(fb, out, outlen);
  }
  if (mode == SB200_MODE_3XMIXED) {
    if (gemm_mix_applies(M, N, K, addressable != 0)) {
      const int clusters = sm_count / 2 > 0 ? sm_count / 2 : 1;
      const int tn = choose_tile_n(M, N, round_up(K, GEMM_BK) / GEMM_BK, clusters, 3);
      const long long tiles = ((M + PAIR_BM - 1) / PAIR_BM) * ((N + tn - 1) / tn);
      const int stages = tn == 256 ? PairCfg<5, 256>::kStages : tn == 128 ? PairCfg<5, 128>::kStages : PairCfg<5, 64>::kStages;
      char fb[256];
      snprintf(fb, sizeof fb, "pair mixed tile=%dx%d stages=%d tiles=%lld waves=%lld workspace=%zu launches=7", PAIR_BM, tn, stages,
               tiles, (tiles + clusters - 1) / clusters, gemm_mix_workspace_need(M, N, K));
      return copy_out(fb, out, outlen);
    }
    mode = SB200_MODE_3XTF32;
  }
  const GemmRoute r = route_gemm(mode, M, N, K, addressable != 0, sm_count, M);
  char buf[256];
  snprintf(buf, sizeof buf, "%s %s tile=%dx%d stages=%d tiles=%lld waves=%lld workspace=%zu launches=%d",
           r.pair ? "pair" : "single", r.direct ? "direct" : "panels", r.pair ? PAIR_BM : GEMM_BM, r.tile_n, r.stages, r.tiles,
           r.waves, r.workspace, r.direct ? (mode == SB200_MODE_3XTF32 ? 2 : 1) : 3);
  return copy_out(buf, out, outlen);
}

int sb200_vector_add_f32(int dev, uint64_t stream, uint64_t c, uint64_t a, uint64_t b, int64_t n) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  return run_map(*d, as_stream(stream), OP_VECADD, c, 0, a, b, 0.0f, n);
}

int sb200_stream_triad_f32(int dev, uint64_t stream, uint64_t a, uint64_t b, uint64_t c, float scalar, int64_t n) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  return run_map(*d, as_stream(stream), OP_TRIAD, a, 0, b, c, scalar, n);
}

int sb200_chain_triad_square_f32(int dev, uint64_t stream, uint64_t dd, uint64_t a_out, uint64_t b, uint64_t c, float scalar,
                                 int64_t n) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  return run_map(*d, as_stream(stream), a_out ? OP_CHAIN_KEEP : OP_CHAIN, dd, a_out, b, c, scalar, n);
}

int sb200_set_mode(int mode) {
  if (!sb200::valid_mode(mode)) return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  g_mode.store(mode);
  return SB200_OK;
}

int sb200_mixed_plan(float max_a, float max_b, int32_t out[5]) {
  if (!out) return fail(SB200_ERR_INVALID_VALUE, "null output");
  uint32_t ua, ub;
  memcpy(&ua, &max_a, 4);
  memcpy(&ub, &max_b, 4);
  const MixCtl c = mix_plan(ua & 0x7fffffffu, ub & 0x7fffffffu);
  out[0] = c.ok;
  out[1] = c.rescale_stages;
  out[2] = c.first_scale;
  out[3] = c.shift_a;
  out[4] = c.shift_b;
  return SB200_OK;
}

int sb200_set_lockstep(int setting) {
  if (setting < -1 || setting > 1) return fail(SB200_ERR_INVALID_VALUE, "lockstep setting must be -1 (by k-loop length), 0 or 1");
  g_lockstep.store(setting);
  return SB200_OK;
}

int sb200_set_mixed_min_macs(int64_t macs) {
  if (macs < 0) return fail(SB200_ERR_INVALID_VALUE, "negative threshold");
  g_mix_min_macs.store(macs);
  return SB200_OK;
}

int sb200_set_gemm_tile_n(int tile_n) {
  if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256)
    return fail(SB200_ERR_INVALID_VALUE, "tile columns must be 0 (automatic), 64, 128 or 256, not %d", tile_n);
  g_tile_n.store(tile_n);
  return SB200_OK;
}

int sb200_set_gemm_variant(int variant) {
  if (variant < 0 || variant > 3)
    return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM variant %d (0 auto, 1 single, 2 pair, 3 pair with panels)", variant);
  g_gemm_variant.store(variant);
  return SB200_OK;
}

int sb200_set_l2_policy(int bits) {
  if (bits < -1 || bits > 63 || (bits >= 0 && ((bits & 3) == 3 || ((bits >> 2) & 3) == 3 || ((bits >> 4) & 3) == 3)))
    return fail(SB200_ERR_INVALID_VALUE, "L2 policy bits %d: three 2-bit fields, each 0 (normal), 1 (evict first) or 2 (evict last)", bits);
  g_l2_policy.store(bits);
  return SB200_OK;
}

int sb200_get_mode(int* mode) {
  if (!mode) return fail(SB200_ERR_INVALID_VALUE, "null mode pointer");
  *mode = current_mode();
  return SB200_OK;
}

int sb200_fill_f32(int dev, uint64_t stream, uint64_t dptr, int64_t n, uint64_t seed, uint64_t stream_id, int kind, double sigma,
                   int64_t first) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (n < 0 || kind < 0 || kind > 2) return fail(SB200_ERR_INVALID_VALUE, "bad fill arguments");
  if (n == 0) return SB200_OK;
  if (!dptr || (dptr & 3)) return fail(SB200_ERR_INVALID_VALUE, "fill needs a 4-byte aligned device pointer");
  if ((rc = check_extent(*d, dptr, static_cast<uint64_t>(n) * 4, "fill destination"))) return rc;
  long long grid = (n + 255) / 256;
  const long long cap = static_cast<long long>(d->sm_count) * 16;
  if (grid > cap) grid = cap;
  fill_kernel<<<static_cast<unsigned>(grid), 256, 0, as_stream(stream)>>>(as_ptr<float>(dptr), n, seed, stream_id, kind, sigma,
                                                                          first);
  return launch_check("fill_kernel");
}

int sb200_enable_profiling(int on) {
  g_profiling.store(on ? 1 : 0);
  return SB200_OK;
}

int sb200_profile_gemm_read(int dev, uint64_t* calls, double* prep_ms, double* main_ms) {
  if (!calls || !prep_ms || !main_ms) return fail(SB200_ERR_INVALID_VALUE, "null result pointer");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  std::vector<DeviceState::ProfRec> recs;
  {
    std::lock_guard<std::mutex> lock(d->mu);
    recs.swap(d->prof);
  }
  *calls = recs.size();
  *prep_ms = 0.0;
  *main_ms = 0.0;
  for (auto& r : recs) {
    float a = 0.f, b = 0.f;
    cudaError_t e = cudaEventSynchronize(r.e2);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&a, r.e0, r.e1);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&b, r.e1, r.e2);
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
    cudaEventDestroy(r.e2);
    if (e != cudaSuccess) return cuda_fail(e, "reading GEMM profile events");
    *prep_ms += a;
    *main_ms += b;
  }
  return SB200_OK;
}

int sb200_selftest_wait_timeout(int dev, uint32_t limit_ms) {
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  if (limit_ms == 0 || limit_ms > 1000) return fail(SB200_ERR_INVALID_VALUE, "limit must be 1..1000 ms");
  d->status_armed.store(true);
  wait_timeout_probe_kernel<<<1, 32>>>(d->status, static_cast<unsigned long long>(limit_ms) * 1000000ull);
  return launch_check("wait_timeout_probe_kernel");
}

int sb200_launch_count(uint64_t* count) {
  if (!count) return fail(SB200_ERR_INVALID_VALUE, "null count pointer");
  *count = g_launches.load();
  return SB200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// GEMM for callers that must not allocate device memory
// ---------------------------------------------------------------------------
// sb200_gemm_f32 keeps its TF32 operand panels in a grow-only workspace that it
// obtains with cudaMalloc (and releases with cudaFree when it has to grow).
// Two kinds of caller cannot live with that.  A host framework whose own
// caching allocator already holds all of the GPU's memory makes every further
// cudaMalloc fail.  And a caller that keeps other streams busy, or that calls
// from a latency-critical loop, cannot afford the device-wide synchronisation
// that cudaMalloc / cudaFree imply.  The variant below computes the same
// result with the same kernels, but its panels live in a fixed array that is
// part of the library image, so the call allocates nothing at all: no
// cudaMalloc, no cudaFree, no pinned host memory, no CUDA events.
//
// Price and rules:
//  * Every GPU on which the library is loaded carries the array (32 MiB) from
//    load to exit.
//  * Problem sizes are limited by it: the panels need
//    (M + N) * roundup(K, 32) * 4 bytes, twice that in 3xTF32 mode (each part
//    rounded up to 1 KiB); larger problems are refused with SB200_ERR_TOO_LARGE.
//    1024^3 in 3xTF32 mode and 1448^3 in TF32 mode fit.
//  * All calls on a device share the one array and it keeps whatever the last
//    call left in it.  Nothing in it has to start at zero: each call rewrites
//    every panel element it later reads, including the zero padding of K.
//    For the same reason two calls that overlap on the GPU (different streams,
//    or different host threads) race on the panels; serialise them.
//  * The first call on each device looks up the array's device address.  Make
//    that first call before any stream capture begins.
//  * Every call waits on `stream` until its kernels have finished and then reads
//    a status word back with a synchronous copy, so that a device-side wait that
//    ran out of time is reported by the call that suffered it, as
//    SB200_ERR_TIMEOUT.  Do not issue it on a stream that is being captured.
//  * Operands that lie inside buffers from sb200_mem_alloc are checked against
//    the end of their buffer exactly as sb200_gemm_f32 does (SB200_ERR_BOUNDS).
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(32) << 20;

// In host code these two names are only stand-ins for the device objects; the
// addresses kernels may use come from cudaGetSymbolAddress (noalloc_setup).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
static __device__ int g_noalloc_status;

struct NoAllocDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int* status = nullptr;             // device address of g_noalloc_status on this device
  int sm_count = 0;
};
NoAllocDevice g_noalloc[kMaxDevices];
std::mutex g_noalloc_mu;

// Once per device, with that device current.
int noalloc_setup(int dev, NoAllocDevice** out) {
  if (dev < 0 || dev >= kMaxDevices) return fail(SB200_ERR_INVALID_VALUE, "device index %d out of range", dev);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(SB200_ERR_NO_DEVICE, "no CUDA device available");
  }
  if (dev >= count) return fail(SB200_ERR_INVALID_VALUE, "device index %d but only %d device(s)", dev, count);
  CU_TRY(cudaSetDevice(dev));
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  NoAllocDevice& nd = g_noalloc[dev];
  if (!nd.ready) {
    int major = 0, sms = 0;
    CU_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    CU_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10) return fail(SB200_ERR_NO_DEVICE, "device %d is not sm_100; this library carries sm_100a code only", dev);
    void* p = nullptr;
    CU_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    nd.scratch = static_cast<unsigned char*>(p);
    CU_TRY(cudaGetSymbolAddress(&p, g_noalloc_status));
    nd.status = static_cast<int*>(p);
    CU_TRY(cudaMemset(nd.status, 0, sizeof(int)));
    nd.sm_count = sms;
    nd.ready = true;
  }
  *out = &nd;
  return SB200_OK;
}

template <int MODE>
int launch_gemm_fixed_scratch(const NoAllocDevice& nd, cudaStream_t st, long long M, long long N, long long K, const float* A,
                              long long lda, const float* B, long long ldb, GemmParams gp) {
  using Cfg = GemmCfg<MODE>;
  CU_TRY(cudaFuncSetAttribute(gemm_tf32_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(Cfg::kSmemBytes)));
  const long long kp = round_up(K, GEMM_BK);
  const size_t a_bytes = round_up(M * kp * 4, 1024), b_bytes = round_up(N * kp * 4, 1024);
  float* a_hi = reinterpret_cast<float*>(nd.scratch);
  float* b_hi = reinterpret_cast<float*>(nd.scratch + a_bytes);
  float* a_lo = MODE == 3 ? reinterpret_cast<float*>(nd.scratch + a_bytes + b_bytes) : a_hi;
  float* b_lo = MODE == 3 ? reinterpret_cast<float*>(nd.scratch + 2 * a_bytes + b_bytes) : b_hi;
  int rc;
  {
    long long grid = (M * (kp >> 2) + 255) / 256;
    const long long cap = static_cast<long long>(nd.sm_count) * 16;
    if (grid > cap) grid = cap;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 3) == 0) ? 1 : 0;
    prep_a_kernel<MODE><<<static_cast<unsigned>(grid), 256, 0, st>>>(A, lda, a_hi, a_lo, static_cast<int>(M),
                                                                      static_cast<int>(K), static_cast<int>(kp), vec_ok);
    if ((rc = launch_check("prep_a_kernel"))) return rc;
  }
  {
    long long grid = (kp >> 5) * ((N + 31) >> 5);
    const long long cap = static_cast<long long>(nd.sm_count) * 32;
    if (grid > cap) grid = cap;
    prep_b_kernel<MODE><<<static_cast<unsigned>(grid), dim3(32, 8), 0, st>>>(B, ldb, b_hi, b_lo, static_cast<int>(K),
                                                                               static_cast<int>(N), static_cast<int>(kp));
    if ((rc = launch_check("prep_b_kernel"))) return rc;
  }
  CUtensorMap ma_hi, mb_hi, ma_lo, mb_lo;
  if ((rc = encode_panel_map(&ma_hi, a_hi, kp, M, GEMM_BM))) return rc;
  if ((rc = encode_panel_map(&mb_hi, b_hi, kp, N, GEMM_BN))) return rc;
  if ((rc = encode_panel_map(&ma_lo, a_lo, kp, M, GEMM_BM))) return rc;
  if ((rc = encode_panel_map(&mb_lo, b_lo, kp, N, GEMM_BN))) return rc;
  gp.num_k_blocks = static_cast<int>(kp / GEMM_BK);
  gp.tiles_m = static_cast<int>((M + GEMM_BM - 1) / GEMM_BM);
  gp.tiles_n = static_cast<int>((N + GEMM_BN - 1) / GEMM_BN);
  gp.status = nd.status;
  derive_params(&gp);
  const long long tiles = static_cast<long long>(gp.tiles_m) * gp.tiles_n;
  const unsigned grid = static_cast<unsigned>(tiles < nd.sm_count ? tiles : nd.sm_count);
  gemm_tf32_kernel<MODE><<<grid, GEMM_THREADS, Cfg::kSmemBytes, st>>>(ma_hi, mb_hi, ma_lo, mb_lo, gp);
  return launch_check("gemm_tf32_kernel");
}

}  // namespace

extern "C" int sb200_gemm_f32_noalloc(int dev, uint64_t stream, int mode, int64_t M, int64_t N, int64_t K, uint64_t A,
                                      int64_t lda, uint64_t B, int64_t ldb, uint64_t D, int64_t ldd, float alpha, uint64_t C,
                                      int64_t ldc, float beta, uint64_t bias, int act) {
  if (mode != SB200_MODE_3XTF32 && mode != SB200_MODE_TF32) return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (M < 0 || N < 0 || K < 0) return fail(SB200_ERR_INVALID_VALUE, "negative GEMM dimension (M=%lld N=%lld K=%lld)",
                                           (long long)M, (long long)N, (long long)K);
  if (act != SB200_ACT_NONE && act != SB200_ACT_RELU) return fail(SB200_ERR_INVALID_VALUE, "unknown activation %d", act);
  if (M > 0 && N > 0 && K > 0) {
    if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24))
      return fail(SB200_ERR_TOO_LARGE, "GEMM dimension beyond the fixed scratch (M=%lld N=%lld K=%lld)", (long long)M,
                  (long long)N, (long long)K);
    const size_t need = gemm_workspace_need(mode, M, N, K);
    if (need > kNoAllocScratchBytes)
      return fail(SB200_ERR_TOO_LARGE,
                  "this problem needs %zu bytes of operand panels but the allocation-free entry point has a fixed %zu-byte "
                  "scratch; use sb200_gemm_f32 or a smaller problem",
                  need, kNoAllocScratchBytes);
  }
  if (M == 0 || N == 0) return SB200_OK;
  if (!D || (K > 0 && (!A || !B))) return fail(SB200_ERR_INVALID_VALUE, "null device pointer passed to GEMM");
  if ((K > 0 && lda < K) || (K > 0 && ldb < N) || ldd < N || (C && ldc < N))
    return fail(SB200_ERR_INVALID_VALUE, "leading dimension smaller than the row length");
  if ((A | B | C | D | bias) & 3) return fail(SB200_ERR_ALIGNMENT, "float32 matrices must be 4-byte aligned");
  NoAllocDevice* nd;
  int rc = noalloc_setup(dev, &nd);
  if (rc) return rc;
  {
    // operands inside buffers from sb200_mem_alloc must end inside them (a table lookup: allocates nothing)
    DeviceState& ds = g_dev[dev];
    auto extent = [](long long rows, long long cols, long long ld) { return static_cast<uint64_t>((rows - 1) * ld + cols) * 4; };
    if (K > 0 && ((rc = check_extent(ds, A, extent(M, K, lda), "GEMM operand A")) ||
                  (rc = check_extent(ds, B, extent(K, N, ldb), "GEMM operand B"))))
      return rc;
    if ((rc = check_extent(ds, D, extent(M, N, ldd), "GEMM result D")) || (rc = check_extent(ds, C, extent(M, N, ldc), "GEMM operand C")) ||
        (rc = check_extent(ds, bias, static_cast<uint64_t>(N) * 4, "GEMM bias")))
      return rc;
  }
  cudaStream_t st = as_stream(stream);
  GemmParams gp;
  memset(&gp, 0, sizeof gp);
  gp.M = static_cast<int>(M);
  gp.N = static_cast<int>(N);
  gp.D = as_ptr<float>(D);
  gp.ldd = ldd;
  gp.C = as_ptr<const float>(C);
  gp.ldc = ldc;
  gp.bias = as_ptr<const float>(bias);
  gp.alpha = alpha;
  gp.beta = beta;
  gp.act = act;
  gp.status = nd->status;
  if (K == 0) {
    long long grid = (M * N + 255) / 256;
    const long long cap = static_cast<long long>(nd->sm_count) * 16;
    if (grid > cap) grid = cap;
    gemm_k0_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(gp);
    rc = launch_check("gemm_k0_kernel");
  } else if (mode == SB200_MODE_3XTF32) {
    rc = launch_gemm_fixed_scratch<3>(*nd, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  } else {
    rc = launch_gemm_fixed_scratch<1>(*nd, st, M, N, K, as_ptr<const float>(A), lda, as_ptr<const float>(B), ldb, gp);
  }
  if (rc) return rc;
  CU_TRY(cudaStreamSynchronize(st));
  int flag = 0;
  CU_TRY(cudaMemcpy(&flag, nd->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag != 0) {
    CU_TRY(cudaMemset(nd->status, 0, sizeof(int)));
    return fail(SB200_ERR_TIMEOUT, "a bounded device-side wait expired in the GEMM pipeline (site 0x%x)", flag);
  }
  return SB200_OK;
}

// ---------------------------------------------------------------------------
// GEMM on host operands, transfers pipelined with compute
// ---------------------------------------------------------------------------
// The reference moves whole vectors with synchronous copies before and after a
// launch (sarek/core/Transfer.ml:229-322: to_device, kernel, to_cpu).  Here the
// same end-to-end operation is one call that overlaps the three phases: B and
// the bias go first; A and C then stream in by row blocks on one stream while
// a second stream runs the GEMM of the blocks that have arrived and a third
// copies finished blocks of D back (PCIe carries both directions at once).
// B's panels are prepared once and reused by every row block.
extern "C" int sb200_gemm_f32_host(int dev, int mode, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                                   const float* B, int64_t ldb, float* D, int64_t ldd, float alpha, const float* C,
                                   int64_t ldc, float beta, const float* bias, int act) {
  if (!sb200::valid_mode(mode))
    return fail(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (M < 0 || N < 0 || K < 0) return fail(SB200_ERR_INVALID_VALUE, "negative GEMM dimension");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL - 64) return fail(SB200_ERR_TOO_LARGE, "GEMM dimension beyond 2^31-1");
  if (act != SB200_ACT_NONE && act != SB200_ACT_RELU) return fail(SB200_ERR_INVALID_VALUE, "unknown activation %d", act);
  if (M == 0 || N == 0) return SB200_OK;
  if (!D || (K > 0 && (!A || !B))) return fail(SB200_ERR_INVALID_VALUE, "null host pointer passed to GEMM");
  if ((K > 0 && lda < K) || (K > 0 && ldb < N) || ldd < N || (C && ldc < N))
    return fail(SB200_ERR_INVALID_VALUE, "leading dimension smaller than the row length");
  DeviceState* d;
  int rc = device_ready(dev, &d);
  if (rc) return rc;
  std::lock_guard<std::mutex> host_call_lock(d->host_call_mu);
  if ((rc = ensure_pipe_streams(*d))) return rc;
  // device mirrors, packed: A[M x K], B[K x N], C[M x N] (if any), D[M x N], bias[N]
  auto al = [](size_t b) { return (b + 255) / 256 * 256; };
  const size_t szA = al(size_t(M) * K * 4), szB = al(size_t(K) * N * 4), szC = C ? al(size_t(M) * N * 4) : 0,
               szD = al(size_t(M) * N * 4), szBias = bias ? al(size_t(N) * 4) : 0;
  const size_t need = szA + szB + szC + szD + szBias + 256;
  if (need > d->host_stage_bytes) {
    if (d->host_stage) {
      CU_TRY(cudaDeviceSynchronize());
      CU_TRY(cudaFree(d->host_stage));
      d->host_stage = nullptr;
      d->host_stage_bytes = 0;
    }
    CU_TRY(cudaMalloc(&d->host_stage, need));
    d->host_stage_bytes = need;
  }
  uint8_t* base = static_cast<uint8_t*>(d->host_stage);
  float* dA = reinterpret_cast<float*>(base);
  float* dB = reinterpret_cast<float*>(base + szA);
  float* dC = C ? reinterpret_cast<float*>(base + szA + szB) : nullptr;
  float* dD = reinterpret_cast<float*>(base + szA + szB + szC);
  float* dBias = bias ? reinterpret_cast<float*>(base + szA + szB + szC + szD) : nullptr;

  // row blocks, multiples of 256 rows so that block edges are tile edges: about eight equal ones, the last of
  // them halved down to 256 rows, because what follows the last inbound copy — that block's GEMM and its
  // copy back — is the part of the call that nothing overlaps
  long long block_rows = (M + 7) / 8;
  block_rows = (block_rows + 255) / 256 * 256;
  if (block_rows > M) block_rows = M;
  std::vector<std::pair<long long, long long>> blocks;  // (first row, rows)
  {
    long long r = 0;
    while (M - r > block_rows) {
      blocks.emplace_back(r, block_rows);
      r += block_rows;
    }
    long long rem = M - r;
    while (rem > 256) {
      const long long h = (rem / 2 + 255) / 256 * 256;
      if (h >= rem) break;
      blocks.emplace_back(r, h);
      r += h;
      rem -= h;
    }
    if (rem > 0) blocks.emplace_back(r, rem);
  }
  const int nblocks = static_cast<int>(blocks.size());

  // Pageable host operands (what a Bigarray is): asynchronous copies from pageable memory are neither
  // asynchronous nor fast, so such a call moves its operands with the staged copier instead — several host
  // threads through pinned slots — block by block, synchronously for the host, while the GEMM of the block
  // before runs on the compute stream.  Needs contiguous rows; strided pageable operands take the plain path.
  const bool contiguous = (K == 0 || (lda == K && ldb == N)) && ldd == N && (!C || ldc == N);
  const bool any_pageable = staged_copy_enabled() && contiguous &&
                            ((K > 0 && (host_memory_is_pageable(A) || host_memory_is_pageable(B))) ||
                             (C && host_memory_is_pageable(C)) || host_memory_is_pageable(D));
  if (any_pageable) {
    auto copy_in = [&](void* dst, const void* src, size_t bytes) -> int {
      if (bytes == 0) return 0;
      if (bytes >= (size_t(1) << 20) && host_memory_is_pageable(src)) return staged_copy_to_device(dev, dst, src, bytes, false);
      // a copy from pageable memory may return once the data is staged, before the DMA has landed, and the
      // compute stream is non-blocking: wait for the legacy stream so that the kernel cannot read early
      cudaError_t ce = cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
      if (ce == cudaSuccess) ce = cudaStreamSynchronize(0);
      return static_cast<int>(ce);
    };
    auto copy_out = [&](void* dst, const void* src, size_t bytes) -> int {
      if (bytes == 0) return 0;
      if (bytes >= (size_t(1) << 20) && host_memory_is_pageable(dst)) return staged_copy_to_host(dev, dst, src, bytes, false);
      return static_cast<int>(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    };
    std::vector<cudaEvent_t> done(nblocks, nullptr);
    std::thread* out_thread_ptr = nullptr;
    auto finish = [&](int code, const char* what) -> int {
      if (out_thread_ptr && out_thread_ptr->joinable()) out_thread_ptr->join();
      cudaDeviceSynchronize();
      for (auto e : done) if (e) cudaEventDestroy(e);
      if (code > 0) return cuda_fail(static_cast<cudaError_t>(code), what);
      return code;
    };
    std::atomic<int> out_error{0};
    std::thread out_thread;
    out_thread_ptr = &out_thread;
    auto copy_block_out = [&](int blk) {
      cudaSetDevice(dev);
      int oe = static_cast<int>(cudaEventSynchronize(done[blk]));
      const long long p0 = blocks[blk].first, prows = blocks[blk].second;
      if (!oe) oe = copy_out(D + p0 * N, dD + p0 * N, size_t(prows) * N * 4);
      if (oe) out_error.store(oe);
    };
    int e = 0;
    if (K > 0 && (e = copy_in(dB, B, size_t(K) * N * 4))) return finish(e, "copy of B");
    if (bias && (e = copy_in(dBias, bias, size_t(N) * 4))) return finish(e, "copy of bias");
    for (int i = 0; i < nblocks; ++i) {
      const long long r0 = blocks[i].first, rows = blocks[i].second;
      if (K > 0 && (e = copy_in(dA + r0 * K, A + r0 * K, size_t(rows) * K * 4))) return finish(e, "copy of an A block");
      if (C && (e = copy_in(dC + r0 * N, C + r0 * N, size_t(rows) * N * 4))) return finish(e, "copy of a C block");
      GemmParams gp;
      memset(&gp, 0, sizeof gp);
      gp.M = static_cast<int>(rows);
      gp.N = static_cast<int>(N);
      gp.D = dD + r0 * N;
      gp.ldd = N;
      gp.C = dC ? dC + r0 * N : nullptr;
      gp.ldc = N;
      gp.bias = dBias;
      gp.alpha = alpha;
      gp.beta = beta;
      gp.act = act;
      if (K == 0) {
        long long grid = (rows * N + 255) / 256;
        const long long cap = static_cast<long long>(d->sm_count) * 16;
        if (grid > cap) grid = cap;
        gemm_k0_kernel<<<static_cast<unsigned>(grid), 256, 0, d->pipe_compute>>>(gp);
        rc = launch_check("gemm_k0_kernel");
      } else if (mode == SB200_MODE_3XF16) {  // fp16 panels are prepared per row block (B's with every block)
        rc = launch_gemm_f16<true>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
      } else if (mode == SB200_MODE_F16) {
        rc = launch_gemm_f16<false>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
      } else if (mode == SB200_MODE_3XMIXED && gemm_mix_applies(rows, N, K, operands_addressable(dA + r0 * K, K, dB, N))) {
        rc = launch_gemm_mix(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
      } else if (mode == SB200_MODE_3XTF32 || mode == SB200_MODE_3XMIXED) {
        // a block the mixed mode leaves to 3xTF32 finds the scratch holding fp16 panels: B's low parts are made anew
        rc = launch_gemm_mode<3>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp, block_rows,
                                 mode == SB200_MODE_3XTF32 && i > 0);
      } else {
        rc = launch_gemm_mode<1>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp, block_rows, i > 0);
      }
      if (rc) return finish(rc, "");
      if ((e = static_cast<int>(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming)))) return finish(e, "event");
      if ((e = static_cast<int>(cudaEventRecord(done[i], d->pipe_compute)))) return finish(e, "event");
      // the block before goes back on a thread of its own, beside the next block's copies in
      if (out_thread.joinable()) out_thread.join();
      if (out_error.load()) return finish(out_error.load(), "copy of a D block");
      if (i > 0) out_thread = std::thread(copy_block_out, i - 1);
    }
    if (out_thread.joinable()) out_thread.join();
    if (out_error.load()) return finish(out_error.load(), "copy of a D block");
    copy_block_out(nblocks - 1);
    if (out_error.load()) return finish(out_error.load(), "copy of a D block");
    rc = finish(0, "");
    return rc ? rc : check_status_word(*d);
  }

  std::vector<cudaEvent_t> ev_in(nblocks), ev_done(nblocks);
  cudaEvent_t ev_b = nullptr;
  auto cleanup = [&]() {
    if (ev_b) cudaEventDestroy(ev_b);
    for (auto e : ev_in) if (e) cudaEventDestroy(e);
    for (auto e : ev_done) if (e) cudaEventDestroy(e);
  };
  for (auto& e : ev_in) e = nullptr;
  for (auto& e : ev_done) e = nullptr;
#define PIPE_TRY(call)                          \
  do {                                          \
    cudaError_t e__ = (call);                   \
    if (e__ != cudaSuccess) {                   \
      cudaDeviceSynchronize();                  \
      cleanup();                                \
      return cuda_fail(e__, #call);             \
    }                                           \
  } while (0)
  PIPE_TRY(cudaEventCreateWithFlags(&ev_b, cudaEventDisableTiming));
  for (int i = 0; i < nblocks; ++i) {
    PIPE_TRY(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
    PIPE_TRY(cudaEventCreateWithFlags(&ev_done[i], cudaEventDisableTiming));
  }
  // inbound stream: B and bias first, then the row blocks of A and C
  if (K > 0) PIPE_TRY(cudaMemcpy2DAsync(dB, size_t(N) * 4, B, size_t(ldb) * 4, size_t(N) * 4, size_t(K), cudaMemcpyHostToDevice, d->pipe_in));
  if (bias) PIPE_TRY(cudaMemcpyAsync(dBias, bias, size_t(N) * 4, cudaMemcpyHostToDevice, d->pipe_in));
  PIPE_TRY(cudaEventRecord(ev_b, d->pipe_in));
  for (int i = 0; i < nblocks; ++i) {
    const long long r0 = blocks[i].first, rows = blocks[i].second;
    if (K > 0)
      PIPE_TRY(cudaMemcpy2DAsync(dA + r0 * K, size_t(K) * 4, A + r0 * lda, size_t(lda) * 4, size_t(K) * 4, size_t(rows),
                                 cudaMemcpyHostToDevice, d->pipe_in));
    if (C)
      PIPE_TRY(cudaMemcpy2DAsync(dC + r0 * N, size_t(N) * 4, C + r0 * ldc, size_t(ldc) * 4, size_t(N) * 4, size_t(rows),
                                 cudaMemcpyHostToDevice, d->pipe_in));
    PIPE_TRY(cudaEventRecord(ev_in[i], d->pipe_in));
  }
  // compute stream: one GEMM per row block, B's panels prepared by the first
  PIPE_TRY(cudaStreamWaitEvent(d->pipe_compute, ev_b, 0));
  for (int i = 0; i < nblocks && rc == SB200_OK; ++i) {
    const long long r0 = blocks[i].first, rows = blocks[i].second;
    PIPE_TRY(cudaStreamWaitEvent(d->pipe_compute, ev_in[i], 0));
    GemmParams gp;
    memset(&gp, 0, sizeof gp);
    gp.M = static_cast<int>(rows);
    gp.N = static_cast<int>(N);
    gp.D = dD + r0 * N;
    gp.ldd = N;
    gp.C = dC ? dC + r0 * N : nullptr;
    gp.ldc = N;
    gp.bias = dBias;
    gp.alpha = alpha;
    gp.beta = beta;
    gp.act = act;
    if (K == 0) {
      long long grid = (rows * N + 255) / 256;
      const long long cap = static_cast<long long>(d->sm_count) * 16;
      if (grid > cap) grid = cap;
      gemm_k0_kernel<<<static_cast<unsigned>(grid), 256, 0, d->pipe_compute>>>(gp);
      rc = launch_check("gemm_k0_kernel");
    } else if (mode == SB200_MODE_3XF16) {
      rc = launch_gemm_f16<true>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
    } else if (mode == SB200_MODE_F16) {
      rc = launch_gemm_f16<false>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
    } else if (mode == SB200_MODE_3XMIXED && gemm_mix_applies(rows, N, K, operands_addressable(dA + r0 * K, K, dB, N))) {
      rc = launch_gemm_mix(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp);
    } else if (mode == SB200_MODE_3XTF32 || mode == SB200_MODE_3XMIXED) {
      rc = launch_gemm_mode<3>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp, block_rows,
                               mode == SB200_MODE_3XTF32 && i > 0);
    } else {
      rc = launch_gemm_mode<1>(*d, d->pipe_compute, rows, N, K, dA + r0 * K, K, dB, N, gp, block_rows, i > 0);
    }
    if (rc == SB200_OK) PIPE_TRY(cudaEventRecord(ev_done[i], d->pipe_compute));
    // outbound stream: the finished block of D
    if (rc == SB200_OK) {
      PIPE_TRY(cudaStreamWaitEvent(d->pipe_out, ev_done[i], 0));
      PIPE_TRY(cudaMemcpy2DAsync(D + r0 * ldd, size_t(ldd) * 4, dD + r0 * N, size_t(N) * 4, size_t(N) * 4, size_t(rows),
                                 cudaMemcpyDeviceToHost, d->pipe_out));
    }
  }
  cudaError_t e1 = cudaStreamSynchronize(d->pipe_in), e2 = cudaStreamSynchronize(d->pipe_compute),
              e3 = cudaStreamSynchronize(d->pipe_out);
  cleanup();
#undef PIPE_TRY
  if (rc) return rc;
  if (e1 != cudaSuccess) return cuda_fail(e1, "inbound copies");
  if (e2 != cudaSuccess) return cuda_fail(e2, "GEMM row blocks");
  if (e3 != cudaSuccess) return cuda_fail(e3, "outbound copies");
  return check_status_word(*d);
}
