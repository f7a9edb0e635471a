// sb200_group.cu — one host process driving several GPUs: device groups and the row-sharded GEMM.
//
// The reference's host is a single OCaml process whose multi-device model is "partition the vector, launch
// once per device" (sarek/core/Vector.ml:273-296 with the split rule of sarek/core/Vector_storage.ml:261-272;
// peer access is bound but never used, sarek-cuda/Cuda_bindings.ml:472-493).  This file is that model for the
// GEMM path, inside the library: a group owns one stream set per GPU and, for more than one GPU, an NCCL
// communicator per GPU (ncclCommInitAll, NCCL loaded with dlopen when the first multi-GPU group is made).
// A sharded product splits the rows of A, C and D by the reference's rule, replicates B and the bias from the
// first GPU into each GPU's own memory with ncclBroadcast, runs the per-device operator (sb200_gemm_f32) on
// every GPU's stream, and leaves the result either as row blocks, or gathered on every GPU — by the GEMM
// epilogue's own stores into the peers' copies (sb200_gemm_f32_gather; peer access enabled between the
// group's GPUs) or by NCCL (in-place all-gather, or one broadcast per block when the blocks differ in size).
// Only this library's kernels store to peer memory, with plain stores; no library kernel is handed a peer
// pointer, and every TMA load in the library reads the issuing GPU's own memory into the issuing block.
//
// Everything here is built from the public per-device entry points, so a group of one GPU behaves exactly
// as those do.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <unordered_set>
#include <vector>

#include "../../include/sb200.h"
#include "internal.hpp"
#include "transfer.hpp"

using sb200::set_error;

namespace {

constexpr int kMaxGroup = 8;

// ---- NCCL through dlopen: the library has no link-time dependency on it -------------------------------
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle) return SB200_OK;
  // One NCCL per process: a copy that the host program has already loaded (a framework's bundled one, say) is
  // taken as it is; otherwise SAREK_B200_NCCL names the file, and the system's libnccl.so.2 is the default.
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) {
    const char* named = getenv("SAREK_B200_NCCL");
    if (named && *named) h = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
  }
  for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
    if (h) break;
    h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
  }
  if (!h) return set_error(SB200_ERR_COMM, "NCCL is needed for a group of more than one GPU and could not be loaded: %s", dlerror());
  NcclApi api;
  api.handle = h;
  bool ok = true;
  auto sym = [&](const char* n) {
    void* p = dlsym(h, n);
    if (!p) ok = false;
    return p;
  };
  api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
  api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
  api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
  api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  if (!ok) return set_error(SB200_ERR_COMM, "the NCCL library that was found lacks an entry point this library uses");
  g_nccl = api;
  return SB200_OK;
}

#define GCU_TRY(call)                                                                                             \
  do {                                                                                                            \
    cudaError_t e__ = (call);                                                                                     \
    if (e__ != cudaSuccess) {                                                                                     \
      cudaGetLastError();                                                                                         \
      return set_error(static_cast<int>(e__), "%s: %s (%s)", #call, cudaGetErrorString(e__), cudaGetErrorName(e__)); \
    }                                                                                                             \
  } while (0)

#define NCCL_TRY(call)                                                                           \
  do {                                                                                           \
    ncclResult_t r__ = (call);                                                                   \
    if (r__ != ncclSuccess) return set_error(SB200_ERR_COMM, "%s: %s", #call, g_nccl.GetErrorString(r__)); \
  } while (0)

struct Buf {  // grow-only device buffer
  void* p = nullptr;
  size_t bytes = 0;
};

struct Group {
  int n = 0;
  int dev[kMaxGroup];
  ncclComm_t comm[kMaxGroup];
  cudaStream_t s_main[kMaxGroup], s_in[kMaxGroup], s_out[kMaxGroup];
  cudaEvent_t ev0[kMaxGroup], ev1[kMaxGroup];
  bool peer_ok = true;   // every GPU of the group can store into every other's memory
  Buf b_rep[kMaxGroup];  // replicas of B and bias on the GPUs other than the first
  Buf bias_rep[kMaxGroup];
  uint64_t rep_b_src = 0, rep_bias_src = 0;  // what the replicas currently hold (for SB200_SHARD_B_RESIDENT)
  size_t rep_b_bytes = 0;
  Buf stage[kMaxGroup];  // host-operand form: device mirrors of the operands
  float last_ms = 0.f;
  std::mutex mu;  // one call per group at a time
};

std::mutex g_groups_mu;
std::unordered_set<Group*> g_groups;

Group* find_group(uint64_t h) {
  Group* g = reinterpret_cast<Group*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lock(g_groups_mu);
  return g_groups.count(g) ? g : nullptr;
}

int grow(Buf* b, size_t bytes) {
  if (bytes <= b->bytes) return SB200_OK;
  if (b->p) {
    GCU_TRY(cudaDeviceSynchronize());
    GCU_TRY(cudaFree(b->p));
    b->p = nullptr;
    b->bytes = 0;
  }
  GCU_TRY(cudaMalloc(&b->p, bytes));
  b->bytes = bytes;
  return SB200_OK;
}

// The reference's split rule: the first (total mod parts) parts get one more (sarek/core/Vector_storage.ml:261-272).
void split(int64_t total, int parts, int index, int64_t* first, int64_t* count) {
  const int64_t base = total / parts, rem = total % parts;
  *count = base + (index < rem ? 1 : 0);
  *first = base * index + (index < rem ? index : rem);
}

void release(Group* g) {
  for (int i = 0; i < g->n; ++i) {
    if (cudaSetDevice(g->dev[i]) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    if (g->comm[i]) g_nccl.CommDestroy(g->comm[i]);
    for (cudaStream_t s : {g->s_main[i], g->s_in[i], g->s_out[i]})
      if (s) cudaStreamDestroy(s);
    for (cudaEvent_t e : {g->ev0[i], g->ev1[i]})
      if (e) cudaEventDestroy(e);
    for (Buf* b : {&g->b_rep[i], &g->bias_rep[i], &g->stage[i]})
      if (b->p) cudaFree(b->p);
  }
  cudaGetLastError();
}

}  // namespace

extern "C" {

int sb200_group_create(int ngpus, const int* devices, uint64_t* group) {
  if (!group) return set_error(SB200_ERR_INVALID_VALUE, "null group pointer");
  *group = 0;
  if (ngpus < 1 || ngpus > kMaxGroup)
    return set_error(SB200_ERR_INVALID_VALUE, "a group has between 1 and %d GPUs, not %d", kMaxGroup, ngpus);
  int count = 0;
  int rc = sb200_device_count(&count);
  if (rc) return rc;
  if (count == 0) return set_error(SB200_ERR_NO_DEVICE, "no sm_100 device available");
  int dev[kMaxGroup];
  for (int i = 0; i < ngpus; ++i) {
    dev[i] = devices ? devices[i] : i;
    if (dev[i] < 0 || dev[i] >= count)
      return set_error(SB200_ERR_INVALID_VALUE, "group member %d is device %d but %d device(s) are usable", i, dev[i], count);
    for (int j = 0; j < i; ++j)
      if (dev[j] == dev[i]) return set_error(SB200_ERR_INVALID_VALUE, "device %d appears twice in the group", dev[i]);
  }
  if (ngpus > 1 && (rc = load_nccl())) return rc;
  Group* g = new Group();
  g->n = ngpus;
  for (int i = 0; i < kMaxGroup; ++i) {
    g->dev[i] = i < ngpus ? dev[i] : -1;
    g->comm[i] = nullptr;
    g->s_main[i] = g->s_in[i] = g->s_out[i] = nullptr;
    g->ev0[i] = g->ev1[i] = nullptr;
  }
  auto bail = [&](int code) {
    release(g);
    delete g;
    return code;
  };
  for (int i = 0; i < ngpus; ++i) {
    if ((rc = sb200_device_set_current(dev[i]))) return bail(rc);
    cudaError_t e = cudaStreamCreateWithFlags(&g->s_main[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g->s_in[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g->s_out[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&g->ev0[i]);
    if (e == cudaSuccess) e = cudaEventCreate(&g->ev1[i]);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return bail(set_error(static_cast<int>(e), "creating the streams of device %d: %s", dev[i], cudaGetErrorString(e)));
    }
    // peer access for the fused gather: this GPU's kernels store into the other members' memory
    for (int j = 0; j < ngpus; ++j) {
      if (j == i) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, dev[i], dev[j]) != cudaSuccess || !can) {
        cudaGetLastError();
        g->peer_ok = false;
        continue;
      }
      e = cudaDeviceEnablePeerAccess(dev[j], 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) g->peer_ok = false;
      cudaGetLastError();
    }
  }
  if (ngpus > 1) {
    ncclResult_t r = g_nccl.CommInitAll(g->comm, ngpus, dev);
    if (r != ncclSuccess) return bail(set_error(SB200_ERR_COMM, "ncclCommInitAll: %s", g_nccl.GetErrorString(r)));
  }
  {
    std::lock_guard<std::mutex> lock(g_groups_mu);
    g_groups.insert(g);
  }
  *group = reinterpret_cast<uintptr_t>(g);
  return SB200_OK;
}

int sb200_group_destroy(uint64_t group) {
  Group* g = reinterpret_cast<Group*>(static_cast<uintptr_t>(group));
  {
    std::lock_guard<std::mutex> lock(g_groups_mu);
    if (!g_groups.erase(g)) return group ? set_error(SB200_ERR_INVALID_HANDLE, "unknown group") : SB200_OK;
  }
  release(g);
  delete g;
  return SB200_OK;
}

int sb200_group_size(uint64_t group, int* ngpus) {
  Group* g = find_group(group);
  if (!g || !ngpus) return set_error(SB200_ERR_INVALID_HANDLE, "unknown group");
  *ngpus = g->n;
  return SB200_OK;
}

int sb200_group_device(uint64_t group, int index, int* dev) {
  Group* g = find_group(group);
  if (!g || !dev) return set_error(SB200_ERR_INVALID_HANDLE, "unknown group");
  if (index < 0 || index >= g->n) return set_error(SB200_ERR_INVALID_VALUE, "group member %d of %d", index, g->n);
  *dev = g->dev[index];
  return SB200_OK;
}

int sb200_row_block(int64_t total, int parts, int index, int64_t* first, int64_t* count) {
  if (!first || !count || total < 0 || parts < 1 || index < 0 || index >= parts)
    return set_error(SB200_ERR_INVALID_VALUE, "row block %d of %d parts of %lld rows", index, parts, static_cast<long long>(total));
  split(total, parts, index, first, count);
  return SB200_OK;
}

int sb200_group_last_ms(uint64_t group, float* ms) {
  Group* g = find_group(group);
  if (!g || !ms) return set_error(SB200_ERR_INVALID_HANDLE, "unknown group");
  *ms = g->last_ms;
  return SB200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Row-sharded GEMM on device-resident operands
// ---------------------------------------------------------------------------------------------------
namespace {

inline uint64_t h(cudaStream_t s) { return reinterpret_cast<uintptr_t>(s); }

// Replicates `count` floats from the first member's `src` into each other member's replica buffer and
// enqueues the broadcast on every member's main stream; ptr_out[i] is the copy member i reads.
int replicate(Group* g, uint64_t src, size_t count, Buf* reps, uint64_t* ptr_out, bool resident) {
  ptr_out[0] = src;
  if (!src || count == 0) {
    for (int i = 1; i < g->n; ++i) ptr_out[i] = 0;
    return SB200_OK;
  }
  for (int i = 1; i < g->n; ++i) {
    GCU_TRY(cudaSetDevice(g->dev[i]));
    int rc = grow(&reps[i], count * 4);
    if (rc) return rc;
    ptr_out[i] = reinterpret_cast<uintptr_t>(reps[i].p);
  }
  if (resident || g->n == 1) return SB200_OK;
  NCCL_TRY(g_nccl.GroupStart());
  for (int i = 0; i < g->n; ++i) {
    void* buf = reinterpret_cast<void*>(static_cast<uintptr_t>(ptr_out[i]));
    ncclResult_t r = g_nccl.Broadcast(buf, buf, count, ncclFloat, 0, g->comm[i], g->s_main[i]);
    if (r != ncclSuccess) {
      g_nccl.GroupEnd();
      return set_error(SB200_ERR_COMM, "ncclBroadcast: %s", g_nccl.GetErrorString(r));
    }
  }
  NCCL_TRY(g_nccl.GroupEnd());
  return SB200_OK;
}

int finish(Group* g) {
  int first_rc = SB200_OK;
  for (int i = 0; i < g->n; ++i) {
    cudaSetDevice(g->dev[i]);
    cudaEventRecord(g->ev1[i], g->s_main[i]);
  }
  float worst = 0.f;
  for (int i = 0; i < g->n; ++i) {
    int rc = sb200_stream_synchronize(g->dev[i], h(g->s_main[i]));  // also reports a device-side wait that ran out
    if (rc && !first_rc) first_rc = rc;
    float ms = 0.f;
    if (!rc && cudaEventElapsedTime(&ms, g->ev0[i], g->ev1[i]) == cudaSuccess && ms > worst) worst = ms;
    cudaGetLastError();
  }
  g->last_ms = worst;
  return first_rc;
}

}  // namespace

extern "C" int sb200_gemm_sharded(uint64_t group, int mode, int64_t M, int64_t N, int64_t K, const uint64_t* a_shards,
                                  int64_t lda, uint64_t b, int64_t ldb, const uint64_t* d, int64_t ldd, float alpha,
                                  const uint64_t* c_shards, int64_t ldc, float beta, uint64_t bias, int act, int flags) {
  Group* g = find_group(group);
  if (!g) return set_error(SB200_ERR_INVALID_HANDLE, "unknown group");
  if (M < 0 || N < 0 || K < 0) return set_error(SB200_ERR_INVALID_VALUE, "negative GEMM dimension");
  if (!a_shards || !d) return set_error(SB200_ERR_INVALID_VALUE, "null shard table");
  if (flags & ~(SB200_SHARD_GATHER_FUSED | SB200_SHARD_GATHER_NCCL | SB200_SHARD_B_RESIDENT))
    return set_error(SB200_ERR_INVALID_VALUE, "unknown flag bits 0x%x", flags);
  if ((flags & SB200_SHARD_GATHER_FUSED) && (flags & SB200_SHARD_GATHER_NCCL))
    return set_error(SB200_ERR_INVALID_VALUE, "choose one way to gather the result");
  const bool gather = flags & (SB200_SHARD_GATHER_FUSED | SB200_SHARD_GATHER_NCCL);
  const bool fused = (flags & SB200_SHARD_GATHER_FUSED) != 0;
  const int n = g->n;
  if (n > 1) {
    if (K > 0 && ldb != N) return set_error(SB200_ERR_INVALID_VALUE, "B must be contiguous (ldb == N) to be broadcast");
    if ((flags & SB200_SHARD_GATHER_NCCL) && ldd != N)
      return set_error(SB200_ERR_INVALID_VALUE, "D must be contiguous (ldd == N) to be gathered by NCCL");
    if (fused && !g->peer_ok)
      return set_error(SB200_ERR_UNSUPPORTED, "the group's GPUs cannot all store into each other's memory; gather with NCCL instead");
  }
  std::lock_guard<std::mutex> lock(g->mu);
  for (int i = 0; i < n; ++i) {
    GCU_TRY(cudaSetDevice(g->dev[i]));
    GCU_TRY(cudaEventRecord(g->ev0[i], g->s_main[i]));
  }
  if (M == 0 || N == 0) return finish(g);
  // B and the bias: from the first GPU into every GPU's own memory
  uint64_t b_at[kMaxGroup], bias_at[kMaxGroup];
  const size_t b_count = static_cast<size_t>(K) * static_cast<size_t>(N);
  const bool resident = (flags & SB200_SHARD_B_RESIDENT) && g->rep_b_src == b && g->rep_b_bytes == b_count * 4 &&
                        g->rep_bias_src == bias;
  int rc = replicate(g, K > 0 ? b : 0, b_count, g->b_rep, b_at, resident);
  if (!rc) rc = replicate(g, bias, static_cast<size_t>(N), g->bias_rep, bias_at, resident);
  if (rc) {
    finish(g);
    return rc;
  }
  g->rep_b_src = b;
  g->rep_b_bytes = b_count * 4;
  g->rep_bias_src = bias;
  // the row blocks
  int64_t first[kMaxGroup], rows[kMaxGroup];
  for (int i = 0; i < n; ++i) split(M, n, i, &first[i], &rows[i]);
  for (int i = 0; i < n && !rc; ++i) {
    if (rows[i] == 0) continue;
    const uint64_t c_i = c_shards ? c_shards[i] : 0;
    if (!d[i] || (K > 0 && !a_shards[i])) {
      rc = set_error(SB200_ERR_INVALID_VALUE, "null shard pointer for group member %d", i);
      break;
    }
    if (gather && fused && n > 1) {
      uint64_t copies[kMaxGroup];
      copies[0] = d[i];
      int m = 1;
      for (int j = 0; j < n; ++j)
        if (j != i) copies[m++] = d[j];
      rc = sb200_gemm_f32_gather(g->dev[i], h(g->s_main[i]), mode, rows[i], N, K, a_shards[i], lda, b_at[i], ldb, copies, n,
                                 first[i], ldd, alpha, c_i, ldc, beta, bias_at[i], act);
    } else {
      const uint64_t d_i = gather ? d[i] + static_cast<uint64_t>(first[i]) * static_cast<uint64_t>(ldd) * 4 : d[i];
      rc = sb200_gemm_f32(g->dev[i], h(g->s_main[i]), mode, rows[i], N, K, a_shards[i], lda, b_at[i], ldb, d_i, ldd, alpha, c_i,
                          ldc, beta, bias_at[i], act);
    }
  }
  if (!rc && (flags & SB200_SHARD_GATHER_NCCL) && n > 1) {
    bool equal = true;
    for (int i = 1; i < n; ++i) equal = equal && rows[i] == rows[0];
    ncclResult_t r = g_nccl.GroupStart();
    for (int i = 0; i < n && r == ncclSuccess; ++i) {
      float* whole = reinterpret_cast<float*>(static_cast<uintptr_t>(d[i]));
      if (equal) {
        // row blocks of a row-major matrix are contiguous: the gather runs in place
        r = g_nccl.AllGather(whole + first[i] * N, whole, static_cast<size_t>(rows[i]) * N, ncclFloat, g->comm[i], g->s_main[i]);
      } else {
        for (int j = 0; j < n && r == ncclSuccess; ++j)
          if (rows[j] > 0)
            r = g_nccl.Broadcast(whole + first[j] * N, whole + first[j] * N, static_cast<size_t>(rows[j]) * N, ncclFloat, j,
                                 g->comm[i], g->s_main[i]);
      }
    }
    ncclResult_t r2 = g_nccl.GroupEnd();
    if (r == ncclSuccess) r = r2;
    if (r != ncclSuccess) rc = set_error(SB200_ERR_COMM, "gathering D: %s", g_nccl.GetErrorString(r));
  }
  const int rc2 = finish(g);
  return rc ? rc : rc2;
}

// ---------------------------------------------------------------------------------------------------
// Row-sharded GEMM on host operands
// ---------------------------------------------------------------------------------------------------
// What a single-process host with its data in host memory calls: B crosses PCIe once, a band of rows
// over each GPU's link, and is assembled everywhere over NVLink (ncclAllGather); every GPU pulls only its own rows of A and C
// and pushes only its own rows of D, over its own PCIe link, driven by a host thread of its own.  Within a
// GPU the rows move in a few chunks so that the copy in of one chunk, the GEMM of the one before and the
// copy out of the one before that overlap.  Pinned host memory (sb200_host_alloc) is copied asynchronously;
// contiguous pageable memory goes through the staged copier of transfer.cc.
#include <string>
#include <thread>

namespace {

struct HostCall {
  int mode;
  int64_t M, N, K;
  const float *A, *B, *C, *bias;
  float* D;
  int64_t lda, ldb, ldc, ldd;
  float alpha, beta;
  int act;
};

struct MemberResult {
  int rc = SB200_OK;
  std::string msg;
};

constexpr int kHostChunks = 4;

size_t al256(size_t b) { return (b + 255) / 256 * 256; }

// Host -> device copy of `rows` rows of `cols` floats (row strides in elements), ordered on `st`.
int copy_in(int dev, cudaStream_t st, float* dst, const float* src, int64_t rows, int64_t cols, int64_t src_ld, bool staged) {
  if (rows == 0 || cols == 0) return SB200_OK;
  if (staged && src_ld == cols) {
    GCU_TRY(cudaStreamSynchronize(st));
    const int e = sb200::staged_copy_to_device(dev, dst, src, static_cast<size_t>(rows) * cols * 4, false);
    if (e) return set_error(e, "staged copy to device %d failed: %s", dev, cudaGetErrorString(static_cast<cudaError_t>(e)));
    return SB200_OK;
  }
  GCU_TRY(cudaMemcpy2DAsync(dst, static_cast<size_t>(cols) * 4, src, static_cast<size_t>(src_ld) * 4, static_cast<size_t>(cols) * 4,
                            static_cast<size_t>(rows), cudaMemcpyHostToDevice, st));
  return SB200_OK;
}

// The row block of one member: B and the bias are already on their way on the member's main stream (the broadcast was
// enqueued there), so the GEMMs launched on that stream below follow their arrival.
void member_main(Group* g, int i, const HostCall* hc, int64_t first, int64_t rows, float* dB, float* dBias, float* dA, float* dC,
                 float* dD, MemberResult* out) {
  auto fail_here = [&](int rc) {
    out->rc = rc;
    out->msg = sb200_last_error_string();
  };
  const int dev = g->dev[i];
  cudaError_t e = cudaSetDevice(dev);
  if (e != cudaSuccess) return fail_here(set_error(static_cast<int>(e), "cudaSetDevice(%d): %s", dev, cudaGetErrorString(e)));
  const HostCall& c = *hc;
  const bool staged_a = sb200::staged_copy_enabled() && c.K > 0 && sb200::host_memory_is_pageable(c.A);
  const bool staged_c = sb200::staged_copy_enabled() && c.C && sb200::host_memory_is_pageable(c.C);
  const bool staged_d = sb200::staged_copy_enabled() && sb200::host_memory_is_pageable(c.D) && c.ldd == c.N;
  // Row chunks: four when anything goes through the staged copier (it wants large pieces); from page-locked memory
  // eight, and the last of them cut again into a half and two quarters, because the last chunk's GEMM and copy out
  // hide behind nothing (SAREK_B200_PIPE_TAPER=0: four equal chunks always).
  static const bool taper = [] {
    const char* e = getenv("SAREK_B200_PIPE_TAPER");
    return !(e && e[0] == '0');
  }();
  const bool fine = taper && !(staged_a || staged_c || staged_d);
  static const int fine_chunks = [] {  // SAREK_B200_GROUP_CHUNKS: chunks per GPU from page-locked memory (4..64)
    const char* e = getenv("SAREK_B200_GROUP_CHUNKS");
    const int v = e ? atoi(e) : 0;
    return v >= 4 && v <= 64 ? v : 2 * kHostChunks;
  }();
  const int nchunks = fine ? fine_chunks : kHostChunks;
  int64_t chunk = (rows + nchunks - 1) / nchunks;
  chunk = (chunk + 255) / 256 * 256;  // chunk edges on tile edges
  if (chunk <= 0) chunk = 256;
  std::vector<int64_t> cuts;  // first row of every chunk, then `rows`
  {
    int64_t r = 0;
    while (rows - r > chunk) {
      cuts.push_back(r);
      r += chunk;
    }
    for (int split = 0; split < 2 && fine && rows - r >= 512; ++split) {
      cuts.push_back(r);
      r += ((rows - r) / 2 + 255) / 256 * 256;
    }
    if (r < rows) cuts.push_back(r);
    cuts.push_back(rows);
  }
  std::vector<cudaEvent_t> ev_in, ev_done;
  auto cleanup = [&] {
    cudaStreamSynchronize(g->s_in[i]);
    cudaStreamSynchronize(g->s_main[i]);
    cudaStreamSynchronize(g->s_out[i]);
    for (auto ev : ev_in) cudaEventDestroy(ev);
    for (auto ev : ev_done) cudaEventDestroy(ev);
    cudaGetLastError();
  };
  int rc = SB200_OK;
  auto copy_out = [&](int64_t r0, int64_t nr, cudaEvent_t done) -> int {
    float* dst = c.D + (first + r0) * c.ldd;
    const float* src = dD + r0 * c.N;
    if (staged_d) {
      cudaError_t ce = cudaEventSynchronize(done);
      if (ce != cudaSuccess) return set_error(static_cast<int>(ce), "waiting for a row chunk on device %d", dev);
      const int se = sb200::staged_copy_to_host(dev, dst, src, static_cast<size_t>(nr) * c.N * 4, false);
      if (se) return set_error(se, "staged copy from device %d failed: %s", dev, cudaGetErrorString(static_cast<cudaError_t>(se)));
      return SB200_OK;
    }
    GCU_TRY(cudaStreamWaitEvent(g->s_out[i], done, 0));
    GCU_TRY(cudaMemcpy2DAsync(dst, static_cast<size_t>(c.ldd) * 4, src, static_cast<size_t>(c.N) * 4, static_cast<size_t>(c.N) * 4,
                              static_cast<size_t>(nr), cudaMemcpyDeviceToHost, g->s_out[i]));
    return SB200_OK;
  };
  int64_t prev_r0 = -1, prev_nr = 0;
  cudaEvent_t prev_done = nullptr;
  for (size_t ci = 0; ci + 1 < cuts.size() && !rc; ++ci) {
    const int64_t r0 = cuts[ci], nr = cuts[ci + 1] - r0;
    cudaEvent_t in = nullptr, done = nullptr;
    if (cudaEventCreateWithFlags(&in, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&done, cudaEventDisableTiming) != cudaSuccess) {
      rc = set_error(SB200_ERR_INVALID_VALUE, "creating events on device %d", dev);
      break;
    }
    ev_in.push_back(in);
    ev_done.push_back(done);
    if (c.K > 0) rc = copy_in(dev, g->s_in[i], dA + r0 * c.K, c.A + (first + r0) * c.lda, nr, c.K, c.lda, staged_a);
    if (!rc && c.C) rc = copy_in(dev, g->s_in[i], dC + r0 * c.N, c.C + (first + r0) * c.ldc, nr, c.N, c.ldc, staged_c);
    if (rc) break;
    if (cudaEventRecord(in, g->s_in[i]) != cudaSuccess || cudaStreamWaitEvent(g->s_main[i], in, 0) != cudaSuccess) {
      rc = set_error(SB200_ERR_INVALID_VALUE, "ordering a row chunk on device %d", dev);
      break;
    }
    rc = sb200_gemm_f32(dev, h(g->s_main[i]), c.mode, nr, c.N, c.K, reinterpret_cast<uintptr_t>(dA + r0 * c.K), c.K,
                        reinterpret_cast<uintptr_t>(dB), c.N, reinterpret_cast<uintptr_t>(dD + r0 * c.N), c.N, c.alpha,
                        dC ? reinterpret_cast<uintptr_t>(dC + r0 * c.N) : 0, c.N, c.beta, reinterpret_cast<uintptr_t>(dBias), c.act);
    if (rc) break;
    if (cudaEventRecord(done, g->s_main[i]) != cudaSuccess) {
      rc = set_error(SB200_ERR_INVALID_VALUE, "recording a row chunk on device %d", dev);
      break;
    }
    // the chunk before goes back while this one computes
    if (prev_done) rc = copy_out(prev_r0, prev_nr, prev_done);
    prev_r0 = r0;
    prev_nr = nr;
    prev_done = done;
  }
  if (!rc && prev_done) rc = copy_out(prev_r0, prev_nr, prev_done);
  if (rc) {
    fail_here(rc);
    cleanup();
    return;
  }
  e = cudaStreamSynchronize(g->s_out[i]);
  if (e != cudaSuccess) fail_here(set_error(static_cast<int>(e), "copying D back from device %d: %s", dev, cudaGetErrorString(e)));
  cleanup();
}

}  // namespace

extern "C" int sb200_gemm_sharded_host(uint64_t group, int mode, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                                       const float* B, int64_t ldb, float* D, int64_t ldd, float alpha, const float* C,
                                       int64_t ldc, float beta, const float* bias, int act) {
  Group* g = find_group(group);
  if (!g) return set_error(SB200_ERR_INVALID_HANDLE, "unknown group");
  if (!sb200::valid_mode(mode))
    return set_error(SB200_ERR_INVALID_VALUE, "unknown GEMM mode %d", mode);
  if (M < 0 || N < 0 || K < 0) return set_error(SB200_ERR_INVALID_VALUE, "negative GEMM dimension");
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL - 64) return set_error(SB200_ERR_TOO_LARGE, "GEMM dimension beyond 2^31-1");
  if (act != SB200_ACT_NONE && act != SB200_ACT_RELU) return set_error(SB200_ERR_INVALID_VALUE, "unknown activation %d", act);
  if (M == 0 || N == 0) return SB200_OK;
  if (!D || (K > 0 && (!A || !B))) return set_error(SB200_ERR_INVALID_VALUE, "null host pointer passed to GEMM");
  if ((K > 0 && lda < K) || (K > 0 && ldb < N) || ldd < N || (C && ldc < N))
    return set_error(SB200_ERR_INVALID_VALUE, "leading dimension smaller than the row length");
  std::lock_guard<std::mutex> lock(g->mu);
  const int n = g->n;
  const HostCall hc{mode, M, N, K, A, B, C, bias, D, lda, ldb, ldc, ldd, alpha, beta, act};
  int64_t first[kMaxGroup], rows[kMaxGroup];
  float *dB[kMaxGroup], *dBias[kMaxGroup], *dA[kMaxGroup], *dC[kMaxGroup], *dD[kMaxGroup];
  // B crosses PCIe once: in equal bands of rows, one per GPU and link, assembled on every GPU by an in-place all-gather
  // over NVLink (SAREK_B200_GROUP_SPLIT_B=0: whole over the first GPU's link, then a broadcast)
  static const bool split_env = [] {
    const char* e = getenv("SAREK_B200_GROUP_SPLIT_B");
    return !(e && e[0] == '0');
  }();
  const bool split_b = split_env && n > 1 && K >= n;
  const int64_t band_rows = (K + n - 1) / n;  // the last band may be shorter; the buffer holds n whole bands
  const size_t szB = al256(static_cast<size_t>(split_b ? band_rows * n : K) * N * 4), szBias = bias ? al256(static_cast<size_t>(N) * 4) : 0;
  for (int i = 0; i < n; ++i) {
    split(M, n, i, &first[i], &rows[i]);
    const size_t szA = al256(static_cast<size_t>(rows[i]) * K * 4), szC = C ? al256(static_cast<size_t>(rows[i]) * N * 4) : 0,
                 szD = al256(static_cast<size_t>(rows[i]) * N * 4);
    GCU_TRY(cudaSetDevice(g->dev[i]));
    int rc = grow(&g->stage[i], szB + szBias + szA + szC + szD + 256);
    if (rc) return rc;
    uint8_t* p = static_cast<uint8_t*>(g->stage[i].p);
    dB[i] = reinterpret_cast<float*>(p);
    dBias[i] = bias ? reinterpret_cast<float*>(p + szB) : nullptr;
    dA[i] = reinterpret_cast<float*>(p + szB + szBias);
    dC[i] = C ? reinterpret_cast<float*>(p + szB + szBias + szA) : nullptr;
    dD[i] = reinterpret_cast<float*>(p + szB + szBias + szA + szC);
  }
  // B and the bias: over PCIe to the first GPU, over NVLink to the rest
  GCU_TRY(cudaSetDevice(g->dev[0]));
  GCU_TRY(cudaEventRecord(g->ev0[0], g->s_main[0]));
  const bool staged_b = sb200::staged_copy_enabled() && K > 0 && sb200::host_memory_is_pageable(B);
  int rc = SB200_OK;
  if (split_b) {
    for (int i = 0; i < n && !rc; ++i) {
      const int64_t k0 = i * band_rows, kr = std::min<int64_t>(band_rows, K - k0);
      if (kr <= 0) continue;
      GCU_TRY(cudaSetDevice(g->dev[i]));
      rc = copy_in(g->dev[i], g->s_main[i], dB[i] + k0 * N, B + k0 * ldb, kr, N, ldb, staged_b);
    }
    GCU_TRY(cudaSetDevice(g->dev[0]));
  } else if (K > 0) {
    rc = copy_in(g->dev[0], g->s_main[0], dB[0], B, K, N, ldb, staged_b);
  }
  if (!rc && bias) GCU_TRY(cudaMemcpyAsync(dBias[0], bias, static_cast<size_t>(N) * 4, cudaMemcpyHostToDevice, g->s_main[0]));
  if (rc) return rc;
  if (n > 1) {
    NCCL_TRY(g_nccl.GroupStart());
    ncclResult_t r = ncclSuccess;
    for (int i = 0; i < n && r == ncclSuccess; ++i) {
      if (split_b)
        r = g_nccl.AllGather(dB[i] + static_cast<size_t>(i) * band_rows * N, dB[i], static_cast<size_t>(band_rows) * N, ncclFloat,
                             g->comm[i], g->s_main[i]);
      else if (K > 0)
        r = g_nccl.Broadcast(dB[i], dB[i], static_cast<size_t>(K) * N, ncclFloat, 0, g->comm[i], g->s_main[i]);
      if (bias && r == ncclSuccess) r = g_nccl.Broadcast(dBias[i], dBias[i], static_cast<size_t>(N), ncclFloat, 0, g->comm[i], g->s_main[i]);
    }
    ncclResult_t r2 = g_nccl.GroupEnd();
    if (r == ncclSuccess) r = r2;
    if (r != ncclSuccess) return set_error(SB200_ERR_COMM, "broadcast of B: %s", g_nccl.GetErrorString(r));
  }
  // one host thread per GPU for the row blocks (the calling thread takes the last member)
  MemberResult res[kMaxGroup];
  std::vector<std::thread> threads;
  for (int i = 0; i + 1 < n; ++i)
    threads.emplace_back(member_main, g, i, &hc, first[i], rows[i], dB[i], dBias[i], dA[i], dC[i], dD[i], &res[i]);
  member_main(g, n - 1, &hc, first[n - 1], rows[n - 1], dB[n - 1], dBias[n - 1], dA[n - 1], dC[n - 1], dD[n - 1], &res[n - 1]);
  for (auto& t : threads) t.join();
  for (int i = 0; i < n; ++i)
    if (res[i].rc) return set_error(res[i].rc, "%s", res[i].msg.c_str());
  // a device-side wait that ran out is reported by the synchronise of each GPU
  for (int i = 0; i < n; ++i)
    if ((rc = sb200_stream_synchronize(g->dev[i], h(g->s_main[i])))) return rc;
  return SB200_OK;
}
