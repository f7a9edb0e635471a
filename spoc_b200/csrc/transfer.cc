// transfer.cc — staged copies between pageable host memory and the device.
//
// The reference moves whole vectors with one synchronous cuMemcpyHtoD / cuMemcpyDtoH from the
// Bigarray that backs the vector (sarek/core/Transfer.ml:229-322, sarek-cuda/Cuda_api.ml:191-243).
// A Bigarray is ordinary pageable memory, and a pageable copy runs far below the link rate because
// the driver stages it through one internal buffer on one thread.  Here a large pageable copy is
// cut into chunks that several host threads move through pinned staging slots, each thread with
// its own stream and two slots, so the host-side memcpy of one chunk overlaps the DMA of others.
// The call stays synchronous: it returns when the last byte has arrived.
#include "transfer.hpp"

#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

namespace sb200 {
namespace {

constexpr size_t kSlotBytes = size_t(4) << 20;  // a staging slot; chunks are at most this large
constexpr int kMaxLanes = 8;
constexpr int kMaxDevices = 16;

struct Lane {
  cudaStream_t stream = nullptr;
  void* slot[2] = {nullptr, nullptr};
  cudaEvent_t ev[2] = {nullptr, nullptr};
};

struct Job;

// Lanes of one device and direction.  Lane 0 is driven by the thread that calls the copy; lanes 1.. have a
// worker thread each, started with the lane and parked on a condition variable between copies (starting
// threads per copy cost as much as the copy itself for 16-64 MiB).  Pools are never destroyed: their
// parked workers end with the process.
struct Pool {
  std::mutex mu;  // one staged transfer per device and direction at a time
  int lanes = 0;
  Lane lane[kMaxLanes];
  std::mutex wm;
  std::condition_variable wake, done;
  unsigned long generation = 0;
  Job* job = nullptr;
  bool job_to_device = true;
  int job_workers = 0;  // lanes taking part in the current copy, lane 0 included
  int running = 0;      // worker threads still busy with it
};
Pool* g_pool[kMaxDevices][2];  // [device][0 = to the device, 1 = to the host]: the two directions can run side by side
std::mutex g_pool_mu;

Pool* pool_for(int dev, bool to_device) {
  std::lock_guard<std::mutex> lock(g_pool_mu);
  Pool*& p = g_pool[dev][to_device ? 0 : 1];
  if (!p) p = new Pool();
  return p;
}

int lane_count() {
  static int n = [] {
    if (const char* e = getenv("SAREK_B200_COPY_THREADS")) {
      int v = atoi(e);
      if (v >= 1) return v > kMaxLanes ? kMaxLanes : v;
    }
    unsigned hc = std::thread::hardware_concurrency();
    int v = static_cast<int>(hc / 2);
    return v < 2 ? 2 : (v > kMaxLanes ? kMaxLanes : v);
  }();
  return n;
}

void to_device_worker(Job* j, Lane* l);
void to_host_worker(Job* j, Lane* l);

void worker_main(Pool* p, int lane_index) {
  unsigned long seen = 0;
  for (;;) {
    Job* job;
    bool to_device;
    {
      std::unique_lock<std::mutex> lk(p->wm);
      p->wake.wait(lk, [&] { return p->generation != seen; });
      seen = p->generation;
      if (lane_index >= p->job_workers) continue;  // a small copy: this lane sits it out
      job = p->job;
      to_device = p->job_to_device;
    }
    (to_device ? to_device_worker : to_host_worker)(job, &p->lane[lane_index]);
    {
      std::lock_guard<std::mutex> lk(p->wm);
      if (--p->running == 0) p->done.notify_one();
    }
  }
}

cudaError_t ensure_pool(Pool& p) {
  const int want = lane_count();
  for (; p.lanes < want; ++p.lanes) {
    Lane& l = p.lane[p.lanes];
    cudaError_t e = cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking);
    for (int s = 0; s < 2 && e == cudaSuccess; ++s) {
      e = cudaMallocHost(&l.slot[s], kSlotBytes);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&l.ev[s], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) return e;  // the lanes built so far stay usable
    if (p.lanes > 0) std::thread(worker_main, &p, p.lanes).detach();
  }
  return cudaSuccess;
}

struct Job {
  int dev;
  char* dev_ptr;
  char* host_ptr;
  size_t bytes;
  size_t chunk;  // bytes per chunk: large copies use whole slots, small ones are cut finer so that every lane
                 // gets several chunks and its host copy overlaps its DMA
  size_t nchunks;
  std::atomic<size_t> next{0};
  std::atomic<int> error{0};
};

void note(Job& j, cudaError_t e) {
  if (e != cudaSuccess) {
    int expected = 0;
    j.error.compare_exchange_strong(expected, static_cast<int>(e));
  }
}

void to_device_worker(Job* j, Lane* l) {
  note(*j, cudaSetDevice(j->dev));
  bool used[2] = {false, false};
  int s = 0;
  while (j->error.load() == 0) {
    const size_t i = j->next.fetch_add(1);
    if (i >= j->nchunks) break;
    const size_t off = i * j->chunk, len = (j->bytes - off < j->chunk) ? j->bytes - off : j->chunk;
    if (used[s]) note(*j, cudaEventSynchronize(l->ev[s]));  // the slot's previous DMA has read it
    memcpy(l->slot[s], j->host_ptr + off, len);
    note(*j, cudaMemcpyAsync(j->dev_ptr + off, l->slot[s], len, cudaMemcpyHostToDevice, l->stream));
    note(*j, cudaEventRecord(l->ev[s], l->stream));
    used[s] = true;
    s ^= 1;
  }
  note(*j, cudaStreamSynchronize(l->stream));
}

void to_host_worker(Job* j, Lane* l) {
  note(*j, cudaSetDevice(j->dev));
  int s = 0;
  bool pending = false;
  size_t p_off = 0, p_len = 0;
  int p_slot = 0;
  auto drain = [&] {
    if (!pending) return;
    note(*j, cudaEventSynchronize(l->ev[p_slot]));
    if (j->error.load() == 0) memcpy(j->host_ptr + p_off, l->slot[p_slot], p_len);
    pending = false;
  };
  while (j->error.load() == 0) {
    const size_t i = j->next.fetch_add(1);
    if (i >= j->nchunks) break;
    const size_t off = i * j->chunk, len = (j->bytes - off < j->chunk) ? j->bytes - off : j->chunk;
    note(*j, cudaMemcpyAsync(l->slot[s], j->dev_ptr + off, len, cudaMemcpyDeviceToHost, l->stream));
    note(*j, cudaEventRecord(l->ev[s], l->stream));
    drain();  // the previous chunk's host copy overlaps this chunk's DMA
    pending = true;
    p_off = off;
    p_len = len;
    p_slot = s;
    s ^= 1;
  }
  drain();
  note(*j, cudaStreamSynchronize(l->stream));
}

int run(int dev, void* dev_ptr, void* host_ptr, size_t bytes, bool to_device, bool after_device_work) {
  if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  Pool& p = *pool_for(dev, to_device);
  std::lock_guard<std::mutex> lock(p.mu);
  cudaError_t e = ensure_pool(p);
  if (p.lanes == 0) return static_cast<int>(e);
  cudaGetLastError();
  if (after_device_work) {
    // a synchronous copy on the default stream waits for the work launched before it; keep that order
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  Job j;
  j.dev = dev;
  j.dev_ptr = static_cast<char*>(dev_ptr);
  j.host_ptr = static_cast<char*>(host_ptr);
  j.bytes = bytes;
  {
    size_t c = bytes / (static_cast<size_t>(p.lanes) * 4);
    c = (c + (size_t(256) << 10) - 1) / (size_t(256) << 10) * (size_t(256) << 10);
    if (c < (size_t(512) << 10)) c = size_t(512) << 10;
    if (c > kSlotBytes) c = kSlotBytes;
    j.chunk = c;
  }
  j.nchunks = (bytes + j.chunk - 1) / j.chunk;
  const int workers = static_cast<int>(j.nchunks < static_cast<size_t>(p.lanes) ? j.nchunks : p.lanes);
  {
    std::lock_guard<std::mutex> lk(p.wm);
    p.job = &j;
    p.job_to_device = to_device;
    p.job_workers = workers;
    p.running = workers - 1;
    ++p.generation;
  }
  p.wake.notify_all();
  (to_device ? to_device_worker : to_host_worker)(&j, &p.lane[0]);  // the calling thread is lane 0
  {
    std::unique_lock<std::mutex> lk(p.wm);
    p.done.wait(lk, [&] { return p.running == 0; });
    p.job = nullptr;
  }
  return j.error.load();
}

}  // namespace

bool staged_copy_enabled() {
  static bool on = [] {
    const char* e = getenv("SAREK_B200_STAGED_COPY");
    return !(e && e[0] == '0');
  }();
  return on;
}

bool host_memory_is_pageable(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;  // unknown: leave it to the plain copy
  }
  return attr.type == cudaMemoryTypeUnregistered;
}

int staged_copy_to_device(int dev, void* dst, const void* src, size_t bytes, bool after_device_work) {
  return run(dev, dst, const_cast<void*>(src), bytes, true, after_device_work);
}

int staged_copy_to_host(int dev, void* dst, const void* src, size_t bytes, bool after_device_work) {
  return run(dev, const_cast<void*>(src), dst, bytes, false, after_device_work);
}

}  // namespace sb200
