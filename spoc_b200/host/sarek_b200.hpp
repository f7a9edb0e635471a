// sarek_b200.hpp — C++ host side of the B200 plugin, above the C ABI.
//
// The reference's host language (OCaml) has no toolchain where this library is
// built, so the plugin's host half is written in C++ with the members, argument
// meaning and error behaviour of the interface it stands for:
//
//   sarek_b200::Backend        Framework_sig.BACKEND  (spoc/framework/Framework_sig.ml:137-350),
//                              arranged like sarek-cuda/Cuda_plugin.ml:146-224
//   Backend::Device/Stream/Memory/Event/Kernel   the nested modules of BACKEND
//   Backend::run_source        Cuda_plugin.ml:174-210 (compile cached, bind args in order, launch)
//   sarek_b200::Vector         Spoc_core.Vector for float32 (sarek/core/Vector_types.ml:198-229):
//                              host storage + lazily allocated device buffer + location state
//   sarek_b200::run_vectors    Sarek.Execute.run_vectors (sarek/sarek/Execute.ml:197-216,231-304,
//                              321-335,520-543): transfer, expand Vec -> (buffer, int32 length),
//                              launch, mark every vector argument stale on the CPU
//   sarek_b200::fusion::*      Sarek_fusion (sarek/sarek/Sarek_fusion.ml) over IR text
//
// Errors are exceptions (BackendError, UnsupportedConstruct), like Cuda_api.Cuda_error
// (sarek-cuda/Cuda_api.ml:27-31) and Backend_error (spoc/framework/Backend_error.ml:21-78).
// Header-only; link with -lsarek_b200.  Nothing here computes.
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "../../include/sb200.h"

namespace sarek_b200 {

struct BackendError : std::runtime_error {
  int code;
  BackendError(int c, const std::string& m) : std::runtime_error("[sarek-b200] error " + std::to_string(c) + ": " + m), code(c) {}
};
struct UnsupportedConstruct : BackendError {
  using BackendError::BackendError;
};

inline void check(int rc) {
  if (rc == SB200_OK) return;
  const std::string msg = sb200_last_error_string();
  if (rc == SB200_ERR_UNSUPPORTED) throw UnsupportedConstruct(rc, msg);
  throw BackendError(rc, msg);
}

struct Dims {  // Framework_sig.dims
  uint32_t x = 1, y = 1, z = 1;
};
inline Dims dims1d(uint32_t x) { return {x, 1, 1}; }
inline Dims dims2d(uint32_t x, uint32_t y) { return {x, y, 1}; }

// Framework_sig.run_source_arg
// host: the array the device buffer has yet to be filled from (null: the device copy is current); host_copy: the
// page-locked array a result may be sent back to behind its kernel (null: leave it on the device)
struct RSA_Buffer { uint64_t device_ptr; int length; const void* host = nullptr; void* host_copy = nullptr; };
struct RSA_Int32 { int32_t v; };
struct RSA_Int64 { int64_t v; };
struct RSA_Float32 { float v; };
struct RSA_Float64 { double v; };
using RunSourceArg = std::variant<RSA_Buffer, RSA_Int32, RSA_Int64, RSA_Float32, RSA_Float64>;

class Backend {
 public:
  static constexpr const char* name = "B200";
  static constexpr const char* execution_model = "JIT";
  static constexpr const char* source_lang = "SarekIR_sexp";

  // ---- Device ----------------------------------------------------------
  struct DeviceT {
    int id = 0;
    std::string name;
    uint64_t total_mem = 0;
    int cc_major = 0, cc_minor = 0, sm_count = 0;
  };
  struct DeviceM {
    Backend* b;
    void init() const { check(sb200_init()); }
    int count() const {
      int n = 0;
      check(sb200_device_count(&n));
      return n;
    }
    const DeviceT& get(int idx) const {
      auto it = b->devices_.find(idx);
      if (it == b->devices_.end()) {
        sb200_device_info info;
        check(sb200_device_get_info(idx, &info));
        DeviceT d{idx, info.name, info.total_mem, info.cc_major, info.cc_minor, info.sm_count};
        it = b->devices_.emplace(idx, d).first;
      }
      return it->second;
    }
    void set_current(const DeviceT& d) const {
      check(sb200_device_set_current(d.id));
      b->current_ = d.id;
    }
    int get_current_device() const { return b->current_; }
    void synchronize(const DeviceT& d) const { check(sb200_device_synchronize(d.id)); }
  };

  // ---- Stream / Event --------------------------------------------------
  struct StreamT { int dev; uint64_t handle; };
  struct StreamM {
    StreamT create(const DeviceT& d) const {
      uint64_t h = 0;
      check(sb200_stream_create(d.id, &h));
      return {d.id, h};
    }
    void destroy(StreamT& s) const {
      check(sb200_stream_destroy(s.dev, s.handle));
      s.handle = 0;
    }
    void synchronize(const StreamT& s) const { check(sb200_stream_synchronize(s.dev, s.handle)); }
    StreamT default_stream(const DeviceT& d) const { return {d.id, 0}; }
  };
  struct EventT { int dev; uint64_t handle; };
  struct EventM {
    Backend* b;
    EventT create() const {
      uint64_t h = 0;
      check(sb200_event_create(b->current_, &h));
      return {b->current_, h};
    }
    void destroy(EventT& e) const {
      check(sb200_event_destroy(e.dev, e.handle));
      e.handle = 0;
    }
    void record(const EventT& e, const StreamT& s) const { check(sb200_event_record(e.dev, e.handle, s.handle)); }
    void synchronize(const EventT& e) const { check(sb200_event_synchronize(e.dev, e.handle)); }
    float elapsed(const EventT& start, const EventT& stop) const {
      float ms = 0;
      check(sb200_event_elapsed_ms(start.dev, start.handle, stop.handle, &ms));
      return ms;
    }
  };

  // ---- Memory ----------------------------------------------------------
  struct Buffer {
    int dev = 0;
    uint64_t ptr = 0;
    size_t size = 0;       // elements
    size_t elem_size = 0;  // bytes
  };
  struct MemoryM {
    Buffer alloc_custom(const DeviceT& d, size_t size, size_t elem_size) const {
      uint64_t p = 0;
      check(sb200_mem_alloc(d.id, size * elem_size, &p));
      return {d.id, p, size, elem_size};
    }
    Buffer alloc(const DeviceT& d, size_t size) const { return alloc_custom(d, size, sizeof(float)); }
    void free(Buffer& b) const { check(sb200_mem_free(b.dev, b.ptr)); }  // idempotent in the library
    void host_ptr_to_device(const void* src, size_t bytes, const Buffer& dst) const {
      check(sb200_memcpy_htod(dst.dev, dst.ptr, src, bytes));
    }
    void device_to_host_ptr(const Buffer& src, void* dst, size_t bytes) const {
      check(sb200_memcpy_dtoh(src.dev, dst, src.ptr, bytes));
    }
    void device_to_device(const Buffer& src, const Buffer& dst) const {
      check(sb200_memcpy_dtod(dst.dev, dst.ptr, src.ptr, std::min(src.size * src.elem_size, dst.size * dst.elem_size)));
    }
    size_t size(const Buffer& b) const { return b.size; }
    uint64_t device_ptr(const Buffer& b) const { return b.ptr; }
    bool is_zero_copy(const Buffer&) const { return false; }
  };

  // ---- Kernel ----------------------------------------------------------
  struct KernelT { int dev; uint64_t handle; };
  struct Args {
    std::vector<sb200_arg> items;  // positional: set_arg_* append and ignore their index, as the reference's do
  };
  struct KernelM {
    Backend* b;
    KernelT compile(const DeviceT& d, const std::string& name, const std::string& source) const {
      uint64_t h = 0;
      check(sb200_kernel_compile(d.id, source.c_str(), name.c_str(), &h));
      return {d.id, h};
    }
    KernelT compile_cached(const DeviceT& d, const std::string& name, const std::string& source) const {
      auto key = std::make_pair(d.id, source);
      auto it = b->kernels_.find(key);
      if (it == b->kernels_.end()) it = b->kernels_.emplace(key, compile(d, name, source)).first;
      return it->second;
    }
    void clear_cache() const {
      for (auto& kv : b->kernels_) sb200_kernel_destroy(kv.second.handle);
      b->kernels_.clear();
    }
    int kind(const KernelT& k) const {
      int v = 0;
      check(sb200_kernel_kind(k.handle, &v));
      return v;
    }
    std::string describe(const KernelT& k) const {
      char buf[512];
      check(sb200_kernel_describe(k.handle, buf, sizeof buf));
      return buf;
    }
    Args create_args() const { return {}; }
    static sb200_arg make(int tag) {
      sb200_arg a;
      std::memset(&a, 0, sizeof a);
      a.tag = tag;
      return a;
    }
    void set_arg_buffer(Args& a, int, const Buffer& buf) const { auto x = make(SB200_ARG_BUFFER); x.v.buffer = buf.ptr; a.items.push_back(x); }
    void set_arg_ptr(Args& a, int, uint64_t p) const { auto x = make(SB200_ARG_BUFFER); x.v.buffer = p; a.items.push_back(x); }
    void set_arg_int32(Args& a, int, int32_t v) const { auto x = make(SB200_ARG_I32); x.v.i32 = v; a.items.push_back(x); }
    void set_arg_int64(Args& a, int, int64_t v) const { auto x = make(SB200_ARG_I64); x.v.i64 = v; a.items.push_back(x); }
    void set_arg_float32(Args& a, int, float v) const { auto x = make(SB200_ARG_F32); x.v.f32 = v; a.items.push_back(x); }
    void set_arg_float64(Args& a, int, double v) const { auto x = make(SB200_ARG_F64); x.v.f64 = v; a.items.push_back(x); }
    void launch(const KernelT& k, const Args& a, Dims grid, Dims block, uint32_t shared_mem, uint64_t stream = 0) const {
      const uint32_t g[3] = {grid.x, grid.y, grid.z}, bl[3] = {block.x, block.y, block.z};
      check(sb200_kernel_launch(k.handle, a.items.data(), static_cast<int>(a.items.size()), g, bl, shared_mem, stream));
    }
    // The launch that also uploads (host[i] non-null: fill argument i's buffer from there first) and, for page-locked
    // host_copy entries of vectors a matmul writes, sends the result back behind the kernel; returns one flag per argument.
    std::vector<int32_t> launch_from_host(const KernelT& k, const Args& a, const std::vector<const void*>& host,
                                          const std::vector<void*>& host_copy, Dims grid, Dims block, uint32_t shared_mem,
                                          uint64_t stream = 0) const {
      const uint32_t g[3] = {grid.x, grid.y, grid.z}, bl[3] = {block.x, block.y, block.z};
      std::vector<int32_t> coming(a.items.size() + 1, 0);
      check(sb200_kernel_launch_from_host(k.handle, a.items.data(), static_cast<int>(a.items.size()), host.data(), host_copy.data(),
                                          coming.data(), g, bl, shared_mem, stream));
      coming.resize(a.items.size());
      return coming;
    }
  };

  Backend() : Device{this}, Event{this}, Kernel{this} {}
  ~Backend() { Kernel.clear_cache(); }
  Backend(const Backend&) = delete;
  Backend& operator=(const Backend&) = delete;

  DeviceM Device;
  StreamM Stream;
  MemoryM Memory;
  EventM Event;
  KernelM Kernel;

  bool is_available() const {
    int n = 0;
    return sb200_device_count(&n) == SB200_OK && n > 0;
  }
  // IR -> source: the IR text is its own source language
  std::string generate_source(const std::string& ir) const { return ir; }
  void enable_profiling() const { check(sb200_enable_profiling(1)); }
  void disable_profiling() const { check(sb200_enable_profiling(0)); }
  void set_mode(int mode) const { check(sb200_set_mode(mode)); }

  // Returns, per argument, whether its result is already on its way back to its host_copy array.
  std::vector<int32_t> run_source(const std::string& source, const std::string& lang, const std::string& kernel_name, Dims block,
                                  Dims grid, uint32_t shared_mem, const std::vector<RunSourceArg>& args) {
    if (lang != source_lang) throw BackendError(SB200_ERR_UNSUPPORTED, "run_source: source language " + lang + " not supported");
    const DeviceT& dev = Device.get(Device.get_current_device());
    KernelT k = Kernel.compile_cached(dev, kernel_name, source);
    Args ka = Kernel.create_args();
    int i = 0;
    std::vector<const void*> host(args.size() + 1, nullptr);
    std::vector<void*> host_copy(args.size() + 1, nullptr);
    bool from_host = false;
    for (const RunSourceArg& a : args) {
      if (auto* p = std::get_if<RSA_Buffer>(&a)) {
        Kernel.set_arg_ptr(ka, i, p->device_ptr);
        host[i] = p->host;
        host_copy[i] = p->host_copy;
        from_host = from_host || p->host || p->host_copy;
      }
      else if (auto* q = std::get_if<RSA_Int32>(&a)) Kernel.set_arg_int32(ka, i, q->v);
      else if (auto* r = std::get_if<RSA_Int64>(&a)) Kernel.set_arg_int64(ka, i, r->v);
      else if (auto* s = std::get_if<RSA_Float32>(&a)) Kernel.set_arg_float32(ka, i, s->v);
      else Kernel.set_arg_float64(ka, i, std::get<RSA_Float64>(a).v);
      ++i;
    }
    if (from_host) return Kernel.launch_from_host(k, ka, host, host_copy, grid, block, shared_mem);
    Kernel.launch(k, ka, grid, block, shared_mem);
    return std::vector<int32_t>(args.size(), 0);
  }

 private:
  int current_ = 0;
  std::map<int, DeviceT> devices_;
  std::map<std::pair<int, std::string>, KernelT> kernels_;
};

// ---- Vector / run_vectors ------------------------------------------------
class Vector {
 public:
  enum Location { CPU, Both, Stale_CPU };
  Vector(Backend& b, size_t n) : backend_(&b), host_(n, 0.0f) {}
  Vector(Backend& b, std::vector<float> data) : backend_(&b), host_(std::move(data)) {}
  ~Vector() {
    if (prefetch_dev_ >= 0) sb200_prefetch_wait(prefetch_dev_);  // no exception leaves a destructor
    prefetch_dev_ = -1;
    free_buffer();
    if (pinned_) sb200_host_unregister(host_.data());
  }
  Vector(const Vector&) = delete;
  Vector& operator=(const Vector&) = delete;

  size_t length() const { return host_.size(); }
  Location location() const { return loc_; }
  void to_device(const Backend::DeviceT& dev) {
    if (!buf_.ptr) buf_ = backend_->Memory.alloc(dev, host_.size());
    if (loc_ == CPU) {
      note_transfer();
      backend_->Memory.host_ptr_to_device(host_.data(), host_.size() * sizeof(float), buf_);
      loc_ = Both;
    }
  }
  // For run_vectors: the device buffer exists afterwards; returns the host array when the launch has to upload it
  // (the launch call moves it, overlapped with the kernel where it can), null when the device copy is current.
  const float* pending_upload(const Backend::DeviceT& dev) {
    finish_prefetch();  // nothing may still be writing the host array when it is read for an upload
    if (!buf_.ptr) buf_ = backend_->Memory.alloc(dev, host_.size());
    if (loc_ != CPU) return nullptr;
    note_transfer();
    return host_.data();
  }
  void uploaded() {
    if (loc_ == CPU) loc_ = Both;
  }
  float* pinned_host() { return pinned_ ? host_.data() : nullptr; }
  void result_coming_back(int dev) { prefetch_dev_ = dev; }
  const std::vector<float>& to_array() {
    if (finish_prefetch() && loc_ == Stale_CPU) {  // the launch that made the host copy stale has already sent the result back
      note_transfer();
      loc_ = Both;
    }
    if (loc_ == Stale_CPU) {
      note_transfer();
      backend_->Memory.device_to_host_ptr(buf_, host_.data(), host_.size() * sizeof(float));
      loc_ = Both;
    }
    return host_;
  }
  float get(size_t i) { return to_array().at(i); }
  void set(size_t i, float v) {
    to_array();
    host_.at(i) = v;
    loc_ = CPU;
  }
  void mark_stale() {
    if (loc_ == Both) loc_ = Stale_CPU;
  }
  void free_buffer() {
    finish_prefetch();
    if (buf_.ptr) {
      sb200_mem_free(buf_.dev, buf_.ptr);
      buf_ = {};
      if (loc_ == Stale_CPU) loc_ = CPU;  // the device copy is gone; what the host holds is all there is
    }
  }
  const Backend::Buffer& buffer() const { return buf_; }

 private:
  bool finish_prefetch() {
    if (prefetch_dev_ < 0) return false;
    const int dev = prefetch_dev_;
    prefetch_dev_ = -1;
    check(sb200_prefetch_wait(dev));
    return true;
  }
  // The vector owns its host array for its whole life, so the array can be pinned in place: a vector of 16 MiB or
  // more that is moved a second time is registered with the driver, and this and every later transfer run at the
  // pinned rate; the destructor unregisters.
  void note_transfer() {
    if (++transfers_ == 2 && !pinned_ && host_.size() * sizeof(float) >= (size_t(16) << 20))
      pinned_ = sb200_host_register(host_.data(), host_.size() * sizeof(float)) == SB200_OK;
  }
  Backend* backend_;
  std::vector<float> host_;
  Backend::Buffer buf_;
  Location loc_ = CPU;
  int transfers_ = 0;
  bool pinned_ = false;
  int prefetch_dev_ = -1;  // device whose outbound stream is bringing the result back to host_
};

struct ScalarArg {
  enum Kind { Int32, Int64, Float32, Float64 } kind;
  double f = 0;
  int64_t i = 0;
  static ScalarArg int32(int32_t v) { return {Int32, double(v), v}; }
  static ScalarArg int64(int64_t v) { return {Int64, double(v), v}; }
  static ScalarArg float32(float v) { return {Float32, v, int64_t(v)}; }
  static ScalarArg float64(double v) { return {Float64, v, int64_t(v)}; }
};
using ExecArg = std::variant<Vector*, ScalarArg>;

inline void run_vectors(Backend& backend, const Backend::DeviceT& device, const std::string& ir, const std::vector<ExecArg>& args,
                        Dims block, Dims grid, uint32_t shared_mem = 0, const std::string& kernel_name = "sarek_kern") {
  std::vector<RunSourceArg> rs;
  for (const ExecArg& a : args) {
    if (auto* v = std::get_if<Vector*>(&a)) {
      // Transfer.to_device of the reference, folded into the launch call so that the library can overlap the two
      const float* host = (*v)->pending_upload(device);
      rs.push_back(RSA_Buffer{(*v)->buffer().ptr, static_cast<int>((*v)->length()), host, (*v)->pinned_host()});
      rs.push_back(RSA_Int32{static_cast<int32_t>((*v)->length())});
    } else {
      const ScalarArg& s = std::get<ScalarArg>(a);
      switch (s.kind) {
        case ScalarArg::Int32: rs.push_back(RSA_Int32{static_cast<int32_t>(s.i)}); break;
        case ScalarArg::Int64: rs.push_back(RSA_Int64{s.i}); break;
        case ScalarArg::Float32: rs.push_back(RSA_Float32{static_cast<float>(s.f)}); break;
        case ScalarArg::Float64: rs.push_back(RSA_Float64{s.f}); break;
      }
    }
  }
  backend.Device.set_current(device);
  const std::vector<int32_t> coming =
      backend.run_source(backend.generate_source(ir), Backend::source_lang, kernel_name, block, grid, shared_mem, rs);
  size_t pos = 0;  // position in rs: a vector takes two places (buffer, length), a scalar one
  for (const ExecArg& a : args) {
    if (auto* v = std::get_if<Vector*>(&a)) {
      (*v)->uploaded();  // the launch call returns when its uploads have completed
      if (coming[pos]) (*v)->result_coming_back(device.id);
      (*v)->mark_stale();
      pos += 2;
    } else {
      pos += 1;
    }
  }
}

// ---- Sarek_fusion over IR text ---------------------------------------------
namespace fusion {
inline bool can_fuse(const std::string& p, const std::string& c, const std::string& inter) {
  int r = 0;
  check(sb200_ir_can_fuse(p.c_str(), c.c_str(), inter.c_str(), &r));
  return r != 0;
}
inline std::string fuse(const std::string& p, const std::string& c, const std::string& inter) {
  std::string out(1 << 20, '\0');
  check(sb200_ir_fuse(p.c_str(), c.c_str(), inter.c_str(), &out[0], static_cast<int>(out.size())));
  out.resize(std::strlen(out.c_str()));
  return out;
}
// try_fuse_all: empty optional-like result (false) when the reference returns None
inline bool try_fuse_all(const std::string& p, const std::string& c, const std::string& inter, std::string* fused) {
  std::string out(1 << 20, '\0');
  int f = 0;
  check(sb200_ir_fuse_as(p.c_str(), c.c_str(), inter.c_str(), SB200_FUSE_TRY_ALL, &out[0], static_cast<int>(out.size()), &f));
  out.resize(std::strlen(out.c_str()));
  if (f) *fused = out;
  return f != 0;
}
// this backend's extension: fusion of the guarded `let tid = .. in if tid < n then ..` kernel form
inline bool fuse_guarded(const std::string& p, const std::string& c, const std::string& inter, std::string* fused) {
  std::string out(1 << 20, '\0');
  int f = 0;
  check(sb200_ir_fuse_as(p.c_str(), c.c_str(), inter.c_str(), SB200_FUSE_GUARDED, &out[0], static_cast<int>(out.size()), &f));
  out.resize(std::strlen(out.c_str()));
  if (f) *fused = out;
  return f != 0;
}
}  // namespace fusion

// ---- several GPUs of one process ----------------------------------------------
// The reference's multi-device model is to partition a vector and launch once per device
// (sarek/core/Vector.ml:273-296, split rule sarek/core/Vector_storage.ml:261-272).  A DeviceGroup is that model
// for the GEMM path over the library's group entry points: the library owns streams, NCCL communicators and
// the replicas of B; this class passes pointers and sizes.
class DeviceGroup {
 public:
  enum Gather { None = 0, Fused = SB200_SHARD_GATHER_FUSED, Nccl = SB200_SHARD_GATHER_NCCL };
  explicit DeviceGroup(const std::vector<int>& devices) : devices_(devices) {
    check(sb200_group_create(static_cast<int>(devices.size()), devices.data(), &handle_));
  }
  DeviceGroup(const DeviceGroup&) = delete;
  DeviceGroup& operator=(const DeviceGroup&) = delete;
  ~DeviceGroup() {
    if (handle_) sb200_group_destroy(handle_);
  }
  size_t size() const { return devices_.size(); }
  // (first row, rows) of member `index` when m rows are split over the group
  std::pair<int64_t, int64_t> row_block(int64_t m, int index) const {
    int64_t first = 0, count = 0;
    check(sb200_row_block(m, static_cast<int>(devices_.size()), index, &first, &count));
    return {first, count};
  }
  // D = act(alpha*A.B + beta*C + bias) on device-resident row shards; returns the device time in ms
  float gemm(int mode, int64_t m, int64_t n, int64_t k, const std::vector<uint64_t>& a_shards, uint64_t b,
             const std::vector<uint64_t>& d, float alpha = 1.0f, const std::vector<uint64_t>* c_shards = nullptr, float beta = 0.0f,
             uint64_t bias = 0, int act = SB200_ACT_NONE, Gather gather = None, bool b_resident = false) {
    check(sb200_gemm_sharded(handle_, mode, m, n, k, a_shards.data(), k, b, n, d.data(), n, alpha,
                             c_shards ? c_shards->data() : nullptr, n, beta, bias, act,
                             static_cast<int>(gather) | (b_resident ? SB200_SHARD_B_RESIDENT : 0)));
    float ms = 0.f;
    check(sb200_group_last_ms(handle_, &ms));
    return ms;
  }
  // the same on host operands (row-major contiguous); d is written in place
  void gemm_host(int mode, int64_t m, int64_t n, int64_t k, const float* a, const float* b, float* d, float alpha = 1.0f,
                 const float* c = nullptr, float beta = 0.0f, const float* bias = nullptr, int act = SB200_ACT_NONE) {
    check(sb200_gemm_sharded_host(handle_, mode, m, n, k, a, k, b, n, d, n, alpha, c, n, beta, bias, act));
  }

 private:
  std::vector<int> devices_;
  uint64_t handle_ = 0;
};

}  // namespace sarek_b200
