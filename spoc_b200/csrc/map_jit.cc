// map_jit.cc — run-time compilation and launch of generated element-wise map
// kernels (the backend's counterpart of the reference's NVRTC path,
// sarek-cuda/Cuda_nvrtc.ml:263-389 and sarek-cuda/Cuda_api.ml:315-487, except
// that the target is sm_100a itself, not PTX clamped to compute_90).
//
// NVRTC is loaded with dlopen when the first generic map is compiled; the
// driver entry points come from the CUDA runtime, so the library links
// against neither.  There is no fallback: when NVRTC or the driver is
// missing the call fails with an error message.
#include "map_jit.hpp"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <mutex>

#include "../../include/sb200.h"

namespace sb200 {
namespace {

typedef struct _nvrtcProgram* nvrtcProgram;
typedef int nvrtcResult;

struct Nvrtc {
  void* handle = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
  const char* (*GetErrorString)(nvrtcResult) = nullptr;
};
Nvrtc g_nvrtc;
std::once_flag g_nvrtc_once;
std::string g_nvrtc_error;

void load_nvrtc() {
  static const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                                "/usr/local/cuda/lib64/libnvrtc.so", "libnvrtc.so.13"};
  for (const char* n : names) {
    g_nvrtc.handle = dlopen(n, RTLD_LAZY | RTLD_LOCAL);
    if (g_nvrtc.handle) break;
  }
  if (!g_nvrtc.handle) {
    g_nvrtc_error = "libnvrtc not found (tried libnvrtc.so.12, libnvrtc.so, /usr/local/cuda/lib64)";
    return;
  }
#define LOAD(field, sym)                                                        \
  g_nvrtc.field = reinterpret_cast<decltype(g_nvrtc.field)>(dlsym(g_nvrtc.handle, sym)); \
  if (!g_nvrtc.field) g_nvrtc_error = std::string("libnvrtc lacks ") + sym;
  LOAD(CreateProgram, "nvrtcCreateProgram")
  LOAD(CompileProgram, "nvrtcCompileProgram")
  LOAD(GetCUBINSize, "nvrtcGetCUBINSize")
  LOAD(GetCUBIN, "nvrtcGetCUBIN")
  LOAD(GetProgramLogSize, "nvrtcGetProgramLogSize")
  LOAD(GetProgramLog, "nvrtcGetProgramLog")
  LOAD(DestroyProgram, "nvrtcDestroyProgram")
  LOAD(GetErrorString, "nvrtcGetErrorString")
#undef LOAD
}

struct Driver {
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**,
                           void**) = nullptr;
  bool ok = false;
};
Driver g_drv;
std::once_flag g_drv_once;

void load_driver() {
  auto get = [](const char* name) -> void* {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return fn;
  };
  g_drv.ModuleLoadData = reinterpret_cast<decltype(g_drv.ModuleLoadData)>(get("cuModuleLoadData"));
  g_drv.ModuleGetFunction = reinterpret_cast<decltype(g_drv.ModuleGetFunction)>(get("cuModuleGetFunction"));
  g_drv.ModuleUnload = reinterpret_cast<decltype(g_drv.ModuleUnload)>(get("cuModuleUnload"));
  g_drv.LaunchKernel = reinterpret_cast<decltype(g_drv.LaunchKernel)>(get("cuLaunchKernel"));
  g_drv.ok = g_drv.ModuleLoadData && g_drv.ModuleGetFunction && g_drv.ModuleUnload && g_drv.LaunchKernel;
}

}  // namespace

int jit_compile_cubin(const std::string& source, const std::string& name, std::string* cubin, std::string* err) {
  std::call_once(g_nvrtc_once, load_nvrtc);
  if (!g_nvrtc_error.empty()) {
    *err = g_nvrtc_error;
    return SB200_ERR_UNSUPPORTED;
  }
  nvrtcProgram prog = nullptr;
  nvrtcResult r = g_nvrtc.CreateProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
  if (r != 0) {
    *err = std::string("nvrtcCreateProgram: ") + g_nvrtc.GetErrorString(r);
    return SB200_ERR_UNSUPPORTED;
  }
  // -fmad=false: the Native backend never contracts a*b+c
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-fmad=false", "-default-device"};
  r = g_nvrtc.CompileProgram(prog, 4, opts);
  if (r != 0) {
    size_t n = 0;
    g_nvrtc.GetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n) g_nvrtc.GetProgramLog(prog, &log[0]);
    *err = std::string("NVRTC failed to compile the generated map kernel: ") + g_nvrtc.GetErrorString(r) + "\n" + log;
    g_nvrtc.DestroyProgram(&prog);
    return SB200_ERR_UNSUPPORTED;
  }
  size_t size = 0;
  r = g_nvrtc.GetCUBINSize(prog, &size);
  if (r == 0) {
    cubin->assign(size, '\0');
    r = g_nvrtc.GetCUBIN(prog, &(*cubin)[0]);
  }
  g_nvrtc.DestroyProgram(&prog);
  if (r != 0 || size == 0) {
    *err = std::string("nvrtcGetCUBIN: ") + g_nvrtc.GetErrorString(r);
    return SB200_ERR_UNSUPPORTED;
  }
  return SB200_OK;
}

int jit_load(const std::string& cubin, bool reduce, JitModule* out, std::string* err) {
  std::call_once(g_drv_once, load_driver);
  if (!g_drv.ok) {
    *err = "CUDA driver entry points for module loading are unavailable";
    return SB200_ERR_NO_DEVICE;
  }
  CUmodule mod = nullptr;
  CUresult r = g_drv.ModuleLoadData(&mod, cubin.data());
  if (r != CUDA_SUCCESS) {
    *err = "cuModuleLoadData failed with CUresult " + std::to_string(static_cast<int>(r));
    return static_cast<int>(r);
  }
  CUfunction fv = nullptr, fs = nullptr, fr = nullptr;
  if (reduce) {
    r = g_drv.ModuleGetFunction(&fr, mod, "sb200_reduce");
  } else if ((r = g_drv.ModuleGetFunction(&fv, mod, "sb200_map_vec")) == CUDA_SUCCESS) {
    r = g_drv.ModuleGetFunction(&fs, mod, "sb200_map_scalar");
  }
  if (r != CUDA_SUCCESS) {
    g_drv.ModuleUnload(mod);
    *err = "cuModuleGetFunction failed with CUresult " + std::to_string(static_cast<int>(r));
    return static_cast<int>(r);
  }
  out->module = mod;
  out->vec_fn = fv;
  out->scalar_fn = fs;
  out->reduce_fn = fr;
  return SB200_OK;
}

void jit_unload(JitModule* m) {
  if (m->module && g_drv.ok) g_drv.ModuleUnload(static_cast<CUmodule>(m->module));
  m->module = m->vec_fn = m->scalar_fn = m->reduce_fn = nullptr;
}

int jit_launch(void* fn, unsigned grid, unsigned block, void* stream, void** args, std::string* err) {
  CUresult r = g_drv.LaunchKernel(static_cast<CUfunction>(fn), grid, 1, 1, block, 1, 1, 0, static_cast<CUstream>(stream), args, nullptr);
  if (r != CUDA_SUCCESS) {
    *err = "cuLaunchKernel failed with CUresult " + std::to_string(static_cast<int>(r));
    return static_cast<int>(r);
  }
  return SB200_OK;
}

}  // namespace sb200
