// map_jit.hpp — run-time compilation (NVRTC, sm_100a) and launch of generated map kernels.
#pragma once
#include <string>

namespace sb200 {

struct JitModule {
  void* module = nullptr;     // CUmodule
  void* vec_fn = nullptr;     // CUfunction sb200_map_vec
  void* scalar_fn = nullptr;  // CUfunction sb200_map_scalar
  void* reduce_fn = nullptr;  // CUfunction sb200_reduce (block-reduction kernels)
};

// source -> cubin for sm_100a.  Needs libnvrtc at run time, no GPU.
int jit_compile_cubin(const std::string& source, const std::string& name, std::string* cubin, std::string* err);
// cubin -> module + the two kernels, in the current device's context.
int jit_load(const std::string& cubin, bool reduce, JitModule* out, std::string* err);
void jit_unload(JitModule* m);
int jit_launch(void* fn, unsigned grid, unsigned block, void* stream, void** args, std::string* err);

}  // namespace sb200
