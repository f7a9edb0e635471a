// internal.hpp — what the library's translation units share besides the public C ABI.
#pragma once

namespace sb200 {

// Records a failure for sb200_last_error_string() on the calling thread and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// The numeric modes every GEMM entry point takes.
inline bool valid_mode(int mode) {
  return mode == SB200_MODE_3XTF32 || mode == SB200_MODE_TF32 || mode == SB200_MODE_3XF16 || mode == SB200_MODE_F16 ||
         mode == SB200_MODE_3XMIXED;
}

}  // namespace sb200
