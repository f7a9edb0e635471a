// internal.hpp — what the library's translation units share besides the public C ABI.
#pragma once

namespace sb200 {

// Records a failure for sb200_last_error_string() on the calling thread and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

}  // namespace sb200
