// Thread-local last-error string shared by all host entry points.  Host code never calls
// exit() on a CUDA error (the reference's CUCHECK/CUDACHECK macros do,
// csrc/nvl_shared_buffer.cuh:17-39); it records a message and returns a non-zero code that
// the Python layer turns into an exception.
#pragma once
#include <cstdarg>
#include <cstdio>

namespace mep {
char* last_error_buf();
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 1024, fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace mep

#define MEP_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess)                                                             \
      return mep::fail(-100 - (int)_e, "%s failed: %s (%s:%d)", #expr,                 \
                       cudaGetErrorString(_e), __FILE__, __LINE__);                    \
  } while (0)
