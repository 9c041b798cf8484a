#include "host/errors.h"

namespace mep {
char* last_error_buf() {
  static thread_local char buf[1024] = {0};
  return buf;
}
}  // namespace mep

extern "C" const char* mep_last_error() { return mep::last_error_buf(); }
