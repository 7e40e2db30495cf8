// Thread-local last-error string of the C ABI.
#include <stdarg.h>

#include "common.cuh"

namespace bolt {
namespace {
thread_local char g_last_error[512] = "";
}
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_last_error; }
}  // namespace bolt

extern "C" const char* bolt_last_error(void) { return bolt::last_error(); }
extern "C" int bolt_abi_version(void) { return BOLT_ABI_VERSION; }
