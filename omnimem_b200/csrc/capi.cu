// Error string and version of the C ABI.
#include "common.cuh"

#include <string>

namespace nsa {
namespace {
thread_local char g_error[512] = "";
}
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_error; }
}  // namespace nsa

extern "C" const char* nsa_last_error(void) { return nsa::get_error(); }
extern "C" const char* nsa_version(void) { return "omnimem_b200 0.1 (sm_100a)"; }
