// Status and error text for the C ABI.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace fracssm {
static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace fracssm

extern "C" int fracssm_abi_version(void) { return FRACSSM_ABI_VERSION; }
extern "C" const char *fracssm_last_error(void) { return fracssm::g_err; }
