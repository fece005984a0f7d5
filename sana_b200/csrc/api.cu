// Status plumbing and device queries shared by every entry point.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace sana {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static long long g_exchange_wait_ns = 2000000000LL;
long long exchange_wait_limit_ns() { return g_exchange_wait_ns; }

}  // namespace sana

extern "C" int sana_exchange_set_wait_limit_ns(int64_t ns) {
  if (ns < 0) return sana::fail(SANA_ERR_INVALID, "sana_exchange_set_wait_limit_ns: negative limit");
  sana::g_exchange_wait_ns = ns == 0 ? 2000000000LL : (long long)ns;
  return SANA_OK;
}

extern "C" int sana_abi_version(void) { return 1; }
extern "C" const char* sana_last_error(void) { return sana::g_err; }
