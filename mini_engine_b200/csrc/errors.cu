// Last-error text of the library (one per thread).
#include "common.cuh"
#include <string.h>

static thread_local char g_error[1024] = "";

void me_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

ME_API const char* me_last_error() { return g_error; }

ME_API int me_abi_version() { return 1; }

static bool g_pdl = true;
bool me_pdl_enabled() { return g_pdl; }
int me_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}
ME_API int me_device_sm_count() { return me_sm_count(); }
// Switch programmatic dependent launch on (default) or off for all later launches.
ME_API void me_set_pdl(int on) { g_pdl = on != 0; }
