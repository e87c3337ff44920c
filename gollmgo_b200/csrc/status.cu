// Error reporting shared by all launchers, and the library's version probe.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_err[512] = "";

int gg_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int gg_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return GG_OK;
}

bool gg_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("GOLLMGO_B200_NO_PDL");
    on = (v && v[0] && v[0] != '0') ? 0 : 1;
  }
  return on == 1;
}

extern "C" const char* gg_last_error() { return g_err; }

// Compute capability of the current device as major*10+minor, or -1.
extern "C" int gg_device_capability() {
  int dev = 0, major = 0, minor = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
  return major * 10 + minor;
}
