// Library state shared by all entry points: error text, device properties.
#include "tsb_common.cuh"
#include <string.h>
#include <stdlib.h>

namespace tsb {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  // One cached value per device ordinal; the library is used with one device
  // per process in multi-GPU runs but tests may switch devices.
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  return dev;
}

bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("TSB_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace tsb

extern "C" const char *tsb_last_error(void) { return tsb::g_err; }
extern "C" int tsb_version(void) { return 1000; }
extern "C" int tsb_sm_count(void) { return tsb::sm_count(); }
