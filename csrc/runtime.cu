// Small host-side services of the library: status word readback, device facts, build string.
#include <cuda_runtime.h>
#include <stdlib.h>

#include "api.h"

extern "C" int zse_status_read(const void* status_dev, uint32_t* out4) {
  return cudaMemcpy(out4, status_dev, 16, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : ZSE_ERR_DRIVER;
}

extern "C" int zse_device_info(int* sm_count, int* cc_major, int* cc_minor, int64_t* total_mem, int64_t* free_mem) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ZSE_ERR_DRIVER;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return ZSE_ERR_DRIVER;
  size_t f = 0, t = 0;
  if (cudaMemGetInfo(&f, &t) != cudaSuccess) return ZSE_ERR_DRIVER;
  *sm_count = p.multiProcessorCount;
  *cc_major = p.major;
  *cc_minor = p.minor;
  *total_mem = int64_t(t);
  *free_mem = int64_t(f);
  return 0;
}

namespace zse {
static int g_pdl = -1;
int pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("ZSE_PDL");
    g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}
}  // namespace zse

extern "C" void zse_set_pdl(int on) { zse::g_pdl = on ? 1 : 0; }
extern "C" int zse_get_pdl(void) { return zse::pdl_enabled(); }

extern "C" const char* zse_build_info(void) { return "zse_b200 native library, sm_100a, " __DATE__ " " __TIME__; }
