// Small host-side services of the library: status word readback, device facts, build string.
#include <cuda_runtime.h>

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

extern "C" const char* zse_build_info(void) { return "zse_b200 native library, sm_100a, " __DATE__ " " __TIME__; }
