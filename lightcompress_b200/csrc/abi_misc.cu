// Version, status strings and device selection of the C ABI.
#include "lc_common.cuh"

extern "C" LC_API int lc_version(void) { return 100; }

extern "C" LC_API const char* lc_status_string(int status) {
  switch (status) {
    case LC_OK: return "ok";
    case LC_ERR_ARG: return "invalid argument";
    case LC_ERR_SHAPE: return "unsupported shape";
    case LC_ERR_ALIGN: return "misaligned pointer or pitch";
    case LC_ERR_ARCH: return "device is not sm_100";
    case LC_ERR_WORKSPACE: return "workspace too small";
    case LC_ERR_NOT_PD: return "matrix not positive definite";
    case LC_ERR_TIMEOUT: return "device-side wait timed out";
    case LC_ERR_CUDA: return "CUDA error";
    default: return "unknown status";
  }
}

extern "C" LC_API int lc_set_device(int device) {
  if (device < 0) return LC_ERR_ARG;
  LC_CHECK_CUDA(cudaSetDevice(device));
  return LC_OK;
}
