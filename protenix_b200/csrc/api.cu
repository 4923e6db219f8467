// Version and status text of the C ABI.
#include "px_common.cuh"

extern "C" int32_t px_version(void) { return 100; }

extern "C" const char* px_status_string(int32_t status) {
  switch (status) {
    case PX_OK: return "ok";
    case PX_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, misaligned pointer or wrong leading dimension)";
    case PX_ERR_UNSUPPORTED: return "shape or dtype outside the compiled specialisations (c_z=128, 4 heads x 32, expansion 4)";
    case PX_ERR_LAUNCH: return "the CUDA runtime refused the kernel launch";
    case PX_ERR_WORKSPACE: return "workspace too small";
    case PX_ERR_TOO_LARGE: return "N exceeds the capacity of the built-in scratch array (N <= 128)";
    default: return "unknown status";
  }
}
