// Version and status text of the C ABI.
#include "px_common.cuh"

namespace px {
unsigned int contract_error_flags();
unsigned int flash_error_flags();
unsigned int transition_error_flags();
unsigned int trimul_in_error_flags();
unsigned int triatt_in_error_flags();
unsigned int triatt_out_error_flags();
unsigned int trimul_out_error_flags();
unsigned int pair_bias_error_flags();
unsigned int recycle_error_flags();
}  // namespace px

// Synchronises the device and returns (and clears) the flags recorded by bounded waits that ran out.
// Bits 0-7: contraction kernel, bits 8-15: flash-attention kernel, bits 16-23: transition kernel,
// bits 24-31: projection and output stages.
extern "C" int32_t px_device_error_flags(uint32_t* flags) {
  if (!flags) return PX_ERR_BAD_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return PX_ERR_LAUNCH;
  *flags = px::contract_error_flags() | (px::flash_error_flags() << 8) | (px::transition_error_flags() << 16) |
           ((px::trimul_in_error_flags() | px::triatt_in_error_flags() | px::triatt_out_error_flags() | px::trimul_out_error_flags() | px::pair_bias_error_flags() |
            px::recycle_error_flags()) << 24);
  return PX_OK;
}

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
