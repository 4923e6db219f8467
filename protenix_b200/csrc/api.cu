// Version and status text of the C ABI.
#include "px_common.cuh"

namespace px {
#define PX_FAMILY(name) unsigned int name##_error_flags(); int name##_set_wait_limit(long long);
PX_FAMILY(contract) PX_FAMILY(flash) PX_FAMILY(transition) PX_FAMILY(trimul_in) PX_FAMILY(trimul_out)
PX_FAMILY(triatt_in) PX_FAMILY(triatt_out) PX_FAMILY(pair_bias) PX_FAMILY(recycle) PX_FAMILY(selftest) PX_FAMILY(peer) PX_FAMILY(opm)
#undef PX_FAMILY
}  // namespace px

namespace {
typedef unsigned int (*FlagsFn)();
typedef int (*LimitFn)(long long);
// one entry per kernel family = one bit of the flag word, in the order of PX_FAMILY_* in the header
const FlagsFn kFlagFns[PX_N_FAMILIES] = {px::contract_error_flags, px::flash_error_flags, px::transition_error_flags,
                                         px::trimul_in_error_flags, px::trimul_out_error_flags, px::triatt_in_error_flags,
                                         px::triatt_out_error_flags, px::pair_bias_error_flags, px::recycle_error_flags,
                                         px::selftest_error_flags, px::peer_error_flags, px::opm_error_flags};
const LimitFn kLimitFns[PX_N_FAMILIES] = {px::contract_set_wait_limit, px::flash_set_wait_limit, px::transition_set_wait_limit,
                                          px::trimul_in_set_wait_limit, px::trimul_out_set_wait_limit, px::triatt_in_set_wait_limit,
                                          px::triatt_out_set_wait_limit, px::pair_bias_set_wait_limit, px::recycle_set_wait_limit,
                                          px::selftest_set_wait_limit, px::peer_set_wait_limit, px::opm_set_wait_limit};
}  // namespace

// Synchronises the device and returns (and clears) what the bounded waits recorded: bit f of *flags is set when a wait
// of kernel family f ran out; detail[f] (optional, PX_N_FAMILIES words) holds that family's wait codes, which name
// the pipeline role that gave up (0x80000000: the word could not be read).
extern "C" int32_t px_device_error_detail(uint32_t* flags, uint32_t* detail) {
  if (!flags) return PX_ERR_BAD_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return PX_ERR_LAUNCH;
  uint32_t word = 0;
  for (int f = 0; f < PX_N_FAMILIES; ++f) {
    const uint32_t v = kFlagFns[f]();
    if (v) word |= 1u << f;
    if (detail) detail[f] = v;
  }
  *flags = word;
  return PX_OK;
}

extern "C" int32_t px_device_error_flags(uint32_t* flags) { return px_device_error_detail(flags, nullptr); }

// Replaces the limit (clock cycles) of every bounded wait on the current device; cycles <= 0 restores the default.
extern "C" int32_t px_set_wait_limit_cycles(int64_t cycles) {
  const long long c = cycles > 0 ? (long long)cycles : (1ll << 28);
  for (int f = 0; f < PX_N_FAMILIES; ++f)
    if (kLimitFns[f](c) != 0) return PX_ERR_LAUNCH;
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
