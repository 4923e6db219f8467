// Triangle multiplication: input projection, channel-batched contraction, output stage.
#include "px_common.cuh"

namespace px {

// Stage 1 (the gated input projections) lives in trimul_in_tc.cu.
// Stage 2 (the channel-batched contraction) lives in contract_tcgen05.cu.

// Stage 3 (the gated output projection) lives in trimul_out_tc.cu.

static size_t trimul_elems(int64_t n) { return (size_t)kC * n * px_ld(n); }

}  // namespace px

using namespace px;

extern "C" int64_t px_ld(int64_t n) { return (n + 7) / 8 * 8; }

// a, b, x in fp16, then room for the standardised fp16 copy of an fp32 z
extern "C" int64_t px_trimul_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  return (int64_t)(3 * trimul_elems(n) * 2 + (size_t)n * n * kC * 2);
}

extern "C" int32_t px_triangle_multiplication(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                              const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                              const float* ln_out_b, const px_w16* w_ap, const px_w16* w_ag,
                                              const px_w16* w_bp, const px_w16* w_bg, const px_f16* w_z,
                                              const px_w16* w_g, void* workspace, int64_t workspace_bytes, int64_t n,
                                              int32_t incoming, int32_t add_residual, float eps, void* stream) {
  if (!workspace || n <= 0) return PX_ERR_BAD_ARG;
  if (workspace_bytes < px_trimul_workspace_bytes(n)) return PX_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return PX_ERR_BAD_ARG;
  const int64_t ld = px_ld(n);
  px_f16* a = (px_f16*)workspace;
  px_f16* b = a + trimul_elems(n);
  px_f16* x = b + trimul_elems(n);
  px_f16* zn = x + trimul_elems(n);
  const void* rows = z_in;                 // the rows the tensor core multiplies: bf16 z itself, or ...
  int32_t rows_dtype = z_dtype, s;
  if (z_dtype == PX_F32) {                 // ... the standardised fp16 copy of an fp32 z (shared by stages 1 and 3)
    s = px_standardise_rows((const float*)z_in, zn, n * n, eps, stream);
    if (s != PX_OK) return s;
    rows = zn;
    rows_dtype = PX_F16;
  }
  s = px_trimul_in_proj(rows, rows_dtype, mask, ln_in_w, ln_in_b, w_ap, w_ag, w_bp, w_bg, a, b, n, n, ld, incoming, eps,
                        stream);
  if (s != PX_OK) return s;
  s = px_trimul_contract(a, b, x, kC, n, ld, stream);
  if (s != PX_OK) return s;
  return px_trimul_out(x, z_in, zn, z_out, z_dtype, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_z, w_g, n, n, ld,
                       add_residual, eps, stream);
}

// =========================================================================================
// Triangle multiplication for callers that cannot allocate device memory.
//
// The three stages need scratch for a, b and x.  Here that scratch is a fixed array that is part
// of the loaded library image, so the call needs no workspace from the caller and makes no
// cudaMalloc / cudaFree.  The array is 16 MiB (N <= 128) and every GPU that loads the library
// holds it until the process exits.
// =========================================================================================
constexpr int64_t kStaticMaxN = PX_STATIC_MAX_N;
constexpr size_t kStaticScratchBytes = 4 * (size_t)px::kC * kStaticMaxN * kStaticMaxN * 2;   // a, b, x, zn in fp16
static __device__ __align__(256) unsigned char g_trimul_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the scratch array per device ordinal.  In host code the array's name is only a
// handle for the runtime, not a device address: the address has to be asked for, once per device,
// with that device current.  Benign race: two threads may both ask and store the same value.
void* g_static_scratch_addr[kMaxDevices] = {};

int32_t static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PX_ERR_LAUNCH;
  void* p = g_static_scratch_addr[dev];
  if (!p) {
    cudaError_t e = cudaGetSymbolAddress(&p, g_trimul_static_scratch);
    if (e != cudaSuccess || !p) return PX_ERR_LAUNCH;
    g_static_scratch_addr[dev] = p;
  }
  *out = p;
  return PX_OK;
}
}  // namespace

extern "C" int64_t px_static_max_n(void) { return kStaticMaxN; }

extern "C" int32_t px_triangle_multiplication_static(const void* z_in, void* z_out, int32_t z_dtype,
                                                     const float* mask, const float* ln_in_w, const float* ln_in_b,
                                                     const float* ln_out_w, const float* ln_out_b,
                                                     const px_w16* w_ap, const px_w16* w_ag, const px_w16* w_bp,
                                                     const px_w16* w_bg, const px_f16* w_z, const px_w16* w_g,
                                                     int64_t n, int32_t incoming, int32_t add_residual, float eps,
                                                     void* stream) {
  if (n <= 0) return PX_ERR_BAD_ARG;
  if (n > kStaticMaxN) return PX_ERR_TOO_LARGE;
  void* scratch = nullptr;
  int32_t s = static_scratch(&scratch);
  if (s != PX_OK) return s;
  // Layout for this N: a | b | x, each [128][N][ld] fp16, then the standardised copy of an fp32 z.  Every
  // element a stage reads was written earlier in the same call (the projection also writes the zero pad
  // columns), so nothing left by a previous call, possibly with another N, has to be cleared.
  return px_triangle_multiplication(z_in, z_out, z_dtype, mask, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_ap, w_ag, w_bp,
                                    w_bg, w_z, w_g, scratch, (int64_t)kStaticScratchBytes, n, incoming, add_residual,
                                    eps, stream);
}
