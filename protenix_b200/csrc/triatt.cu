// Triangle attention (4 heads x 32): input projection, flash attention with pair bias, output stage.
#include <math_constants.h>

#include "px_common.cuh"

namespace px {

constexpr int kH = 4;   // heads
constexpr int kD = 32;  // head width

// Stage 1 (the q, k, v and bias projections) lives in triatt_in_tc.cu.
// Stage 2 (the attention core) lives in flash_tcgen05.cu.

// Stage 3 (gating and the output projection) lives in triatt_out_tc.cu.

static size_t att_qkv_elems(int64_t n) { return (size_t)n * kH * px_ld(n) * kD; }
static size_t align256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace px

using namespace px;

// workspace layout: q | k | v | o (fp16) | bias (fp32 [4][n][ldm]) | mask_bias (fp32 [n][ldm]) | tile flags |
// standardised fp16 copy of an fp32 z
extern "C" int64_t px_triatt_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  const int64_t ld = px_ld_mask(n);
  return (int64_t)(3 * align256(att_qkv_elems(n) * 2) + align256((size_t)n * n * kC * 2) +
                   align256((size_t)kH * n * ld * 4) + align256((size_t)n * ld * 4) +
                   align256((size_t)px_triatt_flash_scratch_bytes(n, n)) + align256((size_t)n * n * kC * 2));
}

extern "C" int32_t px_triangle_attention(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                         const float* ln_w, const float* ln_b, const px_w16* w_bias,
                                         const px_w16* w_q, const px_w16* w_k, const px_w16* w_v,
                                         const px_w16* w_g, const px_f16* w_o, void* workspace,
                                         int64_t workspace_bytes, int64_t n, int32_t ending, int32_t add_residual,
                                         float eps, float inf, void* stream) {
  if (!workspace || n <= 0 || ((uintptr_t)workspace & 255)) return PX_ERR_BAD_ARG;
  if (workspace_bytes < px_triatt_workspace_bytes(n)) return PX_ERR_WORKSPACE;
  const int64_t ld = px_ld_mask(n);
  unsigned char* p = (unsigned char*)workspace;
  px_f16* q = (px_f16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_f16* k = (px_f16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_f16* v = (px_f16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_f16* o = (px_f16*)p;
  p += align256((size_t)n * n * kC * 2);
  float* bias = (float*)p;
  p += align256((size_t)kH * n * ld * 4);
  float* mbias = (float*)p;
  p += align256((size_t)n * ld * 4);
  void* flags = (void*)p;
  p += align256((size_t)px_triatt_flash_scratch_bytes(n, n));
  px_f16* zn = (px_f16*)p;
  const void* rows = z_in;                 // the rows the tensor core multiplies: bf16 z itself, or ...
  int32_t rows_dtype = z_dtype, s;
  if (z_dtype == PX_F32) {                 // ... the standardised fp16 copy of an fp32 z (shared by stages 1 and 3)
    s = px_standardise_rows((const float*)z_in, zn, n * n, eps, stream);
    if (s != PX_OK) return s;
    rows = zn;
    rows_dtype = PX_F16;
  }
  s = px_triatt_in_proj(rows, rows_dtype, mask, ln_w, ln_b, w_q, w_k, w_v, w_bias, q, k, v, bias, mbias, n, n, ld, ending,
                        eps, inf, stream);
  if (s != PX_OK) return s;
  s = px_triatt_flash(q, k, v, bias, mbias, o, flags, n, n, ld, stream);
  if (s != PX_OK) return s;
  return px_triatt_out(o, z_in, zn, z_out, z_dtype, ln_w, ln_b, w_g, w_o, n, n, ending, add_residual, eps, stream);
}
