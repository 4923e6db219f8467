// Pair-bias projection of the single-representation branch.
#include "px_common.cuh"

namespace px {

// =========================================================================================
// out[h][row] = (W LN(z[row]))[h], h < n_heads <= 16.  HBM-bound: 128*sizeof(Tz) read,
// 4*n_heads written per row.
// =========================================================================================
struct PairBiasSmem {
  bf16 A[128 * kLdA];
  bf16 W[16 * kLdA];
  float zero_beta[kC];
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
pair_bias_kernel(const Tz* __restrict__ z, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                 const bf16* __restrict__ w, float* __restrict__ out, int64_t rows, int n_heads, float eps) {
  __shared__ PairBiasSmem sm;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t row0 = (int64_t)blockIdx.x * 128;
  {
    const int r = tid >> 4, ch = tid & 15;
    cp_async16(smem_u32(sm.W + r * kLdA + ch * 8), w + (size_t)(r < n_heads ? r : 0) * kC + ch * 8, r < n_heads);
    cp_async_commit();
  }
  if (tid < kC) sm.zero_beta[tid] = ln_b ? ln_b[tid] : 0.f;
  __syncthreads();
  ln_tile_rows<Tz>(sm.A, warp, lane, ln_w, sm.zero_beta, eps, [&](int r) -> const Tz* {
    return (row0 + r) < rows ? z + (size_t)(row0 + r) * kC : nullptr;
  });
  cp_async_wait<0>();
  __syncthreads();
  uint32_t afr[8][4];
  load_a_frags(afr, sm.A, warp, lane);
  float acc[2][4];
  acc[0][0] = acc[0][1] = acc[0][2] = acc[0][3] = 0.f;
  acc[1][0] = acc[1][1] = acc[1][2] = acc[1][3] = 0.f;
  warp_gemm_k128<0, 2, 2>(acc, afr, sm.W, lane);
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int head = 8 * j + 2 * tq + e;
      if (head < n_heads) {
        const int64_t r = row0 + 16 * warp + g;
        if (r < rows) out[(size_t)head * rows + r] = acc[j][e];
        if (r + 8 < rows) out[(size_t)head * rows + r + 8] = acc[j][2 + e];
      }
    }
}

}  // namespace px

using namespace px;

extern "C" int32_t px_pair_bias_proj(const void* z, int32_t z_dtype, const float* ln_w, const float* ln_b,
                                     const px_bf16* w, float* out, int64_t rows, int32_t n_heads, float eps,
                                     void* stream) {
  if (!z || !ln_w || !w || !out || rows < 0) return PX_ERR_BAD_ARG;
  if (n_heads <= 0 || n_heads > 16) return PX_ERR_UNSUPPORTED;
  if (rows == 0) return PX_OK;
  const int64_t ctas = (rows + 127) / 128;
  if (ctas > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == PX_F32)
    pair_bias_kernel<float><<<(unsigned)ctas, 256, 0, st>>>((const float*)z, ln_w, ln_b, (const bf16*)w, out, rows,
                                                            n_heads, eps);
  else if (z_dtype == PX_BF16)
    pair_bias_kernel<bf16><<<(unsigned)ctas, 256, 0, st>>>((const bf16*)z, ln_w, ln_b, (const bf16*)w, out, rows,
                                                           n_heads, eps);
  else
    return PX_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
