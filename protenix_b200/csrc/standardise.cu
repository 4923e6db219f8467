// Standardised fp16 copy of the rows of an fp32 pair tensor:  zn[row] = fp16( (z[row] - mean) * rsqrt(var + eps) ).
//
// The kernels that consume LayerNorm'd rows of z multiply 16-bit operands on the tensor core.  For a bf16 z they take
// the stored rows as they are; for an fp32 z they take this copy: one pass over z per sub-module (the projection and
// the output stage of a triangle update normalise the same z with the same LayerNorm, so they share the copy), after
// which the rows reach the tensor core by TMA exactly like bf16 rows.  A standardised row lies within +-sqrt(128), so
// fp16 cannot overflow, and its 11-bit significand is what makes the fp32 path more accurate than the bf16 one.
// gamma and beta are not applied here: the consumers fold them into their weights.
//
// HBM-bound: 512 bytes read and 256 written per row.  One warp per row (a row is one coalesced 16-byte load per
// lane), eight rows in flight per warp so that the loads overlap and the shuffle chains interleave; mean and variance
// in two passes over the registers.
#include "px_common.cuh"

namespace px {

constexpr int kStdRowsPerBatch = 8;

__global__ void __launch_bounds__(256) standardise_rows_kernel(const float* __restrict__ z, __half* __restrict__ zn,
                                                               long long rows, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  constexpr int kB = kStdRowsPerBatch;
  for (long long r0 = warp * kB; r0 < rows; r0 += nwarps * kB) {
    float4 v[kB];
    float acc[kB];
#pragma unroll
    for (int j = 0; j < kB; ++j)
      v[j] = r0 + j < rows ? __ldcs(reinterpret_cast<const float4*>(z + (size_t)(r0 + j) * kC) + lane)
                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kB; ++j) acc[j] = (v[j].x + v[j].y) + (v[j].z + v[j].w);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int j = 0; j < kB; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      const float mean = acc[j] * (1.0f / kC);
      v[j].x -= mean, v[j].y -= mean, v[j].z -= mean, v[j].w -= mean;
      acc[j] = fmaf(v[j].x, v[j].x, v[j].y * v[j].y) + fmaf(v[j].z, v[j].z, v[j].w * v[j].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int j = 0; j < kB; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      if (r0 + j < rows) {
        const float rstd = rsqrtf(acc[j] * (1.0f / kC) + eps);
        *reinterpret_cast<uint2*>(zn + (size_t)(r0 + j) * kC + 4 * lane) =
            make_uint2(pack_f16x2(v[j].x * rstd, v[j].y * rstd), pack_f16x2(v[j].z * rstd, v[j].w * rstd));
      }
    }
  }
}

// z[i] += upd[i] for an fp32 tensor and an fp16 update (the row-sharded path adds the ending-node update, computed
// where the columns live and returned in fp16, to the rows it owns).  HBM-bound; eight elements per thread and step.
__global__ void __launch_bounds__(256) add_update_kernel(float* __restrict__ z, const __half* __restrict__ upd, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(upd) + i);
    float4 a = reinterpret_cast<const float4*>(z)[2 * i], b = reinterpret_cast<const float4*>(z)[2 * i + 1];
    const float2 u0 = unpack_f16x2(u.x), u1 = unpack_f16x2(u.y), u2 = unpack_f16x2(u.z), u3 = unpack_f16x2(u.w);
    a.x += u0.x, a.y += u0.y, a.z += u1.x, a.w += u1.y;
    b.x += u2.x, b.y += u2.y, b.z += u3.x, b.w += u3.y;
    reinterpret_cast<float4*>(z)[2 * i] = a;
    reinterpret_cast<float4*>(z)[2 * i + 1] = b;
  }
}

}  // namespace px

extern "C" int32_t px_add_update_rows(float* z, const px_f16* upd, int64_t rows, void* stream) {
  if (!z || !upd || rows < 0 || (((uintptr_t)z | (uintptr_t)upd) & 15)) return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long n8 = (long long)rows * (px::kC / 8);
  long long grid = (n8 + 255) / 256;
  if (grid > 8ll * sms) grid = 8ll * sms;
  px::add_update_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(z, (const __half*)upd, n8);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int32_t px_standardise_rows(const float* z, px_f16* zn, int64_t rows, float eps, void* stream) {
  if (!z || !zn || rows < 0 || (((uintptr_t)z | (uintptr_t)zn) & 15)) return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long batches = (rows + px::kStdRowsPerBatch - 1) / px::kStdRowsPerBatch;
  long long grid = (batches + 7) / 8;                    // eight warps per CTA
  if (grid > 8ll * sms) grid = 8ll * sms;                // a multiple of the SM count, eight CTAs resident per SM
  px::standardise_rows_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(z, (__half*)zn, (long long)rows, eps);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
