// Row-shared dropout fused with the residual add (training path of dropout_add_rowwise,
// protenix/model/modules/fused_ops.py:190-224):
//   out[b][r][k] = residual[b][r][k] + x[b][r][k] * mask[b][k]        k over the last two axes (C x D), r over rows
// The mask (zeros and 1 / (1 - p), one value per (b, k), shared by all rows r) is drawn by the caller; with
// residual == NULL the product alone is written (the gradient of x).  The product is rounded to the storage type
// before the add, as the two separate tensor operations of the reference's own fallback do, so results are the
// same to the bit.  HBM-bound: three tensors of traffic, 16-byte accesses when the row length allows.
#include <cuda_fp16.h>

#include "px_common.cuh"

namespace px {

template <typename T>
struct Rnd;
template <>
struct Rnd<float> {
  static __device__ __forceinline__ float ld(float v) { return v; }
  static __device__ __forceinline__ float st(float v) { return v; }
};
template <>
struct Rnd<bf16> {
  static __device__ __forceinline__ float ld(bf16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ bf16 st(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Rnd<__half> {
  static __device__ __forceinline__ float ld(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half st(float v) { return __float2half_rn(v); }
};

template <typename T, int VEC>
__global__ void __launch_bounds__(256) scale_add_rowwise_kernel(const T* __restrict__ residual, const T* __restrict__ x,
                                                                const T* __restrict__ mask, T* __restrict__ out,
                                                                long long rows, long long cd, long long total) {
  struct alignas(sizeof(T) * VEC) V {
    T v[VEC];
  };
  const long long step = (long long)gridDim.x * blockDim.x * VEC;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += step) {
    const long long k = i % cd, b = i / (rows * cd);       // VEC divides cd: a vector never straddles a row
    const V xv = *reinterpret_cast<const V*>(x + i);
    const V mv = *reinterpret_cast<const V*>(mask + b * cd + k);
    V rv, ov;
    if (residual) rv = *reinterpret_cast<const V*>(residual + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const T prod = Rnd<T>::st(__fmul_rn(Rnd<T>::ld(xv.v[e]), Rnd<T>::ld(mv.v[e])));
      ov.v[e] = residual ? Rnd<T>::st(__fadd_rn(Rnd<T>::ld(rv.v[e]), Rnd<T>::ld(prod))) : prod;
    }
    *reinterpret_cast<V*>(out + i) = ov;
  }
}

template <typename T>
static cudaError_t launch_scale_add(const void* residual, const void* x, const void* mask, void* out, long long batches,
                                    long long rows, long long cd, cudaStream_t st) {
  const long long total = batches * rows * cd;
  if (total == 0) return cudaSuccess;
  constexpr int kWide = 16 / (int)sizeof(T);
  const bool wide = cd % kWide == 0 &&
                    ((((uintptr_t)residual | (uintptr_t)x | (uintptr_t)mask | (uintptr_t)out) & 15) == 0);
  const long long work = wide ? total / kWide : total;
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (wide)
    scale_add_rowwise_kernel<T, kWide><<<(int)blocks, 256, 0, st>>>((const T*)residual, (const T*)x, (const T*)mask, (T*)out,
                                                                  rows, cd, total);
  else
    scale_add_rowwise_kernel<T, 1><<<(int)blocks, 256, 0, st>>>((const T*)residual, (const T*)x, (const T*)mask, (T*)out, rows,
                                                              cd, total);
  return cudaGetLastError();
}

}  // namespace px

extern "C" int32_t px_scale_add_rowwise(const void* residual, const void* x, const void* mask, void* out, int64_t batches,
                                        int64_t rows, int64_t cd, int32_t dtype, void* stream) {
  if (batches < 0 || rows < 0 || cd < 0) return PX_ERR_BAD_ARG;
  if (batches * rows * cd == 0) return PX_OK;
  if (!x || !mask || !out) return PX_ERR_BAD_ARG;
  cudaError_t e;
  switch (dtype) {
    case PX_F32: e = px::launch_scale_add<float>(residual, x, mask, out, batches, rows, cd, (cudaStream_t)stream); break;
    case PX_BF16: e = px::launch_scale_add<px::bf16>(residual, x, mask, out, batches, rows, cd, (cudaStream_t)stream); break;
    case PX_F16: e = px::launch_scale_add<__half>(residual, x, mask, out, batches, rows, cd, (cudaStream_t)stream); break;
    default: return PX_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
