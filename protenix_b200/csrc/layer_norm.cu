// Stand-alone LayerNorm forward over the last axis (general width, fp32 / bf16 / fp16).
//
// HBM-bound: 2 * cols * sizeof(T) algorithmic bytes per row.  One warp owns a row; the row is
// held in registers between the statistics and the write-back (cols <= 32*VEC*kMaxIt), so x is
// read from HBM exactly once.  VEC is the widest vector (up to 16 bytes) that divides cols.
// Rows that fit 4..32 lanes x 16 bytes (the pair representation's 128 channels in any of the three types, the
// template embedder's 64) take ln_fwd_rows16: every lane moves 16 bytes, a warp works on 32/LANES rows at once and
// keeps four such groups in flight.
#include <cuda_fp16.h>

#include "px_common.cuh"

namespace px {

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Cvt<bf16> {
  static __device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Vec {
  T v[VEC];
};

constexpr int kMaxIt = 8;

// Register-resident path: cols <= 32 * VEC * kMaxIt.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) ln_fwd_cached(const T* __restrict__ x, const T* __restrict__ gamma,
                                                     const T* __restrict__ beta, T* __restrict__ y,
                                                     float* __restrict__ mean_out, float* __restrict__ invvar_out,
                                                     int64_t rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int nvec = cols / VEC;
  const float inv_c = 1.0f / (float)cols;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const Vec<T, VEC>* xr = reinterpret_cast<const Vec<T, VEC>*>(x + row * cols);
    float v[kMaxIt][VEC];
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxIt; ++it) {
      int i = lane + 32 * it;
      if (i < nvec) {
        Vec<T, VEC> t = xr[i];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          v[it][e] = Cvt<T>::to_f(t.v[e]);
          s += v[it][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[it][e] = 0.f;
      }
    }
    const float mean = warp_sum(s) * inv_c;
    float q = 0.f;
#pragma unroll
    for (int it = 0; it < kMaxIt; ++it) {
      if (lane + 32 * it < nvec) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float d = v[it][e] - mean;
          q += d * d;
        }
      }
    }
    const float var = fmaxf(warp_sum(q) * inv_c, 0.f);
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (invvar_out) invvar_out[row] = rstd;
    }
    Vec<T, VEC>* yr = reinterpret_cast<Vec<T, VEC>*>(y + row * cols);
#pragma unroll
    for (int it = 0; it < kMaxIt; ++it) {
      int i = lane + 32 * it;
      if (i < nvec) {
        Vec<T, VEC> g, b, o;
        if (gamma) g = reinterpret_cast<const Vec<T, VEC>*>(gamma)[i];
        if (beta) b = reinterpret_cast<const Vec<T, VEC>*>(beta)[i];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          float r = (v[it][e] - mean) * rstd;
          if (gamma) r *= Cvt<T>::to_f(g.v[e]);
          if (beta) r += Cvt<T>::to_f(b.v[e]);
          o.v[e] = Cvt<T>::from_f(r);
        }
        yr[i] = o;
      }
    }
  }
}

// Rows of exactly LANES x 16 bytes, LANES a power of two <= 32: a group of LANES lanes owns a row.
template <typename T, int LANES>
__global__ void __launch_bounds__(256) ln_fwd_rows16(const T* __restrict__ x, const T* __restrict__ gamma,
                                                     const T* __restrict__ beta, T* __restrict__ y,
                                                     float* __restrict__ mean_out, float* __restrict__ invvar_out,
                                                     int64_t rows, float eps) {
  constexpr int VEC = 16 / (int)sizeof(T), kCols = VEC * LANES, kR = 32 / LANES;
  constexpr int kB = 4;                                  // row groups in flight per warp (2 and 8 measured slower)
  const int lane = threadIdx.x & 31, sub = lane / LANES, li = lane % LANES;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  float g[VEC], b[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    g[e] = gamma ? Cvt<T>::to_f(gamma[li * VEC + e]) : 1.f;
    b[e] = beta ? Cvt<T>::to_f(beta[li * VEC + e]) : 0.f;
  }
  for (int64_t r0 = warp0 * (kB * kR); r0 < rows; r0 += nwarps * (kB * kR)) {
    float v[kB][VEC], acc[kB];
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      const int64_t row = r0 + j * kR + sub;
      Vec<T, VEC> t;
      if (row < rows) {                                  // one 16-byte streaming load per lane
        const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(x + row * kCols) + li);
        t = *reinterpret_cast<const Vec<T, VEC>*>(&raw);
      }
      acc[j] = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        v[j][e] = row < rows ? Cvt<T>::to_f(t.v[e]) : 0.f;
        acc[j] += v[j][e];
      }
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1)
#pragma unroll
      for (int j = 0; j < kB; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    float mean[kB];
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      mean[j] = acc[j] * (1.0f / kCols);
      acc[j] = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        v[j][e] -= mean[j];
        acc[j] = fmaf(v[j][e], v[j][e], acc[j]);
      }
    }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1)
#pragma unroll
      for (int j = 0; j < kB; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
#pragma unroll
    for (int j = 0; j < kB; ++j) {
      const int64_t row = r0 + j * kR + sub;
      if (row < rows) {
        const float rstd = rsqrtf(acc[j] * (1.0f / kCols) + eps);
        if (li == 0) {
          if (mean_out) mean_out[row] = mean[j];
          if (invvar_out) invvar_out[row] = rstd;
        }
        Vec<T, VEC> o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.v[e] = Cvt<T>::from_f(fmaf(v[j][e] * rstd, g[e], b[e]));
        reinterpret_cast<Vec<T, VEC>*>(y + row * kCols)[li] = o;
      }
    }
  }
}

template <typename T, int LANES>
static cudaError_t launch_rows16(const void* x, const void* g, const void* b, void* y, float* mean, float* invvar,
                                 int64_t rows, float eps, cudaStream_t st) {
  const int64_t rows_per_cta = 8 * 4 * (32 / LANES);
  int64_t ctas = (rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = 148 * 8;                           // eight CTAs of 256 threads resident per SM
  if (ctas > cap) ctas = cap;
  ln_fwd_rows16<T, LANES><<<(unsigned)ctas, 256, 0, st>>>((const T*)x, (const T*)g, (const T*)b, (T*)y, mean, invvar, rows,
                                                          eps);
  return cudaGetLastError();
}

// Wide rows: three passes over the row (the second and third hit L1/L2).
template <typename T>
__global__ void __launch_bounds__(256) ln_fwd_wide(const T* __restrict__ x, const T* __restrict__ gamma,
                                                   const T* __restrict__ beta, T* __restrict__ y,
                                                   float* __restrict__ mean_out, float* __restrict__ invvar_out,
                                                   int64_t rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float inv_c = 1.0f / (float)cols;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const T* xr = x + row * cols;
    float s = 0.f;
    for (int i = lane; i < cols; i += 32) s += Cvt<T>::to_f(xr[i]);
    const float mean = warp_sum(s) * inv_c;
    float q = 0.f;
    for (int i = lane; i < cols; i += 32) {
      float d = Cvt<T>::to_f(xr[i]) - mean;
      q += d * d;
    }
    const float rstd = rsqrtf(fmaxf(warp_sum(q) * inv_c, 0.f) + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (invvar_out) invvar_out[row] = rstd;
    }
    T* yr = y + row * cols;
    for (int i = lane; i < cols; i += 32) {
      float r = (Cvt<T>::to_f(xr[i]) - mean) * rstd;
      if (gamma) r *= Cvt<T>::to_f(gamma[i]);
      if (beta) r += Cvt<T>::to_f(beta[i]);
      yr[i] = Cvt<T>::from_f(r);
    }
  }
}

template <typename T, int VEC>
static cudaError_t launch_cached(const void* x, const void* g, const void* b, void* y, float* mean, float* invvar,
                                 int64_t rows, int cols, float eps, cudaStream_t st) {
  const int warps_per_cta = 8;
  int64_t ctas = (rows + warps_per_cta - 1) / warps_per_cta;
  const int64_t cap = 148 * 8 * 4;  // a few waves of resident CTAs; warps stride over the rows
  if (ctas > cap) ctas = cap;
  ln_fwd_cached<T, VEC><<<(unsigned)ctas, 256, 0, st>>>((const T*)x, (const T*)g, (const T*)b, (T*)y, mean, invvar,
                                                         rows, cols, eps);
  return cudaGetLastError();
}

template <typename T>
static cudaError_t dispatch(const void* x, const void* g, const void* b, void* y, float* mean, float* invvar,
                            int64_t rows, int cols, float eps, cudaStream_t st) {
  constexpr int kMaxVec = 16 / (int)sizeof(T);
  auto aligned = [&](int vec) {
    uintptr_t m = (uintptr_t)(sizeof(T) * vec) - 1;
    return cols % vec == 0 && cols <= 32 * vec * kMaxIt && !((uintptr_t)x & m) && !((uintptr_t)y & m) &&
           !((uintptr_t)g & m) && !((uintptr_t)b & m);
  };
  if (cols % kMaxVec == 0 && aligned(kMaxVec)) {       // rows of 4..32 lanes x 16 bytes
    switch (cols / kMaxVec) {
      case 32: return launch_rows16<T, 32>(x, g, b, y, mean, invvar, rows, eps, st);
      case 16: return launch_rows16<T, 16>(x, g, b, y, mean, invvar, rows, eps, st);
      case 8: return launch_rows16<T, 8>(x, g, b, y, mean, invvar, rows, eps, st);
      case 4: return launch_rows16<T, 4>(x, g, b, y, mean, invvar, rows, eps, st);
      default: break;
    }
  }
  if (kMaxVec >= 8 && aligned(8) && cols >= 32 * 8)
    return launch_cached<T, (kMaxVec >= 8 ? 8 : 1)>(x, g, b, y, mean, invvar, rows, cols, eps, st);
  if (aligned(4)) return launch_cached<T, 4>(x, g, b, y, mean, invvar, rows, cols, eps, st);
  if (aligned(2)) return launch_cached<T, 2>(x, g, b, y, mean, invvar, rows, cols, eps, st);
  if (aligned(1)) return launch_cached<T, 1>(x, g, b, y, mean, invvar, rows, cols, eps, st);
  const int warps_per_cta = 8;
  int64_t ctas = (rows + warps_per_cta - 1) / warps_per_cta;
  if (ctas > 148 * 32) ctas = 148 * 32;
  ln_fwd_wide<T><<<(unsigned)ctas, 256, 0, st>>>((const T*)x, (const T*)g, (const T*)b, (T*)y, mean, invvar, rows,
                                                 cols, eps);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// Backward.  With xhat = (x - mean) * invvar and g = dy * gamma (g = dy without a scale):
//   dx = invvar * (g - mean_c(g) - xhat * mean_c(g * xhat)),   dgamma = sum_rows dy * xhat,   dbeta = sum_rows dy.
// One warp per row, two passes over the row (the second is served by L1/L2); the column sums of a CTA's rows are
// collected in shared memory and added to an fp32 scratch of 2 * cols values with one atomic per column and CTA,
// which a second kernel converts to the parameter type.
template <typename T>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                     const float* __restrict__ mean, const float* __restrict__ invvar,
                                                     const T* __restrict__ gamma, T* __restrict__ dx,
                                                     float* __restrict__ scratch, long long rows, int cols) {
  extern __shared__ float ln_bwd_sums[];                 // [2][cols]: dgamma, dbeta partial sums of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (scratch) {
    for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) ln_bwd_sums[c] = 0.f;
    __syncthreads();
  }
  const float inv_cols = 1.0f / (float)cols;
  for (long long row = (long long)blockIdx.x * warps + warp; row < rows; row += (long long)gridDim.x * warps) {
    const T* xr = x + (size_t)row * cols;
    const T* dyr = dy + (size_t)row * cols;
    const float mu = mean[row], rs = invvar[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float g = Cvt<T>::to_f(dyr[c]) * (gamma ? Cvt<T>::to_f(gamma[c]) : 1.0f);
      s1 += g;
      s2 += g * ((Cvt<T>::to_f(xr[c]) - mu) * rs);
    }
    s1 = warp_sum(s1) * inv_cols;
    s2 = warp_sum(s2) * inv_cols;
    T* dxr = dx + (size_t)row * cols;
    for (int c = lane; c < cols; c += 32) {
      const float d = Cvt<T>::to_f(dyr[c]), xh = (Cvt<T>::to_f(xr[c]) - mu) * rs;
      const float g = d * (gamma ? Cvt<T>::to_f(gamma[c]) : 1.0f);
      dxr[c] = Cvt<T>::from_f(rs * (g - s1 - xh * s2));
      if (scratch) {
        atomicAdd(&ln_bwd_sums[c], d * xh);
        atomicAdd(&ln_bwd_sums[cols + c], d);
      }
    }
  }
  if (scratch) {
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) atomicAdd(&scratch[c], ln_bwd_sums[c]);
  }
}

template <typename T>
__global__ void ln_bwd_finish_kernel(const float* __restrict__ scratch, T* __restrict__ dgamma, T* __restrict__ dbeta,
                                     int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  if (dgamma) dgamma[c] = Cvt<T>::from_f(scratch[c]);
  if (dbeta) dbeta[c] = Cvt<T>::from_f(scratch[cols + c]);
}

template <typename T>
static cudaError_t dispatch_bwd(const void* dy, const void* x, const float* mean, const float* invvar, const void* gamma,
                                void* dx, void* dgamma, void* dbeta, float* scratch, long long rows, int cols,
                                cudaStream_t st) {
  const bool sums = dgamma || dbeta;
  const size_t smem = sums ? (size_t)2 * cols * sizeof(float) : 0;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(ln_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return cudaErrorInvalidValue;
  if (sums) {
    const cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)2 * cols * sizeof(float), st);
    if (e != cudaSuccess) return e;
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + 7) / 8;
  const int grid = (int)(want < 4ll * sms ? want : 4ll * sms);
  if (rows > 0)
    ln_bwd_kernel<T><<<grid, 256, smem, st>>>((const T*)dy, (const T*)x, mean, invvar, (const T*)gamma, (T*)dx,
                                              sums ? scratch : nullptr, rows, cols);
  if (sums)
    ln_bwd_finish_kernel<T><<<(cols + 255) / 256, 256, 0, st>>>(scratch, (T*)dgamma, (T*)dbeta, cols);
  return cudaGetLastError();
}

}  // namespace px

extern "C" int32_t px_layer_norm_bwd(const void* dy, const void* x, const float* mean, const float* invvar,
                                     const void* gamma, void* dx, void* dgamma, void* dbeta, float* scratch,
                                     int64_t rows, int64_t cols, int32_t dtype, void* stream) {
  if (cols <= 0 || cols > 16384 || rows < 0) return PX_ERR_BAD_ARG;
  if ((dgamma || dbeta) && !scratch) return PX_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows > 0 && (!dy || !x || !mean || !invvar || !dx)) return PX_ERR_BAD_ARG;
  cudaError_t e;
  switch (dtype) {   // rows == 0 still runs the (empty) reduction so that the parameter gradients come out as zeros
    case PX_F32: e = px::dispatch_bwd<float>(dy, x, mean, invvar, gamma, dx, dgamma, dbeta, scratch, rows, (int)cols, st); break;
    case PX_BF16: e = px::dispatch_bwd<px::bf16>(dy, x, mean, invvar, gamma, dx, dgamma, dbeta, scratch, rows, (int)cols, st); break;
    case PX_F16: e = px::dispatch_bwd<__half>(dy, x, mean, invvar, gamma, dx, dgamma, dbeta, scratch, rows, (int)cols, st); break;
    default: return PX_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int32_t px_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean,
                                     float* invvar, int64_t rows, int64_t cols, float eps, int32_t dtype,
                                     void* stream) {
  if (rows == 0 && cols > 0) return PX_OK;  // empty input: nothing to launch, pointers may be null
  if (!x || !y || rows < 0 || cols <= 0 || cols > (1 << 30)) return PX_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  switch (dtype) {
    case PX_F32: e = px::dispatch<float>(x, gamma, beta, y, mean, invvar, rows, (int)cols, eps, st); break;
    case PX_BF16: e = px::dispatch<px::bf16>(x, gamma, beta, y, mean, invvar, rows, (int)cols, eps, st); break;
    case PX_F16: e = px::dispatch<__half>(x, gamma, beta, y, mean, invvar, rows, (int)cols, eps, st); break;
    default: return PX_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
