// SwiGLU transition for 128-channel rows and the pair-bias projection of the single branch.
#include "px_common.cuh"

namespace px {

// =========================================================================================
// x_out = [x +] W_o( silu(W_a LN(x)) * (W_b LN(x)) ), hidden width 512 processed in 16 chunks
// of 32: the [rows][512] intermediates live in registers only.  One CTA = 128 rows.
// Tensor-bound once fused: 393216 FLOP per row against 2*128*sizeof(T) bytes.
// =========================================================================================
constexpr int kTrLdO = 32 + 8;  // row stride of a W_o chunk [128 out][32 hidden]

struct TransitionSmem {
  bf16 A[128 * kLdA];
  bf16 Wab[2][64 * kLdA];     // rows 0..31: W_a chunk, rows 32..63: W_b chunk
  bf16 Wo[2][128 * kTrLdO];   // W_o[:, 32q .. 32q+32)
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
transition_kernel(const Tz* __restrict__ x_in, Tz* __restrict__ x_out, const float* __restrict__ ln_w,
                  const float* __restrict__ ln_b, const bf16* __restrict__ w_a, const bf16* __restrict__ w_b,
                  const bf16* __restrict__ w_o, int64_t rows, int add_residual, float eps) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TransitionSmem& sm = *reinterpret_cast<TransitionSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t row0 = (int64_t)blockIdx.x * 128;

  auto load_chunk = [&](int q, int buf) {
    load_w_rows(sm.Wab[buf], 0, w_a, 32 * q, 32, tid);
    load_w_rows(sm.Wab[buf], 32, w_b, 32 * q, 32, tid);
    for (int idx = tid; idx < 128 * 4; idx += 256) {
      const int r = idx >> 2, ch = idx & 3;
      cp_async16(smem_u32(sm.Wo[buf] + r * kTrLdO + ch * 8), w_o + (size_t)r * 512 + 32 * q + ch * 8, true);
    }
    cp_async_commit();
  };
  load_chunk(0, 0);

  ln_tile_rows<Tz>(sm.A, warp, lane, ln_w, ln_b, eps, [&](int r) -> const Tz* {
    return (row0 + r) < rows ? x_in + (size_t)(row0 + r) * kC : nullptr;
  });
  __syncwarp();

  float out[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) out[j][0] = out[j][1] = out[j][2] = out[j][3] = 0.f;

  const int arow = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int akof = (lane >> 4) * 8;
  const int nrow = (lane & 7) + (lane >> 4) * 8;
  const int kof = ((lane >> 3) & 1) * 8;

  for (int q = 0; q < 16; ++q) {
    if (q + 1 < 16) {
      load_chunk(q + 1, (q + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* Wab = sm.Wab[q & 1];
    const bf16* Wo = sm.Wo[q & 1];
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, smem_u32(sm.A + arow * kLdA + ks * 16 + akof));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, smem_u32(Wab + (np * 16 + nrow) * kLdA + ks * 16 + kof));
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    // h = silu(a) * b as A fragments: 32 hidden columns = 2 k-steps
    uint32_t hf[2][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float h0 = acc[j][0] * sigmoidf_fast(acc[j][0]) * acc[j + 4][0];
      float h1 = acc[j][1] * sigmoidf_fast(acc[j][1]) * acc[j + 4][1];
      float h2 = acc[j][2] * sigmoidf_fast(acc[j][2]) * acc[j + 4][2];
      float h3 = acc[j][3] * sigmoidf_fast(acc[j][3]) * acc[j + 4][3];
      hf[j >> 1][(j & 1) * 2] = pack_bf16x2(h0, h1);
      hf[j >> 1][(j & 1) * 2 + 1] = pack_bf16x2(h2, h3);
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, smem_u32(Wo + (np * 16 + nrow) * kTrLdO + ks * 16 + kof));
        mma_bf16(out[2 * np], hf[ks], b[0], b[1]);
        mma_bf16(out[2 * np + 1], hf[ks], b[2], b[3]);
      }
    __syncthreads();
  }
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int col = 8 * j + 2 * tq;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int64_t r = row0 + 16 * warp + g + 8 * hh;
      if (r < rows) {
        const size_t off = (size_t)r * kC + col;
        float v0 = out[j][2 * hh], v1 = out[j][2 * hh + 1];
        if (add_residual) {
          float2 res = load2(x_in + off);
          v0 += res.x;
          v1 += res.y;
        }
        store2(x_out + off, v0, v1);
      }
    }
  }
}

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

extern "C" int32_t px_transition(const void* x_in, void* x_out, int32_t dtype, const float* ln_w, const float* ln_b,
                                 const px_bf16* w_a, const px_bf16* w_b, const px_bf16* w_o, int64_t rows,
                                 int32_t add_residual, float eps, void* stream) {
  if (!x_in || !x_out || !ln_w || !ln_b || !w_a || !w_b || !w_o || rows < 0) return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  const int64_t ctas = (rows + 127) / 128;
  if (ctas > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const size_t smem = sizeof(TransitionSmem);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == PX_F32) {
    if (cudaFuncSetAttribute(transition_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    transition_kernel<float><<<(unsigned)ctas, 256, smem, st>>>((const float*)x_in, (float*)x_out, ln_w, ln_b,
                                                                (const bf16*)w_a, (const bf16*)w_b, (const bf16*)w_o,
                                                                rows, add_residual, eps);
  } else if (dtype == PX_BF16) {
    if (cudaFuncSetAttribute(transition_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    transition_kernel<bf16><<<(unsigned)ctas, 256, smem, st>>>((const bf16*)x_in, (bf16*)x_out, ln_w, ln_b,
                                                               (const bf16*)w_a, (const bf16*)w_b, (const bf16*)w_o,
                                                               rows, add_residual, eps);
  } else {
    return PX_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

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
