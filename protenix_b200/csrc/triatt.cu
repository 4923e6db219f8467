// Triangle attention (4 heads x 32): input projection, flash attention with pair bias, output stage.
#include <math_constants.h>

#include "px_common.cuh"

namespace px {

constexpr int kH = 4;   // heads
constexpr int kD = 32;  // head width

// Stage 1 (the q, k, v and bias projections) lives in triatt_in_tc.cu.
// Stage 2 (the attention core) lives in flash_tcgen05.cu.

// =========================================================================================
// Stage 3: z_out(u,t) = [z(u,t) +] W_o (o[u][t] * sigmoid(W_g LN(z(u,t)))).
// HBM-bound: reads 256 (o) + 128*sizeof(Tz), writes 128*sizeof(Tz) per pair element.
// =========================================================================================
struct TriAttOutSmem {
  bf16 A[128 * kLdA];
  bf16 O[128 * kLdA];
  bf16 W[2][64 * kLdA];
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
triatt_out_kernel(const bf16* __restrict__ o, const Tz* __restrict__ z_in, Tz* __restrict__ z_out,
                  const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w_g,
                  const bf16* __restrict__ w_o, int n_u, int n, int swap, int add_residual, float eps) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TriAttOutSmem& sm = *reinterpret_cast<TriAttOutSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, t0 = blockIdx.x * 128;

  // o tile rows [t][128]
  for (int idx = tid; idx < 128 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    const bool p = (t0 + r) < n;
    cp_async16(smem_u32(sm.O + r * kLdA + ch * 8), p ? (o + ((size_t)u * n + t0 + r) * kC + ch * 8) : o, p);
  }
  cp_async_commit();
  auto load_chunk = [&](int c, int buf) {
    load_w_rows(sm.W[buf], 0, (c < 2) ? w_g : w_o, 64 * (c & 1), 64, tid);
    cp_async_commit();
  };
  load_chunk(0, 0);

  auto pair_index = [&](int t) -> size_t { return swap ? ((size_t)t * n_u + u) : ((size_t)u * n + t); };
  ln_tile_rows<Tz>(sm.A, warp, lane, ln_w, ln_b, eps, [&](int r) -> const Tz* {
    int t = t0 + r;
    return t < n ? z_in + pair_index(t) * kC : nullptr;
  });
  __syncwarp();
  uint32_t afr[8][4];
  load_a_frags(afr, sm.A, warp, lane);

  const int g = lane >> 2, tq = lane & 3;
  const int rl = 16 * warp + g;  // local rows rl, rl + 8
  uint32_t og[8][4];             // gated o as A fragments of the output projection
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (c + 1 < 4) {
      load_chunk(c + 1, (c + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    if (c < 2) {
      warp_gemm_k128<0, 8, 8>(acc, afr, sm.W[c & 1], lane);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 64 * c + 8 * j + 2 * tq;
        float2 o0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sm.O + rl * kLdA + col));
        float2 o1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sm.O + (rl + 8) * kLdA + col));
        const uint32_t lo = pack_bf16x2(o0.x * sigmoidf_fast(acc[j][0]), o0.y * sigmoidf_fast(acc[j][1]));
        const uint32_t hi = pack_bf16x2(o1.x * sigmoidf_fast(acc[j][2]), o1.y * sigmoidf_fast(acc[j][3]));
        const int ks = 4 * c + (j >> 1);
        og[ks][(j & 1) * 2] = lo;
        og[ks][(j & 1) * 2 + 1] = hi;
      }
    } else {
      warp_gemm_k128<0, 8, 8>(acc, og, sm.W[c & 1], lane);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 64 * (c & 1) + 8 * j + 2 * tq;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int t = t0 + rl + 8 * hh;
          if (t < n) {
            const size_t off = pair_index(t) * kC + col;
            float v0 = acc[j][2 * hh], v1 = acc[j][2 * hh + 1];
            if (add_residual) {
              float2 r = load2(z_in + off);
              v0 += r.x;
              v1 += r.y;
            }
            store2(z_out + off, v0, v1);
          }
        }
      }
    }
    __syncthreads();
  }
}

static size_t att_qkv_elems(int64_t n) { return (size_t)n * kH * px_ld(n) * kD; }
static size_t align256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace px

using namespace px;

extern "C" int32_t px_triatt_out(const px_bf16* o, const void* z_in, void* z_out, int32_t z_dtype, const float* ln_w,
                                 const float* ln_b, const px_bf16* w_g, const px_bf16* w_o, int64_t n_u, int64_t n_t,
                                 int32_t ending, int32_t add_residual, float eps, void* stream) {
  if (!o || !z_in || !z_out || !ln_w || !ln_b || !w_g || !w_o || n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768)
    return PX_ERR_BAD_ARG;
  dim3 grid((unsigned)((n_t + 127) / 128), (unsigned)n_u);
  const size_t smem = sizeof(TriAttOutSmem);
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == PX_F32) {
    if (cudaFuncSetAttribute(triatt_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_out_kernel<float><<<grid, 256, smem, st>>>((const bf16*)o, (const float*)z_in, (float*)z_out, ln_w, ln_b,
                                                      (const bf16*)w_g, (const bf16*)w_o, (int)n_u, (int)n_t, ending,
                                                      add_residual, eps);
  } else if (z_dtype == PX_BF16) {
    if (cudaFuncSetAttribute(triatt_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_out_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)o, (const bf16*)z_in, (bf16*)z_out, ln_w, ln_b,
                                                     (const bf16*)w_g, (const bf16*)w_o, (int)n_u, (int)n_t, ending,
                                                     add_residual, eps);
  } else {
    return PX_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

// workspace layout: q | k | v | o (bf16) | bias (fp32 [4][n][ldm]) | mask_bias (fp32 [n][ldm]) | tile flags
extern "C" int64_t px_triatt_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  const int64_t ld = px_ld_mask(n);
  return (int64_t)(3 * align256(att_qkv_elems(n) * 2) + align256((size_t)n * n * kC * 2) +
                   align256((size_t)kH * n * ld * 4) + align256((size_t)n * ld * 4) +
                   (size_t)px_triatt_flash_scratch_bytes(n, n));
}

extern "C" int32_t px_triangle_attention(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                         const float* ln_w, const float* ln_b, const px_bf16* w_bias,
                                         const px_bf16* w_q, const px_bf16* w_k, const px_bf16* w_v,
                                         const px_bf16* w_g, const px_bf16* w_o, void* workspace,
                                         int64_t workspace_bytes, int64_t n, int32_t ending, int32_t add_residual,
                                         float eps, float inf, void* stream) {
  if (!workspace || n <= 0 || ((uintptr_t)workspace & 255)) return PX_ERR_BAD_ARG;
  if (workspace_bytes < px_triatt_workspace_bytes(n)) return PX_ERR_WORKSPACE;
  const int64_t ld = px_ld_mask(n);
  unsigned char* p = (unsigned char*)workspace;
  px_bf16* q = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* k = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* v = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* o = (px_bf16*)p;
  p += align256((size_t)n * n * kC * 2);
  float* bias = (float*)p;
  p += align256((size_t)kH * n * ld * 4);
  float* mbias = (float*)p;
  p += align256((size_t)n * ld * 4);
  void* flags = (void*)p;
  int32_t s = px_triatt_in_proj(z_in, z_dtype, mask, ln_w, ln_b, w_q, w_k, w_v, w_bias, q, k, v, bias, mbias, n, n,
                                ld, ending, eps, inf, stream);
  if (s != PX_OK) return s;
  s = px_triatt_flash(q, k, v, bias, mbias, o, flags, n, n, ld, stream);
  if (s != PX_OK) return s;
  return px_triatt_out(o, z_in, z_out, z_dtype, ln_w, ln_b, w_g, w_o, n, n, ending, add_residual, eps, stream);
}
