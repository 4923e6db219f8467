// Shared device helpers for the sm_100a Pairformer kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/px_b200.h"

namespace px {

typedef __nv_bfloat16 bf16;

constexpr int kC = 128;        // pair channels handled by the fused kernels
constexpr int kPad = 8;        // bf16 elements of padding per shared-memory row (16 bytes)
constexpr int kLdA = kC + kPad;  // row stride of a [rows][128] bf16 operand tile in shared memory
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16-byte asynchronous copy global -> shared; when !pred the destination is zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// bf16 -> fp32 is a 16-bit shift: spelled out so that it runs on the integer pipe, not the conversion unit
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- typed access to the residual stream (fp32 or bf16 storage) -------------------------
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
  return unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p));
}
__device__ __forceinline__ void store2(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void store2(bf16* p, float a, float b) {
  *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(a, b);
}

// eight consecutive channels of a row

// ---- LayerNorm of a 128-channel tile into a bf16 operand tile ----------------------------
// Warp `warp` normalises rows [16*warp, 16*warp+16) of a 128-row tile; lane l owns channels
// 4l..4l+3.  row_ptr(r) returns the global address of row r or nullptr when the row is out of
// range (the operand row is then zero).  Only __syncwarp() is needed before the same warp
// reads its rows back with ldmatrix.
template <typename Tz, typename RowPtr>
__device__ __forceinline__ void ln_tile_rows(bf16* sA, int warp, int lane, const float* __restrict__ gamma,
                                             const float* __restrict__ beta, float eps, RowPtr row_ptr) {
  const float4 g4 = *reinterpret_cast<const float4*>(gamma + 4 * lane);
  const float4 b4 = *reinterpret_cast<const float4*>(beta + 4 * lane);
#pragma unroll
  for (int rr = 0; rr < 16; rr += 4) {
    float4 x[4];
    bool ok[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const Tz* p = row_ptr(16 * warp + rr + q);
      ok[q] = (p != nullptr);
      x[q] = ok[q] ? load4(p + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float mean = warp_sum(x[q].x + x[q].y + x[q].z + x[q].w) * (1.0f / kC);
      float d0 = x[q].x - mean, d1 = x[q].y - mean, d2 = x[q].z - mean, d3 = x[q].w - mean;
      float var = warp_sum(d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3) * (1.0f / kC);
      float rstd = rsqrtf(var + eps);
      uint2 o;
      if (ok[q]) {
        o.x = pack_bf16x2(d0 * rstd * g4.x + b4.x, d1 * rstd * g4.y + b4.y);
        o.y = pack_bf16x2(d2 * rstd * g4.z + b4.z, d3 * rstd * g4.w + b4.w);
      } else {
        o.x = 0u;
        o.y = 0u;
      }
      *reinterpret_cast<uint2*>(sA + (16 * warp + rr + q) * kLdA + 4 * lane) = o;
    }
  }
}

// A fragments (16 rows x 128 k) of this warp's rows, 8 k-steps of 16.
__device__ __forceinline__ void load_a_frags(uint32_t (&a)[8][4], const bf16* sA, int warp, int lane) {
  const int row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int kof = (lane >> 4) * 8;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) ldmatrix_x4(a[ks], smem_u32(sA + row * kLdA + ks * 16 + kof));
}
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const bf16* sA, int ld, int warp, int lane, int ks) {
  const int row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int kof = (lane >> 4) * 8;
  ldmatrix_x4(a, smem_u32(sA + row * ld + ks * 16 + kof));
}

// acc[nt] (nt in [NT0, NT0+NT), NT even) += A(16x128) * W^T where sW holds rows n (stride kLdA) of W[n][k].
template <int NT0, int NT, int NACC>
__device__ __forceinline__ void warp_gemm_k128(float (&acc)[NACC][4], const uint32_t (&a)[8][4], const bf16* sW,
                                               int lane) {
  const int nrow = (lane & 7) + (lane >> 4) * 8;
  const int kof = ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, smem_u32(sW + ((NT0 + 2 * np) * 8 + nrow) * kLdA + ks * 16 + kof));
      mma_bf16(acc[NT0 + 2 * np], a[ks], b[0], b[1]);
      mma_bf16(acc[NT0 + 2 * np + 1], a[ks], b[2], b[3]);
    }
  }
}

}  // namespace px
