// Shared device helpers for the sm_100a Pairformer kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/px_b200.h"

namespace px {

typedef __nv_bfloat16 bf16;

constexpr int kC = 128;        // pair channels handled by the fused kernels
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Two fp32 -> one f16x2 word (round to nearest; values beyond the fp16 range saturate to +-65504 instead of inf).
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 unpack_f16x2(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}
// The two 16-bit operand formats of the tensor-core kernels: bf16 (kF16 = false) and fp16 (kF16 = true).
template <bool kF16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  return kF16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}
template <bool kF16>
__device__ __forceinline__ float2 unpack16x2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack16x2<true>(uint32_t u) {
  return unpack_f16x2(u);
}
// bf16 -> fp32 is a 16-bit shift: spelled out so that it runs on the integer pipe, not the conversion unit
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}

template <>
__device__ __forceinline__ float2 unpack16x2<false>(uint32_t u) {
  return unpack_bf16x2(u);
}
template <bool kF16>
__device__ __forceinline__ uint16_t round16(float v) {
  return kF16 ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
// (1, 1) as a pair of bf16 or of fp16
__host__ __device__ constexpr uint32_t ones16x2(bool f16) { return f16 ? 0x3C003C00u : 0x3F803F80u; }

// Packed fp32 arithmetic (sm_100): two elements per issue slot.  Pays where the issue slots are the scarce resource
// (flash attention: -7 %); the SwiGLU of the transition kernel got 22 % slower with it and stays scalar.
// (a0, a1) += (b0, b1) as one packed instruction: half the issue slots of two scalar additions.
__device__ __forceinline__ void add2(float& a0, float& a1, float b0, float b1) {
  asm("{\n .reg .b64 x, y;\n mov.b64 x, {%0, %1};\n mov.b64 y, {%2, %3};\n add.f32x2 x, x, y;\n mov.b64 {%0, %1}, x;\n}\n"
      : "+f"(a0), "+f"(a1)
      : "f"(b0), "f"(b1));
}

// (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1) as one packed instruction.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n .reg .b64 a, b, c, d;\n mov.b64 a, {%2, %3};\n mov.b64 b, {%4, %5};\n mov.b64 c, {%6, %7};\n"
      " fma.rn.f32x2 d, a, b, c;\n mov.b64 {%0, %1}, d;\n}\n"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
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


}  // namespace px
