// Triangle attention core on the 5th-generation tensor cores (4 heads x 32).
//
//   o[u][q][h*32+d] = softmax_k( q[u,h,q,:] . k[u,h,k,:] + bias[h][q][k] + mask_bias[u][k] ) v[u,h,k,d]
//
// One CTA = (head h, 128 queries, 4 attended rows u), 10 warps:
//   warps 0..3  softmax group 0: rows u0+0 and u0+2   (each thread owns one query row)
//   warps 4..7  softmax group 1: rows u0+1 and u0+3
//   warp 8      TMA producer: the four Q tiles once, then per work item a K tile [128 keys][32] (64-byte
//               swizzle) and a transposed V tile [32 d][128 keys] (128-byte swizzle, two boxes) into a
//               3-stage ring; per key tile the pair-bias tile [128 q][128 k] fp32 (four 128-byte-swizzled
//               boxes) into a 2-deep ring.  The bias tile is shared by the four rows.
//   warp 9      MMA issuer (one thread): S = Q K^T (M=128, N=128, K=32) into one of two TMEM buffers; after
//               the group has turned S into P (bf16, written back over S in TMEM), O_u += P V with P as the
//               TMEM-resident A operand (M=128, N=48, K=128).  Row 32 of the value operand is all ones, so
//               column 32 of O_u accumulates the softmax denominators.
// Work items are ordered (key tile, row); consecutive items alternate between the two groups, so the
// tensor core computes the next S while a group is busy with exponentials.
//
// Softmax is online in base 2 with a lazy reference maximum: the reference only moves (and O_u is rescaled
// through TMEM) when the tile maximum exceeds it by more than 8, so probabilities stay below 2^8.
// Exponentials use the packed bf16 ex2 (P feeds a bf16 MMA anyway).  Every mbarrier wait is bounded.
#include <math_constants.h>

#include "px_tcgen05.cuh"

namespace px {

constexpr int kFH = 4, kFD = 32;
constexpr int kFRows = 4;                 // attended rows per CTA
constexpr int kFStages = 3;               // K/V ring
constexpr int kFQBytes = 128 * 64;        // [128][32] bf16
constexpr int kFKBytes = 128 * 64;
constexpr int kFVBox = 32 * 128;          // one TMA box of the value tile: 32 rows x 64 keys
constexpr int kFVSub = 48 * 128;          // shared footprint of one half (48 operand rows: 32 d, ones, 15 zero)
constexpr int kFStageBytes = kFKBytes + 2 * kFVSub;
constexpr int kFBiasBytes = 128 * 128 * 4;
constexpr int kFON = 48;                  // columns of an O accumulator (32 d + denominator + pad)
constexpr uint32_t kFCols = 512;
constexpr float kRescaleGap = 8.0f;

struct FlashBars {
  uint64_t q_full, kv_full[kFStages], kv_empty[kFStages], bias_full[2], bias_empty[2], s_full[2], p_ready[2], o_done;
  uint32_t tmem_base;
};

struct FlashLayout {
  static constexpr int q = 0;
  static constexpr int kv = q + kFRows * kFQBytes;
  static constexpr int bias = kv + kFStages * kFStageBytes;
  static constexpr int bars = bias + 2 * kFBiasBytes;
  static constexpr int total = bars + (int)sizeof(FlashBars);
};

__global__ void __launch_bounds__(320, 1)
triatt_flash_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_b,
                       const float* __restrict__ mb, const unsigned char* __restrict__ tile_masked,
                       bf16* __restrict__ o, int n_u, int n, int ldm, int nkt) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  FlashBars& bars = *reinterpret_cast<FlashBars*>(sm + FlashLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128, h = blockIdx.y, u0 = blockIdx.z * kFRows;
  const int n_items = nkt * kFRows;

  if (threadIdx.x == 0) {
    mbar_init(&bars.q_full, 1);
    for (int s = 0; s < kFStages; ++s) {
      mbar_init(&bars.kv_full[s], 1);
      mbar_init(&bars.kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.bias_full[b], 1);
      mbar_init(&bars.bias_empty[b], 8);
      mbar_init(&bars.s_full[b], 1);
      mbar_init(&bars.p_ready[b], 4);
    }
    mbar_init(&bars.o_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // operand rows 32..47 of every value half-tile: row 32 = ones (denominator column), the rest zero.  The
  // TMA boxes only ever write rows 0..31.  Rows 32..39 are one 8-row swizzle group; row 32 is its row 0,
  // whose 16-byte pieces are not permuted.
  for (int i = threadIdx.x; i < kFStages * 2 * (16 * 128 / 16); i += blockDim.x) {
    const int half = i / 128, piece = i % 128;                    // 128 pieces of 16 bytes per 16 rows
    const int stage = half >> 1, sub = half & 1;
    uint4 v = (piece < 8) ? make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u) : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(sm + FlashLayout::kv + stage * kFStageBytes + kFKBytes + sub * kFVSub + 32 * 128 +
                              piece * 16) = v;
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes above -> MMA reads
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(kFCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  // TMEM columns: S/P buffer g at 128*g, O accumulator of row r at 256 + 48*r

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(&bars.q_full, kFRows * kFQBytes);
      for (int r = 0; r < kFRows; ++r)  // rows past n_u: coordinate beyond the tensor -> zero fill
        tma_load_3d(smem_u32(sm + FlashLayout::q + r * kFQBytes), &map_q, &bars.q_full, 0, q0, (u0 + r) * kFH + h);
      for (int i = 0; i < n_items && ok; ++i) {
        const int kt = i / kFRows, r = i % kFRows;
        if (r == 0) {
          const int b = kt & 1;
          ok = mbar_wait(&bars.bias_empty[b], ((kt >> 1) & 1) ^ 1, 1u);
          if (!ok) break;
          mbar_expect_tx(&bars.bias_full[b], kFBiasBytes);
          for (int c = 0; c < 4; ++c)
            tma_load_3d(smem_u32(sm + FlashLayout::bias + b * kFBiasBytes + c * (128 * 128)), &map_b,
                        &bars.bias_full[b], kt * 128 + c * 32, q0, h);
        }
        const int s = i % kFStages;
        ok = mbar_wait(&bars.kv_empty[s], ((i / kFStages) & 1) ^ 1, 2u);
        if (!ok) break;
        mbar_expect_tx(&bars.kv_full[s], kFKBytes + 2 * kFVBox);
        const uint32_t base = smem_u32(sm + FlashLayout::kv + s * kFStageBytes);
        const int uh = (u0 + r) * kFH + h;
        tma_load_3d(base, &map_k, &bars.kv_full[s], 0, kt * 128, uh);
        tma_load_3d(base + kFKBytes, &map_v, &bars.kv_full[s], kt * 128, 0, uh);
        tma_load_3d(base + kFKBytes + kFVSub, &map_v, &bars.kv_full[s], kt * 128 + 64, 0, uh);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128), idesc_o = umma_idesc_bf16(128, kFON);
      bool ok = mbar_wait(&bars.q_full, 0, 4u);
      auto issue_s = [&](int i) -> bool {  // S(i) = Q_r K^T into buffer (i & 1)
        const int s = i % kFStages, r = i % kFRows;
        if (!mbar_wait(&bars.kv_full[s], (i / kFStages) & 1, 8u)) return false;
        tc_fence_after();
        const uint64_t dq = umma_desc_sw64(smem_u32(sm + FlashLayout::q + r * kFQBytes));
        const uint64_t dk = umma_desc_sw64(smem_u32(sm + FlashLayout::kv + s * kFStageBytes));
        umma_bf16(tmem_base + 128 * (i & 1), dq, dk, idesc_s, 0u);
        umma_bf16(tmem_base + 128 * (i & 1), dq + 2, dk + 2, idesc_s, 1u);
        umma_commit(&bars.s_full[i & 1]);
        return true;
      };
      if (ok && n_items > 0) ok = issue_s(0);
      if (ok && n_items > 1) ok = issue_s(1);
      for (int i = 0; i < n_items && ok; ++i) {
        const int g = i & 1, s = i % kFStages, kt = i / kFRows, r = i % kFRows;
        ok = mbar_wait(&bars.p_ready[g], (i >> 1) & 1, 16u);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vbase = smem_u32(sm + FlashLayout::kv + s * kFStageBytes + kFKBytes);
        const uint32_t d_o = tmem_base + 256 + kFON * r, a_p = tmem_base + 128 * g;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 16 keys per step: 8 TMEM columns of P, 32 bytes of the value rows
          const uint64_t dv = umma_desc_sw128(vbase + (ks >> 2) * kFVSub) + 2 * (ks & 3);
          umma_bf16_ts(d_o, a_p + 8 * ks, dv, idesc_o, (kt | ks) ? 1u : 0u);
        }
        umma_commit(&bars.kv_empty[s]);
        if (i + 2 < n_items) ok = issue_s(i + 2);
      }
      if (ok) umma_commit(&bars.o_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int g = warp >> 2, qw = warp & 3;
    const int row = 32 * qw + lane;                 // query row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(32 * qw) << 16;
    const uint32_t t_s = tmem_base + lane_addr + 128 * g;
    float m_ref[2] = {-CUDART_INF_F, -CUDART_INF_F};
    bool ok = true;
    for (int kt = 0; kt < nkt && ok; ++kt) {
      const float* bias_tile = reinterpret_cast<const float*>(sm + FlashLayout::bias + (kt & 1) * kFBiasBytes);
      for (int rr = 0; rr < 2 && ok; ++rr) {
        const int r = 2 * rr + g;                   // row of this item inside the CTA's group of four
        const int j = 2 * kt + rr;                  // this group's item counter
        if (rr == 0) ok = mbar_wait(&bars.bias_full[kt & 1], (kt >> 1) & 1, 32u);
        ok = ok && mbar_wait(&bars.s_full[g], j & 1, 64u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float s[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t t[32];
          tmem_ld32(t_s + 32 * c, t);
          tmem_wait_ld();
          // bias: box c holds columns 32c..32c+31 of all 128 rows, 128-byte rows, 16-byte pieces swizzled
          const float* brow = bias_tile + c * (128 * 32) + row * 32;
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const float4 b4 = *reinterpret_cast<const float4*>(brow + ((p ^ (row & 7)) << 2));
            s[32 * c + 4 * p + 0] = __uint_as_float(t[4 * p + 0]) + b4.x;
            s[32 * c + 4 * p + 1] = __uint_as_float(t[4 * p + 1]) + b4.y;
            s[32 * c + 4 * p + 2] = __uint_as_float(t[4 * p + 2]) + b4.z;
            s[32 * c + 4 * p + 3] = __uint_as_float(t[4 * p + 3]) + b4.w;
          }
        }
        const int u = u0 + r;
        const bool urow = u < n_u;
        if (!urow || tile_masked[(size_t)(urow ? u : 0) * nkt + kt]) {   // warp-uniform
          const float* mrow = mb + (size_t)(urow ? u : 0) * ldm + kt * 128;
#pragma unroll
          for (int c4 = 0; c4 < 32; ++c4) {
            const float4 m4 = __ldg(reinterpret_cast<const float4*>(mrow) + c4);
            s[4 * c4 + 0] += m4.x;
            s[4 * c4 + 1] += m4.y;
            s[4 * c4 + 2] += m4.z;
            s[4 * c4 + 3] += m4.w;
          }
        }
        float mt = s[0];
#pragma unroll
        for (int c = 1; c < 128; ++c) mt = fmaxf(mt, s[c]);
        if (kt == 0) {
          m_ref[rr] = mt;                           // first tile: the P.V product overwrites O
        } else if (__any_sync(0xffffffffu, mt > m_ref[rr] + kRescaleGap)) {
          const float m_new = (mt > m_ref[rr] + kRescaleGap) ? mt : m_ref[rr];
          const float alpha = fast_exp2(m_ref[rr] - m_new);
          m_ref[rr] = m_new;
          const uint32_t t_o = tmem_base + lane_addr + 256 + kFON * r;
          uint32_t a[32], b[16];
          tmem_ld32(t_o, a);
          tmem_ld16(t_o + 32, b);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) a[c] = __float_as_uint(__uint_as_float(a[c]) * alpha);
#pragma unroll
          for (int c = 0; c < 16; ++c) b[c] = __float_as_uint(__uint_as_float(b[c]) * alpha);
          tmem_st32(t_o, a);
          tmem_st16(t_o + 32, b);
        }
        const float mr = m_ref[rr];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t w[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) w[e] = exp2_bf16x2(s[64 * c + 2 * e] - mr, s[64 * c + 2 * e + 1] - mr);
          tmem_st32(t_s + 32 * c, w);               // P overwrites the first 64 columns of S
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars.p_ready[g]);
          if (rr == 1) mbar_arrive(&bars.bias_empty[kt & 1]);
        }
      }
    }
    // ---- epilogue: o = O / denominator for this group's two rows
    ok = ok && mbar_wait(&bars.o_done, 0, 128u);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int qi = q0 + row;
      for (int rr = 0; rr < 2; ++rr) {
        const int r = 2 * rr + g, u = u0 + r;
        uint32_t a[32], b[16];
        const uint32_t t_o = tmem_base + lane_addr + 256 + kFON * r;
        tmem_ld32(t_o, a);
        tmem_ld16(t_o + 32, b);
        tmem_wait_ld();
        if (u < n_u && qi < n) {
          const float inv = 1.0f / __uint_as_float(b[0]);
          bf16* dst = o + ((size_t)u * n + qi) * kC + h * kFD;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(a[8 * v + 0]) * inv, __uint_as_float(a[8 * v + 1]) * inv);
            pk.y = pack_bf16x2(__uint_as_float(a[8 * v + 2]) * inv, __uint_as_float(a[8 * v + 3]) * inv);
            pk.z = pack_bf16x2(__uint_as_float(a[8 * v + 4]) * inv, __uint_as_float(a[8 * v + 5]) * inv);
            pk.w = pack_bf16x2(__uint_as_float(a[8 * v + 6]) * inv, __uint_as_float(a[8 * v + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + 8 * v) = pk;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (g_tc_error != 0) {  // a wait ran out: let copies that may still be in flight land before leaving
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
    __syncthreads();
  }
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFCols) : "memory");
  }
}

// tile_masked[u][kt] = 1 when any key of the 128-key tile kt carries a non-zero mask bias for row u
__global__ void flash_tile_flags_kernel(const float* __restrict__ mb, unsigned char* __restrict__ flags, int n_u, int ldm,
                                        int nkt) {
  const int u = blockIdx.x, kt = blockIdx.y;
  const float v = mb[(size_t)u * ldm + kt * 128 + threadIdx.x];
  const int any = __syncthreads_or(v != 0.0f);
  if (threadIdx.x == 0) flags[(size_t)u * nkt + kt] = (unsigned char)(any ? 1 : 0);
}

unsigned int flash_error_flags() {
  unsigned int v = 0;
  return read_clear_tc_error(&v) == 0 ? v : 0x800000u;
}

}  // namespace px

using namespace px;

extern "C" int64_t px_ld_mask(int64_t n) { return (n + 127) / 128 * 128; }

extern "C" int64_t px_triatt_flash_scratch_bytes(int64_t n_u, int64_t n) {
  if (n_u <= 0 || n <= 0) return 0;
  return (n_u * ((n + 127) / 128) + 255) / 256 * 256;
}

extern "C" int32_t px_triatt_flash(const px_bf16* q, const px_bf16* k, const px_bf16* v, const float* bias,
                                   const float* mask_bias, px_bf16* o, void* scratch, int64_t n_u, int64_t n,
                                   int64_t ldm, void* stream) {
  if (!q || !k || !v || !bias || !mask_bias || !o || !scratch || n_u <= 0 || n <= 0 || n_u > 32768 || n > 32768 ||
      ldm != px_ld_mask(n))
    return PX_ERR_BAD_ARG;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)bias | (uintptr_t)mask_bias | (uintptr_t)o) & 15)
    return PX_ERR_BAD_ARG;
  const int64_t ldt = px_ld(n);
  const int nkt = (int)((n + 127) / 128);
  CUtensorMap mq, mk, mv, mbias;
  const uint64_t uh = (uint64_t)n_u * kFH;
  // q, k: [n_u*4][n][32] bf16, box [1][128][32], 64-byte swizzle
  if (!make_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, q, kFD, (uint64_t)n, uh, kFD * 2, (uint64_t)n * kFD * 2, kFD,
                   128, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !make_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k, kFD, (uint64_t)n, uh, kFD * 2, (uint64_t)n * kFD * 2, kFD,
                   128, CU_TENSOR_MAP_SWIZZLE_64B) ||
      // v (transposed): [n_u*4][32][n keys, row stride ldt] bf16, box [1][32][64], 128-byte swizzle
      !make_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, v, (uint64_t)n, kFD, uh, (uint64_t)ldt * 2,
                   (uint64_t)kFD * ldt * 2, 64, kFD, CU_TENSOR_MAP_SWIZZLE_128B) ||
      // pair bias: [4][n q][n k, row stride ldm] fp32, box [1][128][32], 128-byte swizzle
      !make_map_3d(&mbias, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, bias, (uint64_t)n, (uint64_t)n, kFH, (uint64_t)ldm * 4,
                   (uint64_t)n * ldm * 4, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return PX_ERR_LAUNCH;
  cudaStream_t st = (cudaStream_t)stream;
  flash_tile_flags_kernel<<<dim3((unsigned)n_u, (unsigned)nkt), 128, 0, st>>>(mask_bias, (unsigned char*)scratch,
                                                                                (int)n_u, (int)ldm, nkt);
  const size_t smem = FlashLayout::total + 1024;
  if (cudaFuncSetAttribute(triatt_flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  dim3 grid((unsigned)((n + 127) / 128), kFH, (unsigned)((n_u + kFRows - 1) / kFRows));
  triatt_flash_tc_kernel<<<grid, 320, smem, st>>>(mq, mk, mv, mbias, mask_bias, (const unsigned char*)scratch, (bf16*)o,
                                                  (int)n_u, (int)n, (int)ldm, nkt);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
