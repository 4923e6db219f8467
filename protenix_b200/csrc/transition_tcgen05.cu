// SwiGLU transition for 128-channel rows on the 5th-generation tensor cores:
//   x_out = [x +] W_o( silu(W_a LN(x)) * (W_b LN(x)) ),  hidden width 512, the [rows][512] intermediates never
//   leave the SM (tensor memory -> registers -> tensor memory).
//
// One CTA = 256 rows = two M-tiles of 128, 12 warps:
//   warps 0..7   LayerNorm + epilogue.  Warp w first normalises rows 32w..32w+31 (lanes across channels,
//                coalesced) and writes them as the K-major, 128-byte-swizzled A operand of its tile.  Then each
//                thread owns one row: per 64-wide hidden chunk it pulls a|b (128 fp32 columns) out of tensor
//                memory, forms h = silu(a) * b, and writes h (bf16) back over the first 32 columns as the A
//                operand of the second product; at the end it adds the residual and stores the row.
//   warp 8       TMA producer: per hidden chunk the rows 64c..64c+63 of W_a and W_b (two 64-wide k panels each)
//                and the columns 64c..64c+63 of W_o, 48 KB, 3-stage ring.  Weights are re-read from L2 by every
//                CTA: 384 KB per 256 rows.
//   warps 9, 10  one MMA-issuing thread per M-tile (tcgen05 instructions cost ~100 cycles of issue each):
//                H_m = A_m [W_a;W_b]_c^T  (M=128, N=128, K=128) and OUT_m += h_m W_o,c^T (M=128, N=128, K=64, h as
//                the TMEM-resident A operand).  While the epilogue warps of one tile work on H, the tensor core
//                serves the other tile.
//   warp 11      idle (completes the control warpgroup, which hands its registers to the epilogue warpgroups)
// Tensor memory: H_0 | H_1 | OUT_0 | OUT_1, 128 columns each.  Every mbarrier wait is bounded.
#include "px_tcgen05.cuh"

namespace px {

constexpr int kTrStages = 3;
constexpr int kTrABytes = 2 * 128 * 128;            // one M-tile: two k panels of [128 rows][64 k] bf16
constexpr int kTrW1Bytes = 2 * 128 * 128;           // [W_a chunk; W_b chunk]: two k panels of [128 rows][64 k]
constexpr int kTrW2Bytes = 128 * 128;               // W_o chunk: [128 out rows][64 hidden]
constexpr int kTrStageBytes = kTrW1Bytes + kTrW2Bytes;
constexpr int kTrChunks = 8;                        // 512 hidden / 64

struct TransBars {
  uint64_t a_ready[2], w_full[kTrStages], w_empty[kTrStages], h_full[2], hp_ready[2], out_done[2];
  uint32_t tmem_base;
};
struct TransLayout {
  static constexpr int a = 0;
  static constexpr int w = a + 2 * kTrABytes;
  static constexpr int bars = w + kTrStages * kTrStageBytes;
  static constexpr int total = bars + (int)sizeof(TransBars);
};

#ifdef PX_TRANS_TRACE
__device__ long long g_trans_trace[1024];
#define TR_TRACE(slot, idx) \
  if (blockIdx.x == 0 && lane == 0) g_trans_trace[(slot) * 16 + (idx)] = clock64();
#else
#define TR_TRACE(slot, idx)
#endif

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <typename Tz>
__global__ void __launch_bounds__(384, 1)
transition_tc_kernel(const __grid_constant__ CUtensorMap map_wa, const __grid_constant__ CUtensorMap map_wb,
                     const __grid_constant__ CUtensorMap map_wo, const Tz* __restrict__ x_in, Tz* __restrict__ x_out,
                     const float* __restrict__ ln_w, const float* __restrict__ ln_b, long long rows, int add_residual,
                     float eps) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TransBars& bars = *reinterpret_cast<TransBars*>(sm + TransLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row0 = (long long)blockIdx.x * 256;

  if (threadIdx.x == 0) {
    for (int m = 0; m < 2; ++m) {
      mbar_init(&bars.a_ready[m], 4);
      mbar_init(&bars.h_full[m], 1);
      mbar_init(&bars.hp_ready[m], 4);
      mbar_init(&bars.out_done[m], 1);
    }
    for (int s = 0; s < kTrStages; ++s) {
      mbar_init(&bars.w_full[s], 1);
      mbar_init(&bars.w_empty[s], 2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;\n");
    if (warp == 8 && lane == 0) {
      // ---------------------------------------------------------------- weight producer
      bool ok = true;
      for (int c = 0; c < kTrChunks && ok; ++c) {
        const int s = c % kTrStages;
        ok = mbar_wait(&bars.w_empty[s], ((c / kTrStages) & 1) ^ 1, 1u);
        if (!ok) break;
        mbar_expect_tx(&bars.w_full[s], kTrStageBytes);
        const uint32_t base = smem_u32(sm + TransLayout::w + s * kTrStageBytes);
        for (int p = 0; p < 2; ++p) {  // k panel p: rows 0..63 from W_a, rows 64..127 from W_b
          tma_load_3d(base + p * 16384, &map_wa, &bars.w_full[s], 64 * p, 64 * c, 0);
          tma_load_3d(base + p * 16384 + 8192, &map_wb, &bars.w_full[s], 64 * p, 64 * c, 0);
        }
        tma_load_3d(base + kTrW1Bytes, &map_wo, &bars.w_full[s], 64 * c, 0, 0);
      }
    } else if ((warp == 9 || warp == 10) && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer of M-tile m
      const int m = warp - 9;
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
      const uint32_t a_addr = smem_u32(sm + TransLayout::a + m * kTrABytes);
      const uint32_t d_h = tmem_base + 128 * m, d_out = tmem_base + 256 + 128 * m;
      TR_TRACE(30 + m, 0);
      bool ok = mbar_wait(&bars.a_ready[m], 0, 2u);
      TR_TRACE(30 + m, 1);
      for (int c = 0; c < kTrChunks && ok; ++c) {
        const int s = c % kTrStages;
        TR_TRACE(0 + 4 * m, c);
        ok = mbar_wait(&bars.w_full[s], (c / kTrStages) & 1, 4u);
        if (!ok) break;
        TR_TRACE(1 + 4 * m, c);
        tc_fence_after();
        const uint32_t wbase = smem_u32(sm + TransLayout::w + s * kTrStageBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16(d_h, umma_desc_sw128(a_addr + (ks >> 2) * 16384) + 2 * (ks & 3),
                    umma_desc_sw128(wbase + (ks >> 2) * 16384) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
        umma_commit(&bars.h_full[m]);
        TR_TRACE(2 + 4 * m, c);
        ok = mbar_wait(&bars.hp_ready[m], c & 1, 8u);
        if (!ok) break;
        TR_TRACE(3 + 4 * m, c);
        tc_fence_after();
        const uint64_t dwo = umma_desc_sw128(wbase + kTrW1Bytes);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_bf16_ts(d_out, d_h + 8 * ks, dwo + 2 * ks, idesc, (c | ks) ? 1u : 0u);
        umma_commit(&bars.w_empty[s]);
      }
      if (ok) umma_commit(&bars.out_done[m]);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;\n");
    const int m = warp >> 2, qw = warp & 3;
    // ------------------------------------------------------------------ LayerNorm -> swizzled A operand
    {
      unsigned char* sa = sm + TransLayout::a + m * kTrABytes;
      const float4 g4 = *reinterpret_cast<const float4*>(ln_w + 4 * lane);
      const float4 b4 = *reinterpret_cast<const float4*>(ln_b + 4 * lane);
      const int panel_off = (lane >> 4) * 16384 + (lane & 1) * 8, chunk = (lane & 15) >> 1;
      // eight rows per batch: all loads first, then eight independent reductions
#pragma unroll 1
      for (int rb = 0; rb < 32; rb += 8) {
        float4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const long long grow = row0 + 128 * m + 32 * qw + rb + j;
          x[j] = grow < rows ? load4(x_in + (size_t)grow * kC + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = x[j].x + x[j].y + x[j].z + x[j].w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += __shfl_xor_sync(0xffffffffu, sum[j], o);
        float var[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float mean = sum[j] * (1.0f / kC);
          x[j].x -= mean;
          x[j].y -= mean;
          x[j].z -= mean;
          x[j].w -= mean;
          var[j] = x[j].x * x[j].x + x[j].y * x[j].y + x[j].z * x[j].z + x[j].w * x[j].w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int j = 0; j < 8; ++j) var[j] += __shfl_xor_sync(0xffffffffu, var[j], o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = 32 * qw + rb + j;                  // row inside the M-tile
          const long long grow = row0 + 128 * m + r;
          const float rstd = rsqrtf(var[j] * (1.0f / kC) + eps);
          uint2 o = make_uint2(0u, 0u);
          if (grow < rows) {
            o.x = pack_bf16x2(x[j].x * rstd * g4.x + b4.x, x[j].y * rstd * g4.y + b4.y);
            o.y = pack_bf16x2(x[j].z * rstd * g4.z + b4.z, x[j].w * rstd * g4.w + b4.w);
          }
          *reinterpret_cast<uint2*>(sa + panel_off + r * 128 + ((chunk ^ (r & 7)) << 4)) = o;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a_ready[m]);
    }
    // ------------------------------------------------------------------ per-chunk SwiGLU in registers
    const uint32_t lane_addr = (uint32_t)(32 * qw) << 16;
    const uint32_t t_h = tmem_base + lane_addr + 128 * m, t_out = tmem_base + lane_addr + 256 + 128 * m;
    bool ok = true;
    for (int c = 0; c < kTrChunks && ok; ++c) {
      if (qw == 0) { TR_TRACE(8 + 4 * m, c); }
      ok = mbar_wait(&bars.h_full[m], c & 1, 16u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (qw == 0) { TR_TRACE(9 + 4 * m, c); }
      tc_fence_after();
      uint32_t a[64], b[64];
      {
        uint32_t(&a0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&a[0]);
        uint32_t(&a1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&a[32]);
        uint32_t(&b0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&b[0]);
        uint32_t(&b1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&b[32]);
        tmem_ld32(t_h, a0);
        tmem_ld32(t_h + 32, a1);
        tmem_ld32(t_h + 64, b0);
        tmem_ld32(t_h + 96, b1);
        tmem_wait_ld();
      }
      if (qw == 0) { TR_TRACE(10 + 4 * m, c); }
      uint32_t w[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        // silu(a) * b = 0.5 * a * b * (1 + tanh(a / 2)): one special-function op per element
        const float a0 = __uint_as_float(a[2 * e]), a1 = __uint_as_float(a[2 * e + 1]);
        const float h0 = 0.5f * a0 * __uint_as_float(b[2 * e]), h1 = 0.5f * a1 * __uint_as_float(b[2 * e + 1]);
        w[e] = pack_bf16x2(fmaf(h0, tanh_fast(0.5f * a0), h0), fmaf(h1, tanh_fast(0.5f * a1), h1));
      }
      tmem_st32(t_h, w);                                   // h overwrites the first 32 columns of H
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.hp_ready[m]);
      if (qw == 0) { TR_TRACE(11 + 4 * m, c); }
    }
    // ------------------------------------------------------------------ residual + store, one row per thread
    if (qw == 0) { TR_TRACE(32 + m, 0); }
    ok = ok && mbar_wait(&bars.out_done[m], 0, 32u);
    ok = __all_sync(0xffffffffu, ok);
    if (qw == 0) { TR_TRACE(32 + m, 1); }
    if (ok) {
      tc_fence_after();
      // The A operand of this tile is no longer read: its first 16 KB stage 32-column blocks of the result,
      // [128 rows][32 fp32], 16-byte pieces swizzled by row.  Thread r writes row r; the same warp then reads its
      // 32 rows back with 8 lanes per row, adds the residual and stores 4 rows per instruction, coalesced.
      unsigned char* stg = sm + TransLayout::a + m * kTrABytes;
      const int srow = 32 * qw + lane;
      const int rsub = lane >> 3, piece = lane & 7;          // reader: row within a group of 4, 16-byte piece
#pragma unroll 1
      for (int q = 0; q < 4; ++q) {
        uint32_t r[32];
        tmem_ld32(t_out + 32 * q, r);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(stg + srow * 128 + ((c ^ (srow & 7)) << 4)) =
              make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rl = 32 * qw + 4 * it + rsub;
          const long long grow = row0 + 128 * m + rl;
          const float4 v = *reinterpret_cast<const float4*>(stg + rl * 128 + ((piece ^ (rl & 7)) << 4));
          if (grow < rows) {
            const size_t off = (size_t)grow * kC + 32 * q + 4 * piece;
            float4 val = v;
            if (add_residual) {
              const float4 res = load4(x_in + off);
              val.x += res.x;
              val.y += res.y;
              val.z += res.z;
              val.w += res.w;
            }
            store2(x_out + off, val.x, val.y);
            store2(x_out + off + 2, val.z, val.w);
          }
        }
        __syncwarp();
      }
    }
  }

  if (warp < 8 && (warp & 3) == 0) { TR_TRACE(32 + (warp >> 2), 2); }
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

#ifdef PX_TRANS_TRACE
}  // namespace px
extern "C" __attribute__((visibility("default"))) int px_debug_trans_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, px::g_trans_trace, sizeof(long long) * 1024);
}
namespace px {
#endif

unsigned int transition_error_flags() {
  unsigned int v = 0;
  return read_clear_tc_error(&v) == 0 ? v : 0x80u;
}

template <typename Tz>
static int32_t launch_transition(const void* x_in, void* x_out, const float* ln_w, const float* ln_b, const px_bf16* w_a,
                                 const px_bf16* w_b, const px_bf16* w_o, int64_t rows, int32_t add_residual, float eps,
                                 cudaStream_t st) {
  CUtensorMap ma, mb, mo;
  // W_a, W_b: [512 rows][128 k] bf16, box [64 rows][64 k]; W_o: [128 rows][512 k], box [128 rows][64 k]
  if (!make_map_3d(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w_a, 128, 512, 1, 256, 512 * 256, 64, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map_3d(&mb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w_b, 128, 512, 1, 256, 512 * 256, 64, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map_3d(&mo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, w_o, 512, 128, 1, 1024, 128 * 1024, 64, 128,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return PX_ERR_LAUNCH;
  const size_t smem = TransLayout::total + 1024;
  if (cudaFuncSetAttribute(transition_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t ctas = (rows + 255) / 256;
  transition_tc_kernel<Tz><<<(unsigned)ctas, 384, smem, st>>>(ma, mb, mo, (const Tz*)x_in, (Tz*)x_out, ln_w, ln_b,
                                                              (long long)rows, add_residual, eps);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_transition(const void* x_in, void* x_out, int32_t dtype, const float* ln_w, const float* ln_b,
                                 const px_bf16* w_a, const px_bf16* w_b, const px_bf16* w_o, int64_t rows,
                                 int32_t add_residual, float eps, void* stream) {
  if (!x_in || !x_out || !ln_w || !ln_b || !w_a || !w_b || !w_o || rows < 0) return PX_ERR_BAD_ARG;
  if (((uintptr_t)x_in | (uintptr_t)x_out | (uintptr_t)w_a | (uintptr_t)w_b | (uintptr_t)w_o) & 15) return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  if ((rows + 255) / 256 > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  if (dtype == PX_F32)
    return launch_transition<float>(x_in, x_out, ln_w, ln_b, w_a, w_b, w_o, rows, add_residual, eps, (cudaStream_t)stream);
  if (dtype == PX_BF16)
    return launch_transition<bf16>(x_in, x_out, ln_w, ln_b, w_a, w_b, w_o, rows, add_residual, eps, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
