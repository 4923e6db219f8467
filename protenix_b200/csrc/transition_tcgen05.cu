// SwiGLU transition for 128-channel rows on the 5th-generation tensor cores:
//   x_out = [x +] W_o( silu(W_a LN(x)) * (W_b LN(x)) ),  hidden width 512, the [rows][512] intermediates never
//   leave the SM (tensor memory -> registers -> tensor memory).  Both products take fp16 operands, whatever the
//   storage type of x: the rows pass through registers for the LayerNorm anyway, a normalised row and the weights
//   lie far inside the fp16 range, and fp16 keeps three more bits than bf16 (h saturates at +-65504).
//
// Persistent kernel, one CTA per SM, 128 rows per tile, three tiles in flight: while the tensor core works through
// the eight 64-wide hidden chunks of one tile, the next tile is being normalised and the previous one written out.
//
//   warps 0..7    SwiGLU: a thread owns one row and half of the current hidden chunk: it pulls a|b out of tensor
//                 memory, forms h = silu(a) * b, and writes h (fp16) back over the first 32 columns of the same
//                 H buffer as the A operand of the second product.  The two H buffers alternate.
//   warps 8..11   LayerNorm: lanes across channels (coalesced), eight rows in flight per warp; the normalised rows
//                 are written as the K-major, 128-byte-swizzled A operand of the first product (two buffers).
//   warps 12..15  output: accumulator -> shared staging -> + residual -> coalesced stores (two accumulators).
//   warp 16       TMA producer of the weight chunks: rows 64c..64c+63 of W_a and W_b and columns 64c..64c+63 of
//                 W_o, 48 KB, 3-stage ring (the weights are re-read from L2 for every tile: 384 KB per 128 rows).
//   warps 17, 18  MMA issuers: H = A [W_a;W_b]_c^T (M=128, N=128, K=128) and OUT += h W_o,c^T (M=128, N=128, K=64, h
//                 as the TMEM-resident A operand).  Two threads because a tcgen05.mma costs its issuing thread
//                 about 100 cycles.
// Tensor memory: H_0 | H_1 | OUT_0 | OUT_1, 128 columns each.  Every mbarrier wait is bounded.
#include "px_rowpipe.cuh"

namespace px {

constexpr int kTrStages = 3;
constexpr int kTrABytes = 2 * 128 * 128;            // one tile: two k panels of [128 rows][64 k] fp16
constexpr int kTrW1Bytes = 2 * 128 * 128;           // [W_a chunk; W_b chunk]: two k panels of [128 rows][64 k]
constexpr int kTrW2Bytes = 128 * 128;               // W_o chunk: [128 out rows][64 hidden]
constexpr int kTrStageBytes = kTrW1Bytes + kTrW2Bytes;
constexpr int kTrChunks = 8;                        // 512 hidden / 64
constexpr int kTrWarps = 20;
constexpr int kTrThreads = 32 * kTrWarps;

struct TransBars {
  uint64_t a_full[2], a_free[2], w_full[kTrStages], w_empty[kTrStages], h_full[2], h_free[2], p_ready[2], out_full[2],
      out_free[2];
  uint32_t tmem_base;
};
struct TransLayout {
  static constexpr int a = 0;                                  // two normalised tiles
  static constexpr int w = a + 2 * kTrABytes;                  // weight ring
  static constexpr int stg = w + kTrStages * kTrStageBytes;    // output staging: [128 rows][32 fp32]
  static constexpr int bars = stg + 128 * 128;
  static constexpr int total = bars + (int)sizeof(TransBars);
};

// Four consecutive channels as they are stored (8 or 16 bytes), so that loads can be kept in flight cheaply.
template <typename Tz>
struct Raw4;
template <>
struct Raw4<bf16> {
  uint2 v;
  __device__ __forceinline__ void load(const bf16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void zero() { v = make_uint2(0u, 0u); }
  __device__ __forceinline__ float4 get() const {
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
};
template <>
struct Raw4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ float4 get() const { return v; }
};

template <typename Tz>
__global__ void __launch_bounds__(kTrThreads, 1)
transition_tc_kernel(const __grid_constant__ CUtensorMap map_wa, const __grid_constant__ CUtensorMap map_wb,
                     const __grid_constant__ CUtensorMap map_wo, const Tz* __restrict__ x_in, Tz* __restrict__ x_out,
                     const float* __restrict__ ln_w, const float* __restrict__ ln_b, long long rows, int n_tiles,
                     int add_residual, float eps) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TransBars& bars = *reinterpret_cast<TransBars*>(sm + TransLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first_tile = blockIdx.x, tile_step = gridDim.x;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.a_full[b], 4);
      mbar_init(&bars.a_free[b], 1);
      mbar_init(&bars.h_full[b], 1);
      mbar_init(&bars.h_free[b], 1);
      mbar_init(&bars.p_ready[b], 8);
      mbar_init(&bars.out_full[b], 1);
      mbar_init(&bars.out_free[b], 4);
    }
    for (int s = 0; s < kTrStages; ++s) {
      mbar_init(&bars.w_full[s], 1);
      mbar_init(&bars.w_empty[s], 2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 16) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 16) {
    if (lane != 0) {
      // nothing: the control threads are lane 0 of their warps
    } else if (warp == 16) {
      // ---------------------------------------------------------------- weight producer
      int j = 0;                                      // chunk counter over all tiles of this CTA
      bool ok = true;
      for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step) {
        for (int c = 0; c < kTrChunks && ok; ++c, ++j) {
          const int s = j % kTrStages;
          ok = mbar_wait(&bars.w_empty[s], ((j / kTrStages) & 1) ^ 1, 1u);
          if (!ok) break;
          mbar_expect_tx(&bars.w_full[s], kTrStageBytes);
          const uint32_t base = smem_u32(sm + TransLayout::w + s * kTrStageBytes);
          for (int p = 0; p < 2; ++p) {  // k panel p: rows 0..63 from W_a, rows 64..127 from W_b
            tma_load_3d(base + p * 16384, &map_wa, &bars.w_full[s], 64 * p, 64 * c, 0);
            tma_load_3d(base + p * 16384 + 8192, &map_wb, &bars.w_full[s], 64 * p, 64 * c, 0);
          }
          tma_load_3d(base + kTrW1Bytes, &map_wo, &bars.w_full[s], 64 * c, 0, 0);
        }
      }
    } else if (warp == 17) {
      // ---------------------------------------------------------------- first product: H = A [W_a;W_b]_c^T
      constexpr uint32_t idesc = umma_idesc_f16(128, 128);
      int j = 0, k = 0;
      bool ok = true;
      for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++k) {
        const int ab = k & 1;
        ok = mbar_wait(&bars.a_full[ab], (k >> 1) & 1, 2u);
        const uint32_t a_addr = smem_u32(sm + TransLayout::a + ab * kTrABytes);
        for (int c = 0; c < kTrChunks && ok; ++c, ++j) {
          const int s = j % kTrStages, hb = j & 1;
          ok = mbar_wait(&bars.w_full[s], (j / kTrStages) & 1, 4u) && mbar_wait(&bars.h_free[hb], ((j >> 1) & 1) ^ 1, 4u);
          if (!ok) break;
          tc_fence_after();
          const uint32_t wbase = smem_u32(sm + TransLayout::w + s * kTrStageBytes);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16(tmem_base + 128 * hb, umma_desc_sw128(a_addr + (ks >> 2) * 16384) + 2 * (ks & 3),
                      umma_desc_sw128(wbase + (ks >> 2) * 16384) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
          umma_commit(&bars.h_full[hb]);
          umma_commit(&bars.w_empty[s]);                // this thread's share of the reads of the stage
        }
        if (ok) umma_commit(&bars.a_free[ab]);          // the tile has been read for the last time
      }
    } else if (warp == 18) {
      // ---------------------------------------------------------------- second product: OUT += h W_o,c^T
      constexpr uint32_t idesc = umma_idesc_f16(128, 128);
      int j = 0, k = 0;
      bool ok = true;
      for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++k) {
        const int ob = k & 1;
        ok = mbar_wait(&bars.out_free[ob], ((k >> 1) & 1) ^ 1, 8u);
        for (int c = 0; c < kTrChunks && ok; ++c, ++j) {
          const int s = j % kTrStages, hb = j & 1;
          ok = mbar_wait(&bars.w_full[s], (j / kTrStages) & 1, 4u) && mbar_wait(&bars.p_ready[hb], (j >> 1) & 1, 8u);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dwo = umma_desc_sw128(smem_u32(sm + TransLayout::w + s * kTrStageBytes) + kTrW1Bytes);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_bf16_ts(tmem_base + 256 + 128 * ob, tmem_base + 128 * hb + 8 * ks, dwo + 2 * ks, idesc, (c | ks) ? 1u : 0u);
          umma_commit(&bars.h_free[hb]);
          umma_commit(&bars.w_empty[s]);
        }
        if (ok) umma_commit(&bars.out_full[ob]);
      }
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ output rows: residual + store
    const int qw = warp - 12;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * qw) << 16);
    // Staging holds 32-column blocks of the result, [128 rows][32 fp32], 16-byte pieces swizzled by row.  Thread r
    // writes row r; the same warp then reads its 32 rows back with 8 lanes per row, adds the residual and stores
    // 4 rows per instruction, coalesced.
    unsigned char* stg = sm + TransLayout::stg;
    const int srow = 32 * qw + lane;
    const int rsub = lane >> 3, piece = lane & 7;          // reader: row within a group of 4, 16-byte piece
    int k = 0;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
      const int ob = k & 1;
      const long long row0 = (long long)tile * 128;
      // the residual values of a 32-column block are requested one block ahead (the first before the wait)
      Raw4<Tz> res[8], res_next[8];
      auto request = [&](Raw4<Tz>(&dst)[8], int q) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const long long grow = row0 + 32 * qw + 4 * it + rsub;
          if (add_residual && grow < rows) {
            dst[it].load(x_in + (size_t)grow * kC + 32 * q + 4 * piece);
          } else {
            dst[it].zero();
          }
        }
      };
      request(res_next, 0);
      bool ok = mbar_wait(&bars.out_full[ob], (k >> 1) & 1, 32u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int it = 0; it < 8; ++it) res[it] = res_next[it];
        if (q + 1 < 4) request(res_next, q + 1);
        uint32_t r[32];
        tmem_ld32(lane_addr + 256 + 128 * ob + 32 * q, r);
        tmem_wait_ld();
        if (q == 3) {                                      // this warp has read its part of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.out_free[ob]);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(stg + srow * 128 + ((c ^ (srow & 7)) << 4)) =
              make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rl = 32 * qw + 4 * it + rsub;
          const long long grow = row0 + rl;
          const float4 v = *reinterpret_cast<const float4*>(stg + rl * 128 + ((piece ^ (rl & 7)) << 4));
          if (grow < rows) {
            const size_t off = (size_t)grow * kC + 32 * q + 4 * piece;
            const float4 rs = res[it].get();
            store2(x_out + off, fmaf(2.0f, v.x, rs.x), fmaf(2.0f, v.y, rs.y));      // the second product is of h / 2
            store2(x_out + off + 2, fmaf(2.0f, v.z, rs.z), fmaf(2.0f, v.w, rs.w));
          }
        }
        __syncwarp();
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ LayerNorm -> swizzled A operand
    const int qw = warp - 8;
    // The normalised rows enter the first product halved: a' = a / 2 is the argument of the gate's tanh, b' = b / 2,
    // and h' = a' b' (1 + tanh a') = silu(a) b / 2 is what the SwiGLU warps write; the output warps double the second
    // product.  Powers of two: nothing changes but two multiplications per hidden element that are no longer needed.
    float4 g4 = *reinterpret_cast<const float4*>(ln_w + 4 * lane);
    float4 b4 = *reinterpret_cast<const float4*>(ln_b + 4 * lane);
    g4.x *= 0.5f, g4.y *= 0.5f, g4.z *= 0.5f, g4.w *= 0.5f;
    b4.x *= 0.5f, b4.y *= 0.5f, b4.z *= 0.5f, b4.w *= 0.5f;
    const int panel_off = (lane >> 4) * 16384 + (lane & 1) * 8, chunk = (lane & 15) >> 1;
    int k = 0;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
      const int ab = k & 1;
      const long long row0 = (long long)tile * 128;
      bool ok = mbar_wait(&bars.a_free[ab], ((k >> 1) & 1) ^ 1, 16u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      unsigned char* sa = sm + TransLayout::a + ab * kTrABytes;
      // eight rows per batch; the next batch is requested (as stored) before this one is reduced
      Raw4<Tz> raw[8];
      auto request = [&](int rb) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const long long grow = row0 + 32 * qw + rb + j;
          if (grow < rows) {
            raw[j].load(x_in + (size_t)grow * kC + 4 * lane);
          } else {
            raw[j].zero();
          }
        }
      };
      request(0);
#pragma unroll 1
      for (int rb = 0; rb < 32; rb += 8) {
        float4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = raw[j].get();
        if (rb + 8 < 32) request(rb + 8);
        float sum[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = x[j].x + x[j].y + x[j].z + x[j].w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += __shfl_xor_sync(0xffffffffu, sum[j], o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float mean = sum[j] * (1.0f / kC);
          x[j].x -= mean;
          x[j].y -= mean;
          x[j].z -= mean;
          x[j].w -= mean;
          sum[j] = x[j].x * x[j].x + x[j].y * x[j].y + x[j].z * x[j].z + x[j].w * x[j].w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += __shfl_xor_sync(0xffffffffu, sum[j], o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = 32 * qw + rb + j;                  // row inside the tile
          const long long grow = row0 + r;
          const float rstd = rsqrtf(sum[j] * (1.0f / kC) + eps);
          uint2 o = make_uint2(0u, 0u);
          if (grow < rows) {
            o.x = pack_f16x2(x[j].x * rstd * g4.x + b4.x, x[j].y * rstd * g4.y + b4.y);
            o.y = pack_f16x2(x[j].z * rstd * g4.z + b4.z, x[j].w * rstd * g4.w + b4.w);
          }
          *reinterpret_cast<uint2*>(sa + panel_off + r * 128 + ((chunk ^ (r & 7)) << 4)) = o;
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a_full[ab]);
    }
  } else {
    // ------------------------------------------------------------------ SwiGLU in registers
    // All eight warps work on the current hidden chunk (lane quarter x half of its 64 columns), so that the second
    // product can start after half the time; the H buffers alternate from chunk to chunk.
    const int half = warp >> 2, qw = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * qw) << 16);
    int j = 0;                                        // chunk counter over all tiles of this CTA
    bool ok = true;
    for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step) {
      for (int c = 0; c < kTrChunks && ok; ++c, ++j) {
        const int hb = j & 1;
        const uint32_t t_h = lane_addr + 128 * hb;
        ok = mbar_wait(&bars.h_full[hb], (j >> 1) & 1, 64u);
        ok = named_barrier_all(2, 256, ok);                // all eight warps go on, or none
        if (!ok) break;
        tc_fence_after();
        uint32_t w[16];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t a[16], b[16];
          tmem_ld16(t_h + 32 * half + 16 * hh, a);
          tmem_ld16(t_h + 64 + 32 * half + 16 * hh, b);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            // silu(a) * b / 2 = a' b' (1 + tanh a') with a' = a / 2, b' = b / 2 as the accumulators hold them:
            // one special-function op, one multiplication and one fused multiply-add per element
            const float a0 = __uint_as_float(a[2 * e]), a1 = __uint_as_float(a[2 * e + 1]);
            const float h0 = a0 * __uint_as_float(b[2 * e]), h1 = a1 * __uint_as_float(b[2 * e + 1]);
            w[8 * hh + e] = pack_f16x2(fmaf(h0, tanh_fast(a0), h0), fmaf(h1, tanh_fast(a1), h1));
          }
        }
        // h overwrites the first 32 columns of H; all warps must have read their a before any of them writes:
        // the a columns 0..31 of the half-0 warps are exactly where h lands
        named_barrier(2, 256);
        tmem_st16(t_h + 16 * half, w);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.p_ready[hb]);
      }
    }
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 16) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(transition)

template <typename Tz>
static int32_t launch_transition(const void* x_in, void* x_out, const float* ln_w, const float* ln_b, const px_bf16* w_a,
                                 const px_bf16* w_b, const px_bf16* w_o, int64_t rows, int32_t add_residual, float eps,
                                 cudaStream_t st) {
  CUtensorMap ma, mb, mo;
  // W_a, W_b: [512 rows][128 k] fp16, box [64 rows][64 k]; W_o: [128 rows][512 k], box [128 rows][64 k]
  if (!make_map_3d(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w_a, 128, 512, 1, 256, 512 * 256, 64, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map_3d(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w_b, 128, 512, 1, 256, 512 * 256, 64, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map_3d(&mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w_o, 512, 128, 1, 1024, 128 * 1024, 64, 128,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return PX_ERR_LAUNCH;
  const size_t smem = TransLayout::total + 1024;
  if (cudaFuncSetAttribute(transition_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t n_tiles = (rows + 127) / 128;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  transition_tc_kernel<Tz><<<grid, kTrThreads, smem, st>>>(ma, mb, mo, (const Tz*)x_in, (Tz*)x_out, ln_w, ln_b,
                                                           (long long)rows, (int)n_tiles, add_residual, eps);
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
  if ((rows + 127) / 128 > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  if (dtype == PX_F32)
    return launch_transition<float>(x_in, x_out, ln_w, ln_b, w_a, w_b, w_o, rows, add_residual, eps, (cudaStream_t)stream);
  if (dtype == PX_BF16)
    return launch_transition<bf16>(x_in, x_out, ln_w, ln_b, w_a, w_b, w_o, rows, add_residual, eps, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
