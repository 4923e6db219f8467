// Triangle attention, stage 1 on the 5th-generation tensor cores:
//   LN(z) -> q, k [u][h][t][32] (q pre-scaled by log2(e)/sqrt(32)), v transposed [u][h][32][ld] (zero pad columns),
//   in fp16 (projections of standardised rows: far inside its range), bias[h][u][t] = log2(e) * (W_bias LN(z))_h (zero
//   pad columns) and mask_bias[u][t] = log2(e) * inf * (mask - 1) (-inf in the pad columns) in fp32, for the pair
//   element (u, t) = z[u][t] (starting node) or z[t][u] (ending node).
//
// Persistent kernel, one CTA per SM, on the row-tile pipeline of px_rowpipe.cuh (TMA-fed raw rows, LayerNorm folded
// into the resident weights plus one correction K step, row statistics from a tensor-core Gram product).  The CTAs
// work in pairs on the same tiles; CTA parity picks two of the four heads.
//
//   warps 0..7    epilogue of q | k: a thread owns one pair element and both heads of q (warps 0..3) or k (4..7):
//                 64-byte runs per head, coalesced across the warp.
//   warps 8..15   epilogue of v | bias: v goes through a [64 d][128 t] staging tile and a TMA store (the transpose),
//                 the two bias values of the row are written directly.
//   warps 16..19  one thread per row: statistics, correction row, scale pair, mask bias.
//   warp 20       TMA producer; warps 21, 22 MMA issuers of the two products (N = 128 and N = 80), warp 23 of the
//                 statistics product.
// Algorithmic HBM traffic per pair element: 256 + 4 read, 3*256 + 16 + 4 written.  Every wait is bounded.
#include <math_constants.h>

#include "px_rowpipe.cuh"

namespace px {

constexpr int kAiH = 4, kAiD = 32;
constexpr int kAiW1Panel = 80 * 128;           // [v 64 | bias 16][64 k]
constexpr int kAiStageOut = 64 * 256;          // [64 d][128 t] fp16
constexpr int kAiWarps = 24;
constexpr int kAiThreads = 32 * kAiWarps;
constexpr uint32_t kAiColGram = 256;           // tensor memory: q|k (128) | v|bias (80) | - | statistics (144);
                                               // standardised rows: a second set of accumulators at 256 instead

struct AiBars {
  TileBars tile;
  uint64_t acc_full[2][2], acc_free[2][2];   // [product][accumulator]
  uint32_t tmem_base;
};
struct AiLayout {
  static constexpr int w0 = 0;                                  // [q 64 | k 64][128 k]
  static constexpr int w1 = w0 + kOperandBytes;                 // [v 64 | bias 16][128 k]
  static constexpr int wx0 = w1 + 2 * kAiW1Panel;               // correction panels
  static constexpr int wx1 = wx0 + 128 * 32;
  static constexpr int a = wx1 + 128 * 32;                      // row-tile ring
  static constexpr int ax = a + kTileStages * kTileBytes;
  static constexpr int out = ax + kTileSlots * kTileExtra;      // v staging
  static constexpr int scale = out + kAiStageOut;               // float2 (rstd, rstd or 0 beyond n) per row and slot
  static constexpr int bars = scale + kTileSlots * 128 * 8;
  static constexpr int total = bars + (int)sizeof(AiBars);
};
static_assert(AiLayout::total + 1024 <= 232448, "shared memory budget");
static_assert(AiLayout::a % 1024 == 0, "tile ring must keep the swizzle alignment");

// kF16: the rows are the standardised fp16 copy of an fp32 pair tensor (fp16 weights); otherwise bf16 rows of z.
template <bool kF16>
__global__ void __launch_bounds__(kAiThreads, 1)
triatt_in_tc_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_v,
                    const float* __restrict__ mask, const float* __restrict__ ln_w,
                    const float* __restrict__ ln_b, const bf16* __restrict__ w_q, const bf16* __restrict__ w_k,
                    const bf16* __restrict__ w_v, const bf16* __restrict__ w_bias, bf16* __restrict__ q_out,
                    bf16* __restrict__ k_out, float* __restrict__ bias_out, float* __restrict__ mb_out, int n_u, int n,
                    int ldm, int swap, float eps, float inf, int tiles_t, int n_tiles) {
  constexpr int kAiAcc = kF16 ? 2 : 1;   // accumulators per product: the products of tile k+1 run beside the epilogue of k
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  AiBars& bars = *reinterpret_cast<AiBars*>(sm + AiLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hpair = blockIdx.x & 1;                      // this CTA's heads: 2*hpair, 2*hpair + 1
  TileCtx ctx;
  ctx.tiles = sm + AiLayout::a;
  ctx.extras = sm + AiLayout::ax;
  ctx.bars = &bars.tile;
  ctx.first_tile = blockIdx.x >> 1;
  ctx.tile_step = gridDim.x >> 1;
  ctx.n_tiles = n_tiles;
  ctx.tiles_t = tiles_t;
  ctx.n_u = n_u;
  ctx.n_t = n;
  ctx.swap = swap;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    tile_bars_init(bars.tile, 2, kF16);
    for (int b = 0; b < 4; ++b) {
      mbar_init(&bars.acc_full[b >> 1][b & 1], 1);
      mbar_init(&bars.acc_free[b >> 1][b & 1], 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 20) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {
    // weights -> resident operands (q carries the softmax scale, the bias rows log2(e))
    const float qscale = kLog2e * rsqrtf((float)kAiD);
    fold_weight_rows<kF16, kF16>(sm + AiLayout::w0, sm + AiLayout::wx0, 0, kPanelBytes, w_q, 64 * hpair, 64, ln_w, ln_b, qscale, warp,
                     kAiWarps, lane);
    fold_weight_rows<kF16, kF16>(sm + AiLayout::w0, sm + AiLayout::wx0, 64, kPanelBytes, w_k, 64 * hpair, 64, ln_w, ln_b, 1.0f, warp,
                     kAiWarps, lane);
    fold_weight_rows<kF16, kF16>(sm + AiLayout::w1, sm + AiLayout::wx1, 0, kAiW1Panel, w_v, 64 * hpair, 64, ln_w, ln_b, 1.0f, warp,
                     kAiWarps, lane);
    fold_weight_rows<kF16, kF16>(sm + AiLayout::w1, sm + AiLayout::wx1, 64, kAiW1Panel, w_bias, 2 * hpair, 2, ln_w, ln_b, kLog2e, warp,
                     kAiWarps, lane);
    // rows 66..79 of the second operand (and of its correction panel) are padding
    for (int i = threadIdx.x; i < 14 * 18; i += kAiThreads) {
      const int r = 66 + i / 18, piece = i % 18;
      unsigned char* dst = piece < 16 ? sm + AiLayout::w1 + operand_piece_offset(r, piece, kAiW1Panel)
                                      : sm + AiLayout::wx1 + r * 32 + (piece - 16) * 16;
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    tile_write_ones<kF16>(ctx.tiles, threadIdx.x, kAiThreads);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 20) {
    if (lane == 0) {
      if (warp == 20) {
        tile_producer_loop(ctx, &map_z);
      } else if (warp == 23) {
        if (!kF16) tile_gram_loop<kF16>(ctx, tmem_base + kAiColGram);   // standardised rows: nothing to measure
      } else if (warp == 21) {
        tile_product_loop(ctx, tmem_base, smem_u32(sm + AiLayout::w0), kPanelBytes, smem_u32(sm + AiLayout::wx0),
                          umma_idesc_16(128, 128, kF16, kF16), bars.acc_full[0], bars.acc_free[0], kAiAcc, 256);
      } else {
        tile_product_loop(ctx, tmem_base + 128, smem_u32(sm + AiLayout::w1), kAiW1Panel, smem_u32(sm + AiLayout::wx1),
                          umma_idesc_16(128, 80, kF16, kF16), bars.acc_full[1], bars.acc_free[1], kAiAcc, 256);
      }
    }
  } else if (warp >= 16) {
    // ------------------------------------------------------------------ row statistics, one thread per row
    float2* scale = reinterpret_cast<float2*>(sm + AiLayout::scale);
    tile_stats_loop<kF16>(ctx, eps, tmem_base + kAiColGram, warp - 16, lane, [&](int k, int u, int t, int r, float rstd) {
      scale[(k % kTileSlots) * 128 + r] = make_float2(rstd, t < n ? rstd : 0.f);
      if (hpair == 0 && t < ldm) {                       // mask bias, -inf in the pad columns [n, ldm)
        float mv = -CUDART_INF_F;
        if (t < n)
          mv = mask ? (__ldg(mask + (swap ? ((size_t)t * n_u + u) : ((size_t)u * n + t))) - 1.0f) * inf * kLog2e : 0.f;
        mb_out[(size_t)u * ldm + t] = mv;
      }
    });
  } else if (warp < 8) {
    // ------------------------------------------------------------------ epilogue of q | k
    const int which = warp >> 2, qw = warp & 3;          // 0: q, 1: k
    const int row = 32 * qw + lane;
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * qw) << 16) + 64 * which;
    bf16* out = which ? k_out : q_out;
    int k = 0;
    for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
      const int u = tile / tiles_t, t = (tile % tiles_t) * 128 + row;
      const int ab = kAiAcc == 2 ? (k & 1) : 0, an = kAiAcc == 2 ? (k >> 1) : k;
      bool ok = mbar_wait(&bars.acc_full[0][ab], an & 1, 32u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float rstd = reinterpret_cast<const float2*>(sm + AiLayout::scale)[(k % kTileSlots) * 128 + row].x;
      uint32_t h0[32], h1[32];
      tmem_ld32(t_acc + 256 * ab, h0);
      tmem_ld32(t_acc + 256 * ab + 32, h1);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free[0][ab]);  // this warp has read its part of the accumulator
      if (t < n) {
        auto emit = [&](const uint32_t(&v)[32], int head) {
          uint4* dst = reinterpret_cast<uint4*>(out + (((size_t)u * kAiH + head) * n + t) * kAiD);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_f16x2(rstd * __uint_as_float(v[8 * j + 0]), rstd * __uint_as_float(v[8 * j + 1]));
            o.y = pack_f16x2(rstd * __uint_as_float(v[8 * j + 2]), rstd * __uint_as_float(v[8 * j + 3]));
            o.z = pack_f16x2(rstd * __uint_as_float(v[8 * j + 4]), rstd * __uint_as_float(v[8 * j + 5]));
            o.w = pack_f16x2(rstd * __uint_as_float(v[8 * j + 6]), rstd * __uint_as_float(v[8 * j + 7]));
            dst[j] = o;
          }
        };
        emit(h0, 2 * hpair);
        emit(h1, 2 * hpair + 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue of v | bias
    const int half = (warp >> 2) & 1, qw = warp & 3;
    const int row = 32 * qw + lane;
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * qw) << 16) + 128 + 32 * half;
    const bool leader = (threadIdx.x & 255) == 0;
    unsigned char* stage = sm + AiLayout::out + (32 * half) * 256 + row * 2;
    int k = 0;
    bool ok = true;
    for (int tile = ctx.first_tile; tile < n_tiles && ok; tile += ctx.tile_step, ++k) {
      const int u = tile / tiles_t, t0 = (tile % tiles_t) * 128, t = t0 + row;
      const int ab = kAiAcc == 2 ? (k & 1) : 0, an = kAiAcc == 2 ? (k >> 1) : k;
      ok = mbar_wait(&bars.acc_full[1][ab], an & 1, 64u);
      // the store that last read the staging buffer (one tile ago) must be through with it
      if (leader) tma_store_wait_read<0>();
      ok = named_barrier_all(1, 256, ok);                  // all eight warps go on, or none
      if (!ok) break;
      tc_fence_after();
      const float2 sc = reinterpret_cast<const float2*>(sm + AiLayout::scale)[(k % kTileSlots) * 128 + row];
      uint32_t v[32], b[16];
      tmem_ld32(t_acc + 256 * ab, v);
      if (half == 0) tmem_ld16(tmem_base + ((uint32_t)(32 * qw) << 16) + 256 * ab + 128 + 64, b);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free[1][ab]);  // this warp has read its part of the accumulator
#pragma unroll
      for (int e = 0; e < 32; ++e)
        *reinterpret_cast<__half*>(stage + e * 256) = __float2half_rn(sc.y * __uint_as_float(v[e]));
      if (half == 0 && t < ldm) {                        // zero in the pad columns [n, ldm)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          bias_out[((size_t)(2 * hpair + e) * n_u + u) * ldm + t] = sc.y * __uint_as_float(b[e]);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      named_barrier(1, 256);
      if (leader) {
        tma_store_3d(&map_v, smem_u32(sm + AiLayout::out), t0, u * 128 + 64 * hpair, 0);
        tma_store_commit();
      }
    }
    if (leader) tma_store_wait<0>();
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 20) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(triatt_in)

template <bool kF16>
static int32_t launch_triatt_in(const void* z, const float* mask, const float* ln_w, const float* ln_b,
                                const px_bf16* w_q, const px_bf16* w_k, const px_bf16* w_v, const px_bf16* w_bias,
                                px_f16* q, px_f16* k, px_f16* v, float* bias, float* mask_bias, int64_t n_u,
                                int64_t n, int64_t ldm, int32_t ending, float eps, float inf, cudaStream_t st) {
  CUtensorMap mz, mv;
  const CUtensorMapDataType zt = kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // pair element (u, t) is row u*n + t of z, or row t*n_u + u when the two indices are exchanged
  const bool ok = ending ? make_map_3d(&mz, zt, z, 128, (uint64_t)n_u, (uint64_t)n, 256, (uint64_t)n_u * 256, 64, 1,
                                       CU_TENSOR_MAP_SWIZZLE_128B, 128)
                         : make_map_3d(&mz, zt, z, 128, (uint64_t)n, (uint64_t)n_u, 256, (uint64_t)n * 256, 64, 128,
                                       CU_TENSOR_MAP_SWIZZLE_128B, 1);
  if (!ok) return PX_ERR_LAUNCH;
  // v is [n_u * 128 rows (u, head, d)][ldt]: a store writes [64 rows][128 t]
  const uint64_t ldt = (uint64_t)px_ld(n);
  if (!make_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, v, ldt, (uint64_t)n_u * 128, 1, ldt * 2, ldt * 2 * n_u * 128, 128,
                   64, CU_TENSOR_MAP_SWIZZLE_NONE, 1))
    return PX_ERR_LAUNCH;
  const size_t smem = AiLayout::total + 1024;
  if (cudaFuncSetAttribute(triatt_in_tc_kernel<kF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_t = (n + 127) / 128, n_tiles = tiles_t * n_u;   // 128-wide tiles cover the pad columns up to ldm
  if (n_tiles > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int pairs = (int)(n_tiles < sm_count() / 2 ? n_tiles : sm_count() / 2);
  triatt_in_tc_kernel<kF16><<<2 * pairs, kAiThreads, smem, st>>>(mz, mv, mask, ln_w, ln_b, (const bf16*)w_q,
                                                               (const bf16*)w_k, (const bf16*)w_v, (const bf16*)w_bias,
                                                               (bf16*)q, (bf16*)k, bias, mask_bias, (int)n_u, (int)n,
                                                               (int)ldm, ending, eps, inf, (int)tiles_t, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_triatt_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w,
                                     const float* ln_b, const px_bf16* w_q, const px_bf16* w_k, const px_bf16* w_v,
                                     const px_bf16* w_bias, px_f16* q, px_f16* k, px_f16* v, float* bias,
                                     float* mask_bias, int64_t n_u, int64_t n_t, int64_t ldm, int32_t ending,
                                     float eps, float inf, void* stream) {
  if (!z || !ln_w || !ln_b || !w_q || !w_k || !w_v || !w_bias || !q || !k || !v || !bias || !mask_bias)
    return PX_ERR_BAD_ARG;
  if (n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768 || ldm != px_ld_mask(n_t)) return PX_ERR_BAD_ARG;
  if (((uintptr_t)z | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)w_q | (uintptr_t)w_k | (uintptr_t)w_v |
       (uintptr_t)w_bias | (uintptr_t)ln_w | (uintptr_t)ln_b) & 15)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F16)   // standardised rows of an fp32 pair tensor (px_standardise_rows)
    return launch_triatt_in<true>(z, mask, ln_w, ln_b, w_q, w_k, w_v, w_bias, q, k, v, bias, mask_bias, n_u, n_t, ldm,
                                   ending, eps, inf, (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_triatt_in<false>(z, mask, ln_w, ln_b, w_q, w_k, w_v, w_bias, q, k, v, bias, mask_bias, n_u, n_t, ldm,
                                  ending, eps, inf, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
