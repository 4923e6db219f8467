// Triangle multiplication, stage 1 on the 5th-generation tensor cores:
//   a[c][u][t] = mask * (W_ap LN(z))_c * sigmoid((W_ag LN(z))_c),  b likewise, for the pair element (u, t),
//   stored channel-major in fp16 with the contraction index t contiguous.  (a and b are products of a bounded gate
//   and a projection of a standardised row: far inside the fp16 range, and fp16 keeps three more bits than bf16.)
//
// Persistent kernel, one CTA per SM.  A tile is 128 pair elements (one u, 128 consecutive t); the CTAs work in
// pairs on the same sequence of tiles, each CTA producing 64 of the 128 channels of a and of b (the second read of
// a tile comes from L2).  Halving the weights a CTA keeps resident leaves shared memory for output staging and
// tensor memory for the row statistics (px_rowpipe.cuh has the parts shared with the other row kernels):
//   * The weights stay in shared memory for the whole kernel with gamma and the 1/2 of the sigmoid folded in;
//     LayerNorm's mean and beta terms enter the product as one extra K step (see px_rowpipe.cuh).
//   * The row statistics come from the tensor core as well: Z Z^T has the sums of squares on its diagonal, and 16
//     rows of ones kept behind every tile in shared memory add the plain sums as columns 128..143 of that product.
//     Variance = E[x^2] - mean^2 in fp32: accurate while |mean| is not orders of magnitude above the deviation.
//   * The gated outputs are staged as [channel][t] in shared memory (two-byte stores, conflict-free) and leave
//     through TMA stores, 256-byte runs per channel.
//
//   warps 0..7    epilogue of output a: a thread owns one pair element (accumulator lane) and 32 of the CTA's 64
//                 channels; warps 8..15 do the same for output b, concurrently.
//   warps 16..19  one thread per row: reads the two statistics out of tensor memory, writes the correction row and
//                 the row's scale pair.
//   warp 20       TMA producer of the row tiles (bf16 rows of z, or standardised fp16 rows), two-stage ring.
//   warps 21..23  MMA issuers (a tcgen05.mma costs its issuing thread 100 cycles and more, so the work is split):
//                 warp 21 output a, warp 22 output b, each 8 MMAs M=128 (t) N=128 (projection | gate) K=16 plus the
//                 correction step; warp 23 the statistics product (8 MMAs, N=144).
// Algorithmic HBM traffic per pair element: 256 + 4 read, 512 written.  Every mbarrier wait is bounded.
#include "px_rowpipe.cuh"

namespace px {

constexpr int kTiWExtra = 128 * 32;            // [128 rows][16 k] weight-side correction panel
constexpr int kTiStageOut = 64 * 256;          // [64 channels][128 t] fp16
constexpr int kTiWarps = 24;
constexpr int kTiThreads = 32 * kTiWarps;
constexpr uint32_t kTiColGram = 256;           // tensor memory: out a | out b | statistics (144 columns); standardised
                                               // rows need no statistics product: a second pair of accumulators there

struct TiBars {
  TileBars tile;
  uint64_t acc_full[2][2], acc_free[2][2];   // [output][accumulator]
  uint32_t tmem_base;
};
struct TiLayout {
  static constexpr int w = 0;                                   // per output: [projection 64 | gate 64][128 k]
  static constexpr int wx = w + 2 * kOperandBytes;              // per output: correction panel
  static constexpr int a = wx + 2 * kTiWExtra;                  // row-tile ring
  static constexpr int ax = a + kTileStages * kTileBytes;       // row-tile correction panels
  static constexpr int out = ax + kTileSlots * kTileExtra;      // output staging, one buffer per output
  static constexpr int scale = out + 2 * kTiStageOut;           // float2 (rstd, rstd*mask/2) per row and slot
  static constexpr int bars = scale + kTileSlots * 128 * 8;
  static constexpr int total = bars + (int)sizeof(TiBars);
};
static_assert(TiLayout::total + 1024 <= 232448, "shared memory budget");

// kF16: the rows are the standardised fp16 copy of an fp32 pair tensor (fp16 weights); otherwise bf16 rows of z.
template <bool kF16>
__global__ void __launch_bounds__(kTiThreads, 1)
trimul_in_tc_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const float* __restrict__ mask,
                    const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w_ap,
                    const bf16* __restrict__ w_ag, const bf16* __restrict__ w_bp, const bf16* __restrict__ w_bg,
                    int n_u, int n_t, int swap, float eps, int tiles_t, int n_tiles) {
  constexpr int kTiAcc = kF16 ? 2 : 1;   // accumulators per output: the products of tile k+1 run beside the epilogue of k
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TiBars& bars = *reinterpret_cast<TiBars*>(sm + TiLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chan0 = 64 * (blockIdx.x & 1);               // this CTA's channels of a and b
  TileCtx ctx;
  ctx.tiles = sm + TiLayout::a;
  ctx.extras = sm + TiLayout::ax;
  ctx.bars = &bars.tile;
  ctx.first_tile = blockIdx.x >> 1;
  ctx.tile_step = gridDim.x >> 1;
  ctx.n_tiles = n_tiles;
  ctx.tiles_t = tiles_t;
  ctx.n_u = n_u;
  ctx.n_t = n_t;
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
    // weights -> resident operands; the gate rows carry the 1/2 of sigmoid(x) = 1/2 + 1/2 tanh(x/2)
    unsigned char* w0 = sm + TiLayout::w;
    unsigned char* x0 = sm + TiLayout::wx;
    fold_weight_rows<kF16, kF16>(w0, x0, 0, kPanelBytes, w_ap, chan0, 64, ln_w, ln_b, 1.0f, warp, kTiWarps, lane);
    fold_weight_rows<kF16, kF16>(w0, x0, 64, kPanelBytes, w_ag, chan0, 64, ln_w, ln_b, 0.5f, warp, kTiWarps, lane);
    fold_weight_rows<kF16, kF16>(w0 + kOperandBytes, x0 + kTiWExtra, 0, kPanelBytes, w_bp, chan0, 64, ln_w, ln_b, 1.0f, warp, kTiWarps, lane);
    fold_weight_rows<kF16, kF16>(w0 + kOperandBytes, x0 + kTiWExtra, 64, kPanelBytes, w_bg, chan0, 64, ln_w, ln_b, 0.5f, warp, kTiWarps, lane);
    tile_write_ones<kF16>(ctx.tiles, threadIdx.x, kTiThreads);
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
        if (!kF16) tile_gram_loop<kF16>(ctx, tmem_base + kTiColGram);   // standardised rows: nothing to measure
      } else {
        const int ph = warp - 21;                          // MMA issuer of output ph
        tile_product_loop(ctx, tmem_base + 128 * ph, smem_u32(sm + TiLayout::w) + ph * kOperandBytes, kPanelBytes,
                          smem_u32(sm + TiLayout::wx) + ph * kTiWExtra, umma_idesc_16(128, 128, kF16, kF16), bars.acc_full[ph],
                          bars.acc_free[ph], kTiAcc, 256);
      }
    }
  } else if (warp >= 16) {
    // ------------------------------------------------------------------ row statistics, one thread per row
    float2* scale = reinterpret_cast<float2*>(sm + TiLayout::scale);
    tile_stats_loop<kF16>(ctx, eps, tmem_base + kTiColGram, warp - 16, lane, [&](int k, int u, int t, int r, float rstd) {
      float mk = 0.f;
      if (t < n_t) mk = mask ? __ldg(mask + (swap ? ((size_t)t * n_u + u) : ((size_t)u * n_t + t))) : 1.f;
      scale[(k % kTileSlots) * 128 + r] = make_float2(rstd, 0.5f * rstd * mk);
    });
  } else {
    // ------------------------------------------------------------------ epilogue of output ph
    const int ph = warp >> 3, half = (warp >> 2) & 1, qw = warp & 3;
    const int row = 32 * qw + lane;                      // this thread's pair element = accumulator lane
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * qw) << 16) + 128 * ph + 32 * half;
    const bool leader = (threadIdx.x & 255) == 0;
    const CUtensorMap* map_out = ph ? &map_b : &map_a;
    unsigned char* stage = sm + TiLayout::out + ph * kTiStageOut + (32 * half) * 256 + row * 2;
    int k = 0;
    bool ok = true;
    for (int tile = ctx.first_tile; tile < n_tiles && ok; tile += ctx.tile_step, ++k) {
      const int u = tile / tiles_t, t0 = (tile % tiles_t) * 128;
      const int ab = kTiAcc == 2 ? (k & 1) : 0, an = kTiAcc == 2 ? (k >> 1) : k;
      const uint32_t t_buf = t_acc + 256 * ab;
      ok = mbar_wait(&bars.acc_full[ph][ab], an & 1, 32u);
      // the store that last read the staging buffer (one tile ago) must be through with it
      if (leader) tma_store_wait_read<0>();
      ok = named_barrier_all(1 + ph, 256, ok);             // all eight warps go on, or none
      if (!ok) break;
      tc_fence_after();
      const float2 sc = reinterpret_cast<const float2*>(sm + TiLayout::scale)[(k % kTileSlots) * 128 + row];
      // mask * p * sigmoid(g) = h + h * tanh(g / 2) with h = mask * p / 2 (the halves are folded in)
      auto emit = [&](const uint32_t(&p)[16], const uint32_t(&g)[16], int hh) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float h = sc.y * __uint_as_float(p[e]);
          const float v = fmaf(h, tanh_fast(sc.x * __uint_as_float(g[e])), h);
          *reinterpret_cast<__half*>(stage + (16 * hh + e) * 256) = __float2half_rn(v);
        }
      };
      uint32_t p0[16], g0[16], p1[16], g1[16];
      tmem_ld16(t_buf, p0);
      tmem_ld16(t_buf + 64, g0);
      tmem_ld16(t_buf + 16, p1);
      tmem_ld16(t_buf + 64 + 16, g1);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free[ph][ab]);  // this warp has read its part of the accumulator
      emit(p0, g0, 0);
      emit(p1, g1, 1);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      named_barrier(1 + ph, 256);
      if (leader) {
        tma_store_3d(map_out, smem_u32(sm + TiLayout::out + ph * kTiStageOut), t0, u, chan0);
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

PX_DEFINE_FAMILY_HOOKS(trimul_in)

template <bool kF16>
static int32_t launch_trimul_in(const void* z, const float* mask, const float* ln_w, const float* ln_b,
                                const px_w16* w_ap, const px_w16* w_ag, const px_w16* w_bp, const px_w16* w_bg,
                                px_f16* a, px_f16* b, int64_t n_u, int64_t n_t, int64_t ld, int32_t incoming, float eps,
                                cudaStream_t st) {
  CUtensorMap mz, ma, mb;
  const CUtensorMapDataType zt = kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // pair element (u, t) is row u*n_t + t of z, or row t*n_u + u when the two indices are exchanged
  const bool ok = incoming ? make_map_3d(&mz, zt, z, 128, (uint64_t)n_u, (uint64_t)n_t, 256, (uint64_t)n_u * 256, 64, 1,
                                         CU_TENSOR_MAP_SWIZZLE_128B, 128)
                           : make_map_3d(&mz, zt, z, 128, (uint64_t)n_t, (uint64_t)n_u, 256, (uint64_t)n_t * 256, 64, 128,
                                         CU_TENSOR_MAP_SWIZZLE_128B, 1);
  if (!ok) return PX_ERR_LAUNCH;
  // outputs [128 channels][n_u][ld]: a store writes [64 channels][one u][128 t]
  if (!make_map_3d(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, (uint64_t)ld, (uint64_t)n_u, 128, (uint64_t)ld * 2,
                   (uint64_t)n_u * ld * 2, 128, 1, CU_TENSOR_MAP_SWIZZLE_NONE, 64) ||
      !make_map_3d(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, b, (uint64_t)ld, (uint64_t)n_u, 128, (uint64_t)ld * 2,
                   (uint64_t)n_u * ld * 2, 128, 1, CU_TENSOR_MAP_SWIZZLE_NONE, 64))
    return PX_ERR_LAUNCH;
  const size_t smem = TiLayout::total + 1024;
  if (cudaFuncSetAttribute(trimul_in_tc_kernel<kF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_t = (ld + 127) / 128, n_tiles = tiles_t * n_u;
  if (n_tiles > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int pairs = (int)(n_tiles < sm_count() / 2 ? n_tiles : sm_count() / 2);
  trimul_in_tc_kernel<kF16><<<2 * pairs, kTiThreads, smem, st>>>(mz, ma, mb, mask, ln_w, ln_b, (const bf16*)w_ap,
                                                                 (const bf16*)w_ag, (const bf16*)w_bp, (const bf16*)w_bg,
                                                                 (int)n_u, (int)n_t, incoming, eps, (int)tiles_t,
                                                                 (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_trimul_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w,
                                     const float* ln_b, const px_w16* w_ap, const px_w16* w_ag,
                                     const px_w16* w_bp, const px_w16* w_bg, px_f16* a, px_f16* b, int64_t n_u,
                                     int64_t n_t, int64_t ld, int32_t incoming, float eps, void* stream) {
  if (!z || !ln_w || !ln_b || !w_ap || !w_ag || !w_bp || !w_bg || !a || !b) return PX_ERR_BAD_ARG;
  if (n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768 || ld != px_ld(n_t)) return PX_ERR_BAD_ARG;
  if (((uintptr_t)z | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w_ap | (uintptr_t)w_ag | (uintptr_t)w_bp |
       (uintptr_t)w_bg | (uintptr_t)ln_w | (uintptr_t)ln_b) & 15)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F16)   // standardised rows of an fp32 pair tensor (px_standardise_rows)
    return launch_trimul_in<true>(z, mask, ln_w, ln_b, w_ap, w_ag, w_bp, w_bg, a, b, n_u, n_t, ld, incoming, eps,
                                  (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_trimul_in<false>(z, mask, ln_w, ln_b, w_ap, w_ag, w_bp, w_bg, a, b, n_u, n_t, ld, incoming, eps,
                                   (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
