// Pair bias of the single-representation attention on the 5th-generation tensor cores:
//   out[h][row] = (W LN(z[row]))[h], h < n_heads <= 16, fp32, for every pair element (row) of z.
//
// Persistent kernel, one CTA per SM, 128 rows per tile, on the row-tile pipeline of px_rowpipe.cuh (TMA-fed raw rows,
// LayerNorm folded into the resident 16 x 128 weight plus one correction K step, row statistics from a tensor-core
// Gram product).  HBM-bound: 128*sizeof(Tz) bytes read and 4*n_heads written per row.
//   warps 0..3  epilogue: a thread owns one row, reads its 16 accumulator columns and writes n_heads floats
//               (coalesced across the warp for every head);
//   warps 4..7  one thread per row: statistics, correction row, the row's rstd;
//   warp 8      TMA producer; warp 9 MMA issuer of the projection (M=128, N=16), warp 10 of the statistics product.
// Every mbarrier wait is bounded.
#include "px_rowpipe.cuh"

namespace px {

constexpr int kPbWarps = 12;
constexpr int kPbThreads = 32 * kPbWarps;
constexpr int kPbWPanel = 16 * 128;            // [16 heads][64 k] bf16
constexpr uint32_t kPbColGram = 32;            // tensor memory: projection (16 of 32 columns) | statistics (144)

struct PbBars {
  TileBars tile;
  uint64_t acc_full, acc_free;
  uint32_t tmem_base;
};
struct PbLayout {
  static constexpr int w = 0;                                   // [16][128 k] as two k panels
  static constexpr int wx = w + 2 * kPbWPanel;                  // correction panel [16][16 k]
  static constexpr int a = wx + 1024;                           // row-tile ring
  static constexpr int ax = a + kTileStages * kTileBytes;
  static constexpr int scale = ax + kTileSlots * kTileExtra;    // rstd per row and slot
  static constexpr int bars = scale + kTileSlots * 128 * 4;
  static constexpr int total = bars + (int)sizeof(PbBars);
};
static_assert(PbLayout::total + 1024 <= 232448, "shared memory budget");
static_assert(PbLayout::a % 1024 == 0, "tile ring must keep the swizzle alignment");

static __device__ float g_zero_beta[128];      // stands in for a LayerNorm without bias

// kF16: the rows are the standardised fp16 copy of an fp32 pair tensor (fp16 weights); otherwise bf16 rows of z.
template <bool kF16>
__global__ void __launch_bounds__(kPbThreads, 1)
pair_bias_tc_kernel(const __grid_constant__ CUtensorMap map_z, const float* __restrict__ ln_w,
                    const float* __restrict__ ln_b, const bf16* __restrict__ w, float* __restrict__ out, long long rows,
                    int n_heads, float eps, int n_tiles) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  PbBars& bars = *reinterpret_cast<PbBars*>(sm + PbLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TileCtx ctx;
  ctx.tiles = sm + PbLayout::a;
  ctx.extras = sm + PbLayout::ax;
  ctx.bars = &bars.tile;
  ctx.first_tile = blockIdx.x;
  ctx.tile_step = gridDim.x;
  ctx.n_tiles = n_tiles;
  ctx.tiles_t = n_tiles;                                 // the rows are one long line of tiles: u = 0, t = row
  ctx.n_u = 1;
  ctx.n_t = (int)rows;
  ctx.swap = 0;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    tile_bars_init(bars.tile, 1, kF16);
    mbar_init(&bars.acc_full, 1);
    mbar_init(&bars.acc_free, 4);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {
    fold_weight_rows<kF16, kF16>(sm + PbLayout::w, sm + PbLayout::wx, 0, kPbWPanel, w, 0, n_heads, ln_w, ln_b ? ln_b : g_zero_beta, 1.0f,
                     warp, kPbWarps, lane);
    // operand and correction rows of the heads that do not exist
    for (int i = threadIdx.x; i < (16 - n_heads) * 18; i += kPbThreads) {
      const int r = n_heads + i / 18, piece = i % 18;
      unsigned char* dst = piece < 16 ? sm + PbLayout::w + operand_piece_offset(r, piece, kPbWPanel)
                                      : sm + PbLayout::wx + r * 32 + (piece - 16) * 16;
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
    tile_write_ones<kF16>(ctx.tiles, threadIdx.x, kPbThreads);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 8) {
    if (lane == 0) {
      if (warp == 8) {
        tile_producer_loop(ctx, &map_z);
      } else if (warp == 9) {
        tile_product_loop(ctx, tmem_base, smem_u32(sm + PbLayout::w), kPbWPanel, smem_u32(sm + PbLayout::wx),
                          umma_idesc_16(128, 16, kF16, kF16), &bars.acc_full, &bars.acc_free);
      } else if (warp == 10) {
        if (!kF16) tile_gram_loop<kF16>(ctx, tmem_base + kPbColGram);   // standardised rows: nothing to measure
      }
    }
  } else if (warp >= 4) {
    float* scale = reinterpret_cast<float*>(sm + PbLayout::scale);
    tile_stats_loop<kF16>(ctx, eps, tmem_base + kPbColGram, warp - 4, lane,
                        [&](int k, int u, int t, int r, float rstd) { scale[(k % kTileSlots) * 128 + r] = rstd; });
  } else {
    // ------------------------------------------------------------------ epilogue
    const int row = 32 * warp + lane;
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * warp) << 16);
    int k = 0;
    for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
      const long long t = (long long)tile * 128 + row;
      bool ok = mbar_wait(&bars.acc_full, k & 1, 32u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float rstd = reinterpret_cast<const float*>(sm + PbLayout::scale)[(k % kTileSlots) * 128 + row];
      uint32_t acc[16];
      tmem_ld16(t_acc, acc);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free);
      if (t < rows) {
#pragma unroll
        for (int h = 0; h < 16; ++h)
          if (h < n_heads) out[(size_t)h * rows + t] = rstd * __uint_as_float(acc[h]);
      }
    }
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(pair_bias)

template <bool kF16>
static int32_t launch_pair_bias(const void* z, const float* ln_w, const float* ln_b, const px_bf16* w, float* out,
                                int64_t rows, int32_t n_heads, float eps, cudaStream_t st) {
  CUtensorMap mz;
  if (!make_map_3d(&mz, kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, z, 128, (uint64_t)rows, 1,
                   256, (uint64_t)rows * 256, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B, 1))
    return PX_ERR_LAUNCH;
  const size_t smem = PbLayout::total + 1024;
  if (cudaFuncSetAttribute(pair_bias_tc_kernel<kF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t n_tiles = (rows + 127) / 128;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  pair_bias_tc_kernel<kF16><<<grid, kPbThreads, smem, st>>>(mz, ln_w, ln_b, (const bf16*)w, out, (long long)rows,
                                                          n_heads, eps, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_pair_bias_proj(const void* z, int32_t z_dtype, const float* ln_w, const float* ln_b,
                                     const px_bf16* w, float* out, int64_t rows, int32_t n_heads, float eps,
                                     void* stream) {
  if (!z || !ln_w || !w || !out || rows < 0) return PX_ERR_BAD_ARG;
  if (n_heads <= 0 || n_heads > 16) return PX_ERR_UNSUPPORTED;
  if (((uintptr_t)z | (uintptr_t)w | (uintptr_t)ln_w | (uintptr_t)ln_b) & 15) return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  if (rows > 0x3fffffff) return PX_ERR_UNSUPPORTED;
  if (z_dtype == PX_F16) return launch_pair_bias<true>(z, ln_w, ln_b, w, out, rows, n_heads, eps, (cudaStream_t)stream);
  if (z_dtype == PX_BF16) return launch_pair_bias<false>(z, ln_w, ln_b, w, out, rows, n_heads, eps, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
