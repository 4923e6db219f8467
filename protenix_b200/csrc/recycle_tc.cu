// Recycling update of the pair representation on the 5th-generation tensor cores:
//   out[row] = z_init[row] + W LN(z[row]),   W [128][128], one row per pair element
// (protenix/model/protenix.py:246: z = z_init + linear_no_bias_z_cycle(layernorm_z_cycle(z))).
//
// Persistent kernel, one CTA per SM, 128 rows per tile, on the row-tile pipeline of px_rowpipe.cuh (TMA-fed raw rows,
// LayerNorm folded into the resident weight plus one correction K step, row statistics from a tensor-core Gram
// product).  HBM-bound: per row 128*sizeof(Tz) bytes of z and of z_init are read and as many written.
//   warps 0..7   output rows: a thread owns one row and 64 of its channels, adds rstd * accumulator to the z_init
//                tile in shared memory (brought in by TMA, in place) and one thread stores the tile by TMA;
//                fp32 rows read z_init from global memory and use plain stores;
//   warps 8..11  one thread per row: statistics, correction row, the row's rstd;
//   warp 12      TMA producer (z tiles and z_init tiles); warp 13 MMA issuer of the projection (M=128, N=128),
//   warp 14      MMA issuer of the statistics product.
// `out` may be the same buffer as `z` or as `z_init`: a tile is written only after all of its reads.
// Every mbarrier wait is bounded.
#include <cstring>

#include "px_rowpipe.cuh"

namespace px {

constexpr int kRcWarps = 15;
constexpr int kRcThreads = 32 * kRcWarps;
constexpr uint32_t kRcColGram = 128;           // tensor memory: projection (128 columns) | statistics (144)

struct RcBars {
  TileBars tile;
  uint64_t acc_full, acc_free, res_full[kTileStages], res_empty[kTileStages];
  uint32_t tmem_base;
};
struct RcLayout {
  static constexpr int w = 0;                                   // [128][128 k] as two k panels
  static constexpr int wx = w + kOperandBytes;                  // correction panel [128][16 k]
  static constexpr int a = wx + 128 * 32;                       // row-tile ring
  static constexpr int ax = a + kTileStages * kTileBytes;
  static constexpr int res = ax + kTileSlots * kTileExtra;      // z_init tiles, then the output tiles, in place
  static constexpr int scale = res + kTileStages * kOperandBytes;  // rstd per row and slot
  static constexpr int bars = scale + kTileSlots * 128 * 4;
  static constexpr int total = bars + (int)sizeof(RcBars);
};
static_assert(RcLayout::total + 1024 <= 232448, "shared memory budget");
static_assert(RcLayout::a % 1024 == 0 && RcLayout::res % 1024 == 0, "tiles must keep the swizzle alignment");

static __device__ float g_rc_zero_beta[128];   // stands in for a LayerNorm without bias

template <typename Tz>
__global__ void __launch_bounds__(kRcThreads, 1)
recycle_tc_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_init,
                  const __grid_constant__ CUtensorMap map_out, const Tz* z_init, Tz* out,
                  const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w,
                  long long rows, float eps, int n_tiles) {
  constexpr bool kTma = sizeof(Tz) == 2;               // bf16: z_init and out go through shared memory and TMA
  constexpr bool kF16 = !kTma;                           // fp32: the rows of z arrive as a standardised fp16 copy
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  RcBars& bars = *reinterpret_cast<RcBars*>(sm + RcLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TileCtx ctx;
  ctx.tiles = sm + RcLayout::a;
  ctx.extras = sm + RcLayout::ax;
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
    mbar_init(&bars.acc_free, 8);
    for (int s = 0; s < kTileStages; ++s) {
      mbar_init(&bars.res_full[s], 1);
      mbar_init(&bars.res_empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 12) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  fold_weight_rows<kF16, kF16>(sm + RcLayout::w, sm + RcLayout::wx, 0, kPanelBytes, w, 0, 128, ln_w, ln_b ? ln_b : g_rc_zero_beta, 1.0f,
                   warp, kRcWarps, lane);
  tile_write_ones<kF16>(ctx.tiles, threadIdx.x, kRcThreads);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 12) {
    if (lane == 0) {
      if (warp == 12) {
        // z tile into the operand ring and (bf16) the z_init tile into the output ring
        int k = 0;
        for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
          const int s = k % kTileStages, n = k / kTileStages;
          if (!mbar_wait(&bars.tile.a_empty[s], (n & 1) ^ 1, 1u)) break;
          mbar_expect_tx(&bars.tile.raw_full[s], kOperandBytes);
          const uint32_t dst = smem_u32(ctx.tiles + s * kTileBytes);
          for (int p = 0; p < 2; ++p) tma_load_3d(dst + p * kTilePanel, &map_z, &bars.tile.raw_full[s], 64 * p, tile * 128, 0);
          if (kTma) {
            if (!mbar_wait(&bars.res_empty[s], (n & 1) ^ 1, 1u)) break;
            mbar_expect_tx(&bars.res_full[s], kOperandBytes);
            const uint32_t rdst = smem_u32(sm + RcLayout::res + s * kOperandBytes);
            for (int p = 0; p < 2; ++p) tma_load_3d(rdst + p * kPanelBytes, &map_init, &bars.res_full[s], 64 * p, tile * 128, 0);
          }
        }
      } else if (warp == 13) {
        tile_product_loop(ctx, tmem_base, smem_u32(sm + RcLayout::w), kPanelBytes, smem_u32(sm + RcLayout::wx),
                          umma_idesc_16(128, 128, kF16, kF16), &bars.acc_full, &bars.acc_free);
      } else if (warp == 14) {
        if (!kF16) tile_gram_loop<kF16>(ctx, tmem_base + kRcColGram);   // standardised rows: nothing to measure
      }
    }
  } else if (warp >= 8) {
    float* scale = reinterpret_cast<float*>(sm + RcLayout::scale);
    tile_stats_loop<kF16>(ctx, eps, tmem_base + kRcColGram, warp - 8, lane,
                        [&](int k, int u, int t, int r, float rstd) { scale[(k % kTileSlots) * 128 + r] = rstd; });
  } else {
    // ------------------------------------------------------------------ output rows
    const int half = (warp >> 2) & 1, qw = warp & 3;
    const int row = 32 * qw + lane;
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * qw) << 16) + 64 * half;
    const bool leader = threadIdx.x == 0;
    int k = 0;
    bool ok = true;
    for (int tile = ctx.first_tile; tile < n_tiles && ok; tile += ctx.tile_step, ++k) {
      const int s = k % kTileStages, n = k / kTileStages;
      // fp32 rows: this warp's 32 rows and their z_init values for the first 32 channels, requested before the wait
      const long long first_row = (long long)tile * 128 + 32 * qw;
      const int valid = rows - first_row < 32 ? (rows - first_row > 0 ? (int)(rows - first_row) : 0) : 32;
      RowsOutReq rq;
      if (!kTma) {
        rows_out_request(rq, reinterpret_cast<const float*>(z_init), first_row, 1, valid, 64 * half, lane, true);
        // z_init of the next tile is asked of L2 now (both 32-channel blocks of this warp's rows)
        const long long r2 = (long long)(tile + ctx.tile_step) * 128 + 32 * qw + lane;
        if (r2 < rows) {
          const float* p2 = reinterpret_cast<const float*>(z_init) + (size_t)r2 * kC + 64 * half;
          asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p2));
          asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p2 + 32));
        }
      }
      ok = mbar_wait(&bars.acc_full, k & 1, 32u);
      if (kTma) ok = ok && mbar_wait(&bars.res_full[s], n & 1, 33u);
      ok = named_barrier_all(1, 256, ok);                  // all eight warps go on, or none
      if (!ok) break;
      tc_fence_after();
      const float rstd = reinterpret_cast<const float*>(sm + RcLayout::scale)[(k % kTileSlots) * 128 + row];
      unsigned char* rtile = sm + RcLayout::res + s * kOperandBytes;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t acc[32];
        tmem_ld32(t_acc + 32 * hh, acc);
        tmem_wait_ld();
        if (hh == 1) {                                     // this warp has read its part of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.acc_free);
        }
        if (kTma) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            unsigned char* piece = rtile + operand_piece_offset(row, 8 * half + 4 * hh + j);
            const uint4 iv = *reinterpret_cast<const uint4*>(piece);
            const uint32_t iw[4] = {iv.x, iv.y, iv.z, iv.w};
            uint32_t ow[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 r2 = unpack_bf16x2(iw[e]);
              ow[e] = pack_bf16x2_int(fmaf(rstd, __uint_as_float(acc[8 * j + 2 * e]), r2.x),
                                      fmaf(rstd, __uint_as_float(acc[8 * j + 2 * e + 1]), r2.y));
            }
            *reinterpret_cast<uint4*>(piece) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        } else {
          // fp32 rows: coalesced through a warp-private 4 KB staging area in the z_init ring, which this mode does
          // not otherwise use (z_init is read straight from global memory, in the arrangement of the stores)
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = rstd * __uint_as_float(acc[e]);
          rows_out_store(sm + RcLayout::res + warp * 4096, v, rq, reinterpret_cast<float*>(out), first_row, 1, valid,
                         64 * half + 32 * hh, lane);
          if (hh == 0)
            rows_out_request(rq, reinterpret_cast<const float*>(z_init), first_row, 1, valid, 64 * half + 32, lane, true);
        }
      }
      if (kTma) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        named_barrier(1, 256);
        if (leader) {
          for (int p = 0; p < 2; ++p) tma_store_3d(&map_out, smem_u32(rtile + p * kPanelBytes), 64 * p, tile * 128, 0);
          tma_store_commit();
          tma_store_wait_read<0>();                        // the store has read the tile: hand it back
          mbar_arrive(&bars.res_empty[s]);
        }
      }
    }
    if (kTma && leader) tma_store_wait<0>();
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 12) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(recycle)

template <typename Tz>
static int32_t launch_recycle(const void* z, const void* z_init, void* out, const float* ln_w, const float* ln_b,
                              const px_bf16* w, int64_t rows, float eps, cudaStream_t st) {
  CUtensorMap mz, mi, mo;
  // the rows of z: bf16 as stored, or the standardised fp16 copy
  if (!make_map_3d(&mz, sizeof(Tz) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, z, 128,
                   (uint64_t)rows, 1, 256, (uint64_t)rows * 256, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B, 1))
    return PX_ERR_LAUNCH;
  if (sizeof(Tz) == 2) {
    const void* base[2] = {z_init, out};
    CUtensorMap* maps[2] = {&mi, &mo};
    for (int i = 0; i < 2; ++i)
      if (!make_map_3d(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base[i], 128, (uint64_t)rows, 1, 256, (uint64_t)rows * 256,
                       64, 128, CU_TENSOR_MAP_SWIZZLE_128B, 1))
        return PX_ERR_LAUNCH;
  } else {
    memset(&mi, 0, sizeof(mi));
    memset(&mo, 0, sizeof(mo));
  }
  const size_t smem = RcLayout::total + 1024;
  if (cudaFuncSetAttribute(recycle_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t n_tiles = (rows + 127) / 128;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  recycle_tc_kernel<Tz><<<grid, kRcThreads, smem, st>>>(mz, mi, mo, (const Tz*)z_init, (Tz*)out, ln_w, ln_b,
                                                        (const bf16*)w, (long long)rows, eps, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_recycle_update(const void* z, const void* z_init, void* out, int32_t z_dtype, const float* ln_w,
                                     const float* ln_b, const px_bf16* w, int64_t rows, float eps, void* stream) {
  if (!z || !z_init || !out || !ln_w || !w || rows < 0) return PX_ERR_BAD_ARG;
  if (((uintptr_t)z | (uintptr_t)z_init | (uintptr_t)out | (uintptr_t)w | (uintptr_t)ln_w | (uintptr_t)ln_b) & 15)
    return PX_ERR_BAD_ARG;
  if (rows == 0) return PX_OK;
  if (rows > 0x3fffff80) return PX_ERR_UNSUPPORTED;
  if (z_dtype == PX_F32) return launch_recycle<float>(z, z_init, out, ln_w, ln_b, w, rows, eps, (cudaStream_t)stream);
  if (z_dtype == PX_BF16) return launch_recycle<bf16>(z, z_init, out, ln_w, ln_b, w, rows, eps, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
