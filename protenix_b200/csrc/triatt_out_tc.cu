// Triangle attention, stage 3 on the 5th-generation tensor cores:
//   z_out(u,t) = [z_in(u,t) +] W_o ( o[u][t] * sigmoid(W_g LN(z_in(u,t))) ),
//   (u,t) = z[u][t] (starting node) or z[t][u] (ending node); z_out may alias z_in.
// Three forms (kMode): 0 = z stored as bf16 (rows multiplied as stored, output through shared memory and TMA);
// 1 = z stored as fp32 (the rows arrive as their standardised fp16 copy, residual and output fp32, coalesced through
// a staging area); 2 = only the standardised fp16 rows are at hand and the update itself is wanted, in fp16, without
// residual (the row-sharded path computes the ending-node update where the columns live and adds it where the rows
// live, so that 16-bit tensors cross NVLink in both directions).
//
// Persistent kernel, one CTA per SM, on the row-tile pipeline of px_rowpipe.cuh (TMA-fed raw rows, LayerNorm folded
// into the resident gate weights plus one correction K step, row statistics from a tensor-core Gram product).  A
// stage of the ring holds the z tile and the o tile of 128 pair elements.  Both products of a tile run on the
// tensor core; the gated rows go from registers back into tensor memory as the A operand of the second product and
// never touch shared memory.
//
//   warps 0..7    gate: a thread owns one pair element and 64 channels: g from the accumulator, o from the
//                 swizzled tile (fp16), o * sigmoid(g) packed to fp16 into tensor memory.
//   warps 8..15   output: accumulator + residual (the raw z tile still in shared memory), packed to bf16 over the
//                 o tile in place, which then leaves through a TMA store; the store addresses z[u][t] or z[t][u],
//                 so the ending node costs nothing extra.  fp32 rows are written with plain stores instead.
//   warps 16..19  one thread per row: statistics, correction row, the row's rstd.
//   warp 20       TMA producer (z and o tiles); warp 21 MMA issuer of the gate product, warp 22 of the output
//                 product (A operand in tensor memory), warp 23 of the statistics product.
// Tensor memory: gate accumulator (128) | gated rows, two fp16 per column (64) | output accumulator (128) |
// statistics (144).  Algorithmic HBM traffic per pair element: 256 + 128*sizeof(Tz) read, 128*sizeof(Tz) written.
// Every mbarrier wait is bounded.
#include <cstring>

#include "px_rowpipe.cuh"

namespace px {

constexpr int kAoWarps = 24;
constexpr int kAoThreads = 32 * kAoWarps;
constexpr uint32_t kAoColG = 0, kAoColA2 = 128, kAoColOut = 192, kAoColGram = 320;

struct AoBars {
  TileBars tile;
  uint64_t g_full, g_free, a2_ready, a2_free, out_full, out_free;
  uint32_t tmem_base;
};
struct AoLayout {
  static constexpr int wg = 0;                                  // gate weights, LayerNorm folded in
  static constexpr int wo = wg + kOperandBytes;                 // output weights
  static constexpr int wx = wo + kOperandBytes;                 // gate correction panel
  static constexpr int a = wx + 128 * 32;                       // z tiles
  static constexpr int ax = a + kTileStages * kTileBytes;       // z correction panels
  static constexpr int o = ax + kTileSlots * kTileExtra;        // o tiles (later the output rows)
  static constexpr int scale = o + kTileStages * kOperandBytes; // rstd per row and slot
  static constexpr int bars = scale + kTileSlots * 128 * 4;
  static constexpr int total = bars + (int)sizeof(AoBars);
};
static_assert(AoLayout::total + 1024 <= 232448, "shared memory budget");
static_assert(AoLayout::a % 1024 == 0 && AoLayout::o % 1024 == 0, "tiles must keep the swizzle alignment");

template <int kMode>
__global__ void __launch_bounds__(kAoThreads, 1)
triatt_out_tc_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_o,
                     const __grid_constant__ CUtensorMap map_out, const void* __restrict__ z_in, void* __restrict__ z_out,
                     const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w_g,
                     const bf16* __restrict__ w_o, int n_u, int n, int swap, int add_residual, float eps, int tiles_t,
                     int n_tiles) {
  constexpr bool kTma = kMode != 1;                      // 16-bit output: packed over the o tile, leaves through TMA
  constexpr bool kF16 = kMode != 0;                      // the z tile is a standardised fp16 copy; o, W_o always fp16
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  AoBars& bars = *reinterpret_cast<AoBars*>(sm + AoLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TileCtx ctx;
  ctx.tiles = sm + AoLayout::a;
  ctx.extras = sm + AoLayout::ax;
  ctx.bars = &bars.tile;
  ctx.first_tile = blockIdx.x;
  ctx.tile_step = gridDim.x;
  ctx.n_tiles = n_tiles;
  ctx.tiles_t = tiles_t;
  ctx.n_u = n_u;
  ctx.n_t = n;
  ctx.swap = swap;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    // a stage is read by the statistics product, the gate product and the output warps
    tile_bars_init(bars.tile, 2, kF16);
    mbar_init(&bars.g_full, 1);
    mbar_init(&bars.g_free, 8);
    mbar_init(&bars.a2_ready, 8);
    mbar_init(&bars.a2_free, 1);
    mbar_init(&bars.out_full, 1);
    mbar_init(&bars.out_free, 8);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 20) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {
    // the gate rows carry the 1/2 of sigmoid(x) = 1/2 + 1/2 tanh(x/2)
    fold_weight_rows<kF16, kF16>(sm + AoLayout::wg, sm + AoLayout::wx, 0, kPanelBytes, w_g, 0, 128, ln_w, ln_b, 0.5f, warp,
                                 kAoWarps, lane);
    // the output weights multiply the fp16 rows o * sigmoid(g) and arrive as fp16
    fold_weight_rows<true, true>(sm + AoLayout::wo, nullptr, 0, kPanelBytes, w_o, 0, 128, nullptr, nullptr, 1.0f, warp,
                                 kAoWarps, lane);
    tile_write_ones<kF16>(ctx.tiles, threadIdx.x, kAoThreads);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 20) {
    if (lane == 0) {
      if (warp == 20) {
        // ---------------------------------------------------------------- tile producer: z (bf16 rows) and o
        int k = 0;
        for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
          const int s = k % kTileStages, m = k / kTileStages;
          if (!mbar_wait(&bars.tile.a_empty[s], (m & 1) ^ 1, 1u)) break;
          const int u = tile / tiles_t, t0 = (tile % tiles_t) * 128;
          mbar_expect_tx(&bars.tile.raw_full[s], 2 * kOperandBytes);
          const uint32_t zdst = smem_u32(ctx.tiles + s * kTileBytes), odst = smem_u32(sm + AoLayout::o + s * kOperandBytes);
          for (int p = 0; p < 2; ++p) {
            tma_load_3d(zdst + p * kTilePanel, &map_z, &bars.tile.raw_full[s], 64 * p, swap ? u : t0, swap ? t0 : u);
            tma_load_3d(odst + p * kPanelBytes, &map_o, &bars.tile.raw_full[s], 64 * p, t0, u);
          }
        }
      } else if (warp == 23) {
        if (!kF16) tile_gram_loop<kF16>(ctx, tmem_base + kAoColGram);   // standardised rows: nothing to measure
      } else if (warp == 21) {
        tile_product_loop(ctx, tmem_base + kAoColG, smem_u32(sm + AoLayout::wg), kPanelBytes, smem_u32(sm + AoLayout::wx),
                          umma_idesc_16(128, 128, kF16, kF16), &bars.g_full, &bars.g_free);
      } else {
        // ---------------------------------------------------------------- output product, A operand in tensor memory
        constexpr uint32_t idesc = umma_idesc_f16(128, 128);
        const uint32_t wo_addr = smem_u32(sm + AoLayout::wo);
        int k = 0;
        for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
          if (!mbar_wait(&bars.a2_ready, k & 1, 4u) || !mbar_wait(&bars.out_free, (k & 1) ^ 1, 8u)) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16_ts(tmem_base + kAoColOut, tmem_base + kAoColA2 + 8 * ks,
                         umma_desc_sw128(wo_addr + (ks >> 2) * kPanelBytes) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
          umma_commit(&bars.out_full);
          umma_commit(&bars.a2_free);
        }
      }
    }
  } else if (warp >= 16) {
    // ------------------------------------------------------------------ row statistics, one thread per row
    float* scale = reinterpret_cast<float*>(sm + AoLayout::scale);
    tile_stats_loop<kF16>(ctx, eps, tmem_base + kAoColGram, warp - 16, lane,
                        [&](int k, int u, int t, int r, float rstd) { scale[(k % kTileSlots) * 128 + r] = rstd; });
  } else if (warp < 8) {
    // ------------------------------------------------------------------ gate: o * sigmoid(g) -> tensor memory
    const int half = warp >> 2, qw = warp & 3;
    const int row = 32 * qw + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * qw) << 16);
    int k = 0;
    for (int tile = ctx.first_tile; tile < n_tiles; tile += ctx.tile_step, ++k) {
      const int s = k % kTileStages;
      bool ok = mbar_wait(&bars.g_full, k & 1, 32u) && mbar_wait(&bars.a2_free, (k & 1) ^ 1, 32u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float rstd = reinterpret_cast<const float*>(sm + AoLayout::scale)[(k % kTileSlots) * 128 + row];
      const unsigned char* otile = sm + AoLayout::o + s * kOperandBytes;
      uint32_t packed[32];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t g[32];
        tmem_ld32(lane_addr + kAoColG + 64 * half + 32 * hh, g);
        tmem_wait_ld();
        if (hh == 1) {                                   // this warp has read its part of the gate accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.g_free);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 ov = *reinterpret_cast<const uint4*>(otile + operand_piece_offset(row, 8 * half + 4 * hh + j));
          const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 o2 = unpack_f16x2(ow[e]);
            const float s0 = fmaf(0.5f, tanh_fast(rstd * __uint_as_float(g[8 * j + 2 * e])), 0.5f);
            const float s1 = fmaf(0.5f, tanh_fast(rstd * __uint_as_float(g[8 * j + 2 * e + 1])), 0.5f);
            packed[16 * hh + 4 * j + e] = pack_f16x2(o2.x * s0, o2.y * s1);
          }
        }
      }
      tmem_st32(lane_addr + kAoColA2 + 32 * half, packed);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a2_ready);
    }
  } else {
    // ------------------------------------------------------------------ output rows
    const int half = (warp >> 2) & 1, qw = warp & 3;
    const int row = 32 * qw + lane;
    const uint32_t t_out = tmem_base + ((uint32_t)(32 * qw) << 16) + kAoColOut + 64 * half;
    const bool leader = (threadIdx.x & 255) == 0;
    int k = 0;
    bool ok = true;
    for (int tile = ctx.first_tile; tile < n_tiles && ok; tile += ctx.tile_step, ++k) {
      const int s = k % kTileStages;
      const int u = tile / tiles_t, t0 = (tile % tiles_t) * 128;
      // fp32 rows: this warp's 32 rows (u, t0 + 32 qw + i) in units of 128-channel rows of z, and their residual
      // values for the first 32 channels, requested before the wait (the second block's lines are asked of L2)
      const long long first_row = swap ? (long long)(t0 + 32 * qw) * n_u + u : (long long)u * n + t0 + 32 * qw;
      const long long row_stride = swap ? n_u : 1;
      const int valid = n - (t0 + 32 * qw) < 32 ? (n - (t0 + 32 * qw) > 0 ? n - (t0 + 32 * qw) : 0) : 32;
      RowsOutReq rq;
      if (!kTma) {
        rows_out_request(rq, reinterpret_cast<const float*>(z_in), first_row, row_stride, valid, 64 * half, lane,
                         add_residual != 0);
        if (add_residual && lane < valid)
          asm volatile("prefetch.global.L2 [%0];\n" ::"l"(reinterpret_cast<const float*>(z_in) +
                                                            (size_t)(first_row + lane * row_stride) * kC + 64 * half + 32));
        // and both blocks of the next tile, so that its requests hit L2
        const int nt = tile + ctx.tile_step;
        if (add_residual && nt < n_tiles) {
          const int u2 = nt / tiles_t, t2 = (nt % tiles_t) * 128 + 32 * qw + lane;
          if (t2 < n) {
            const float* p2 = reinterpret_cast<const float*>(z_in) + (size_t)(swap ? (long long)t2 * n_u + u2 : (long long)u2 * n + t2) * kC + 64 * half;
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p2));
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p2 + 32));
          }
        }
      }
      ok = mbar_wait(&bars.out_full, k & 1, 64u);
      ok = named_barrier_all(1, 256, ok);                  // all eight warps go on, or none
      if (!ok) break;
      tc_fence_after();
      unsigned char* otile = sm + AoLayout::o + s * kOperandBytes;
      const unsigned char* ztile = ctx.tiles + s * kTileBytes;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t acc[32];
        tmem_ld32(t_out + 32 * hh, acc);
        tmem_wait_ld();
        if (hh == 1) {                                   // this warp has read its part of the output accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.out_free);
        }
        if (kTma) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int piece = 8 * half + 4 * hh + j;
            uint32_t w[4];
            if (add_residual) {
              const uint4 zv = *reinterpret_cast<const uint4*>(ztile + operand_piece_offset(row, piece, kTilePanel));
              const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 r2 = unpack16x2<kF16>(zw[e]);
                w[e] = pack16x2<kF16>(__uint_as_float(acc[8 * j + 2 * e]) + r2.x, __uint_as_float(acc[8 * j + 2 * e + 1]) + r2.y);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack16x2<kF16>(__uint_as_float(acc[8 * j + 2 * e]), __uint_as_float(acc[8 * j + 2 * e + 1]));
            }
            *reinterpret_cast<uint4*>(otile + operand_piece_offset(row, piece)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
          // fp32 rows: coalesced through a warp-private staging area inside the o tile, which the gate warps and
          // the tensor core have finished reading (8 warps x 4 KB)
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(acc[e]);
          rows_out_store(otile + (warp & 7) * 4096, v, rq, reinterpret_cast<float*>(z_out), first_row, row_stride, valid,
                         64 * half + 32 * hh, lane);
          if (hh == 0)
            rows_out_request(rq, reinterpret_cast<const float*>(z_in), first_row, row_stride, valid, 64 * half + 32, lane,
                             add_residual != 0);
        }
      }
      if (kTma) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        named_barrier(1, 256);
        if (leader) {
          for (int p = 0; p < 2; ++p)
            tma_store_3d(&map_out, smem_u32(otile + p * kPanelBytes), 64 * p, swap ? u : t0, swap ? t0 : u);
          tma_store_commit();
          tma_store_wait_read<0>();                        // the store has read the stage: hand it back
          mbar_arrive(&bars.tile.a_empty[s]);
        }
      } else {
        named_barrier(1, 256);
        if (leader) mbar_arrive(&bars.tile.a_empty[s]);
      }
    }
    if (kTma && leader) tma_store_wait<0>();
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 20) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(triatt_out)

template <int kMode>
static int32_t launch_triatt_out(const px_f16* o, const void* z_in, const px_f16* zn, void* z_out, const float* ln_w, const float* ln_b,
                                 const px_bf16* w_g, const px_bf16* w_o, int64_t n_u, int64_t n, int32_t ending,
                                 int32_t add_residual, float eps, cudaStream_t st) {
  CUtensorMap mz, mo, mout;
  // operand rows: bf16 z itself, or the standardised fp16 copy of an fp32 z; pair element (u, t) is row u*n + t, or
  // row t*n_u + u when the two indices are exchanged
  const CUtensorMapDataType zt = kMode == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const void* zrows = kMode == 1 ? (const void*)zn : z_in;
  if (!(ending ? make_map_3d(&mz, zt, zrows, 128, (uint64_t)n_u, (uint64_t)n, 256, (uint64_t)n_u * 256, 64, 1,
                             CU_TENSOR_MAP_SWIZZLE_128B, 128)
               : make_map_3d(&mz, zt, zrows, 128, (uint64_t)n, (uint64_t)n_u, 256, (uint64_t)n * 256, 64, 128,
                             CU_TENSOR_MAP_SWIZZLE_128B, 1)))
    return PX_ERR_LAUNCH;
  if (kMode != 1) {
    if (!(ending ? make_map_3d(&mout, zt, z_out, 128, (uint64_t)n_u, (uint64_t)n, 256, (uint64_t)n_u * 256, 64, 1,
                               CU_TENSOR_MAP_SWIZZLE_128B, 128)
                 : make_map_3d(&mout, zt, z_out, 128, (uint64_t)n, (uint64_t)n_u, 256, (uint64_t)n * 256, 64, 128,
                               CU_TENSOR_MAP_SWIZZLE_128B, 1)))
      return PX_ERR_LAUNCH;
  } else {
    memset(&mout, 0, sizeof(mout));
  }
  if (!make_map_3d(&mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, o, 128, (uint64_t)n, (uint64_t)n_u, 256, (uint64_t)n * 256, 64,
                   128, CU_TENSOR_MAP_SWIZZLE_128B, 1))
    return PX_ERR_LAUNCH;
  const size_t smem = AoLayout::total + 1024;
  if (cudaFuncSetAttribute(triatt_out_tc_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_t = (n + 127) / 128, n_tiles = tiles_t * n_u;
  if (n_tiles > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  triatt_out_tc_kernel<kMode><<<grid, kAoThreads, smem, st>>>(mz, mo, mout, z_in, z_out, ln_w, ln_b,
                                                           (const bf16*)w_g, (const bf16*)w_o, (int)n_u, (int)n, ending,
                                                           add_residual, eps, (int)tiles_t, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_triatt_out(const px_f16* o, const void* z_in, const px_f16* zn, void* z_out, int32_t z_dtype,
                                 const float* ln_w, const float* ln_b, const px_w16* w_g, const px_f16* w_o, int64_t n_u,
                                 int64_t n_t, int32_t ending, int32_t add_residual, float eps, void* stream) {
  if (!o || !z_in || !z_out || !ln_w || !ln_b || !w_g || !w_o || n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F32 && (!zn || ((uintptr_t)zn & 15))) return PX_ERR_BAD_ARG;
  if (((uintptr_t)o | (uintptr_t)z_in | (uintptr_t)z_out | (uintptr_t)w_g | (uintptr_t)w_o | (uintptr_t)ln_w |
       (uintptr_t)ln_b) & 15)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F16)   // z_in: standardised fp16 rows; z_out: the update in fp16 (no residual to add)
    return add_residual ? PX_ERR_BAD_ARG
                        : launch_triatt_out<2>(o, z_in, nullptr, z_out, ln_w, ln_b, w_g, w_o, n_u, n_t, ending, 0, eps,
                                               (cudaStream_t)stream);
  if (z_dtype == PX_F32)
    return launch_triatt_out<1>(o, z_in, zn, z_out, ln_w, ln_b, w_g, w_o, n_u, n_t, ending, add_residual, eps,
                                    (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_triatt_out<0>(o, z_in, nullptr, z_out, ln_w, ln_b, w_g, w_o, n_u, n_t, ending, add_residual, eps,
                                   (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
