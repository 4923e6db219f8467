// Triangle multiplication, stage 3 on the 5th-generation tensor cores:
//   z_out[i][j] = [z_in[i][j] +] (W_z LN_out(x[:, i, j])) * sigmoid(W_g LN_in(z_in[i][j])),
//   x [128 channels][n_i][ld] fp16, channel-major and scaled by PX_TRIMUL_X_SCALE as the contraction leaves it
//   (LN_out runs with eps * scale^2, which gives exactly LN_out of the unscaled x).
//
// Persistent kernel, one CTA per SM, 128 pair elements (one i, 128 consecutive j) per tile.  Both LayerNorms are
// folded into the resident weights plus one shared correction K step (px_rowpipe.cuh); nothing is normalised or
// transposed on the way in:
//   * the z tile arrives by TMA as a K-major operand (rows of 128 channels): the bf16 rows of z themselves, or, for an
//     fp32 z, its standardised fp16 copy `zn` (px_standardise_rows), whose statistics are known;
//   * the x tile arrives by TMA exactly as it lies in memory, [128 channels][128 j], and is used as an MN-major
//     operand: the tensor core reads it transposed;
//   * the statistics of both come from Gram products (diagonal = sums of squares) and from 16 rows of ones kept
//     behind each weight matrix (columns 128..143 of the two accumulators = plain sums).
//
//   warps 0..15   epilogue: a thread owns one pair element and 32 channels: p * sigmoid(g) + residual (the raw z
//                 tile in shared memory), packed to bf16 over the z tile in place, which leaves through a TMA store.
//                 fp32 rows are written with plain stores instead.
//   warps 16..19  one thread per row: both sets of statistics, the correction row, the scale pair.
//   warp 20       TMA producer (z and x tiles); warps 21, 22 MMA issuers of the gate and of the projection product,
//                 warp 23 of the two statistics products.
// Tensor memory: gate accumulator (144) | projection accumulator (144) | statistics (128, z then x).
// Algorithmic HBM traffic per pair element: 256 + 128*sizeof(Tz) read, 128*sizeof(Tz) written.  Every wait is bounded.
#include <cstring>

#include "px_rowpipe.cuh"

namespace px {

constexpr int kToWarps = 24;
constexpr int kToThreads = 32 * kToWarps;
constexpr int kToWPanel = 144 * 128;           // [128 weight rows + 16 rows of ones][64 k]
constexpr int kToWBytes = 2 * kToWPanel;
constexpr int kToWExtra = 144 * 32;
constexpr int kToStages = 2;
constexpr int kToSlots = kToStages + 1;
constexpr uint32_t kToColG = 0, kToColP = 144, kToColGram = 288;

struct ToBars {
  uint64_t raw_full[kToStages], a_ready[kToStages], a_empty[kToStages];
  uint64_t gram_full, gram_free, main_full, acc_full, acc_free;
  uint32_t tmem_base;
};
struct ToLayout {
  static constexpr int wg = 0;                                  // gate weights | ones
  static constexpr int wz = wg + kToWBytes;                     // projection weights | ones
  static constexpr int wxg = wz + kToWBytes;                    // correction panels (k 0..7: z, k 8..15: x)
  static constexpr int wxz = wxg + kToWExtra;
  static constexpr int zt = wxz + kToWExtra;                    // z tiles (later the output rows)
  static constexpr int xt = zt + kToStages * kOperandBytes;     // x tiles, [128 c][64 j] per j block
  static constexpr int ax = xt + kToStages * kOperandBytes;     // tile-side correction panels
  static constexpr int scale = ax + kToStages * 128 * 32;       // float2 (rstd_z, rstd_x) per row and slot
  static constexpr int bars = scale + kToSlots * 128 * 8;
  static constexpr int total = bars + (int)sizeof(ToBars);
};
static_assert(ToLayout::zt % 1024 == 0 && ToLayout::xt % 1024 == 0, "tiles must keep the swizzle alignment");
static_assert(ToLayout::total + 1024 <= 232448, "shared memory budget");

template <typename Tz>
__global__ void __launch_bounds__(kToThreads, 1)
trimul_out_tc_kernel(const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ CUtensorMap map_out, const Tz* __restrict__ z_in, Tz* __restrict__ z_out,
                     const float* __restrict__ ln_in_w, const float* __restrict__ ln_in_b,
                     const float* __restrict__ ln_out_w, const float* __restrict__ ln_out_b, const bf16* __restrict__ w_z,
                     const bf16* __restrict__ w_g, int n_i, int n, int add_residual, float eps, int tiles_j, int n_tiles) {
  constexpr bool kTma = sizeof(Tz) == 2;               // bf16: residual from the z tile, output through TMA
  constexpr bool kF16 = !kTma;                           // operand format of the z side; the x side is always fp16
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  ToBars& bars = *reinterpret_cast<ToBars*>(sm + ToLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    for (int s = 0; s < kToStages; ++s) {
      mbar_init(&bars.raw_full[s], 1);
      mbar_init(&bars.a_ready[s], 4);
      mbar_init(&bars.a_empty[s], 4);                      // three issuing threads and the store of the output rows
    }
    mbar_init(&bars.gram_full, 1);
    mbar_init(&bars.gram_free, 4);
    mbar_init(&bars.main_full, 2);
    mbar_init(&bars.acc_full, 2);
    mbar_init(&bars.acc_free, 16);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 20) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  {
    // weights -> resident operands; the gate rows carry the 1/2 of sigmoid(x) = 1/2 + 1/2 tanh(x/2).  The z
    // statistics use k 0..7 of the correction step, the x statistics k 8..15.
    fold_weight_rows<kF16, kF16>(sm + ToLayout::wg, sm + ToLayout::wxg, 0, kToWPanel, w_g, 0, 128, ln_in_w, ln_in_b, 0.5f, warp, kToWarps,
                     lane, 0);
    fold_weight_rows<true, true>(sm + ToLayout::wz, sm + ToLayout::wxz, 0, kToWPanel, w_z, 0, 128, ln_out_w, ln_out_b, 1.0f, warp, kToWarps,
                     lane, 1);
    for (int i = threadIdx.x; i < 2 * 2 * 16 * 8; i += kToThreads) {   // rows of ones behind both weights
      const int panel = i >> 7, piece = i & 127;
      const uint32_t one = ones16x2(panel >= 2 || kF16);     // panels 0, 1: gate weights, 2, 3: projection
      *reinterpret_cast<uint4*>(sm + ToLayout::wg + panel * kToWPanel + 128 * 128 + piece * 16) = make_uint4(one, one, one, one);
    }
    for (int i = threadIdx.x; i < 2 * 16 * 2; i += kToThreads)         // ... which take no correction
      *reinterpret_cast<uint4*>(sm + ToLayout::wxg + (i >> 5) * kToWExtra + 128 * 32 + (i & 31) * 16) = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < kToStages * 128 * 2; i += kToThreads)  // tile-side panels start out finite
      *reinterpret_cast<uint4*>(sm + ToLayout::ax + i * 16) = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  const int first_tile = blockIdx.x, tile_step = gridDim.x;

  if (warp >= 20) {
    if (lane == 0) {
      if (warp == 20) {
        // ---------------------------------------------------------------- tile producer: z (bf16 rows) and x
        int k = 0;
        for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
          const int s = k % kToStages, m = k / kToStages;
          if (!mbar_wait(&bars.a_empty[s], (m & 1) ^ 1, 1u)) break;
          const int i = tile / tiles_j, j0 = (tile % tiles_j) * 128;
          mbar_expect_tx(&bars.raw_full[s], 2 * kOperandBytes);
          const uint32_t zdst = smem_u32(sm + ToLayout::zt + s * kOperandBytes), xdst = smem_u32(sm + ToLayout::xt + s * kOperandBytes);
          for (int p = 0; p < 2; ++p) {
            tma_load_3d(zdst + p * kPanelBytes, &map_z, &bars.raw_full[s], 64 * p, j0, i);
            tma_load_3d(xdst + p * kPanelBytes, &map_x, &bars.raw_full[s], j0 + 64 * p, i, 0);
          }
        }
      } else if (warp == 23) {
        // ---------------------------------------------------------------- statistics products: Z Z^T, then X^T X
        constexpr uint32_t idesc_z = umma_idesc_16(128, 128, kF16, kF16), idesc_x = umma_idesc_f16(128, 128, true, true);
        int k = 0;
        for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
          const int s = k % kToStages, m = k / kToStages;
          // bf16 rows: two phases of the statistics accumulator per tile (z, then x); standardised rows have known
          // statistics, so only x is measured and the phases alternate from tile to tile
          if (!mbar_wait(&bars.raw_full[s], m & 1, 2u) || !mbar_wait(&bars.gram_free, kF16 ? ((k & 1) ^ 1) : 1u, 2u)) break;
          tc_fence_after();
          const uint32_t z_addr = smem_u32(sm + ToLayout::zt + s * kOperandBytes), x_addr = smem_u32(sm + ToLayout::xt + s * kOperandBytes);
          if (!kF16) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t d = umma_desc_sw128(z_addr + (ks >> 2) * kPanelBytes) + 2 * (ks & 3);
              umma_bf16(tmem_base + kToColGram, d, d, idesc_z, ks ? 1u : 0u);
            }
            umma_commit(&bars.gram_full);
            if (!mbar_wait(&bars.gram_free, 0u, 2u)) break;
            tc_fence_after();
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t d = umma_desc_mn_sw128(x_addr + ks * 2048, kPanelBytes, 1024);
            umma_bf16(tmem_base + kToColGram, d, d, idesc_x, ks ? 1u : 0u);
          }
          umma_commit(&bars.gram_full);
          umma_commit(&bars.a_empty[s]);
        }
      } else {
        // ---------------------------------------------------------------- gate (warp 21) / projection (warp 22) product
        const bool proj = warp == 22;
        const uint32_t idesc = proj ? umma_idesc_f16(128, 144, true, false) : umma_idesc_16(128, 144, kF16, kF16);
        const uint32_t d_tmem = tmem_base + (proj ? kToColP : kToColG);
        const uint32_t w_addr = smem_u32(sm + (proj ? ToLayout::wz : ToLayout::wg));
        const uint64_t wx_desc = umma_desc_sw32(smem_u32(sm + (proj ? ToLayout::wxz : ToLayout::wxg)));
        int k = 0;
        for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
          const int s = k % kToStages, m = k / kToStages;
          if (!mbar_wait(&bars.raw_full[s], m & 1, 4u) || !mbar_wait(&bars.acc_free, (k & 1) ^ 1, 8u)) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sm + (proj ? ToLayout::xt : ToLayout::zt) + s * kOperandBytes);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t a_desc = proj ? umma_desc_mn_sw128(a_addr + ks * 2048, kPanelBytes, 1024)
                                         : umma_desc_sw128(a_addr + (ks >> 2) * kPanelBytes) + 2 * (ks & 3);
            umma_bf16(d_tmem, a_desc, umma_desc_sw128(w_addr + (ks >> 2) * kToWPanel) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
          }
          umma_commit(&bars.main_full);                        // the sums (columns 128..143) are there
          if (!mbar_wait(&bars.a_ready[s], m & 1, 4u)) break;  // the correction step needs the statistics
          tc_fence_after();
          umma_bf16(d_tmem, umma_desc_sw32(smem_u32(sm + ToLayout::ax + s * 128 * 32)), wx_desc,
                    umma_idesc_bf16(128, 144, false, false), 1u);
          umma_commit(&bars.acc_full);
          umma_commit(&bars.a_empty[s]);
        }
      }
    }
  } else if (warp >= 16) {
    // ------------------------------------------------------------------ row statistics, one thread per row
    const int qw = warp - 16, r = 32 * qw + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * qw) << 16);
    float2* scale = reinterpret_cast<float2*>(sm + ToLayout::scale);
    int k = 0;
    bool ok = true;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++k) {
      const int s = k % kToStages;
      float sumsq[2] = {0.f, 0.f};
#pragma unroll
      for (int which = kF16 ? 1 : 0; which < 2; ++which) {   // 0: z (bf16 rows only), 1: x
        ok = mbar_wait(&bars.gram_full, kF16 ? (k & 1) : which, 16u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t diag[32];
        tmem_ld32(lane_addr + kToColGram + 32 * qw, diag);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.gram_free);
        sumsq[which] = select_own(diag, lane);
      }
      if (!ok) break;
      ok = mbar_wait(&bars.main_full, k & 1, 16u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sz[16], sx[16];
      tmem_ld16(lane_addr + kToColG + 128, sz);
      tmem_ld16(lane_addr + kToColP + 128, sx);
      tmem_wait_ld();
      tc_fence_before();
      float rstd[2];
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        float mean = __uint_as_float(which ? sx[0] : sz[0]) * (1.0f / kC);
        const float var = fmaxf(sumsq[which] * (1.0f / kC) - mean * mean, 0.f);
        const float e = which ? eps * (PX_TRIMUL_X_SCALE * PX_TRIMUL_X_SCALE) : eps;   // x arrives scaled
        float std = sqrtf(var + e);
        rstd[which] = rsqrtf(var + e);
        if (kF16 && which == 0) mean = 0.f, std = 1.f, rstd[0] = 1.f;   // standardised rows: known statistics
        // rstd * (W'x - mean * s + std * t): the row side of the correction step holds (-mean, std)
        write_correction_row(sm + ToLayout::ax + s * 128 * 32, r, -mean, std, false, which, false);
      }
      scale[(k % kToSlots) * 128 + r] = make_float2(rstd[0], rstd[1]);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a_ready[s]);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int part = warp >> 2, qw = warp & 3;
    const int row = 32 * qw + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * qw) << 16);
    const bool leader = threadIdx.x == 0;
    int k = 0;
    bool ok = true;
    for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++k) {
      const int s = k % kToStages;
      const int i = tile / tiles_j, j0 = (tile % tiles_j) * 128;
      RowsOutReq rq;
      if (!kTma) {                                         // the residual values are requested before the wait
        const int valid = n - (j0 + 32 * qw) < 32 ? (n - (j0 + 32 * qw) > 0 ? n - (j0 + 32 * qw) : 0) : 32;
        rows_out_request(rq, reinterpret_cast<const float*>(z_in), (long long)i * n + j0 + 32 * qw, 1, valid, 32 * part, lane,
                         add_residual != 0);
        // the residual lines of the next tile are asked of L2 now: a tile later they are a hit, not a trip to HBM
        const int nt = tile + tile_step;
        if (add_residual && nt < n_tiles) {
          const int i2 = nt / tiles_j, j2 = (nt % tiles_j) * 128 + 32 * qw + lane;
          if (j2 < n)
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(reinterpret_cast<const float*>(z_in) + ((size_t)i2 * n + j2) * kC + 32 * part));
        }
      }
      ok = mbar_wait(&bars.acc_full, k & 1, 32u);
      ok = named_barrier_all(1, 512, ok);                  // all sixteen warps go on, or none
      if (!ok) break;
      tc_fence_after();
      const float2 sc = reinterpret_cast<const float2*>(sm + ToLayout::scale)[(k % kToSlots) * 128 + row];
      unsigned char* ztile = sm + ToLayout::zt + s * kOperandBytes;
      uint32_t g[32], p[32];
      tmem_ld32(lane_addr + kToColG + 32 * part, g);
      tmem_ld32(lane_addr + kToColP + 32 * part, p);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_free);          // this warp has read its part of the accumulators
      float v[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        // p * sigmoid(g) = h + h * tanh(g / 2) with h = p / 2 (the half of g is folded into the weights)
        const float h = 0.5f * sc.y * __uint_as_float(p[e]);
        v[e] = fmaf(h, tanh_fast(sc.x * __uint_as_float(g[e])), h);
      }
      if (kTma) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          unsigned char* piece = ztile + operand_piece_offset(row, 4 * part + q);
          uint32_t w[4];
          if (add_residual) {
            const uint4 zv = *reinterpret_cast<const uint4*>(piece);
            const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 r2 = unpack_bf16x2(zw[e]);
              w[e] = pack_bf16x2_int(v[8 * q + 2 * e] + r2.x, v[8 * q + 2 * e + 1] + r2.y);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) w[e] = pack_bf16x2_int(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
          }
          *reinterpret_cast<uint4*>(piece) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        named_barrier(1, 512);
        if (leader) {
          for (int pnl = 0; pnl < 2; ++pnl) tma_store_3d(&map_out, smem_u32(ztile + pnl * kPanelBytes), 64 * pnl, j0, i);
          tma_store_commit();
          tma_store_wait_read<0>();                          // the store has read the stage: hand it back
          mbar_arrive(&bars.a_empty[s]);
        }
      } else {
        // fp32 rows: coalesced through a warp-private staging area inside the stage's tiles, which the tensor core
        // has finished reading (16 warps x 4 KB = the z tile and the x tile)
        unsigned char* stg = sm + (warp < 8 ? ToLayout::zt : ToLayout::xt) + s * kOperandBytes + (warp & 7) * 4096;
        const int valid = n - (j0 + 32 * qw) < 32 ? (n - (j0 + 32 * qw) > 0 ? n - (j0 + 32 * qw) : 0) : 32;
        rows_out_store(stg, v, rq, reinterpret_cast<float*>(z_out), (long long)i * n + j0 + 32 * qw, 1, valid, 32 * part, lane);
        named_barrier(1, 512);
        if (leader) mbar_arrive(&bars.a_empty[s]);
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

PX_DEFINE_FAMILY_HOOKS(trimul_out)

template <typename Tz>
static int32_t launch_trimul_out(const px_f16* x, const void* z_in, const px_f16* zn, void* z_out, const float* ln_in_w, const float* ln_in_b,
                                 const float* ln_out_w, const float* ln_out_b, const px_bf16* w_z, const px_bf16* w_g,
                                 int64_t n_i, int64_t n, int64_t ld, int32_t add_residual, float eps, cudaStream_t st) {
  CUtensorMap mz, mx, mout;
  // operand rows: bf16 z itself, or the standardised fp16 copy of an fp32 z
  if (!make_map_3d(&mz, sizeof(Tz) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   sizeof(Tz) == 2 ? z_in : (const void*)zn, 128, (uint64_t)n, (uint64_t)n_i, 256, (uint64_t)n * 256, 64, 128,
                   CU_TENSOR_MAP_SWIZZLE_128B, 1))
    return PX_ERR_LAUNCH;
  if (sizeof(Tz) == 2) {
    if (!make_map_3d(&mout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, z_out, 128, (uint64_t)n, (uint64_t)n_i, 256, (uint64_t)n * 256,
                     64, 128, CU_TENSOR_MAP_SWIZZLE_128B, 1))
      return PX_ERR_LAUNCH;
  } else {
    memset(&mout, 0, sizeof(mout));
  }
  // x [128 channels][n_i][ld]: a load brings [128 channels][one i][64 j]
  if (!make_map_3d(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)ld, (uint64_t)n_i, 128, (uint64_t)ld * 2,
                   (uint64_t)n_i * ld * 2, 64, 1, CU_TENSOR_MAP_SWIZZLE_128B, 128))
    return PX_ERR_LAUNCH;
  const size_t smem = ToLayout::total + 1024;
  if (cudaFuncSetAttribute(trimul_out_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_j = (n + 127) / 128, n_tiles = tiles_j * n_i;
  if (n_tiles > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  trimul_out_tc_kernel<Tz><<<grid, kToThreads, smem, st>>>(mz, mx, mout, (const Tz*)z_in, (Tz*)z_out, ln_in_w, ln_in_b,
                                                           ln_out_w, ln_out_b, (const bf16*)w_z, (const bf16*)w_g, (int)n_i,
                                                           (int)n, add_residual, eps, (int)tiles_j, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_trimul_out(const px_f16* x, const void* z_in, const px_f16* zn, void* z_out, int32_t z_dtype,
                                 const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                 const float* ln_out_b, const px_f16* w_z, const px_w16* w_g, int64_t n_i,
                                 int64_t n_j, int64_t ld, int32_t add_residual, float eps, void* stream) {
  if (!x || !z_in || !z_out || !ln_in_w || !ln_in_b || !ln_out_w || !ln_out_b || !w_z || !w_g) return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F32 && (!zn || ((uintptr_t)zn & 15))) return PX_ERR_BAD_ARG;
  if (n_i <= 0 || n_j <= 0 || n_i > 32768 || n_j > 32768 || ld != px_ld(n_j)) return PX_ERR_BAD_ARG;
  if (((uintptr_t)x | (uintptr_t)z_in | (uintptr_t)z_out | (uintptr_t)w_z | (uintptr_t)w_g | (uintptr_t)ln_in_w |
       (uintptr_t)ln_in_b | (uintptr_t)ln_out_w | (uintptr_t)ln_out_b) & 15)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F32)
    return launch_trimul_out<float>(x, z_in, zn, z_out, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_z, w_g, n_i, n_j, ld,
                                    add_residual, eps, (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_trimul_out<bf16>(x, z_in, nullptr, z_out, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_z, w_g, n_i, n_j, ld,
                                   add_residual, eps, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
