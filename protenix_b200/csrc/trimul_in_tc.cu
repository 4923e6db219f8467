// Triangle multiplication, stage 1 on the 5th-generation tensor cores:
//   a[c][u][t] = mask * (W_ap LN(z))_c * sigmoid((W_ag LN(z))_c),  b likewise, for the pair element (u, t),
//   stored channel-major with the contraction index t contiguous.
//
// Persistent kernel, one CTA per SM, 128 pair elements (one u, 128 consecutive t) per tile.  The four weight
// matrices stay in shared memory for the whole kernel with gamma and the 1/2 of the sigmoid folded in; LayerNorm's
// mean and beta terms enter the product as one extra K step, so the epilogue multiplies by the row's rstd and nothing
// else.
//
//   warps 0..7    epilogue: a thread owns one pair element (accumulator lane) and 64 of the 128 channels.  For a
//                 fixed channel the 32 lanes of a warp hold 32 consecutive t: the channel-major output is written
//                 as coalesced 64-byte runs, two bytes per lane.
//   warps 8..15   two threads per row of the tile: LayerNorm statistics (bf16 rows: read from the operand that TMA
//                 wrote; fp32 rows: read from global memory and written standardised), the correction row and the
//                 mask value.
//   warp 16       TMA producer of the bf16 row tiles, two-stage ring.
//   warp 17       MMA issuer: per tile and per output (a, b) 9 MMAs M=128 (t) N=256 (projection | gate) K=16 into
//                 one of two 256-column accumulator buffers, so the epilogue of one output overlaps the products of
//                 the next.
// Algorithmic HBM traffic per pair element: 128*sizeof(Tz) + 4 read, 512 written.  Every mbarrier wait is bounded.
#include <cstring>

#include "px_rowpipe.cuh"

namespace px {

constexpr int kTiStages = 2;
constexpr int kTiSlots = kTiStages + 1;   // row-scale slots: the epilogue reads them after the operand is freed
constexpr int kTiWPanel = 256 * 128;      // [256 rows: projection | gate][64 k] bf16
constexpr int kTiWExtra = 256 * 32;       // [256 rows][16 k] correction panel
constexpr int kTiAExtra = 128 * 32;
constexpr int kTiEpiWarps = 8;            // 4 lane quarters x 2 channel halves
constexpr int kTiStatWarps = 8;           // two threads per row of the tile
constexpr int kTiWarps = kTiEpiWarps + kTiStatWarps + 2;  // + TMA producer, MMA issuer
constexpr int kTiThreads = 32 * kTiWarps;

struct TiBars {
  uint64_t raw_full[kTiStages], a_ready[kTiStages], a_empty[kTiStages], acc_full[2], acc_free[2];
  uint32_t tmem_base;
};
struct TiLayout {
  static constexpr int w = 0;                                   // per output: two k panels
  static constexpr int wx = w + 4 * kTiWPanel;                  // per output: correction panel
  static constexpr int a = wx + 2 * kTiWExtra;                  // row-tile ring
  static constexpr int ax = a + kTiStages * kOperandBytes;      // row-tile correction panels
  static constexpr int scale = ax + kTiStages * kTiAExtra;      // float2 (rstd, rstd*mask/2) per row and slot
  static constexpr int bars = scale + kTiSlots * 128 * 8;
  static constexpr int total = bars + (int)sizeof(TiBars);
};

template <typename Tz>
__global__ void __launch_bounds__(kTiThreads, 1)
trimul_in_tc_kernel(const __grid_constant__ CUtensorMap map_z, const Tz* __restrict__ z, const float* __restrict__ mask,
                    const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w_ap,
                    const bf16* __restrict__ w_ag, const bf16* __restrict__ w_bp, const bf16* __restrict__ w_bg,
                    bf16* __restrict__ a_out, bf16* __restrict__ b_out, int n_u, int n_t, int ld, int swap, float eps,
                    int tiles_t, int n_tiles) {
  constexpr bool kTma = sizeof(Tz) == 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TiBars& bars = *reinterpret_cast<TiBars*>(sm + TiLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTiStages; ++s) {
      mbar_init(&bars.raw_full[s], 1);
      mbar_init(&bars.a_ready[s], kTiStatWarps);
      mbar_init(&bars.a_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.acc_full[b], 1);
      mbar_init(&bars.acc_free[b], kTiEpiWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == kTiEpiWarps + kTiStatWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // weights -> resident operands; the gate rows carry the 1/2 of sigmoid(x) = 1/2 + 1/2 tanh(x/2)
  {
    unsigned char* w0 = sm + TiLayout::w;
    unsigned char* x0 = sm + TiLayout::wx;
    fold_weight_rows(w0, x0, 0, kTiWPanel, w_ap, 0, 128, ln_w, ln_b, 1.0f, warp, kTiWarps, lane);
    fold_weight_rows(w0, x0, 128, kTiWPanel, w_ag, 0, 128, ln_w, ln_b, 0.5f, warp, kTiWarps, lane);
    fold_weight_rows(w0 + 2 * kTiWPanel, x0 + kTiWExtra, 0, kTiWPanel, w_bp, 0, 128, ln_w, ln_b, 1.0f, warp, kTiWarps, lane);
    fold_weight_rows(w0 + 2 * kTiWPanel, x0 + kTiWExtra, 128, kTiWPanel, w_bg, 0, 128, ln_w, ln_b, 0.5f, warp, kTiWarps, lane);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  if (warp == 0) { ROW_TRACE(12, 0); }

  if (warp >= kTiEpiWarps + kTiStatWarps) {
    if (warp == kTiEpiWarps + kTiStatWarps && lane == 0 && kTma) {
      // ---------------------------------------------------------------- row-tile producer (bf16 rows)
      int k = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++k) {
        const int s = k % kTiStages, n = k / kTiStages;
        if (!mbar_wait(&bars.a_empty[s], (n & 1) ^ 1, 1u)) break;
        ROW_TRACE(0, k);
        const int u = tile / tiles_t, t0 = (tile % tiles_t) * 128;
        mbar_expect_tx(&bars.raw_full[s], kOperandBytes);
        const uint32_t dst = smem_u32(sm + TiLayout::a + s * kOperandBytes);
        for (int p = 0; p < 2; ++p)
          tma_load_3d(dst + p * kPanelBytes, &map_z, &bars.raw_full[s], 64 * p, swap ? u : t0, swap ? t0 : u);
      }
    } else if (warp == kTiEpiWarps + kTiStatWarps + 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = umma_idesc_bf16(128, 256);
      const uint32_t w_addr = smem_u32(sm + TiLayout::w), wx_addr = smem_u32(sm + TiLayout::wx);
      int k = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++k) {
        const int s = k % kTiStages, n = k / kTiStages;
        // The products over the stored rows need only the tile; the correction step waits for the statistics,
        // which are computed meanwhile.
        if (kTma) {
          ok = mbar_wait(&bars.raw_full[s], n & 1, 2u);
        } else {
          ok = mbar_wait(&bars.a_ready[s], n & 1, 4u);
        }
        if (!ok) break;
        ROW_TRACE(1, k);
        const uint32_t a_addr = smem_u32(sm + TiLayout::a + s * kOperandBytes);
        const uint64_t ax_desc = umma_desc_sw32(smem_u32(sm + TiLayout::ax + s * kTiAExtra));
        for (int ph = 0; ph < 2 && ok; ++ph) {
          ok = mbar_wait(&bars.acc_free[ph], (k & 1) ^ 1, 8u);
          if (!ok) break;
          ROW_TRACE(2 + 2 * ph, k);
          tc_fence_after();
          const uint32_t wm = w_addr + 2 * ph * kTiWPanel;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_bf16(tmem_base + 256 * ph, umma_desc_sw128(a_addr + (ks >> 2) * kPanelBytes) + 2 * (ks & 3),
                      umma_desc_sw128(wm + (ks >> 2) * kTiWPanel) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
          if (kTma && ph == 0) {
            ok = mbar_wait(&bars.a_ready[s], n & 1, 4u);
            if (!ok) break;
            tc_fence_after();
          }
          umma_bf16(tmem_base + 256 * ph, ax_desc, umma_desc_sw32(wx_addr + ph * kTiWExtra), idesc, 1u);
          umma_commit(&bars.acc_full[ph]);
          ROW_TRACE(3 + 2 * ph, k);
        }
        if (ok) umma_commit(&bars.a_empty[s]);
      }
    }
  } else if (warp >= kTiEpiWarps) {
    // ------------------------------------------------------------------ row statistics, two threads per row
    const int r = (threadIdx.x - 32 * kTiEpiWarps) >> 1, half = threadIdx.x & 1;
    int k = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++k) {
      const int s = k % kTiStages, n = k / kTiStages;
      const int u = tile / tiles_t, t = (tile % tiles_t) * 128 + r;
      unsigned char* op = sm + TiLayout::a + s * kOperandBytes;
      const size_t pair = swap ? ((size_t)t * n_u + u) : ((size_t)u * n_t + t);
      float mk = 0.f;
      if (t < n_t && half == 0) mk = mask ? __ldg(mask + pair) : 1.f;
      float mean = 0.f, rstd = 1.f;
      if (kTma) {
        ok = mbar_wait(&bars.raw_full[s], n & 1, 16u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (warp == kTiEpiWarps) { ROW_TRACE(6, k); }
        row_stats_from_operand(op, r, half, eps, mean, rstd);
      } else {
        ok = mbar_wait(&bars.a_empty[s], (n & 1) ^ 1, 16u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (half == 0)
          standardise_row_to_operand(op, r, t < n_t ? reinterpret_cast<const float*>(z) + pair * kC : nullptr, eps);
      }
      if (half == 0) {
        // rstd * (W'x - mean * s + std * t): the row side of the correction step holds (-mean, std)
        write_correction_row(sm + TiLayout::ax + s * kTiAExtra, r, -mean, 1.0f / rstd, false);
        reinterpret_cast<float2*>(sm + TiLayout::scale)[(k % kTiSlots) * 128 + r] = make_float2(rstd, 0.5f * rstd * mk);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a_ready[s]);
      if (warp == kTiEpiWarps) { ROW_TRACE(7, k); }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int part = warp >> 2, qw = warp & 3;
    const int row = 32 * qw + lane;                      // this thread's pair element = accumulator lane
    const uint32_t t_acc = tmem_base + ((uint32_t)(32 * qw) << 16);
    const int ch_stride = n_u * ld;                      // elements between channels (both factors <= 32768)
    int k = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++k) {
      const int u = tile / tiles_t, t = (tile % tiles_t) * 128 + row;
      const bool live = t < ld;
#pragma unroll
      for (int ph = 0; ph < 2; ++ph) {
        ok = mbar_wait(&bars.acc_full[ph], k & 1, 32u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (warp == 0) { ROW_TRACE(8 + 2 * ph, k); }
        tc_fence_after();
        const float2 sc = reinterpret_cast<const float2*>(sm + TiLayout::scale)[(k % kTiSlots) * 128 + row];
        bf16* dst = (ph ? b_out : a_out) + ((size_t)(64 * part) * n_u + u) * ld + t;
        const uint32_t t_p = t_acc + 256 * ph + 64 * part, t_g = t_p + 128;
        // 16 channels: mask * p * sigmoid(g) = h + h * tanh(g / 2) with h = mask * p / 2 (the halves are folded in)
        auto emit = [&](const uint32_t(&p)[16], const uint32_t(&g)[16]) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float h = sc.y * __uint_as_float(p[e]);
            const float v = fmaf(h, tanh_fast(sc.x * __uint_as_float(g[e])), h);
            if (live) store_bf16_int(dst, v);
            dst += ch_stride;
          }
        };
        // two register sets: the next 16 columns are on their way while the current ones are worked on
        uint32_t p0[16], g0[16], p1[16], g1[16];
        tmem_ld16(t_p, p0);
        tmem_ld16(t_g, g0);
#pragma unroll 1
        for (int jj = 0; jj < 4; jj += 2) {
          tmem_wait_ld();
          tmem_ld16(t_p + 16 * (jj + 1), p1);
          tmem_ld16(t_g + 16 * (jj + 1), g1);
          emit(p0, g0);
          tmem_wait_ld();
          if (jj == 0) {
            tmem_ld16(t_p + 32, p0);
            tmem_ld16(t_g + 32, g0);
          } else {                                       // this warp has read its part of the buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.acc_free[ph]);
          }
          emit(p1, g1);
        }
        if (warp == 0) { ROW_TRACE(9 + 2 * ph, k); }
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
  if (warp == kTiEpiWarps + kTiStatWarps) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

#ifdef PX_ROW_TRACE
}  // namespace px
extern "C" __attribute__((visibility("default"))) int px_debug_row_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, px::g_row_trace, sizeof(long long) * 1024);
}
namespace px {
#endif

unsigned int trimul_in_error_flags() {
  unsigned int v = 0;
  return read_clear_tc_error(&v) == 0 ? v : 0x80u;
}

template <typename Tz>
static int32_t launch_trimul_in(const void* z, const float* mask, const float* ln_w, const float* ln_b,
                                const px_bf16* w_ap, const px_bf16* w_ag, const px_bf16* w_bp, const px_bf16* w_bg,
                                px_bf16* a, px_bf16* b, int64_t n_u, int64_t n_t, int64_t ld, int32_t incoming, float eps,
                                cudaStream_t st) {
  CUtensorMap mz;
  if (sizeof(Tz) == 2) {
    // pair element (u, t) is row u*n_t + t of z, or row t*n_u + u when the two indices are exchanged
    const bool ok = incoming ? make_map_3d(&mz, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, z, 128, (uint64_t)n_u, (uint64_t)n_t,
                                           256, (uint64_t)n_u * 256, 64, 1, CU_TENSOR_MAP_SWIZZLE_128B, 128)
                             : make_map_3d(&mz, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, z, 128, (uint64_t)n_t, (uint64_t)n_u,
                                           256, (uint64_t)n_t * 256, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B, 1);
    if (!ok) return PX_ERR_LAUNCH;
  } else {
    memset(&mz, 0, sizeof(mz));
  }
  const size_t smem = TiLayout::total + 1024;
  if (cudaFuncSetAttribute(trimul_in_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_t = (ld + 127) / 128, n_tiles = tiles_t * n_u;
  if (n_tiles > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
  trimul_in_tc_kernel<Tz><<<grid, kTiThreads, smem, st>>>(mz, (const Tz*)z, mask, ln_w, ln_b, (const bf16*)w_ap, (const bf16*)w_ag,
                                                   (const bf16*)w_bp, (const bf16*)w_bg, (bf16*)a, (bf16*)b, (int)n_u,
                                                   (int)n_t, (int)ld, incoming, eps, (int)tiles_t, (int)n_tiles);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_trimul_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w,
                                     const float* ln_b, const px_bf16* w_ap, const px_bf16* w_ag,
                                     const px_bf16* w_bp, const px_bf16* w_bg, px_bf16* a, px_bf16* b, int64_t n_u,
                                     int64_t n_t, int64_t ld, int32_t incoming, float eps, void* stream) {
  if (!z || !ln_w || !ln_b || !w_ap || !w_ag || !w_bp || !w_bg || !a || !b) return PX_ERR_BAD_ARG;
  if (n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768 || ld != px_ld(n_t)) return PX_ERR_BAD_ARG;
  if (((uintptr_t)z | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w_ap | (uintptr_t)w_ag | (uintptr_t)w_bp |
       (uintptr_t)w_bg | (uintptr_t)ln_w | (uintptr_t)ln_b) & 15)
    return PX_ERR_BAD_ARG;
  if (z_dtype == PX_F32)
    return launch_trimul_in<float>(z, mask, ln_w, ln_b, w_ap, w_ag, w_bp, w_bg, a, b, n_u, n_t, ld, incoming, eps,
                                   (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_trimul_in<bf16>(z, mask, ln_w, ln_b, w_ap, w_ag, w_bp, w_bg, a, b, n_u, n_t, ld, incoming, eps,
                                  (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
