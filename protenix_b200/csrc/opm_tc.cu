// Outer product mean of the MSA module, the N^2-heavy part on the 5th-generation tensor cores
// (protenix/model/triangular/layers.py:657-780, c_hidden = 32, c_z = 128):
//
//   outer[i][j][c][e] = sum_s a[s][i][c] * b[s][j][e]                 px_opm_outer: the contraction kernel of the
//                                                                      triangle multiplication (contract_tcgen05.cu)
//                                                                      on operands [(i,c)][s] and [(j,e)][s]
//   z_out[i][j][:] = [z_in[i][j][:] +] (W_out . outer[i][j][:] + bias) * inv_norm[i][j]          this file
//
// The first stage leaves x[(i,c)][(j,e)] = 2^-6 outer in fp16, one row per (i, c).  For a fixed i the 1024 inputs
// of pair (i, j) are the 32 x 32 block at rows 32 i + c, columns 32 j + e: seen as a 3-D tensor (e, j, row) a TMA box
// [4 c][128 j][32 e] with the 64-byte swizzle is, per c, exactly a K-major UMMA operand of 128 rows (j) x 32 k (e),
// so the gather of the reference's reshape costs nothing.  W_out[o][32 c + e] is cut the same way.
//
// Persistent kernel, one CTA per SM, 192 threads, tile = (i, 128 j):
//   warp 0      TMA producer: per stage 4 c-slabs of x (32 KB) and the matching 4 slabs of W_out (32 KB, from L2),
//               3-stage ring
//   warp 1      one thread: 8 x tcgen05.mma M=128 (j) N=128 (o) K=16 per stage, 8 stages per tile, two accumulators
//   warps 2..5  epilogue: (acc * 2^6 + bias) * inv_norm + residual; fp32 rows go out coalesced through a 4 KB
//               staging area per warp, bf16 rows as 64-byte runs
// HBM-bound: 2048 bytes of x per pair element against 2 * 128 * 1024 FLOP.  Every mbarrier wait is bounded.
// The entry point takes a block of n_i rows i (pointers of x, inv_norm and z at the block's first row), so that a
// caller can bound the size of x: (32 n_i) x (32 N) fp16.
#include "px_rowpipe.cuh"

namespace px {

constexpr int kOpCc = 4;                       // c-slabs per stage
constexpr int kOpSlab = 128 * 64;              // [128 rows][32 k] fp16, 64-byte swizzle
constexpr int kOpStageBytes = 2 * kOpCc * kOpSlab;
constexpr int kOpStages = 3;
constexpr int kOpKSteps = 32 / kOpCc;          // stages per tile
constexpr uint32_t kOpCols = 256;              // two fp32 accumulators of 128 columns

struct OpBars {
  uint64_t full[kOpStages], empty[kOpStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};
struct OpLayout {
  static constexpr int ring = 0;
  static constexpr int stg = ring + kOpStages * kOpStageBytes;   // 4 warps x 4 KB
  static constexpr int bars = stg + 4 * 4096;
  static constexpr int total = bars + (int)sizeof(OpBars);
};
static_assert(OpLayout::total + 1024 <= 232448, "shared memory budget");

template <typename Tz>
__global__ void __launch_bounds__(192, 1)
opm_out_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const float* __restrict__ bias, const float* __restrict__ inv_norm, const Tz* z_in,
                  Tz* z_out, int n, int add_residual, int tiles_j, int total_tiles) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  OpBars& bars = *reinterpret_cast<OpBars*>(sm + OpLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    for (int s = 0; s < kOpStages; ++s) {
      mbar_init(&bars.full[s], 1);
      mbar_init(&bars.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.acc_full[b], 1);
      mbar_init(&bars.acc_empty[b], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(kOpCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int i = tile / tiles_j, j0 = (tile % tiles_j) * 128;
        for (int kc = 0; kc < kOpKSteps && ok; ++kc, ++it) {
          const int s = it % kOpStages;
          ok = mbar_wait(&bars.empty[s], ((it / kOpStages) & 1) ^ 1, 1u);
          if (!ok) break;
          mbar_expect_tx(&bars.full[s], kOpStageBytes);
          const uint32_t sa = smem_u32(sm + OpLayout::ring + s * kOpStageBytes);
          tma_load_3d(sa, &map_x, &bars.full[s], 0, j0, 32 * i + kOpCc * kc);            // [4 c][128 j][32 e]
          tma_load_3d(sa + kOpCc * kOpSlab, &map_w, &bars.full[s], 0, 0, kOpCc * kc);     // [4 c][128 o][32 e]
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(128, 128);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t ab = tcount & 1;
        ok = mbar_wait(&bars.acc_empty[ab], ((tcount >> 1) & 1) ^ 1, 2u);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + 128 * ab;
        for (int kc = 0; kc < kOpKSteps; ++kc, ++it) {
          const int s = it % kOpStages;
          ok = mbar_wait(&bars.full[s], (it / kOpStages) & 1, 4u);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(sm + OpLayout::ring + s * kOpStageBytes);
#pragma unroll
          for (int cc = 0; cc < kOpCc; ++cc) {
            const uint64_t da = umma_desc_sw64(sa + cc * kOpSlab), db = umma_desc_sw64(sa + (kOpCc + cc) * kOpSlab);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)   // 16 fp16 = 32 bytes = 2 units of the start-address field
              umma_bf16(d_tmem, da + 2 * ks, db + 2 * ks, idesc, (kc | cc | ks) ? 1u : 0u);
          }
          umma_commit(&bars.empty[s]);
        }
        if (!ok) break;
        umma_commit(&bars.acc_full[ab]);
      }
    }
  } else {
    constexpr bool kF32 = sizeof(Tz) == 4;
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    unsigned char* stg = sm + OpLayout::stg + q * 4096;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
      const int i = tile / tiles_j, j0 = (tile % tiles_j) * 128;
      const uint32_t ab = tcount & 1;
      const int j = j0 + 32 * q + lane;
      const long long first_row = (long long)i * n + j0 + 32 * q;
      const int valid = n - (j0 + 32 * q) < 32 ? (n - (j0 + 32 * q) > 0 ? n - (j0 + 32 * q) : 0) : 32;
      const float scale = j < n ? __ldg(inv_norm + (size_t)i * n + j) : 0.f;
      RowsOutReq rq;
      if (kF32) rows_out_request(rq, reinterpret_cast<const float*>(z_in), first_row, 1, valid, 0, lane, add_residual != 0);
      ok = mbar_wait(&bars.acc_full[ab], (tcount >> 1) & 1, 8u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + 128 * ab + 32 * cc, r);
        tmem_wait_ld();
        if (cc == 3) {                            // this warp has read its part of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.acc_empty[ab]);
        }
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e)
          v[e] = (__uint_as_float(r[e]) * (1.0f / PX_TRIMUL_X_SCALE) + __ldg(bias + 32 * cc + e)) * scale;
        if (kF32) {
          rows_out_store(stg, v, rq, reinterpret_cast<float*>(z_out), first_row, 1, valid, 32 * cc, lane);
          if (cc < 3)
            rows_out_request(rq, reinterpret_cast<const float*>(z_in), first_row, 1, valid, 32 * (cc + 1), lane,
                             add_residual != 0);
        } else if (j < n) {
          const size_t off = ((size_t)i * n + j) * kC + 32 * cc;
          const bf16* zi = reinterpret_cast<const bf16*>(z_in) + off;
          bf16* zo = reinterpret_cast<bf16*>(z_out) + off;
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            uint32_t w[4];
            if (add_residual) {
              const uint4 zv = *reinterpret_cast<const uint4*>(zi + 8 * p);
              const uint32_t zw[4] = {zv.x, zv.y, zv.z, zv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 r2 = unpack_bf16x2(zw[e]);
                w[e] = pack_bf16x2_int(v[8 * p + 2 * e] + r2.x, v[8 * p + 2 * e + 1] + r2.y);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) w[e] = pack_bf16x2_int(v[8 * p + 2 * e], v[8 * p + 2 * e + 1]);
            }
            *reinterpret_cast<uint4*>(zo + 8 * p) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kOpCols) : "memory");
  }
}

PX_DEFINE_FAMILY_HOOKS(opm)

template <typename Tz>
static int32_t launch_opm_out(const px_f16* x, const px_f16* w_out, const float* bias, const float* inv_norm,
                              const void* z_in, void* z_out, int64_t n_i, int64_t n, int32_t add_residual,
                              cudaStream_t st) {
  CUtensorMap mx, mw;
  // x [32 n_i rows (i, c)][32 n columns (j, e)] seen as (e, j, row): box [4 rows][128 j][32 e], 64-byte swizzle
  if (!make_map_3d(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, 32, (uint64_t)n, (uint64_t)n_i * 32, 64, (uint64_t)n * 64, 32, 128,
                   CU_TENSOR_MAP_SWIZZLE_64B, kOpCc) ||
      // W_out [128 o][32 c][32 e] seen as (e, o, c): box [4 c][128 o][32 e]
      !make_map_3d(&mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, w_out, 32, 128, 32, 2048, 64, 32, 128, CU_TENSOR_MAP_SWIZZLE_64B,
                   kOpCc))
    return PX_ERR_LAUNCH;
  const size_t smem = OpLayout::total + 1024;
  if (cudaFuncSetAttribute(opm_out_tc_kernel<Tz>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return PX_ERR_LAUNCH;
  const int64_t tiles_j = (n + 127) / 128, total = tiles_j * n_i;
  if (total > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int grid = (int)(total < sm_count() ? total : sm_count());
  opm_out_tc_kernel<Tz><<<grid, 192, smem, st>>>(mx, mw, bias, inv_norm, (const Tz*)z_in, (Tz*)z_out, (int)n, add_residual,
                                                 (int)tiles_j, (int)total);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

}  // namespace px

using namespace px;

extern "C" int32_t px_opm_out(const px_f16* x, const px_f16* w_out, const float* bias, const float* inv_norm,
                              const void* z_in, void* z_out, int32_t z_dtype, int64_t n_i, int64_t n,
                              int32_t add_residual, void* stream) {
  if (!x || !w_out || !bias || !inv_norm || !z_out || (add_residual && !z_in) || n <= 0 || n > 32768 || n_i <= 0 ||
      n_i > n)
    return PX_ERR_BAD_ARG;
  if ((((uintptr_t)x | (uintptr_t)w_out | (uintptr_t)bias | (uintptr_t)z_in | (uintptr_t)z_out) & 15) || ((uintptr_t)inv_norm & 3))
    return PX_ERR_BAD_ARG;          // inv_norm is read one value at a time: a block of rows may start anywhere
  if (z_dtype == PX_F32)
    return launch_opm_out<float>(x, w_out, bias, inv_norm, z_in, z_out, n_i, n, add_residual, (cudaStream_t)stream);
  if (z_dtype == PX_BF16)
    return launch_opm_out<bf16>(x, w_out, bias, inv_norm, z_in, z_out, n_i, n, add_residual, (cudaStream_t)stream);
  return PX_ERR_UNSUPPORTED;
}
