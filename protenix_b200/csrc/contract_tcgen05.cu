// Triangle-multiplication contraction on the 5th-generation tensor cores:
//   x[c][i][j] = 2^-6 sum_k a[c][i][k] * b[c][j][k]      (fp16 in, fp32 accumulate, fp16 out)
// The LayerNorm that consumes x does not see a common factor (its epsilon is scaled to match), and the factor 2^-6
// keeps sums over thousands of k inside the fp16 range.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer: A tile [128 i][64 k] and B tile [256 j][64 k] per k-block, 128-byte swizzle,
//               4-stage ring guarded by full/empty mbarriers
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16) four times per k-block;
//               tcgen05.commit releases the shared-memory stage and, after the last k-block, publishes
//               the accumulator
//   warps 2..5  epilogue: tcgen05.ld of the fp32 accumulator (each warp its own 32 TMEM lanes = 32 rows),
//               scale, convert to fp16, 16-byte stores
// The accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue of tile t overlaps the
// main loop of tile t+1.  Ragged edges need no predicates on the load side: the TMA zero-fills rows
// >= N and k >= ld.  Tiles are ordered channel-major so that a channel's operands (2 * N * ld * 2
// bytes) stay in L2 while its tiles are computed.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a flag in g_tc_error, the
// role stops issuing work, and the kernel still frees its TMEM and returns.
#include "px_tcgen05.cuh"

namespace px {

constexpr int kTcBM = 128, kTcBN = 256, kTcBK = 64, kTcStages = 4;
constexpr int kTcABytes = kTcBM * kTcBK * 2, kTcBBytes = kTcBN * kTcBK * 2;
constexpr int kTcStageBytes = kTcABytes + kTcBBytes;
constexpr uint32_t kTcCols = 512;  // two 256-column fp32 accumulators

struct TcBarriers {
  uint64_t full[kTcStages], empty[kTcStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

__global__ void __launch_bounds__(192, 1)
trimul_contract_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          bf16* __restrict__ x, int n, int ld_k, int ld, int tiles_i, int tiles_j, int total_tiles) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // operand ring first (1024-byte aligned for the 128-byte swizzle), barriers after it
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TcBarriers& bars = *reinterpret_cast<TcBarriers*>(ring + kTcStages * kTcStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = (ld_k + kTcBK - 1) / kTcBK;      // ld_k: extent of the contraction index; ld: row stride of x

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
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
                 "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = bars.tmem_base;

  auto tile_coords = [&](int tile, int& c, int& i0, int& j0) {
    const int per_c = tiles_i * tiles_j;
    c = tile / per_c;
    const int r = tile - c * per_c;
    i0 = (r / tiles_j) * kTcBM;
    j0 = (r % tiles_j) * kTcBN;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int c, i0, j0;
        tile_coords(tile, c, i0, j0);
        for (int kt = 0; kt < nk && ok; ++kt, ++it) {
          const int s = it % kTcStages;
          const uint32_t ph = (it / kTcStages) & 1;
          ok = mbar_wait(&bars.empty[s], ph ^ 1, 1u);
          if (!ok) break;
          mbar_expect_tx(&bars.full[s], kTcStageBytes);
          const uint32_t sa = smem_u32(ring + s * kTcStageBytes);
          tma_load_3d(sa, &map_a, &bars.full[s], kt * kTcBK, i0, c);
          tma_load_3d(sa + kTcABytes, &map_b, &bars.full[s], kt * kTcBK, j0, c);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t ab = tcount & 1, aph = (tcount >> 1) & 1;
        ok = mbar_wait(&bars.acc_empty[ab], aph ^ 1, 2u);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t d_tmem = tmem_base + ab * kTcBN;
        for (int kt = 0; kt < nk; ++kt, ++it) {
          const int s = it % kTcStages;
          const uint32_t ph = (it / kTcStages) & 1;
          ok = mbar_wait(&bars.full[s], ph, 4u);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t sa = smem_u32(ring + s * kTcStageBytes);
          const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kTcABytes);
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k)  // 16 bf16 = 32 bytes = 2 units of the start-address field
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, umma_idesc_f16(kTcBM, kTcBN), (kt | k) ? 1u : 0u);
          umma_commit(&bars.empty[s]);
        }
        if (!ok) break;
        umma_commit(&bars.acc_full[ab]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
      int c, i0, j0;
      tile_coords(tile, c, i0, j0);
      const uint32_t ab = tcount & 1, aph = (tcount >> 1) & 1;
      ok = mbar_wait(&bars.acc_full[ab], aph, 8u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int i = i0 + 32 * q + lane;
      bf16* xrow = x + ((size_t)c * n + (i < n ? i : 0)) * ld;
#pragma unroll 1
      for (int cc = 0; cc < kTcBN / 32; ++cc) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + ab * kTcBN + cc * 32, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (i < n) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int j = j0 + cc * 32 + v * 8;
            if (j < ld) {
              uint4 o;
              constexpr float sc = PX_TRIMUL_X_SCALE;
              o.x = pack_f16x2(sc * __uint_as_float(r[8 * v + 0]), sc * __uint_as_float(r[8 * v + 1]));
              o.y = pack_f16x2(sc * __uint_as_float(r[8 * v + 2]), sc * __uint_as_float(r[8 * v + 3]));
              o.z = pack_f16x2(sc * __uint_as_float(r[8 * v + 4]), sc * __uint_as_float(r[8 * v + 5]));
              o.w = pack_f16x2(sc * __uint_as_float(r[8 * v + 6]), sc * __uint_as_float(r[8 * v + 7]));
              *reinterpret_cast<uint4*>(xrow + j) = o;
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.acc_empty[ab]);
    }
  }

  // teardown: everybody meets, then the allocating warp frees the tensor memory
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  cta_teardown_sync();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTcCols) : "memory");
  }
}

// [channels][n rows][ld k] bf16 tensor, box = [1][box_rows][64], 128-byte swizzle, zero fill outside.
static bool make_operand_map(CUtensorMap* map, const void* base, int64_t channels, int64_t n, int64_t ld,
                             uint32_t box_rows) {
  return make_map_3d(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, (uint64_t)ld, (uint64_t)n, (uint64_t)channels,
                     (uint64_t)ld * 2, (uint64_t)n * ld * 2, kTcBK, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

PX_DEFINE_FAMILY_HOOKS(contract)

}  // namespace px

using namespace px;

static int sm_count_contract() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

extern "C" int32_t px_trimul_contract(const px_bf16* a, const px_bf16* b, px_bf16* x, int64_t channels, int64_t n,
                                      int64_t ld, void* stream) {
  if (!a || !b || !x || channels <= 0 || channels > 65535 || n <= 0 || n > 32768 || ld != px_ld(n))
    return PX_ERR_BAD_ARG;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)x) & 15) return PX_ERR_BAD_ARG;
  CUtensorMap ma, mb;
  if (!make_operand_map(&ma, a, channels, n, ld, kTcBM) || !make_operand_map(&mb, b, channels, n, ld, kTcBN))
    return PX_ERR_LAUNCH;
  const int tiles_i = (int)((n + kTcBM - 1) / kTcBM), tiles_j = (int)((n + kTcBN - 1) / kTcBN);
  const int total = tiles_i * tiles_j * (int)channels;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = total < sms ? total : sms;
  const size_t smem = (size_t)kTcStages * kTcStageBytes + sizeof(TcBarriers) + 1024;
  if (cudaFuncSetAttribute(trimul_contract_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  trimul_contract_tc_kernel<<<grid, 192, smem, (cudaStream_t)stream>>>(ma, mb, (bf16*)x, (int)n, (int)ld, (int)ld,
                                                                       tiles_i, tiles_j, total);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

// The same kernel for the outer product of the MSA module: one "channel", a_t [rows_a][ld_k] against
// b_t [rows_b][ld_k] (rows = 32 x tokens), contraction over the ld_k (padded) MSA rows; x is [rows_a][rows_b].
extern "C" int32_t px_opm_outer(const px_f16* a_t, const px_f16* b_t, px_f16* x, int64_t rows_a, int64_t rows_b,
                                int64_t ld_k, void* stream) {
  if (!a_t || !b_t || !x || rows_a <= 0 || rows_a > (1 << 20) || rows_b <= 0 || rows_b > (1 << 20) || rows_b % 8 ||
      ld_k <= 0 || ld_k % 8 || ld_k > (1 << 20))
    return PX_ERR_BAD_ARG;
  if (((uintptr_t)a_t | (uintptr_t)b_t | (uintptr_t)x) & 15) return PX_ERR_BAD_ARG;
  CUtensorMap ma, mb;
  if (!make_operand_map(&ma, a_t, 1, rows_a, ld_k, kTcBM) || !make_operand_map(&mb, b_t, 1, rows_b, ld_k, kTcBN))
    return PX_ERR_LAUNCH;
  const int64_t ti = (rows_a + kTcBM - 1) / kTcBM, tj = (rows_b + kTcBN - 1) / kTcBN;
  if (ti * tj > 0x7fffffff) return PX_ERR_UNSUPPORTED;
  const int tiles_i = (int)ti, tiles_j = (int)tj;
  const int total = tiles_i * tiles_j;
  const int sms = sm_count_contract();
  const int grid = total < sms ? total : sms;
  const size_t smem = (size_t)kTcStages * kTcStageBytes + sizeof(TcBarriers) + 1024;
  if (cudaFuncSetAttribute(trimul_contract_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  trimul_contract_tc_kernel<<<grid, 192, smem, (cudaStream_t)stream>>>(ma, mb, (bf16*)x, (int)rows_a, (int)ld_k,
                                                                       (int)rows_b, tiles_i, tiles_j, total);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

