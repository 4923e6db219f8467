// Pieces shared by the persistent, TMA-fed row kernels (LayerNorm'd 128-channel rows times resident weights).
//
// Operand formats.  Rows of a bf16 pair tensor are multiplied as they are stored, against bf16 weights.  For an fp32
// pair tensor the kernels read a standardised fp16 copy of the rows, (x - mean) * rstd, that px_standardise_rows
// writes (a standardised row lies within +-sqrt(128), so fp16's range is safe and its three extra mantissa bits cut
// the operand rounding error eightfold), against fp16 weights; such rows carry mean 0 and deviation 1, so their
// correction step only adds the beta term.  `kF16` names the format of a product's operands; the correction step
// is a separate MMA and always takes bf16 head/tail pairs.
//
// LayerNorm is not applied to the operand.  With W' = W diag(gamma), s = W' 1, t = W beta and std = 1/rstd,
//     W LN(x) = rstd * ( W' x - mean * s + std * t ),
// so the tensor core multiplies the rows exactly as they are stored (bf16 rows go from global memory to the swizzled
// operand by TMA without passing through registers).  The two correction terms ride along as one extra K step of 16:
// the row side holds (-mean, std) and the weight side (s, t), each split into a bf16 head and tail so that the
// products carry about 17 bits.  What is left for the epilogue is one multiplication by the row's rstd.
#pragma once
#include "px_tcgen05.cuh"

namespace px {

constexpr int kPanelBytes = 128 * 128;        // [128 rows][64 k] bf16, 128-byte swizzle
constexpr int kOperandBytes = 2 * kPanelBytes;  // [128 rows][128 k] as two k panels

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 -> one bf16x2 word (one conversion instruction; measured at 64 lanes per clock and SM on B200, half the
// FMA rate and four times the special-function rate).
__device__ __forceinline__ uint32_t pack_bf16x2_int(float lo, float hi) { return pack_bf16x2(lo, hi); }

// Byte offset of the 16-byte piece holding channels 8*piece16..8*piece16+7 of row r inside a [128][128] operand.
__device__ __forceinline__ int operand_piece_offset(int r, int piece16, int panel_bytes = kPanelBytes) {
  return (piece16 >> 3) * panel_bytes + r * 128 + (((piece16 & 7) ^ (r & 7)) << 4);
}

// bf16 head and tail of an fp32 value: head + tail carries about 17 significant bits.
__device__ __forceinline__ void split_bf16(float v, uint32_t& head, uint32_t& tail) {
  const bf16 h = __float2bfloat16_rn(v);
  const bf16 t = __float2bfloat16_rn(v - __bfloat162float(h));
  head = (uint32_t)__bfloat16_as_ushort(h);
  tail = (uint32_t)__bfloat16_as_ushort(t);
}

// Row r of a correction panel ([rows][16 k] bf16, 32-byte swizzle).  One 8-wide half of the row (`khalf`: k = 0..7 or
// k = 8..15) pairs up x with the other side's first value in its k = 0..3 and y with its second value in k = 4..7;
// `weight_side` picks the interleaving so that the four head/tail products of each pair meet:
// row side (xh, xh, xl, xl, yh, yh, yl, yl), weight side (xh, xl, xh, xl, yh, yl, yh, yl).
// The other half of the row is zeroed when `zero_other` is set (it must never hold anything but finite values).
__device__ __forceinline__ void write_correction_row(unsigned char* panel, int r, float x, float y, bool weight_side,
                                                     int khalf = 0, bool zero_other = true) {
  uint32_t xh, xl, yh, yl;
  split_bf16(x, xh, xl);
  split_bf16(y, yh, yl);
  uint4 v;
  if (weight_side) {
    v.x = xh | (xl << 16), v.y = v.x, v.z = yh | (yl << 16), v.w = v.z;
  } else {
    v.x = xh | (xh << 16), v.y = xl | (xl << 16), v.z = yh | (yh << 16), v.w = yl | (yl << 16);
  }
  const int sw = ((r >> 2) & 1) ^ khalf;
  *reinterpret_cast<uint4*>(panel + r * 32 + (sw << 4)) = v;
  if (zero_other) *reinterpret_cast<uint4*>(panel + r * 32 + ((sw ^ 1) << 4)) = make_uint4(0u, 0u, 0u, 0u);
}

// Rounds to bf16 and stores two bytes.
__device__ __forceinline__ void store_bf16_int(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// 16-bit weight values -> fp32 (`kF16`: the weights are fp16, otherwise bf16).
template <bool kF16>
__device__ __forceinline__ float4 load4_w16(const uint16_t* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack16x2<kF16>(u.x), b = unpack16x2<kF16>(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

// Folds gamma (and `scale`) into rows [row_begin, row_begin + count) of a [*][128] 16-bit weight (format kInF16) and
// writes them in the operand format kOutF16 as rows dst_row0.. of a K-major swizzled operand with `panel_bytes` per
// 64-wide k panel; the matching rows of the correction panel `extra` receive (s, t): s = sum_c W'[row][c] over the
// rounded values, t = scale * sum_c W[row][c] * beta[c].  Warp-per-row; called by `nwarps` warps with consecutive
// `warp` numbers.  gamma == nullptr: no LayerNorm to fold (plain copy with `scale`, no correction row).
template <bool kInF16, bool kOutF16>
__device__ __forceinline__ void fold_weight_rows(unsigned char* dst, unsigned char* extra, int dst_row0, int panel_bytes,
                                                 const bf16* __restrict__ W, int row_begin, int count,
                                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                                 float scale, int warp, int nwarps, int lane, int khalf = 0) {
  const float4 g4 = gamma ? *reinterpret_cast<const float4*>(gamma + 4 * lane) : make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 b4 = gamma ? *reinterpret_cast<const float4*>(beta + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
  for (int i = warp; i < count; i += nwarps) {
    const float4 w = load4_w16<kInF16>(reinterpret_cast<const uint16_t*>(W) + (size_t)(row_begin + i) * kC + 4 * lane);
    const uint32_t lo = pack16x2<kOutF16>(w.x * g4.x * scale, w.y * g4.y * scale);
    const uint32_t hi = pack16x2<kOutF16>(w.z * g4.z * scale, w.w * g4.w * scale);
    const int r = i + dst_row0;
    *reinterpret_cast<uint2*>(dst + operand_piece_offset(r, lane >> 1, panel_bytes) + (lane & 1) * 8) = make_uint2(lo, hi);
    if (gamma) {
      const float2 f0 = unpack16x2<kOutF16>(lo), f1 = unpack16x2<kOutF16>(hi);
      const float s = warp_sum(f0.x + f0.y + f1.x + f1.y);
      const float t = warp_sum(w.x * b4.x + w.y * b4.y + w.z * b4.z + w.w * b4.w) * scale;
      if (lane == 0) write_correction_row(extra, r, s, t, true, khalf);
    }
  }
}

// The register of a 32-entry array that belongs to this lane (arr[lane] without local memory).
__device__ __forceinline__ float select_own(const uint32_t (&arr)[32], int lane) {
  uint32_t v = 0;
#pragma unroll
  for (int e = 0; e < 32; ++e) v = (lane == e) ? arr[e] : v;
  return __uint_as_float(v);
}

// TMA store of a 3-D box from shared memory (bulk async group of the calling thread).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];\n"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// Waits until at most N of this thread's store groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}
// Barrier over `threads` threads that also returns whether `ok` held on all of them, so that a group can leave a
// loop together after one of its waits ran out.
__device__ __forceinline__ bool named_barrier_all(int id, int threads, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 q, %1, 0;\n bar.red.and.pred p, %2, %3, q;\n selp.b32 %0, 1, 0, p;\n}\n"
      : "=r"(r)
      : "r"((uint32_t)ok), "r"(id), "r"(threads)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// Mean and 1/std of one bf16 row already in the swizzled operand at `op` (row r), computed by two threads, each
// over 64 channels (`half` = 0/1; the two threads are neighbouring lanes).  One pass: sums of (x - x0) and
// (x - x0)^2 with the row's first element as pivot, which keeps the variance accurate when |mean| >> std.
__device__ __forceinline__ void row_stats_from_operand(const unsigned char* op, int r, int half, float eps, float& mean,
                                                       float& rstd) {
  const float x0 = __uint_as_float(*reinterpret_cast<const uint32_t*>(op + operand_piece_offset(r, 0)) << 16);
  float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // pieces 4*half..4*half+3 of both k panels: the 8 lanes of a quarter warp touch 8 distinct bank groups
    const int p = ((i >> 2) << 3) + 4 * half + (i & 3);
    const uint4 v = *reinterpret_cast<const uint4*>(op + operand_piece_offset(r, p));
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    float e;
    e = a.x - x0, s0 += e, q0 = fmaf(e, e, q0);
    e = a.y - x0, s1 += e, q1 = fmaf(e, e, q1);
    e = b.x - x0, s0 += e, q0 = fmaf(e, e, q0);
    e = b.y - x0, s1 += e, q1 = fmaf(e, e, q1);
    e = c.x - x0, s0 += e, q0 = fmaf(e, e, q0);
    e = c.y - x0, s1 += e, q1 = fmaf(e, e, q1);
    e = d.x - x0, s0 += e, q0 = fmaf(e, e, q0);
    e = d.y - x0, s1 += e, q1 = fmaf(e, e, q1);
  }
  float s = s0 + s1, q = q0 + q1;
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  q += __shfl_xor_sync(0xffffffffu, q, 1);
  const float m = s * (1.0f / kC);
  mean = x0 + m;
  rstd = rsqrtf(fmaxf(q * (1.0f / kC) - m * m, 0.f) + eps);
}

// ---------------------------------------------------------------------------------------------------------------
// Row tiles: the part of the pipeline that is the same for every kernel that consumes LayerNorm'd pair rows.
// A tile is 128 pair elements (one u, 128 consecutive t); element (u, t) is row u*n_t + t of z, or row t*n_u + u when
// the two indices are exchanged (`swap`).  A stage of the ring holds the tile as two k panels of 144 rows (the
// last 16 rows are ones, see below) and the tile's correction panel.
//   * producer thread: TMA loads of the rows (bf16 rows of z, or the standardised fp16 copy of an fp32 z);
//   * statistics issuer thread: Z Z^T | Z 1 (M=128, N=144) into tensor memory: the diagonal holds each row's sum
//     of squares and columns 128..143 its plain sum;
//   * statistics threads (one per row): variance = E[x^2] - mean^2 in fp32 (accurate while |mean| is not orders of
//     magnitude above the deviation), correction row (-mean, std), and whatever the kernel wants per row.  For
//     standardised rows the statistics are known: (0, 1).
// ---------------------------------------------------------------------------------------------------------------
constexpr int kTileStages = 2;
constexpr int kTileSlots = 4;    // slots of everything written per tile by the statistics warps (scales, correction
                                 // rows, the a_ready barrier): read after the stage is freed, by an epilogue that may
                                 // run two tiles behind the products when the accumulators are double-buffered
constexpr int kTilePanel = 144 * 128;          // [128 rows + 16 rows of ones][64 k] bf16
constexpr int kTileBytes = 2 * kTilePanel;
constexpr int kTileExtra = 128 * 32;           // [128 rows][16 k] correction panel
constexpr uint32_t kGramCols = 144;

struct TileBars {
  // raw_full: tile in shared memory; a_ready: statistics, correction rows and scales written;
  // a_empty: every MMA that reads the stage is complete (one commit per issuing thread)
  uint64_t raw_full[kTileStages], a_ready[kTileSlots], a_empty[kTileStages], gram_full, gram_free;
};
struct TileCtx {
  unsigned char* tiles;     // kTileStages x kTileBytes
  unsigned char* extras;    // kTileSlots x kTileExtra (the correction step of a tile runs after its stage is freed)
  TileBars* bars;
  int first_tile, tile_step, n_tiles, tiles_t, n_u, n_t, swap;
};

// readers: how many arrivals free a stage besides the statistics side, which adds one (the thread that issues the
// statistics product) or, for standardised rows, four (the statistics warps, which only watch the tile arrive).
__device__ __forceinline__ void tile_bars_init(TileBars& b, int readers, bool standardised) {
  for (int s = 0; s < kTileStages; ++s) {
    mbar_init(&b.raw_full[s], 1);
    mbar_init(&b.a_empty[s], readers + (standardised ? 4 : 1));
  }
  for (int s = 0; s < kTileSlots; ++s) mbar_init(&b.a_ready[s], 4);
  mbar_init(&b.gram_full, 1);
  mbar_init(&b.gram_free, 4);
}

// The 16 rows of ones behind every tile panel (never overwritten: a tile load covers 128 rows).
template <bool kF16>
__device__ __forceinline__ void tile_write_ones(unsigned char* tiles, int tid, int nthreads) {
  constexpr uint32_t one = ones16x2(kF16);
  for (int i = tid; i < kTileStages * 2 * 16 * 8; i += nthreads) {
    const int panel = i >> 7, piece = i & 127;
    *reinterpret_cast<uint4*>(tiles + panel * kTilePanel + 128 * 128 + piece * 16) = make_uint4(one, one, one, one);
  }
}

// One thread: TMA loads of the bf16 tiles.
__device__ __forceinline__ void tile_producer_loop(const TileCtx& c, const CUtensorMap* map_z) {
  int k = 0;
  for (int tile = c.first_tile; tile < c.n_tiles; tile += c.tile_step, ++k) {
    const int s = k % kTileStages, n = k / kTileStages;
    if (!mbar_wait(&c.bars->a_empty[s], (n & 1) ^ 1, 1u)) break;
    const int u = tile / c.tiles_t, t0 = (tile % c.tiles_t) * 128;
    mbar_expect_tx(&c.bars->raw_full[s], kOperandBytes);
    const uint32_t dst = smem_u32(c.tiles + s * kTileBytes);
    for (int p = 0; p < 2; ++p)
      tma_load_3d(dst + p * kTilePanel, map_z, &c.bars->raw_full[s], 64 * p, c.swap ? u : t0, c.swap ? t0 : u);
  }
}

// One thread: the statistics product of every tile into tensor-memory columns [gram_col, gram_col + 144).
template <bool kF16>
__device__ __forceinline__ void tile_gram_loop(const TileCtx& c, uint32_t tmem_gram) {
  constexpr uint32_t idesc_gram = umma_idesc_16(128, kGramCols, kF16, kF16);
  int k = 0;
  for (int tile = c.first_tile; tile < c.n_tiles; tile += c.tile_step, ++k) {
    const int s = k % kTileStages, n = k / kTileStages;
    if (!mbar_wait(&c.bars->raw_full[s], n & 1, 2u) || !mbar_wait(&c.bars->gram_free, (k & 1) ^ 1, 2u)) break;
    tc_fence_after();
    const uint32_t a_addr = smem_u32(c.tiles + s * kTileBytes);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint64_t d = umma_desc_sw128(a_addr + (ks >> 2) * kTilePanel) + 2 * (ks & 3);
      umma_bf16(tmem_gram, d, d, idesc_gram, ks ? 1u : 0u);
    }
    umma_commit(&c.bars->gram_full);
    umma_commit(&c.bars->a_empty[s]);
  }
}

// Four warps, one thread per row (`qw` = warp's lane quarter, 0..3).  per_row(k, u, t, r, rstd) is called once per
// tile and row with the row's 1/std, before a_ready is signalled.  `kStandardised`: the rows are a standardised copy
// (mean 0, deviation 1 by construction), so the correction row is (0, 1) and the factor is 1.
template <bool kStandardised, typename PerRow>
__device__ __forceinline__ void tile_stats_loop(const TileCtx& c, float eps, uint32_t tmem_gram, int qw, int lane,
                                                PerRow per_row) {
  const int r = 32 * qw + lane;
  const uint32_t t_gram = tmem_gram + ((uint32_t)(32 * qw) << 16);
  int k = 0;
  bool ok = true;
  for (int tile = c.first_tile; tile < c.n_tiles; tile += c.tile_step, ++k) {
    const int s = k % kTileStages;
    const int u = tile / c.tiles_t, t = (tile % c.tiles_t) * 128 + r;
    float mean = 0.f, std = 1.f, rstd = 1.f;
    if (kStandardised) {
      // nothing to measure (no statistics product runs in this mode): the arrival of the tile only paces this loop,
      // so that the slots it writes are those of tiles in flight
      ok = mbar_wait(&c.bars->raw_full[s], (k / kTileStages) & 1, 16u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars->a_empty[s]);   // seen: the stage may move on (no phase can be missed)
    } else {
      ok = mbar_wait(&c.bars->gram_full, k & 1, 16u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t diag[32], sums[16];
      tmem_ld32(t_gram + 32 * qw, diag);
      tmem_ld16(t_gram + 128, sums);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars->gram_free);
      mean = __uint_as_float(sums[0]) * (1.0f / kC);
      const float var = fmaxf(select_own(diag, lane) * (1.0f / kC) - mean * mean, 0.f);
      rstd = rsqrtf(var + eps);
      std = sqrtf(var + eps);
    }
    // rstd * (W'x - mean * s + std * t): the row side of the correction step holds (-mean, std)
    write_correction_row(c.extras + (k % kTileSlots) * kTileExtra, r, -mean, std, false);
    per_row(k, u, t, r, rstd);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.bars->a_ready[k % kTileSlots]);
  }
}

// One thread: for every tile, 8 MMAs M=128 (rows) x N (weight rows of `w_addr`, two k panels of w_panel bytes) into
// tensor-memory column d_tmem, then the correction step against the weight-side panel at wx_addr.  acc_full/acc_free
// hand the accumulator back and forth with the epilogue warps: arrays of n_acc barriers, tile k uses accumulator
// k % n_acc at d_tmem + (k % n_acc) * acc_cols (n_acc = 1 or 2).
__device__ __forceinline__ void tile_product_loop(const TileCtx& c, uint32_t d_tmem, uint32_t w_addr, int w_panel,
                                                  uint32_t wx_addr, uint32_t idesc, uint64_t* acc_full,
                                                  uint64_t* acc_free, int n_acc = 1, uint32_t acc_cols = 0) {
  const uint64_t wx_desc = umma_desc_sw32(wx_addr);
  // the correction step multiplies bf16 head/tail pairs whatever the format of the main operands; M and N as `idesc`
  const uint32_t idesc_corr = idesc | (1u << 7) | (1u << 10);
  int k = 0;
  for (int tile = c.first_tile; tile < c.n_tiles; tile += c.tile_step, ++k) {
    const int s = k % kTileStages, n = k / kTileStages;
    const int ab = n_acc == 2 ? (k & 1) : 0, an = n_acc == 2 ? (k >> 1) : k;
    const uint32_t d = d_tmem + ab * acc_cols;
    if (!mbar_wait(&c.bars->raw_full[s], n & 1, 4u) || !mbar_wait(&acc_free[ab], (an & 1) ^ 1, 8u)) break;
    tc_fence_after();
    const uint32_t a_addr = smem_u32(c.tiles + s * kTileBytes);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_bf16(d, umma_desc_sw128(a_addr + (ks >> 2) * kTilePanel) + 2 * (ks & 3),
                umma_desc_sw128(w_addr + (ks >> 2) * w_panel) + 2 * (ks & 3), idesc, ks ? 1u : 0u);
    // This thread's reads of the stage end here: the producer may refill it while the statistics of the tile are
    // still on their way.  The correction step reads the tile's slot of the correction ring; slot k % 4 (rows, scales
    // and the a_ready barrier alike) is rewritten for tile k + 4, whose stage is handed out only after the products
    // of tile k + 2, which this thread issues after the correction step below and which wait for the epilogue of
    // tile k (at the latest) to have read its scales and its accumulator.
    umma_commit(&c.bars->a_empty[s]);
    if (!mbar_wait(&c.bars->a_ready[k % kTileSlots], (k / kTileSlots) & 1, 4u)) break;   // needs the statistics
    tc_fence_after();
    umma_bf16(d, umma_desc_sw32(smem_u32(c.extras + (k % kTileSlots) * kTileExtra)), wx_desc, idesc_corr, 1u);
    umma_commit(&acc_full[ab]);
  }
}

// fp32 output rows, coalesced.  A thread of the epilogue owns one row (its accumulator lane) and 32 consecutive
// channels of it; written as they are, a warp's store would touch 32 rows 512 bytes apart.  Instead the warp passes
// its [32 rows][32 channels] block through a private 4 KB staging area (rows of 128 bytes, 16-byte pieces swizzled
// by row) and reads it back with 8 lanes per row, so that every global access of the warp covers four rows x 128
// contiguous bytes.  `res` holds the residual values of the same block in the read-back arrangement, loaded by
// rows_out_request before the accumulator is waited for (zeros without a residual).
struct RowsOutReq {
  float4 v[8];
};
// first_row: index (inside the tensor, in rows of 128 channels) of the warp's row 0; row_stride: distance in rows
// between consecutive rows of the warp (1, or n_u for a column slab); rows_valid: how many of the 32 rows exist.
__device__ __forceinline__ void rows_out_request(RowsOutReq& rq, const float* __restrict__ z, long long first_row,
                                                 long long row_stride, int rows_valid, int chan0, int lane, bool want) {
  const int rsub = lane >> 3, piece = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rl = 4 * it + rsub;
    rq.v[it] = (want && rl < rows_valid)
                   ? __ldg(reinterpret_cast<const float4*>(z + (size_t)(first_row + rl * row_stride) * kC + chan0) + piece)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
__device__ __forceinline__ void rows_out_store(unsigned char* stg, const float (&v)[32], const RowsOutReq& rq,
                                               float* __restrict__ out, long long first_row, long long row_stride,
                                               int rows_valid, int chan0, int lane) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) =
        make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
  const int rsub = lane >> 3, piece = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rl = 4 * it + rsub;
    float4 o = *reinterpret_cast<const float4*>(stg + rl * 128 + ((piece ^ (rl & 7)) << 4));
    if (rl < rows_valid) {
      o.x += rq.v[it].x, o.y += rq.v[it].y, o.z += rq.v[it].z, o.w += rq.v[it].w;
      *(reinterpret_cast<float4*>(out + (size_t)(first_row + rl * row_stride) * kC + chan0) + piece) = o;
    }
  }
  __syncwarp();
}

// Number of SMs of the current device (cached per device ordinal).
static inline int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace px
