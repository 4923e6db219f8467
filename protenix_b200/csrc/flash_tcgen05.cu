// Triangle attention core on the 5th-generation tensor cores (4 heads x 32).
//
//   o[u][q][h*32+d] = softmax_k( q[u,h,q,:] . k[u,h,k,:] + bias[h][q][k] + mask_bias[u][k] ) v[u,h,k,d]
//
// q, k, v and o are fp16 (projections of standardised rows and convex combinations of them: far inside its range;
// fp16 keeps three more bits than bf16), the pair bias, the logits, the softmax and the accumulators fp32.
//
// One CTA = (head h, 128 queries, 6 attended rows u), 16 warps:
//   warps 0..11   three softmax groups of four warps; group g owns rows u0+2g, u0+2g+1, each thread one query row.
//                 The kernel is bound by the latency of a group's chain (wait S, load, add, reduce, exponentials,
//                 store P), not by any one unit, so three groups are kept in flight per SM.  Per work item a thread
//                 adds its 64 pair-bias values from the shared tile (the bias does not depend on u: all six rows
//                 use the same tile), and keeps the softmax denominator of its row in a register.
//   warps 12..14  one control thread per group (tcgen05 and TMA instructions cost ~100 cycles of issue each, so
//                 one issuing thread for all groups would be the bottleneck).  It loads the group's Q tiles once
//                 and, per work item, a K tile [64 keys][32] (64-byte swizzle) and a transposed V tile
//                 [32 d][64 keys] (128-byte swizzle) into the group's 4-stage ring; issues S = Q K^T (M=128, N=64,
//                 K=32) into the group's S buffer in tensor memory; and, once the group has written P (fp16) into
//                 its P buffer, issues O_u += P V with P as the TMEM-resident A operand (M=128, N=32, K=64).  S of
//                 the next item is issued as soon as the group has pulled the current S into registers, so it is
//                 ready when the group comes back.
//   warp 15       one thread loads the pair-bias tiles [128 q][64 k] fp32 (two 128-byte-swizzled boxes, 2-deep ring).
// Tensor memory: S (3 x 64) | P (3 x 32, two fp16 per column) | O (6 x 32).
//
// Letting the tensor core add the bias (S += I B with an identity operand and the bias tile as an MN-major fp16
// operand: eight more MMAs per item) was measured and lost: 7.8 ms against 6.3 ms at N=1536.  The 48 instructions
// it takes off every softmax thread weigh less than the ten MMA issues it puts on the group's control thread.
//
// Softmax is online in base 2 with a lazy reference maximum: the reference only moves (and O_u is rescaled
// through TMEM) when the tile maximum exceeds it by more than 8, so probabilities stay below 2^8.
// Exponentials are fp32 (three pairs in four by ex2, the fourth by a cubic on the FMA pipe); P is their rounding to
// fp16, the denominators sum the fp32 values.  Every mbarrier wait is bounded.
#include <math_constants.h>

#include "px_tcgen05.cuh"

namespace px {

constexpr int kFH = 4, kFD = 32;
constexpr int kFGroups = 3;               // softmax groups per CTA
constexpr int kFRpg = 2;                  // attended rows per group
constexpr int kFRows = kFGroups * kFRpg;  // attended rows per CTA
constexpr int kFKT = 64;                  // keys per work item
constexpr int kFStages = 4;               // K/V ring of each group (work items = (key tile, row))
constexpr int kFQBytes = 128 * 64;        // [128][32] fp16
constexpr int kFKBytes = kFKT * 64;       // [64][32] fp16
constexpr int kFVBox = 32 * 128;          // the TMA box of the value tile: 32 rows x 64 keys
constexpr int kFVBytes = 32 * 128;        // [32 d][64 keys] fp16
constexpr int kFStageBytes = kFKBytes + kFVBytes;
constexpr int kFBiasBytes = 128 * kFKT * 4;
constexpr int kFON = 32;                  // columns of an O accumulator
constexpr uint32_t kFCols = 512;
constexpr int kFColS = 0, kFColP = kFGroups * kFKT, kFColO = kFColP + kFGroups * (kFKT / 2);  // TMEM column map
constexpr float kRescaleGap = 8.0f;
constexpr int kFThreads = 32 * (4 * kFGroups + 4);
static_assert(kFColO + kFRows * kFON <= 512, "tensor memory budget");

struct FlashBars {
  uint64_t q_full[kFGroups], kv_full[kFGroups][kFStages], bias_full[2], bias_empty[2], s_full[kFGroups],
      s_free[kFGroups], p_ready[kFGroups], pv_done[kFGroups];
  uint32_t tmem_base;
};

struct FlashLayout {
  static constexpr int q = 0;
  static constexpr int kv = q + kFRows * kFQBytes;
  static constexpr int bias = kv + kFGroups * kFStages * kFStageBytes;
  static constexpr int bars = bias + 2 * kFBiasBytes;
  static constexpr int total = bars + (int)sizeof(FlashBars);
};
static_assert(FlashLayout::kv % 1024 == 0 && FlashLayout::bias % 1024 == 0 && kFStageBytes % 1024 == 0, "swizzle alignment");

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for two arguments on the FMA pipe (the special-function unit delivers 16 ex2 per clock and SM and is the
// busiest unit of this kernel): x = n + f with n = round(x) taken from the mantissa after adding 1.5 * 2^23,
// 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding of P), 2^n added into the exponent
// field.  Arguments below -126 (masked or padded keys) give 2^-126.
constexpr int kFPolyEvery = 4;   // every fourth pair of exponentials takes this path
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  constexpr float kMagic = 12582912.f;
  constexpr float c0 = 0.9999280571937561f, c1 = 0.6932610273361206f, c2 = 0.2426111102104187f, c3 = 0.05517144873738289f;
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  float t0 = x0, t1 = x1;
  add2(t0, t1, kMagic, kMagic);
  float n0 = t0, n1 = t1;
  add2(n0, n1, -kMagic, -kMagic);
  float f0, f1, q0, q1;
  fma2(f0, f1, n0, n1, -1.f, -1.f, x0, x1);
  fma2(q0, q1, f0, f1, c3, c3, c2, c2);
  fma2(q0, q1, q0, q1, f0, f1, c1, c1);
  fma2(q0, q1, q0, q1, f0, f1, c0, c0);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

__global__ void __launch_bounds__(kFThreads, 1)
triatt_flash_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_b,
                       const float* __restrict__ mb, const unsigned long long* __restrict__ tile_masked,
                       bf16* __restrict__ o, int n_u, int n, int ldm, int nkt) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  FlashBars& bars = *reinterpret_cast<FlashBars*>(sm + FlashLayout::bars);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128, h = blockIdx.y, u0 = blockIdx.z * kFRows;

  if (cta_skip_after_error()) return;   // an earlier bounded wait gave up: do not start new work
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars.bias_full[b], 1);
      mbar_init(&bars.bias_empty[b], 4 * kFGroups);
    }
    for (int g = 0; g < kFGroups; ++g) {
      mbar_init(&bars.q_full[g], 1);
      for (int s = 0; s < kFStages; ++s) mbar_init(&bars.kv_full[g][s], 1);
      mbar_init(&bars.s_full[g], 1);
      mbar_init(&bars.s_free[g], 4);
      mbar_init(&bars.p_ready[g], 4);
      mbar_init(&bars.pv_done[g], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 4 * kFGroups) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&bars.tmem_base)),
                 "r"(kFCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;

  if (warp >= 4 * kFGroups) {
    // ------------------------------------------------------------------ control thread of group g
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;\n");   // registers go to the softmax warpgroups (with 24 the
                                                             // control threads spill: 6.02 ms against 5.91 at N=1536)
    const int g = warp - 4 * kFGroups;
    if (g == kFGroups && lane == 0) {
      // ---------------------------------------------------------------- pair-bias loader (all six rows share a tile)
      for (int kt = 0; kt < nkt; ++kt) {
        const int b = kt & 1;
        if (!mbar_wait(&bars.bias_empty[b], ((kt >> 1) & 1) ^ 1, 1u)) break;
        mbar_expect_tx(&bars.bias_full[b], kFBiasBytes);
        for (int c = 0; c < kFKT / 32; ++c)
          tma_load_3d(smem_u32(sm + FlashLayout::bias + b * kFBiasBytes + c * (128 * 128)), &map_b, &bars.bias_full[b],
                      kt * kFKT + c * 32, q0, h);
      }
    } else if (g < kFGroups && lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, kFKT), idesc_o = umma_idesc_f16(128, kFON);
      const int n_items = nkt * kFRpg;              // work item i = (key tile i / 3, row i % 3 of the group)
      const uint32_t q_addr = smem_u32(sm + FlashLayout::q + g * kFRpg * kFQBytes);
      const uint32_t ring = smem_u32(sm + FlashLayout::kv + g * kFStages * kFStageBytes);
      const uint32_t d_s = tmem_base + kFColS + kFKT * g, d_p = tmem_base + kFColP + (kFKT / 2) * g;
      const uint32_t d_o = tmem_base + kFColO + kFON * kFRpg * g;
      const int uh0 = (u0 + g * kFRpg) * kFH + h;   // rows past n_u: coordinate beyond the tensor -> zero fill
      bool ok = true;
      auto load_kv = [&](int i) {                   // K and V tiles of item i into stage i % kFStages
        const int s = i % kFStages, kt = i / kFRpg, uh = uh0 + (i % kFRpg) * kFH;
        mbar_expect_tx(&bars.kv_full[g][s], kFKBytes + kFVBox);
        tma_load_3d(ring + s * kFStageBytes, &map_k, &bars.kv_full[g][s], 0, kt * kFKT, uh);
        tma_load_3d(ring + s * kFStageBytes + kFKBytes, &map_v, &bars.kv_full[g][s], kt * kFKT, 0, uh);
      };
      auto issue_s = [&](int i) {                   // S(i) = Q_r K^T
        const int s = i % kFStages;
        if (!mbar_wait(&bars.kv_full[g][s], (i / kFStages) & 1, 8u)) return false;
        tc_fence_after();
        const uint64_t dq = umma_desc_sw64(q_addr + (i % kFRpg) * kFQBytes), dk = umma_desc_sw64(ring + s * kFStageBytes);
        umma_bf16(d_s, dq, dk, idesc_s, 0u);
        umma_bf16(d_s, dq + 2, dk + 2, idesc_s, 1u);
        umma_commit(&bars.s_full[g]);
        return true;
      };
      mbar_expect_tx(&bars.q_full[g], kFRpg * kFQBytes);
      for (int r = 0; r < kFRpg; ++r) tma_load_3d(q_addr + r * kFQBytes, &map_q, &bars.q_full[g], 0, q0, uh0 + r * kFH);
      for (int i = 0; i < kFStages - 1 && i < n_items; ++i) load_kv(i);   // first use of these stages
      ok = ok && mbar_wait(&bars.q_full[g], 0, 4u);
      ok = ok && issue_s(0);
      for (int i = 0; i < n_items && ok; ++i) {
        const int kt = i / kFRpg, r = i % kFRpg;
        if (i + 1 < n_items) {                      // next S as soon as the group holds the current one in registers
          ok = mbar_wait(&bars.s_free[g], i & 1, 2u) && issue_s(i + 1);
          if (!ok) break;
        }
        if (i + kFStages - 1 < n_items) {           // refill: that stage was last read by P.V of item i-1
          if (i >= 1) ok = mbar_wait(&bars.pv_done[g], (i - 1) & 1, 32u);
          if (!ok) break;
          load_kv(i + kFStages - 1);
        }
        ok = mbar_wait(&bars.p_ready[g], i & 1, 16u);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dv = umma_desc_sw128(ring + (i % kFStages) * kFStageBytes + kFKBytes);
#pragma unroll
        for (int ks = 0; ks < kFKT / 16; ++ks)  // 16 keys per step: 8 TMEM columns of P, 32 bytes of the value rows
          umma_bf16_ts(d_o + kFON * r, d_p + 8 * ks, dv + 2 * ks, idesc_o, (kt | ks) ? 1u : 0u);
        umma_commit(&bars.pv_done[g]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;\n");
    const int g = warp >> 2, qw = warp & 3;
    const int row = 32 * qw + lane;                 // query row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(32 * qw) << 16;
    const uint32_t t_s = tmem_base + lane_addr + kFColS + kFKT * g;
    const uint32_t t_p = tmem_base + lane_addr + kFColP + (kFKT / 2) * g;
    const uint32_t t_o = tmem_base + lane_addr + kFColO + kFON * kFRpg * g;
    const int ug = u0 + kFRpg * g;                  // first row of this group
    const int words = (nkt + 63) / 64;              // mask-flag words per row: one bit per 64-key tile
    unsigned long long flag_word[kFRpg];
    float m_ref[kFRpg], l_sum[kFRpg];             // reference maximum and denominator of this thread's query per row
#pragma unroll
    for (int r = 0; r < kFRpg; ++r) {
      flag_word[r] = 0;
      m_ref[r] = -CUDART_INF_F;
      l_sum[r] = 0.f;
    }
    bool ok = true;
    for (int kt = 0; kt < nkt && ok; ++kt) {
      if ((kt & 63) == 0) {
#pragma unroll
        for (int r = 0; r < kFRpg; ++r)
          flag_word[r] = (ug + r < n_u) ? __ldg(tile_masked + (size_t)(ug + r) * words + (kt >> 6)) : ~0ull;
      }
      ok = mbar_wait(&bars.bias_full[kt & 1], (kt >> 1) & 1, 64u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float* bias_tile = reinterpret_cast<const float*>(sm + FlashLayout::bias + (kt & 1) * kFBiasBytes);
#pragma unroll
      for (int r = 0; r < kFRpg; ++r) {
        const int i = kt * kFRpg + r;               // this group's work item
        ok = mbar_wait(&bars.s_full[g], i & 1, 128u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float s[kFKT];
        {
          uint32_t(&t0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
          uint32_t(&t1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
          tmem_ld32(t_s, t0);
          tmem_ld32(t_s + 32, t1);
          tmem_wait_ld();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.s_free[g]);  // S is in registers: the next S may be computed
        // + pair bias: box c of the tile holds columns 32c..32c+31 of all 128 rows, 128-byte rows, 16-byte pieces
        // swizzled by row
#pragma unroll
        for (int c = 0; c < kFKT / 32; ++c) {
          const float* brow = bias_tile + c * (128 * 32) + row * 32;
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const float4 b4 = *reinterpret_cast<const float4*>(brow + ((p ^ (row & 7)) << 2));
            add2(s[32 * c + 4 * p + 0], s[32 * c + 4 * p + 1], b4.x, b4.y);
            add2(s[32 * c + 4 * p + 2], s[32 * c + 4 * p + 3], b4.z, b4.w);
          }
        }
        if (r == kFRpg - 1) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.bias_empty[kt & 1]);   // this warp is done with the bias tile
        }
        if ((flag_word[r] >> (kt & 63)) & 1ull) {     // warp-uniform
          const int u = (ug + r < n_u) ? ug + r : 0;
          const float4* mrow = reinterpret_cast<const float4*>(mb + (size_t)u * ldm + kt * kFKT);
#pragma unroll
          for (int c4 = 0; c4 < kFKT / 4; ++c4) {
            const float4 m4 = __ldg(mrow + c4);
            add2(s[4 * c4 + 0], s[4 * c4 + 1], m4.x, m4.y);
            add2(s[4 * c4 + 2], s[4 * c4 + 3], m4.z, m4.w);
          }
        }
        // tile maximum: four independent chains, so the reduction costs about 8 dependent steps
        float mq[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mq[c] = max3(s[16 * c], s[16 * c + 1], s[16 * c + 2]);
#pragma unroll
          for (int e = 3; e + 1 < 16; e += 2) mq[c] = max3(mq[c], s[16 * c + e], s[16 * c + e + 1]);
          mq[c] = fmaxf(mq[c], s[16 * c + 15]);
        }
        const float mt = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
        // Does the reference maximum have to move?  Rare after the first tiles (warp-uniform decision).
        const bool first = (kt == 0);
        const bool move = !first && __any_sync(0xffffffffu, mt > m_ref[r] + kRescaleGap);
        float alpha = 1.0f;
        if (first) {
          m_ref[r] = mt;                              // first tile: the P.V product overwrites O
        } else if (move) {
          const float m_new = (mt > m_ref[r] + kRescaleGap) ? mt : m_ref[r];
          alpha = fast_exp2(m_ref[r] - m_new);
          m_ref[r] = m_new;
        }
        uint32_t w[kFKT / 2];
        float l0 = 0.f, l1 = 0.f;
        {
          const float nm = -m_ref[r];
#pragma unroll
          for (int e = 0; e < kFKT / 2; ++e) {
            // fp32 exponentials; P is their rounding to nearest fp16 (one conversion per pair), which is unbiased,
            // so the denominator can sum the fp32 values themselves.
            add2(s[2 * e], s[2 * e + 1], nm, nm);
            float p0, p1;
            if (e % kFPolyEvery == kFPolyEvery - 1) {
              exp2_poly2(s[2 * e], s[2 * e + 1], p0, p1);
            } else {
              p0 = fast_exp2(s[2 * e]);
              p1 = fast_exp2(s[2 * e + 1]);
            }
            w[e] = pack_f16x2(p0, p1);
            add2(l0, l1, p0, p1);
          }
        }
        l_sum[r] = l_sum[r] * alpha + (l0 + l1);
        // P.V of the previous item must be through before O is rescaled or the P buffer overwritten
        if (i >= 1) {
          ok = mbar_wait(&bars.pv_done[g], (i - 1) & 1, 256u);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if (move) {
#pragma unroll
          for (int c = 0; c < kFON / 16; ++c) {
            uint32_t a[16];
            tmem_ld16(t_o + kFON * r + 16 * c, a);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) a[e] = __float_as_uint(__uint_as_float(a[e]) * alpha);
            tmem_st16(t_o + kFON * r + 16 * c, a);
          }
        }
        {
          uint32_t(&w0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&w[0]);
          tmem_st32(t_p, w0);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.p_ready[g]);
      }
    }
    // ---- epilogue: o = O / denominator for this group's rows
    ok = ok && mbar_wait(&bars.pv_done[g], (nkt * kFRpg - 1) & 1, 512u);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int qi = q0 + row;
#pragma unroll
      for (int r = 0; r < kFRpg; ++r) {
        uint32_t a[32];
        tmem_ld32(t_o + kFON * r, a);
        tmem_wait_ld();
        if (ug + r < n_u && qi < n) {
          const float inv = 1.0f / l_sum[r];
          bf16* dst = o + ((size_t)(ug + r) * n + qi) * kC + h * kFD;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            pk.x = pack_f16x2(__uint_as_float(a[8 * v + 0]) * inv, __uint_as_float(a[8 * v + 1]) * inv);
            pk.y = pack_f16x2(__uint_as_float(a[8 * v + 2]) * inv, __uint_as_float(a[8 * v + 3]) * inv);
            pk.z = pack_f16x2(__uint_as_float(a[8 * v + 4]) * inv, __uint_as_float(a[8 * v + 5]) * inv);
            pk.w = pack_f16x2(__uint_as_float(a[8 * v + 6]) * inv, __uint_as_float(a[8 * v + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + 8 * v) = pk;
          }
        }
      }
    }
  }

  tc_fence_before();
  cta_teardown_sync();
  if (warp == 4 * kFGroups) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFCols) : "memory");
  }
}

// Bit (kt & 63) of flags[u][kt >> 6] is set when any key of the 64-key tile kt carries a non-zero mask bias
// for row u.  One CTA per (u, word); each warp handles tiles warp, warp + 4, ...
__global__ void flash_tile_flags_kernel(const float* __restrict__ mb, unsigned long long* __restrict__ flags, int ldm,
                                        int nkt) {
  __shared__ unsigned long long word;
  const int u = blockIdx.x, w = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) word = 0ull;
  __syncthreads();
  for (int t = warp; t < 64; t += 4) {
    const int kt = 64 * w + t;
    if (kt >= nkt) break;
    const float* p = mb + (size_t)u * ldm + kt * kFKT;
    const bool any = __any_sync(0xffffffffu, p[lane] != 0.0f || p[lane + 32] != 0.0f);
    if (any && lane == 0) atomicOr(&word, 1ull << t);
  }
  __syncthreads();
  if (threadIdx.x == 0) flags[(size_t)u * gridDim.y + w] = word;
}

PX_DEFINE_FAMILY_HOOKS(flash)

}  // namespace px

using namespace px;

extern "C" int64_t px_ld_mask(int64_t n) { return (n + 127) / 128 * 128; }

extern "C" int64_t px_triatt_flash_scratch_bytes(int64_t n_u, int64_t n) {
  if (n_u <= 0 || n <= 0) return 0;
  return (n_u * ((((n + kFKT - 1) / kFKT) + 63) / 64) * 8 + 255) / 256 * 256;
}

extern "C" int32_t px_triatt_flash(const px_f16* q, const px_f16* k, const px_f16* v, const float* bias,
                                   const float* mask_bias, px_f16* o, void* scratch, int64_t n_u, int64_t n,
                                   int64_t ldm, void* stream) {
  if (!q || !k || !v || !bias || !mask_bias || !o || !scratch || n_u <= 0 || n <= 0 || n_u > 32768 || n > 32768 ||
      ldm != px_ld_mask(n))
    return PX_ERR_BAD_ARG;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)bias | (uintptr_t)mask_bias | (uintptr_t)o) & 15)
    return PX_ERR_BAD_ARG;
  const int64_t ldt = px_ld(n);
  const int nkt = (int)((n + kFKT - 1) / kFKT);
  CUtensorMap mq, mk, mv, mbias;
  const uint64_t uh = (uint64_t)n_u * kFH;
  // q, k: [n_u*4][n][32] fp16, box [1][128][32], 64-byte swizzle
  if (!make_map_3d(&mq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, q, kFD, (uint64_t)n, uh, kFD * 2, (uint64_t)n * kFD * 2, kFD,
                   128, CU_TENSOR_MAP_SWIZZLE_64B) ||
      !make_map_3d(&mk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, k, kFD, (uint64_t)n, uh, kFD * 2, (uint64_t)n * kFD * 2, kFD,
                   kFKT, CU_TENSOR_MAP_SWIZZLE_64B) ||
      // v (transposed): [n_u*4][32][n keys, row stride ldt] fp16, box [1][32][64], 128-byte swizzle
      !make_map_3d(&mv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, v, (uint64_t)n, kFD, uh, (uint64_t)ldt * 2,
                   (uint64_t)kFD * ldt * 2, 64, kFD, CU_TENSOR_MAP_SWIZZLE_128B) ||
      // pair bias: [4][n q][n k, row stride ldm] fp32, box [1][128][32], 128-byte swizzle
      !make_map_3d(&mbias, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, bias, (uint64_t)n, (uint64_t)n, kFH, (uint64_t)ldm * 4,
                   (uint64_t)n * ldm * 4, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return PX_ERR_LAUNCH;
  cudaStream_t st = (cudaStream_t)stream;
  if ((uintptr_t)scratch & 7) return PX_ERR_BAD_ARG;
  flash_tile_flags_kernel<<<dim3((unsigned)n_u, (unsigned)((nkt + 63) / 64)), 128, 0, st>>>(
      mask_bias, (unsigned long long*)scratch, (int)ldm, nkt);
  const size_t smem = FlashLayout::total + 1024;
  if (cudaFuncSetAttribute(triatt_flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  dim3 grid((unsigned)((n + 127) / 128), kFH, (unsigned)((n_u + kFRows - 1) / kFRows));
  triatt_flash_tc_kernel<<<grid, kFThreads, smem, st>>>(mq, mk, mv, mbias, mask_bias, (const unsigned long long*)scratch, (bf16*)o,
                                                  (int)n_u, (int)n, (int)ldm, nkt);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
