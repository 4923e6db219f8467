// Triangle attention (4 heads x 32): input projection, flash attention with pair bias, output stage.
#include <math_constants.h>

#include "px_common.cuh"

namespace px {

constexpr int kH = 4;   // heads
constexpr int kD = 32;  // head width

// =========================================================================================
// Stage 1: LN(z) -> q,k,v [u][h][t][32] (q pre-scaled), bias[h][u][t], mask_bias[u][t].
// One CTA = (u, 128 consecutive t).  Pair element for (u,t): z[u][t] (starting) or z[t][u] (ending).
// HBM-bound: reads 128*sizeof(Tz)+4, writes 3*256 + 16 + 4/.. bytes per pair element.
// =========================================================================================
struct TriAttInSmem {
  bf16 A[128 * kLdA];
  bf16 W[2][64 * kLdA];
  bf16 S[64 * kLdA];  // transposed staging of a v chunk: [channel][t]
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
triatt_in_proj_kernel(const Tz* __restrict__ z, const float* __restrict__ mask, const float* __restrict__ ln_w,
                      const float* __restrict__ ln_b, const bf16* __restrict__ w_q, const bf16* __restrict__ w_k,
                      const bf16* __restrict__ w_v, const bf16* __restrict__ w_bias, bf16* __restrict__ q_out,
                      bf16* __restrict__ k_out, bf16* __restrict__ v_out, float* __restrict__ bias_out,
                      float* __restrict__ mb_out, int n_u, int n, int ldm, int ldt, int swap, float eps, float inf) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TriAttInSmem& sm = *reinterpret_cast<TriAttInSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, t0 = blockIdx.x * 128;

  auto load_chunk = [&](int c, int buf) {
    if (c < 6) {
      const bf16* w = (c < 2) ? w_q : (c < 4 ? w_k : w_v);
      load_w_rows(sm.W[buf], 0, w, 64 * (c & 1), 64, tid);
    } else {  // bias projection: 4 real rows, rows 4..15 zero
      const int r = tid >> 4, ch = tid & 15;
      cp_async16(smem_u32(sm.W[buf] + r * kLdA + ch * 8), w_bias + (size_t)(r < kH ? r : 0) * kC + ch * 8, r < kH);
    }
    cp_async_commit();
  };
  load_chunk(0, 0);

  // z (and the mask) is [n_u][n] pair elements, or [n][n_u] when the two indices are exchanged
  auto pair_index = [&](int t) -> size_t { return swap ? ((size_t)t * n_u + u) : ((size_t)u * n + t); };
  ln_tile_rows<Tz>(sm.A, warp, lane, ln_w, ln_b, eps, [&](int r) -> const Tz* {
    int t = t0 + r;
    return t < n ? z + pair_index(t) * kC : nullptr;
  });
  __syncwarp();
  uint32_t afr[8][4];
  load_a_frags(afr, sm.A, warp, lane);

  if (tid < 128) {  // mask bias, -inf in the pad columns [n, ldm)
    const int t = t0 + tid;
    if (t < ldm) {
      float mv = -CUDART_INF_F;
      if (t < n) mv = mask ? (mask[pair_index(t)] - 1.0f) * inf * kLog2e : 0.f;
      mb_out[(size_t)u * ldm + t] = mv;
    }
  }

  const int g = lane >> 2, tq = lane & 3;
  const int tr = t0 + 16 * warp + g;
  const float qscale = kLog2e * rsqrtf((float)kD);
  for (int c = 0; c < 7; ++c) {
    if (c + 1 < 7) {
      load_chunk(c + 1, (c + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    if (c >= 4 && c < 6) {
      // v is stored transposed, [u][h][d][t] with t contiguous (row stride ldt, zero pad columns), so
      // that the value tile is a K-major operand of the P.V product
      warp_gemm_k128<0, 8, 8>(acc, afr, sm.W[c & 1], lane);
      const int r0 = 16 * warp + g;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int ch = 8 * j + 2 * tq;
        sm.S[ch * kLdA + r0] = __float2bfloat16_rn(acc[j][0]);
        sm.S[(ch + 1) * kLdA + r0] = __float2bfloat16_rn(acc[j][1]);
        sm.S[ch * kLdA + r0 + 8] = __float2bfloat16_rn(acc[j][2]);
        sm.S[(ch + 1) * kLdA + r0 + 8] = __float2bfloat16_rn(acc[j][3]);
      }
      __syncthreads();
      {
        const int ch = tid >> 2, seg = tid & 3;  // 64 channels x 4 segments of 32 t
        const size_t row = (((size_t)u * kH + 2 * (c & 1) + (ch >> 5)) * kD + (ch & 31)) * ldt;
#pragma unroll
        for (int h8 = 0; h8 < 4; ++h8) {
          const int t = t0 + seg * 32 + h8 * 8;
          if (t < ldt)
            *reinterpret_cast<uint4*>(v_out + row + t) =
                *reinterpret_cast<const uint4*>(sm.S + ch * kLdA + seg * 32 + h8 * 8);
        }
      }
    } else if (c < 4) {
      warp_gemm_k128<0, 8, 8>(acc, afr, sm.W[c & 1], lane);
      bf16* dst = (c < 2) ? q_out : k_out;
      const float sc = (c < 2) ? qscale : 1.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int head = 2 * (c & 1) + (j >> 2);
        const int d = (j & 3) * 8 + 2 * tq;
        const size_t base = ((size_t)u * kH + head) * n;
        if (tr < n)
          *reinterpret_cast<uint32_t*>(dst + (base + tr) * kD + d) = pack_bf16x2(acc[j][0] * sc, acc[j][1] * sc);
        if (tr + 8 < n)
          *reinterpret_cast<uint32_t*>(dst + (base + tr + 8) * kD + d) = pack_bf16x2(acc[j][2] * sc, acc[j][3] * sc);
      }
    } else {
      warp_gemm_k128<0, 2, 8>(acc, afr, sm.W[c & 1], lane);
      if (tq < 2) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int head = 2 * tq + e;
          // zero in the pad columns [n, ldm)
          if (tr < ldm) bias_out[((size_t)head * n_u + u) * ldm + tr] = tr < n ? acc[0][e] * kLog2e : 0.f;
          if (tr + 8 < ldm) bias_out[((size_t)head * n_u + u) * ldm + tr + 8] = tr + 8 < n ? acc[0][2 + e] * kLog2e : 0.f;
        }
      }
    }
    __syncthreads();
  }
}

// =========================================================================================
// Stage 2: flash attention.  One CTA = (64 queries, head h, R attended rows u); 4 warps x 16
// queries.  For every 64-key tile the pair-bias fragment [q][k] is fetched once (prefetched one
// tile ahead into registers) and reused by the R rows; logits start as bias + mask_bias in the
// accumulator of the q.k product.  K, V and mask_bias tiles arrive through a double-buffered
// cp.async pipeline.  bias and mask_bias rows are padded to a multiple of 64 keys (bias 0,
// mask_bias -inf in the pad) so the inner loop carries no column predicates.
// =========================================================================================
constexpr int kFaLd = kD + 8;  // shared row stride of q/k/v tiles (80 bytes: conflict-free ldmatrix)

constexpr int kFaLdV = 64 + 8;  // row stride of a transposed value tile [32 d][64 keys]

template <int R>
struct FlashSmem {
  bf16 Q[R][64 * kFaLd];
  bf16 K[2][R][64 * kFaLd];
  bf16 V[2][R][kD * kFaLdV];
  float MB[2][R][64];
};

template <int R>
__global__ void __launch_bounds__(128, 2)
triatt_flash_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                    const float* __restrict__ bias, const float* __restrict__ mb, bf16* __restrict__ o, int n_u,
                    int n, int ldm, int ldt) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FlashSmem<R>& sm = *reinterpret_cast<FlashSmem<R>*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = blockIdx.x * 64, h = blockIdx.y, u0 = blockIdx.z * R;
  const int g = lane >> 2, tq = lane & 3;
  const int nkt = (n + 63) / 64;

  auto rows_base = [&](int r) -> size_t { return ((size_t)(u0 + r) * kH + h) * n; };
  auto load_kv = [&](int kt, int stage) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool urow = (u0 + r) < n_u;
      const size_t base = urow ? rows_base(r) : 0;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int idx = tid + 128 * it, row = idx >> 2, ch = idx & 3;
        const bool p = urow && (kt * 64 + row) < n;
        const size_t off = p ? (base + kt * 64 + row) * kD + ch * 8 : 0;
        cp_async16(smem_u32(sm.K[stage][r] + row * kFaLd + ch * 8), k + off, p);
        // value tile, transposed: 32 rows (d) x 64 keys, 8 pieces of 16 bytes per row
        const int d = idx >> 3, kc = idx & 7;
        const bool pv = urow && (kt * 64 + kc * 8) < ldt;
        const size_t offv = pv ? (((size_t)(u0 + r) * kH + h) * kD + d) * ldt + kt * 64 + kc * 8 : 0;
        cp_async16(smem_u32(sm.V[stage][r] + d * kFaLdV + kc * 8), v + offv, pv);
      }
    }
    if (tid < R * 16) {
      const int r = tid >> 4, ch = tid & 15;
      const bool urow = (u0 + r) < n_u;
      cp_async16(smem_u32(&sm.MB[stage][r][ch * 4]), mb + (urow ? (size_t)(u0 + r) * ldm + kt * 64 + ch * 4 : 0), urow);
    }
  };
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const bool urow = (u0 + r) < n_u;
    const size_t base = urow ? rows_base(r) : 0;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = tid + 128 * it, row = idx >> 2, ch = idx & 3;
      const bool p = urow && (q0 + row) < n;
      cp_async16(smem_u32(sm.Q[r] + row * kFaLd + ch * 8), q + (p ? (base + q0 + row) * kD + ch * 8 : 0), p);
    }
  }
  load_kv(0, 0);
  cp_async_commit();

  uint32_t qf[R][2][4];
  // oacc[r][0..3]: output columns; oacc[r][4]: row sums of P, produced by the same MMA against a
  // constant "ones" column, so they are rescaled together with the output.
  float oacc[R][5][4], mrow[R][2];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    mrow[r][0] = mrow[r][1] = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 5; ++j) oacc[r][j][0] = oacc[r][j][1] = oacc[r][j][2] = oacc[r][j][3] = 0.f;
  }
  const uint32_t ones_b = (g == 0) ? 0x3F803F80u : 0u;  // B fragment of a [16 x 8] tile whose column 0 is 1
  const int qr = q0 + 16 * warp + g;  // this thread's query rows: qr and qr + 8
  // rows of the pair bias this thread reads (clamped: out-of-range queries are never stored)
  const float* brow0 = bias + ((size_t)h * n + min(qr, n - 1)) * ldm + 2 * tq;
  const float* brow1 = bias + ((size_t)h * n + min(qr + 8, n - 1)) * ldm + 2 * tq;
  float2 bnext[8][2];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    bnext[j][0] = *reinterpret_cast<const float2*>(brow0 + 8 * j);
    bnext[j][1] = *reinterpret_cast<const float2*>(brow1 + 8 * j);
  }

  for (int kt = 0; kt < nkt; ++kt) {
    cp_async_wait<0>();
    __syncthreads();
    if (kt + 1 < nkt) load_kv(kt + 1, (kt + 1) & 1);
    cp_async_commit();
    if (kt == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) load_a_frag(qf[r][ks], sm.Q[r], kFaLd, warp, lane, ks);
    }
    // pair-bias fragment of this tile (shared by the R rows); fetch the next tile's behind the math
    float2 bcur[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      bcur[j][0] = bnext[j][0];
      bcur[j][1] = bnext[j][1];
    }
    if (kt + 1 < nkt) {
      const int ko = (kt + 1) * 64;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        bnext[j][0] = *reinterpret_cast<const float2*>(brow0 + ko + 8 * j);
        bnext[j][1] = *reinterpret_cast<const float2*>(brow1 + ko + 8 * j);
      }
    }
    const int stage = kt & 1;
#pragma unroll
    for (int r = 0; r < R; ++r) {  // rows past the end run on zero tiles and are not stored
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 mv = *reinterpret_cast<const float2*>(&sm.MB[stage][r][8 * j + 2 * tq]);
        s[j][0] = bcur[j][0].x + mv.x;
        s[j][1] = bcur[j][0].y + mv.y;
        s[j][2] = bcur[j][1].x + mv.x;
        s[j][3] = bcur[j][1].y + mv.y;
      }
      // S += Q K^T
      {
        const bf16* Ks = sm.K[stage][r];
        const int nrow = (lane & 7) + (lane >> 4) * 8;
        const int kof = ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_u32(Ks + (np * 16 + nrow) * kFaLd + ks * 16 + kof));
            mma_bf16(s[2 * np], qf[r][ks], b[0], b[1]);
            mma_bf16(s[2 * np + 1], qf[r][ks], b[2], b[3]);
          }
      }
      // online softmax (base 2)
      float mx0 = s[0][0], mx1 = s[0][2];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(mrow[r][0], mx0), mn1 = fmaxf(mrow[r][1], mx1);
      const float al0 = fast_exp2(mrow[r][0] - mn0), al1 = fast_exp2(mrow[r][1] - mn1);
      mrow[r][0] = mn0;
      mrow[r][1] = mn1;
      uint32_t pf[4][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pf[j >> 1][(j & 1) * 2] = exp2_bf16x2(s[j][0] - mn0, s[j][1] - mn0);
        pf[j >> 1][(j & 1) * 2 + 1] = exp2_bf16x2(s[j][2] - mn1, s[j][3] - mn1);
      }
#pragma unroll
      for (int j = 0; j < 5; ++j) {
        oacc[r][j][0] *= al0;
        oacc[r][j][1] *= al0;
        oacc[r][j][2] *= al1;
        oacc[r][j][3] *= al1;
      }
      // O += P V
      {
        const bf16* Vs = sm.V[stage][r];
        const int drow = (lane & 7) + (lane >> 4) * 8;
        const int kof2 = ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
          for (int dp = 0; dp < 2; ++dp) {
            uint32_t b[4];
            ldmatrix_x4(b, smem_u32(Vs + (dp * 16 + drow) * kFaLdV + kk * 16 + kof2));
            mma_bf16(oacc[r][2 * dp], pf[kk], b[0], b[1]);
            mma_bf16(oacc[r][2 * dp + 1], pf[kk], b[2], b[3]);
          }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) mma_bf16(oacc[r][4], pf[kk], ones_b, ones_b);
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (u0 + r >= n_u) continue;
    // row sums sit in column 0 of the extra tile: lane 4*g of each quad holds them
    const float l0 = __shfl_sync(0xffffffffu, oacc[r][4][0], lane & ~3);
    const float l1 = __shfl_sync(0xffffffffu, oacc[r][4][2], lane & ~3);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    bf16* orow = o + ((size_t)(u0 + r) * n) * kC + h * kD;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = 8 * j + 2 * tq;
      if (qr < n)
        *reinterpret_cast<uint32_t*>(orow + (size_t)qr * kC + d) = pack_bf16x2(oacc[r][j][0] * i0, oacc[r][j][1] * i0);
      if (qr + 8 < n)
        *reinterpret_cast<uint32_t*>(orow + (size_t)(qr + 8) * kC + d) =
            pack_bf16x2(oacc[r][j][2] * i1, oacc[r][j][3] * i1);
    }
  }
}

// =========================================================================================
// Stage 3: z_out(u,t) = [z(u,t) +] W_o (o[u][t] * sigmoid(W_g LN(z(u,t)))).
// HBM-bound: reads 256 (o) + 128*sizeof(Tz), writes 128*sizeof(Tz) per pair element.
// =========================================================================================
struct TriAttOutSmem {
  bf16 A[128 * kLdA];
  bf16 O[128 * kLdA];
  bf16 W[2][64 * kLdA];
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
triatt_out_kernel(const bf16* __restrict__ o, const Tz* __restrict__ z_in, Tz* __restrict__ z_out,
                  const float* __restrict__ ln_w, const float* __restrict__ ln_b, const bf16* __restrict__ w_g,
                  const bf16* __restrict__ w_o, int n_u, int n, int swap, int add_residual, float eps) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TriAttOutSmem& sm = *reinterpret_cast<TriAttOutSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int u = blockIdx.y, t0 = blockIdx.x * 128;

  // o tile rows [t][128]
  for (int idx = tid; idx < 128 * 16; idx += 256) {
    const int r = idx >> 4, ch = idx & 15;
    const bool p = (t0 + r) < n;
    cp_async16(smem_u32(sm.O + r * kLdA + ch * 8), p ? (o + ((size_t)u * n + t0 + r) * kC + ch * 8) : o, p);
  }
  cp_async_commit();
  auto load_chunk = [&](int c, int buf) {
    load_w_rows(sm.W[buf], 0, (c < 2) ? w_g : w_o, 64 * (c & 1), 64, tid);
    cp_async_commit();
  };
  load_chunk(0, 0);

  auto pair_index = [&](int t) -> size_t { return swap ? ((size_t)t * n_u + u) : ((size_t)u * n + t); };
  ln_tile_rows<Tz>(sm.A, warp, lane, ln_w, ln_b, eps, [&](int r) -> const Tz* {
    int t = t0 + r;
    return t < n ? z_in + pair_index(t) * kC : nullptr;
  });
  __syncwarp();
  uint32_t afr[8][4];
  load_a_frags(afr, sm.A, warp, lane);

  const int g = lane >> 2, tq = lane & 3;
  const int rl = 16 * warp + g;  // local rows rl, rl + 8
  uint32_t og[8][4];             // gated o as A fragments of the output projection
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (c + 1 < 4) {
      load_chunk(c + 1, (c + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    if (c < 2) {
      warp_gemm_k128<0, 8, 8>(acc, afr, sm.W[c & 1], lane);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 64 * c + 8 * j + 2 * tq;
        float2 o0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sm.O + rl * kLdA + col));
        float2 o1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sm.O + (rl + 8) * kLdA + col));
        const uint32_t lo = pack_bf16x2(o0.x * sigmoidf_fast(acc[j][0]), o0.y * sigmoidf_fast(acc[j][1]));
        const uint32_t hi = pack_bf16x2(o1.x * sigmoidf_fast(acc[j][2]), o1.y * sigmoidf_fast(acc[j][3]));
        const int ks = 4 * c + (j >> 1);
        og[ks][(j & 1) * 2] = lo;
        og[ks][(j & 1) * 2 + 1] = hi;
      }
    } else {
      warp_gemm_k128<0, 8, 8>(acc, og, sm.W[c & 1], lane);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = 64 * (c & 1) + 8 * j + 2 * tq;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int t = t0 + rl + 8 * hh;
          if (t < n) {
            const size_t off = pair_index(t) * kC + col;
            float v0 = acc[j][2 * hh], v1 = acc[j][2 * hh + 1];
            if (add_residual) {
              float2 r = load2(z_in + off);
              v0 += r.x;
              v1 += r.y;
            }
            store2(z_out + off, v0, v1);
          }
        }
      }
    }
    __syncthreads();
  }
}

static size_t att_qkv_elems(int64_t n) { return (size_t)n * kH * px_ld(n) * kD; }
static size_t align256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace px

using namespace px;

static bool att_bad_dims(int64_t n_u, int64_t n, int64_t ldm) {
  return n_u <= 0 || n <= 0 || n_u > 32768 || n > 32768 || ldm != px_ld_mask(n);
}

extern "C" int32_t px_triatt_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w,
                                     const float* ln_b, const px_bf16* w_q, const px_bf16* w_k, const px_bf16* w_v,
                                     const px_bf16* w_bias, px_bf16* q, px_bf16* k, px_bf16* v, float* bias,
                                     float* mask_bias, int64_t n_u, int64_t n_t, int64_t ldm, int32_t ending,
                                     float eps, float inf, void* stream) {
  if (!z || !ln_w || !ln_b || !w_q || !w_k || !w_v || !w_bias || !q || !k || !v || !bias || !mask_bias ||
      att_bad_dims(n_u, n_t, ldm))
    return PX_ERR_BAD_ARG;
  dim3 grid((unsigned)((n_t + 127) / 128), (unsigned)n_u);  // 128-wide tiles cover the pad columns up to ldm too
  const size_t smem = sizeof(TriAttInSmem);
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == PX_F32) {
    if (cudaFuncSetAttribute(triatt_in_proj_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_in_proj_kernel<float><<<grid, 256, smem, st>>>(
        (const float*)z, mask, ln_w, ln_b, (const bf16*)w_q, (const bf16*)w_k, (const bf16*)w_v,
        (const bf16*)w_bias, (bf16*)q, (bf16*)k, (bf16*)v, bias, mask_bias, (int)n_u, (int)n_t, (int)ldm, (int)px_ld(n_t), ending,
        eps, inf);
  } else if (z_dtype == PX_BF16) {
    if (cudaFuncSetAttribute(triatt_in_proj_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_in_proj_kernel<bf16><<<grid, 256, smem, st>>>(
        (const bf16*)z, mask, ln_w, ln_b, (const bf16*)w_q, (const bf16*)w_k, (const bf16*)w_v, (const bf16*)w_bias,
        (bf16*)q, (bf16*)k, (bf16*)v, bias, mask_bias, (int)n_u, (int)n_t, (int)ldm, (int)px_ld(n_t), ending, eps,
        inf);
  } else {
    return PX_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

constexpr int kFlashR = 2;

extern "C" int32_t px_triatt_flash(const px_bf16* q, const px_bf16* k, const px_bf16* v, const float* bias,
                                   const float* mask_bias, px_bf16* o, int64_t n_u, int64_t n, int64_t ldm,
                                   void* stream) {
  if (!q || !k || !v || !bias || !mask_bias || !o || att_bad_dims(n_u, n, ldm)) return PX_ERR_BAD_ARG;
  dim3 grid((unsigned)((n + 63) / 64), kH, (unsigned)((n_u + kFlashR - 1) / kFlashR));
  const size_t smem = sizeof(FlashSmem<kFlashR>);
  if (cudaFuncSetAttribute(triatt_flash_kernel<kFlashR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return PX_ERR_LAUNCH;
  triatt_flash_kernel<kFlashR><<<grid, 128, smem, (cudaStream_t)stream>>>(
      (const bf16*)q, (const bf16*)k, (const bf16*)v, bias, mask_bias, (bf16*)o, (int)n_u, (int)n, (int)ldm,
      (int)px_ld(n));
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int32_t px_triatt_out(const px_bf16* o, const void* z_in, void* z_out, int32_t z_dtype, const float* ln_w,
                                 const float* ln_b, const px_bf16* w_g, const px_bf16* w_o, int64_t n_u, int64_t n_t,
                                 int32_t ending, int32_t add_residual, float eps, void* stream) {
  if (!o || !z_in || !z_out || !ln_w || !ln_b || !w_g || !w_o || n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768)
    return PX_ERR_BAD_ARG;
  dim3 grid((unsigned)((n_t + 127) / 128), (unsigned)n_u);
  const size_t smem = sizeof(TriAttOutSmem);
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == PX_F32) {
    if (cudaFuncSetAttribute(triatt_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_out_kernel<float><<<grid, 256, smem, st>>>((const bf16*)o, (const float*)z_in, (float*)z_out, ln_w, ln_b,
                                                      (const bf16*)w_g, (const bf16*)w_o, (int)n_u, (int)n_t, ending,
                                                      add_residual, eps);
  } else if (z_dtype == PX_BF16) {
    if (cudaFuncSetAttribute(triatt_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    triatt_out_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)o, (const bf16*)z_in, (bf16*)z_out, ln_w, ln_b,
                                                     (const bf16*)w_g, (const bf16*)w_o, (int)n_u, (int)n_t, ending,
                                                     add_residual, eps);
  } else {
    return PX_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int64_t px_ld_mask(int64_t n) { return (n + 63) / 64 * 64; }

// workspace layout: q | k | v | o (bf16) | bias (fp32 [4][n][ldm]) | mask_bias (fp32 [n][ldm])
extern "C" int64_t px_triatt_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  const int64_t ld = px_ld_mask(n);
  return (int64_t)(3 * align256(att_qkv_elems(n) * 2) + align256((size_t)n * n * kC * 2) +
                   align256((size_t)kH * n * ld * 4) + align256((size_t)n * ld * 4));
}

extern "C" int32_t px_triangle_attention(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                         const float* ln_w, const float* ln_b, const px_bf16* w_bias,
                                         const px_bf16* w_q, const px_bf16* w_k, const px_bf16* w_v,
                                         const px_bf16* w_g, const px_bf16* w_o, void* workspace,
                                         int64_t workspace_bytes, int64_t n, int32_t ending, int32_t add_residual,
                                         float eps, float inf, void* stream) {
  if (!workspace || n <= 0 || ((uintptr_t)workspace & 255)) return PX_ERR_BAD_ARG;
  if (workspace_bytes < px_triatt_workspace_bytes(n)) return PX_ERR_WORKSPACE;
  const int64_t ld = px_ld_mask(n);
  unsigned char* p = (unsigned char*)workspace;
  px_bf16* q = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* k = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* v = (px_bf16*)p;
  p += align256(att_qkv_elems(n) * 2);
  px_bf16* o = (px_bf16*)p;
  p += align256((size_t)n * n * kC * 2);
  float* bias = (float*)p;
  p += align256((size_t)kH * n * ld * 4);
  float* mbias = (float*)p;
  int32_t s = px_triatt_in_proj(z_in, z_dtype, mask, ln_w, ln_b, w_q, w_k, w_v, w_bias, q, k, v, bias, mbias, n, n,
                                ld, ending, eps, inf, stream);
  if (s != PX_OK) return s;
  s = px_triatt_flash(q, k, v, bias, mbias, o, n, n, ld, stream);
  if (s != PX_OK) return s;
  return px_triatt_out(o, z_in, z_out, z_dtype, ln_w, ln_b, w_g, w_o, n, n, ending, add_residual, eps, stream);
}
