// Triangle multiplication: input projection, channel-batched contraction, output stage.
#include "px_common.cuh"

namespace px {

// Stage 1 (the gated input projections) lives in trimul_in_tc.cu.
// Stage 2 (the channel-batched contraction) lives in contract_tcgen05.cu.

// =========================================================================================
// Stage 3: z_out = [z +] W_z LN_out(x) * sigmoid(W_g LN_in(z)).  One CTA = (i, 128 consecutive j).
// x arrives channel-major (256-byte runs per channel) and is transposed through shared memory.
// HBM-bound: reads 256 (x) + sizeof(Tz)*128 (z), writes sizeof(Tz)*128 per pair element.
// =========================================================================================
struct TriMulOutSmem {
  bf16 A1[128 * kLdA];      // LN_out(x) rows [j][c]
  bf16 XS[128 * kLdA];      // raw x tile [c][j]; later reused for LN_in(z) rows [j][c]
  bf16 W[2][64 * kLdA];     // rows 0..31 of W_z chunk, rows 32..63 of W_g chunk
  float red[2][128];
  float stat[2][128];       // mean, rstd per j
};

template <typename Tz>
__global__ void __launch_bounds__(256, 2)
trimul_out_kernel(const bf16* __restrict__ x, const Tz* __restrict__ z_in, Tz* __restrict__ z_out,
                  const float* __restrict__ ln_in_w, const float* __restrict__ ln_in_b,
                  const float* __restrict__ ln_out_w, const float* __restrict__ ln_out_b,
                  const bf16* __restrict__ w_z, const bf16* __restrict__ w_g, int n_i, int n, int ld, int add_residual,
                  float eps) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TriMulOutSmem& sm = *reinterpret_cast<TriMulOutSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int i = blockIdx.y, j0 = blockIdx.x * 128;

  // x tile: 128 channels x 128 j (16-byte pieces, zero beyond ld)
  for (int idx = tid; idx < 128 * 16; idx += 256) {
    const int c = idx >> 4, seg = idx & 15;
    const int j = j0 + seg * 8;
    const bool p = j < ld;
    cp_async16(smem_u32(sm.XS + c * kLdA + seg * 8), p ? (x + ((size_t)c * n_i + i) * ld + j) : x, p);
  }
  cp_async_commit();
  auto load_chunk = [&](int q, int buf) {
    load_w_rows(sm.W[buf], 0, w_z, 32 * q, 32, tid);
    load_w_rows(sm.W[buf], 32, w_g, 32 * q, 32, tid);
    cp_async_commit();
  };
  load_chunk(0, 0);
  cp_async_wait<1>();
  __syncthreads();

  // statistics over c for each j: two threads per j, each half of the channels
  {
    const int j = tid & 127, half = tid >> 7;
    float s = 0.f;
#pragma unroll 8
    for (int c = 0; c < 64; ++c) s += __bfloat162float(sm.XS[(64 * half + c) * kLdA + j]);
    sm.red[half][j] = s;
    __syncthreads();
    const float mean = (sm.red[0][j] + sm.red[1][j]) * (1.0f / kC);
    float qv = 0.f;
#pragma unroll 8
    for (int c = 0; c < 64; ++c) {
      float d = __bfloat162float(sm.XS[(64 * half + c) * kLdA + j]) - mean;
      qv += d * d;
    }
    __syncthreads();
    sm.red[half][j] = qv;
    __syncthreads();
    if (half == 0) {
      sm.stat[0][j] = mean;
      sm.stat[1][j] = rsqrtf((sm.red[0][j] + sm.red[1][j]) * (1.0f / kC) + eps);
    }
    __syncthreads();
  }
  // transpose + normalise into A1: warp handles its own 16 rows j; lane = jj + 8*cc
  {
    const int jj = lane & 7, cc = lane >> 3;
#pragma unroll 4
    for (int it = 0; it < 32; ++it) {
      const int j = 16 * warp + (it & 1) * 8 + jj;
      const int c = ((it >> 1) * 4 + cc) * 2;
      const float mean = sm.stat[0][j], rstd = sm.stat[1][j];
      float v0 = (__bfloat162float(sm.XS[c * kLdA + j]) - mean) * rstd * ln_out_w[c] + ln_out_b[c];
      float v1 = (__bfloat162float(sm.XS[(c + 1) * kLdA + j]) - mean) * rstd * ln_out_w[c + 1] + ln_out_b[c + 1];
      if (j0 + j >= n) v0 = v1 = 0.f;
      *reinterpret_cast<uint32_t*>(sm.A1 + j * kLdA + c) = pack_bf16x2(v0, v1);
    }
  }
  __syncthreads();  // every warp is done with the raw x tile
  ln_tile_rows<Tz>(sm.XS, warp, lane, ln_in_w, ln_in_b, eps, [&](int r) -> const Tz* {
    int j = j0 + r;
    return j < n ? z_in + ((size_t)i * n + j) * kC : nullptr;
  });
  __syncwarp();
  uint32_t a1[8][4], a2[8][4];
  load_a_frags(a1, sm.A1, warp, lane);
  load_a_frags(a2, sm.XS, warp, lane);

  const int g = lane >> 2, tq = lane & 3;
  const int jr = j0 + 16 * warp + g;
  for (int q = 0; q < 4; ++q) {
    if (q + 1 < 4) {
      load_chunk(q + 1, (q + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    warp_gemm_k128<0, 4, 8>(acc, a1, sm.W[q & 1], lane);
    warp_gemm_k128<4, 4, 8>(acc, a2, sm.W[q & 1], lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = 32 * q + 8 * j + 2 * tq;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int jrow = jr + 8 * h;
        if (jrow < n) {
          const size_t off = ((size_t)i * n + jrow) * kC + col;
          float v0 = acc[j][2 * h] * sigmoidf_fast(acc[j + 4][2 * h]);
          float v1 = acc[j][2 * h + 1] * sigmoidf_fast(acc[j + 4][2 * h + 1]);
          if (add_residual) {
            float2 r = load2(z_in + off);
            v0 += r.x;
            v1 += r.y;
          }
          store2(z_out + off, v0, v1);
        }
      }
    }
    __syncthreads();  // all warps done with W[q&1] before it is refilled two chunks later
  }
}

static size_t trimul_elems(int64_t n) { return (size_t)kC * n * px_ld(n); }

}  // namespace px

using namespace px;

extern "C" int64_t px_ld(int64_t n) { return (n + 7) / 8 * 8; }

static bool bad_dims(int64_t n_u, int64_t n_t, int64_t ld) {
  return n_u <= 0 || n_t <= 0 || n_u > 32768 || n_t > 32768 || ld != px_ld(n_t);
}

extern "C" int32_t px_trimul_out(const px_bf16* x, const void* z_in, void* z_out, int32_t z_dtype,
                                 const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                 const float* ln_out_b, const px_bf16* w_z, const px_bf16* w_g, int64_t n_i,
                                 int64_t n_j, int64_t ld, int32_t add_residual, float eps, void* stream) {
  if (!x || !z_in || !z_out || !ln_in_w || !ln_in_b || !ln_out_w || !ln_out_b || !w_z || !w_g ||
      bad_dims(n_i, n_j, ld))
    return PX_ERR_BAD_ARG;
  dim3 grid((unsigned)((n_j + 127) / 128), (unsigned)n_i);
  const size_t smem = sizeof(TriMulOutSmem);
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == PX_F32) {
    if (cudaFuncSetAttribute(trimul_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    trimul_out_kernel<float><<<grid, 256, smem, st>>>((const bf16*)x, (const float*)z_in, (float*)z_out, ln_in_w,
                                                      ln_in_b, ln_out_w, ln_out_b, (const bf16*)w_z,
                                                      (const bf16*)w_g, (int)n_i, (int)n_j, (int)ld, add_residual,
                                                      eps);
  } else if (z_dtype == PX_BF16) {
    if (cudaFuncSetAttribute(trimul_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return PX_ERR_LAUNCH;
    trimul_out_kernel<bf16><<<grid, 256, smem, st>>>((const bf16*)x, (const bf16*)z_in, (bf16*)z_out, ln_in_w,
                                                     ln_in_b, ln_out_w, ln_out_b, (const bf16*)w_z, (const bf16*)w_g,
                                                     (int)n_i, (int)n_j, (int)ld, add_residual, eps);
  } else {
    return PX_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
extern "C" int64_t px_trimul_workspace_bytes(int64_t n) {
  if (n <= 0) return 0;
  return (int64_t)(3 * trimul_elems(n) * sizeof(bf16));
}

extern "C" int32_t px_triangle_multiplication(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                              const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                              const float* ln_out_b, const px_bf16* w_ap, const px_bf16* w_ag,
                                              const px_bf16* w_bp, const px_bf16* w_bg, const px_bf16* w_z,
                                              const px_bf16* w_g, void* workspace, int64_t workspace_bytes, int64_t n,
                                              int32_t incoming, int32_t add_residual, float eps, void* stream) {
  if (!workspace || n <= 0) return PX_ERR_BAD_ARG;
  if (workspace_bytes < px_trimul_workspace_bytes(n)) return PX_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return PX_ERR_BAD_ARG;
  const int64_t ld = px_ld(n);
  px_bf16* a = (px_bf16*)workspace;
  px_bf16* b = a + trimul_elems(n);
  px_bf16* x = b + trimul_elems(n);
  int32_t s = px_trimul_in_proj(z_in, z_dtype, mask, ln_in_w, ln_in_b, w_ap, w_ag, w_bp, w_bg, a, b, n, n, ld,
                                incoming, eps, stream);
  if (s != PX_OK) return s;
  s = px_trimul_contract(a, b, x, kC, n, ld, stream);
  if (s != PX_OK) return s;
  return px_trimul_out(x, z_in, z_out, z_dtype, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_z, w_g, n, n, ld,
                       add_residual, eps, stream);
}

// =========================================================================================
// Triangle multiplication for callers that cannot allocate device memory.
//
// The three stages need scratch for a, b and x.  Here that scratch is a fixed array that is part
// of the loaded library image, so the call needs no workspace from the caller and makes no
// cudaMalloc / cudaFree.  The array is 12 MiB (N <= 128) and every GPU that loads the library
// holds it until the process exits.
// =========================================================================================
constexpr int64_t kStaticMaxN = PX_STATIC_MAX_N;
constexpr size_t kStaticScratchBytes = 3 * (size_t)px::kC * kStaticMaxN * kStaticMaxN * sizeof(px::bf16);
static __device__ __align__(256) unsigned char g_trimul_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the scratch array per device ordinal.  In host code the array's name is only a
// handle for the runtime, not a device address: the address has to be asked for, once per device,
// with that device current.  Benign race: two threads may both ask and store the same value.
void* g_static_scratch_addr[kMaxDevices] = {};

int32_t static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PX_ERR_LAUNCH;
  void* p = g_static_scratch_addr[dev];
  if (!p) {
    cudaError_t e = cudaGetSymbolAddress(&p, g_trimul_static_scratch);
    if (e != cudaSuccess || !p) return PX_ERR_LAUNCH;
    g_static_scratch_addr[dev] = p;
  }
  *out = p;
  return PX_OK;
}
}  // namespace

extern "C" int64_t px_static_max_n(void) { return kStaticMaxN; }

extern "C" int32_t px_triangle_multiplication_static(const void* z_in, void* z_out, int32_t z_dtype,
                                                     const float* mask, const float* ln_in_w, const float* ln_in_b,
                                                     const float* ln_out_w, const float* ln_out_b,
                                                     const px_bf16* w_ap, const px_bf16* w_ag, const px_bf16* w_bp,
                                                     const px_bf16* w_bg, const px_bf16* w_z, const px_bf16* w_g,
                                                     int64_t n, int32_t incoming, int32_t add_residual, float eps,
                                                     void* stream) {
  if (n <= 0) return PX_ERR_BAD_ARG;
  if (n > kStaticMaxN) return PX_ERR_TOO_LARGE;
  void* scratch = nullptr;
  int32_t s = static_scratch(&scratch);
  if (s != PX_OK) return s;
  // Layout for this N: a | b | x, each [128][N][ld] bf16.  Every element a stage reads was written
  // earlier in the same call (the projection also writes the zero pad columns), so nothing left by
  // a previous call, possibly with another N, has to be cleared.
  return px_triangle_multiplication(z_in, z_out, z_dtype, mask, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_ap, w_ag, w_bp,
                                    w_bg, w_z, w_g, scratch, (int64_t)kStaticScratchBytes, n, incoming, add_residual,
                                    eps, stream);
}
