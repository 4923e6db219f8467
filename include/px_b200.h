/*
 * px_b200 -- C ABI of the sm_100a Pairformer pair-representation kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a `cudaStream_t` passed as `void*`; NULL = the legacy default stream), launches
 * asynchronously on that stream and returns PX_OK or a negative status.  Nothing here
 * allocates device memory: intermediate tensors are carved from a caller-provided
 * workspace whose size the `*_workspace_bytes` functions report.  No exception crosses
 * this boundary.  Entry points are re-entrant across streams as long as calls do not
 * share output or workspace memory.
 *
 * Conventions
 *   - N            number of tokens; the pair tensor z is [N][N][128], row-major, channel last.
 *   - z_dtype      storage type of the residual stream: PX_F32 or PX_BF16.  All matrix products
 *                  take 16-bit operands and accumulate in fp32.  Rows of a bf16 z are multiplied as
 *                  they are stored (bf16 x bf16).  For an fp32 z the kernels multiply a standardised
 *                  fp16 copy of the rows, zn = (z - mean) * rstd, written by px_standardise_rows
 *                  (fp16 x fp16: a standardised row cannot leave the fp16 range, and fp16 keeps three
 *                  more mantissa bits).  The composite entry points make that copy in their
 *                  workspace; the stage entry points take it as an argument: stages that only
 *                  read LayerNorm'd rows accept PX_BF16 (the rows of z) or PX_F16 (the copy),
 *                  stages that also add the residual take z (PX_BF16 or PX_F32) and, for PX_F32, zn.  Every intermediate 16-bit tensor (a, b, x, q, k, v, o)
 *                  is fp16 in both cases.
 *   - weights      16-bit, row-major [out_features][in_features] exactly as the reference's
 *                  nn.Linear.weight, cast by the caller: px_w16 parameters take the format of the z
 *                  they multiply (bf16 for PX_BF16, fp16 for PX_F32); px_f16 weight parameters
 *                  (they multiply an fp16 intermediate) take fp16 always.  LayerNorm scale/offset fp32.
 *   - mask         fp32 [N][N] (1 = keep, 0 = masked) or NULL for all ones.
 *   - ld           px_ld(N): N rounded up to a multiple of 8; row stride (in elements) of the
 *                  intermediate tensors so that every row starts on a 16-byte boundary.
 *   - n_u, n_t     the stage entry points work on a rectangular slab of pair elements (u, t),
 *                  u < n_u, t < n_t: the whole pair tensor (n_u = n_t = N) or, when z is sharded
 *                  by rows over several GPUs, the local rows (n_u = N / ranks, n_t = N).  The slab
 *                  is stored [n_u][n_t][128]; with `incoming` / `ending` set it is stored
 *                  [n_t][n_u][128] and read transposed.
 *
 * The reference interfaces each entry point stands in for are cited as file:line of
 * bytedance/Protenix v2.0.0.
 */
#ifndef PX_B200_H_
#define PX_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PX_OK 0
#define PX_ERR_BAD_ARG (-1)     /* null pointer, non-positive size, misaligned pointer */
#define PX_ERR_UNSUPPORTED (-2) /* shape / dtype outside the compiled specialisations   */
#define PX_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch                  */
#define PX_ERR_WORKSPACE (-4)   /* workspace too small                                  */
#define PX_ERR_TOO_LARGE (-5)   /* N beyond the capacity of the built-in scratch array  */

#define PX_STATIC_MAX_N 128     /* largest N px_triangle_multiplication_static accepts  */

#define PX_F32 0
#define PX_BF16 1
#define PX_F16 2

typedef uint16_t px_bf16; /* storage of one bfloat16 */
typedef uint16_t px_f16;  /* storage of one IEEE half */
typedef uint16_t px_w16;  /* a weight element: bfloat16 when z_dtype is PX_BF16, half when it is PX_F32 */

/* The contraction stores x = PX_TRIMUL_X_SCALE * sum_k a b, so that sums over thousands of k stay inside the fp16
 * range; the output stage normalises x with eps * PX_TRIMUL_X_SCALE^2, which is LayerNorm of the unscaled x. */
#define PX_TRIMUL_X_SCALE 0.015625f

#if defined(__GNUC__)
#define PX_API __attribute__((visibility("default")))
#else
#define PX_API
#endif

/* Library version (major*10000 + minor*100 + patch). */
PX_API int32_t px_version(void);
/* Static, human-readable text for a status code. */
PX_API const char* px_status_string(int32_t status);
/* Leading dimension used for intermediates: N rounded up to a multiple of 8. */
PX_API int64_t px_ld(int64_t n);
/* Row stride of the attention bias tensors: N rounded up to a multiple of 128 (one key tile). */
PX_API int64_t px_ld_mask(int64_t n);

/* ---- LayerNorm op ---------------------------------------------------------------------
 * y = (x - mean) * rsqrt(var + eps) * gamma + beta over the last axis of x[rows][cols];
 * gamma and/or beta may be NULL (the four affine variants).  x, y, gamma, beta share `dtype`
 * (PX_F32, PX_BF16, PX_F16); mean and invvar are fp32 [rows] (may be NULL when not wanted).
 * Replaces the pybind functions forward_{none,with_bias,with_weight,with_both}_affine of
 * protenix/model/layer_norm/kernel/layer_norm_cuda.cpp:142-160 (wrapper :73-90, kernel
 * layer_norm_cuda_kernel.cu:145-388).  Unlike the reference it launches on `stream`. */
PX_API int32_t px_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* invvar,
                          int64_t rows, int64_t cols, float eps, int32_t dtype, void* stream);
/* Backward of the same op: dx (type of x), and, when wanted (non-NULL), dgamma and dbeta (type of x, [cols]).
 * mean and invvar are the fp32 statistics the forward returned; gamma NULL = no scale.  scratch: 2 * cols floats of
 * device memory when dgamma or dbeta is wanted (zeroed here).  cols <= 16384.
 * Replaces backward_{none,with_bias,with_weight,with_both}_affine of
 * protenix/model/layer_norm/kernel/layer_norm_cuda.cpp:162-179 (kernels layer_norm_cuda_kernel.cu:412-977). */
PX_API int32_t px_layer_norm_bwd(const void* dy, const void* x, const float* mean, const float* invvar, const void* gamma,
                          void* dx, void* dgamma, void* dbeta, float* scratch, int64_t rows, int64_t cols,
                          int32_t dtype, void* stream);

/* ---- Standardised copy of fp32 rows --------------------------------------------------------
 * zn[row] = fp16((z[row] - mean) * rsqrt(var + eps)) over `rows` rows of 128 channels: LayerNorm without scale and
 * offset (the consumers fold those into their weights).  One copy serves every stage that normalises the same z with
 * the same eps.  HBM-bound, 768 bytes per row.  No counterpart in the reference (its LayerNorm kernel writes the
 * normalised tensor in the input's type, protenix/model/layer_norm/kernel/layer_norm_cuda_kernel.cu:145-388). */
PX_API int32_t px_standardise_rows(const float* z, px_f16* zn, int64_t rows, float eps, void* stream);
/* z[row] += upd[row] over `rows` rows of 128 channels, z fp32, upd fp16: adds an update that was computed elsewhere
 * (px_triatt_out with z_dtype PX_F16) to the residual stream.  No counterpart in the reference. */
PX_API int32_t px_add_update_rows(float* z, const px_f16* upd, int64_t rows, void* stream);

/* ---- Triangle multiplication (outgoing / incoming) ---------------------------------------
 * Stage 1: zn = LN(z); a = mask * sigmoid(W_ag zn) * (W_ap zn); b likewise.  a and b are
 * written channel-major, contraction index contiguous: a[c][i][k] (row stride ld), zero in
 * the pad columns k >= N.  For `incoming` the two token indices are exchanged on the way out
 * (a[c][i][k] holds the reference's a[k][i][c]) so that stage 2 is the same product for both.
 * Replaces protenix/model/triangular/triangular.py:535-543. */
PX_API int32_t px_trimul_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w, const float* ln_b,
                          const px_w16* w_ap, const px_w16* w_ag, const px_w16* w_bp, const px_w16* w_bg,
                          px_f16* a, px_f16* b, int64_t n_u, int64_t n_t, int64_t ld, int32_t incoming, float eps,
                          void* stream);
/* Stage 2: x[c][i][j] = PX_TRIMUL_X_SCALE * sum_k a[c][i][k] * b[c][j][k] for the 128 channels (fp16 in, fp32
 * accumulate, fp16 out, row stride ld) on the tcgen05 tensor cores: persistent kernel, TMA-fed
 * 128x256x64 tiles, fp32 accumulators in tensor memory, double-buffered epilogue.  a, b, x must be
 * 16-byte aligned.  Replaces _combine_projections, protenix/model/triangular/triangular.py:123-150. */
PX_API int32_t px_trimul_contract(const px_f16* a, const px_f16* b, px_f16* x, int64_t channels, int64_t n, int64_t ld,
                           void* stream);
/* Device-side waits are bounded: a kernel whose wait runs out records a flag, stops issuing work, frees what it
 * holds and returns; kernels launched while a flag is set return without working.  The call synchronises the
 * device, then returns and clears the record: bit f of *flags (PX_FAMILY_*) is set when a wait of kernel family f
 * gave up -- the outputs written since the last call are then not valid.  px_device_error_detail also fills
 * detail[PX_N_FAMILIES] with the wait codes of each family (which pipeline role gave up).  No counterpart in the
 * reference (torch reports asynchronous failures through the CUDA error state). */
#define PX_FAMILY_CONTRACT 0
#define PX_FAMILY_FLASH 1
#define PX_FAMILY_TRANSITION 2
#define PX_FAMILY_TRIMUL_IN 3
#define PX_FAMILY_TRIMUL_OUT 4
#define PX_FAMILY_TRIATT_IN 5
#define PX_FAMILY_TRIATT_OUT 6
#define PX_FAMILY_PAIR_BIAS 7
#define PX_FAMILY_RECYCLE 8
#define PX_FAMILY_SELFTEST 9
#define PX_FAMILY_PEER 10 /* px_peer_barrier: a rank did not arrive; detail bit r names the rank (mod 16) */
#define PX_FAMILY_OPM 11
#define PX_N_FAMILIES 12
PX_API int32_t px_device_error_flags(uint32_t* flags);
PX_API int32_t px_device_error_detail(uint32_t* flags, uint32_t* detail);
/* Limit of every bounded wait on the current device, in SM clock cycles (default 2^28, about 0.14 s); cycles <= 0
 * restores the default.  No counterpart in the reference. */
PX_API int32_t px_set_wait_limit_cycles(int64_t cycles);
/* Launches a one-CTA kernel whose wait can never complete (an mbarrier nobody arrives on).  It gives up after the
 * wait limit, sets bit PX_FAMILY_SELFTEST and writes 1 to *out_word (device memory); launched while that flag is
 * still set it writes 2 and returns at once.  Exercises the give-up path without faulting the GPU.  No counterpart in
 * the reference. */
PX_API int32_t px_selftest_wait_timeout(uint32_t* out_word, void* stream);
/* Stage 3: z_out = [z_in +] W_z LN_out(x) * sigmoid(W_g LN_in(z_in)).  z_out may alias z_in.  zn: the standardised
 * copy of z_in when z_dtype is PX_F32 (NULL otherwise).
 * Replaces protenix/model/triangular/triangular.py:559-565. */
PX_API int32_t px_trimul_out(const px_f16* x, const void* z_in, const px_f16* zn, void* z_out, int32_t z_dtype, const float* ln_in_w,
                      const float* ln_in_b, const float* ln_out_w, const float* ln_out_b, const px_f16* w_z,
                      const px_w16* w_g, int64_t n_i, int64_t n_j, int64_t ld, int32_t add_residual, float eps,
                      void* stream);
/* Bytes of workspace px_triangle_multiplication needs for N tokens (a, b and x). */
PX_API int64_t px_trimul_workspace_bytes(int64_t n);
/* The three stages in sequence.  Stands in for TriangleMultiplicativeUpdate.forward,
 * protenix/model/triangular/triangular.py:470-570 (and for the cuEquivariance call
 * :28-90 the reference can dispatch to). */
PX_API int32_t px_triangle_multiplication(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                   const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                   const float* ln_out_b, const px_w16* w_ap, const px_w16* w_ag,
                                   const px_w16* w_bp, const px_w16* w_bg, const px_f16* w_z, const px_w16* w_g,
                                   void* workspace, int64_t workspace_bytes, int64_t n, int32_t incoming,
                                   int32_t add_residual, float eps, void* stream);

/* Triangle multiplication without any workspace argument, for callers that must not or cannot
 * allocate device memory: a plug-in running inside a host application that has handed all device
 * memory to its own pool (cudaMalloc then fails), or a latency-critical thread that must avoid
 * cudaMalloc/cudaFree because they synchronise the device.  The scratch for a, b, x and the
 * standardised copy of an fp32 z is a 16 MiB array inside the library image (held by every GPU that loads the library until the
 * process exits), so N is limited to PX_STATIC_MAX_N = 128; a larger N returns PX_ERR_TOO_LARGE.
 * The call itself allocates nothing.  Its first call on a device looks up the array's device
 * address (cudaGetSymbolAddress, with that device current); make that first call before any stream
 * capture.  All calls on one device share the one array: calls that overlap on the GPU (different
 * streams, or different host threads without ordering) race on it and must be serialised by the
 * caller.  Nothing needs clearing between calls: each call writes every scratch element it reads.
 * Results are those of px_triangle_multiplication on the same inputs.
 * This entry point has no counterpart in the reference. */
PX_API int32_t px_triangle_multiplication_static(const void* z_in, void* z_out, int32_t z_dtype, const float* mask,
                                          const float* ln_in_w, const float* ln_in_b, const float* ln_out_w,
                                          const float* ln_out_b, const px_w16* w_ap, const px_w16* w_ag,
                                          const px_w16* w_bp, const px_w16* w_bg, const px_f16* w_z,
                                          const px_w16* w_g, int64_t n, int32_t incoming, int32_t add_residual,
                                          float eps, void* stream);
/* PX_STATIC_MAX_N as seen by the loaded library. */
PX_API int64_t px_static_max_n(void);

/* ---- Triangle attention (starting / ending node), 4 heads x 32 -------------------------
 * Stage 1: xn = LN(z); q,k,v = W xn written per attended row u as [u][h][t][32] fp16 (v transposed: [u][h][32][ld(n_t)]) with q
 * pre-scaled by log2(e)/sqrt(32); bias[h][u][t] = log2(e) * (W_b xn)[u][t][h] (fp32, row
 * stride ldm = px_ld_mask(N), zero in the pad columns); mask_bias[u][t] = log2(e) * inf *
 * (mask - 1) (fp32, row stride ldm, -infinity in the pad columns).  For the
 * ending node the pair element read for (u,t) is z[t][u] and mask[t][u], which is what the
 * reference obtains by transposing z (protenix/model/modules/pairformer.py:160-168).
 * Replaces protenix/model/triangular/triangular.py:683-692 and layers.py:361-382. */
PX_API int32_t px_triatt_in_proj(const void* z, int32_t z_dtype, const float* mask, const float* ln_w, const float* ln_b,
                          const px_w16* w_q, const px_w16* w_k, const px_w16* w_v, const px_w16* w_bias,
                          px_f16* q, px_f16* k, px_f16* v, float* bias, float* mask_bias, int64_t n_u, int64_t n_t,
                          int64_t ldm, int32_t ending, float eps, float inf, void* stream);
/* Stage 2: o[u][t][h*32+d] = softmax_k(q.k + bias[h][t][k] + mask_bias[u][k]) v on the tcgen05
 * tensor cores: TMA-fed, logits and probabilities live in tensor memory only, online softmax in
 * base 2.  v is the transposed layout [u][h][32][ld(n)] written by stage 1; `scratch` needs
 * px_triatt_flash_scratch_bytes(n_u, n) bytes (per-tile mask flags).  All pointers 16-byte aligned.
 * Replaces the back-ends selected in protenix/model/triangular/layers.py:441-469 (_attention
 * :276-296, the Triton kernel protenix/model/tri_attention/forward.py:22-188, DS4Sci and
 * cuEquivariance calls). */
PX_API int32_t px_triatt_flash(const px_f16* q, const px_f16* k, const px_f16* v, const float* bias,
                        const float* mask_bias, px_f16* o, void* scratch, int64_t n_u, int64_t n, int64_t ldm,
                        void* stream);
PX_API int64_t px_triatt_flash_scratch_bytes(int64_t n_u, int64_t n);
/* Stage 3: z_out(u,t) = [z_in(u,t) +] W_o (o[u][t] * sigmoid(W_g LN(z_in(u,t)))), where (u,t)
 * addresses z[u][t] (starting) or z[t][u] (ending).  z_out may alias z_in.  zn: the standardised copy of z_in
 * (same layout) when z_dtype is PX_F32 (NULL otherwise).  z_dtype PX_F16: z_in is itself the standardised fp16 copy
 * and z_out receives the update alone, in fp16 (add_residual must be 0): for callers that add the update elsewhere.
 * Replaces Attention._wrap_up, protenix/model/triangular/layers.py:384-398. */
PX_API int32_t px_triatt_out(const px_f16* o, const void* z_in, const px_f16* zn, void* z_out, int32_t z_dtype, const float* ln_w,
                      const float* ln_b, const px_w16* w_g, const px_f16* w_o, int64_t n_u, int64_t n_t, int32_t ending,
                      int32_t add_residual, float eps, void* stream);
PX_API int64_t px_triatt_workspace_bytes(int64_t n);
/* The three stages in sequence.  Stands in for TriangleAttention.forward,
 * protenix/model/triangular/triangular.py:657-715. */
PX_API int32_t px_triangle_attention(const void* z_in, void* z_out, int32_t z_dtype, const float* mask, const float* ln_w,
                              const float* ln_b, const px_w16* w_bias, const px_w16* w_q, const px_w16* w_k,
                              const px_w16* w_v, const px_w16* w_g, const px_f16* w_o, void* workspace,
                              int64_t workspace_bytes, int64_t n, int32_t ending, int32_t add_residual, float eps,
                              float inf, void* stream);

/* ---- Transition (SwiGLU), c = 128, expansion 4 -------------------------------------------
 * x_out = [x_in +] W_o( silu(W_a LN(x_in)) * (W_b LN(x_in)) ) over rows of 128 channels; the
 * [rows][512] intermediates stay on chip.  x_out may alias x_in.  The rows pass through registers for the LayerNorm
 * whatever their storage type, so both products take fp16 operands and the three weights are fp16 always.
 * Replaces Transition.forward, protenix/model/modules/primitives.py:190-230. */
PX_API int32_t px_transition(const void* x_in, void* x_out, int32_t dtype, const float* ln_w, const float* ln_b,
                      const px_f16* w_a, const px_f16* w_b, const px_f16* w_o, int64_t rows, int32_t add_residual,
                      float eps, void* stream);

/* ---- Pair bias for the single-representation attention ----------------------------------
 * out[h][row] = (W LN(z[row]))[h] for h < n_heads (<= 16), fp32; ln_b may be NULL.  z_dtype PX_BF16 (rows of z) or
 * PX_F16 (standardised copy of an fp32 z).
 * Replaces protenix/model/modules/transformer.py:185-188. */
PX_API int32_t px_pair_bias_proj(const void* z, int32_t z_dtype, const float* ln_w, const float* ln_b, const px_w16* w,
                          float* out, int64_t rows, int32_t n_heads, float eps, void* stream);

/* ---- Recycling update of the pair representation ------------------------------------------
 * out[row] = z_init[row] + W LN(z[row]) for `rows` rows of 128 channels (W [128][128] in the format of z,
 * z_init and out of one dtype, PX_BF16 or PX_F32; z the bf16 rows, or for PX_F32 their standardised fp16 copy);
 * ln_b may be NULL; out may be z or z_init.
 * Replaces protenix/model/protenix.py:246
 * (z = z_init + linear_no_bias_z_cycle(layernorm_z_cycle(z))). */
PX_API int32_t px_recycle_update(const void* z, const void* z_init, void* out, int32_t z_dtype, const float* ln_w,
                          const float* ln_b, const px_w16* w, int64_t rows, float eps, void* stream);

/* ---- Outer product mean of the MSA module (c_hidden = 32, c_z = 128) ------------------------
 * Stage 1: x[32 i + c][32 j + e] = PX_TRIMUL_X_SCALE * sum_s a_t[32 i + c][s] * b_t[32 j + e][s], fp16, where a_t and
 * b_t are the masked projections of the normalised MSA embedding laid out [rows = 32 N][ld_k] with the MSA row s
 * contiguous (ld_k a multiple of 8, pad columns zero): a_t has rows_a = 32 n_i rows (a block of n_i tokens i), b_t
 * rows_b = 32 N, and x is [rows_a][rows_b].  The tensor-core contraction of the triangle multiplication on one
 * "channel".
 * Stage 2: z_out[i][j][:] = [z_in[i][j][:] +] (W_out (x[i, j block] / PX_TRIMUL_X_SCALE) + bias) * inv_norm[i][j], with
 * W_out fp16 [128][1024] (input index 32 c + e, as the reference flattens), bias fp32 [128], inv_norm fp32 [N][N] =
 * 1 / (sum_s mask[s][i] mask[s][j] + eps); z PX_F32 or PX_BF16 [N][N][128]; z_out may alias z_in.  The call covers
 * n_i rows i: x, inv_norm, z_in and z_out point at the first of them (x is then the [32 n_i][32 N] block of stage 1).
 * Replace OuterProductMean._opm and the normalisation, protenix/model/triangular/layers.py:685-695 and :770-777
 * (the einsum, the reshape, linear_out, the division). */
PX_API int32_t px_opm_outer(const px_f16* a_t, const px_f16* b_t, px_f16* x, int64_t rows_a, int64_t rows_b, int64_t ld_k,
                     void* stream);
PX_API int32_t px_opm_out(const px_f16* x, const px_f16* w_out, const float* bias, const float* inv_norm, const void* z_in,
                   void* z_out, int32_t z_dtype, int64_t n_i, int64_t n, int32_t add_residual, void* stream);

/* ---- Row-shared dropout + residual add (training path) ---------------------------------------
 * out[b][r][k] = residual[b][r][k] + x[b][r][k] * mask[b][k] for tensors [batches][rows][cd] and a mask [batches][cd]
 * of zeros and 1 / (1 - p) in the same type (PX_F32, PX_BF16, PX_F16), one value per (b, k) shared by all rows;
 * residual NULL: the product alone (the gradient with respect to x).  The product is rounded to the storage type before
 * the add.  Replaces the Triton kernels behind dropout_add_rowwise, protenix/model/modules/fused_ops.py:40-187 (forward
 * and backward), whose mask comes from a counter-based generator inside the kernel; here the caller draws it. */
PX_API int32_t px_scale_add_rowwise(const void* residual, const void* x, const void* mask, void* out, int64_t batches,
                             int64_t rows, int64_t cd, int32_t dtype, void* stream);

/* ---- Exchange between the GPUs of one box (row-sharded path) ------------------------------
 * No counterpart in the reference (which runs the Pairformer on one GPU).  A peer buffer is a
 * cudaMalloc allocation whose 64-byte handle other processes on the same machine can open;
 * px_copy_2d copies `height` rows of `width_bytes` (pointers, pitches and width multiples of 16
 * bytes) with a hand-written kernel: 16-byte loads and stores, dst may be an opened peer buffer
 * (plain stores over NVLink; no TMA, no multicast).  Ordering across GPUs is the caller's job:
 * px_peer_barrier after the copies, before the receiver's kernels. */
#define PX_PEER_HANDLE_BYTES 64
PX_API int32_t px_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle);
PX_API int32_t px_peer_open(const unsigned char* handle, void** ptr);
PX_API int32_t px_peer_close(void* ptr);
PX_API int32_t px_peer_free(void* ptr);
PX_API int32_t px_copy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width_bytes,
                          int64_t height, void* stream);
/* The copy of px_copy_2d issued to the copy engines (cudaMemcpy2DAsync): uses no SM, overlaps any kernel; for wide
 * rows.  No alignment requirement. */
PX_API int32_t px_copy_2d_dma(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width_bytes,
                              int64_t height, void* stream);
/* Barrier between the `world` (<= PX_COPY_BATCH_MAX) ranks of a box, stream-ordered on every rank: completes on a
 * rank once every rank has reached its call with the same `epoch`, i.e. once everybody's earlier copies are in place.
 * flag_arrays[r] is rank r's flag array (at least `world` 32-bit words in a peer buffer, zero at the start) as mapped
 * into this process; `epoch` is 1 for the first barrier on these arrays and grows by one per barrier, on all ranks
 * alike.  One warp: system-scope release stores into the peers' arrays, bounded acquire polling of the own one.  A
 * rank that does not arrive within the wait limit sets PX_FAMILY_PEER in px_device_error_flags on the waiting ranks.
 * Every rank must run on its own GPU.  No counterpart in the reference. */
PX_API int32_t px_peer_barrier(void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch, void* stream);
/* The same copy geometry for `count` (<= PX_COPY_BATCH_MAX) source/destination pairs in one launch. */
#define PX_COPY_BATCH_MAX 16
PX_API int32_t px_copy_2d_batch(void* const* dst, const void* const* src, int32_t count, int64_t dpitch, int64_t spitch,
                                int64_t width_bytes, int64_t height, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PX_B200_H_ */
