/*
 * nslq_b200.h -- C ABI of the B200 (sm_100a) quantized-linear library.
 *
 * Drop-in boundary for NSL's quantized-linear path: BitLinear (ternary W1.58 x
 * int8 activations, exact int32 accumulation) and W4A16 (uint4 group-quantised
 * weights x 16-bit activations, fp32 accumulation).  Plain pointers and sizes
 * only; every data pointer is a CUDA device pointer unless a comment says host.
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *
 * Conventions follow NSL's extern "C" runtime (docs/abi/README.md:80-113 in the
 * NSL tree): handles are raw pointers, outputs are caller-allocated, nothing
 * unwinds across the boundary.  Core functions return a status (0 = ok, < 0 =
 * error, text from nslq_last_error()); the shims with NSL's own names keep
 * NSL's behaviour (print + abort on a bad dtype/shape, print + return 0 on null).
 *
 * There is no CPU fallback anywhere in this library: every entry point that
 * computes launches CUDA kernels and fails with NSLQ_ERR_CUDA if it cannot.
 */
#ifndef NSLQ_B200_H
#define NSLQ_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define NSLQ_OK                0
#define NSLQ_ERR_ARG          -1 /* null pointer, bad enum, misaligned pointer      */
#define NSLQ_ERR_SHAPE        -2 /* shape the path cannot represent (e.g. K % 4)    */
#define NSLQ_ERR_CUDA         -3 /* a CUDA runtime call or launch failed            */
#define NSLQ_ERR_UNSUPPORTED  -4 /* valid request with no kernel for it             */
#define NSLQ_ERR_WORKSPACE    -5 /* workspace missing or too small                  */
#define NSLQ_ERR_COMM         -6 /* NCCL missing or a collective failed             */
#define NSLQ_ERR_TIMEOUT      -7 /* a bounded wait on a collective reached its deadline */
#define NSLQ_ERR_IO           -8 /* a file cannot be read or is not the container it should be */

/* ---- dtype tags: NSL's NslTensor.dtype wire tags -------------------------
 * crates/nsl-runtime/src/tensor/mod.rs:246-256 */
#define NSLQ_DTYPE_F64   0
#define NSLQ_DTYPE_F32   1
#define NSLQ_DTYPE_FP16  2
#define NSLQ_DTYPE_BF16  3
#define NSLQ_DTYPE_INT8  4
#define NSLQ_DTYPE_I32   9

/* Library/ABI version (major*100 + minor) and the last error text of the
 * calling thread (never NULL; valid until that thread's next failing call). */
int         nslq_version(void);
const char *nslq_last_error(void);

/* Every wait inside the kernels (mbarrier phases of the tensor-core kernels, the
 * landing of a weight slab) is bounded; a kernel whose wait expires records a
 * nonzero code and ends normally instead of spinning.  nslq_decode_attention
 * records 0x901 when it found its position outside [0, max_ctx) and did nothing.
 * This reads those words of the current device into *status (0 = nothing
 * happened) and clears them.  The reads are ordinary device-to-host copies on
 * the legacy default stream: they wait for work issued before them on blocking
 * streams; work on non-blocking streams must be synchronised by the caller. */
int nslq_device_status(int *status);

/* Kernels are launched with the programmatic-dependent-launch attribute, so that
 * a kernel's weight prefetch overlaps the tail of the kernel before it in the
 * stream (each kernel waits for its predecessor before touching its inputs or
 * outputs).  enable = 0 turns the attribute off process-wide; default on. */
void nslq_set_dependent_launch(int enable);

/* ========================================================================== */
/* Stage 1: per-token absmax int8 activation quantisation                      */
/* ========================================================================== */
/*
 * Replaces absmax_scale_row + quantize_row_int8
 * (crates/nsl-codegen/tests/bitnet_reference_impl.rs:46-70) and the fused
 * absmax phase of the reference GPU kernel
 * (crates/nsl-codegen/src/bitnet/phases/absmean_quant.rs:62-177).
 *
 *   scale[r] = max_k |x[r,k]|            (NaN ignored; 0 for an all-zero row)
 *   q[r,k]   = round_half_away(clamp(x[r,k] * (127/scale[r]), -127, 127)) as i8
 *
 * x: [M,K] row-major, x_dtype in {F32, FP16, BF16}.  Outputs (each may be NULL
 * except scale):
 *   q_plain [M,K] int8   natural k order (what the reference returns)
 *   q_perm  [M,K] int8   the order the matmul kernels consume: inside every
 *                        aligned group of 16 k, position 4*i+j holds k = 4*j+i
 *                        (requires K % 16 == 0)
 *   scale   [M]   f32
 *   rowsum  [M]   int32  sum_k q[r,k]
 */
int nslq_act_quant_i8(const void *x, int x_dtype, int64_t M, int64_t K,
                      int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum,
                      void *stream);

/*
 * RMSNorm fused in front of the quantisation: the `fused_rmsnorm` prologue that NSL's BitNet
 * kernel config names but never emits (crates/nsl-codegen/src/bitnet/config.rs:23-31).
 *
 *   rms[r] = sqrt(sum_k x[r,k]^2 / K + eps)           f64, like nsl_tensor_rmsnorm
 *   h[r,k] = (f32)(x[r,k] / rms[r] * weight[k])       (crates/nsl-runtime/src/tensor/mod.rs:3016-3035)
 *   then scale/q/rowsum of h exactly as nslq_act_quant_i8.
 *
 * weight: f32 [K].  h_out (f32 [M,K]) may be NULL: the normalised row then never reaches memory.
 * K must be a multiple of 16 and at most 12288; all buffers 16-byte aligned.  The sum of squares
 * is a tree reduction (the reference adds sequentially), so h can differ from the reference in
 * the last bit of a few elements; everything after h is exact.
 */
int nslq_rmsnorm_act_quant_i8(const void *x, int x_dtype, const float *weight, double eps,
                              int64_t M, int64_t K, float *h_out,
                              int8_t *q_plain, int8_t *q_perm, float *scale, int32_t *rowsum,
                              void *stream);

/*
 * SiLU(gate) * up fused in front of the quantisation of the down projection's input (SwiGLU FFN of
 * the BitNet decoder; gate, up and down live in stdlib-level model code of NSL, so this is a fused
 * neighbour of the linear like the RMSNorm prologue, not a replacement of a runtime function):
 *   h[r,k] = (f32)( gate[r,k] / (1 + exp(-gate[r,k])) * up[r,k] )       fp32 arithmetic
 *   then scale/q/rowsum of h exactly as nslq_act_quant_i8.
 * gate, up: [M,K] of the same dtype in {F32, FP16, BF16} with row strides gate_ld, up_ld in elements
 * (K when packed; larger when they are column slices of one fused gate|up projection output; rows
 * must stay 16-byte aligned); h_out (f32 [M,K]) may be NULL.
 * K % 16 == 0, K <= 12288, buffers 16-byte aligned.
 */
int nslq_swiglu_act_quant_i8(const void *gate, const void *up, int dtype, int64_t M, int64_t K,
                             int64_t gate_ld, int64_t up_ld, float *h_out, int8_t *q_plain, int8_t *q_perm, float *scale,
                             int32_t *rowsum, void *stream);

/*
 * Decoder step between the q/k/v projections and the output projection, one launch: rotate-half
 * RoPE of q and k at position *pos (stdlib/nsl/nn/rope.nsl:10-17: frequency table
 * concat(freqs, freqs)), append of k and v to the KV cache, and causal single-query attention
 * over keys 0..*pos with grouped heads (stdlib/nsl/nn/gqa.nsl:66-95).  No runtime entry point of
 * NSL does this in one call; it stands in for rope.forward + scaled_dot_product_attention on the
 * newest token.
 *
 *   q      bf16 [B,H,D]      k_new, v_new  bf16 [B,Hkv,D]      (projection outputs, before RoPE);
 *          *_batch_stride = elements between consecutive sequences (H*D resp. Hkv*D when packed;
 *          larger when q, k, v are column slices of one fused projection output), multiples of 4
 *   k_cache, v_cache  bf16 [B,Hkv,max_ctx,D]   row *pos is written, rows 0..*pos are read
 *   cos_table, sin_table  f32 [max_ctx, D/2]
 *   pos    device pointer to the int64 position (read by the kernel, so a CUDA graph can advance it)
 *   out    bf16 [B,H,D]
 * D % 4 == 0, D <= 128, H % Hkv == 0, max_ctx % 4 == 0.  fp32 arithmetic.  A position outside
 * [0, max_ctx) makes the kernel do nothing (out and the caches keep their bytes) and record
 * 0x901 in the status word nslq_device_status reads: a replayed decode loop must be stopped by
 * its host before the cache is full.
 */
int nslq_decode_attention(const void *q, const void *k_new, const void *v_new,
                          int64_t q_batch_stride, int64_t k_batch_stride, int64_t v_batch_stride,
                          void *k_cache, void *v_cache,
                          const float *cos_table, const float *sin_table, const int64_t *pos,
                          int64_t B, int64_t H, int64_t Hkv, int64_t D, int64_t max_ctx,
                          float sm_scale, void *out, void *stream);

/*
 * The rotary embedding of a prompt and its cache writes in one launch (RotaryEmbedding.forward,
 * stdlib/nsl/nn/rope.nsl:41-68: x * cos + rotate_half(x) * sin with cos/sin = concat(freqs, freqs)): q [B*T, H*D]
 * is rotated in place, k [B*T, Hkv*D] is rotated into k_cache[b, h, pos0 + t, :] and v copied into v_cache
 * ([B, Hkv, max_ctx, D]); token row r belongs to sequence r / T at position pos0 + r % T.  All BF16; cos_t, sin_t
 * [max_ctx, D/2] F32; q_ld, k_ld, v_ld: elements between token rows (so q, k, v may be column blocks of one fused
 * projection).  Each product and each sum is rounded separately in fp32 and the result once to bf16 -- the bits of the
 * same expression evaluated operation by operation on fp32 tensors.  nslq_decode_attention continues from pos0 + T.
 */
int nslq_rope_kv_prefill(void *q, const void *k, const void *v, int64_t q_ld, int64_t k_ld, int64_t v_ld,
                         void *k_cache, void *v_cache, const float *cos_t, const float *sin_t,
                         int64_t B, int64_t T, int64_t pos0, int64_t H, int64_t Hkv, int64_t D, int64_t max_ctx,
                         void *stream);

/*
 * The three remaining launches of a greedy decode step, each one runtime function of NSL as one launch on
 * device-resident data (one CTA per row; launch-latency work):
 *
 *  nslq_embed_gather   out[r,:] = (f32) table[tokens[r],:]   nsl_tensor_embedding_lookup
 *                      (crates/nsl-runtime/src/tensor/mod.rs:2592-2680).  table [V,H] F32/FP16/BF16, tokens int64 [B].
 *                      The reference bounds-checks host-resident ids and aborts; these ids live on the device,
 *                      so the kernel checks: an id outside [0,V) gives a row of zeros and status 0xA01
 *                      (nslq_device_status).
 *  nslq_rmsnorm_rows   y[r,k] = (f32)(x[r,k] / rms[r] * weight[k]), rms = sqrt(mean x^2 + eps) in f64
 *                      (nsl_tensor_rmsnorm, crates/nsl-runtime/src/tensor/mod.rs:3016-3035; the sum of squares
 *                      is a tree, as in nslq_rmsnorm_act_quant_i8), then rounded to y_dtype in {F32,FP16,BF16}.
 *  nslq_argmax_rows    out[r] = lowest index of the largest element of x[r,0:V] (row stride ld elements);
 *                      a NaN never wins, a row with nothing above -inf gives 0: the loop of nsl_tensor_argmax
 *                      (crates/nsl-runtime/src/sampling.rs:322-400).  int64 indices (the reference returns
 *                      them as f64).  `counter` (device int64, may be NULL) is incremented by one: the
 *                      position of a decode loop that lives on the device.
 */
int nslq_embed_gather(const void *table, int table_dtype, int64_t V, int64_t H, const int64_t *tokens, int64_t B,
                      float *out, void *stream);
int nslq_rmsnorm_rows(const float *x, const float *weight, double eps, int64_t M, int64_t K, void *y, int y_dtype,
                      void *stream);
int nslq_argmax_rows(const void *x, int x_dtype, int64_t M, int64_t V, int64_t ld, int64_t *out, int64_t *counter,
                     void *stream);

/* ========================================================================== */
/* BitLinear (ternary W1.58 A8)                                                */
/* ========================================================================== */
typedef struct nslq_bitlinear nslq_bitlinear_t;

/*
 * Wraps a packed ternary weight in NSL's own layout, zero-copy: row-major
 * [N = out_dim][K/4] bytes, four consecutive-k trits per byte, HIGH-BITS-FIRST,
 * code = trit + 1 (crates/nsl-codegen/src/bitnet/pack.rs:38-43; weight layout
 * crates/nsl-codegen/src/bitnet/mod.rs:97-103).  `weight_scale` is the
 * per-tensor absmean scale the loader produces
 * (crates/nsl-codegen/src/bitnet/loader.rs:47-56).  The buffer is borrowed and
 * must outlive the handle.  K % 4 == 0 (NSL's own constraint,
 * crates/nsl-codegen/src/bitnet/mod.rs:134-139).
 */
int  nslq_bitlinear_create(const uint8_t *packed, int64_t N, int64_t K, float weight_scale,
                           nslq_bitlinear_t **out);
void nslq_bitlinear_destroy(nslq_bitlinear_t *w);

/*
 * NSL's packed representation rejects the reserved code 0b11 (try_unpack_byte,
 * crates/nsl-codegen/src/bitnet/pack.rs:60-67; KAT bytes 0xFF and 0xC0).  The kernels do not look:
 * they would multiply such a field as +2.  This pass counts the bytes of the weight that hold it
 * (one reduction kernel, then a synchronisation of `stream`), stores the count in *invalid_bytes
 * (may be NULL) and returns NSLQ_ERR_ARG when it is not zero.  Call it once after
 * nslq_bitlinear_create for weights of unknown origin.
 */
int nslq_bitlinear_validate(const nslq_bitlinear_t *w, int64_t *invalid_bytes, void *stream);

/* Bytes of device scratch nslq_bitlinear_forward needs for M tokens of width K
 * (quantised activations, scales, row sums). */
int64_t nslq_bitlinear_workspace_bytes(int64_t M, int64_t K);

/*
 * y[M,N] = BitLinear(x[M,K]).  Replaces the fused reference kernel
 * nsl_bitnet_b158_gemm_* (crates/nsl-codegen/src/bitnet/mod.rs:133-307) and its
 * CPU statement forward_reference
 * (crates/nsl-codegen/tests/bitnet_reference_impl.rs:101-141):
 *
 *   acc[r,c] = sum_k q[r,k] * W[c,k]                      exact int32
 *   y[r,c]   = ((scale[r] / 127) * (float)acc) * weight_scale
 *              [+ bias[c]] [+ residual[r,c]]               each step rounded to f32
 *
 * (finalize order: crates/nsl-codegen/src/bitnet/phases/finalize.rs:39-80).
 * x_dtype, y_dtype in {F32, FP16, BF16}.  acc_out (int32 [M,N]), bias (f32 [N])
 * and residual (f32 [M,N]) may be NULL.  workspace: device memory of at least
 * nslq_bitlinear_workspace_bytes(M,K), 256-byte aligned, private to this call
 * until the stream reaches the end of it.
 */
int nslq_bitlinear_forward(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M,
                           void *y, int y_dtype, int32_t *acc_out,
                           const float *bias, const float *residual,
                           void *workspace, int64_t workspace_bytes, void *stream);

/*
 * Same product on activations already quantised by nslq_act_quant_i8 (q_perm,
 * scale, rowsum), so several projections of one input share one quantisation.
 */
int nslq_bitlinear_forward_quantized(const nslq_bitlinear_t *w, const int8_t *q_perm,
                                     const float *scale, const int32_t *rowsum, int64_t M,
                                     void *y, int y_dtype, int32_t *acc_out,
                                     const float *bias, const float *residual, void *stream);

/*
 * nslq_bitlinear_forward with the launch in front of it folded in: the input rows are
 *   RMSNorm(x) with `norm_weight`, `eps`      (= nslq_rmsnorm_act_quant_i8, then forward_quantized), or
 *   SiLU(gate) * up                           (= nslq_swiglu_act_quant_i8,  then forward_quantized),
 * with the same bits as those two calls.  For one token (a decode step) every CTA of the one launch
 * forms and quantises the rows for itself -- NSL's BitNet kernel config names this prologue (`fused_rmsnorm`,
 * crates/nsl-codegen/src/bitnet/config.rs:23-31) and never emits it; from two tokens on (measured: the CTAs' repeated work then costs more than a launch), or when a row
 * does not fit the CTA's shared memory next to the weights, the call issues the two launches itself and
 * needs the workspace of nslq_bitlinear_forward (pass it always).  K % 64 == 0; gate, up: [M,K], packed.
 */
int nslq_bitlinear_forward_rmsnorm(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M,
                                   const float *norm_weight, double eps, void *y, int y_dtype, int32_t *acc_out,
                                   const float *bias, const float *residual,
                                   void *workspace, int64_t workspace_bytes, void *stream);
int nslq_bitlinear_forward_swiglu(const nslq_bitlinear_t *w, const void *gate, const void *up, int dtype, int64_t M,
                                  void *y, int y_dtype, int32_t *acc_out,
                                  const float *bias, const float *residual,
                                  void *workspace, int64_t workspace_bytes, void *stream);

/*
 * Sibling projections of the same rows -- q, k and v of an attention block, gate and up of an MLP: the
 * reference's `BitLinear.forward` is called once per projection on the same normalised input
 * (stdlib/nsl/quant/bitlinear.nsl:74-88) -- as one call.  ys[i] [M, layers[i]->N] gets exactly the bits of
 * nslq_bitlinear_forward_rmsnorm(layers[i], x, ..., ys[i], ...) (norm_weight != NULL) or of
 * nslq_bitlinear_forward(layers[i], x, ..., ys[i], ...) (norm_weight == NULL) without bias or residual.  For one
 * token all layers share ONE launch (each CTA quantises the rows for itself and multiplies a slab of one
 * layer's weights); above that the rows are normalised and quantised once (which needs the workspace of
 * nslq_bitlinear_forward: pass it always) and the layers share one launch of the streaming kernel where that kernel
 * would take each of them (up to 16 rows of small matrices), else each layer is one launch.  1 <= n_layers <= 4; all layers the same K, K % 64 == 0.
 */
int nslq_bitlinear_forward_multi(const nslq_bitlinear_t *const *layers, int n_layers, const void *x, int x_dtype, int64_t M,
                                 const float *norm_weight, double eps, void *const *ys, int y_dtype,
                                 void *workspace, int64_t workspace_bytes, void *stream);

/*
 * nslq_bitlinear_forward without a caller workspace.  (No counterpart in NSL: the
 * reference has no GPU entry point for this path at all.)
 *
 * For hosts that cannot give the library device memory of their own accord: NSL's
 * runtime routes every device allocation through its caching allocator and frees
 * on its own schedule, so a plug-in has no buffer it may hold on to; a decode loop
 * that must not stall cannot call cudaMalloc, which synchronises the whole device;
 * a library loaded after the device was fully reserved has nothing left to ask
 * for.  The scratch (quantised activations, scales, row sums) lives instead in a
 * fixed area of nslq_noalloc_scratch_bytes() = 512 KiB inside the library's device
 * image -- every GPU that loads the library carries it until the process ends --
 * and the call itself requests no memory, on the host or the device (no cudaMalloc,
 * cudaFree or allocating library routine).
 *
 *  - Sizes: nslq_bitlinear_workspace_bytes(M, K) must fit the area (e.g. 16 tokens
 *    of width 16384, or 128 of width 3200); larger requests return
 *    NSLQ_ERR_WORKSPACE and say so.  No bias / residual / accumulator outputs.
 *  - The first call on each device looks up the area's device address (with that
 *    device current).  With CUDA's lazy module loading that look-up can be the moment
 *    the driver places the library's image -- its 512 KiB included -- on the device,
 *    so it is the one call that may take device memory and time.  Make that first
 *    call during set-up, before any stream capture begins.
 *  - All calls on a device share the one area, and it keeps the previous call's
 *    bytes.  Nothing needs clearing (each call overwrites what it reads), but two
 *    calls whose kernels can overlap on the GPU -- different streams, or different
 *    host threads on different streams -- race on it: keep them on one stream or
 *    order them yourself.
 *  - Results are identical to nslq_bitlinear_forward on the same inputs.
 */
int     nslq_bitlinear_forward_noalloc(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M,
                                       void *y, int y_dtype, void *stream);
int64_t nslq_noalloc_scratch_bytes(void);

/* ========================================================================== */
/* W4A16 (uint4 group-quantised weights, 16-bit activations)                   */
/* ========================================================================== */
typedef struct nslq_w4a16 nslq_w4a16_t;

/*
 * Weight stored as an NSL QuantizedTensor of shape [N,K], INT4, per-group along
 * axis 1 stores it (crates/nsl-runtime/src/quantize.rs:27-51, :366-417): codes
 * two per byte over the flat index n*K+k, low nibble = even k; one scale and one
 * zero point per (n, k/group); dequantisation (q - zp) * scale
 * (quantize.rs:263-266).  codes are borrowed; scales/zero points are converted
 * once into the library's own small f32 tables.
 *   scale_dtype: F32, BF16, FP16 or F64;  zp_packed: 0 = one u8 per group,
 *   1 = two uint4 per byte (low nibble = even group index over the flat n*G+g).
 */
int nslq_w4a16_create_nk(const uint8_t *codes, const void *scales, int scale_dtype,
                         const uint8_t *zero_points, int zp_packed,
                         int64_t N, int64_t K, int64_t group_size, nslq_w4a16_t **out);

/*
 * Weight in NSL's AwqPackedWeight form (crates/nsl-runtime/src/awq.rs:29-45):
 * logical [K,N], nibble index row*N+col, f64 scales and f64 float zeros indexed
 * [g*N+col], dequantisation q*scale+zero (awq.rs:74-76).  Re-laid out once on the
 * GPU into the [N,K] streaming order; nothing is borrowed.
 */
int nslq_w4a16_create_awq_kn(const uint8_t *data, const double *scales, const double *zeros,
                             int64_t K, int64_t N, int64_t group_size, nslq_w4a16_t **out);
/*
 * Weight stored as an NSL QuantizedTensor of shape [K,N] -- the orientation nsl_qtensor_matmul_mixed
 * requires (crates/nsl-runtime/src/quantize.rs:547-573) -- INT4, device pointers: nibble index k*N+n
 * (low nibble = even index), scales f32 and zero points u8 indexed as the reference indexes them
 * (quantize.rs:366-417).  Accepted: per tensor; per channel along axis 1 (one scale per column n);
 * per group along axis 0 (one scale per run of `group_size` rows k, shared by every column -- what
 * `per_group` means for a [K,N] tensor in the reference).  Re-laid out once on the GPU into the
 * [N,K] streaming order; nothing is borrowed.  Other granularities: NSLQ_ERR_UNSUPPORTED.
 */
int nslq_w4a16_create_qtensor_kn(const uint8_t *data, const float *scale, const uint8_t *zero_point,
                                 int64_t K, int64_t N, int granularity, int gran_axis, int64_t group_size,
                                 nslq_w4a16_t **out);
void nslq_w4a16_destroy(nslq_w4a16_t *w);

/*
 * y[M,N] = x[M,K] @ dequant(W)^T with fp32 accumulation.  Replaces
 * awq_matmul_cpu (crates/nsl-runtime/src/awq.rs:202-226) and the
 * dequantise-then-matmul of nsl_qtensor_matmul_mixed
 * (crates/nsl-runtime/src/quantize.rs:547-585).  x_dtype in {BF16, FP16, F32},
 * y_dtype in {BF16, FP16, F32}.
 */
int nslq_w4a16_forward(const nslq_w4a16_t *w, const void *x, int x_dtype, int64_t M,
                       void *y, int y_dtype, void *stream);

/*
 * The same product for fp32 activations (NSL's default dtype for GPU tensors,
 * crates/nsl-runtime/src/cuda/mod.rs:395-551) on the 16-bit kernels, without rounding x: each
 * element is split into three bf16 parts whose sum is x exactly, the kernels run on the 3M
 * stacked rows (the weights are still streamed once) and the three parts of the result are
 * added in fp32.  scratch: device memory of
 * nslq_w4a16_f32x_scratch_bytes(w, M), 256-byte aligned.
 */
int64_t nslq_w4a16_f32x_scratch_bytes(const nslq_w4a16_t *w, int64_t M);
int nslq_w4a16_forward_f32x(const nslq_w4a16_t *w, const float *x, int64_t M, void *y, int y_dtype,
                            void *scratch, int64_t scratch_bytes, void *stream);

/* ========================================================================== */
/* Pack-at-load: the reference's weight quantisers, on the GPU                 */
/* ========================================================================== */
/*
 * quantize_float_to_ternary (crates/nsl-codegen/src/bitnet/loader.rs:126-193):
 * scale = (sum |w|, added sequentially in f32) / numel; trit = round_half_away(
 * clamp(w / (scale > 0 ? scale : 1), -1, 1)); four trits per byte, HIGH-BITS-FIRST.
 * The sum keeps the reference's order (one thread adds), so `packed` and `*scale`
 * are the reference's bytes.  w: numel elements (F32 / FP16 / BF16), numel % 4 == 0
 * (the reference's AlignmentError otherwise); packed: numel/4 bytes; scale: one
 * float in device memory (it is the weight_scale of nslq_bitlinear_create).
 */
int nslq_ternary_quantize_pack(const void *w, int w_dtype, int64_t numel, uint8_t *packed, float *scale,
                               void *stream);

/*
 * load_bitnet_b158_safetensors (crates/nsl-codegen/src/bitnet/loader.rs:200-220): every tensor of the
 * safetensors file at `path` whose name ends in one of the seven BitLinear projection suffixes
 * (.self_attn.{q,k,v,o}_proj.weight, .mlp.{gate,up,down}_proj.weight; loader.rs:100-111), stored as F32,
 * F16 or BF16, is copied to the current device and quantised there by nslq_ternary_quantize_pack.  An
 * entry of the set is the reference's LoadedTernaryWeight (loader.rs:47-56): name, packed bytes (in DEVICE
 * memory, owned by the set: pass them to nslq_bitlinear_create with N = shape[0], K = shape[1]), the
 * shape from the header, and the absmean scale (= weight_scale).  Entries come in the order of their
 * bytes in the file (the reference's order is that of a hash map).  Errors, as the reference's
 * LoaderError: NSLQ_ERR_IO (Io, Safetensors: unreadable file, malformed header, byte ranges that do not
 * match shape or file), NSLQ_ERR_SHAPE (AlignmentError: element count % 4), NSLQ_ERR_UNSUPPORTED
 * (UnsupportedDtype); nothing is returned then.  Other tensors (embeddings, norms, lm_head) are skipped,
 * as in the reference.  Synchronises `stream` once per tensor: a load-time call.
 */
typedef struct nslq_ternary_set nslq_ternary_set_t;
int nslq_bitnet_load_safetensors(const char *path, void *stream, nslq_ternary_set_t **out);
int64_t nslq_ternary_set_size(const nslq_ternary_set_t *set);
int nslq_ternary_set_entry(const nslq_ternary_set_t *set, int64_t i, const char **name, const uint8_t **packed,
                           int64_t *packed_bytes, const int64_t **shape, int *ndim, float *scale);
void nslq_ternary_set_destroy(nslq_ternary_set_t *set);

/*
 * nsl_qtensor_quantize for INT4, per-group along axis 1 of a [N,K] tensor
 * (crates/nsl-runtime/src/quantize.rs:224-266, :366-417): f64 arithmetic, scale =
 * (max-min)/15 (stored f32), zp = round(-min/scale) clamped, q = round(x/scale+zp)
 * clamped; the constant-group branch of compute_scale_zp included.  Outputs are what
 * nslq_w4a16_create_nk takes: codes [N*K/2] (low nibble = even k), scale f32 [N,G],
 * zero_point u8 [N,G].  w: F64 or F32; K and group_size even.
 */
int nslq_int4_quantize_nk(const void *w, int w_dtype, int64_t N, int64_t K, int64_t group_size,
                          uint8_t *codes, float *scale, uint8_t *zero_point, void *stream);

/*
 * nsl_qtensor_quantize and nsl_qtensor_dequantize in every form the reference has
 * (crates/nsl-runtime/src/quantize.rs:283-426, :436-537): dtype 0 = INT8 (codes 0..255), 1 = INT4 (two
 * codes per byte over the flat row-major index, low nibble = even index); granularity 0 = per tensor,
 * 1 = per channel along `axis`, 2 = per group of `group_size` along `axis`, for a tensor of up to 8
 * dimensions (`shape`: HOST array).  f64 arithmetic as in compute_scale_zp / quantize_val /
 * dequantize_val (quantize.rs:224-266); minimum and maximum by atomics (order-independent), so data,
 * scale (f32) and zero_point (u8) are the reference's bytes.  nslq_qtensor_num_scales = compute_num_scales
 * (quantize.rs:72-96) sizes scale and zero_point.  src: F64 or F32 device tensor; dequantise writes F64 (what
 * the reference returns) or F32.  quantize allocates a small scratch and synchronises `stream`: a load-time call.
 */
int64_t nslq_qtensor_num_scales(const int64_t *shape, int ndim, int granularity, int axis, int64_t group_size);
int nslq_qtensor_quantize(const void *src, int src_dtype, const int64_t *shape, int ndim, int dtype, int granularity,
                          int axis, int64_t group_size, uint8_t *data, float *scale, uint8_t *zero_point, void *stream);
int nslq_qtensor_dequantize(const uint8_t *data, const float *scale, const uint8_t *zero_point, const int64_t *shape, int ndim,
                            int dtype, int granularity, int axis, int64_t group_size, void *out, int out_dtype, void *stream);

/*
 * awq_quantize_cpu (crates/nsl-runtime/src/awq.rs:104-144): weight [K,N] (F64 or F32),
 * groups along K per column, scale = (max-min)/15 (1.0 if the range is < 1e-10),
 * zero = min, q = clamp(round((v-zero)/scale), 0, 15); nibble index row*N+col.  Outputs
 * are what nslq_w4a16_create_awq_kn takes: data [K*N/2], scales/zeros f64 [G*N].
 * K*N must be a multiple of 8.
 */
int nslq_awq_quantize_kn(const void *w, int w_dtype, int64_t K, int64_t N, int64_t group_size,
                         uint8_t *data, double *scales, double *zeros, void *stream);

/* ========================================================================== */
/* Column-parallel sharding                                                    */
/* ========================================================================== */
/*
 * Rank `rank` of `world` owns output rows [row0, row0+rows) of W[out,in] -- the
 * contiguous dim-0 split of NSL's shard math
 * (crates/nsl-runtime/src/tensor_parallel/sharding.rs:18-58).  N % world != 0 is
 * NSLQ_ERR_SHAPE, as in the reference.
 */
int nslq_shard_rows(int64_t N, int world, int rank, int64_t *row0, int64_t *rows);

/*
 * The communicator of a column-sharded run: one process per GPU on one node.  Follows NSL's
 * NCCL backend (crates/nsl-runtime/src/tensor_parallel/collective.rs:854-1130): rank 0 mints
 * a unique id (nslq_shard_unique_id, NSLQ_UNIQUE_ID_BYTES bytes of host memory), the host
 * hands it to every rank by its own means (NSL: a shared-memory broadcast), and every rank
 * calls nslq_shard_init with the device it will use current.  The join runs under a watchdog:
 * if the clique is not complete after NSL_NCCL_TIMEOUT_SECS (default 300) the process is
 * aborted with a message, as the reference does, because a peer that died before joining would
 * otherwise leave the others waiting for ever.  NCCL is loaded with dlopen at the first use (a
 * NCCL already in the process is reused), so the library itself loads without it; world == 1
 * needs no NCCL and no id.  At most NSLQ_MAX_RANKS ranks.
 */
#define NSLQ_MAX_RANKS        8
#define NSLQ_UNIQUE_ID_BYTES  128
typedef struct nslq_comm nslq_comm_t;
int  nslq_shard_unique_id(void *id_out);
int  nslq_shard_init(const void *unique_id, int rank, int world, nslq_comm_t **out);
void nslq_shard_destroy(nslq_comm_t *c);
int  nslq_shard_info(const nslq_comm_t *c, int *rank, int *world);

/*
 * The one exchange step of the column-parallel layout, by NCCL: all-gather of the [M, N_local]
 * output shards (ncclAllGather on `stream`; crates/nsl-runtime/src/tensor_parallel/
 * collective.rs:1061-1087).  `gathered` receives the shards rank after rank, [world][M][N_local]
 * -- for M == 1 that already is y[N].  When y_full is not NULL a second small kernel lays the
 * result out as [M][world*N_local] there (y_full must not alias gathered unless M == 1).
 * dtype: any NSLQ_DTYPE_* tag (bytes are moved, not interpreted).  The call only enqueues;
 * nslq_shard_wait is the bounded way to wait for it.
 */
int nslq_allgather_cols(nslq_comm_t *c, const void *y_local, int dtype, int64_t M, int64_t N_local,
                        void *gathered, void *y_full, void *stream);

/*
 * Waits until `stream` has drained, polling instead of blocking: an asynchronous NCCL error or
 * the deadline (timeout_ms; <= 0 = NSL_NCCL_TIMEOUT_SECS) ends the wait with NSLQ_ERR_COMM /
 * NSLQ_ERR_TIMEOUT after the communicator has been aborted (it is unusable afterwards; destroy
 * it).  The reference aborts the process at this point (collective.rs:975-1010); a library
 * leaves that decision to its host.  Not for use during stream capture.
 */
int nslq_shard_wait(nslq_comm_t *c, void *stream, int64_t timeout_ms);

/*
 * Peer memory.  nslq_symm_alloc is collective (every rank calls it, same size, same order): each
 * rank allocates `bytes` of device memory, the ranks exchange CUDA IPC handles over the
 * communicator and map one another's buffers; *local_ptr is this rank's own buffer, zero-filled.
 * The library's kernels reach the peers' copies with plain loads and stores only.  No counterpart
 * in NSL (its NCCL backend has no peer-memory path).
 */
int nslq_symm_alloc(nslq_comm_t *c, int64_t bytes, void **local_ptr);
int nslq_symm_free(nslq_comm_t *c, void *local_ptr);

/*
 * Flag barrier over peer memory, one small kernel on `stream`: every rank announces that the
 * work in front of the barrier on its stream is complete (its stores into peers' buffers
 * included) and waits until every other rank has announced the same.  The wait is bounded
 * (2 s): a rank that never arrives makes the kernel record 0x501 (nslq_shard_status) and
 * return; the context stays usable.  Graph-capturable (the epoch lives in device memory).
 */
int nslq_peer_barrier(nslq_comm_t *c, void *stream);
int nslq_shard_status(nslq_comm_t *c, int *status);

/*
 * All-gather by peer stores: this rank's [M, N_local] block goes to columns
 * [rank*N_local, (rank+1)*N_local) of the [M][world*N_local] result y_full in EVERY rank's copy.
 * y_full must lie inside a buffer of nslq_symm_alloc, at the same offset on every rank; rows of
 * the block must be multiples of 16 bytes.  Completion on the peers is what nslq_peer_barrier
 * announces.
 */
int nslq_peer_allgather_cols(nslq_comm_t *c, const void *y_local, int dtype, int64_t M, int64_t N_local,
                             void *y_full, void *stream);

/*
 * The same exchange by the copy engines: this rank's column block, already in place in its own
 * copy of y_full, is copied into every peer's copy with one strided cudaMemcpy2DAsync per peer
 * on `stream`.  No SM takes part, so the transfer runs under the kernels of other streams -- the
 * form to use when the block is produced by a kernel that fills every SM.
 */
int nslq_peer_push_cols_async(nslq_comm_t *c, void *y_full, int dtype, int64_t M, int64_t N_local, void *stream);

/*
 * BitLinear on this rank's row shard of W with the all-gather fused in: y_full is the whole
 * [M][world*N_shard] result, inside a buffer of nslq_symm_alloc.  For M > 16 the tensor-core
 * GEMM's epilogue stores each finished tile into this rank's copy and into every peer's copy
 * (the transfer overlaps the remaining tiles); for M <= 16 the decode kernel writes the local
 * block and one kernel pushes it.  x (and so its quantisation) is replicated on every rank,
 * hence the accumulators equal the unsharded ones bit for bit.  The caller brackets a group of
 * these calls with nslq_peer_barrier: one before the first store into a buffer the peers may
 * still be reading, one after the last call, before anyone reads y_full.
 * bias: this rank's N_shard entries or NULL.  Workspace as nslq_bitlinear_forward, sized by
 * nslq_bitlinear_gathered_workspace_bytes(M, K, N_shard).  Requires K % 64 == 0.
 * The _quantized form takes activations already quantised by nslq_act_quant_i8; its scratch
 * (M <= 16 only) is M*N_shard*4 bytes rounded up to 256.
 */
int64_t nslq_bitlinear_gathered_workspace_bytes(int64_t M, int64_t K, int64_t N_shard);
/*
 * The kernel capability the gathered calls are built on, usable without a communicator: the
 * [M, N] result is written as columns [col0, col0+N) of rows of `ldy` elements into n_copies
 * (1..8) arrays at once -- y_copies is a HOST array of device pointers to the [M][ldy] arrays.
 * E.g. q, k and v projections writing the column blocks of one fused [M, 3*hidden] buffer, or a
 * test standing in for two ranks on one GPU.  y_scratch as above (M <= 16 only); the form without
 * _quantized quantises x first and takes the workspace of the gathered call.
 */
int nslq_bitlinear_forward_cols(const nslq_bitlinear_t *w, const void *x, int x_dtype, int64_t M,
                                void *const *y_copies, int n_copies, int64_t ldy, int64_t col0, int y_dtype,
                                const float *bias, void *workspace, int64_t workspace_bytes, void *stream);
int nslq_bitlinear_forward_quantized_cols(const nslq_bitlinear_t *w, const int8_t *q_perm, const float *scale,
                                          const int32_t *rowsum, int64_t M, void *const *y_copies, int n_copies,
                                          int64_t ldy, int64_t col0, int y_dtype, const float *bias,
                                          void *y_scratch, int64_t y_scratch_bytes, void *stream);
int nslq_bitlinear_forward_gathered(nslq_comm_t *c, const nslq_bitlinear_t *w_shard, const void *x, int x_dtype,
                                    int64_t M, void *y_full, int y_dtype, const float *bias,
                                    void *workspace, int64_t workspace_bytes, void *stream);
int nslq_bitlinear_forward_quantized_gathered(nslq_comm_t *c, const nslq_bitlinear_t *w_shard, const int8_t *q_perm,
                                              const float *scale, const int32_t *rowsum, int64_t M,
                                              void *y_full, int y_dtype, const float *bias,
                                              void *y_scratch, int64_t y_scratch_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NSLQ_B200_H */
