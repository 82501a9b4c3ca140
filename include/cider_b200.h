/*
 * cider_b200 - C ABI of the B200 (sm_100a) implementation of cider's online
 * activation-quantized linear path.
 *
 * This is the boundary a binding of the reference would attach to.  The
 * reference exposes the path as four nanobind functions of the module
 * `_cider_prim` (csrc/src/prim_bindings.cpp:15-35) that build MLX primitives
 * (csrc/include/w8a8_primitive.h, pergroup_primitive.h, w4a8_primitive.h).
 * Here the same operations take raw DEVICE pointers, sizes and a CUDA stream;
 * no torch / MLX type appears in a signature.
 *
 * Conventions
 *  - All pointers are device pointers on the current CUDA device unless said
 *    otherwise.  fp16 is IEEE binary16 (`__half`), passed as void*.
 *  - `stream` is a cudaStream_t (0 = default stream).  Work is enqueued, never
 *    synchronised; no entry point allocates or frees device memory: scratch is
 *    passed in as `workspace` (size from cider_workspace_bytes()).
 *  - Every function returns CIDER_OK (0) or a negative CIDER_E_* code; a
 *    message for the last failure on the calling thread is available from
 *    cider_last_error().  Invalid arguments never launch a kernel.
 *  - Matrices are dense row-major.  A: [M,K], weights W: [N,K] ("transpose_b"
 *    layout of the reference), outputs [M,N].
 */
#ifndef CIDER_B200_H_
#define CIDER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CIDER_OK 0
#define CIDER_E_INVALID (-1)     /* null pointer, non-positive size, bad enum   */
#define CIDER_E_SHAPE (-2)       /* K % group_size, unsupported group size, ... */
#define CIDER_E_WORKSPACE (-3)   /* workspace missing or too small              */
#define CIDER_E_ALIGNMENT (-4)   /* pointer alignment the kernels rely on       */
#define CIDER_E_CUDA (-5)        /* a CUDA runtime / driver call failed         */
#define CIDER_E_UNSUPPORTED (-6) /* device is not compute capability 10.x       */
#define CIDER_E_DEVICE (-7)      /* a kernel recorded a bounded-wait time-out   */

/* dtype tag for weight scales */
#define CIDER_F32 0
#define CIDER_F16 1

/* op tags for cider_workspace_bytes() */
#define CIDER_OP_PERCHANNEL 1
#define CIDER_OP_PERGROUP 2
#define CIDER_OP_W4A8 3      /* cider_w4a8_linear      (reference packing [K/2, N]) */
#define CIDER_OP_W4A8_ROWS 4 /* cider_w4a8_linear_nk4  (packed rows [N, K/2])      */
#define CIDER_OP_W4A8_ROWS_INT8COPY 5 /* the same entry, lending N*K more bytes (see there) */

/* Library version (major*10000 + minor*100 + patch). */
int cider_version(void);

/* Message of the last failure on this thread ("" if none).  The reference
 * raises C++ exceptions instead (csrc/src/w8a8_primitive.mm:257-262,
 * csrc/src/pergroup_primitive.mm:282-295). */
const char *cider_last_error(void);

/* 1 if CUDA device `device` can run this library (compute capability 10.x),
 * 0 otherwise.  Counterpart of the reference's hardware gate is_available()
 * (cider/ops.py:52-68). */
int cider_device_supported(int device);

/* Bytes of scratch the given op needs for an [M,K] x [N,K] problem: the int8
 * copy of the activations and their per-row scales (the encoder temporaries of
 * csrc/src/w8a8_primitive.mm:184-188), plus for the per-channel linear at M <= 512
 * with few output tiles and a long K the int32 slabs of its split-K form (the per-group
 * linear: fp32 slabs, the same size for every group size), plus for
 * W4A8 on the reference packing the weights transposed into packed rows (N*K/2 bytes;
 * no int8 copy of the weights is ever made for K >= 128, K % 32 == 0 - the kernels
 * expand the nibbles in shared memory / registers; other K take an int8 copy or the
 * plain kernel).  A pure function of the shape.  0 when the op needs none (M == 1
 * per-channel / per-group). */
size_t cider_workspace_bytes(int op, int64_t M, int64_t N, int64_t K);

/* Per-token activation quantisation, fp16 [M,K] (row stride ldx elements) ->
 * int8 [M,K] (dense) + fp32 scale [M].
 *   s = max_k|x| / 127 (0 -> 1), q = int8(clamp(round_half_away(x * (1/s)), -128, 127))
 * Replaces kernel quantize_per_token, cider/kernels/w8a8_quantize.metal:17-87,
 * launched from csrc/src/w8a8_primitive.mm:190-202. */
int cider_quantize_per_token(const void *x_f16, int64_t M, int64_t K, int64_t ldx,
                             void *q_i8, float *scale, void *stream);

/* The quantiser in two halves, for a row whose absmax is not known from the local data
 * alone: a tensor-parallel rank in front of a row-parallel linear holds a K-slice of
 * the activation; the ranks exchange their slice maxima (a max all-reduce of [M] fp32)
 * and every rank then quantises with the scale of the FULL row, which makes the int8
 * activations identical to the single-GPU ones.
 *   cider_row_absmax:          amax[m] = max_k |x[m,k]|
 *   cider_quantize_given_amax: s = amax[m]/127 (0 -> 1), q as in cider_quantize_per_token
 *                              (amax must be >= the row's own absmax), scale[m] = s.
 * No counterpart in the reference, which has no multi-device path; the arithmetic is
 * that of cider/kernels/w8a8_quantize.metal:64-86. */
int cider_row_absmax(const void *x_f16, int64_t M, int64_t K, int64_t ldx, float *amax, void *stream);
int cider_quantize_given_amax(const void *x_f16, int64_t M, int64_t K, int64_t ldx, const float *amax,
                              void *q_i8, float *scale, void *stream);

/* Raw integer GEMM  C[m,n] = sum_k A[m,k]*B[n,k]  (int8,int8 -> exact int32).
 * Replaces int8_matmul_int32, csrc/src/prim_bindings.cpp:33 /
 * csrc/src/w8a8_primitive.mm:280-342 / cider/kernels/w8a8_matmul.metal:301-472. */
int cider_int8_matmul_int32(const void *a_i8, const void *b_i8, int32_t *c,
                            int64_t M, int64_t N, int64_t K, void *stream);

/* W8A8 per-channel linear  y = dequant(quant(x) . W^T) + bias, fp16 [M,N].
 *   M  > 1: quantise x per token, integer GEMM, epilogue
 *           half(float(acc)*sa[m]*sw[n] + float(bias[n]));
 *   M == 1: x is NOT quantised: half(sw[n]*sum_k float(W[n,k])*float(x[k]) + bias[n]).
 * scale_w: fp32 [N]; bias: fp16 [N] or NULL (zeros).
 * Replaces perchannel_linear, csrc/src/prim_bindings.cpp:18 /
 * csrc/src/w8a8_primitive.mm:137-276 (dispatch :157-178 for M == 1). */
int cider_perchannel_linear(const void *x_f16, const void *w_i8, const float *scale_w,
                            const void *bias_f16, void *y_f16, int64_t M, int64_t N,
                            int64_t K, void *workspace, size_t workspace_bytes,
                            void *stream);

/* W8A8 per-group linear.  scale_w: [K/group_size, N] (physically transposed,
 * cider/nn.py:85-88), fp32 or fp16 (`scale_dtype`); group_size in {64,128,256};
 * K % group_size == 0.
 *   M  > 1: accf = sum_g float(acc_g)*sw[g,n] (ascending g), half(accf*sa[m] + bias[n]);
 *   M == 1: half(sum_g sw[g,n]*sum_{k in g} float(W[n,k])*float(x[k]) + bias[n]).
 * Replaces pergroup_linear, csrc/src/prim_bindings.cpp:23 /
 * csrc/src/pergroup_primitive.mm:138-312.  The reference's `new_bias` argument
 * is bound but ignored by its kernels (cider/kernels/pergroup_int8_mv.metal:27)
 * and has no counterpart here. */
int cider_pergroup_linear(const void *x_f16, const void *w_i8, const void *scale_w,
                          int scale_dtype, const void *bias_f16, void *y_f16, int64_t M,
                          int64_t N, int64_t K, int group_size, void *workspace,
                          size_t workspace_bytes, void *stream);

/* W4A8 linear.  packed_w: uint8 [K/2,N] (N contiguous), high nibble = even k,
 * low nibble = odd k, value = nibble - 8.  No bias, no M == 1 special case.
 *   group_size == 0: scale_w [N]           -> half(float(acc)*sa[m]*sw[n])
 *   group_size  > 0: scale_w [K/gs, N]     -> per-group accumulation as above
 * The nibbles are expanded to int8 inside the GEMM, in the shared-memory stage the
 * tensor core reads (the reference expands them in its fragment load,
 * cider/kernels/w4a8_matmul.metal:47-70); this packing is first transposed into rows in
 * the workspace (one pass over N*K/2 bytes; see cider_w4a8_linear_nk4 to skip it).
 * Replaces w4a8_linear, csrc/src/prim_bindings.cpp:29 /
 * csrc/src/w4a8_primitive.mm:175-283 (reference: group_size == 0, fp32 scales). */
int cider_w4a8_linear(const void *x_f16, const void *packed_w, const void *scale_w,
                      int scale_dtype, int group_size, void *y_f16, int64_t M, int64_t N,
                      int64_t K, void *workspace, size_t workspace_bytes, void *stream);

/* The same linear on weights repacked once into rows: w_nk4 [N, K/2] bytes, byte j of
 * row n = (w[n][2j] + 8) << 4 | (w[n][2j+1] + 8), i.e. the reference's nibble convention
 * with K contiguous (cider/ops.py pack_weight_int4 writes [K/2, N], N contiguous, which
 * suits a Metal threadgroup but cannot be streamed row by row).  No counterpart in the
 * reference.  cider_w4a8_repack converts (one pass, at weight-load time).  With rows in
 * this layout a decode-sized call (M <= 16, per-group M <= 64, K % 64 == 0) streams the
 * packed bytes - half the HBM traffic of int8 - and expands the nibbles in registers;
 * larger M runs the tcgen05 GEMM whose converter warps expand the packed rows into the
 * shared-memory stage the MMA reads (K >= 128, K % 32 == 0), so the weights cross HBM as
 * 4-bit values only and no weight scratch is needed.  Arguments, results and errors as
 * cider_w4a8_linear; workspace size from CIDER_OP_W4A8_ROWS; K % 16 == 0.
 * Memory for time: the in-kernel expansion costs shared-memory bandwidth the int8 kernels
 * do not spend (measured 0.86 of the int8 rate per channel, 0.74 per group of 64 at
 * M = 8192).  A caller that passes a workspace of at least
 * cider_workspace_bytes(CIDER_OP_W4A8_ROWS_INT8COPY, ...) bytes (N*K more) gets, beyond decode
 * sizes, an int8 copy made by a pass of its own followed by the int8 kernels: the same
 * results at the int8 rate. */
int cider_w4a8_repack(const void *packed_w_kn, void *w_nk4, int64_t N, int64_t K, void *stream);
int cider_w4a8_linear_nk4(const void *x_f16, const void *w_nk4, const void *scale_w, int scale_dtype,
                          int group_size, void *y_f16, int64_t M, int64_t N, int64_t K, void *workspace,
                          size_t workspace_bytes, void *stream);

/* The per-channel linear above for callers that cannot pass a workspace because
 * they cannot allocate device memory where the call is made (a plugin living
 * inside another program's fixed memory budget, a latency-critical path that
 * must not hit cudaMalloc's device-wide synchronisation, a host runtime without
 * an allocator to borrow from).  No counterpart in the reference.
 *   - Scratch is an array built into the library (about 8.06 MiB of device
 *     memory on every GPU that loads it, held until exit).  Limits for M > 1:
 *     M*K <= 8388608 and M <= 16384, otherwise CIDER_E_WORKSPACE with a message
 *     that names the limit.  M == 1 uses no scratch and has no limit.
 *   - The first call on a device resolves the array's address
 *     (cudaGetSymbolAddress); make that call before any stream capture.
 *   - All calls on one device share the array (it keeps the previous call's
 *     bytes; every byte that is read is rewritten first).  Calls that can run
 *     concurrently on one GPU race: keep them on one stream.
 *   - Calls no cudaMalloc / cudaFree / allocating routine.
 *   - Same kernel choice as cider_linear_prequantized after the quantiser (streaming
 *     kernel for 2 <= M <= 16, tensor-core tiles otherwise).  It never takes the
 *     split-K form that cider_perchannel_linear uses for M <= 512 with few output
 *     tiles and a long K (its int32 slabs do not fit the array): those shapes give
 *     the same bits but may take up to twice as long.
 * Same arguments, results and error codes as cider_perchannel_linear. */
int cider_perchannel_linear_noalloc(const void *x_f16, const void *w_i8, const float *scale_w,
                                    const void *bias_f16, void *y_f16, int64_t M, int64_t N,
                                    int64_t K, void *stream);

/* cider_perchannel_linear for activations and results in HOST memory (x_host
 * [M,K] fp16, y_host [M,N] fp16; pinned memory for full speed, pageable memory
 * works).  Weights, scales and bias stay device pointers.  No counterpart in the
 * reference, which runs on unified memory and has no copies to hide; a caller on a
 * discrete GPU that holds host pointers otherwise pays upload + kernels + download
 * in sequence.  Rows are processed in chunks of chunk_rows (0 = about 16 MB of
 * output per chunk) on three internal streams so that the upload of the next
 * chunk and the download of the previous one overlap the kernels.
 *   - Ordered after the work already queued on `stream`; `stream` resumes when the
 *     last rows are in y_host.  x_host must stay valid and y_host untouched until
 *     then (synchronise `stream`, or an event recorded on it, before reading).
 *   - Staging buffers belong to the library (per device, cudaMalloc on first use,
 *     grown on demand, kept until exit); calls on one device are serialised.  Not
 *     capturable into a CUDA graph.
 *   - Results are bit-identical to cider_perchannel_linear on the same rows (M == 1
 *     takes the matrix-vector path; a last chunk of one row does not). */
int cider_perchannel_linear_host(const void *x_host_f16, const void *w_i8, const float *scale_w,
                                 const void *bias_f16, void *y_host_f16, int64_t M, int64_t N, int64_t K,
                                 int64_t chunk_rows, void *stream);

/* Linear on activations that are already int8 (a_i8 [M,K], scale_a [M]), e.g.
 * produced once by cider_quantize_per_token / cider_rmsnorm_quant and shared by
 * several projections.  group_size 0 = per-channel.  Second half of
 * csrc/src/w8a8_primitive.mm:206-247 and csrc/src/pergroup_primitive.mm:219-272. */
int cider_linear_prequantized(const void *a_i8, const float *scale_a, const void *w_i8,
                              const void *scale_w, int scale_dtype, int group_size,
                              const void *bias_f16, void *y_f16, int64_t M, int64_t N,
                              int64_t K, void *stream);

/* RMSNorm fused with the per-token quantiser:
 *   n = half(float(x) * rsqrt(mean(x^2) + eps) * float(w))  (rounded to fp16 first,
 *   exactly what an unfused norm would hand to the quantiser), then S1 on n.
 * y_f16 may be NULL when only the int8 form is needed.  No counterpart in the
 * reference, whose RMSNorm is an MLX library op in front of quantize_per_token. */
int cider_rmsnorm_quant(const void *x_f16, const void *w_f16, float eps, int64_t M,
                        int64_t K, void *y_f16, void *q_i8, float *scale, void *stream);

/* Residual update fused with the norm (and optionally the quantiser):
 *   x <- half(x + delta) in place (skipped when delta is NULL), n = RMSNorm(x) as
 *   above; n is stored to y_f16 when given, and quantised to (q_i8, scale) when
 *   q_i8 is given.  No counterpart in the reference (MLX library ops). */
int cider_add_rmsnorm_quant(void *x_f16_inout, const void *delta_f16, const void *w_f16, float eps,
                            int64_t M, int64_t K, void *y_f16, void *q_i8, float *scale, void *stream);

/* Per-head q/k RMSNorm + rotary embedding + KV-cache append for the fused
 * projection output qkv [B*T, (nq+2nkv)*D] (D == 128):
 *   q, k heads: n = half(RMSNorm_D(x) * w), then rotate-half rope in fp32 with
 *   angle[d] = pos3[axis[d], t] * inv_freq[d] (d < D/2; `axis` selects the t/h/w
 *   position row per frequency slot: interleaved M-RoPE; all zeros for 1-D rope);
 *   q -> q_out [B, nq, T, D]; k, v -> caches [B, nkv, Tcap, D] at base + t, where
 *   base = *base_dev when base_dev is non-NULL (read on the device, for CUDA-graph
 *   replay) else base_host.  pos3 is int32 [3, pos_stride] on the device.
 *   base_host + T > Tcap is refused with CIDER_E_SHAPE; a device-side base that puts
 *   a token outside [0, Tcap) skips that token's K / V stores and records
 *   CIDER_STATUS_KV_OVERFLOW (read with cider_device_status).
 * Restates the attention prologue of the reference's model code
 * (cider/fused_hybrid.py:177-190); no kernel counterpart there. */
int cider_qk_norm_rope_append(const void *qkv_f16, const void *q_norm_w, const void *k_norm_w,
                              const float *inv_freq, const int8_t *axis, const int32_t *pos3,
                              int64_t pos_stride, const int32_t *base_dev, int64_t base_host, float eps,
                              void *q_out, void *k_cache, void *v_cache, int64_t B, int64_t T, int64_t nq,
                              int64_t nkv, int64_t D, int64_t Tcap, void *stream);

/* SwiGLU: act[m,i] = half(half(silu(g)) * u), g = gate_up[m,i], u = gate_up[m,inter+i]
 * (cider/fused_hybrid.py:205-213 in the reference's model code). */
int cider_silu_mul(const void *gate_up_f16, void *act_f16, int64_t M, int64_t inter, void *stream);

/* cider_quantize_per_token on an attention output still in [B, heads, T, D] layout
 * (what a batched attention kernel writes): q [B*T, heads*D] int8 and scale [B*T],
 * row (b, t) being the concatenation of its heads - the transpose + reshape copy in
 * front of the output projection is never made.  D % 16 == 0, 16-byte aligned. */
int cider_quantize_heads(const void *a_f16, int64_t B, int64_t heads, int64_t T, int64_t D, void *q_i8,
                         float *scale, void *stream);

/* cider_silu_mul followed by cider_quantize_per_token in one pass: q [M,inter] int8
 * and scale [M] of act = half(half(silu(gate)) * up), without writing act.  The
 * down projection of a prefill chunk then runs as cider_linear_prequantized. */
int cider_silu_mul_quant(const void *gate_up_f16, int64_t M, int64_t inter, void *q_i8, float *scale,
                         void *stream);

/* The fused gate/up projection of a prefill chunk with the SwiGLU in its epilogue (per-channel
 * int8 weights, activations already quantised): act [M, N/2] fp16 = half(half(silu(g)) * u) of
 * the fp16 linear outputs g, u - the values cider_linear_prequantized followed by cider_silu_mul
 * produce, without the [M, N] round trip - and rowmax[m] raised to max_i |act[m,i]| (fp32; the
 * caller passes it zeroed, cider_quantize_consume_amax leaves it zeroed again).
 * w_i8 [N, K] (and scale_w [N], bias [N]) hold the rows of the fused projection INTERLEAVED in
 * blocks of 32: rows 64 b .. 64 b + 31 are gate rows 32 b .., rows 64 b + 32 .. 64 b + 63 the up
 * rows 32 b .. (cider_b200.ops.interleave_gate_up builds it).  N % 64 == 0; shapes the tensor-core
 * kernels take (K % 16 == 0, 16-byte aligned operands), else CIDER_E_SHAPE.  No counterpart in
 * the reference (cider/fused_hybrid.py:205-213 runs the linear and the SwiGLU as separate ops). */
int cider_swiglu_linear_prequantized(const void *a_i8, const float *scale_a, const void *w_i8,
                                     const float *scale_w, const void *bias_f16, void *act_f16,
                                     float *rowmax, int64_t M, int64_t N, int64_t K, void *stream);

/* cider_quantize_given_amax that also writes 0 back to amax[m] once the row has read it: the
 * quantiser behind cider_swiglu_linear_prequantized. */
int cider_quantize_consume_amax(const void *x_f16, int64_t M, int64_t K, int64_t ldx, float *amax,
                                void *q_i8, float *scale, void *stream);

/* M == 1 linear (the matrix-vector path of cider_perchannel_linear /
 * cider_pergroup_linear, group_size 0 = per-channel) with the preceding
 * elementwise step folded into the load of the activation:
 *   prologue 0: x [K] as is;
 *   prologue 1: x is a fused [gate | up] vector of length 2K, the activation is
 *               half(half(silu(gate)) * up)               (what cider_silu_mul computes);
 *   prologue 2: v = half(x + delta) (delta may be NULL), written to x_out when
 *               given (x_out must not alias x), activation = RMSNorm(v) * norm_w as in
 *               cider_add_rmsnorm_quant.
 * A batch-1 decode step of a small model is bound by kernel launches, not by
 * HBM; this removes three launches per decoder layer.  No counterpart in the
 * reference (MLX fuses nothing across these ops either).
 * Prologues 1 and 2 need the streaming kernel: K % 64 == 0, 16-byte aligned
 * operands, group_size 0 or 64 * 2^i with N % 8 == 0; otherwise CIDER_E_SHAPE. */
int cider_linear_m1_fused(const void *x_f16, int prologue, const void *delta_f16, const void *norm_w_f16,
                          float eps, void *x_out_f16, const void *w_i8, const void *scale_w, int scale_dtype,
                          int group_size, const void *bias_f16, void *y_f16, int64_t N, int64_t K,
                          void *stream);

/* Split-K single-query attention over an fp16 KV cache (decode step).
 *   q [B,Hq,D]; k_cache, v_cache [B,Hkv,Tcap,D]; out [B,Hq,D]; Hq % Hkv == 0;
 *   attends to positions [0,T), or [0,*length_dev) when length_dev (device
 *   int32, <= T) is given - T then only sizes the split.  Replaces the MLX library call the reference's
 *   model code makes (visible at cider/fused_hybrid.py:192). */
int cider_sdpa_decode(const void *q_f16, const void *k_cache, const void *v_cache,
                      void *out_f16, int64_t B, int64_t Hq, int64_t Hkv, int64_t D,
                      int64_t T, int64_t Tcap, float scale, void *workspace,
                      size_t workspace_bytes, const int32_t *length_dev, void *stream);
size_t cider_sdpa_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T);

/* The same in ONE launch: `tickets` is a device array of B*Hkv uint32 that is zero
 * on entry; the block that finishes last for a (batch, KV head) merges the splits
 * and puts its counter back to zero, so the array can be reused by the next call
 * (also across CUDA-graph replays).  Calls that may run concurrently need separate
 * arrays.  Same arguments and results otherwise. */
int cider_sdpa_decode_tickets(const void *q_f16, const void *k_cache, const void *v_cache,
                              void *out_f16, int64_t B, int64_t Hq, int64_t Hkv, int64_t D,
                              int64_t T, int64_t Tcap, float scale, void *workspace,
                              size_t workspace_bytes, const int32_t *length_dev, uint32_t *tickets,
                              void *stream);

/* One-shot all-reduce (sum) of a small fp16 message between the GPUs of one box, over
 * peer-mapped memory: the exchange step of a tensor-parallel decode step, where every
 * rank holds a partial [M, hidden] result of a row-parallel o_proj / down_proj.  The
 * reference has no multi-device path; the loop this sits in is
 * vlm_service/custom_qwen3vl.py:660-679.  One kernel per rank and call, no host round
 * trip, capturable in a CUDA graph (the call counter lives in device memory).
 *
 * Set-up, once per process (one process per GPU):
 *   cider_peer_alloc   cudaMalloc + zero an "inbox" of `bytes` on the current device and
 *                      return its address and a 64-byte handle (cudaIpcGetMemHandle).  This is
 *                      a set-up call and, with cider_perchannel_linear_host, the only place
 *                      where the library allocates device memory.
 *   cider_peer_open    map a peer's inbox from its handle (exchanged by the caller, e.g.
 *                      through torch.distributed); cider_peer_close unmaps it.
 *   cider_peer_free    release the own inbox (after every peer has closed it).
 *   cider_peer_reset   zero the header of the own inbox (flags and counters) on `stream`; every
 *                      rank must do it, with a host barrier on both sides, after a time-out.
 *   cider_peer_max_bytes  largest message for an inbox of the given size:
 *                      (inbox_bytes - 4096) / 16, rounded down to 256.
 *
 * cider_allreduce_f16: out[i] = half(sum over ranks 0..world-1, in that order, in fp32, of
 *   in[i]) for count halves (a multiple of 8; in / out 16-byte aligned, may alias).  Every rank
 *   gets the same bits.  `inboxes` is a HOST array of `world` device pointers, entry q being
 *   rank q's inbox as mapped in this process (the own allocation at [rank]).  All ranks must
 *   make the same sequence of calls with the same count.  Peers are only ever written to
 *   (plain stores over NVLink; no multicast); the wait for the peers' flags polls local
 *   memory and is bounded by wait_cycles GPU clocks (0 = about a second): when it runs out
 *   the kernel records CIDER_STATUS_PEER_TIMEOUT, writes no result and returns, and the
 *   group has to be reset.  2 <= world <= 8; CIDER_E_WORKSPACE when the message exceeds
 *   cider_peer_max_bytes. */
size_t cider_peer_max_bytes(size_t inbox_bytes);
int cider_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int cider_peer_open(const unsigned char *handle64, void **ptr);
int cider_peer_close(void *ptr);
int cider_peer_free(void *ptr);
int cider_peer_reset(void *own_inbox, void *stream);
int cider_allreduce_f16(const void *in_f16, void *out_f16, int64_t count, int rank, int world,
                        void *const *inboxes, size_t inbox_bytes, int64_t wait_cycles, void *stream);

/* The exchange fused with what follows it in a decoder layer: partial_f16 [M,K] is this
 * rank's partial output of a row-parallel linear;
 *   delta = cider_allreduce_f16(partial), x <- half(x + delta) in place,
 *   n = RMSNorm(x) * norm_w as in cider_add_rmsnorm_quant, stored to y_f16 when given and
 *   quantised per token to (q_i8, scale) when q_i8 is given
 * in ONE kernel (one CTA per row; the row stays in registers from the peer stores to the
 * quantised store).  1 <= M <= 32, K % 8 == 0, K <= 8192, M*K*2 <= cider_peer_max_bytes.
 * Same group, call-sequence rules, bounded wait and status bit as cider_allreduce_f16 (the
 * two share the inbox and its call counters, and may be mixed freely).  No counterpart in
 * the reference. */
int cider_allreduce_add_rmsnorm_quant(const void *partial_f16, void *x_f16_inout, const void *norm_w_f16, float eps,
                                      int64_t M, int64_t K, void *y_f16, void *q_i8, float *scale, int rank,
                                      int world, void *const *inboxes, size_t inbox_bytes, int64_t wait_cycles,
                                      void *stream);

/* cider_qk_norm_rope_append for ONE new token per sequence followed by cider_sdpa_decode
 * (or _tickets when `tickets` is given), in one launch: every block of the attention kernel
 * normalises and rotates the query heads of its group itself (from the raw projection output
 * qkv [B, (Hq + 2 Hkv) * D], D == 128; position ids pos3[:, 0]), and the block whose split
 * holds the newest position appends the new key and value to the caches at position L - 1
 * before it walks its positions, L = *length_dev (or T when length_dev is NULL) being the
 * attended length INCLUDING the new token.  Same arithmetic and roundings as the two separate
 * calls (same bits).  L > Tcap appends nothing and records CIDER_STATUS_KV_OVERFLOW.  Removes
 * one launch per decoder layer from a decode step.  No counterpart in the reference. */
int cider_sdpa_decode_fused(const void *qkv_f16, const void *q_norm_w, const void *k_norm_w, const float *inv_freq,
                            const int8_t *axis, const int32_t *pos3, int64_t pos_stride, float eps, void *k_cache,
                            void *v_cache, void *out_f16, int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T,
                            int64_t Tcap, float scale, void *workspace, size_t workspace_bytes,
                            const int32_t *length_dev, uint32_t *tickets, void *stream);

/* Kernels bound every wait (on shared-memory barriers, on another GPU's flag) and
 * check what only the device knows (a cache position read from device memory); they
 * record a failure in a device status word instead of hanging or writing out of
 * bounds.  Read (synchronises the device) / clear it.  Returns CIDER_OK and stores 0
 * in *status when nothing was recorded; otherwise a mask of the bits below. */
#define CIDER_STATUS_WAIT_TIMEOUT 1u /* a wait on a shared-memory barrier ran out            */
#define CIDER_STATUS_KV_OVERFLOW 4u  /* cider_qk_norm_rope_append: base_dev + t outside the
                                        cache; the K / V stores of that token were skipped  */
#define CIDER_STATUS_PEER_TIMEOUT 8u /* a wait on another GPU's flag ran out                 */
int cider_device_status(unsigned int *status);
int cider_clear_device_status(void);

/* Launch the decode-step kernels (matrix-vector, norm, rope/append, SwiGLU,
 * decode attention) with programmatic dependent launch: a kernel may start while
 * its predecessor in the stream is finishing and waits on the device before it
 * reads the predecessor's output.  Process-wide, off by default; meant to be
 * switched on around the capture of a decode-step CUDA graph.  Results are
 * unchanged. */
int cider_set_programmatic_launch(int enable);

#ifdef __cplusplus
}
#endif
#endif /* CIDER_B200_H_ */
