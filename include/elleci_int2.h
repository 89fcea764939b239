/*
 * elleci_int2.h - C ABI of the B200 (sm_100a) BitNet INT2 linear library (libelleci_int2.so).
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream; the caller owns all memory.
 * Nothing here allocates, synchronises or prints.  Every function returns EL_OK (0) or a negative
 * EL_ERR_* code; el_status_string() names it and el_last_cuda_error() gives the CUDA error code behind
 * EL_ERR_CUDA on the calling thread.  All calls are asynchronous on `stream` and re-entrant across
 * host threads, streams and devices: there is no hidden scratch memory, with one documented exception,
 * el_linear_decode_static, whose scratch is a static device array shared by all calls on a device.
 * The el_set_* tuning calls are process-wide and take effect for calls made after they return.
 *
 * Each declaration cites the interface of the reference project (step325/Elleci-Training-Vast,
 * paths relative to its root) that it replaces.
 *
 * Data formats (identical to the reference's, kernels/int2/int2_packed.cuh:9-86):
 *   W_packed  uint8 [N, ceil(K/4)]  four ternary weights per byte, weight k at bits 2*(k%4) of byte k/4;
 *                                   code 0 = -1, 1 = 0, 2 = +1, 3 = reserved (reads as 0)
 *   H_packed  uint8 [N, ceil(K/2)]  two signed 4-bit hysteresis counters per byte, even k in the low nibble
 *   Xq        int8  [M, K]          quantised activations, row-major
 *   absmax    float [M] or [1]      max |x| of a token row (or of the whole tensor); the dequantisation
 *                                   scale is absmax/127, applied in the GEMM epilogue
 */
#ifndef ELLECI_INT2_H_
#define ELLECI_INT2_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t), passed as an opaque pointer so that the header needs no CUDA include. */
typedef void* el_stream_t;

/* Exported symbol marker (the library is built with hidden default visibility). */
#if defined(__GNUC__)
#define EL_API __attribute__((visibility("default")))
#else
#define EL_API
#endif

/* ---- status codes ---------------------------------------------------------------------------------- */
#define EL_OK                     0
#define EL_ERR_INVALID_ARG       -1   /* a size, dtype or flag is out of range */
#define EL_ERR_NULL_PTR          -2   /* a required pointer is NULL */
#define EL_ERR_ALIGNMENT         -3   /* a pointer or pitch breaks an alignment rule of the requested path */
#define EL_ERR_UNSUPPORTED_SHAPE -4   /* the requested path cannot run this shape (see the function's notes) */
#define EL_ERR_CUDA              -5   /* a CUDA runtime call failed; see el_last_cuda_error() */
#define EL_ERR_DEVICE            -6   /* the current device is not an sm_100 part */
#define EL_ERR_DRIVER            -7   /* the driver refused a tensor-map descriptor */
#define EL_ERR_TOO_LARGE         -8   /* a size exceeds the fixed capacity of the entry point (el_linear_decode_static) */

/* ---- element types of floating-point / output buffers ------------------------------------------------ */
#define EL_F16  0
#define EL_BF16 1
#define EL_F32  2
#define EL_I32  3   /* raw int32 accumulators (outputs only): the bit-exact check of a GEMM */

/* ---- GEMM path selection (flags argument) ------------------------------------------------------------ */
#define EL_PATH_AUTO   0   /* tensor-core (tcgen05) kernel when the shape allows it, CUDA-core kernel otherwise */
#define EL_PATH_SIMPLE 1   /* force the CUDA-core kernel (any shape) */
#define EL_PATH_TC     2   /* require the tcgen05 kernel; EL_ERR_UNSUPPORTED_SHAPE / EL_ERR_ALIGNMENT if it cannot run */
#define EL_PATH_TC_SINGLE 3 /* as EL_PATH_TC, but forward / dX on the single-CTA kernel instead of CTA pairs */
/* May be OR-ed into the path: the CTA-pair kernels keep to 128 registers per thread, so that a kernel which needs no
 * shared memory (el_peer_put on another stream) can run on the same SMs beside them; about 9 % slower on their own. */
#define EL_FLAG_LEAN   0x100

EL_API int el_version(void);
EL_API const char* el_status_string(int status);
EL_API int el_last_cuda_error(void);

/* Device-side error word written by the tensor-core kernels when one of their bounded waits gives up
 * (0 = no error; otherwise a code naming the wait).  `dev_status` arguments below may be NULL. */

/* ---- weight format --------------------------------------------------------------------------------- */

/* Packs int8 ternary weights w[N,K] into W_packed; unused fields of a row's last byte get pad_code (0..3).
 * Replaces Int2LinearTC._pack_int2_cpu (core/bitnet/int2_linear_tc.py:414-436) and the test packer
 * pack_int2 (kernels/tests/kernel_build.py:69-81), which run on the host. */
EL_API int el_pack_ternary(const int8_t* w, uint8_t* W_packed, int N, int K, int pad_code, el_stream_t stream);

/* q = clamp(round_half_even(W/gamma), -1, 1) packed in one pass (padding code 0, as the module packer).
 * Replaces Int2LinearTC.init_from_float (core/bitnet/int2_linear_tc.py:391-412). */
EL_API int el_ternarize_pack(const float* W, float gamma, uint8_t* W_packed, int N, int K, el_stream_t stream);

/* Decodes W_packed into a dense [N,K] matrix of {-1,0,+1}; out_dtype EL_F16 / EL_BF16 / EL_F32, or
 * EL_I32 meaning int8 output.  Replaces int2_unpack_to_fp16 (kernels/int2/int2_unpack.cu:157-174,
 * binding kernels/int2/int2_tc_ops.cpp:476-499). */
EL_API int el_unpack_ternary(const uint8_t* W_packed, void* out, int out_dtype, int N, int K, el_stream_t stream);

/* ---- activation quantisation ------------------------------------------------------------------------ */

/* Per-token absmax int8 quantisation: a[m] = max(max_k |x[m,k]|, eps), q = clamp(rint(x*(127/a)), -128, 127);
 * non-finite inputs count as 0.  x_dtype EL_F16 / EL_BF16 / EL_F32; ldx is the row pitch of x in elements
 * (>= K: a column window of a wider matrix needs no copy); q is dense [M,K].  Replaces
 * BitLinear.activation_quant (model/common/bitnet_legacy.py:58-87), in integer form.
 * mode EL_QUANT_FULL        one pass: row_absmax[m] receives a[m], q the int8 row.
 *      EL_QUANT_ABSMAX_ONLY row_absmax[m] receives the raw max |x[m,:]| (no floor); q is not touched.  A rank that
 *                           holds a column shard reduces these over ranks (max) before quantising.
 *      EL_QUANT_WITH_ABSMAX row_absmax[m] holds the raw maximum on entry (as written by ABSMAX_ONLY, possibly
 *                           reduced over ranks); it is floored at eps in place and the row is quantised with it.
 * Optional gradient folding (both NULL to disable; not with ABSMAX_ONLY): with fold_absmax[M] given, fold_max[1]
 * receives, by an atomic max, max_m(rawmax[m] * (fold_absmax[m]/127)); the caller zeroes fold_max first. */
#define EL_QUANT_FULL        0
#define EL_QUANT_ABSMAX_ONLY 1
#define EL_QUANT_WITH_ABSMAX 2
EL_API int el_quantize_rows(const void* x, int x_dtype, long long ldx, int8_t* q, float* row_absmax, int M, int K,
                            float eps, int mode, const float* fold_absmax, float* fold_max, el_stream_t stream);

/* Per-tensor absmax int8 quantisation: absmax[0] = max finite |x| (the call zeroes it first),
 * q = clamp(roundf(x * (absmax > 1e-8 ? 127/absmax : 0)), -127, 127).  Replaces quantize_activation_async
 * (kernels/int2/int2_activation_quant.cu:313-343, binding kernels/int2/int2_tc_ops.cpp:343-371); the scratch
 * word of the reference is the caller's own absmax buffer here. */
EL_API int el_quantize_tensor(const void* x, int x_dtype, int8_t* q, float* absmax, long long size, el_stream_t stream);

/* out = q * (absmax[0]/127).  Replaces dequantize_activation (int2_activation_quant.cu:290-304,
 * binding int2_tc_ops.cpp:310-337). */
EL_API int el_dequantize_tensor(const int8_t* q, const float* absmax, void* out, int out_dtype, long long size,
                         el_stream_t stream);

/* Gq[m,n] = clamp(rint((dY[m,n] * (x_absmax[m]/127)) * inv), -127, 127), inv = g >= 1e-30 ? 127/g : 0,
 * g = g_absmax[0] (from el_quantize_rows' fold_max).  The per-token activation scale folded into the output
 * gradient makes the weight gradient an exact integer GEMM.  ld_dy is the row pitch of dY in elements; Gq is
 * dense [M,N].  No counterpart in the reference, which forms dW with a library fp16 GEMM
 * (core/bitnet/int2_linear_tc.py:525-537). */
EL_API int el_quantize_grad(const void* dY, int dy_dtype, long long ld_dy, const float* x_absmax, const float* g_absmax,
                            int8_t* Gq, int M, int N, el_stream_t stream);

/* out[m,c] = out_dtype( float(acc[m,c]) * ((absmax[m*absmax_stride]/127) * gamma) ): the GEMM epilogue as a
 * stand-alone pass, for int32 sums that were reduced over ranks first (dX of an N-sharded layer).  The reference
 * has no multi-GPU path; the arithmetic is that of its GEMM epilogue (int2_backward_int8_tc_v2.cu:88-92,233). */
EL_API int el_scale_rows(const int32_t* acc, void* out, int out_dtype, const float* absmax, int absmax_stride,
                         float gamma, int M, int C, el_stream_t stream);

/* ---- pre-linear RMSNorm fused with the per-token quantiser ------------------------------------------ */

/* The reference normalises the activations right before every INT2 linear call
 * (_ExtraRMSNorm, core/bitnet/bitnet_int2_optimized.py:72-86,203-204; _RMSNorm, model/common/bitnet_legacy.py:10-25):
 *   y = dtype( dtype(x * rstd) * dtype(weight) ),  rstd[m] = 1/sqrt(mean_k x[m,k]^2 + norm_eps)  (float32)
 * and quantises y per token.  This call does both in one pass over x (dtype EL_F16/EL_BF16/EL_F32, row pitch ldx
 * elements, weight float32 [K]): q int8 [M,K] and row_absmax [M] exactly as el_quantize_rows(y, quant_eps) gives them,
 * plus rstd [M] for the backward pass.  The sum of squares is accumulated in float64, so the result does not depend on
 * the order of the additions.  Needs K % 8 == 0 and 16-byte aligned rows (EL_ERR_UNSUPPORTED_SHAPE / EL_ERR_ALIGNMENT
 * otherwise). */
EL_API int el_rmsnorm_quantize_rows(const void* x, int x_dtype, long long ldx, const float* weight, float norm_eps,
                                    int8_t* q, float* row_absmax, float* rstd, int M, int K, float quant_eps,
                                    el_stream_t stream);
/* Backward of the normalisation above for an upstream gradient g [M,K] with respect to y (the quantiser is a
 * straight-through estimator, model/common/bitnet_legacy.py:83-87), following autograd through the reference's
 * expression:  gn = dtype(g * dtype(weight));  c[m] = sum_k gn*x;  dx = dtype(gn*rstd - x * (rstd^3 * c / K));
 * dweight[k] = sum_m g[m,k] * dtype(x*rstd)[m,k]  (float32 [K], overwritten).  g, x, dx contiguous [M,K] of `dtype`.
 * `workspace`: el_rmsnorm_backward_workspace_bytes(K) bytes, 16-byte aligned, contents irrelevant.  K % 8 == 0 and
 * K <= 25600. */
EL_API size_t el_rmsnorm_backward_workspace_bytes(int K);
EL_API int el_rmsnorm_backward(const void* g, const void* x, int dtype, const float* weight, const float* rstd, void* dx,
                               float* dweight, void* workspace, size_t workspace_bytes, int M, int K, el_stream_t stream);

/* ---- SwiGLU gate fused with the down projection's norm and quantiser ------------------------------- */

/* The reference's feed-forward block is w3(silu(w1 x) * w2 x) (SwiGLUFFN.forward, model/model.py:107-108); its INT2
 * layer then normalises and quantises that product (core/bitnet/bitnet_int2_optimized.py:201-210).  This call takes
 * the outputs of the gate and up projections (gate, up: [M,H] of `dtype`, common row pitch ld elements, so they may
 * be the two halves of one [M,2H] buffer) and writes what the down projection's GEMM reads:
 *   s = dtype(gate * sigmoid(gate));  h = dtype(s * up);
 *   y = dtype(dtype(h * rstd) * dtype(norm_weight)),  rstd[m] = 1/sqrt(mean_k h[m,k]^2 + norm_eps)   (y = h and rstd
 *   untouched when norm_weight is NULL);  q, row_absmax = per-token quantisation of y as el_quantize_rows gives it.
 * sigmoid(g) = 1/(1 + e^-g) in float32 with a fixed polynomial exponential (about 1 ulp), so the result is the same on
 * every run and reproducible on a CPU; against a float32 library silu it differs by at most one unit of `dtype` on a
 * small fraction of elements.  H % 8 == 0, 16-byte aligned rows. */
EL_API int el_swiglu_quantize_rows(const void* gate, const void* up, int dtype, long long ld, const float* norm_weight,
                                   float norm_eps, int8_t* q, float* row_absmax, float* rstd, int M, int H,
                                   float quant_eps, el_stream_t stream);
/* The input of an INT2 layer as el_rmsnorm_quantize_rows / el_swiglu_quantize_rows form it, written out in `dtype`
 * (y [M,K], contiguous) instead of being quantised: x is the layer input, or the gate when `up` is not NULL
 * (h = dtype(dtype(x*sigmoid(x))*up)); with norm_weight not NULL the row is normalised as _ExtraRMSNorm does
 * (core/bitnet/bitnet_int2_optimized.py:72-86).  Feeding y to el_linear_decode gives, for 1..64 tokens, the output the
 * training-time forward gives for them bit for bit (the decode kernels quantise their tokens themselves): the
 * inference path of Elleci.generate (model/model.py:505-623) through normalised layers.  K % 8 == 0, 16-byte aligned
 * rows. */
EL_API int el_prelinear_rows(const void* x, const void* up, int dtype, long long ld, const float* norm_weight,
                             float norm_eps, void* y, int M, int K, el_stream_t stream);
/* sig[i] = sigmoid(g[i]) in float32 exactly as the two SwiGLU calls compute it (fixed polynomial exponential, correctly
 * rounded reciprocal): lets a port or a test check the arithmetic element by element.  torch's silu, which the
 * reference calls (model/model.py:108), uses the platform's exponential instead. */
EL_API int el_sigmoid_fixed(const float* g, float* sig, long long n, el_stream_t stream);
/* Backward of the call above for the gradient gy [M,H] (contiguous) with respect to y, following autograd through the
 * reference's tensor operations (quantiser = straight-through estimator):
 *   gn = dtype(gy*dtype(w));  c[m] = sum_k gn*h;  dh = dtype(gn*rstd - h*(rstd^3*c/H));  d_norm_weight[k] = sum_m
 *   gy*dtype(h*rstd)  (dh = gy without a norm);  ds = dtype(dh*up);  d_up = dtype(dh*s);
 *   d_gate = dtype((ds*sig) * (1 + gate*(1 - sig))).
 * d_gate, d_up: [M,H] with common row pitch ld_d (may be the halves of one [M,2H] buffer: the gradient of the fused
 * gate|up projection).  workspace: el_swiglu_backward_workspace_bytes(H) bytes, 16-byte aligned (unused without a
 * norm).  H % 8 == 0; H <= 25600 with a norm. */
EL_API size_t el_swiglu_backward_workspace_bytes(int H);
EL_API int el_swiglu_backward(const void* gy, const void* gate, const void* up, int dtype, long long ld,
                              const float* norm_weight, const float* rstd, void* d_gate, void* d_up, long long ld_d,
                              float* d_norm_weight, void* workspace, size_t workspace_bytes, int M, int H,
                              el_stream_t stream);

/* ---- GEMMs ------------------------------------------------------------------------------------------- */

/* Y[m,n] = out_dtype( float(sum_k Xq[m,k]*Wq[n,k]) * ((absmax[m*absmax_stride]/127) * gamma) ).
 * absmax_stride 1 = per-token scales, 0 = one per-tensor scale.  Tensor-core path needs K % 64 == 0 and
 * 16-byte aligned Xq / W_packed.  Replaces int2_matmul_int8_tc_v2 (kernels/int2/int2_matmul_int8_tc_v2.cu:
 * 500-537, binding tc_matmul_int8 kernels/int2/int2_tc_ops.cpp:381-425). */
EL_API int el_gemm_fwd(const int8_t* Xq, const uint8_t* W_packed, void* Y, int out_dtype, const float* absmax,
                int absmax_stride, float gamma, int M, int N, int K, int flags, int32_t* dev_status,
                el_stream_t stream);

/* el_gemm_fwd / el_gemm_dx with a caller-owned workspace that lets a problem with few output tiles use the whole GPU.
 * A GEMM whose output has fewer 256 x 256 tiles than half the GPU's CTA pairs and whose reduction is long (512 tokens
 * through 11008 -> 4096: 32 tiles for 74 pairs, 86 reduction blocks; the per-rank GEMMs of a layer split over eight
 * GPUs) is cut along its reduction into q <= 8 parts
 * that run side by side; each part stores int32 partial sums in the workspace and a second small kernel adds them
 * (exact: the result is bit-identical to the unsplit GEMM) and applies the scaling epilogue.  el_gemm_workspace_bytes
 * (mode 0 = forward, 1 = dX) says how many bytes that takes for a shape, 0 when the shape is not split; with workspace
 * NULL or too small the call runs unsplit, as el_gemm_fwd / el_gemm_dx do.  The workspace (16-byte aligned) needs no
 * initialisation and holds nothing between calls; calls that share one must not overlap on the GPU.  No counterpart in
 * the reference. */
EL_API size_t el_gemm_workspace_bytes(int mode, int M, int N, int K);
EL_API int el_gemm_fwd_ws(const int8_t* Xq, const uint8_t* W_packed, void* Y, int out_dtype, const float* absmax,
                          int absmax_stride, float gamma, int M, int N, int K, int flags, void* workspace,
                          size_t workspace_bytes, int32_t* dev_status, el_stream_t stream);
EL_API int el_gemm_dx_ws(const int8_t* dYq, const uint8_t* W_packed, void* dX, int out_dtype, const float* absmax,
                         int absmax_stride, float gamma, int M, int N, int K, int flags, void* workspace,
                         size_t workspace_bytes, int32_t* dev_status, el_stream_t stream);

/* Forward GEMM of one N-shard fused with the all-gather of the output: the [M,N] result of el_gemm_fwd (N = this
 * rank's rows of W_packed) is written at column col_offset of EVERY matrix Y_all[r] (r < n_ranks <= 8, each [M, ld_total]
 * of out_dtype): the rank's own buffer and the peer-mapped buffers of the other ranks (symmetric memory / IPC
 * mappings).  The epilogue sends each output block with TMA stores over NVLink while later tiles compute; there is no
 * separate collective.  The caller orders the ranks (a barrier after the kernel before any rank reads Y, and before
 * the next call overwrites it).  Needs the tensor-core path (K % 64 == 0), N % 32 == 0 and 16-byte aligned bases,
 * pitch and col_offset.  No counterpart in the reference, which is single-GPU (README.md:58). */
EL_API int el_gemm_fwd_gather(const int8_t* Xq, const uint8_t* W_packed, void* const* Y_all, int n_ranks, long long ld_total,
                              long long col_offset, int out_dtype, const float* absmax, int absmax_stride, float gamma,
                              int M, int N, int K, int32_t* dev_status, el_stream_t stream);

/* dX[m,k] = out_dtype( float(sum_n dYq[m,n]*Wq[n,k]) * ((absmax[m*absmax_stride]/127) * gamma) ).
 * Tensor-core path needs N % 16 == 0 and K % 64 == 0.  Replaces int2_backward_dx_int8_tc_v2
 * (kernels/int2/int2_backward_int8_tc_v2.cu:465-499, binding tc_backward_input_int8 int2_tc_ops.cpp:435-470). */
EL_API int el_gemm_dx(const int8_t* dYq, const uint8_t* W_packed, void* dX, int out_dtype, const float* absmax,
               int absmax_stride, float gamma, int M, int N, int K, int flags, int32_t* dev_status,
               el_stream_t stream);

/* dX GEMM of one N-shard fused with the reduce-scatter of its partial sums: rank `rank` of n_ranks (<= 8) computes the
 * int32 sums of el_gemm_dx over its rows of W_packed and the epilogue stores the token rows [d*M/n_ranks, (d+1)*M/n_ranks)
 * into slot `rank` of parts_all[d], rank d's staging buffer of shape [n_ranks, M/n_ranks, K] int32 (own buffer or a
 * peer mapping; TMA stores over NVLink).  After a barrier, rank d owns all partial sums of its rows:
 * el_reduce_scale_gather adds them (exact), scales by (absmax[m]/127)*gamma and writes the rows into every rank's
 * dX [M,K] (dX_all[r]), which completes the all-reduce.  Rank r produces the token rows in cyclic order starting with
 * its own, so that at any time the ranks store into different owners (one sender per receiving link).
 * Needs M % (32*n_ranks) == 0, N % 16 == 0, K % 64 == 0.  No counterpart in the reference (single-GPU). */
EL_API int el_gemm_dx_scatter(const int8_t* dYq, const uint8_t* W_packed, void* const* parts_all, int n_ranks, int rank,
                              int M, int N, int K, int32_t* dev_status, el_stream_t stream);
EL_API int el_reduce_scale_gather(const int32_t* parts, void* const* dX_all, int n_ranks, int rank, int out_dtype,
                                  const float* absmax, float gamma, int M, int K, el_stream_t stream);

/* Barrier between the n_ranks (<= 8) GPUs of an N-sharded layer, one process per GPU, for the three calls above:
 * flags_all[i] is rank i's array of n_ranks uint32 flags (own memory or a peer mapping, zero before the first
 * barrier); `epoch` counts this group's barriers 1, 2, ... identically on every rank.  The call queues one tiny kernel
 * that publishes `epoch` in every rank's array (after all earlier work of the stream, stores to peers included) and
 * waits until every rank has done the same.  The wait is bounded (seconds); a rank that does not arrive is reported as
 * code 40 + its index in *dev_status.  No counterpart in the reference. */
EL_API int el_peer_barrier(uint32_t* const* flags_all, int n_ranks, int rank, uint32_t epoch, int32_t* dev_status,
                           el_stream_t stream);
/* el_peer_barrier that also delivers one 32-bit word: before it publishes its epoch, the rank copies `word` (device
 * memory, 4 bytes) to byte offset dst_offset of every rank's buffer dst_all[i]; after the barrier every rank holds every
 * rank's word (each rank passes its own offset).  The token-parallel layer exchanges its partial gradient maxima this
 * way, in the barrier it needs anyway, instead of with a launch of its own.  No counterpart in the reference. */
EL_API int el_peer_barrier_put(uint32_t* const* flags_all, int n_ranks, int rank, uint32_t epoch, int32_t* dev_status,
                               const void* word, void* const* dst_all, size_t dst_offset, el_stream_t stream);
/* el_peer_barrier (word == dst_all == NULL) or el_peer_barrier_put whose epoch is not passed but taken from memory: one
 * more than the epoch this rank published last, which every form of the barrier leaves in slot `rank` of the rank's own
 * flag array.  The launch therefore has no argument that changes from barrier to barrier, so a sequence of launches
 * recorded once (CUDA stream capture) can be replayed, each replay being the next barriers; explicit-epoch calls may be
 * mixed in as long as the host keeps counting.  Every rank must use the same sequence of barriers, as before.  No
 * counterpart in the reference. */
EL_API int el_peer_barrier_next(uint32_t* const* flags_all, int n_ranks, int rank, int32_t* dev_status, const void* word,
                                void* const* dst_all, size_t dst_offset, el_stream_t stream);
/* *counter += delta on the device, in stream order (one thread).  Keeps a step counter that kernels read from memory
 * (el_dw_hysteresis_step_ptr) in step with the recorded launches that use it.  No counterpart in the reference. */
EL_API int el_counter_add(int32_t* counter, int delta, el_stream_t stream);
/* Bound of el_peer_barrier's wait, process-wide, for barriers queued from now on: microseconds > 0 sets it, 0 restores
 * the default of a few seconds.  A health check (or a test) that wants a missing rank reported within a millisecond
 * instead of seconds sets it; the barrier then returns with code 40 + rank in *dev_status and the device stays usable. */
EL_API int el_set_peer_barrier_limit_us(long long microseconds);

/* ---- token-parallel layer: every GPU runs forward and dX on its own tokens, the weight update is split by rows ---- */

/* Pushes `bytes` bytes of local memory `src` to byte offset dst_offset of each of the n_dst (<= 8) buffers dst[d] (own
 * memory or peer mappings; plain 16-byte stores over NVLink when everything is 16-byte aligned, 4-byte stores otherwise;
 * 4-byte alignment is the minimum).  The building block of the layer's all-gathers (the int8 tokens every rank needs for
 * its rows of the weight gradient; the updated rows of W_packed every replica needs): each rank pushes its block, a
 * barrier (el_peer_barrier) completes the exchange.  max_ctas > 0 caps the grid, so that a push running beside a GEMM
 * takes few SMs; 0 picks a size that saturates the links.  No counterpart in the reference (single-GPU, README.md:58). */
EL_API int el_peer_put(const void* src, void* const* dst, int n_dst, size_t dst_offset, size_t bytes, int max_ctas,
                       el_stream_t stream);
/* The same push through the copy engines: one asynchronous device-to-device copy per destination, queued on `stream` in
 * the order of dst[] (a rank should list its peers starting with its successor, so that at any moment every GPU receives
 * from one sender).  No SM takes part, so a GEMM running beside the push keeps all of its SMs and registers; any
 * alignment.  No counterpart in the reference. */
EL_API int el_peer_put_dma(const void* src, void* const* dst, int n_dst, size_t dst_offset, size_t bytes, el_stream_t stream);

/* el_quantize_grad for a token-sharded layer, fused with the all-to-all of its result: this rank's M gradient rows
 * dY[M,N] are quantised exactly as el_quantize_grad does, and the column window [d*N/n_ranks, (d+1)*N/n_ranks) of row m is
 * stored at row row_offset + m of Gq_all[d], rank d's receive buffer of shape [M_total, N/n_ranks] int8 (own memory or a
 * peer mapping).  The per-tensor maximum is max(g_slots[0..n_slots)), the ranks' partial maxima exchanged beforehand; it
 * is also written to g_absmax_out[0] (may be NULL) for el_dw_hysteresis.  Needs (N/n_ranks) % 8 == 0, ld_dy % 8 == 0 and a
 * 16-byte aligned dY.  No counterpart in the reference. */
EL_API int el_quantize_grad_scatter(const void* dY, int dy_dtype, long long ld_dy, const float* x_absmax, const float* g_slots,
                                    int n_slots, float* g_absmax_out, void* const* Gq_all, int n_ranks, long long row_offset,
                                    int M, int N, el_stream_t stream);

/* dW[n,k] = float(sum_m Gq[m,n]*Xq[m,k]) * (g_absmax[0]/127)   (out_dtype EL_F32, or EL_I32 for the raw sums).
 * Tensor-core path needs N % 16 == 0 and K % 16 == 0.  Replaces `torch.mm(dY_2d.t(), X_2d).float()`
 * (core/bitnet/int2_linear_tc.py:537, core/bitnet/int2_linear_tc_offload.py:247). */
EL_API int el_gemm_dw(const int8_t* Gq, const int8_t* Xq, void* dW, int out_dtype, const float* g_absmax, int M, int N,
               int K, int flags, int32_t* dev_status, el_stream_t stream);

/* ---- hysteresis ---------------------------------------------------------------------------------------- */

/* One hysteresis update of W_packed / H_packed from a float32 gradient dW[N,K], in place; bit-exact with
 * int2_hysteresis_v2_update (kernels/int2/int2_hysteresis_v2.cu:54-194, binding tc_hysteresis_step_v2
 * kernels/int2/int2_tc_ops.cpp:214-257), including its fast-math flush of float32 denormals when ftz != 0.
 * idx_base offsets the random-number counter (n*K + k) for a row shard of a larger matrix. */
EL_API int el_hysteresis_from_dw(const float* dW, uint8_t* W_packed, uint8_t* H_packed, float lr, float lr_scale,
                          int threshold, float decay_rate, int step, int N, int K, uint32_t idx_base, int ftz,
                          el_stream_t stream);

/* Weight-gradient GEMM fused with the hysteresis update: the int32 sums of el_gemm_dw stay on chip, are scaled
 * by g_absmax[0]/127 and drive the same per-weight update as el_hysteresis_from_dw (ftz on); W_packed and
 * H_packed are rewritten in place and dW never reaches memory.  Needs N % 16 == 0 and K % 32 == 0
 * (EL_ERR_UNSUPPORTED_SHAPE otherwise: use el_gemm_dw + el_hysteresis_from_dw).  Replaces the pair
 * torch.mm + hysteresis_step_v2 of Int2LinearTC.hysteresis_update (core/bitnet/int2_linear_tc.py:483-548). */
EL_API int el_dw_hysteresis(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* W_packed,
                     uint8_t* H_packed, float lr, float lr_scale, int threshold, float decay_rate, int step,
                     uint32_t idx_base, int M, int N, int K, int32_t* dev_status, el_stream_t stream);
/* el_dw_hysteresis with the step number read from device memory (`step`, one int32, read by the kernel when it runs)
 * instead of passed by value: the launch then has no argument that changes from step to step and can be recorded once
 * and replayed; el_counter_add advances the number between replays.  Same update, bit for bit, as el_dw_hysteresis with
 * the value found there.  No counterpart in the reference. */
EL_API int el_dw_hysteresis_step_ptr(const int8_t* Gq, const int8_t* Xq, const float* g_absmax, uint8_t* W_packed,
                                     uint8_t* H_packed, float lr, float lr_scale, int threshold, float decay_rate,
                                     const int32_t* step, uint32_t idx_base, int M, int N, int K, int32_t* dev_status,
                                     el_stream_t stream);

/* ---- small-M ("decode") layer -------------------------------------------------------------------------------- */

/* Y[m,n] = out_dtype( float(sum_k Q(x)[m,k]*Wq[n,k]) * ((absmax[m]/127) * gamma) ) for 1 <= M <= 64 tokens: per-token
 * quantisation of x followed by a weight-streaming tensor-core kernel (operands swapped, stream-K over all SMs), the
 * same integers and the same rounding as el_quantize_rows + el_gemm_fwd.  Needs K % 64 == 0 and 16-byte aligned x,
 * W_packed, xq_scratch and workspace.  Caller-owned scratch: xq_scratch int8 [M,K] and absmax float [M] (overwritten),
 * and `workspace` of el_decode_workspace_bytes(N) bytes, which must be all zero before its first use and is left
 * all zero by every call (partial sums of weight tiles that span several SMs meet there); calls that share a
 * workspace must not overlap on the GPU.  Replaces the scalar kernel the reference falls back to when M < 64
 * (int2_matmul_int8_tc_v2_simple_kernel, kernels/int2/int2_matmul_int8_tc_v2.cu:452-473, dispatch :511-536), the
 * path of Elleci.generate (model/model.py:505-623). */
EL_API size_t el_decode_workspace_bytes(int N);
/* Tuning: calls with at most `max_tokens` tokens (0..8, default 2) take a single-launch CUDA-core GEMV that
 * quantises the tokens itself and touches no scratch; larger ones take the tensor-core kernel.  Process-wide. */
EL_API int el_set_decode_gemv_max_tokens(int max_tokens);
/* Tuning: calls with more tokens than the limit above and at most `max_tokens` (0..64, default 64) whose int8 tokens,
 * taken 32 at a time, fit in shared memory (up to 32*K of about 190 KB) run on the warp-level int8 MMA: up to 8 tokens as
 * one launch that quantises the tokens itself and touches no scratch; more tokens as the row quantiser (into xq_scratch
 * and absmax) followed by one launch per 32 tokens on the quantised tokens, each a programmatic dependent of the launch
 * before it.  The rest take the tcgen05 stream-K kernel.  Process-wide. */
EL_API int el_set_decode_mma_max_tokens(int max_tokens);
/* Tuning, off by default: with `enable` != 0 the single-launch GEMV of el_linear_decode is issued as a programmatic
 * dependent launch.  It may then start while earlier work of the stream still runs; until that work has completed it
 * only loads W_packed, and it reads x and writes Y afterwards.  Enable it only when nothing queued earlier on the
 * stream writes W_packed (inference: the weights are constant).  Consecutive decode calls then overlap their weight
 * loads with the tail of the previous call.  Process-wide; no counterpart in the reference. */
EL_API int el_set_decode_overlap(int enable);
EL_API int el_linear_decode(const void* x, int x_dtype, const uint8_t* W_packed, void* Y, int out_dtype, float gamma,
                            int8_t* xq_scratch, float* absmax, void* workspace, size_t workspace_bytes, int M, int N,
                            int K, int32_t* dev_status, el_stream_t stream);

/* el_linear_decode for callers that cannot give the library any device memory (no counterpart in the reference).
 * Serving processes that forbid cudaMalloc after start-up, runtimes that own the whole memory pool and hosts at
 * their memory budget cannot supply the scratch buffers of el_linear_decode; here the quantised tokens, their
 * scales and the partial-sum workspace live in one static device array inside the library (about 5.3 MB, held by
 * every GPU that loads the library until the process exits).  The caller passes only x [M,K], W_packed and Y [M,N].
 * Limits: M <= 64, N <= 16384, K <= 16384, K % 64 == 0; larger sizes return EL_ERR_TOO_LARGE.  Same results as
 * el_linear_decode.  The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 * The first call on a device resolves the array's address (cudaGetSymbolAddress): make that first call with the
 * device current and before any stream capture.  All calls on a device share the one array, which keeps the
 * contents of the previous call; the parts that must start at zero are cleared on `stream` at the start of each
 * call.  Two calls whose GPU work overlaps (different streams, or threads) race on it: order them. */
EL_API int el_linear_decode_static(const void* x, int x_dtype, const uint8_t* W_packed, void* Y, int out_dtype, float gamma,
                                   int M, int N, int K, int32_t* dev_status, el_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* ELLECI_INT2_H_ */
