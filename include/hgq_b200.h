/*
 * hgq_b200.h -- C ABI of the B200 (sm_100a) kernels behind the HGQ2 quantised-training hot path.
 *
 * Every entry point takes raw device pointers (unless its name ends in _host), element counts,
 * mode enums and a CUDA stream handle (a cudaStream_t passed as void*; NULL = the default
 * stream).  Unless an entry says otherwise it allocates nothing, is asynchronous on the given
 * stream and returns
 *      0          success (the work has been enqueued),
 *      negative   an HGQ_ERR_* argument error (nothing was enqueued),
 *      positive   a cudaError_t raised by a launch or a runtime call.
 * hgq_status_string() turns any of the three into text.
 *
 * The reference (calad0i/HGQ2) has no FFI of its own: it is pure Python on top of Keras and of
 * the third-party `quantizers` package.  Each declaration below therefore cites the Python call
 * site in the reference that it stands in for (path:line inside the HGQ2 tree).
 *
 * Conventions shared by all entries
 *   - tensors are contiguous, row-major fp32 unless noted; `k` (keep_negative) is uint8 in {0,1},
 *     the dtype of the reference variable (fixed_point_quantizer.py:218-224);
 *   - `i` and `f` hold integer-valued floats (the reference passes round_conv()'ed variables,
 *     fixed_point_quantizer.py:248-265,439-445); they are converted with round-to-nearest-even and
 *     must lie in [-100, 100];
 *   - parameter layout: `period` == n (or 0) means k/i/f have one entry per element of x
 *     ("full"); otherwise they hold `period` entries and element e of x uses entry e % period
 *     ("broadcast": the bitwidth tensor is x.shape with the leading homogeneous axes set to 1,
 *     base.py:163-183).  n must be a multiple of period.
 */
#ifndef HGQ_B200_H_
#define HGQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ---------------------------------------------------------------------- */
#define HGQ_OK 0
#define HGQ_ERR_NULL (-1)      /* a required pointer is NULL                                  */
#define HGQ_ERR_SIZE (-2)      /* a count/shape is negative, inconsistent or over a limit     */
#define HGQ_ERR_MODE (-3)      /* unknown round / overflow mode or flag                       */
#define HGQ_ERR_ALIGN (-4)     /* a pointer is not aligned to its element type                */
#define HGQ_ERR_WORKSPACE (-5) /* the scratch buffer passed in is too small                   */
#define HGQ_ERR_DEVICE (-6)    /* the current device is not an sm_100 part                    */
#define HGQ_ERR_TIMEOUT (-7)   /* a bounded device-side wait gave up (status word non-zero)   */

/* ---- modes (names follow the reference's round_mode / overflow_mode strings) ------------- */
enum hgq_round_mode {
    HGQ_ROUND_TRN = 0,      /* floor(x * 2^f) / 2^f                                            */
    HGQ_ROUND_RND = 1,      /* floor(x * 2^f + 0.5) / 2^f                                      */
    HGQ_ROUND_RND_CONV = 2  /* round-half-even(x * 2^f) / 2^f                                  */
};

enum hgq_overflow_mode {
    HGQ_OVERFLOW_NONE = 0,    /* rounding only: stateless_quantizer.round(x, f, ...)            */
    HGQ_OVERFLOW_WRAP = 1,    /* two's-complement wrap into [-k 2^i, 2^i - 2^-f]                */
    HGQ_OVERFLOW_SAT = 2,     /* clip to [-k 2^i, 2^i - 2^-f]                                   */
    HGQ_OVERFLOW_SAT_SYM = 3  /* clip to [-k (2^i - 2^-f), 2^i - 2^-f]                          */
};

/* flags (bit-or) */
#define HGQ_FLAG_TRAINING 1u       /* training=True: WRAP leaves the rounded value unwrapped     */
#define HGQ_FLAG_ZERO_NONPOS 2u    /* eval-only: y = 0 where k+i+f <= 0 (fixed_point_quantizer.py:148-149) */
#define HGQ_FLAG_ABSMAX_ACCUMULATE 4u /* hgq_qdense_fwd: absmax = max(absmax, statistic) instead of being overwritten */

/* ---- library ------------------------------------------------------------------------------ */

/* Text for a status returned by any entry point. Never NULL. */
const char *hgq_status_string(int status);

/* ABI version of this header (bumped on incompatible change). */
int hgq_abi_version(void);

/* Number of kernels this library has launched in the calling process (all entries, all
 * streams).  Used by the benchmark to report how many launches a timed region made. */
int64_t hgq_launch_count(void);

/* ---- K1: elementwise fixed-point quantizer ------------------------------------------------ */

/*
 * Forward.  Stands in for stateless_quantizer(x, k, i, f, training, seed_gen)
 * (call site fixed_point_quantizer.py:142-150) and stateless_quantizer.round(x, f, ...)
 * (call sites fixed_point_quantizer.py:288,295,305,405) of quantizers.fixed_point.
 *
 *   y[e] = overflow(round(x[e], f), k, i, f)
 *
 * absmax (optional, may be NULL): `period` floats that receive max over the broadcast rows of
 * |round(x, f)| -- the reduction x_to_bw_absmax (base.py:185-186) that the WRAP integer-bit
 * tracking consumes (fixed_point_quantizer.py:405-413).  The entry clears it first.
 * With overflow_mode NONE, `k` and `i` may be NULL.
 */
int hgq_quantize_fwd(const float *x, const uint8_t *k, const float *i, const float *f, float *y,
                     float *absmax, int64_t n, int64_t period, int round_mode, int overflow_mode,
                     unsigned flags, void *stream);

/*
 * Scratch bytes hgq_quantize_bwd needs for (n, period); 0 for the full layout.
 */
size_t hgq_quantize_bwd_workspace(int64_t n, int64_t period);

/*
 * Backward (surrogate gradients).  Stands in for the custom gradient of the same two callables.
 * g is the upstream gradient dL/dy.
 *
 *   dx[e]  straight-through, zero where SAT / SAT_SYM clipped
 *   df     -ln2 * (round(x,f) - x) * g on unclipped elements, +-ln2 2^-f g on clipped ones
 *   di     ln2 2^i g on elements clipped at the top, -k ln2 2^i g at the bottom; 0 for WRAP/NONE
 *
 * Full layout: di/df have n entries.  Broadcast layout: di/df have `period` entries holding the
 * sum over the broadcast rows (the backward of bw_to_x, base.py:182-183); partial sums are
 * staged in `workspace` and reduced in a fixed order, so results do not depend on scheduling.
 * di may be NULL (it is identically zero for WRAP / NONE).
 */
int hgq_quantize_bwd(const float *g, const float *x, const uint8_t *k, const float *i,
                     const float *f, float *dx, float *di, float *df, int64_t n, int64_t period,
                     int round_mode, int overflow_mode, unsigned flags, void *workspace,
                     size_t workspace_bytes, void *stream);

/*
 * The same backward for callers that must not allocate device memory -- a plugin inside a framework
 * whose memory pool already owns the GPU, or a service with a fixed memory budget.  This entry has no
 * counterpart in the reference.  It takes no workspace: the column-sum partials of the broadcast
 * layout go to a fixed array of HGQ_NOALLOC_SCRATCH_BYTES inside the library (device memory that every
 * GPU which loads the library holds until the process exits).  It calls no cudaMalloc / cudaFree and
 * no allocating library routine.
 *
 * Limit: hgq_quantize_bwd_workspace(n, period) must not exceed HGQ_NOALLOC_SCRATCH_BYTES, otherwise
 * the call returns HGQ_ERR_SIZE and launches nothing (use hgq_quantize_bwd with your own workspace).
 * The full layout needs no scratch and is never limited.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with the
 * calling thread's current device); make that first call before any stream capture begins.
 * The array used is the CURRENT device's: the calling thread's current device must be the device
 * `stream` belongs to (cudaSetDevice before the call), otherwise the kernels would be handed another
 * GPU's scratch address.
 * All calls on a device share the one array and it keeps the previous call's contents: nothing in it
 * has to be cleared (each call overwrites every word it later reads), but two calls whose kernels
 * overlap on the GPU -- different streams, no ordering between them -- race on it and corrupt each
 * other's di / df.  Serialise them on one stream or with events.
 * Outputs are identical to hgq_quantize_bwd's.
 */
#define HGQ_NOALLOC_SCRATCH_BYTES (8u << 20)
int hgq_quantize_bwd_noalloc(const float *g, const float *x, const uint8_t *k, const float *i,
                             const float *f, float *dx, float *di, float *df, int64_t n,
                             int64_t period, int round_mode, int overflow_mode, unsigned flags,
                             void *stream);

/* ---- K2: fused quantised dense layer ------------------------------------------------------- */

/*
 * Scratch bytes hgq_qdense_fwd needs when the abs-max side output is requested (0 if the shape is not
 * supported by the fused kernel).
 */
size_t hgq_qdense_fwd_workspace(int64_t M, int K, int N, int rows_period);

/*
 * y = act( iq(x) @ wq + bq ) in one pass.  Stands in for QDense.call (layers/core/dense.py:60-68) and for
 * QEinsumDense.call (layers/core/einsum_dense.py:72-83) when the contraction is over the trailing input
 * axis ('...k,kn->...n').
 *
 *   x [M, K] raw activations; qk/qi/qf: the input quantizer's tables, [rows_period, K] entries, row r of
 *   x uses table row r % rows_period (qf == NULL: no input quantizer; qk/qi may be NULL when the overflow
 *   mode is NONE, or WRAP with HGQ_FLAG_TRAINING); wq [K, N] and bq [N] (may be NULL) already quantised;
 *   activation 0 none, 1 relu; y [M, N].
 *   absmax (may be NULL): [rows_period, K] floats receiving max over rows of |round(x, f)| (the statistic
 *   of x_to_bw_absmax, quantizer/internal/base.py:185-186); needs `workspace`.  With HGQ_FLAG_ABSMAX_ACCUMULATE the
 *   statistic is merged into the caller's buffer by atomic max (the caller zeroes it once for all layers of a step): no
 *   workspace and no second launch.
 *   status (may be NULL): device word; bit 0 is set if a bounded device-side wait gave up.
 *
 * The contraction runs on the tensor cores with every operand split exactly into bf16 terms and fp32
 * accumulation, so y equals the fp32 result whenever that is exact, and is within fp32 rounding otherwise.
 * Limits: N <= 128; K as far as the three bf16 weight terms (6 K Npad bytes) fit shared memory beside the tile buffers
 * (256 at 64 outputs, about 1500 at 16; HGQ_ERR_SIZE beyond); rows_period * K <= 8192 when absmax is requested.
 */
int hgq_qdense_fwd(const float *x, const uint8_t *qk, const float *qi, const float *qf, int rows_period,
                   int round_mode, int overflow_mode, unsigned flags, const float *wq, const float *bq,
                   int activation, float *y, float *absmax, int64_t M, int K, int N, void *workspace,
                   size_t workspace_bytes, unsigned *status, void *stream);

/*
 * hgq_qdense_fwd that also returns the sum of y over every group of pool_rows consecutive rows, times pool_scale:
 * pool_out [M / pool_rows, N].  Stands in for a layer followed by a reduction over the axis its rows run along, e.g.
 * `QEinsumDense('bpc,cd->bpd')` followed by `ops.sum(x, axis=1)` / `ops.mean(x, axis=1)` with pool_rows = p (the particle-set
 * models of the reference's examples): the reduction reads the finished blocks on chip instead of reading y back from memory.
 * y is written as usual (the backward pass needs it).  Rows of a group are added in ascending order.
 * Covered: the training-mode case on the warp-specialised kernel with bulk stores (input quantizer that only rounds, K and N
 * multiples of 4, N >= 33, pool_rows 32, 64 or 128 dividing M); hgq_qdense_fwd_pooled_supported says whether a shape is
 * (HGQ_ERR_SIZE otherwise; pool_out == NULL makes the call plain hgq_qdense_fwd).
 */
int hgq_qdense_fwd_pooled_supported(int64_t M, int K, int N, int rows_period, int pool_rows, int want_absmax);
int hgq_qdense_fwd_pooled(const float *x, const uint8_t *qk, const float *qi, const float *qf, int rows_period,
                          int round_mode, int overflow_mode, unsigned flags, const float *wq, const float *bq,
                          int activation, float *y, float *absmax, float *pool_out, int pool_rows, float pool_scale,
                          int64_t M, int K, int N, void *workspace, size_t workspace_bytes, unsigned *status, void *stream);

/*
 * Scratch bytes hgq_qdense_bwd needs (0 if the shape is not supported by the fused backward).
 */
size_t hgq_qdense_bwd_workspace(int64_t M, int K, int N, int rows_period);

/*
 * Backward of hgq_qdense_fwd for a rounding-only input quantizer (training-mode WRAP) or none, in one pass
 * over gy, y and x.  Stands in for the autograd backward of QDense.call / QEinsumDense.call
 * (layers/core/dense.py:60-68, einsum_dense.py:72-83) including the quantizer's surrogate gradient.
 *
 *   G = gy * (y > 0) if y != NULL (ReLU), else gy;   dx = G @ wq^T (straight-through);
 *   dwq = round(x)^T @ G;   dbq = column sums of G;   df[p, k] = sum_{r = p mod rows_period} (-ln2 (round(x) - x)) dx
 *
 * gy, y [M, N]; x [M, K]; qf [rows_period, K] (NULL: no quantizer, then df must be NULL); wq [K, N];
 * dx [M, K] (may be NULL); dwq [K, N]; dbq [N] (may be NULL); df [rows_period, K] (may be NULL).
 * Operands enter the tensor cores as two bf16 terms (16 significant bits), the weights exactly; partial sums are
 * reduced in a fixed order.  Limits: K <= 64, N <= 128, rows_period divides 128.
 */
int hgq_qdense_bwd(const float *gy, const float *y, const float *x, const float *qf, int rows_period,
                   int round_mode, const float *wq, float *dx, float *dwq, float *dbq, float *df, int64_t M,
                   int K, int N, void *workspace, size_t workspace_bytes, unsigned *status, void *stream);
/* The same with x and dx as column slices of wider row-major matrices (row strides ldx, lddx >= K, in floats): a layer
 * with K > 64 runs as one call per block of 64 input columns, each producing its columns of dx, its rows of dwq and its
 * columns of df (dbq is the same in every call).  gy_repeat > 1: gy has M / gy_repeat rows, each serving gy_repeat
 * consecutive rows of x -- the gradient of a sum over an axis (e.g. over the particles of a set), read in place instead
 * of being expanded in memory. */
int hgq_qdense_bwd_strided(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                           int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, float *dwq,
                           float *dbq, float *df, int64_t M, int K, int N, void *workspace, size_t workspace_bytes,
                           unsigned *status, void *stream);
/* The same with dx += (instead of =) when dx_accumulate is non-zero: layers that read the same input (the query, key and value
 * projections of an attention layer) add their input gradients up in place instead of through separate passes over
 * three tensors.  Covered by the warp-specialised kernel only: hgq_qdense_bwd_accumulate_supported says whether a shape is
 * (relu: y is given; has_quantizer: qf is given); HGQ_ERR_SIZE otherwise. */
int hgq_qdense_bwd_accumulate_supported(int K, int N, int rows_period, int relu, int has_quantizer);
int hgq_qdense_bwd_accumulate(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                              int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, int dx_accumulate,
                              float *dwq, float *dbq, float *df, int64_t M, int K, int N, void *workspace, size_t workspace_bytes,
                              unsigned *status, void *stream);

/* ---- K4: quantised softmax ------------------------------------------------------------------ */

/*
 * Forward of the bit-accurate softmax in training mode.  Stands in for QSoftmax.call (layers/softmax.py:114-132,
 * stable form, no mask) with the quantizers of its exp / inverse tables (layers/activation.py:58-61) and its own
 * output quantizer (layers/core/base.py:105-110):
 *   d = max(s) - s; a = Q1(d); e = exp(-a * scaler); b = Q2(e); S = sum b; t = Q3(S); u = Q4(1 / (t + eps)); y = Q5(b u)
 * s, y [R, L] with the softmax over L (32, 64 or 128); R = batches * rows_period.  The quantizers come as HOST arrays
 * of five entries: qk / qi / qf hold device pointers (Q1..Q4: one element each; Q5: [rows_period, L] tables; qk / qi
 * entries may be NULL for a rounding-only quantizer), qrm the round modes, qom the overflow modes (NONE, SAT, SAT_SYM).
 * absmax_exp_in (1 float), absmax_inv_in (1 float) and absmax_out ([rows_period, L]) receive max |round(d)|,
 * max |round(S)| and max |round(b u)|: the statistics the integer-bit tracking of a WRAP quantizer in those three places
 * needs (fixed_point_quantizer.py:401-424); each may be NULL.
 */
int hgq_qsoftmax_fwd(const float *s, float *y, const uint8_t *const *qk, const float *const *qi,
                     const float *const *qf, const int *qrm, const int *qom, float scaler, float eps,
                     float *absmax_exp_in, float *absmax_inv_in, float *absmax_out, int64_t R, int L, int rows_period,
                     void *stream);

size_t hgq_qsoftmax_bwd_workspace(int64_t R, int L, int rows_period);

/*
 * Backward of hgq_qsoftmax_fwd: recomputes the chain from s and returns ds [R, L], the surrogate gradients of Q1..Q4
 * as dscalars8 = (di1, df1, di2, df2, di3, df3, di4, df4) and those of Q5 as df_out / di_out [rows_period, L]
 * (di_out may be NULL).  The gradient of the row maximum is shared evenly among tied maxima.  Sums are reduced in a
 * fixed order.
 */
int hgq_qsoftmax_bwd(const float *gy, const float *s, float *ds, const uint8_t *const *qk,
                     const float *const *qi, const float *const *qf, const int *qrm, const int *qom,
                     float scaler, float eps, float *dscalars8, float *df_out, float *di_out, int64_t R, int L,
                     int rows_period, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Implicit-GEMM 2-D convolution forward on the same tensor-core kernel as hgq_qdense_fwd:
 *   y = act( conv2d(x, wq) + bq ),  channels-last.
 * Stands in for the contraction of QBaseConv.call (layers/conv.py:72-89); the input quantizer is applied beforehand by
 * hgq_quantize_fwd (x here is the already quantised image), because a pixel is shared by up to KH*KW patches.
 *   x [B, H, W, C] with C % 4 == 0; wq [KH*KW*C, N] (the reference's [KH, KW, C, N] kernel flattened); bq [N] or NULL;
 *   y [B, OH, OW, N]; output pixel (oh, ow) tap (kh, kw) reads x[b, oh*stride_h - pad_top + kh*dil_h,
 *   ow*stride_w - pad_left + kw*dil_w, :], zero outside the image.  Patches are gathered straight from the image into
 *   the operand staging (no im2col buffer).  Limits: KH*KW*C <= 640, N <= 128.
 * The transposed convolution that yields dL/dx is the same call on dL/dy with the flipped, transposed kernel.
 */
int hgq_qconv2d_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW);
/* Shapes the unit-stride kernel takes (any channel count: an image whose C is not a multiple of 4 is read with scalar
 * loads instead of being padded in memory). */
int hgq_qconv2d_unit_stride_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW, int dil_h,
                                      int dil_w);
int hgq_qconv2d_fwd(const float *x, int64_t B, int H, int W, int C, const float *wq, const float *bq, int activation,
                    float *y, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w, int dil_h,
                    int dil_w, int pad_top, int pad_left, unsigned *status, void *stream);

/*
 * Convolution weight / bias gradient (the kernel-side half of the autograd backward of QBaseConv.call,
 * layers/conv.py:72-89), patches gathered from the image like hgq_qconv2d_fwd:
 *   G = gy * (y > 0) when y != NULL (ReLU), else G = gy;   gm = G (written only when y != NULL; y and gm come together)
 *   dwq [KH*KW*C, N] = patches(x)^T @ G,   dbq [N] = sum over pixels of G (dbq may be NULL).
 * x [B, H, W, C] (C % 4 == 0, the quantised image the forward saw), gy / y / gm [B, OH, OW, N].
 * Limits: N <= 128, ceil((KH*KW*C + 1) / 128) * roundup(N, 16) <= 512, B*H*W*C < 2^31, pads >= 0.
 * Scratch: hgq_qconv2d_wgrad_workspace bytes (0 = unsupported shape).  Results do not depend on scheduling.
 */
size_t hgq_qconv2d_wgrad_workspace(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW);
int hgq_qconv2d_wgrad(const float *x, const float *gy, const float *y, float *gm, float *dwq, float *dbq, int64_t B,
                      int H, int W, int C, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w,
                      int dil_h, int dil_w, int pad_top, int pad_left, void *workspace, size_t workspace_bytes,
                      unsigned *status, void *stream);

/* ---- K5: channels-last 2-D max pooling ('valid') ----------------------------------------------------------------
 * The keras MaxPooling2D between the QConv2D layers of the reference's convolutional models (QMaxPooling2D,
 * layers/pooling.py:146-167, delegates to the same keras op).  x [B, H, W, C] -> y [B, OH, OW, C] with
 * OH = (H - pool_h) / stride_h + 1; argmax [B, OH, OW, C] holds the winning window position (ph * pool_w + pw, first
 * maximum in scan order) as one byte.  The backward routes gy to those positions (summing where windows overlap).
 */
int hgq_maxpool2d_fwd(const float *x, float *y, unsigned char *argmax, int64_t B, int H, int W, int C, int pool_h,
                      int pool_w, int stride_h, int stride_w, int OH, int OW, void *stream);
int hgq_maxpool2d_bwd(const float *gy, const unsigned char *argmax, float *dx, int64_t B, int H, int W, int C,
                      int pool_h, int pool_w, int stride_h, int stride_w, int OH, int OW, void *stream);

/* ---- K6: per-head products of multi-head attention ---------------------------------------------------------------
 * The two activation-activation contractions of QMultiHeadAttention._compute_attention (layers/attn/mha.py:434-470)
 * and the four products of their backward, on the tensor cores, reading the head-interleaved projections in place.
 * "SHD" = [B, L, H, D] fp32, "HTS" = [B, H, L, L] fp32; L = 64, D = 16 or 32, H even.
 *   kind 0: out_HTS[b,h,t,s] = sum_d x_SHD[b,t,h,d] * y_SHD[b,s,h,d]     (scores = Q K^T;  dP = dO V^T)
 *   kind 1: out_SHD[b,t,h,d] = sum_s x_HTS[b,h,t,s] * y_SHD[b,s,h,d]     (context = P V;   dQ = dS K)
 *   kind 2: out_SHD[b,s,h,d] = sum_t x_HTS[b,h,t,s] * y_SHD[b,t,h,d]     (dV = P^T dO;     dK = dS^T Q)
 * Operands go through two bf16 terms each (exact up to 16 significant bits), fp32 accumulation.
 */
int hgq_attn_heads_supported(int64_t B, int L, int H, int D);
int hgq_attn_heads_matmul(int kind, const float *x, const float *y, float *out, int64_t B, int L, int H, int D,
                          unsigned *status, void *stream);

/* ---- integer-bit tracking of WRAP quantizers (training) ------------------------------------------------------------
 * i_state <- max(i_state - decay, fewest integer bits that hold absmax), in place, one launch:
 *   hgq_track_kif: minimal_i_given_xf, FixedPointQuantizerKIF.call (fixed_point_quantizer.py:25-31, 401-411);
 *   hgq_track_kbi: minimal_i_given_xb, FixedPointQuantizerKBI.call (:16-22, 277-288), then the clamp [lo, hi] of the
 *                  variable's MinMax constraint (pass -INFINITY / INFINITY for none).
 * absmax >= 0 and the raw (unrounded) f / b variables have n elements each; decay is a device scalar.
 */
int hgq_track_kif(const float *absmax, const float *f_raw, float *i_state, const float *decay, int64_t n, void *stream);
int hgq_track_kbi(const float *absmax, const float *b_raw, float *i_state, const float *decay, int symmetric, float lo,
                  float hi, int64_t n, void *stream);

/* ---- softmax cross-entropy from logits, integer labels, mean over the batch ------------------------------------------
 * The task loss the reference's models are compiled with (keras SparseCategoricalCrossentropy(from_logits=True); Keras,
 * not HGQ2, owns it).  loss (device scalar) and dlogits = (softmax - onehot) / B in one pass; C <= 64;
 * workspace: hgq_softmax_xent_workspace(B) bytes.  Deterministic (fixed-order reduction).
 */
size_t hgq_softmax_xent_workspace(int64_t B);
int hgq_softmax_xent(const float *logits, const int64_t *labels, float *loss, float *dlogits, int64_t B, int C,
                     void *workspace, size_t workspace_bytes, void *stream);

/* ---- K3: EBOPs ---------------------------------------------------------------------------- */

/*
 * EBOPs of a dense / einsum-dense layer and the gradient of its loss term.  Stands in for
 * QDense._compute_ebops (layers/core/dense.py:70-80), QEinsumDense._compute_ebops
 * (layers/core/einsum_dense.py:85-93) and the wrapper's `_ebops.assign(cast(ebops, uint32));
 * add_loss(ebops * beta)` (layers/core/base.py:95-104).
 *
 *   e = scale * ( sum_{p,k,n} bw_in[p,k] bw_w[k,n] + mean(bw_bias) * out_size )
 *
 * bw_in [P, K]: input bitwidths at batch 1 (P = product of the free input axes), bw_w [K, N],
 * bw_bias [n_bias] (n_bias = 0: no bias), all integer-valued fp32.  `beta` is a device scalar.
 * Outputs (each may be NULL): ebops = uint32(e); ebops_f = float(e); loss = ebops_f * beta;
 * d_bw_in / d_bw_w / d_bw_bias = d loss / d (the three bitwidth tensors).  The integer sum is
 * exact.  K <= 10240.  One CTA; latency-bound.
 */
int hgq_ebops_dense(const float *bw_in, int64_t P, int64_t K, const float *bw_w, int64_t N,
                    const float *bw_bias, int64_t n_bias, double out_size, double scale,
                    const float *beta, uint32_t *ebops, float *ebops_f, float *loss, float *d_bw_in,
                    float *d_bw_w, float *d_bw_bias, void *stream);

/*
 * hgq_ebops_dense for up to HGQ_EBOPS_BATCH_MAX layers in ONE launch (a block per layer): the terms of a step's dense
 * layers cost one launch latency instead of one per layer.  `descs` is a host array; the fields are hgq_ebops_dense's
 * arguments.
 */
#define HGQ_EBOPS_BATCH_MAX 16
typedef struct {
    const float *bw_in;
    int64_t P, K;
    const float *bw_w;
    int64_t N;
    const float *bw_bias;
    int64_t n_bias;
    double out_size, scale;
    const float *beta;
    uint32_t *ebops;
    float *ebops_f, *loss, *d_bw_in, *d_bw_w, *d_bw_bias;
} hgq_ebops_dense_desc;
int hgq_ebops_dense_batch(const hgq_ebops_dense_desc *descs, int n, void *stream);

/*
 * EBOPs of a channels-last 2-D convolution: sum(conv(bw_in, bw_w)) * scale_main +
 * mean(bw_bias) * out_size * scale_bias (layers/conv.py:91-102).  bw_in [H, W, C],
 * bw_w [KH, KW, C, N]; (OH, OW) is the output size, pad_top / pad_left the implicit zero padding
 * ('valid': 0).  Outputs as for hgq_ebops_dense.  KH*KW*C <= 10240.
 */
int hgq_ebops_conv2d(const float *bw_in, int H, int W, int C, const float *bw_w, int KH, int KW,
                     int N, int OH, int OW, int stride_h, int stride_w, int dil_h, int dil_w,
                     int pad_top, int pad_left, const float *bw_bias, int64_t n_bias, double out_size,
                     double scale_main, double scale_bias, const float *beta, uint32_t *ebops,
                     float *ebops_f, float *loss, float *d_bw_in, float *d_bw_w, float *d_bw_bias,
                     void *stream);

/* ---- optimizer step ------------------------------------------------------------------------ */

/*
 * Adam over one flat bucket of n fp32 parameters, with the bitwidth regulariser and the variable
 * constraints folded in.  Stands in for what Keras' trainer does after backward for the variables
 * HGQ2 creates: optimizer.apply(grads, trainable_variables) followed by variable.constraint(...)
 * (the constraints of src/hgq/constraints/__init__.py:11-69 are attached at
 * fixed_point_quantizer.py:225-241,382-397), and the gradient of the MonoL1 regulariser
 * (src/hgq/regularizers/__init__.py:8-17).
 *   g' = g * grad_scale + l1;  Keras Adam update with (lr, beta1, beta2, eps);  w = clamp(w, lo, hi)
 * lo / hi / l1 are per-element arrays and may be NULL.  `step` is a device counter (starts at 0)
 * that the call reads for the bias correction and then increments.
 */
int hgq_adam_step(float *w, const float *g, float *m, float *v, const float *lo, const float *hi,
                  const float *l1, int64_t n, float lr, float beta1, float beta2, float eps,
                  float grad_scale, long long *step, void *stream);

/* ---- gradient exchange over peer memory, fused with the optimizer update ------------------------ */

/*
 * The data-parallel tail of a step on one node (one process per GPU) as one kernel per rank: every rank publishes its
 * gradient bucket in a buffer its peers have mapped, waits (bounded) for theirs, adds the buckets in rank order and applies
 * hgq_adam_step's update with grad_scale = 1 / world.  No reference counterpart in the HGQ2 tree: it stands in for the
 * gradient all-reduce of Keras' distribution strategy followed by optimizer.apply (see hgq_adam_step).  Plain peer loads
 * over NVLink; no switch-side reduction, no collective library.
 *
 * hgq_peer_exchange_bytes(n): size of one rank's exchange buffer for a bucket of n floats.
 * hgq_peer_buffer_create: cudaMalloc + zero fill on the current device; writes the 64-byte CUDA IPC handle that the other
 *   processes pass to hgq_peer_buffer_open (which maps the buffer and enables peer access).  close / destroy undo them.
 * hgq_adam_step_peers: peer_bufs is a HOST array of `world` device pointers (entry `rank` = this rank's own buffer, the
 *   others as returned by hgq_peer_buffer_open); every rank must call it once per step with the same n, in the same step
 *   order, each on its own GPU.  max_polls bounds every wait (about 0.1-0.2 us per poll); a wait that runs out sets bit 1
 *   of *status (may be NULL) and leaves that part of the parameters untouched.  `g` is left as it was (the local gradients).
 */
size_t hgq_peer_exchange_bytes(int64_t n);
int hgq_peer_buffer_create(size_t bytes, void **dev_ptr, void *ipc_handle_64);
int hgq_peer_buffer_open(const void *ipc_handle_64, void **dev_ptr);
int hgq_peer_buffer_close(void *dev_ptr);
int hgq_peer_buffer_destroy(void *dev_ptr);
int hgq_adam_step_peers(float *w, const float *g, float *m, float *v, const float *lo, const float *hi,
                        const float *l1, int64_t n, float lr, float beta1, float beta2, float eps, long long *step,
                        void *const *peer_bufs, int world, int rank, unsigned max_polls, unsigned *status, void *stream);

/* ---- batched parameter-side work of a training step ------------------------------------------ */

/*
 * Descriptor tables.  A model's quantizers and weight tensors are described once, in arrays of these structs held in
 * DEVICE memory (all pointers inside are device pointers); each entry point below then handles every quantizer / every
 * weight tensor of the model in one launch.  The reference does the same work as eager element-wise operations on each
 * bitwidth-shaped tensor separately.
 */
#define HGQ_SLOT_KIF 0 /* variables (k, i, f): FixedPointQuantizerKIF, fixed_point_quantizer.py:310-458 */
#define HGQ_SLOT_KBI 1 /* variables (k, b, i): FixedPointQuantizerKBI, fixed_point_quantizer.py:153-307 */

typedef struct hgq_slot_desc {
    const float *a_raw;   /* the variable `f` (KIF) or `b` (KBI), n entries                                   */
    float *i_raw;         /* the variable `i` (trainable, or the tracked state of a WRAP quantizer)           */
    const uint8_t *k;     /* the variable `k`                                                                 */
    float *I, *F, *BITS;  /* derived tables: round_conv(i); round_conv(f) or round_conv(b) - round_conv(i);    */
                          /* the `bits` property (fixed_point_quantizer.py:92-97)                             */
    float *dI, *dF, *dBITS; /* gradients of the loss w.r.t. the three derived tables                          */
    float *g_a, *g_i;     /* where the gradients of a_raw / i_raw go (NULL: not trainable)                    */
    const float *absmax;  /* a tracked activation quantizer: max |round(x, f)| per entry; else NULL           */
    const float *decay;   /* the scalar variable i_decay_speed (WRAP), else NULL                              */
    int64_t n;
    int32_t kind;         /* HGQ_SLOT_KIF / HGQ_SLOT_KBI                                                      */
    int32_t om, rm;       /* hgq_overflow_mode, hgq_round_mode of the quantizer                               */
    int32_t symmetric;    /* overflow mode ends in _SYM                                                       */
    int32_t tracked_weight; /* the weights pass tracks this quantizer's integer bits                          */
    float i_lo, i_hi;     /* MinMax constraint of `i` applied while tracking (KBI; +-inf: none)               */
} hgq_slot_desc;

#define HGQ_WEIGHT_QUANTIZE 0    /* wq = stateless_quantizer(w, k, i, f, training=True)                       */
#define HGQ_WEIGHT_ROUND 1       /* wq = stateless_quantizer.round(w, f)                                      */
#define HGQ_WEIGHT_TRACK_ROUND 2 /* WRAP quantizer in training: track the integer bits, then round            */

typedef struct hgq_weight_desc {
    const float *w_raw;  /* the kernel or bias variable, n entries                                            */
    float *wq;           /* its quantised value                                                               */
    const float *dwq;    /* dL/dwq (written by the layer's backward kernel)                                   */
    float *g_w;          /* where dL/dw goes                                                                  */
    int64_t n;
    int32_t slot;        /* index of the quantizer's hgq_slot_desc; its tables have one entry per weight      */
    int32_t mode;        /* HGQ_WEIGHT_*                                                                      */
} hgq_weight_desc;

/*
 * I = round_conv(i), F = round_conv(f) (KIF) or round_conv(b) - round_conv(i) (KBI) for every slot: the properties
 * `i`, `f` of fixed_point_quantizer.py:244-265,431-449.  max_n = the largest n of any slot.
 */
int hgq_tables_forward(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream);

/*
 * After the forward pass: for every slot with `absmax`, the training branch of FixedPointQuantizerKIF.call
 * (fixed_point_quantizer.py:401-411): i <- max(i - decay, ceil(log2(absmax + 2^-f))); then for every slot
 * BITS = relu(I + F) (KIF) or round_conv(b) (KBI), plus k for overflow mode SAT (fixed_point_quantizer.py:92-97,435-437).
 */
int hgq_tables_track_bits(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream);

/*
 * Backward of the two calls above with straight-through rounding: (dI, dF, dBITS) -> gradients of the raw variables.
 * KIF: g_f = dF + dBITS [i + f > 0], g_i = dI + dBITS [i + f > 0];  KBI: g_b = dF + dBITS, g_i = dI - dF.
 */
int hgq_tables_backward(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream);

/*
 * The quantised kernel / bias of every layer (qkernel / qbias, src/hgq/layers/core/dense.py:93-102 and the like),
 * reading the tables hgq_tables_forward made.  HGQ_WEIGHT_TRACK_ROUND entries also run the integer-bit tracking of
 * FixedPointQuantizerKBI.call / KIF.call in training (fixed_point_quantizer.py:277-288,401-411) on the weight itself.
 */
int hgq_weights_forward(const hgq_weight_desc *weights, int n_weights, int64_t max_n, const hgq_slot_desc *slots,
                        void *stream);

/*
 * Surrogate backward of hgq_weights_forward: g_w = dL/dw, and the slot's dI / dF (one entry per weight) are written.
 */
int hgq_weights_backward(const hgq_weight_desc *weights, int n_weights, int64_t max_n, const hgq_slot_desc *slots,
                         void *stream);

/* ---- a stack of small dense layers in one launch --------------------------------------------- */

#define HGQ_CHAIN_MAX_LAYERS 8

/*
 * One layer of the stack: y = act(round_f(x) @ wq + bq) (QDense.call, src/hgq/layers/core/dense.py:60-68, with the
 * training-mode WRAP input quantizer, which only rounds: fixed_point_quantizer.py:403-424).  1 <= K, N <= 64 and the K of a
 * layer equals the N of the one before.  All pointers are device pointers.
 */
typedef struct {
    int K, N;          /* inputs and outputs */
    int relu;          /* 1: ReLU, 0: no activation */
    int round_mode;    /* HGQ_ROUND_* of the input quantizer */
    const float *qf;   /* [K] fractional bits of the input quantizer (integer-valued) */
    const float *wq;   /* [K, N] quantised kernel */
    const float *bq;   /* [N] quantised bias, or NULL */
    float *y;          /* [M, N] the layer's output: written by the forward, read by the backward */
    float *absmax;     /* forward: [K] abs-max of the rounded inputs, merged by atomic max into what is there
                          (the caller clears it once per step), or NULL */
    float *dwq;        /* backward outputs: [K, N] */
    float *dbq;        /*                   [N] or NULL */
    float *df;         /*                   [K] gradient of the fractional bits, or NULL */
} hgq_chain_layer;

/* 1 when the stack fits the kernels (layer count, widths, shared memory), else 0. */
int hgq_dense_chain_supported(int n_layers, const hgq_chain_layer *layers);

/* Scratch bytes hgq_dense_chain_bwd needs (0 when the stack is not supported). */
size_t hgq_dense_chain_workspace(int64_t M, int n_layers, const hgq_chain_layer *layers);

/*
 * Forward of the whole stack on x [M, K of layer 0] in ONE launch: the activations of a 128-row tile stay in shared memory
 * from layer to layer, every layer's output is also written to its `y`.  `layers` is a host array.  The arithmetic is fp32
 * fused multiply-add on the CUDA cores (layers this small are bound by launch and dependency latencies, not by throughput).
 */
int hgq_dense_chain_fwd(const float *x, int64_t M, int n_layers, const hgq_chain_layer *layers, void *stream);

/*
 * Backward of the stack: gy [M, N of the last layer] is the gradient of its output; x and every layer's `y` are the
 * forward's.  Writes dwq / dbq / df of every layer (the ReLU mask is y > 0) and, when dx != NULL, the gradient of x.
 * Two launches: the stack, then a fixed-order reduction of the per-block partial sums (results do not depend on scheduling).
 */
int hgq_dense_chain_bwd(const float *gy, const float *x, float *dx, int64_t M, int n_layers, const hgq_chain_layer *layers,
                        void *workspace, size_t workspace_bytes, void *stream);

/* ---- standalone quantizer on host buffers ------------------------------------------------- */

/*
 * Device staging bytes hgq_quantize_fwd_bwd_host needs for a given chunk size (elements, a
 * multiple of 4).  The caller allocates that much device memory, 256-byte aligned.
 */
size_t hgq_quantize_host_workspace(int64_t chunk_elems);

/*
 * The same computation as hgq_quantize_fwd followed by hgq_quantize_bwd (full layout), for a
 * caller whose tensors live in host memory -- the situation of the reference's CPU path, where
 * stateless_quantizer (fixed_point_quantizer.py:147) and its gradient run on host tensors.
 * Inputs hx,hk,hi,hf (and hg) are read from host memory, outputs hy (and hdx,hdi,hdf) are written
 * to host memory; pinned memory lets copies and kernels overlap.  hg == NULL runs the forward
 * only; hdi may be NULL.  Synchronous: returns when every output byte has landed.  Uses three
 * internal streams per device, created on first use; not re-entrant on one device.
 */
int hgq_quantize_fwd_bwd_host(const float *hx, const uint8_t *hk, const float *hi, const float *hf,
                              const float *hg, float *hy, float *hdx, float *hdi, float *hdf,
                              int64_t n, int round_mode, int overflow_mode, unsigned flags,
                              void *dev_workspace, size_t dev_workspace_bytes, int64_t chunk_elems);

#ifdef __cplusplus
}
#endif
#endif /* HGQ_B200_H_ */
