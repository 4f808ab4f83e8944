/*
 * cortex_b200 -- C ABI of the B200 (sm_100a) compute backend for cortex's
 * dense-layer hot path.
 *
 * Every entry point mirrors one method of the reference's backend protocols:
 *   - operator boundary:  cortex.tensor.math/TensorMath   (src/cortex/tensor/math.clj:11-252)
 *   - device boundary:    cortex.compute.driver protocols (src/cortex/compute/driver.clj:46-203)
 * The argument order and meaning follow the protocol method named in each
 * comment, so a Clojure (JNA / JavaCPP) shim is a 1:1 forwarder.
 *
 * Conventions
 *   - Every function returns 0 on success, a CB200_ERR_* code otherwise;
 *     cb200_last_error() returns a thread-local message for the last failure.
 *   - Buffers are raw device pointers.  Offsets/sub-buffers are pointer
 *     arithmetic done by the caller (as src/cortex/compute/cuda/driver.clj:465-506).
 *   - Scalars travel as double and are cast to the element type of the
 *     destination before use (drv/dtype-cast, src/cortex/compute/cuda/tensor_math.clj:293).
 *   - Nothing here aborts the process or traps on the device.
 *   - The stream handle carries its device; there is no process-global
 *     "current device / current stream" state and no process-global option:
 *     N host threads x N streams are safe (src/cortex/verify/nn/train.clj:211-236
 *     is the usage model).  One stream is driven by one thread at a time.
 */
#ifndef CORTEX_B200_H
#define CORTEX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enumerations (numbered as the reference's wire format) ------------- */

/* resources/datatypes.h:81-92, src/cortex/compute/cuda/driver.clj:354-367 */
enum cb200_dtype {
  CB200_BYTE = 0, CB200_SHORT = 1, CB200_INT = 2, CB200_LONG = 3,
  CB200_FLOAT = 4, CB200_DOUBLE = 5
};

/* src/cortex/compute/cuda/tensor_math.clj:54-72, resources/operations.h:27-45 */
enum cb200_binary_op {
  CB200_ADD = 0, CB200_SUB = 1, CB200_MUL = 2, CB200_DIV = 3, CB200_MIN = 4,
  CB200_MAX = 5, CB200_BIT_AND = 6, CB200_BIT_XOR = 7, CB200_EQ = 8,
  CB200_GT = 9, CB200_GE = 10, CB200_LT = 11, CB200_LE = 12
};

/* src/cortex/compute/cuda/tensor_math.clj:75-92, resources/operations.h:88-102 */
enum cb200_unary_op {
  CB200_FLOOR = 0, CB200_CEIL = 1, CB200_ROUND = 2, CB200_NEG = 3,
  CB200_TANH = 4, CB200_LOGISTIC = 5, CB200_EXP = 6, CB200_SQRT = 7,
  CB200_NOOP = 8
};

/* src/cortex/compute/cuda/tensor_math.clj:624-630, resources/tensor_unary_reduce.cu:9-20 */
enum cb200_reduce_op {
  CB200_RMAX = 0, CB200_RMIN = 1, CB200_RSUM = 2, CB200_RMEAN = 3,
  CB200_RMAGNITUDE = 4, CB200_RMAGNITUDE_SQ = 5
};

/* epilogue activations of the fused extras (no protocol counterpart) */
enum cb200_act { CB200_ACT_NONE = 0, CB200_ACT_RELU = 1, CB200_ACT_TANH = 2, CB200_ACT_LOGISTIC = 3,
                 /* cb200_gemm_bias_act only: softmax! over every output row after bias (a classifier head).  Rows of
                  * up to 16 columns are normalised by the kernel that computes them, wider ones by a second launch. */
                 CB200_ACT_SOFTMAX = 4 };

enum cb200_status {
  CB200_OK = 0,
  CB200_ERR_INVALID = 1,      /* bad argument / descriptor            */
  CB200_ERR_UNSUPPORTED = 2,  /* protocol method outside the hot path */
  CB200_ERR_CUDA = 3,         /* CUDA runtime / driver error          */
  CB200_ERR_TIMEOUT = 4,      /* a bounded device-side wait ran out   */
  CB200_ERR_NOMEM = 5
};

/* ---- tensor descriptor ---------------------------------------------------
 * Wire format of one operand: what dimensions->cuda builds
 * (src/cortex/compute/cuda/tensor_math.clj:34-51) and what
 * resources/index_system.h:16-41 consumes: shape and strides reversed
 * (fastest-changing dimension first), padded to 5 with shape 1 and the
 * outermost stride, plus one optional int32 index array per dimension
 * (NULL = direct).  When index[d] is set, rev_shape[d] is the number of
 * entries of that index array.                                              */
typedef struct cb200_dims {
  int32_t rev_shape[5];
  int32_t rev_strides[5];
  const int32_t* index[5];
} cb200_dims;

/* convolution-descriptor fields (src/cortex/tensor.clj:1322-1348) */
typedef struct cb200_conv_desc {
  int32_t out_channels, in_channels;
  int32_t kernel_width, kernel_height;
  int32_t pad_x, pad_y;
  int32_t stride_x, stride_y;
} cb200_conv_desc;

typedef struct cb200_stream cb200_stream;  /* device + CUDA stream + status word */
typedef struct cb200_event cb200_event;
typedef struct cb200_graph cb200_graph;  /* a captured launch sequence */

/* ---- errors -------------------------------------------------------------- */
/* check-cuda-error: src/cortex/compute/cuda/driver.clj:40-49 */
const char* cb200_last_error(void);

/* ---- PDriver / PDevice (src/cortex/compute/driver.clj:46-61, 74-84) ------ */
/* get-devices */
int cb200_device_count(int* count);
int cb200_device_info(int device, char* name, int name_len, int* sm_count,
                      int* cc_major, int* cc_minor);
/* memory-info-impl */
int cb200_mem_info(int device, size_t* free_bytes, size_t* total_bytes);
/* create-stream-impl */
int cb200_stream_create(int device, cb200_stream** out);
int cb200_stream_destroy(cb200_stream* s);
/* raw cudaStream_t of the stream (for NCCL / interop), as void* */
void* cb200_stream_native(cb200_stream* s);
int cb200_stream_device(cb200_stream* s);
/* allocate-device-buffer-impl */
int cb200_malloc(int device, size_t bytes, void** out);
int cb200_free(int device, void* ptr);
/* allocate-host-buffer-impl (page-locked: src/cortex/compute/cuda/driver.clj:522-542) */
int cb200_host_alloc(size_t bytes, void** out);
int cb200_host_free(void* ptr);
/* The same page-locked buffer placed on the NUMA node the GPU's PCIe slot hangs off (pages bound and
 * touched before they are pinned), so that uploads to that GPU do not cross the socket interconnect:
 * with one process per GPU, eight uploads otherwise compete for one node's memory channels.  *node
 * gets the node used, or -1 when the platform does not report one (then this is cb200_host_alloc).
 * Staging buffers of the reference: allocate-host-buffer-impl, src/cortex/compute/cuda/driver.clj:522-542;
 * the upload path they feed: src/cortex/nn/execute.clj:387-434.  Free with cb200_host_free. */
int cb200_host_alloc_near(int device, size_t bytes, void** out, int* node);
int cb200_device_numa_node(int device, int* node);

/* ---- PStream / PEvent (src/cortex/compute/driver.clj:180-203) ------------ */
/* copy-host->device / copy-device->host / copy-device->device (sizes in bytes) */
int cb200_memcpy_h2d(cb200_stream* s, void* dst_dev, const void* src_host, size_t bytes);
int cb200_memcpy_d2h(cb200_stream* s, void* dst_host, const void* src_dev, size_t bytes);
int cb200_memcpy_d2d(cb200_stream* s, void* dst_dev, const void* src_dev, size_t bytes);
/* memset [stream device-buffer device-offset elem-val elem-count] */
int cb200_memset(cb200_stream* s, int dtype, void* buf, int64_t elem_offset,
                 double value, int64_t n_elems);
/* create-event: records an event on the stream.  timing != 0 keeps timestamps
 * (the reference creates its events with cudaEventDisableTiming,
 * src/cortex/compute/cuda/driver.clj:935-940; timing is an addition). */
int cb200_event_record(cb200_stream* s, int timing, cb200_event** out);
/* sync-event: make `s` wait for the event */
int cb200_stream_wait_event(cb200_stream* s, cb200_event* e);
/* wait-for-event: block the host; also surfaces asynchronous kernel errors
 * (CUDA errors and bounded-wait timeouts recorded in the stream's status word) */
int cb200_event_wait(cb200_event* e);
int cb200_event_elapsed_ms(cb200_event* start, cb200_event* stop, float* ms);
int cb200_event_destroy(cb200_event* e);
/* sync-stream (driver.clj:206-211) */
int cb200_stream_sync(cb200_stream* s);

/* ---- TensorMath (src/cortex/tensor/math.clj) ------------------------------ */
/* assign-constant! :14 */
int cb200_assign_constant(cb200_stream* s, int dtype, void* buf, const cb200_dims* dims,
                          double value, int64_t n_elems);
/* assign! :16-24 (marshals between any two dtypes) */
int cb200_assign(cb200_stream* s, int dest_dtype, void* dest, const cb200_dims* dest_dims,
                 int src_dtype, const void* src, const cb200_dims* src_dims, int64_t n_elems);
/* unary-accum! :26-28   dest = op(alpha*dest) */
int cb200_unary_accum(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                      double alpha, int op, int64_t n_elems);
/* unary-op! :30-33      dest = op(alpha*x) */
int cb200_unary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                   const void* x, const cb200_dims* x_dims, double alpha, int op, int64_t n_elems);
/* binary-accum-constant! :35-40   dest = (alpha*dest) op scalar   (reversed when rev_ops) */
int cb200_binary_accum_constant(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                                double dest_alpha, double scalar, int64_t n_elems, int op, int rev_ops);
/* binary-op-constant! :42-48      dest = (alpha*x) op scalar */
int cb200_binary_op_constant(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                             const void* x, const cb200_dims* x_dims, double x_alpha,
                             double scalar, int64_t n_elems, int op, int rev_ops);
/* binary-accum! :50-61            dest = (alpha*dest) op (beta*y); requires_cas when several
 * element indexes land on one dest address (dest smaller than the op, or indexed) */
int cb200_binary_accum(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                       double dest_alpha, const void* y, const cb200_dims* y_dims, double y_alpha,
                       int64_t n_elems, int op, int rev_ops, int requires_cas);
/* binary-op! :63-69               dest = (alpha*x) op (beta*y) */
int cb200_binary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                    const void* x, const cb200_dims* x_dims, double x_alpha,
                    const void* y, const cb200_dims* y_dims, double y_alpha,
                    int64_t n_elems, int op);
/* unary-reduce! :100-104          out[..., 0] = reduce_j (alpha * in[..., j]) */
int cb200_unary_reduce(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                       double alpha, const void* in, const cb200_dims* in_dims, int op);
/* gemm! :106-115   C = alpha*op(A)*op(B) + beta*C, row-major, ld* = row pitch in elements.
 * a_rows/a_cols are those of op(A) (M, K); b_cols is that of op(B) (N). float and double only. */
int cb200_gemm(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b,
               double alpha, const void* A, int64_t a_rows, int64_t a_cols, int64_t lda,
               const void* B, int64_t b_cols, int64_t ldb, double beta);
/* softmax-eltwise! :177-179 / softmax-spatial! :181-183 */
int cb200_softmax_eltwise(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                          const void* in, const cb200_dims* in_dims);
int cb200_softmax_spatial(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                          const void* in, const cb200_dims* in_dims);
/* choose-convolution-algorithms :191-195 -> workspace element count (this backend needs none
 * and reports 1 so that callers can still allocate a non-empty tensor) */
int cb200_convolution_workspace_size(const cb200_conv_desc* desc, int in_w, int in_h,
                                     int out_w, int out_h, int batch, int64_t* n_elems);
/* convolution-forward! :197-203   NCHW cross-correlation:
 * out = conv(in, w) + out_alpha * out ; workspace may be NULL */
int cb200_convolution_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                              double out_alpha, const void* in, const cb200_dims* in_dims,
                              const void* w, const cb200_dims* w_dims,
                              void* workspace, int64_t workspace_ecount,
                              const cb200_conv_desc* desc);

/* convolution-backward-weights! / convolution-backward-data! (src/cortex/tensor.clj:1469-1493;
 * src/cortex/tensor/math.clj; CPU semantics src/cortex/compute/cpu/tensor_math.clj:1716-1800):
 *   w_grad[C_out, C_in*kH*kW] = w_grad_alpha * w_grad + sum_n out_grad_n[C_out, hw] . unrolled(in_n)[hw, K]
 *   in_grad[N, C_in, H, W]    = in_grad_alpha * in_grad + roll(out_grad_n^T . w)
 * (the CPU backend treats in_grad_alpha as 0 whatever is passed; the layers pass 0).  All tensors dense NCHW /
 * [C_out, K]; float / double; the caller's workspace is not used (the unrolled matrix lives in the stream's own). */
int cb200_convolution_backward_weights(cb200_stream* s, int dtype, void* w_grad, const cb200_dims* w_grad_dims,
                                       double w_grad_alpha, const void* out_grad, const cb200_dims* out_grad_dims,
                                       const void* in, const cb200_dims* in_dims,
                                       void* workspace, int64_t workspace_ecount, const cb200_conv_desc* desc);
int cb200_convolution_backward_data(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims,
                                    double in_grad_alpha, const void* out_grad, const cb200_dims* out_grad_dims,
                                    const void* w, const cb200_dims* w_dims,
                                    void* workspace, int64_t workspace_ecount, const cb200_conv_desc* desc);

/* convolution-forward! without any allocation.  No counterpart in the reference: cortex's backends
 * take a caller-provided workspace tensor instead.  For hosts that cannot call cudaMalloc on this
 * path (all device memory owned by their own pool, or no tolerance for the device-wide
 * synchronisation an allocation implies): the unrolled input lives in a fixed 64 MiB device array
 * that is part of the library image (one per GPU that loads the library, held until exit).
 * Problems whose unrolled matrix batch*outH*outW x roundup4(C_in*kH*kW) elements exceeds 64 MiB are
 * rejected with CB200_ERR_INVALID.  The first call on a device resolves the array's address - make
 * it before any stream capture.  All calls share the array: calls that overlap on the GPU race. */
int cb200_convolution_forward_static(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                                     double out_alpha, const void* in, const cb200_dims* in_dims,
                                     const void* w, const cb200_dims* w_dims, const cb200_conv_desc* desc);

/* Fused extra (no counterpart in the protocol): what ConvolutionLayer.forward + the following ActivationLayer issue
 * as three calls (src/cortex/compute/nn/layers.clj:300-318, 91-103) in the convolution's own epilogue:
 *   out = act(conv(in, w) + out_alpha * out + bias[channel])    bias: [C_out] or NULL; act: enum cb200_act (no softmax)
 * fp32: bias and activation join the epilogue of whichever tensor-core kernel runs the layer (bit-identical to
 * the three calls for no activation / ReLU); fp64: one more pass over the output. */
int cb200_convolution_forward_bias_act(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                                       double out_alpha, const void* in, const cb200_dims* in_dims,
                                       const void* w, const cb200_dims* w_dims, const cb200_conv_desc* desc,
                                       const void* bias, int act);

/* ---- next to the path: ternary-op! family and gemv! ---------------------------
 * ternary-op! / ternary-op-constant! / ternary-op-constant-constant!
 * (src/cortex/tensor/math.clj:71-98; CPU semantics src/cortex/compute/cpu/tensor_math.clj:465-566):
 *   dest = select(alpha*x, beta*y, gamma*z) = (alpha*x >= 0) ? gamma*z : beta*y
 * One entry point serves the three protocol methods: an operand that is a constant has a NULL
 * pointer (and NULL dims) and its scalar holds value * factor, as the reference's
 * order-ternary-args computes it (src/cortex/tensor.clj:792-805); the binding re-expands arg-order. */
enum cb200_ternary_op_t { CB200_TERNARY_SELECT = 0 };
int cb200_ternary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                     const void* x, const cb200_dims* x_dims, double alpha,
                     const void* y, const cb200_dims* y_dims, double beta,
                     const void* z, const cb200_dims* z_dims, double gamma, int64_t n_elems, int op);
/* activation-gradient! (src/cortex/tensor.clj:1256-1283 -> tm/activation-gradient!; CPU semantics
 * src/cortex/compute/cpu/tensor_math.clj:1318-1363; CUDA reference cudnnActivationBackward):
 *   logistic: in_grad = out * (1 - out) * out_grad;  tanh: (1 - out*out) * out_grad;  relu: (out > 0) * out_grad.
 * float / double; float views are computed in double and rounded once (bit-identical to the CPU backend).
 * act: CB200_ACT_RELU / CB200_ACT_TANH / CB200_ACT_LOGISTIC.  in_grad may alias out_grad or out. */
int cb200_activation_gradient(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims,
                              const void* out_grad, const cb200_dims* out_grad_dims,
                              const void* out, const cb200_dims* out_dims, int act, int64_t n_elems);
/* gemv! (src/cortex/tensor/math.clj:116-124, cublasSgemv/Dgemv at src/cortex/compute/cuda/tensor_math.clj:155-173):
 *   c = alpha * op(A) * x + beta * c;  A: a_rows x a_cols row-major with row pitch lda (elements);
 *   trans_a: op(A) = A^T (c then has a_cols entries, x has a_rows); inc_c / inc_x in elements. */
int cb200_gemv(cb200_stream* s, int dtype, void* c, int64_t inc_c, int trans_a, double alpha,
               const void* A, int64_t a_rows, int64_t a_cols, int64_t lda,
               const void* x, int64_t inc_x, double beta);

/* batch-normalize-eltwise! / batch-normalize-spatial! (inference form; src/cortex/tensor/math.clj:125-148,
 * cudnnBatchNormalizationForwardInference at src/cortex/compute/cuda/tensor_math.clj:662-730):
 *   output = (input - mean[c]) * sqrt(1 / (variance[c] + epsilon)) * scale[c] + bias[c]
 * dense buffers; eltwise: input [batch_count, element_count], c = column; spatial: input
 * [batch_count, channel_count, element_count], c = channel.  Uses channel_count elements of stream scratch. */
int cb200_batch_normalize_eltwise(cb200_stream* s, int dtype, void* output, const void* input, const void* means,
                                  const void* variances, const void* scale, const void* bias, double epsilon,
                                  int64_t batch_count, int64_t element_count);
int cb200_batch_normalize_spatial(cb200_stream* s, int dtype, void* output, const void* input, const void* means,
                                  const void* variances, const void* scale, const void* bias, double epsilon,
                                  int64_t batch_count, int64_t channel_count, int64_t element_count);

/* pooling-forward! (src/cortex/tensor/math.clj:205-222; cudnnPoolingForward at
 * src/cortex/compute/cuda/tensor_math.clj:1096-1160).  NCHW dense tensors [batch, channels, h, w]; the output
 * extent is the output tensor's (the caller applies the descriptor's :floor / :ceil rule).  Padding reads 0 and
 * takes part in the maximum, as in the reference CPU backend.  output = result + output_alpha * output. */
enum cb200_pool_op_t { CB200_POOL_MAX = 0, CB200_POOL_AVG = 1, CB200_POOL_AVG_EXC_PAD = 2 };
typedef struct cb200_pool_desc {
  int32_t kernel_width, kernel_height, pad_x, pad_y, stride_x, stride_y, pool_op;
} cb200_pool_desc;
int cb200_pooling_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                          const void* in, const cb200_dims* in_dims, const cb200_pool_desc* desc);

/* pooling-backward! (src/cortex/tensor/math.clj:223-236; cudnnPoolingBackward at
 * src/cortex/compute/cuda/tensor_math.clj:1201-1235; arithmetic after the CPU backend,
 * src/cortex/compute/cpu/tensor_math.clj:1175-1284).  NCHW dense tensors; `in` / `out` are the tensors of the
 * forward call, `out_grad` has the shape of `out`, `in_grad` the shape of `in`.
 *   max:         every input position equal to its window's output receives that window's output gradient;
 *   avg:         output gradient / (kernel_width * kernel_height) to every position of the window inside the image;
 *   avg-exc-pad: the same with the number of window positions inside the image as divisor.
 *   in_grad = in_grad_alpha * in_grad + sum of contributions, summed in the reference's visiting order with every
 *   partial sum rounded to the element type (bit-identical to the CPU backend, which always accumulates onto the
 *   buffer it is given: in_grad_alpha = 1 on that buffer, or 0 on a zeroed one, reproduces it). */
int cb200_pooling_backward(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims, double in_grad_alpha,
                           const void* in, const cb200_dims* in_dims, const void* out, const cb200_dims* out_dims,
                           const void* out_grad, const cb200_dims* out_grad_dims, const cb200_pool_desc* desc);

/* batch-normalize-update-and-apply-eltwise! / -spatial! (src/cortex/tensor/math.clj:137-158;
 * cudnnBatchNormalizationForwardTraining at src/cortex/compute/cuda/tensor_math.clj:727-775; arithmetic after
 * src/cortex/compute/cpu/tensor_math.clj:820-900).  Per channel c over N = batch_count (* element_count) values:
 *   batch_means[c]       = sum(x) / N                      batch_variances[c] = sum((mean - x)^2) / N
 *   running_means[c]     = running_means[c] * (1 - f) + batch_means[c] * f
 *   running_variances[c] = running_variances[c] * (1 - f) + (sum((mean - x)^2) / max(1, N - 1)) * f
 * then output = batch-normalize of input with the batch statistics (the inference call above).  batch_variances
 * holds plain variances (the reference's CUDA backend stores cudnn's 1/sqrt form there; the CPU backend, followed
 * here, stores the variance).  Sums are carried in double. */
int cb200_batch_normalize_update_and_apply_eltwise(cb200_stream* s, int dtype, void* output, const void* input,
                                                   void* batch_means, void* batch_variances, void* running_means,
                                                   void* running_variances, double average_factor, const void* scale,
                                                   const void* bias, double epsilon, int64_t batch_count,
                                                   int64_t element_count);
int cb200_batch_normalize_update_and_apply_spatial(cb200_stream* s, int dtype, void* output, const void* input,
                                                   void* batch_means, void* batch_variances, void* running_means,
                                                   void* running_variances, double average_factor, const void* scale,
                                                   const void* bias, double epsilon, int64_t batch_count,
                                                   int64_t channel_count, int64_t element_count);

/* batch-normalize-gradients-eltwise! / -spatial! (src/cortex/tensor/math.clj:159-174;
 * cudnnBatchNormalizationBackward at src/cortex/compute/cuda/tensor_math.clj:790-850; arithmetic after
 * src/cortex/compute/cpu/tensor_math.clj:903-1032).  batch_means / batch_variances are what update-and-apply
 * wrote.  With inv_std = 1 / sqrt(variance + epsilon), d = scale * output_gradient, xc = input - mean:
 *   bias_gradient[c]  = sum(output_gradient)          scale_gradient[c] = sum(output_gradient * xc * inv_std)
 *   d_var  = sum(d * xc * (-0.5 * (variance + epsilon)^(-3/2)))
 *   d_mean = sum(-d * inv_std) + d_var * sum(-2 * xc) / N
 *   input_gradient = d * inv_std + d_var * 2 * xc / N + d_mean / N
 * `output` and `bias` are part of the protocol signature and are not read. */
int cb200_batch_normalize_gradients_eltwise(cb200_stream* s, int dtype, void* input_gradient, void* scale_gradient,
                                            void* bias_gradient, const void* output_gradient, const void* output,
                                            const void* input, const void* batch_means, const void* batch_variances,
                                            const void* scale, const void* bias, double epsilon, int64_t batch_count,
                                            int64_t element_count);
int cb200_batch_normalize_gradients_spatial(cb200_stream* s, int dtype, void* input_gradient, void* scale_gradient,
                                            void* bias_gradient, const void* output_gradient, const void* output,
                                            const void* input, const void* batch_means, const void* batch_variances,
                                            const void* scale, const void* bias, double epsilon, int64_t batch_count,
                                            int64_t channel_count, int64_t element_count);

/* ---- optimiser steps and rand! (the ring of the training path that touches the flat parameter buffer) ----
 * adam_step: resources/adam.cu:1-36 (the kernel this replaces), src/cortex/optimize/adam.clj:68-102 (CPU
 * arithmetic: double buffers follow it bit for bit, float buffers are evaluated in single precision like the
 * reference's CUDA kernel) and :123-142 (call site: scalars cast to the buffer type; m and v arrive already
 * offset by the parameter offset).  One pass:
 *   g = gradient_alpha*grad;  m = beta1*m + (1-beta1)*g;  v = beta2*v + (1-beta2)*g*g;
 *   param -= alpha * (m / ((1 - pow_beta1_t) * (sqrt(v / (1 - pow_beta2_t)) + epsilon)))        float / double */
int cb200_adam_step(cb200_stream* s, int dtype, double alpha, double beta1, double beta2, double epsilon,
                    double pow_beta1_t, double pow_beta2_t, double gradient_alpha, const void* gradients,
                    void* parameters, void* m, void* v, int64_t n_elems);
/* adadelta_step: resources/adadelta.cu:1-68 (argument order kept), CPU arithmetic
 * java/cortex/compute/optimize/AdadeltaOptimizer.java; call site src/cortex/optimize/adadelta.clj:27-75.
 *   g = gradient_beta*grad;  ga = g*g*decay + ga*(1-decay);  dx = -sqrt(dxa + eps) * g / sqrt(ga + eps);
 *   dxa = dx*dx*decay + dxa*(1-decay);  param += dx                                           float / double */
int cb200_adadelta_step(cb200_stream* s, int dtype, double decay, double epsilon, void* grad_accum, void* dx_accum,
                        double gradient_beta, const void* gradient, void* parameters, int64_t n_elems);
/* rand! (src/cortex/tensor/math.clj:237; distributions src/cortex/tensor.clj:990-1012): float, dense dest.
 *   CB200_RAND_FLAT:     p0 = minimum, p1 = maximum,  dest in [minimum, maximum)
 *   CB200_RAND_GAUSSIAN: p0 = mean,    p1 = variance
 * The protocol carries no seed (the reference draws from SecureRandom / cuRAND's global generator); here the
 * generator is counter-based, so the caller supplies (seed, sequence): the same pair reproduces the same
 * values, a different sequence number gives an independent stream. */
enum cb200_distribution { CB200_RAND_FLAT = 0, CB200_RAND_GAUSSIAN = 1 };
int cb200_rand(cb200_stream* s, void* dest, const cb200_dims* dest_dims, int distribution, double p0, double p1,
               uint64_t seed, uint64_t sequence);

/* lrn-forward! / lrn-backward! (src/cortex/tensor/math.clj:240-252; cudnnLRNCrossChannelForward / Backward at
 * src/cortex/compute/cuda/tensor_math.clj:1277-1335; descriptor defaults src/cortex/tensor.clj:1553-1560).
 * Dense tensors [.., channels, height, width] of rank 3 to 5, all of one shape.  With
 * W(c) = [c - (n-1)/2, c + n - 1 - (n-1)/2] (integer division, clipped) and s(c) = k + (alpha/n) * sum_{W(c)} x^2:
 *   forward:  y = x * s^-beta;   backward:  dx = dy * s^-beta - (2*alpha*beta/n) * x * sum_{j in W(c)} dy_j*y_j/s(j).
 * Float tensors are evaluated in single precision.  The backward call uses one element of stream scratch per element. */
typedef struct cb200_lrn_desc { int32_t n; double k, alpha, beta; } cb200_lrn_desc;
int cb200_lrn_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, const void* in,
                      const cb200_dims* in_dims, const cb200_lrn_desc* desc);
int cb200_lrn_backward(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims, const void* out,
                       const cb200_dims* out_dims, const void* in, const cb200_dims* in_dims, const void* out_grad,
                       const cb200_dims* out_grad_dims, const cb200_lrn_desc* desc);

/* Every method of the protocol (src/cortex/tensor/math.clj) has an entry point above.  This call reports a method
 * name as CB200_ERR_UNSUPPORTED; bindings use it for calls outside the protocol. */
int cb200_unsupported(const char* method_name);

/* ---- fused extras (no counterpart in the protocol) -------------------------
 * What nn-backend/biased-multiply! + the following ActivationLayer issue as three
 * calls (src/cortex/compute/nn/backend.clj:98-112, src/cortex/compute/nn/layers.clj:91-103):
 *   C = act(alpha*op(A)*op(B) + beta*C + bias)   bias: [N] broadcast over rows, or NULL */
int cb200_gemm_bias_act(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b,
                        double alpha, const void* A, int64_t a_rows, int64_t a_cols, int64_t lda,
                        const void* B, int64_t b_cols, int64_t ldb, double beta,
                        const void* bias, int act);
/* ---- launch-sequence capture (no counterpart in the protocol) ----------------
 * Small batches are launch-bound (the MNIST-shaped 128-row forward is three kernels of a few
 * microseconds each): everything enqueued on `s` by this library between capture_begin and
 * capture_end is recorded instead of run, and replayed by ONE cb200_graph_launch.  Rules: run the
 * sequence once normally first (scratch buffers and kernel attributes are set up on first use and
 * must not be created while capturing: a call that would have to grow them returns CB200_ERR_INVALID);
 * no sync / event_wait / malloc / free between begin and end; the graph replays the same buffers, shapes
 * and scalars; destroy it before freeing those buffers and before destroying the stream it was captured
 * on.  The graph also replays the stream's internal workspace addresses: while a graph captured on a
 * stream is alive, a workspace that has to grow is replaced without freeing the old block (it is released
 * with the stream), so earlier graphs stay valid. */
int cb200_graph_capture_begin(cb200_stream* s);
int cb200_graph_capture_end(cb200_stream* s, cb200_graph** out);
int cb200_graph_launch(cb200_graph* g, cb200_stream* s);
int cb200_graph_destroy(cb200_graph* g);

/* ---- multi-GPU extras (no counterpart: the reference has no multi-device code, README.md:48) ----
 * The same fused GEMM whose epilogue ALSO stores every finished tile of the C window to the same
 * row-major position (row*ldc + column from the given base) of up to 7 more buffers, typically the
 * matching column window of the full output on every other GPU: a column-sharded layer then needs no
 * separate all-gather, the transfer overlaps the math tile by tile (plain peer stores over NVLink).
 * peer_C[d] must be addressable from the stream's device (cb200_peer_enable in one process, or a
 * pointer from cb200_ipc_import across processes), have the pitch ldc, and be 16-byte aligned like C
 * for the vector store path.  The caller orders the readers: the stores are complete when the
 * stream reaches the point after this call (event / stream sync, then its own cross-GPU barrier). */
#define CB200_MAX_PEERS 7
int cb200_gemm_bias_act_peers(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b,
                              double alpha, const void* A, int64_t a_rows, int64_t a_cols, int64_t lda,
                              const void* B, int64_t b_cols, int64_t ldb, double beta,
                              const void* bias, int act, int n_peers, void* const* peer_C);
/* One process driving several GPUs: let `device` address `peer_device`'s memory. */
int cb200_peer_enable(int device, int peer_device);
/* One process per GPU: export a cb200_malloc'ed buffer as a 64-byte CUDA IPC handle; another
 * process imports it on its own device (lazy peer access) and closes it when done. */
#define CB200_IPC_HANDLE_BYTES 64
int cb200_ipc_export(int device, void* device_ptr, unsigned char* handle_out);
int cb200_ipc_import(int device, const unsigned char* handle, void** ptr_out);
int cb200_ipc_close(int device, void* ptr);

/* ---- pre-split layer GEMM (no counterpart in the protocol) ----------------------
 * The 3xTF32 GEMM splits every fp32 operand into hi (the value itself) and lo = x - trunc_tf32(x).  In a
 * stack of layers the weights' lo matrix can be computed once and an activation's lo matrix by the layer
 * that produces it; this entry point takes both operands already split and can write its result split:
 *   C = act(alpha * A * B^T + beta * C + bias),  C_lo = C - trunc_tf32(C)   (C_lo may be NULL)
 * A_hi / A_lo: [a_rows, a_cols] row-major, pitch lda; B_hi / B_lo: [b_rows, a_cols] row-major, pitch ldb
 * (the :linear layout: weights [out, in]); C / C_lo: [a_rows, b_rows], pitch ldc.  fp32 only; operands
 * 16-byte aligned, pitches multiples of 4.  cb200_split_lo computes lo for a dense span (inputs, weights). */
int cb200_split_lo(cb200_stream* s, void* lo, const void* x, int64_t n_elems);
int cb200_gemm_bias_act_presplit(cb200_stream* s, void* C, void* C_lo, int64_t ldc, double alpha,
                                 const void* A_hi, const void* A_lo, int64_t a_rows, int64_t a_cols, int64_t lda,
                                 const void* B_hi, const void* B_lo, int64_t b_rows, int64_t ldb, double beta,
                                 const void* bias, int act);

/* One pass over X[rows, cols] (pitch ldx): Y = max(X + bias, 0), rowmax[r] = max_j Y[r,j],
 * rowsum[r] = sum_j Y[r,j].  float/double.  Y may alias X; rowmax/rowsum may be NULL. */
int cb200_bias_relu_rowstats(cb200_stream* s, int dtype, void* Y, int64_t ldy, const void* X,
                             int64_t ldx, const void* bias, int64_t rows, int64_t cols,
                             void* rowmax, void* rowsum);

/* ---- diagnostics (no counterpart in the protocol) -----------------------------------
 * Per-stream options; nothing here is process-global.  They exist so that every kernel behind one entry
 * point can be parity-tested at sizes the automatic choice would route elsewhere, and so that the
 * bounded device-side waits can be made to run out without faulting the GPU. */
enum cb200_stream_option {
  CB200_OPT_GEMM_AUTO_PRESPLIT = 0, /* gemm!: 0 = split-into-workspace + CTA-pair kernel by problem size,
                                       1 = never, 2 = whenever TMA can address the operands */
  CB200_OPT_PRESPLIT_VARIANT = 1,   /* gemm_bias_act_presplit: 0 = by size, 1 = single-CTA tiles, 2 = CTA pairs */
  CB200_OPT_F64_SIMPLE_KERNEL = 2,  /* fp64 gemm!: 1 = always the register-staged kernel */
  CB200_OPT_WAIT_LIMIT_CYCLES = 3,  /* limit of every bounded device-side wait, in SM cycles (0 = default, ~2 s) */
  CB200_OPT_CONV_ROUTE = 5,         /* fp32 convolution-forward!: 0 = by geometry (TMA-fed kernels for stride-1 layers
                                       with a multiple of 16 input channels), 1 = always the thread-gathered kernel,
                                       2 = the TMA kernel that loads one tile per filter tap, never the one that
                                       keeps the input patch in shared memory, 3 = by geometry, but the patch
                                       kernel always behind its layout pre-pass (never the variant that reads
                                       the NCHW input itself) */
  CB200_OPT_GEMM_K_SLICES = 6,      /* fp32 tensor-core gemm! on problems whose tiles leave SMs free: CTAs per tile, each
                                       over a slice of K: 0 = chosen with the tile width by a timing model, 1 = never
                                       slice, n <= 16 = n slices when K has at least 8 k-blocks per slice */
  CB200_OPT_GEMM_TILE_N = 7,        /* fp32 tensor-core gemm!: output tile width, 0 = by size, else 64, 128 or 256 */
  CB200_OPT_GEMM_SLICE_HANDOVER = 8, /* K-sliced fp32 gemm!: 0 = up to 8 slices meet in distributed shared memory (the
                                       slices of a tile are one thread-block cluster), more through L2; 1 = always L2 */
  CB200_OPT_INJECT_FAULT = 4        /* bit 0: the TMA producers of the fp32 tensor-core GEMM issue no loads, so
                                       the consumers' waits run out -> CB200_ERR_TIMEOUT from cb200_stream_sync.
                                       The failure is made on the host side of the barrier protocol; the kernel
                                       unwinds through its normal abort path (no trap, no bad address). */
};
int cb200_stream_set_option(cb200_stream* s, int option, int64_t value);
/* bytes of the stream's workspace, blocks retired because a live graph may still replay them, live graphs */
int cb200_stream_workspace_info(cb200_stream* s, size_t* workspace_bytes, int* retired_blocks, int* live_graphs);
/* One fp32 gemm! on a named kernel: which = 0 the SIMT kernel, 1 the tcgen05 kernel with `flags`
 * (1 = single tf32 term: no hi/lo split, which exposes how the tensor core reads an fp32 word). */
int cb200_gemm_f32_variant(cb200_stream* s, int which, int flags, void* C, int64_t ldc, int trans_a, int trans_b,
                           double alpha, const void* A, int64_t a_rows, int64_t a_cols, int64_t lda, const void* B,
                           int64_t b_cols, int64_t ldb, double beta);

/* number of kernels this library has launched on the stream since creation */
int64_t cb200_launch_count(cb200_stream* s);
/* read and clear the stream's device-side status word (0 = clean) */
int cb200_stream_status(cb200_stream* s, int* code, int* detail);

#ifdef __cplusplus
}
#endif
#endif /* CORTEX_B200_H */
