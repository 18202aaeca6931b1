/*
 * b2c -- C ABI of the B200 convolution / FC back end.
 *
 * Every entry point takes raw device pointers, plain integers and a CUDA stream handle
 * (passed as void*, i.e. a cudaStream_t; NULL = the default stream).  Calls only enqueue
 * work on that stream: no allocation, no implicit device synchronisation, no ownership of
 * caller memory.  The return value is B2C_OK (0) or a negative b2c_status; nothing aborts,
 * throws across the boundary or traps the device.  b2c_status_string() names a status.
 *
 * The citations name the interface of the reference project each entry replaces
 * (paths relative to that project's root).
 */
#ifndef B2C_H
#define B2C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b2c_status {
    B2C_OK = 0,
    B2C_ERR_NULL_POINTER = -1,
    B2C_ERR_BAD_GEOMETRY = -2,     /* non-positive size, empty output, stride/dilation < 1 */
    B2C_ERR_BAD_ENUM = -3,         /* layout / dtype / weight layout / pass out of range */
    B2C_ERR_WORKSPACE_TOO_SMALL = -4,
    B2C_ERR_MISALIGNED = -5,
    B2C_ERR_UNSUPPORTED = -6,      /* shape outside what the requested engine handles */
    B2C_ERR_CUDA = -7,             /* launch failed; see b2c_last_cuda_error() */
    B2C_ERR_TOO_LARGE = -8,        /* size exceeds a fixed capacity of the entry point */
    B2C_ERR_DEVICE_TIMEOUT = -9    /* a bounded in-kernel wait ran out (status word set) */
} b2c_status;

enum { B2C_LAYOUT_NHWC = 0, B2C_LAYOUT_NCHW = 1 };
enum { B2C_F32 = 0, B2C_F64 = 1 };
/* Filter tensor layouts:
 *   CRSK (ci,kh,kw,co)  reference CPU back end, NHWC   pydtnn/layers/conv_2d.py:73-74
 *   KCRS (co,ci,kh,kw)  both back ends, NCHW            pydtnn/layers/conv_2d.py:71-72
 *   KRSC (co,kh,kw,ci)  reference GPU back end, NHWC    pydtnn/backends/gpu/layers/conv_2d_gpu.py:49-51 */
enum { B2C_W_CRSK = 0, B2C_W_KCRS = 1, B2C_W_KRSC = 2 };
enum { B2C_PASS_FPROP = 0, B2C_PASS_DGRAD = 1, B2C_PASS_WGRAD = 2 };
/* Engine selection: AUTO picks the tensor-core kernels when the shape qualifies and the
 * generic FMA kernels otherwise; the other two force one engine (UNSUPPORTED if it cannot). */
enum { B2C_ENGINE_AUTO = 0, B2C_ENGINE_FMA = 1, B2C_ENGINE_TENSOR = 2 };

/* Geometry of one Conv2D layer: the fields of pydtnn/layers/conv_2d.py:31-78, i.e. the
 * argument list of the reference's convolution FFI (b,h,w,c,kn,kh,kw,vpad,hpad,vstr,hstr,
 * vdil,hdil -- pydtnn/backends/cpu/libs/conv_gemm.py:234-248) plus layout/dtype. */
typedef struct b2c_conv_desc {
    int32_t layout;      /* B2C_LAYOUT_* of x, y, dx, dy */
    int32_t dtype;       /* B2C_F32 / B2C_F64 */
    int32_t w_layout;    /* B2C_W_* of w and dw */
    int32_t engine;      /* B2C_ENGINE_* */
    int32_t n, h, w, ci; /* input batch, height, width, channels */
    int32_t co, kh, kw;  /* filters, filter height, width */
    int32_t vpad, hpad, vstr, hstr, vdil, hdil;
} b2c_conv_desc;

/* Per-channel vectors (length co) of the fused inference epilogue
 *   y = relu?( ((conv + bias) - mean) * inv_std * gamma + beta )
 * argument order and arithmetic of pydtnn/backends/cpu/libs/conv_gemm.py:234-248 (bn_mean,
 * bn_inv_std, bn_gamma, bn_beta, relu) and pydtnn/cython_modules/bn_inference_cython.pyx:71-72. */
typedef struct b2c_bn_params {
    const void *mean, *inv_std, *gamma, *beta;
} b2c_bn_params;

const char *b2c_status_string(int status);
const char *b2c_last_cuda_error(void);
int b2c_version(void);
/* Number of kernels this library has launched in the process so far (diagnostic; lets a caller
 * state how many of its launches fall inside a timed region). No counterpart in the reference. */
uint64_t b2c_launch_count(void);

/* Reads and clears the status word the tensor-core kernels set when one of their bounded in-kernel
 * waits runs out (the kernel then skips its remaining work and returns; the context stays usable).
 * Synchronises with the device. Returns B2C_OK or B2C_ERR_DEVICE_TIMEOUT; *detail (may be NULL)
 * receives the raw code. The reference has no counterpart (cuDNN reports through its status). */
int b2c_check_device_status(int *detail);

/* Launches one warp that waits, for at most limit_cycles SM clock cycles (1 .. 2e9), on a barrier nothing arrives
 * at: the wait runs out, the status word is set (detail 7) and the kernel returns.  Lets a host check, on a healthy
 * device, that a timed-out wait is reported by b2c_check_device_status and leaves the context usable. */
int b2c_selftest_bounded_wait(int64_t limit_cycles, void *stream);

/* Scratch bytes a pass needs for this geometry (0 = none).
 * Replaces the process-global cuDNN workspace sizing, pydtnn/backends/gpu/layers/memory_allocation.py:28-49
 * and ConvGemm's pack buffers, pydtnn/backends/cpu/libs/conv_gemm.py:88-94. */
size_t b2c_conv_workspace_bytes(const b2c_conv_desc *desc, int pass);
/* Which engine (B2C_ENGINE_FMA / B2C_ENGINE_TENSOR) a pass would run on; negative = error. */
int b2c_conv_engine_for(const b2c_conv_desc *desc, int pass);

/* y = relu?(bn?(conv(x, w) + bias)); bias, bn may be NULL.
 * Replaces cudnnConvolutionForward + cudnnAddTensor, pydtnn/backends/gpu/layers/conv_2d_gpu.py:170-190,
 * and sconvGemmNHWC/NCHW with trans='N', pydtnn/backends/cpu/libs/conv_gemm.py:234-248. */
int b2c_conv_fprop(const b2c_conv_desc *desc, const void *x, const void *w, const void *bias,
                   const b2c_bn_params *bn, int relu, void *y,
                   void *workspace, size_t workspace_bytes, void *stream);

/* The forward pass for a convolution that feeds a training-mode batch norm (the Conv2D -> BatchNormalization pairs the
 * reference's fusion flags name, pydtnn/parser.py:74-77; the statistics are those of
 * pydtnn/backends/cpu/layers/batch_normalization_cpu.py:65-70): y = conv(x, w) + bias as b2c_conv_fprop writes it, and
 * in `stats` the per-channel sum and sum of squares of y, taken from the tiles on their way to memory, so that the batch
 * norm does not read y a second time for them.  `stats` is an opaque DEVICE buffer of b2c_conv_stats_bytes(desc) bytes
 * (16-byte aligned) that b2c_bn_train_forward_prestats consumes; it is rewritten by every call.  The byte count says
 * how many rows of partial sums the launch leaves, so pass the value b2c_conv_stats_bytes returned to both calls.
 * b2c_conv_stats_bytes returns 0, and b2c_conv_fprop_stats B2C_ERR_UNSUPPORTED, for shapes outside the float32 NHWC
 * tensor-core path (callers then use b2c_conv_fprop and b2c_bn_train_forward). */
size_t b2c_conv_stats_bytes(const b2c_conv_desc *desc);
int b2c_conv_fprop_stats(const b2c_conv_desc *desc, const void *x, const void *w, const void *bias, void *y,
                         void *stats, size_t stats_bytes, void *workspace, size_t workspace_bytes, void *stream);

/* dx = conv_transpose(dy, w) (the scatter-add of row2im / col2im written as a gather).
 * Replaces cudnnConvolutionBackwardData, conv_2d_gpu.py:224-229, and sconvGemm*_back,
 * pydtnn/backends/cpu/libs/conv_gemm.py:311-330. */
int b2c_conv_dgrad(const b2c_conv_desc *desc, const void *dy, const void *w, void *dx,
                   void *workspace, size_t workspace_bytes, void *stream);

/* dw = lower(x)^T dy and, when db != NULL, db = sum over n,h,w of dy.
 * Replaces cudnnConvolutionBackwardFilter + cudnnConvolutionBackwardBias, conv_2d_gpu.py:192-213,
 * and sconvGemm* with trans='Y', conv_gemm.py:225-230. */
int b2c_conv_wgrad(const b2c_conv_desc *desc, const void *x, const void *dy, void *dw, void *db,
                   void *workspace, size_t workspace_bytes, void *stream);

/* The weight gradient for a caller that kept the forward pass's lowered input, as the reference's CPU layer keeps
 * `x_rows` from forward for backward (pydtnn/backends/cpu/layers/conv_2d_cpu.py:191-192, 373).  Few-channel NHWC layers
 * (the network stems: ci not a multiple of 32) write the im2row matrix of x at the start of the workspace in
 * b2c_conv_fprop and would write it again here; b2c_conv_wgrad_lowered skips that when the caller guarantees that
 * `workspace` is the very buffer the layer's last b2c_conv_fprop (same desc, same x) ran with and nothing has written
 * to it since -- in practice a workspace the layer owns.  b2c_conv_keeps_lowered_input(desc) says whether the layer
 * is of that kind (1) or not (0; the call then returns B2C_ERR_UNSUPPORTED and b2c_conv_wgrad is the one to use). */
int b2c_conv_keeps_lowered_input(const b2c_conv_desc *desc);
int b2c_conv_wgrad_lowered(const b2c_conv_desc *desc, const void *x, const void *dy, void *dw, void *db,
                           void *workspace, size_t workspace_bytes, void *stream);

/* The integer index map of the lowering, written to DEVICE memory as int64:
 *   NHWC: map[M][K], NCHW: map[K][M]; entry = flat offset into x or -1 at a padding tap,
 * numbered exactly as pydtnn/cython_modules/im2row_nhwc_cython.pyx:85-97 and
 * im2col_nchw_cython.pyx:112-124.  Uses the same tap arithmetic as the convolution kernels. */
int b2c_conv_index_map(const b2c_conv_desc *desc, int64_t *map, void *stream);

/* FC layer, row-major: y(b,out) = x(b,in) @ w(in,out) + bias; dw = x^T dy; db = sum_b dy;
 * dx = dy @ w^T.  Any of dw, db, dx may be NULL to skip it.
 * Replaces cublasSgemm/Dgemm + cudnnAddTensor + cublas gemv, pydtnn/backends/gpu/layers/fc_gpu.py:105-181. */
size_t b2c_fc_workspace_bytes(int dtype, int batch, int in_features, int out_features, int engine);
int b2c_fc_forward(int dtype, int engine, int batch, int in_features, int out_features,
                   const void *x, const void *w, const void *bias, void *y,
                   void *workspace, size_t workspace_bytes, void *stream);
int b2c_fc_backward(int dtype, int engine, int batch, int in_features, int out_features,
                    const void *x, const void *dy, const void *w, void *dw, void *db, void *dx,
                    void *workspace, size_t workspace_bytes, void *stream);

/* ---- layers either side of the convolution in a training step ------------------------
 * "rows" = n*h*w, channel axis last for NHWC; for NCHW pass layout and (n, c, hw). */

/* Training-mode batch norm. save_mean / save_inv_std (length c) are kept for backward.
 * running_* are updated in place with r = momentum*r + (1-momentum)*batch_stat.
 * Replaces cudnnBatchNormalizationForwardTraining, pydtnn/backends/gpu/layers/batch_normalization_gpu.py:121-131;
 * arithmetic of pydtnn/backends/cpu/layers/batch_normalization_cpu.py:59-76.
 * scratch: at least 128*c doubles; up to about 1200*c doubles lets layers with few channels spread
 * their reduction over more CTAs (the kernels adapt to what they are given). */
int b2c_bn_train_forward(int dtype, int layout, int n, int c, int hw, const void *x, const void *gamma,
                         const void *beta, void *running_mean, void *running_var, double momentum,
                         double eps, int fuse_relu, void *y, void *save_mean, void *save_inv_std,
                         void *scratch, size_t scratch_bytes, void *stream);
/* The same with the residual sum of an addition block folded in: y = relu?(bn(x) + addend), the sum taken on the
 * rounded batch-norm output exactly as a separate add kernel would take it.  For the last batch norm of a residual
 * branch (pydtnn/backends/gpu/layers/addition_block_gpu.py:49-66 sums the branch outputs, the ReLU follows): the
 * batch-norm output and the sum never travel through memory.  Backward is b2c_bn_train_backward on the masked
 * gradient of the sum (no y needed). */
int b2c_bn_train_forward_residual(int dtype, int layout, int n, int c, int hw, const void *x, const void *gamma,
                                  const void *beta, void *running_mean, void *running_var, double momentum,
                                  double eps, const void *addend, int relu, void *y, void *save_mean,
                                  void *save_inv_std, void *scratch, size_t scratch_bytes, void *stream);

/* b2c_bn_train_forward (float32, NHWC) with the batch sums already taken by b2c_conv_fprop_stats on the convolution
 * that wrote x: mean, inverse standard deviation and the running averages come from `stats` (summed in double, in a
 * fixed order), then y = relu?(bn(x) [+ addend]) in one pass over x.  stats_bytes: what b2c_conv_stats_bytes returned
 * for that convolution (B2C_ERR_BAD_GEOMETRY if it is not a whole number of [2][c] float rows).  addend may be NULL (see
 * b2c_bn_train_forward_residual).  scratch: as for b2c_bn_train_forward.  Backward is b2c_bn_train_backward, unchanged. */
int b2c_bn_train_forward_prestats(int n, int c, int hw, const void *x, const void *stats, size_t stats_bytes,
                                  const void *gamma, const void *beta, void *running_mean, void *running_var,
                                  double momentum, double eps, int fuse_relu, const void *addend, void *y,
                                  void *save_mean, void *save_inv_std, void *scratch, size_t scratch_bytes, void *stream);

/* b2c_bn_train_forward for callers that must not allocate and have no scratch buffer to lend: hosts
 * that give all device memory to their own pool at start-up and then forbid allocation (a late
 * cudaMalloc stalls the device and may fail once the pool owns the card).  Same arguments and results
 * as b2c_bn_train_forward without the scratch pair; the partial sums live in a fixed 2 MiB array inside
 * the library (one copy per GPU that loads it, kept until the process ends).
 *  - Limit: c <= 2048 channels, otherwise B2C_ERR_TOO_LARGE ("size exceeds a fixed capacity").
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *    that first call during set-up, before any stream capture begins.
 *  - No cudaMalloc / cudaFree / allocating library call is made, on the first call or later.
 *  - All calls on a device share the one array: calls that can overlap on the GPU (different streams)
 *    race on it; keep them on one stream or order them with events.  The array keeps the previous
 *    call's partial sums, which is harmless: each call overwrites every entry it later reads.
 * This entry point has no counterpart in the reference. */
int b2c_bn_train_forward_static(int dtype, int layout, int n, int c, int hw, const void *x, const void *gamma,
                                const void *beta, void *running_mean, void *running_var, double momentum,
                                double eps, int fuse_relu, void *y, void *save_mean, void *save_inv_std,
                                void *stream);
/* dgamma, dbeta, dx (dx may be NULL). If the forward pass fused the ReLU, dy is first masked by y > 0: pass
 * the forward output as y_for_relu_mask, and/or the forward beta as beta_for_relu_mask.  With beta the float32
 * NHWC path recomputes the mask from x (the same instruction sequence as the forward pass, bit for bit) and
 * does not read y; every other path reads y, so callers pass both.  Both NULL: no ReLU.
 * Replaces cudnnBatchNormalizationBackward, batch_normalization_gpu.py:146-156. scratch: as for the forward pass. */
int b2c_bn_train_backward(int dtype, int layout, int n, int c, int hw, const void *x, const void *dy,
                          const void *y_for_relu_mask, const void *beta_for_relu_mask, const void *gamma,
                          const void *save_mean,
                          const void *save_inv_std, void *dgamma, void *dbeta, void *dx,
                          void *scratch, size_t scratch_bytes, void *stream);
/* y = relu?(((x-mean)*inv_std)*gamma+beta); pydtnn/cython_modules/bn_inference_cython.pyx:71-72. */
int b2c_bn_inference(int dtype, int layout, int n, int c, int hw, const void *x, const void *mean,
                     const void *inv_std, const void *gamma, const void *beta, int relu, void *y, void *stream);

/* y = max(x,0); dx = dy * (y > 0)   pydtnn/backends/gpu/activations/relu_gpu.py:58,66 */
int b2c_relu_forward(int dtype, int64_t count, const void *x, void *y, void *stream);
int b2c_relu_backward(int dtype, int64_t count, const void *dy, const void *y, void *dx, void *stream);
/* acc += other  (residual sum; pydtnn/backends/gpu/layers/addition_block_gpu.py:63,82) */
int b2c_add_inplace(int dtype, int64_t count, void *acc, const void *other, void *stream);

/* out = max(a + b, 0): the residual sum and the ReLU that follows an addition block, in one pass. */
int b2c_add_relu(int dtype, int64_t count, const void *a, const void *b, void *out, void *stream);
/* dx = (y > 0) ? a + b : 0: the sum of the branch gradients at an addition block's input and the backward of the
 * ReLU that feeds the block (y = that ReLU's output), in one pass. */
int b2c_add_relu_backward(int dtype, int64_t count, const void *a, const void *b, const void *y, void *dx, void *stream);

/* Pooling over in-bounds taps only (pydtnn/cython_modules/max_pool_2d_nhwc_cython.pyx:96-113,
 * average_pool_2d_nhwc_cython.pyx:93-111); idx_max is int32 tap number ii*kw+jj.
 * Replaces cudnnPoolingForward/Backward, pydtnn/backends/gpu/layers/abstract_pool_2d_layer_gpu.py:82-102. */
int b2c_pool_forward(int dtype, int layout, int is_max, int n, int h, int w, int c, int kh, int kw,
                     int vpad, int hpad, int vstr, int hstr, int vdil, int hdil,
                     const void *x, void *y, int32_t *idx_max, void *stream);
int b2c_pool_backward(int dtype, int layout, int is_max, int n, int h, int w, int c, int kh, int kw,
                      int vpad, int hpad, int vstr, int hstr, int vdil, int hdil,
                      const void *dy, const int32_t *idx_max, void *dx, void *stream);

/* Row-wise softmax and its backward (pydtnn/backends/cpu/activations/softmax_cpu.py:32-39). */
int b2c_softmax_forward(int dtype, int rows, int cols, const void *x, void *y, void *stream);
int b2c_softmax_backward(int dtype, int rows, int cols, const void *dy, const void *y, void *dx, void *stream);
/* Categorical cross-entropy on probabilities with integer labels: per-row log-likelihood into
 * row_loss (loss = -mean(row_loss)), hit[row] = 1 if arg-max equals the label, and
 * dx = onehot / (-clip(p) * global_batch)
 * (pydtnn/backends/gpu/losses/categorical_cross_entropy_gpu.py:33-58;
 *  pydtnn/backends/gpu/metrics/categorical_accuracy_gpu.py:33-51). */
int b2c_cce_forward_backward(int dtype, int rows, int cols, const void *probs, const int32_t *labels,
                             int global_batch, double eps, void *row_loss, int32_t *hit, void *dx, void *stream);

/* Totals of b2c_cce_forward_backward's per-row outputs, written to DEVICE memory as two doubles:
 * out2[0] = -sum(row_loss) / rows (the batch's mean loss), out2[1] = 100 * sum(hit) / rows (accuracy in per cent;
 * hit may be NULL -> 0).  These are the values the reference divides by the process count and sums over ranks,
 * pydtnn/model.py:426-438; a data-parallel caller all-reduces the two doubles in place. */
int b2c_cce_totals(int dtype, int rows, const void *row_loss, const int32_t *hit, double *out2, void *stream);

/* inv_std[i] = 1 / sqrt(running_var[i] + eps), evaluated in double and rounded once: the per-channel factor of the
 * inference-mode batch norm, pydtnn/layers/batch_normalization.py:61 and
 * pydtnn/backends/cpu/layers/batch_normalization_cpu.py:92-94 (computed there on the host). */
int b2c_bn_inv_std(int dtype, int c, const void *running_var, double eps, void *inv_std, void *stream);

/* Diagnostic: launches `blocks` CTAs of 256 threads that each run `iters` rounds of 8 independent register-resident
 * fused multiply-adds, and reports the floating-point operations of the launch in *flops (may be NULL).  Timed by the
 * caller, it gives the FMA rate the device sustains: the roofline denominator of the FMA engine.  sink: blocks*256
 * elements, never written.  No counterpart in the reference. */
int b2c_probe_fma(int dtype, int blocks, int iters, void *sink, double *flops, void *stream);

/* SGD with momentum over one flat tensor: v = m*v + dw; w -= lr*(decay*w + v)
 * (Nesterov: w -= lr*(decay*w + dw + m*v)); pydtnn/backends/gpu/optimizers/sgd_gpu.py:40-47. */
int b2c_sgd_update(int dtype, int64_t count, void *w, const void *dw, void *velocity,
                   double lr, double momentum, double decay, int nesterov, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B2C_H */
