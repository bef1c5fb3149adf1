/*
 * nectarml_b200 -- C ABI of the B200 (sm_100a) dense-contraction path:
 * Conv2d / ConvTranspose2d / Linear in forward, input-gradient and weight-gradient.
 *
 * Two layers of entry points:
 *
 *  (1) nml_conv_* / nml_linear_*  -- descriptor based, caller-owned outputs and workspace,
 *      explicit stream, no allocation, no synchronisation, int status return.  The one exception
 *      is the first call on each device, which does what nml_init() does (see there).
 *  (2) nml_ref_*                  -- the flat signatures of the reference's host ops
 *      (device pointers as integers + shape ints in, freshly cudaMalloc'ed result out), so a
 *      binding of the reference's `_nectarml.tensor.conv.*` / `_nectarml.tensor.matmul`
 *      names can forward to them one to one.
 *
 * All pointers are device pointers unless stated.  Nothing here takes or returns a torch type.
 */
#ifndef NECTARML_B200_H
#define NECTARML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes (0 = success).  nml_status_string() names them. */
enum {
    NML_OK = 0,
    NML_ERR_INVALID = 1,     /* bad descriptor / argument                                   */
    NML_ERR_WORKSPACE = 2,   /* workspace missing or too small                              */
    NML_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed                         */
    NML_ERR_UNSUPPORTED = 4, /* valid request the kernels do not cover (e.g. groups != 1)   */
    NML_ERR_DEVICE = 5       /* a kernel gave up on a bounded wait (see nml_device_status)  */
};

/* Element types; the values equal the reference's DType enum
 * (nectarml/csrc/include/common/dtype.h:15-21: Float32 = 0, Float16 = 1). */
enum { NML_F32 = 0, NML_F16 = 1 };

/* Activation layouts. The reference only knows NCHW (nectarml/csrc/ops/tensor/conv/conv2d.cpp:71-134);
 * NHWC is this library's native layout and needs no conversion pass. */
enum { NML_NCHW = 0, NML_NHWC = 1 };

/* Arithmetic of the contraction.
 *  NML_MATH_F16    operands rounded to fp16, fp32 accumulation (replaces cublasHgemm,
 *                  conv2d.cpp:111-118, with a wider accumulator)
 *  NML_MATH_3XTF32 fp32 operands split into tf32 hi + lo, three tensor-core products, fp32
 *                  accumulation (replaces cublasSgemm, conv2d.cpp:100-109)
 *  NML_MATH_TF32   single tf32 product (not used by the reference-compatible entry points) */
enum { NML_MATH_F16 = 0, NML_MATH_3XTF32 = 1, NML_MATH_TF32 = 2 };

/* Geometry of one Conv2d (transposed = 0) or ConvTranspose2d (transposed = 1) layer plus the
 * storage formats of the tensors of one call.  batch/c_in/h/w describe the layer's INPUT;
 * the layer's output has c_out channels and the usual output size
 *   conv : (h + 2p - d(k-1) - 1)/s + 1            (nectarml/nn/functional/conv.py:406-407)
 *   convT: (h-1)s - 2p + d(k-1) + 1 + outpad      (nectarml/nn/functional/conv.py:479-482)
 * Weights are [c_out, c_in, kh, kw] for conv and [c_in, c_out, kh, kw] for convT
 * (nectarml/nn/conv.py:287-289), always dense (groups == 1).
 *   in_dtype / in_layout   : the activation tensors read by the call (x, or dy and x)
 *   out_dtype / out_layout : the activation tensor written (y or dx); dw and db are fp32
 *   w_dtype                : weights and bias as stored                                  */
typedef struct nml_conv_desc {
    int batch, c_in, h, w;
    int c_out, kh, kw;
    int stride_h, stride_w;
    int pad_h, pad_w;
    int dil_h, dil_w;
    int outpad_h, outpad_w; /* ConvTranspose2d only */
    int transposed;
    int in_dtype, in_layout;
    int out_dtype, out_layout;
    int w_dtype;
    int math;
    int round_out_f16;      /* forward only: round the result through fp16 before the store,
                               as the reference's autocast forward does (conv2d.cpp:415-435)  */
} nml_conv_desc;

/* y = x * W^T + b with W [out_features, in_features] (nectarml/nn/linear.py:44-47). */
typedef struct nml_linear_desc {
    int rows, in_features, out_features;
    int in_dtype, out_dtype, w_dtype;
    int math;
    int round_out_f16;
} nml_linear_desc;

enum { NML_PASS_FORWARD = 0, NML_PASS_BACKWARD_DATA = 1, NML_PASS_BACKWARD_WEIGHT = 2 };

const char* nml_status_string(int status);

/* One-time set-up of the CURRENT device: looks up the device-side status word (it lives in the
 * library image, nothing is allocated), clears it with a synchronous cudaMemset, loads every
 * kernel of the library and raises the contraction kernel's dynamic shared-memory limit.  Every
 * entry point does this by itself on its first call on a device; call nml_init() explicitly
 * when that first call would otherwise fall inside a CUDA stream capture or a latency-critical
 * section.  Thread-safe; later calls return immediately. */
int nml_init(void);

/* Output size of the layer described by d (height, width). Returns a status. */
int nml_conv_output_size(const nml_conv_desc* d, int* h_out, int* w_out);

/* Bytes of workspace the given pass needs (0 is possible). Returns a status. */
int nml_conv_workspace_size(const nml_conv_desc* d, int pass, size_t* bytes);
int nml_linear_workspace_size(const nml_linear_desc* d, int pass, size_t* bytes);

/* Forward.  Replaces run_conv2d / run_conv_transpose2d and their im2col, bias, transposition
 * and cast kernels (nectarml/csrc/ops/tensor/conv/conv2d.cpp:71-134, 136-211, 401-497).
 * bias may be NULL. */
int nml_conv_forward(const nml_conv_desc* d, const void* x, const void* w, const void* bias, void* y,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Forward for callers that cannot allocate device memory.  It has no counterpart in the
 * reference (whose host ops cudaMalloc freely); it exists for hosts where an allocation call is
 * not an option at the point of the call -- a serving process that has handed every free byte of
 * HBM to its own pool, so cudaMalloc would fail, or a latency-critical loop that must not hit the
 * device-wide synchronisation cudaMalloc / cudaFree imply.  Same arithmetic and same arguments as
 * nml_conv_forward, but no workspace argument: the converted operands go to a 64 MiB
 * (67,108,864-byte) scratch array that is part of the library image, so every GPU that loads
 * the library holds those 64 MiB until the process exits.  The call makes no cudaMalloc, cudaFree
 * or other allocating call.
 *   - A layer whose conversion scratch exceeds 64 MiB is refused with NML_ERR_WORKSPACE (the
 *     message states the need and the limit); use nml_conv_forward with your own workspace.
 *   - The first call on each device looks up the device address of the scratch array (with that
 *     device current) and raises the kernel's shared-memory limit.  Make that first call
 *     before any stream capture begins.
 *   - All calls share the one array, and it keeps what the last call left there.  Each call
 *     rewrites every byte it later reads, so stale contents are harmless, but two calls whose
 *     work overlaps on the GPU (different streams, or different host threads) race on it:
 *     serialise them.
 *   - Kernels launched here report an abandoned bounded wait into a status word beside the
 *     scratch array, not into the word nml_device_status reads.  Calling this function with
 *     d == NULL (other arguments ignored) synchronises the device and returns NML_ERR_DEVICE
 *     if such a give-up was recorded, clearing it. */
int nml_conv_forward_static(const nml_conv_desc* d, const void* x, const void* w, const void* bias, void* y,
                            void* stream);

/* Input gradient: dx from dy.  Replaces run_conv2d_backward_input + col2im
 * (conv2d.cpp:213-274, 499-518) and conv_transpose2d_backward_input (conv2d.cpp:520-542). */
int nml_conv_backward_data(const nml_conv_desc* d, const void* dy, const void* w, void* dx,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Weight gradient (overwrites dw, fp32, weight-shaped) and, when db != NULL, the bias gradient
 * db[c] = sum over batch and pixels of dy (fp32).  dw is bitwise repeatable from run to run: K
 * slices store partial sums into planes of the workspace that a second kernel adds in a fixed
 * order (no atomics); so are y and dx of every forward / input-gradient walk.  Replaces run_conv2d_backward_weight /
 * run_conv_transpose2d_backward_weight (conv2d.cpp:276-335, 337-395) and the three chained
 * reductions of `out_grad.sum(dim=(0,2,3))` (nectarml/cuda/tensor/conv.py:175-176). */
int nml_conv_backward_weight(const nml_conv_desc* d, const void* x, const void* dy, float* dw,
                             float* db, void* workspace, size_t workspace_bytes, void* stream);

/* Linear.  Replaces the permute + cast + cublas + broadcast-add chain behind
 * `x @ W.transpose(1,0) + b` (nectarml/nn/linear.py:44-47,
 * nectarml/core/_tensor/numerical.py:864-907) and its backward (numerical.py:896-904, 662-666):
 *   forward          y [rows,out] = x [rows,in] * W[out,in]^T + b
 *   backward_data    dx[rows,in]  = dy[rows,out] * W[out,in]
 *   backward_weight  dw[out,in]   = dy^T * x,  db[out] = column sums of dy            */
int nml_linear_forward(const nml_linear_desc* d, const void* x, const void* w, const void* bias,
                       void* y, void* workspace, size_t workspace_bytes, void* stream);
int nml_linear_backward_data(const nml_linear_desc* d, const void* dy, const void* w, void* dx,
                             void* workspace, size_t workspace_bytes, void* stream);
int nml_linear_backward_weight(const nml_linear_desc* d, const void* x, const void* dy, float* dw,
                               float* db, void* workspace, size_t workspace_bytes, void* stream);

/* Synchronises the current device and returns NML_OK, or NML_ERR_DEVICE with *code set to the
 * wait that timed out inside a kernel since the last call (and clears it; nml_status_string then
 * names the wait).  The asynchronous
 * entry points above never block, so this is how a caller learns of a device-side give-up. */
int nml_device_status(int* code);

/* Caps the number of SMs the persistent kernels of later launches occupy (their grid and their tile
 * / split-K plan); 0 restores "all SMs".  For callers that run something else on the GPU at the
 * same time: a contraction kernel launched on every SM while an NCCL all-reduce of the previous
 * layer's gradients holds a few of them leaves some of its CTAs waiting for a free SM, and with a
 * static tile schedule those late CTAs set the kernel's duration; launching on `all - reserved`
 * SMs avoids that.  Process-wide; workspace sizes depend on it, so query them under the same
 * limit the call will run under.  The reference has no counterpart (single stream, no overlap). */
int nml_set_sm_limit(int sms);

/* Number of kernels this library has launched in this process (contraction kernel plus its
 * conversion / reduction helpers), for launch accounting. */
long long nml_launch_count(void);

/* Per-launch device timing of the contraction kernel.  After nml_profile_begin(n) each of the
 * next n contraction launches is bracketed by CUDA events on its own stream; nml_profile_end
 * synchronises, writes the durations in milliseconds in launch order and stops recording.
 * Measurement support only: nothing else in the library depends on it. */
int nml_profile_begin(int max_records);
int nml_profile_end(float* ms_out, int capacity, int* count);

/* ---- neighbours of the contraction in a training step (fp16 NHWC = row-major [rows][channels]) ----
 * Batch normalisation over the rows of a [rows][channels] fp16 matrix (N*H*W pixels of an NHWC
 * tensor), fused with what follows it:  y = act(gamma * (x - mean) * rstd + beta [+ residual]),
 * act 0 = none, 1 = ReLU, 2 = LeakyReLU(slope).  mean and rstd = 1/sqrt(biased variance + eps)
 * (fp32, [channels]) are outputs of the forward and inputs of the backward.  Replaces the
 * reference's fp32-NCHW kernels compute_mean_var_welford / normalize / batch_norm_backward
 * (nectarml/csrc/kernels/tensor/fused/norm.cu; Python side nectarml/cuda/tensor/fused/batch_norm.py:10-99)
 * and the activation and residual-add passes around them.  channels: multiple of 8, at most 2048;
 * pointers 16-byte aligned; gamma / beta / residual may be NULL.  Reductions are two-stage in a
 * fixed order: bitwise repeatable.  The workspace holds the partial sums. */
int nml_bn_workspace_size(long long rows, int channels, size_t* bytes);
int nml_bn_forward(const void* x, long long rows, int channels, const float* gamma, const float* beta,
                   const void* residual, int act, float slope, float eps, void* y, float* mean, float* rstd,
                   void* workspace, size_t workspace_bytes, void* stream);
/* With dz = dy * act'(y): dbeta = sum dz, dgamma = sum dz * xhat,
 * dx = gamma * rstd * (dz - dbeta/rows - xhat * dgamma/rows); dres (optional, fp16) = dz, the
 * gradient of the residual input.  y is the forward's output (needed when act != 0). */
int nml_bn_backward(const void* dy, const void* y, const void* x, long long rows, int channels,
                    const float* gamma, const float* mean, const float* rstd, int act, float slope, void* dx,
                    void* dres, float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Max pooling of an NHWC fp16 tensor (channels a multiple of 8), output size (h + 2 pad - k)/stride + 1.
 * The forward also writes one byte per output value naming the window tap that won (`index`,
 * batch * ho * wo * channels bytes); the backward gathers dy through it, writes every element of
 * dx exactly once and uses no atomics.  Replaces the reference's max-pool kernels on this layout
 * (nectarml/csrc/kernels/tensor/pooling.cu) between the stem and the first residual block. */
int nml_maxpool_forward(const void* x, int batch, int h, int w, int channels, int k, int stride, int pad,
                        void* y, void* index, void* stream);
int nml_maxpool_backward(const void* dy, const void* index, int batch, int h, int w, int channels, int k,
                         int stride, int pad, void* dx, void* stream);

/* Gradient plumbing over ONE flat fp32 buffer holding every parameter's gradient (the buffer the
 * weight-gradient entry points wrote into and NCCL all-reduced).  nml_grads_check sets *found_inf
 * (device int) to 1 if any grad * inv_scale is not finite, else 0: one launch, no allocation, no
 * read-back (the reference unscales parameter by parameter with a cudaMalloc and a blocking copy
 * each, nectarml/csrc/ops/amp/amp.cpp:18-37).  nml_sgd_momentum_step applies
 *   g = grad * inv_scale + weight_decay * p;  v = momentum * v + (1 - dampening) * g;  p -= lr * v
 * (nectarml/optim/sgd.py:60-72, nectarml/csrc/kernels/optim/sgd.cu) to the whole buffer in one
 * launch, refreshes the fp16 copy of the parameters (params_f16, may be NULL) and does nothing at
 * all when *found_inf is set.  n: multiple of 4. */
int nml_grads_check(const float* grads, size_t n, float inv_scale, int* found_inf, void* stream);
int nml_sgd_momentum_step(float* params, const float* grads, float* velocity, void* params_f16, size_t n,
                          float lr, float momentum, float dampening, float weight_decay, float inv_scale,
                          const int* found_inf, void* stream);
long long nml_layers_launch_count(void);

/* ---- reference-shaped entry points ------------------------------------------------------
 * Same argument lists as the reference's host ops, which its pybind module registers as
 * `_nectarml.tensor.conv.*` and `_nectarml.tensor.matmul`
 * (nectarml/csrc/python/ops/tensor/conv.h:71-150, matmul.h:10-16, bindings.cpp:41-51).
 * Pointers travel as integers; *result receives a device pointer from the device's stream-ordered
 * memory pool (cudaMallocAsync on the legacy default stream; plain cudaMalloc where a device has no
 * pools) that the caller releases with nml_ref_free -- or with cudaFree, which accepts such pointers:
 * the reference's `free_cuda` path ends in cudaFree (nectarml/csrc/pool/allocator_pool.cpp:75-96).
 * Unlike the reference's raw cudaMalloc / cudaFree per result (its pool is disabled in these
 * translation units, allocator_pool.h:38), this does not synchronise the device on every call.  dtype uses the NML_F32 / NML_F16 values.
 * Like the reference these run on the legacy default stream and are ordered by it.
 * With half_precision != 0 the tensors are fp32 in memory, the contraction runs on fp16
 * operands and the fp32 result holds fp16-rounded values (conv2d.cpp:415-435); otherwise fp32
 * tensors use the 3xTF32 split and fp16 tensors the fp16 path.  The backward entry points take
 * the dtype of the tensors they are handed and always produce fp32 gradients. */
int nml_ref_conv2d(uintptr_t input_ptr, size_t input_size, uintptr_t weight_ptr, size_t weight_size,
                   uintptr_t bias_ptr, size_t bias_size, size_t output_size, int B, int C_in, int H,
                   int W, int C_out, int KH, int KW, int stride_h, int stride_w, int padding_h,
                   int padding_w, int dilation_h, int dilation_w, int groups, int dtype,
                   int half_precision, uintptr_t* result);
int nml_ref_conv_transpose2d(uintptr_t input_ptr, size_t input_size, uintptr_t weight_ptr,
                             size_t weight_size, uintptr_t bias_ptr, size_t bias_size,
                             size_t output_size, int B, int C_in, int H, int W, int C_out, int KH,
                             int KW, int stride_h, int stride_w, int padding_h, int padding_w,
                             int dilation_h, int dilation_w, int output_padding_h,
                             int output_padding_w, int groups, int dtype, int half_precision,
                             uintptr_t* result);
int nml_ref_conv2d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int H,
                                  int W, int C_out, int KH, int KW, int H_out, int W_out,
                                  int stride_h, int stride_w, int padding_h, int padding_w,
                                  int dilation_h, int dilation_w, int groups, int dtype,
                                  uintptr_t* result);
int nml_ref_conv_transpose2d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B,
                                            int C_in, int H, int W, int C_out, int KH, int KW,
                                            int H_out, int W_out, int stride_h, int stride_w,
                                            int padding_h, int padding_w, int dilation_h,
                                            int dilation_w, int groups, int dtype, uintptr_t* result);
int nml_ref_conv2d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int H,
                                   int W, int C_out, int KH, int KW, int H_out, int W_out,
                                   int stride_h, int stride_w, int padding_h, int padding_w,
                                   int dilation_h, int dilation_w, int dtype, uintptr_t* result);
int nml_ref_conv_transpose2d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B,
                                             int C_in, int H, int W, int C_out, int KH, int KW,
                                             int H_out, int W_out, int stride_h, int stride_w,
                                             int padding_h, int padding_w, int dilation_h,
                                             int dilation_w, int dtype, uintptr_t* result);
/* 1-D convolutions (`_nectarml.tensor.conv.conv1d` ... `conv_transpose1d_backward_weight`,
 * nectarml/csrc/python/ops/tensor/conv.h:11-68, called from nectarml/cuda/tensor/conv.py:12-106):
 * tensors are [B, C, L], weights [C_out, C_in, K] ([C_in, C_out, K] transposed); the same rules on
 * dtype, streams and ownership as the 2-D entry points (these have no half_precision flag). */
int nml_ref_conv1d(uintptr_t input_ptr, uintptr_t weight_ptr, uintptr_t bias_ptr, int B, int C_in, int L,
                   int C_out, int K, int stride, int padding, int dilation, int groups, int dtype,
                   uintptr_t* result);
int nml_ref_conv_transpose1d(uintptr_t input_ptr, uintptr_t weight_ptr, uintptr_t bias_ptr, int B, int C_in,
                             int L, int C_out, int K, int stride, int padding, int dilation,
                             int output_padding, int groups, int dtype, uintptr_t* result);
int nml_ref_conv1d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int L,
                                  int C_out, int K, int L_out, int stride, int padding, int dilation,
                                  int groups, int dtype, uintptr_t* result);
int nml_ref_conv_transpose1d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in,
                                            int L, int C_out, int K, int L_out, int stride, int padding,
                                            int dilation, int groups, int dtype, uintptr_t* result);
int nml_ref_conv1d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int L,
                                   int C_out, int K, int L_out, int stride, int padding, int dilation,
                                   int dtype, uintptr_t* result);
int nml_ref_conv_transpose1d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in,
                                             int L, int C_out, int K, int L_out, int stride, int padding,
                                             int dilation, int dtype, uintptr_t* result);
/* C[..., M, N] = A[..., M, K] * B[K, N] (or batched B), row-major
 * (nectarml/csrc/ops/tensor/matmul.cpp:8-48).  a_shape / b_shape are host arrays.  A 2-D B is
 * shared by every batch entry of A (the reference advances B per batch entry even then,
 * matmul.cpp:27,39, and reads past its end). */
int nml_ref_matmul(uintptr_t a_ptr, uintptr_t b_ptr, const int* a_shape, int a_rank,
                   const int* b_shape, int b_rank, int dtype, uintptr_t* result);

/* Releases a pointer returned through *result above (back to the pool, in stream order); the
 * counterpart of the reference's `_nectarml.free_cuda` (nectarml/csrc/ops/system/memory.cpp:33-39). */
int nml_ref_free(uintptr_t ptr);

/* ---- test support ----------------------------------------------------------------------
 * Copies one TMA box of a row-major host-described 4-D tensor (dims fastest first) into a
 * linear device buffer without swizzle, so tests can pin the coordinate, element-stride and
 * zero-fill behaviour the implicit-GEMM address math relies on.  elem_bytes is 2 or 4. */
int nml_debug_tma_box(const void* tensor, int elem_bytes, const int dims[4], const int box[4],
                      const int elem_strides[4], const int coords[4], void* out, size_t out_bytes,
                      void* stream);


/* Give-up path, exercised without a fault: one warp waits with the library's bounded wait on an
 * mbarrier nothing arrives on; after limit_ns (at most 1e8) the wait runs out, the kernel records
 * the wait code in the status word (use_static_word != 0: the word nml_conv_forward_static's
 * kernels report into) and returns.  nml_device_status / the d == NULL form of
 * nml_conv_forward_static then report NML_ERR_DEVICE once. */
int nml_debug_wait_timeout(unsigned long long limit_ns, int use_static_word, void* stream);

/* The same through the contraction kernel itself: a small fp16 Linear forward whose activation
 * boxes are encoded half as tall as the kernel expects, so no pipeline stage ever receives all
 * its bytes; the MMA warp's wait runs out after limit_ns, every role unwinds through its bounded
 * waits, TMEM is freed and the kernel returns (y is left unwritten).  rows <= 4096,
 * in_features <= 1024, out_features <= 128, fp16 tensors only. */
int nml_debug_stalled_linear_forward(const nml_linear_desc* d, const void* x, const void* w, void* y,
                                     void* workspace, size_t workspace_bytes,
                                     unsigned long long limit_ns, void* stream);

/* Blocking device-to-host copy of a result pointer, as the reference's tensor read-back does
 * (nectarml/csrc/ops/system/device/device.cpp:39-64).  Lets a test read what nml_ref_* returned
 * without wrapping the raw pointer in another framework's tensor. */
int nml_debug_copy_to_host(void* host_dst, uintptr_t device_src, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* NECTARML_B200_H */
