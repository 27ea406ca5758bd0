/*
 * repdl_b200 -- C ABI of the bit-reproducible operator backend for NVIDIA B200 (sm_100a).
 *
 * Every entry point replaces one function of microsoft/RepDL's operator backend (the
 * functions its Python layer binds in backend/cuda/bind.cpp:6-19 and calls from
 * repdl/ops.py:12-157) and produces, on the GPU, exactly the bits the reference's CPU
 * backend produces for the same inputs: one fp32 accumulator per output element, updated
 * in the reference's order with IEEE-754 single-rounding FMA / add, no flush-to-zero, no
 * tensor cores, no atomics.
 *
 * Conventions
 *   - All pointers are DEVICE pointers on the CURRENT device unless a comment says host.
 *   - Tensors are fp32, row-major / NCHW, dense unless a leading dimension is passed.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *     Calls are asynchronous: they enqueue work and return.
 *   - Return value: 0 success; negative = invalid argument (REPDL_E_*); positive = the
 *     cudaError_t reported by the launch.  Nothing throws, nothing allocates device
 *     memory unless the comment says so; scratch is passed in by the caller.
 *   - Inputs are never written.  Outputs may not alias inputs.
 */
#ifndef REPDL_B200_H
#define REPDL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define REPDL_OK 0
#define REPDL_E_NULL (-1)      /* a required pointer is NULL */
#define REPDL_E_SHAPE (-2)     /* a dimension is negative or inconsistent */
#define REPDL_E_RANGE (-3)     /* a size exceeds what the kernel indexes (see each call) */
#define REPDL_E_SCRATCH (-4)   /* scratch buffer missing or too small */
#define REPDL_E_UNSUPPORTED (-5)
#define REPDL_E_STATIC_MAX (-6) /* input larger than a built-in (static) scratch array supports */

/* Library version and the compute capability the kernels were compiled for (100). */
int repdl_b200_version(void);
int repdl_b200_sm_arch(void);
/* Human-readable text for a status returned by any call below (static storage). */
const char *repdl_b200_strerror(int status);

/* Max pooling over non-overlapping windows (kernel = stride, no padding, no dilation, floor mode) of
 * `planes` = N * C planes of H x W, and its backward pass.  Not operators of the reference's backend: its
 * layers call torch.nn.functional.max_pool2d, which these replace behind repdl_b200.nn.MaxPool2d.  The
 * forward scan keeps ATen's selection rule (row by row; a value is taken if it is greater than the maximum
 * so far or is a NaN), so the result and the position that receives the gradient are the ones torch picks.
 * index: int32, position h * W + w inside the plane.  Output extent: (H / KH) x (W / KW). */
int repdl_b200_maxpool2d(const float *x, float *y, int *index, int64_t planes, int64_t H, int64_t W,
                         int64_t KH, int64_t KW, void *stream);
int repdl_b200_maxpool2d_backward(const float *grad_y, const int *index, float *grad_x, int64_t planes,
                                  int64_t H, int64_t W, int64_t KH, int64_t KW, void *stream);

/* Strided sub-matrix copy on a stream: `rows` rows of `width_bytes` bytes, source and destination
 * with their own row pitches.  direction 0: host -> device, 1: device -> host, 2: device -> device.
 * No counterpart in the reference (its operators take whole tensors that live on the device): the
 * host-operand step of repdl_b200.dist uploads B by column blocks with it, so that the first product
 * can start before all of B has arrived.  Host memory should be pinned. */
int repdl_b200_copy2d(void *dst, int64_t dst_pitch_bytes, const void *src, int64_t src_pitch_bytes,
                      int64_t width_bytes, int64_t rows, int direction, void *stream);

/* ---- matrix multiplication -------------------------------------------------------------
 * Replaces repdl::cuda::matrix_multiplication::mm (backend/cuda/matrix_multiplication.cu:234-260),
 * bits defined by backend/cpu/matrix_multiplication.cpp:12-36:
 *     C[i][j] = fold over k = 0..K-1 ascending of fmaf(opA(i,k), opB(k,j), .), starting at +0
 * opA(i,k) = transA ? A[k*lda+i] : A[i*lda+k];  opB(k,j) = transB ? B[j*ldb+k] : B[k*ldb+j].
 * C is M x N with row pitch ldc.  Pitches are in elements.  M, N, K >= 0 (K = 0 writes +0). */
int repdl_b200_mm(const float *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                  int transA, int transB, int64_t lda, int64_t ldb, int64_t ldc, void *stream);

/* Row-sharded product for the GPUs of one node (no counterpart in the reference, which has no
 * multi-GPU code): this rank holds rows [row0, row0 + M_local) of op(A) in A_rows and all of B;
 * the kernel computes those rows of C exactly as repdl_b200_mm would and stores every finished
 * tile into the same rows of ALL nranks C buffers (C_of_rank: HOST array of nranks device pointers,
 * each the base of a full C with pitch ldc; peers' buffers must be mapped into this process, e.g.
 * symmetric memory).  When every rank has run its call and the ranks have synchronised, each holds
 * the full C.  No reduction is split across ranks, so the bits equal a single-GPU run. nranks <= 8. */
int repdl_b200_mm_allgather(const float *A_rows, const float *B, float *const *C_of_rank, int nranks,
                            int64_t row0, int64_t M_local, int64_t N, int64_t K, int transA,
                            int transB, int64_t lda, int64_t ldb, int64_t ldc, void *stream);

/* conv2d with the layer's epilogue in the same launch: output = conv2d(input, kernel) + bias[oc], then
 * max(., 0) if relu != 0.  Replaces the launches of Conv2dFunction.forward behind the operator
 * (repdl/nn/conv.py:27-28: `output += bias...`) and of a ReLU that follows the layer; each step is the
 * separately rounded fp32 operation those launches perform (NaN passes through the maximum), so the
 * bits are the same.  bias may be NULL. */
int repdl_b200_conv2d_bias_act(const float *input, const float *kernel, const float *bias, float *output,
                               int64_t N, int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH,
                               int64_t KW, int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                               int64_t groups, int relu, void *stream);

/* ---- convolution -----------------------------------------------------------------------
 * Replace repdl::cuda::convolution::{conv2d, conv2d_grad_input, conv2d_grad_kernel}
 * (backend/cuda/convolution.cu:153-173, 259-277, 359-377); bits defined by
 * backend/cpu/convolution.cpp:12-52, 54-90, 92-128.  NCHW input, [OC][IC/groups][KH][KW]
 * kernel, OH = (H + 2*pH - KH)/sH + 1.  Taps that fall in the padding are skipped, not
 * multiplied by zero.  Only conv2d takes groups (as in the reference). */
int repdl_b200_conv2d(const float *input, const float *kernel, float *output, int64_t N,
                      int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH, int64_t KW,
                      int64_t sH, int64_t sW, int64_t pH, int64_t pW, int64_t groups,
                      void *stream);
int repdl_b200_conv2d_grad_input(const float *grad_output, const float *kernel,
                                 float *grad_input, int64_t N, int64_t IC, int64_t H, int64_t W,
                                 int64_t OC, int64_t KH, int64_t KW, int64_t sH, int64_t sW,
                                 int64_t pH, int64_t pW, void *stream);
int repdl_b200_conv2d_grad_kernel(const float *grad_output, const float *input,
                                  float *grad_kernel, int64_t N, int64_t IC, int64_t H,
                                  int64_t W, int64_t OC, int64_t KH, int64_t KW, int64_t sH,
                                  int64_t sW, int64_t pH, int64_t pW, void *stream);

/* The weight gradient and the bias gradient of one convolution in one pass over grad_output:
 * replaces the pair of calls in Conv2dFunction.backward, repdl/nn/conv.py:45-50
 * (ops.conv2d_grad_kernel, then ops.sum4d_dim023(grad_output)); grad_bias[oc] is the chain over
 * n, oh, ow of backend/cpu/summation.cpp (sum4d_dim023, no averaging), bit for bit.  Offered for the
 * shapes the row-chunk kernel takes (at least 256 chain steps and output rows of a useful length);
 * REPDL_E_UNSUPPORTED otherwise, and the caller makes the two separate calls. */
int repdl_b200_conv2d_grad_kernel_bias(const float *grad_output, const float *input,
                                       float *grad_kernel, float *grad_bias, int64_t N, int64_t IC,
                                       int64_t H, int64_t W, int64_t OC, int64_t KH, int64_t KW,
                                       int64_t sH, int64_t sW, int64_t pH, int64_t pW, void *stream);

/* ---- fixed-order sums --------------------------------------------------------------------
 * Replace repdl::cuda::summation::{sum1d, sum2d_dim0, sum2d_dim1, sum4d_dim023}
 * (backend/cuda/summation.cu:33-43, 59-71, 94-105, 132-144); bits defined by
 * backend/cpu/summation.cpp:12-78: every result is a strict left-to-right fp32 chain from
 * +0, multiplied once by `factor` at the end (1.0f, or float(1.0/count) for a mean).
 *
 * sum1d reproduces one chain of n elements without walking it element by element (per-binade
 * integer summaries prepared in parallel, applied by one thread after an exact validity check;
 * see csrc/sum1d.cu).  It needs scratch: pass a buffer of at least
 * repdl_b200_sum1d_scratch_bytes(n) bytes (0 for short chains; about 1 MB + n/30 bytes otherwise),
 * 256-byte aligned; its contents on entry do not matter and it may be reused by the next call
 * on the same stream (calls that overlap on the GPU must not share it).  n is limited to
 * 2^36 - 2^15 elements (REPDL_E_RANGE beyond). */
size_t repdl_b200_sum1d_scratch_bytes(int64_t n);
int repdl_b200_sum1d(const float *x, float *out, int64_t n, float factor, void *scratch,
                     size_t scratch_bytes, void *stream);
/* Diagnostics (no counterpart in the reference): what the walker of the last finished long-chain
 * call on `scratch` did.  stats must hold 12 values: [0..7) = items in the stream, summaries applied, leaves walked with
 * real adds, spans walked with real adds, leaves in those spans, composed soft runs that did not
 * fit the exact state, composed robust runs that did not fit; [7..12) = cycle counters of the walker
 * thread (zero unless the library was built with -DREPDL_SUM1D_CLOCKS=1).  Synchronous (one small copy). */
int repdl_b200_sum1d_stats(const void *scratch, long long *stats);
/* The same chain sum for callers that cannot allocate device memory at all.  (No counterpart in
 * the reference.)  Some hosts of this library are not allowed to call cudaMalloc or to go through
 * an allocating framework on the path that needs the sum: code running inside a CUDA-graph capture,
 * real-time or interrupt-like callbacks, a process whose memory pool is owned and fully handed out
 * by someone else, or a plugin ABI that only passes inputs and outputs.  For them the scratch of
 * repdl_b200_sum1d lives in a fixed array inside this library's device image (about 10 MB, held by
 * every GPU that loads the library until the process exits), so the caller passes only x and out.
 *   - n may be at most repdl_b200_sum1d_static_max_n() (2^28 elements); a longer chain returns
 *     REPDL_E_STATIC_MAX and does nothing.
 *   - The first call on each device, whatever its n, looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and sets a kernel attribute.  Make that
 *     first call before starting any stream capture.
 *   - Every call on a device shares the one array and it keeps the previous call's contents.
 *     Nothing in it has to be cleared (each call writes every word before reading it), but two calls
 *     whose kernels can overlap on the GPU (different streams) race on it: serialise them.
 *   - No cudaMalloc, cudaFree or other allocating call is made, on any call. */
int64_t repdl_b200_sum1d_static_max_n(void);
int repdl_b200_sum1d_static(const float *x, float *out, int64_t n, float factor, void *stream);
/* out[j] = factor * chain over i of x[i*N + j]   (M rows, N columns) */
int repdl_b200_sum2d_dim0(const float *x, float *out, int64_t M, int64_t N, float factor,
                          void *stream);
/* out[i] = factor * chain over j of x[i*N + j] */
int repdl_b200_sum2d_dim1(const float *x, float *out, int64_t M, int64_t N, float factor,
                          void *stream);
/* out[c] = factor * chain over (n, h*w) of x[n][c][h][w];  HW = H*W */
int repdl_b200_sum4d_dim023(const float *x, float *out, int64_t N, int64_t C, int64_t HW,
                            float factor, void *stream);

/* ---- elementwise math ----------------------------------------------------------------------
 * exp / log replace repdl::cuda::math::{exp2d, log1d} (backend/cuda/math.cu:20-66); bits defined
 * by backend/cpu/math.cpp:14-47: (float)exp((double)x), (float)log((double)x) with glibc's
 * double-precision libm, i.e. exact -> nearest fp64 -> nearest fp32.
 * div / sqrt replace what repdl/ops.py:98-103 and :122-123 compute through ATen: IEEE fp32
 * division and correctly rounded square root, with the x86 NaN conventions of the reference's
 * CPU run (NaN operands come back quieted with sign and payload kept; invalid operations give
 * 0xFFC00000 for div and 0x7FC00000 for sqrt of a negative). */
int repdl_b200_exp(const float *x, float *y, int64_t n, void *stream);
int repdl_b200_log(const float *x, float *y, int64_t n, void *stream);
int repdl_b200_sqrt(const float *x, float *y, int64_t n, void *stream);
int repdl_b200_div_scalar(const float *x, float divisor, float *y, int64_t n, void *stream);
int repdl_b200_div(const float *x, const float *divisor, float *y, int64_t n, void *stream);

/* ---- composites ------------------------------------------------------------------------------
 * Replace repdl::cuda::softmax::softmax (backend/cuda/softmax.cpp:15-21) and
 * repdl::cuda::cross_entropy::cross_entropy (backend/cuda/cross_entropy.cpp:15-24); bits defined by
 * backend/cpu/softmax.cpp:15-21 and backend/cpu/cross_entropy.cpp:15-24.  x is [M][N]; target holds
 * M int64 class indices.  cross_entropy writes one float (the mean loss) to `loss` and needs
 * M floats of scratch for the per-row terms. */
int repdl_b200_softmax(const float *x, float *y, int64_t M, int64_t N, void *stream);
int repdl_b200_cross_entropy(const float *x, const int64_t *target, float *loss, int64_t M,
                             int64_t N, float *row_scratch, void *stream);

/* Gradient of repdl_b200_cross_entropy with respect to x in one launch: replaces the softmax, one_hot,
 * subtraction and two scalings of CrossEntropyFunction.backward (repdl/nn/loss.py:29-33) with the same
 * separately rounded operations: (softmax(x) - one_hot(target)) * float(1.0 / M) * grad_loss[0].
 * grad_loss: one float on the device (the incoming gradient of the mean loss). */
int repdl_b200_cross_entropy_grad(const float *x, const int64_t *target, const float *grad_loss,
                                  float *grad_x, int64_t M, int64_t N, void *stream);

/* ---- optimizer steps ---------------------------------------------------------------------------
 * One launch updates up to 24 parameter tensors (more: several launches).  params / grads / ... are
 * HOST arrays of `ntensors` device pointers, sizes holds the element counts.  Every operation is
 * rounded separately in fp32 in the order of the Python update it replaces.
 *
 * repdl_b200_adam_step replaces the per-tensor loop of Adam.step, microsoft/RepDL
 * repdl/optim.py:56-83 (CUDA tensors reach ATen element-wise kernels and repdl.ops.sqrt / div there):
 *   g' = fma(p, weight_decay, g) if weight_decay != 0;  m = fma(g', 1-beta1, m*beta1);
 *   v = v*beta2 + (g'*g')*(1-beta2);  [vmax = maximum(vmax, v) if max_exp_avg_sq != NULL]
 *   p += (m / (sqrt(v or vmax) / sqrt_bias_correction2 + eps)) * neg_step_size
 * with the scalars already converted to fp32 the way ATen converts Python scalars
 * (neg_step_size = -(lr / bias_correction1)).
 *
 * repdl_b200_sgd_step: p += g * neg_lr (two roundings, the style of repdl/optim.py:83; the reference
 * itself ships no SGD). */
int repdl_b200_sgd_step(float *const *params, const float *const *grads, const int64_t *sizes,
                        int ntensors, float neg_lr, void *stream);
int repdl_b200_adam_step(float *const *params, const float *const *grads, float *const *exp_avg,
                         float *const *exp_avg_sq, float *const *max_exp_avg_sq,
                         const int64_t *sizes, int ntensors, float beta1, float one_minus_beta1,
                         float beta2, float one_minus_beta2, float sqrt_bias_correction2, float eps,
                         float neg_step_size, float weight_decay, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* REPDL_B200_H */
