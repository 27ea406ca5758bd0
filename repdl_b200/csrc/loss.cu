// Fused softmax and cross-entropy for sm_100a, with the per-element operation order of
// microsoft/RepDL backend/cpu/softmax.cpp:15-21 and backend/cpu/cross_entropy.cpp:15-24:
//   z_ij = x_ij - max_j x_ij                       (one fp32 subtraction)
//   e_ij = (float)exp((double)z_ij)                (crmath.cuh)
//   s_i  = e_i0 + e_i1 + ... left to right         (fp32 chain from +0)
//   softmax:        y_ij = e_ij / s_i              (IEEE division)
//   cross entropy:  l_i = (float)log((double)s_i) - z_i,target_i ; loss = float(1.0/M) * (l_0 + l_1 + ...)
// The reference needs ten launches for a [256, 10] input; here a row is one thread's work and the
// whole op is one launch (softmax) or two (cross entropy: rows, then the chain over rows).
#include "common.cuh"
#include "crmath.cuh"

namespace repdl_b200 {
namespace {

constexpr int LOSS_THREADS = 128;

// Row maximum the way ATen's max(dim) defines it: a NaN anywhere in the row wins.
__device__ __forceinline__ float row_max(const float *__restrict__ row, int64_t N)
{
    float m = __ldg(row);
    for (int64_t j = 1; j < N; j++) {
        float v = __ldg(row + j);
        if (v != v) {
            if (m == m) m = v;
        } else if (m == m && v > m) {
            m = v;
        }
    }
    return m;
}

__global__ void __launch_bounds__(LOSS_THREADS)
softmax_rows_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t M, int64_t N)
{
    int64_t i = (int64_t)blockIdx.x * LOSS_THREADS + threadIdx.x;
    if (i >= M) return;
    const float *row = x + i * N;
    float *out = y + i * N;
    const float m = row_max(row, N);
    float s = 0.0f;
    for (int64_t j = 0; j < N; j++) {
        float e = cr_exp(__fsub_rn(__ldg(row + j), m));
        out[j] = e;
        s = __fadd_rn(s, e);
    }
    for (int64_t j = 0; j < N; j++) out[j] = cr_div(out[j], s);
}

__global__ void __launch_bounds__(LOSS_THREADS)
xent_rows_kernel(const float *__restrict__ x, const int64_t *__restrict__ target,
                 float *__restrict__ per_row, int64_t M, int64_t N)
{
    int64_t i = (int64_t)blockIdx.x * LOSS_THREADS + threadIdx.x;
    if (i >= M) return;
    const float *row = x + i * N;
    const float m = row_max(row, N);
    float s = 0.0f;
    for (int64_t j = 0; j < N; j++) s = __fadd_rn(s, cr_exp(__fsub_rn(__ldg(row + j), m)));
    const int64_t t = target[i];
    // an out-of-range class index has no defined result in the reference (ATen's gather raises);
    // here it yields NaN instead of reading outside the row
    const float zt = (t >= 0 && t < N) ? __fsub_rn(__ldg(row + t), m) : __uint_as_float(0x7FC00000u);
    per_row[i] = __fsub_rn(cr_log(s), zt);
}

// Gradient of the mean cross-entropy loss with respect to the logits, one row per thread: the softmax
// of softmax_rows_kernel, then the three separately rounded steps of the reference's backward
// (repdl/nn/loss.py:29-33): minus one_hot(target), times float(1 / M), times the incoming gradient.
__global__ void __launch_bounds__(LOSS_THREADS)
xent_grad_rows_kernel(const float *__restrict__ x, const int64_t *__restrict__ target, const float *__restrict__ g,
                      float *__restrict__ y, int64_t M, int64_t N, float inv_m)
{
    int64_t i = (int64_t)blockIdx.x * LOSS_THREADS + threadIdx.x;
    if (i >= M) return;
    const float *row = x + i * N;
    float *out = y + i * N;
    const float m = row_max(row, N);
    float s = 0.0f;
    for (int64_t j = 0; j < N; j++) {
        float e = cr_exp(__fsub_rn(__ldg(row + j), m));
        out[j] = e;
        s = __fadd_rn(s, e);
    }
    const int64_t t = target[i];
    const float gin = __ldg(g);
    for (int64_t j = 0; j < N; j++) {
        float v = __fsub_rn(cr_div(out[j], s), j == t ? 1.0f : 0.0f);
        v = __fmul_rn(v, inv_m);
        out[j] = __fmul_rn(v, gin);
    }
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_cross_entropy_grad(const float *x, const int64_t *target, const float *grad_loss,
                                             float *grad_x, int64_t M, int64_t N, void *stream)
{
    clear_stale_error();
    if (M <= 0 || N <= 0) return REPDL_E_SHAPE;
    if (!x || !target || !grad_loss || !grad_x) return REPDL_E_NULL;
    int64_t blocks = (M + LOSS_THREADS - 1) / LOSS_THREADS;
    if (blocks > 0x7FFFFFFF) return REPDL_E_RANGE;
    xent_grad_rows_kernel<<<(unsigned)blocks, LOSS_THREADS, 0, (cudaStream_t)stream>>>(
        x, target, grad_loss, grad_x, M, N, (float)(1.0 / (double)M));
    return launch_status();
}

extern "C" int repdl_b200_softmax(const float *x, float *y, int64_t M, int64_t N, void *stream)
{
    clear_stale_error();
    if (M < 0 || N < 0) return REPDL_E_SHAPE;
    if (M == 0 || N == 0) return REPDL_OK;
    if (!x || !y) return REPDL_E_NULL;
    int64_t blocks = (M + LOSS_THREADS - 1) / LOSS_THREADS;
    if (blocks > 0x7FFFFFFF) return REPDL_E_RANGE;
    softmax_rows_kernel<<<(unsigned)blocks, LOSS_THREADS, 0, (cudaStream_t)stream>>>(x, y, M, N);
    return launch_status();
}

extern "C" int repdl_b200_cross_entropy(const float *x, const int64_t *target, float *loss,
                                        int64_t M, int64_t N, float *row_scratch, void *stream)
{
    clear_stale_error();
    if (M <= 0 || N <= 0) return REPDL_E_SHAPE;
    if (!x || !target || !loss) return REPDL_E_NULL;
    if (!row_scratch) return REPDL_E_SCRATCH;
    int64_t blocks = (M + LOSS_THREADS - 1) / LOSS_THREADS;
    if (blocks > 0x7FFFFFFF) return REPDL_E_RANGE;
    xent_rows_kernel<<<(unsigned)blocks, LOSS_THREADS, 0, (cudaStream_t)stream>>>(x, target,
                                                                                 row_scratch, M, N);
    int e = launch_status();
    if (e) return e;
    // mean over rows: the same single chain as sum1d with factor float(1.0 / M)
    // (backend/cpu/summation.cpp:15)
    const float factor = (float)(1.0 / (double)M);
    return sum1d_plain(row_scratch, loss, M, factor, (cudaStream_t)stream);
}
