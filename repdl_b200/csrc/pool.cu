// Max pooling over non-overlapping windows (kernel size = stride, no padding, no dilation) for sm_100a.
//
// Not an operator of the reference's backend: its layers call torch's max_pool2d, whose CUDA backward
// kernel is written for overlapping windows and is the slowest element-wise launch of the CNN training
// step.  Both kernels here are plain streams.  The forward kernel keeps ATen's selection rule -- scan
// the window row by row, take a value if it is greater than the maximum so far or is a NaN -- so the
// maximum and the position that receives the gradient are the ones torch picks (on the CPU as well:
// aten/src/ATen/native/cpu/MaxPoolKernel.cpp uses the same test).
#include "common.cuh"

namespace repdl_b200 {
namespace {

constexpr int POOL_THREADS = 256;

// (IT: unsigned for tensors below 2^31 elements -- 64-bit divisions cost more than the memory traffic)
template <typename IT>
__global__ void __launch_bounds__(POOL_THREADS)
maxpool_forward_kernel(const float *__restrict__ X, float *__restrict__ Y, int *__restrict__ IDX, int64_t total, int H,
                       int W, int OH, int OW, int KH, int KW)
{
    const IT stride = (IT)gridDim.x * POOL_THREADS, n = (IT)total;
    for (IT i = (IT)blockIdx.x * POOL_THREADS + threadIdx.x; i < n; i += stride) {
        const IT r = i / (IT)OW;
        const int ow = (int)(i - r * (IT)OW);
        const IT plane = r / (IT)OH;
        const int oh = (int)(r - plane * (IT)OH);
        const float *xp = X + (int64_t)plane * H * W;
        const int h0 = oh * KH, w0 = ow * KW;
        float best = -__int_as_float(0x7F800000);  // -inf
        int at = h0 * W + w0;
        for (int kh = 0; kh < KH; kh++) {
            for (int kw = 0; kw < KW; kw++) {
                const int p = (h0 + kh) * W + w0 + kw;
                const float v = __ldg(xp + p);
                if (v > best || v != v) best = v, at = p;
            }
        }
        Y[i] = best;
        IDX[i] = at;
    }
}

// Every input element lies in at most one window; it receives that window's gradient if it is the
// element the forward pass selected, else zero (elements below or right of the last whole window: zero).
template <typename IT>
__global__ void __launch_bounds__(POOL_THREADS)
maxpool_backward_kernel(const float *__restrict__ GY, const int *__restrict__ IDX, float *__restrict__ GX,
                        int64_t total, int H, int W, int OH, int OW, int KH, int KW)
{
    const IT stride = (IT)gridDim.x * POOL_THREADS, n = (IT)total;
    for (IT i = (IT)blockIdx.x * POOL_THREADS + threadIdx.x; i < n; i += stride) {
        const IT r = i / (IT)W;
        const int w = (int)(i - r * (IT)W);
        const IT plane = r / (IT)H;
        const int h = (int)(r - plane * (IT)H);
        const int oh = h / KH, ow = w / KW;
        float g = 0.0f;
        if (oh < OH && ow < OW) {
            const int64_t o = ((int64_t)plane * OH + oh) * OW + ow;
            if (__ldg(IDX + o) == h * W + w) g = __ldg(GY + o);
        }
        GX[i] = g;
    }
}

// four consecutive columns per thread (W a multiple of 4, 16-byte aligned gradient): one row decode and one
// 16-byte store for four elements
__global__ void __launch_bounds__(POOL_THREADS)
maxpool_backward4_kernel(const float *__restrict__ GY, const int *__restrict__ IDX, float *__restrict__ GX,
                         unsigned total4, int H, int W, int OH, int OW, int KH, int KW)
{
    const unsigned stride = gridDim.x * POOL_THREADS, W4 = (unsigned)W / 4;
    for (unsigned i = blockIdx.x * POOL_THREADS + threadIdx.x; i < total4; i += stride) {
        const unsigned r = i / W4;
        const int w0 = (int)(i - r * W4) * 4;
        const unsigned plane = r / (unsigned)H;
        const int h = (int)(r - plane * (unsigned)H);
        const int oh = h / KH;
        float g[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (oh < OH) {
            const int64_t orow = ((int64_t)plane * OH + oh) * OW;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int ow = (w0 + j) / KW;
                if (ow < OW && __ldg(IDX + orow + ow) == h * W + w0 + j) g[j] = __ldg(GY + orow + ow);
            }
        }
        *reinterpret_cast<float4 *>(GX + (int64_t)i * 4) = make_float4(g[0], g[1], g[2], g[3]);
    }
}

static unsigned pool_grid(int64_t total)
{
    int64_t blocks = (total + POOL_THREADS - 1) / POOL_THREADS;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_maxpool2d(const float *x, float *y, int *index, int64_t planes, int64_t H, int64_t W,
                                    int64_t KH, int64_t KW, void *stream)
{
    clear_stale_error();
    if (planes < 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || KH > H || KW > W) return REPDL_E_SHAPE;
    if (H * W >= 0x7FFFFFFF) return REPDL_E_RANGE;
    const int64_t OH = H / KH, OW = W / KW, total = planes * OH * OW;
    if (total == 0) return REPDL_OK;
    if (!x || !y || !index) return REPDL_E_NULL;
    if (planes * H * W < 0x7FFFFFFF)
        maxpool_forward_kernel<unsigned><<<pool_grid(total), POOL_THREADS, 0, (cudaStream_t)stream>>>(
            x, y, index, total, (int)H, (int)W, (int)OH, (int)OW, (int)KH, (int)KW);
    else
        maxpool_forward_kernel<int64_t><<<pool_grid(total), POOL_THREADS, 0, (cudaStream_t)stream>>>(
            x, y, index, total, (int)H, (int)W, (int)OH, (int)OW, (int)KH, (int)KW);
    return launch_status();
}

extern "C" int repdl_b200_maxpool2d_backward(const float *grad_y, const int *index, float *grad_x, int64_t planes,
                                             int64_t H, int64_t W, int64_t KH, int64_t KW, void *stream)
{
    clear_stale_error();
    if (planes < 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || KH > H || KW > W) return REPDL_E_SHAPE;
    if (H * W >= 0x7FFFFFFF) return REPDL_E_RANGE;
    const int64_t OH = H / KH, OW = W / KW, total = planes * H * W;
    if (total == 0) return REPDL_OK;
    if (!grad_y || !index || !grad_x) return REPDL_E_NULL;
    if (total < 0x7FFFFFFF && W % 4 == 0 && aligned16(grad_x))
        maxpool_backward4_kernel<<<pool_grid(total / 4), POOL_THREADS, 0, (cudaStream_t)stream>>>(
            grad_y, index, grad_x, (unsigned)(total / 4), (int)H, (int)W, (int)OH, (int)OW, (int)KH, (int)KW);
    else if (total < 0x7FFFFFFF)
        maxpool_backward_kernel<unsigned><<<pool_grid(total), POOL_THREADS, 0, (cudaStream_t)stream>>>(
            grad_y, index, grad_x, total, (int)H, (int)W, (int)OH, (int)OW, (int)KH, (int)KW);
    else
        maxpool_backward_kernel<int64_t><<<pool_grid(total), POOL_THREADS, 0, (cudaStream_t)stream>>>(
            grad_y, index, grad_x, total, (int)H, (int)W, (int)OH, (int)OW, (int)KH, (int)KW);
    return launch_status();
}
