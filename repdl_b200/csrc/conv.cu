// Bit-reproducible 2-D convolution (forward, input gradient, kernel gradient) for sm_100a.
//
// Contract (microsoft/RepDL backend/cpu/convolution.cpp:12-128): every output element is ONE fp32
// accumulator started at +0 and updated with a single-rounding fmaf per tap in the reference's
// loop order; taps that fall into the padding are SKIPPED (not multiplied by zero -- a zero
// product would turn an accumulator of -0 into +0 and a non-finite weight into NaN).
//
// The kernels in this file are the direct form: one thread owns one output element and walks its
// chain exactly as the reference's loops do.  Threads of a warp own adjacent output elements, so
// the loads of one tap are coalesced along the innermost dimension.
#include "common.cuh"

namespace repdl_b200 {
namespace {

struct ConvDims {
    int N, IC, H, W, OC, KH, KW, OH, OW, sH, sW, pH, pW, groups;
};

constexpr int CONV_THREADS = 128;

// conv2d: backend/cpu/convolution.cpp:24-50.  Thread -> (n, oc, oh, ow) with ow fastest.
__global__ void __launch_bounds__(CONV_THREADS)
conv2d_direct_kernel(const float *__restrict__ I, const float *__restrict__ Kw,
                     float *__restrict__ O, ConvDims d, int64_t total)
{
    int64_t idx = (int64_t)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (idx >= total) return;
    int ow = (int)(idx % d.OW);
    int64_t r = idx / d.OW;
    int oh = (int)(r % d.OH);
    r /= d.OH;
    int oc = (int)(r % d.OC);
    int n = (int)(r / d.OC);
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    const int g = oc / OCg;
    const int h0 = oh * d.sH - d.pH, w0 = ow * d.sW - d.pW;
    const float *ip = I + ((int64_t)n * d.IC + (int64_t)g * ICg) * d.H * d.W;
    const float *kp = Kw + (int64_t)oc * ICg * d.KH * d.KW;
    float acc = 0.0f;
    for (int i = 0; i < ICg; i++) {
        for (int kh = 0; kh < d.KH; kh++) {
            int h = h0 + kh;
            if (h < 0 || h >= d.H) continue;
            for (int kw = 0; kw < d.KW; kw++) {
                int w = w0 + kw;
                if (w < 0 || w >= d.W) continue;
                acc = __fmaf_rn(__ldg(ip + ((int64_t)i * d.H + h) * d.W + w),
                                __ldg(kp + (i * d.KH + kh) * d.KW + kw), acc);
            }
        }
    }
    O[idx] = acc;
}

// conv2d_grad_input: backend/cpu/convolution.cpp:65-88.  Thread -> (n, ic, h, w), w fastest.
// The reference computes oh = (h - kh + pH) / sH with C++ truncating division and keeps the tap
// only if the remainder is zero and 0 <= oh < OH; a negative numerator is never kept (either the
// quotient is negative, or it truncates to 0 with a non-zero remainder).
__global__ void __launch_bounds__(CONV_THREADS)
conv2d_grad_input_direct_kernel(const float *__restrict__ GO, const float *__restrict__ Kw,
                                float *__restrict__ GI, ConvDims d, int64_t total)
{
    int64_t idx = (int64_t)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (idx >= total) return;
    int w = (int)(idx % d.W);
    int64_t r = idx / d.W;
    int h = (int)(r % d.H);
    r /= d.H;
    int ic = (int)(r % d.IC);
    int n = (int)(r / d.IC);
    const float *gp = GO + (int64_t)n * d.OC * d.OH * d.OW;
    float acc = 0.0f;
    for (int oc = 0; oc < d.OC; oc++) {
        const float *kp = Kw + ((int64_t)oc * d.IC + ic) * d.KH * d.KW;
        for (int kh = 0; kh < d.KH; kh++) {
            int nh = h - kh + d.pH;
            if (nh < 0) continue;
            int oh = nh / d.sH;
            if (oh >= d.OH || oh * d.sH != nh) continue;
            for (int kw = 0; kw < d.KW; kw++) {
                int nw = w - kw + d.pW;
                if (nw < 0) continue;
                int ow = nw / d.sW;
                if (ow >= d.OW || ow * d.sW != nw) continue;
                acc = __fmaf_rn(__ldg(gp + ((int64_t)oc * d.OH + oh) * d.OW + ow),
                                __ldg(kp + kh * d.KW + kw), acc);
            }
        }
    }
    GI[idx] = acc;
}

// conv2d_grad_kernel: backend/cpu/convolution.cpp:102-126.  Thread -> (oc, ic, kh, kw); the chain
// runs over (n, oh, ow) -- batch * OH * OW steps that cannot be split.
__global__ void __launch_bounds__(CONV_THREADS)
conv2d_grad_kernel_direct_kernel(const float *__restrict__ GO, const float *__restrict__ I,
                                 float *__restrict__ GK, ConvDims d, int64_t total)
{
    int64_t idx = (int64_t)blockIdx.x * CONV_THREADS + threadIdx.x;
    if (idx >= total) return;
    int kw = (int)(idx % d.KW);
    int64_t r = idx / d.KW;
    int kh = (int)(r % d.KH);
    r /= d.KH;
    int ic = (int)(r % d.IC);
    int oc = (int)(r / d.IC);
    float acc = 0.0f;
    for (int n = 0; n < d.N; n++) {
        const float *gp = GO + ((int64_t)n * d.OC + oc) * d.OH * d.OW;
        const float *ip = I + ((int64_t)n * d.IC + ic) * d.H * d.W;
        for (int oh = 0; oh < d.OH; oh++) {
            int h = oh * d.sH - d.pH + kh;
            if (h < 0 || h >= d.H) continue;
            for (int ow = 0; ow < d.OW; ow++) {
                int w = ow * d.sW - d.pW + kw;
                if (w < 0 || w >= d.W) continue;
                acc = __fmaf_rn(__ldg(gp + oh * d.OW + ow), __ldg(ip + h * d.W + w), acc);
            }
        }
    }
    GK[idx] = acc;
}

int fill_dims(ConvDims &d, int64_t N, int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH,
              int64_t KW, int64_t sH, int64_t sW, int64_t pH, int64_t pW, int64_t groups)
{
    if (N < 0 || IC <= 0 || H <= 0 || W <= 0 || OC <= 0 || KH <= 0 || KW <= 0 || sH <= 0 ||
        sW <= 0 || pH < 0 || pW < 0 || groups <= 0)
        return REPDL_E_SHAPE;
    if (IC % groups || OC % groups) return REPDL_E_SHAPE;
    if (H + 2 * pH < KH || W + 2 * pW < KW) return REPDL_E_SHAPE;
    const int64_t lim = 0x7FFFFFFF;
    if (N > lim || IC > lim || H > lim || W > lim || OC > lim || KH > lim || KW > lim || sH > lim ||
        sW > lim || pH > lim || pW > lim)
        return REPDL_E_RANGE;
    if (IC * KH * KW > lim || H * W > lim) return REPDL_E_RANGE;
    d.N = (int)N; d.IC = (int)IC; d.H = (int)H; d.W = (int)W; d.OC = (int)OC;
    d.KH = (int)KH; d.KW = (int)KW; d.sH = (int)sH; d.sW = (int)sW; d.pH = (int)pH; d.pW = (int)pW;
    d.groups = (int)groups;
    d.OH = (int)((H + 2 * pH - KH) / sH + 1);
    d.OW = (int)((W + 2 * pW - KW) / sW + 1);
    return REPDL_OK;
}

int blocks_for(int64_t total, unsigned &blocks)
{
    int64_t b = (total + CONV_THREADS - 1) / CONV_THREADS;
    if (b > 0x7FFFFFFF) return REPDL_E_RANGE;
    blocks = (unsigned)b;
    return REPDL_OK;
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_conv2d(const float *input, const float *kernel, float *output, int64_t N,
                                 int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH,
                                 int64_t KW, int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                                 int64_t groups, void *stream)
{
    clear_stale_error();
    ConvDims d;
    int e = fill_dims(d, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW, groups);
    if (e) return e;
    int64_t total = (int64_t)d.N * d.OC * d.OH * d.OW;
    if (total == 0) return REPDL_OK;
    if (!input || !kernel || !output) return REPDL_E_NULL;
    unsigned blocks;
    if ((e = blocks_for(total, blocks))) return e;
    conv2d_direct_kernel<<<blocks, CONV_THREADS, 0, (cudaStream_t)stream>>>(input, kernel, output,
                                                                            d, total);
    return launch_status();
}

extern "C" int repdl_b200_conv2d_grad_input(const float *grad_output, const float *kernel,
                                            float *grad_input, int64_t N, int64_t IC, int64_t H,
                                            int64_t W, int64_t OC, int64_t KH, int64_t KW,
                                            int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                                            void *stream)
{
    clear_stale_error();
    ConvDims d;
    int e = fill_dims(d, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW, 1);
    if (e) return e;
    int64_t total = (int64_t)d.N * d.IC * d.H * d.W;
    if (total == 0) return REPDL_OK;
    if (!grad_output || !kernel || !grad_input) return REPDL_E_NULL;
    unsigned blocks;
    if ((e = blocks_for(total, blocks))) return e;
    conv2d_grad_input_direct_kernel<<<blocks, CONV_THREADS, 0, (cudaStream_t)stream>>>(
        grad_output, kernel, grad_input, d, total);
    return launch_status();
}

extern "C" int repdl_b200_conv2d_grad_kernel(const float *grad_output, const float *input,
                                             float *grad_kernel, int64_t N, int64_t IC, int64_t H,
                                             int64_t W, int64_t OC, int64_t KH, int64_t KW,
                                             int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                                             void *stream)
{
    clear_stale_error();
    ConvDims d;
    int e = fill_dims(d, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW, 1);
    if (e) return e;
    int64_t total = (int64_t)d.OC * d.IC * d.KH * d.KW;
    if (!grad_output || !input || !grad_kernel) return REPDL_E_NULL;
    unsigned blocks;
    if ((e = blocks_for(total, blocks))) return e;
    conv2d_grad_kernel_direct_kernel<<<blocks, CONV_THREADS, 0, (cudaStream_t)stream>>>(
        grad_output, input, grad_kernel, d, total);
    return launch_status();
}
