// Bit-reproducible 2-D convolution (forward, input gradient, kernel gradient) for sm_100a.
//
// Contract (microsoft/RepDL backend/cpu/convolution.cpp:12-128): every output element is ONE fp32
// accumulator started at +0 and updated with a single-rounding fmaf per tap in the reference's
// loop order; taps that fall into the padding are SKIPPED (not multiplied by zero -- a zero
// product would turn an accumulator of -0 into +0 and a non-finite weight into NaN).
//
// Three forms live in this file.
//   direct : one thread owns one output element and walks its chain exactly as the reference's
//            loops do (always exact; used for kernels with more than 64 taps, for gradients with
//            very short chains and as the per-tile fallback of the other forms);
//   chains : conv2d_grad_kernel -- few outputs, each a chain over batch x OH x OW steps: warps that
//            only multiply (one chain per thread) fed by warps that only stage operands into shared
//            memory, see the two kernels further down; optionally with the bias gradient fused in;
//   GEMM   : conv2d and conv2d_grad_input as an implicit GEMM on the FP32 FMA pipe -- the same
//            register-blocked main loop as mm (8 x 8 outputs per thread, K in slabs of 16 through
//            double-buffered shared memory), with the im2col matrix gathered on the fly.  A tap that
//            falls into the padding enters the FMA as +0.0 instead of being skipped.  That is the
//            identity for every accumulator except -0, and an accumulator that started at +0 can
//            only become -0 when a non-zero product underflows to zero; so each CTA watches its
//            operands while loading them and, if it meets a non-finite value or a non-zero value
//            below 2^-51 (sums of products of larger values cannot round to zero), discards its tile
//            and recomputes it with the direct form.  Wrong bits are therefore impossible, not
//            merely unlikely.
#include "common.cuh"

namespace repdl_b200 {
namespace {

struct ConvDims {
    int N, IC, H, W, OC, KH, KW, OH, OW, sH, sW, pH, pW, groups;
    unsigned long long m40_khw, m40_kw, m40_ow;  // ceil(2^40 / (KH*KW)), / KW, / OW: division by multiplication
    // epilogue of the forward convolution (repdl_b200_conv2d_bias_act): bias[oc] is added to the finished
    // chain with one separately rounded fp32 addition, then max(., 0); both are what the layer's own
    // element-wise kernels would do to the stored result, so the bits are the same
    const float *bias;
    int relu;
};

// the two epilogue steps on one finished output of channel oc (NaN passes through the maximum, as in ATen's clamp)
__device__ __forceinline__ float conv_finish(float v, const ConvDims &d, int oc)
{
    if (d.bias) v = __fadd_rn(v, __ldg(d.bias + oc));
    if (d.relu) v = v != v ? v : fmaxf(v, 0.0f);
    return v;
}

// k / dv with m40 = ceil(2^40 / dv): exact whenever k * dv < 2^40 (callers keep k < 2^24, dv < 2^16).
__device__ __forceinline__ int fastdiv(int k, unsigned long long m40)
{
    return (int)(((unsigned long long)(unsigned)k * m40) >> 40);
}

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
    O[idx] = conv_finish(acc, d, oc);
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

// ------------------------------------------------------------------------------------------------
// exact per-element chains as device functions (the fallback of the GEMM form)
// ------------------------------------------------------------------------------------------------
__device__ __noinline__ float conv2d_exact(const float *__restrict__ I, const float *__restrict__ Kw,
                                              const ConvDims &d, int n, int oc, int oh, int ow)
{
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    const int g = oc / OCg;
    const int h0 = oh * d.sH - d.pH, w0 = ow * d.sW - d.pW;
    const float *ip = I + ((int64_t)n * d.IC + (int64_t)g * ICg) * d.H * d.W;
    const float *kp = Kw + (int64_t)oc * ICg * d.KH * d.KW;
    float acc = 0.0f;
    for (int i = 0; i < ICg; i++)
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
    return acc;
}

__device__ __noinline__ float conv2d_grad_input_exact(const float *__restrict__ GO,
                                                         const float *__restrict__ Kw,
                                                         const ConvDims &d, int n, int ic, int h, int w)
{
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
    return acc;
}

// ------------------------------------------------------------------------------------------------
// implicit GEMM.  MODE 0: conv2d        C[oc][col] , col = (n, oh, ow), k = (ic, kh, kw)
//                 MODE 1: grad_input    C[ic][col] , col = (n, h, w),   k = (oc, kh, kw)
// ------------------------------------------------------------------------------------------------
constexpr int CG_BK = 16, CG_BN = 128;

// Value needs the exact path: non-finite, or non-zero and below 2^-51.  With every non-zero operand
// at least 2^-51 in magnitude every product is a multiple of 2^-102 and at least 2^-102, far above the
// subnormal range, so no product underflows and no sum of such values can round to zero from a
// non-zero exact value: an accumulator that started at +0 then never becomes -0 (an exact
// cancellation gives +0), which is what makes a +0.0 padding tap the identity.
__device__ __forceinline__ bool cg_unsafe(float v)
{
    const unsigned ax = __float_as_uint(v) & 0x7FFFFFFFu;
    return (ax - 1u < 0x25FFFFFFu) || ax >= 0x7F800000u;  // 0 < |v| < 2^-51, or inf / NaN
}

template <int BM, int MODE, bool S1>  // S1: stride 1 in both directions (no divisions in the gather)
__global__ void __launch_bounds__((BM / 8) * (CG_BN / 8))
conv_gemm_kernel(const float *__restrict__ Src, const float *__restrict__ Kw, float *__restrict__ Out,
                 ConvDims d)
{
    constexpr int NT = (BM / 8) * (CG_BN / 8);
    constexpr int PA = BM + 4, PB = CG_BN + 4;
    constexpr int NVA = BM * CG_BK / 4 / NT;     // 4-element groups of A per thread per slab
    constexpr int NVB = CG_BN * CG_BK / 4 / NT;  // 4-column groups of B per thread per slab
    __shared__ __align__(16) float As[2][CG_BK][PA];
    __shared__ __align__(16) float Bs[2][CG_BK][PB];

    const int t = threadIdx.x, lane = t & 31, wid = t >> 5;
    const int tx = (wid % 2) * 8 + (lane & 7);   // 16 threads along the columns
    const int ty = (wid / 2) * 4 + (lane >> 3);  // BM / 8 threads along the rows
    const int g = blockIdx.z;
    const int KHW = d.KH * d.KW;
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    // GEMM extents and the geometry of the gathered operand
    const int M = MODE == 0 ? OCg : d.IC;
    const int K = MODE == 0 ? ICg * KHW : d.OC * KHW;
    const int outW = MODE == 0 ? d.OW : d.W, outHW = MODE == 0 ? d.OH * d.OW : d.H * d.W;
    const int srcH = MODE == 0 ? d.H : d.OH, srcW = MODE == 0 ? d.W : d.OW;
    const int srcPlanes = MODE == 0 ? d.IC : d.OC;
    const int64_t ncols = (int64_t)d.N * outHW;
    const int m0 = blockIdx.y * BM;
    const int64_t col0 = (int64_t)blockIdx.x * CG_BN;

    // ---- B gather: this thread always serves the same 4 columns ----
    const int bxq = t % (CG_BN / 4), bk0 = t / (CG_BN / 4);  // NT is a multiple of CG_BN / 4
    int64_t b_base[4];
    int b_y[4], b_x[4];
    bool b_ok[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int64_t col = col0 + bxq * 4 + j;
        b_ok[j] = col < ncols;
        const int64_t cc = b_ok[j] ? col : 0;
        const int n = (int)(cc / outHW), p = (int)(cc % outHW);
        b_y[j] = p / outW, b_x[j] = p % outW;
        b_base[j] = ((int64_t)n * srcPlanes + (MODE == 0 ? g * ICg : 0)) * srcH * srcW;
    }
    // Whenever the source position is linear in (kh, kw) -- conv2d at any stride, grad_input at
    // stride 1 -- an element's address is (a term of the column) + (a term of k), and whether the tap
    // falls into the padding is one bit of a per-column mask over the KH * KW <= 64 taps; both
    // column terms are computed once, so an element costs a shift, a test, an add and the load.
    constexpr bool LIN = MODE == 0 || S1;
    const float *b_ptr[4];
    unsigned long long b_mask[4];
    if (LIN) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int y0 = MODE == 0 ? b_y[j] * d.sH - d.pH : b_y[j] + d.pH;
            const int x0 = MODE == 0 ? b_x[j] * d.sW - d.pW : b_x[j] + d.pW;
            b_ptr[j] = Src + (b_base[j] + (int64_t)y0 * srcW + x0);
            unsigned long long m = 0;
            if (b_ok[j]) {
                for (int kh = 0, r = 0; kh < d.KH; kh++) {
                    const int sy = MODE == 0 ? y0 + kh : y0 - kh;
                    for (int kw = 0; kw < d.KW; kw++, r++) {
                        const int sx = MODE == 0 ? x0 + kw : x0 - kw;
                        if (sy >= 0 && sy < srcH && sx >= 0 && sx < srcW) m |= 1ull << r;
                    }
                }
            }
            b_mask[j] = m;
        }
    }
    // k-dependent half of the gather: tap index r and address term of k (LIN only)
    auto decodeK = [&](int k, int &r, int &kterm) {
        const int plane = fastdiv(k, d.m40_khw);
        r = k - plane * KHW;
        const int kh = fastdiv(r, d.m40_kw), kw = r - kh * d.KW;
        const int tap = kh * srcW + kw;
        kterm = plane * srcH * srcW + (MODE == 0 ? tap : -tap);
    };
    auto gatherB = [&](int k, int j) -> float {
        if (k >= K || !b_ok[j]) return 0.0f;
        const int plane = fastdiv(k, d.m40_khw), r = k - plane * KHW;
        const int kh = fastdiv(r, d.m40_kw), kw = r - kh * d.KW;
        int sy, sx;
        if (MODE == 0) {
            sy = b_y[j] * d.sH - d.pH + kh;
            sx = b_x[j] * d.sW - d.pW + kw;
            if (sy < 0 || sy >= srcH || sx < 0 || sx >= srcW) return 0.0f;
        } else {
            const int nh = b_y[j] + d.pH - kh, nw = b_x[j] + d.pW - kw;
            if (nh < 0 || nw < 0) return 0.0f;
            sy = nh / d.sH, sx = nw / d.sW;
            if (sy >= srcH || sx >= srcW || sy * d.sH != nh || sx * d.sW != nw) return 0.0f;
        }
        return __ldg(Src + b_base[j] + ((int64_t)plane * srcH + sy) * srcW + sx);
    };
    // ---- A fetch: weights.  MODE 0: row m of [OC][K]; MODE 1: (ic = m, k = (oc, r)) ----
    auto fetchA = [&](int m, int k) -> float {
        if (k >= K) return -0.0f;  // K tail: (-0) * (+0) = -0, the identity of the accumulation
        if (m >= M) return 0.0f;
        if (MODE == 0) return __ldg(Kw + ((int64_t)(g * OCg + m)) * K + k);
        const int oc = fastdiv(k, d.m40_khw), r = k - oc * KHW;
        return __ldg(Kw + ((int64_t)oc * d.IC + m) * KHW + r);
    };

    float av[NVA][4], bv[NVB][4];
    bool unsafe = false;
    auto load_slab = [&](int k0) {
#pragma unroll
        for (int i = 0; i < NVA; i++) {
            const int idx = t + NT * i;
            const int m = idx / (CG_BK / 4), kq = (idx % (CG_BK / 4)) * 4;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                av[i][e] = fetchA(m0 + m, k0 + kq + e);
                unsafe |= cg_unsafe(av[i][e]);
            }
        }
#pragma unroll
        for (int i = 0; i < NVB; i++) {
            const int k = k0 + bk0 + (NT / (CG_BN / 4)) * i;
            if (LIN) {
                int r = 0, kterm = 0;
                if (k < K) decodeK(k, r, kterm);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const bool ok = k < K && ((b_mask[j] >> r) & 1ull) != 0;
                    bv[i][j] = ok ? __ldg(b_ptr[j] + kterm) : 0.0f;
                    unsafe |= cg_unsafe(bv[i][j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    bv[i][j] = gatherB(k, j);
                    unsafe |= cg_unsafe(bv[i][j]);
                }
            }
        }
    };
    auto store_slab = [&](int buf) {
#pragma unroll
        for (int i = 0; i < NVA; i++) {
            const int idx = t + NT * i;
            const int m = idx / (CG_BK / 4), kq = (idx % (CG_BK / 4)) * 4;
#pragma unroll
            for (int e = 0; e < 4; e++) As[buf][kq + e][m] = av[i][e];
        }
#pragma unroll
        for (int i = 0; i < NVB; i++) {
            const int kl = bk0 + (NT / (CG_BN / 4)) * i;
            *reinterpret_cast<float4 *>(&Bs[buf][kl][bxq * 4]) = make_float4(bv[i][0], bv[i][1], bv[i][2], bv[i][3]);
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    const int nk = (K + CG_BK - 1) / CG_BK;
    load_slab(0);
    store_slab(0);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++) {
        const int cur = kt & 1;
        const bool more = kt + 1 < nk;
        if (more) load_slab((kt + 1) * CG_BK);
#pragma unroll
        for (int k = 0; k < CG_BK; k++) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[cur][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[cur][k][BM / 2 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[cur][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[cur][k][CG_BN / 2 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        if (more) store_slab(cur ^ 1);
        __syncthreads();
    }
    // did any thread of this CTA meet an operand that makes the +0 padding unsafe?
    const bool redo = __syncthreads_or(unsafe ? 1 : 0) != 0;

#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? ty * 4 + i : BM / 2 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t colq = col0 + (h ? CG_BN / 2 : 0) + tx * 4;
            if (colq >= ncols) continue;
            const int n = (int)(colq / outHW), p = (int)(colq % outHW);
            const int plane = MODE == 0 ? g * OCg + m : m;
            const int planes = MODE == 0 ? d.OC : d.IC;
            float c[4] = {acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]};
            if (redo) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int64_t col = colq + j;
                    if (col >= ncols) break;
                    const int nn = (int)(col / outHW), pp = (int)(col % outHW);
                    c[j] = MODE == 0 ? conv2d_exact(Src, Kw, d, nn, plane, pp / outW, pp % outW)
                                     : conv2d_grad_input_exact(Src, Kw, d, nn, plane, pp / outW, pp % outW);
                }
            }
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < 4; j++) c[j] = conv_finish(c[j], d, plane);
            }
            float *dst = Out + ((int64_t)n * planes + plane) * outHW + p;
            if (p + 3 < outHW && (outHW & 3) == 0 && (reinterpret_cast<uintptr_t>(Out) & 15u) == 0) {
                *reinterpret_cast<float4 *>(dst) = make_float4(c[0], c[1], c[2], c[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int64_t col = colq + j;
                    if (col >= ncols) break;
                    const int nn = (int)(col / outHW), pp = (int)(col % outHW);
                    Out[((int64_t)nn * planes + plane) * outHW + pp] = c[j];
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Stride-1 3 x 3 convolutions through a staged source window (conv2d, and conv2d_grad_input, which
// at stride 1 is a convolution of grad_output with the taps walked backwards).
//
// The on-the-fly im2col of conv_gemm_kernel costs address arithmetic, a load and an operand check
// per GATHERED element, i.e. 9 times per source element.  Here a CTA owns a strip of R output rows
// of one image for up to 64 output channels, and per chunk of 8 reduction planes it stages
//   * the source window of the strip (R + 2 rows, padding materialised as +0.0): 4-byte cp.async
//     copies from offsets that a thread computes once per CTA, and
//   * the chunk's weights, read along k with 16-byte loads and scattered to [k][channel]
// into double-buffered shared memory; every staged value is checked once.  The main loop then needs
// no index arithmetic: a thread owns 8 channels x 2 groups of 4 consecutive pixels of a row; for one
// (plane, kh) the 6 window values of a group arrive as two 16-byte loads and serve all 3 taps, so a
// k-step is 64 FFMA for 2 loads of weights and 2/3 of a load of pixels.  k runs (plane, kh, kw)
// ascending, the reference's chain order; planes past the end enter as (-0) * (+0) = -0, the
// identity.  Padding as +0.0 is exact under the same operand watch and per-tile exact fallback as
// conv_gemm_kernel.
// ------------------------------------------------------------------------------------------------
constexpr int CW_PC = 8;             // reduction planes per chunk
constexpr int CW_KC = CW_PC * 9;     // k-steps per chunk

struct WinGeom {
    int M, planes;       // GEMM rows (output channels of this launch); reduction planes
    int outH, outW;      // output image
    int srcH, srcW;      // source image
    int R, strips;       // output rows per strip; strips per image
    int G4, pairs;       // 4-pixel groups per output row; pairs of groups per CTA
    int WR, WP;          // window rows (R + 2); window pitch in floats (a multiple of 4)
    int y_off, x_off;    // window (0, 0) is source (strip's first output row + y_off, x_off)
    int active;          // threads that own outputs (OG * pairs); the rest only stage
    int vecw;            // weights may be read with 16-byte loads
};

#ifndef REPDL_CW_MINB
#define REPDL_CW_MINB 2
#endif
#ifndef REPDL_CW_UNROLL
#define REPDL_CW_UNROLL 1
#endif
template <int MODE, int OG, int NTH>
__global__ void __launch_bounds__(NTH, NTH <= 192 ? REPDL_CW_MINB : 1)
conv_window_kernel(const float *__restrict__ Src, const float *__restrict__ Kw, float *__restrict__ Out,
                   ConvDims d, WinGeom w)
{
    constexpr int BM = OG * 8, PA = BM + 4;
    constexpr int NWQ = (BM * CW_KC / 4 + NTH - 1) / NTH;  // 16-byte weight groups per thread
    extern __shared__ __align__(16) float cw_smem[];
    const int plane_floats = w.WR * w.WP;
    const int win_floats = CW_PC * plane_floats;
    const int stage_floats = win_floats + CW_KC * PA;
    const int t = threadIdx.x;
    constexpr int nt = NTH;
    const int og = t % OG, pair = t / OG;
    const int strip = blockIdx.x % w.strips, n = blockIdx.x / w.strips;
    const int m0 = blockIdx.y * BM, g = blockIdx.z;
    const int r0 = strip * w.R;
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    const int64_t srcHW = (int64_t)w.srcH * w.srcW;
    const float *src_n =
        Src + ((int64_t)n * (MODE == 0 ? d.IC : d.OC) + (MODE == 0 ? g * ICg : 0)) * srcHW;
    const int K = w.planes * 9;
    const bool owner = t < w.active;

    int grow[2], gcol[2];
    bool gok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int grp = pair + h * w.pairs;
        gok[h] = owner && grp < w.R * w.G4;
        const int gg = gok[h] ? grp : 0;
        grow[h] = gg / w.G4;
        gcol[h] = (gg - grow[h] * w.G4) * 4;
    }
    // where each window element comes from (the same for every plane): offset inside a source plane,
    // or -1 for padding; a table in shared memory, filled once per CTA
    int *woff = reinterpret_cast<int *>(cw_smem + 2 * stage_floats);
    for (int e = t; e < plane_floats; e += nt) {
        const int row = e / w.WP, col = e - row * w.WP;
        const int sy = r0 + w.y_off + row, sx = w.x_off + col;
        woff[e] = (sy >= 0 && sy < w.srcH && sx >= 0 && sx < w.srcW) ? sy * w.srcW + sx : -1;
    }
    __syncthreads();

    auto stage_window = [&](int chunk, float *win) {
        const float *sp = src_n + (int64_t)chunk * CW_PC * srcHW;
        const int np = min(CW_PC, w.planes - chunk * CW_PC);  // planes of this chunk that exist
        for (int e = t; e < plane_floats; e += nt) {
            const int off = woff[e];
            const float *s0 = sp + (off >= 0 ? off : 0);
            float *dst = win + e;
#pragma unroll
            for (int p = 0; p < CW_PC; p++) {
                const bool ok = off >= 0 && p < np;
                cp_async_4_zfill(dst + p * plane_floats, ok ? s0 + p * srcHW : sp, ok);
            }
        }
        cp_async_commit();
    };
    bool unsafe = false;
    auto check_window = [&](const float *win) {
        for (int e = t; e < plane_floats; e += nt) {
#pragma unroll
            for (int p = 0; p < CW_PC; p++) unsafe |= cg_unsafe(win[p * plane_floats + e]);
        }
    };
    // weights of one chunk: global -> registers (16 bytes along k) -> As[k][channel]
    float4 wq[NWQ];
    auto load_weights_slow = [&](int chunk) {
#pragma unroll
        for (int i = 0; i < NWQ; i++) {
            const int idx = t + i * nt;
            wq[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (idx >= BM * (CW_KC / 4)) continue;
            int ch, kl;
            const float *src;
            if (MODE == 0) {  // row (channel) of [OC][K], k contiguous
                ch = idx / (CW_KC / 4), kl = (idx - ch * (CW_KC / 4)) * 4;
                src = Kw + (int64_t)(g * OCg + m0 + ch) * K + chunk * CW_KC + kl;
            } else {  // plane p = oc: a contiguous block [IC][9]; here j = ic * 9 + r
                const int p = idx / (BM * 9 / 4), j = (idx - p * (BM * 9 / 4)) * 4;
                ch = j, kl = p;  // decoded element by element below
                src = Kw + ((int64_t)(chunk * CW_PC + p) * d.IC + m0) * 9 + j;
            }
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                bool in;
                if (MODE == 0)
                    in = m0 + ch < w.M && chunk * CW_KC + kl + e < K;
                else
                    in = m0 + (ch + e) / 9 < w.M && chunk * CW_PC + kl < w.planes;
                v[e] = 0.0f;
                if (in && !w.vecw) v[e] = __ldg(src + e);
            }
            if (w.vecw) {
                bool all;
                if (MODE == 0)
                    all = m0 + ch < w.M && chunk * CW_KC + kl + 3 < K;
                else
                    all = m0 + (ch + 3) / 9 < w.M && chunk * CW_PC + kl < w.planes;
                if (all) {
                    const float4 q = ldg_f4(src);
                    v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        bool in;
                        if (MODE == 0)
                            in = m0 + ch < w.M && chunk * CW_KC + kl + e < K;
                        else
                            in = m0 + (ch + e) / 9 < w.M && chunk * CW_PC + kl < w.planes;
                        if (in) v[e] = __ldg(src + e);
                    }
                }
            }
            wq[i] = make_float4(v[0], v[1], v[2], v[3]);
        }
    };
    auto store_weights_slow = [&](int chunk, float *As) {
#pragma unroll
        for (int i = 0; i < NWQ; i++) {
            const int idx = t + i * nt;
            if (idx >= BM * (CW_KC / 4)) continue;
            const float v[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int ch, kl;
                if (MODE == 0) {
                    ch = idx / (CW_KC / 4), kl = (idx - ch * (CW_KC / 4)) * 4 + e;
                } else {
                    const int p = idx / (BM * 9 / 4), j = (idx - p * (BM * 9 / 4)) * 4 + e;
                    ch = j / 9, kl = p * 9 + (j - ch * 9);
                }
                // past the last plane: (-0) * (+0) = -0, the identity; channels past M: zero rows
                const bool ktail = chunk * CW_KC + kl >= K;
                As[kl * PA + ch] = ktail ? -0.0f : v[e];
                unsafe |= cg_unsafe(v[e]);
            }
        }
    };

    // The usual case -- a full tile of channels, a full chunk of planes, 16-byte aligned weight rows --
    // works from offsets computed once per CTA: per group of 4 consecutive weights one global offset
    // (relative to the chunk) and the shared-memory positions of its 4 elements.
    const bool wfast = w.vecw && m0 + BM <= w.M;
    int wg_off[NWQ], ws_off[NWQ][MODE == 0 ? 1 : 4];
#pragma unroll
    for (int i = 0; i < NWQ; i++) {
        const int idx = t + i * nt;
        wg_off[i] = -1;
        if (idx < BM * (CW_KC / 4)) {
            if (MODE == 0) {
                const int ch = idx / (CW_KC / 4), kl = (idx - ch * (CW_KC / 4)) * 4;
                wg_off[i] = (g * OCg + m0 + ch) * K + kl;
                ws_off[i][0] = kl * PA + ch;
            } else {
                const int pp = idx / (BM * 9 / 4), j = (idx - pp * (BM * 9 / 4)) * 4;
                wg_off[i] = (pp * d.IC + m0) * 9 + j;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int ch = (j + e) / 9;
                    ws_off[i][MODE == 0 ? 0 : e] = (pp * 9 + (j + e - ch * 9)) * PA + ch;
                }
            }
        }
    }
    auto load_weights = [&](int chunk) {
        if (!(wfast && (chunk + 1) * CW_PC <= w.planes)) {
            load_weights_slow(chunk);
            return;
        }
        const float *base = Kw + (MODE == 0 ? (int64_t)chunk * CW_KC : (int64_t)chunk * CW_PC * d.IC * 9);
#pragma unroll
        for (int i = 0; i < NWQ; i++)
            if (wg_off[i] >= 0) wq[i] = ldg_f4(base + wg_off[i]);
    };
    auto store_weights = [&](int chunk, float *As) {
        if (!(wfast && (chunk + 1) * CW_PC <= w.planes)) {
            store_weights_slow(chunk, As);
            return;
        }
#pragma unroll
        for (int i = 0; i < NWQ; i++) {
            if (wg_off[i] < 0) continue;
            const float v[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                As[MODE == 0 ? ws_off[i][0] + e * PA : ws_off[i][MODE == 0 ? 0 : e]] = v[e];
                unsafe |= cg_unsafe(v[e]);
            }
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    const int nchunks = (w.planes + CW_PC - 1) / CW_PC;
    stage_window(0, cw_smem);
    load_weights(0);
    store_weights(0, cw_smem + win_floats);
    for (int c = 0; c < nchunks; c++) {
        float *cur = cw_smem + (c & 1) * stage_floats, *nxt = cw_smem + ((c + 1) & 1) * stage_floats;
        cp_async_wait<0>();
        check_window(cur);
        __syncthreads();  // chunk c is complete, and every thread has left chunk c - 1
        const bool more = c + 1 < nchunks;
        if (more) {
            stage_window(c + 1, nxt);
            load_weights(c + 1);
        }
        if (owner) {
            // 24 (plane, kh) rows: the window rows of both pixel groups and the weight rows advance
            // by constant strides (kh walks the window downwards for conv2d, upwards for grad_input)
            const float *row0 = cur + (grow[0] + (MODE == 0 ? 0 : 2)) * w.WP + gcol[0];
            const float *row1 = cur + (grow[1] + (MODE == 0 ? 0 : 2)) * w.WP + gcol[1];
            const float *ak = cur + win_floats + og * 4;
            const int step_kh = MODE == 0 ? w.WP : -w.WP;
            const int step_p = plane_floats - 3 * step_kh;
            constexpr int kUnroll = REPDL_CW_UNROLL;
#pragma unroll kUnroll
            for (int it = 0, kh = 0; it < CW_PC * 3; it++) {
                float bq[2][8];
                {
                    const float4 v0 = *reinterpret_cast<const float4 *>(row0);
                    const float4 v1 = *reinterpret_cast<const float4 *>(row0 + 4);
                    const float4 u0 = *reinterpret_cast<const float4 *>(row1);
                    const float4 u1 = *reinterpret_cast<const float4 *>(row1 + 4);
                    bq[0][0] = v0.x, bq[0][1] = v0.y, bq[0][2] = v0.z, bq[0][3] = v0.w;
                    bq[0][4] = v1.x, bq[0][5] = v1.y, bq[0][6] = v1.z, bq[0][7] = v1.w;
                    bq[1][0] = u0.x, bq[1][1] = u0.y, bq[1][2] = u0.z, bq[1][3] = u0.w;
                    bq[1][4] = u1.x, bq[1][5] = u1.y, bq[1][6] = u1.z, bq[1][7] = u1.w;
                }
#pragma unroll
                for (int kw = 0; kw < 3; kw++) {
                    const float4 a0 = *reinterpret_cast<const float4 *>(ak + kw * PA);
                    const float4 a1 = *reinterpret_cast<const float4 *>(ak + kw * PA + BM / 2);
                    const int o = MODE == 0 ? kw : 2 - kw;
                    const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const float b[8] = {bq[0][o], bq[0][o + 1], bq[0][o + 2], bq[0][o + 3],
                                        bq[1][o], bq[1][o + 1], bq[1][o + 2], bq[1][o + 3]};
#pragma unroll
                    for (int i = 0; i < 8; i++)
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
                }
                ak += 3 * PA;
                const bool last_kh = ++kh == 3;
                if (last_kh) kh = 0;
                row0 += last_kh ? step_kh + step_p : step_kh;
                row1 += last_kh ? step_kh + step_p : step_kh;
            }
        }
        if (more) store_weights(c + 1, nxt + win_floats);
    }
    const bool redo = __syncthreads_or(unsafe ? 1 : 0) != 0;
    if (!owner) return;

    const int planes_out = MODE == 0 ? d.OC : d.IC;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? og * 4 + i : BM / 2 + og * 4 + i - 4);
        if (m >= w.M) continue;
        const int plane = MODE == 0 ? g * OCg + m : m;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int row = r0 + grow[h];
            if (!gok[h] || row >= w.outH) continue;
            float c[4] = {acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]};
            if (redo) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (gcol[h] + j < w.outW)
                        c[j] = MODE == 0 ? conv2d_exact(Src, Kw, d, n, plane, row, gcol[h] + j)
                                         : conv2d_grad_input_exact(Src, Kw, d, n, plane, row, gcol[h] + j);
                }
            }
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < 4; j++) c[j] = conv_finish(c[j], d, plane);
            }
            float *dst = Out + (((int64_t)n * planes_out + plane) * w.outH + row) * w.outW + gcol[h];
            if (gcol[h] + 3 < w.outW && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                *reinterpret_cast<float4 *>(dst) = make_float4(c[0], c[1], c[2], c[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (gcol[h] + j < w.outW) dst[j] = c[j];
            }
        }
    }
}

// Geometry and launch of conv_window_kernel; returns -1 when the shape is not one it takes.
template <int MODE>
int launch_conv_window(const float *src, const float *kw, float *out, const ConvDims &d, cudaStream_t st)
{
    if (d.sH != 1 || d.sW != 1 || d.KW != 3 || d.KH != 3) return -1;
    WinGeom w{};
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    w.M = MODE == 0 ? OCg : d.IC;
    w.planes = MODE == 0 ? ICg : d.OC;
    if (w.planes < CW_PC || w.M < 16) return -1;  // short chains / few channels: the gather kernel
    w.outH = MODE == 0 ? d.OH : d.H, w.outW = MODE == 0 ? d.OW : d.W;
    w.srcH = MODE == 0 ? d.H : d.OH, w.srcW = MODE == 0 ? d.W : d.OW;
    w.y_off = MODE == 0 ? -d.pH : d.pH - 2;
    w.x_off = MODE == 0 ? -d.pW : d.pW - 2;
    w.G4 = (w.outW + 3) / 4;
    w.WP = w.G4 * 4 + 4;  // a group reads 8 floats from its first pixel on
    const int OG = w.M >= 48 ? 8 : 4, BM = OG * 8;
    const int smem_limit = 100 * 1024;  // two CTAs per SM
    // rows per strip: at least 128 owning threads where the image allows it (the staging of a chunk
    // is shared by more outputs), then the fewest idle output slots
    int bestR = 0;
    double best = 0.0;
    for (int R = 1; R <= w.outH; R++) {
        const int pairs = (R * w.G4 + 1) / 2;
        if (OG * pairs > 256) break;
        const int64_t stage_floats = (int64_t)CW_PC * (R + 2) * w.WP + (int64_t)CW_KC * (BM + 4);
        if ((2 * stage_floats + (int64_t)(R + 2) * w.WP) * 4 > smem_limit) break;
        const int threads = OG * pairs <= 128 ? 128 : (OG * pairs <= 192 ? 192 : 256);
        const int strips = (w.outH + R - 1) / R;
        double eff = (double)w.outH * w.outW / ((double)strips * pairs * 8);
        if (OG * pairs < 128) eff *= (double)(OG * pairs) / 128.0;
        if (eff >= best - 1e-9) best = eff, bestR = R;  // ties: the taller strip
    }
    if (bestR == 0 || best < 0.55) return -1;
    w.R = bestR;
    w.strips = (w.outH + w.R - 1) / w.R;
    w.pairs = (w.R * w.G4 + 1) / 2;
    w.WR = w.R + 2;
    w.active = OG * w.pairs;
    const int threads = w.active <= 128 ? 128 : (w.active <= 192 ? 192 : 256);
    // 16-byte weight loads: rows of [OC][K] (or blocks of [IC][9]) that start on 16-byte boundaries
    const int K = w.planes * 9;
    w.vecw = aligned16(kw) && (MODE == 0 ? (K % 4 == 0) : ((int64_t)d.IC * 9 % 4 == 0 && w.M % 4 == 0 && BM % 4 == 0));
    if (MODE == 1 && (BM * 9) % 4 != 0) w.vecw = 0;
    const int64_t gx = (int64_t)w.strips * d.N;
    const int groups = MODE == 0 ? d.groups : 1;
    const int gy = (w.M + BM - 1) / BM;
    if (gx > 0x7FFFFFFF || gy > 65535 || groups > 65535) return -1;
    const int smem = (int)((2 * ((int64_t)CW_PC * w.WR * w.WP + (int64_t)CW_KC * (BM + 4)) + (int64_t)w.WR * w.WP) * 4);
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)groups);
#define REPDL_CW_LAUNCH(OGV, NTV)                                                                  \
    do {                                                                                           \
        static unsigned long long done = 0;                                                        \
        /* opt in once for the largest size any shape may ask for, not for this shape's */         \
        const int e = ensure_smem(conv_window_kernel<MODE, OGV, NTV>, smem_limit, &done);          \
        if (e) return e;                                                                           \
        conv_window_kernel<MODE, OGV, NTV><<<grid, NTV, smem, st>>>(src, kw, out, d, w);           \
    } while (0)
    if (OG == 8) {
        if (threads == 128) REPDL_CW_LAUNCH(8, 128);
        else if (threads == 192) REPDL_CW_LAUNCH(8, 192);
        else REPDL_CW_LAUNCH(8, 256);
    } else {
        if (threads == 128) REPDL_CW_LAUNCH(4, 128);
        else if (threads == 192) REPDL_CW_LAUNCH(4, 192);
        else REPDL_CW_LAUNCH(4, 256);
    }
#undef REPDL_CW_LAUNCH
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// conv2d with short chains (IC/groups * KH * KW <= 64 taps: a first layer over one or three input
// planes).  Such a convolution is bound by its output stream, not by FMAs, and the implicit GEMM's
// gather costs more than the arithmetic.  Here a thread owns one output pixel and CS_OC output
// channels: it walks the taps in the reference's order (ic, kh, kw), loads its input value of a tap
// once (coalesced over the pixels of a warp), reads the CS_OC weights of that tap from shared memory
// by broadcast, and skips a tap that falls into the padding exactly as the reference does (so no
// operand watch and no fallback are needed).  Stores are coalesced per channel.
// ------------------------------------------------------------------------------------------------
constexpr int CS_OC = 32, CS_THREADS = 256, CS_KMAX = 64;

// KB > 0: at most KB taps, all loaded before the first FMA (their latencies overlap); KB = 0: any number up
// to CS_KMAX, loaded one by one.
template <int KB>
__global__ void __launch_bounds__(CS_THREADS)
conv_short_kernel(const float *__restrict__ X, const float *__restrict__ Wt, float *__restrict__ Y, ConvDims d,
                  long long npix)
{
    __shared__ __align__(16) float Ws[CS_KMAX][CS_OC];
    __shared__ int toff[CS_KMAX], tkh[CS_KMAX], tkw[CS_KMAX];
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    const int K = ICg * d.KH * d.KW;
    const int grp = blockIdx.z, oc0 = blockIdx.y * CS_OC;  // oc0 within the group
    for (int i = threadIdx.x; i < K * CS_OC; i += CS_THREADS) {
        const int k = i / CS_OC, o = i - k * CS_OC;
        Ws[k][o] = oc0 + o < OCg ? __ldg(Wt + ((int64_t)(grp * OCg + oc0 + o)) * K + k) : 0.0f;
    }
    for (int k = threadIdx.x; k < K; k += CS_THREADS) {
        const int ic = k / (d.KH * d.KW), r = k - ic * d.KH * d.KW;
        tkh[k] = r / d.KW, tkw[k] = r - (r / d.KW) * d.KW;
        toff[k] = (ic * d.H + tkh[k]) * d.W + tkw[k];
    }
    __syncthreads();
    const long long pix = (long long)blockIdx.x * CS_THREADS + threadIdx.x;
    if (pix >= npix) return;
    const int OHW = d.OH * d.OW;
    const int n = (int)(pix / OHW), rem = (int)(pix - (long long)n * OHW);
    const int oh = rem / d.OW, ow = rem - oh * d.OW;
    const int h0 = oh * d.sH - d.pH, w0 = ow * d.sW - d.pW;
    const float *xn = X + ((int64_t)n * d.IC + (int64_t)grp * ICg) * d.H * d.W;
    const int base = h0 * d.W + w0;  // may be negative; only valid taps are dereferenced
    float acc[CS_OC];
#pragma unroll
    for (int o = 0; o < CS_OC; o++) acc[o] = 0.0f;
    auto tap = [&](float x, int k) {
        const float4 *w4 = reinterpret_cast<const float4 *>(Ws[k]);
#pragma unroll
        for (int q = 0; q < CS_OC / 4; q++) {
            const float4 w = w4[q];
            acc[4 * q + 0] = __fmaf_rn(x, w.x, acc[4 * q + 0]);
            acc[4 * q + 1] = __fmaf_rn(x, w.y, acc[4 * q + 1]);
            acc[4 * q + 2] = __fmaf_rn(x, w.z, acc[4 * q + 2]);
            acc[4 * q + 3] = __fmaf_rn(x, w.w, acc[4 * q + 3]);
        }
    };
    auto in_image = [&](int k) {
        return (unsigned)(h0 + tkh[k]) < (unsigned)d.H && (unsigned)(w0 + tkw[k]) < (unsigned)d.W;
    };
    // the reference skips taps in the padding: nothing is added for them
    if (KB > 0) {
        float x[KB > 0 ? KB : 1];
        unsigned valid = 0;
#pragma unroll
        for (int k = 0; k < KB; k++) {
            const bool v = k < K && in_image(k);
            x[k] = v ? __ldg(xn + base + toff[k]) : 0.0f;
            valid |= (v ? 1u : 0u) << k;
        }
#pragma unroll
        for (int k = 0; k < KB; k++)
            if ((valid >> k) & 1u) tap(x[k], k);
    } else {
        for (int k = 0; k < K; k++)
            if (in_image(k)) tap(__ldg(xn + base + toff[k]), k);
    }
    float *yp = Y + ((int64_t)n * d.OC + (int64_t)grp * OCg + oc0) * OHW + rem;
#pragma unroll
    for (int o = 0; o < CS_OC; o++)
        if (oc0 + o < OCg) yp[(int64_t)o * OHW] = conv_finish(acc[o], d, grp * OCg + oc0 + o);
}

template <int MODE>
int launch_conv_gemm(const float *src, const float *kw, float *out, const ConvDims &d, cudaStream_t st)
{
    const int ICg = d.IC / d.groups, OCg = d.OC / d.groups;
    const int M = MODE == 0 ? OCg : d.IC;
    const int outHW = MODE == 0 ? d.OH * d.OW : d.H * d.W;
    const int64_t ncols = (int64_t)d.N * outHW;
    const int64_t gx = (ncols + CG_BN - 1) / CG_BN;
    const int groups = MODE == 0 ? d.groups : 1;
    if (gx > 0x7FFFFFFF || groups > 65535) return REPDL_E_RANGE;
    {
        const int e = launch_conv_window<MODE>(src, kw, out, d, st);
        if (e >= 0) return e;
    }
    if (MODE == 0 && ICg * d.KH * d.KW <= CS_KMAX && (int64_t)d.IC * d.H * d.W < 0x7FFFFFFF &&
        (OCg + CS_OC - 1) / CS_OC <= 65535 && (ncols + CS_THREADS - 1) / CS_THREADS <= 0x7FFFFFFF) {
        dim3 grid((unsigned)((ncols + CS_THREADS - 1) / CS_THREADS), (unsigned)((OCg + CS_OC - 1) / CS_OC),
                  (unsigned)groups);
        const int K = ICg * d.KH * d.KW;
        if (K <= 16)
            conv_short_kernel<16><<<grid, CS_THREADS, 0, st>>>(src, kw, out, d, (long long)ncols);
        else if (K <= 32)
            conv_short_kernel<32><<<grid, CS_THREADS, 0, st>>>(src, kw, out, d, (long long)ncols);
        else
            conv_short_kernel<0><<<grid, CS_THREADS, 0, st>>>(src, kw, out, d, (long long)ncols);
        return launch_status();
    }
    const bool s1 = d.sH == 1 && d.sW == 1;
    if (M <= 32) {
        dim3 grid((unsigned)gx, (unsigned)((M + 31) / 32), (unsigned)groups);
        if (s1)
            conv_gemm_kernel<32, MODE, true><<<grid, 64, 0, st>>>(src, kw, out, d);
        else
            conv_gemm_kernel<32, MODE, false><<<grid, 64, 0, st>>>(src, kw, out, d);
    } else {
        dim3 grid((unsigned)gx, (unsigned)((M + 63) / 64), (unsigned)groups);
        if (grid.y > 65535) return REPDL_E_RANGE;
        if (s1)
            conv_gemm_kernel<64, MODE, true><<<grid, 128, 0, st>>>(src, kw, out, d);
        else
            conv_gemm_kernel<64, MODE, false><<<grid, 128, 0, st>>>(src, kw, out, d);
    }
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// conv2d_grad_kernel: few outputs (OC * IC * KH * KW), each a chain over batch * OH * OW steps that
// must not be split.  The floor is the latency of the dependent FMA chain (4 cycles per step), so
// the kernel is built to sit near that floor: a CTA owns 8 output channels x 32 (or 16) weight
// columns (ic, kh, kw); its first 4 warps (one per scheduler) only multiply -- a thread owns one
// channel x two (one) adjacent columns and issues two shared-memory loads and two (one) FMAs per
// step -- while 4 more warps do nothing but stage the next slab, so the chains never wait for address
// arithmetic or global loads.  k = (n, oh, ow) is walked in slabs of 128 through double-buffered shared
// memory (a slab's 40 loads per thread are all in flight while the previous slab is multiplied,
// which is what hides the L2 latency with only one warp per scheduler).  Every thread stages four k
// of the slab for all rows and columns, so (n, oh, ow) is decoded four times per slab and thread;
// the per-column input offsets are constants of the thread.  Padding
// taps enter as +0.0 under the same operand watch + exact fallback as the GEMM form above.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float conv2d_grad_kernel_exact(const float *__restrict__ GO,
                                                          const float *__restrict__ I, const ConvDims &d,
                                                          int oc, int ic, int kh, int kw)
{
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
    return acc;
}

constexpr int GK_BK = 128, GK_ROWS = 8, GK_THREADS = 256;  // 4 compute warps + 4 staging warps
constexpr int GK_KPT = GK_BK / 32;  // k values staged per thread per slab

// COLS = 32: a thread owns two adjacent columns (two chains); COLS = 16: one column, which puts twice
// as many CTAs on the machine when there are few outputs.
template <int COLS>
__global__ void __launch_bounds__(GK_THREADS)
conv_gk_kernel(const float *__restrict__ GO, const float *__restrict__ I, float *__restrict__ GK,
               ConvDims d)
{
    constexpr int CPT = COLS / 16;      // columns per thread in the compute role
    constexpr int SCOL = COLS / 4;      // columns staged per thread
    // k is the contiguous index of both slabs (pitch GK_BK + 4 floats), so a multiplying thread
    // fetches four consecutive k of its row / column with one LDS.128 -- a quarter of the loads, and
    // each load is four steps ahead of its last use; the staging threads (one k each) store to
    // consecutive addresses
    constexpr int PK = GK_BK + 4;
    __shared__ __align__(16) float As[2][GK_ROWS][PK];
    __shared__ __align__(16) float Bs[2][COLS][PK];
    const bool producer = threadIdx.x >= 128;
    const int t = threadIdx.x & 127;  // index within the role
    const int KHW = d.KH * d.KW, OHW = d.OH * d.OW, HW = d.H * d.W;
    const int ncols = d.IC * KHW;
    const int64_t K = (int64_t)d.N * OHW;
    const int oc0 = blockIdx.y * GK_ROWS, col0 = blockIdx.x * COLS;
    // compute role: one output channel, CPT adjacent columns
    const int crow = t / 16, ccol = (t % 16) * CPT;
    // staging role: k_local = t % 32 + 32 q (q < GK_KPT); rows t/32 + 4 i (i < 2); columns t/32 + 4 i
    const int sk = t % 32, sq = t / 32;
    int col_off[SCOL], col_kh[SCOL], col_kw[SCOL];
    bool col_ok[SCOL];
#pragma unroll
    for (int i = 0; i < SCOL; i++) {
        const int col = col0 + sq + 4 * i;
        col_ok[i] = col < ncols;
        const int c = col_ok[i] ? col : 0;
        const int ic = c / KHW, r = c - ic * KHW;
        col_kh[i] = r / d.KW, col_kw[i] = r - col_kh[i] * d.KW;
        col_off[i] = ic * HW + (col_kh[i] - d.pH) * d.W + (col_kw[i] - d.pW);
    }
    const bool padded = (d.pH | d.pW) != 0;
    // (n, p) of this thread's k values, advanced by GK_BK per slab without divisions
    int kn[GK_KPT], kp[GK_KPT];
#pragma unroll
    for (int q = 0; q < GK_KPT; q++) {
        const int64_t k = sk + 32 * q;
        kn[q] = (int)(k / OHW);
        kp[q] = (int)(k - (int64_t)kn[q] * OHW);
    }
    // two register sets: while one slab is being written to shared memory the loads of the next
    // one are already in flight (the producers run two slabs ahead of the multiplying warps)
    float avA[GK_KPT][2], bvA[GK_KPT][SCOL], avB[GK_KPT][2], bvB[GK_KPT][SCOL];
    bool unsafe = false;
    auto load_slab = [&](float (&av)[GK_KPT][2], float (&bv)[GK_KPT][SCOL]) {
        // loads the slab (kn, kp) point at, then advances them by GK_BK
#pragma unroll
        for (int q = 0; q < GK_KPT; q++) {
            const int n = kn[q], p = kp[q];
            const bool kin = n < d.N;
            const int oh = fastdiv(p, d.m40_ow), ow = p - oh * d.OW;
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int oc = oc0 + sq + 4 * i;
                // K tail: A = -0, B = +0 gives the product -0, the identity of the accumulation
                av[q][i] = !kin ? -0.0f
                                : (oc < d.OC ? __ldg(GO + ((int64_t)n * d.OC + oc) * OHW + p) : 0.0f);
                unsafe |= cg_unsafe(av[q][i]);
            }
            const float *ip = I + (int64_t)(kin ? n : 0) * d.IC * HW + (oh * d.sH) * d.W + ow * d.sW;
#pragma unroll
            for (int i = 0; i < SCOL; i++) {
                bool ok = kin && col_ok[i];
                if (padded) {
                    const int h = oh * d.sH - d.pH + col_kh[i], w = ow * d.sW - d.pW + col_kw[i];
                    ok = ok && h >= 0 && h < d.H && w >= 0 && w < d.W;
                }
                bv[q][i] = ok ? __ldg(ip + col_off[i]) : 0.0f;
                unsafe |= cg_unsafe(bv[q][i]);
            }
            kp[q] += GK_BK;
            while (kp[q] >= OHW) kp[q] -= OHW, kn[q]++;
        }
    };
    auto store_slab = [&](int buf, const float (&av)[GK_KPT][2], const float (&bv)[GK_KPT][SCOL]) {
#pragma unroll
        for (int q = 0; q < GK_KPT; q++) {
#pragma unroll
            for (int i = 0; i < 2; i++) As[buf][sq + 4 * i][sk + 32 * q] = av[q][i];
#pragma unroll
            for (int i = 0; i < SCOL; i++) Bs[buf][sq + 4 * i][sk + 32 * q] = bv[q][i];
        }
    };
    auto multiply_slab = [&](int cur, float (&acc)[CPT]) {
#pragma unroll
        for (int k = 0; k < GK_BK; k += 4) {
            const float4 a = *reinterpret_cast<const float4 *>(&As[cur][crow][k]);
#pragma unroll
            for (int j = 0; j < CPT; j++) {
                const float4 b = *reinterpret_cast<const float4 *>(&Bs[cur][ccol + j][k]);
                acc[j] = __fmaf_rn(a.x, b.x, acc[j]);
                acc[j] = __fmaf_rn(a.y, b.y, acc[j]);
                acc[j] = __fmaf_rn(a.z, b.z, acc[j]);
                acc[j] = __fmaf_rn(a.w, b.w, acc[j]);
            }
        }
    };
    float acc[CPT];
#pragma unroll
    for (int j = 0; j < CPT; j++) acc[j] = 0.0f;
    const int64_t nslab = (K + GK_BK - 1) / GK_BK;
    if (producer) {
        load_slab(avA, bvA);            // slab 0
        store_slab(0, avA, bvA);
        if (nslab > 1) load_slab(avA, bvA);  // slab 1 stays in flight in set A
    }
    __syncthreads();
    // iterations come in pairs so that the register sets have fixed names: entering an even
    // iteration kt, slab kt + 1 is in set A; entering an odd one it is in set B
    for (int64_t kt = 0; kt < nslab; kt += 2) {
        if (producer) {
            if (kt + 2 < nslab) load_slab(avB, bvB);
            if (kt + 1 < nslab) store_slab(1, avA, bvA);
        } else {
            multiply_slab(0, acc);
        }
        __syncthreads();
        if (kt + 1 >= nslab) break;
        if (producer) {
            if (kt + 3 < nslab) load_slab(avA, bvA);
            if (kt + 2 < nslab) store_slab(0, avB, bvB);
        } else {
            multiply_slab(1, acc);
        }
        __syncthreads();
    }
    const bool redo = __syncthreads_or(unsafe ? 1 : 0) != 0;
    const int oc = oc0 + crow;
    if (!producer && oc < d.OC) {
#pragma unroll
        for (int j = 0; j < CPT; j++) {
            const int col = col0 + ccol + j;
            if (col >= ncols) continue;
            float v = acc[j];
            if (redo) {
                const int ic = col / KHW, r = col - ic * KHW;
                v = conv2d_grad_kernel_exact(GO, I, d, oc, ic, r / d.KW, r % d.KW);
            }
            GK[(int64_t)oc * ncols + col] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// conv2d_grad_kernel, row-chunk form (the one used whenever an image's output rows give chunks of a
// useful length).  Same split of roles as above -- warps that only multiply, one chain per thread, and
// 8 warps that only stage -- but the staging warps never touch a value: k is walked image by image in
// chunks of R whole output rows -- the whole image when that fits, up to 768 steps -- or of segments
// of one row when rows are longer than that, every operand element goes global -> shared with one
// 4-byte cp.async (16-byte for grad_output when its rows allow it), three chunks are in flight, and
// the (row, column) decoding of a thread's elements is the same for every chunk, so it is done once.
// What is left per element is the address and the copy.  Padding taps are zero-filled by the copy itself (src-size 0), so only a padded
// convolution needs the operand watch: there the staging threads read back what they copied when it
// has landed, and the CTA falls back to the exact loop for its outputs if a non-finite or vanishing
// value was seen.  A CTA's tile is 8 output channels x 16 weight columns (4 multiplying warps), or
// 4 x 8 (one warp) when there are so few outputs that the larger tile would leave most SMs idle.
// ------------------------------------------------------------------------------------------------
constexpr int GKR_RING = 6;     // groups of 4 steps a multiplying warp loads ahead of its FMAs
constexpr int GKR_STAGES = 3;
constexpr int GKR_KPT = 3;      // steps of a chunk that one staging thread copies, at most
// steps of a chunk after padding to whole rings
__host__ __device__ constexpr int gkr_padded(int len) { return (len + 4 * GKR_RING - 1) / (4 * GKR_RING) * (4 * GKR_RING); }
// row pitch in floats for chunks of at most kmax steps: room for the padded chunk, a multiple of 4
// (16-byte loads), and 4 or 12 modulo 32 so that the 16-byte segments of 4 rows or 8 columns at one
// k fall into different banks
static int gkr_pitch(int kmax)
{
    int p = gkr_padded(kmax);
    while (p % 32 != 4 && p % 32 != 12) p += 4;
    return p;
}
constexpr int GKR_STAGERS = 256;  // staging threads (8 warps)
constexpr int GKR_KMAX = GKR_KPT * GKR_STAGERS;  // longest chunk

__device__ __forceinline__ void cp_async_4(float *smem_dst, const float *gmem_src)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_4z(float *smem_dst, const float *gmem_src, bool ok)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = ok ? 4 : 0;  // 0: nothing is read, the word is zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes)
                 : "memory");
}

// position of a chunk: image n, first output row oh0, first output column ow0
struct GkChunk {
    int n, oh0, ow0;
};

// RW x CB multiplying warps, each owning a patch of 4 output channels x 8 weight columns.
// BIAS: the kernel also adds up the rows of grad_output in the order n, oh, ow of the reference's
// sum4d_dim023 and writes the bias gradient, which saves a separate pass over grad_output.  A bias
// chain is as long as a weight chain.  Where the grid leaves SMs free (bias_sep), one more column
// block of CTAs carries the bias chains alone: those CTAs stage and read the row operand only.
// Otherwise the threads of the first column block carry a second chain, which costs them 0.5 to 0.9
// cycles per step (but a CTA that has to share its SM costs the kernel far more).
template <bool PADDED, int RW, int CB, bool BIAS>
__global__ void __launch_bounds__((RW * CB) * 32 + GKR_STAGERS, 2)
conv_gk_rows_kernel(const float *__restrict__ GO, const float *__restrict__ I, float *__restrict__ GK,
                    float *__restrict__ GB, ConvDims d, int segW, int R, int pitch, int a16, int bias_sep,
                    long long nchunks)
{
    extern __shared__ __align__(16) float gkr_smem[];
    constexpr int ROWS = 4 * RW, COLS = 8 * CB, NCW = RW * CB;
    constexpr int NT = NCW * 32 + GKR_STAGERS;
    const int STAGE = (ROWS + COLS) * pitch;
    const bool producer = threadIdx.x >= NCW * 32;
    const int t = producer ? threadIdx.x - NCW * 32 : threadIdx.x;  // index within the role
    const int KHW = d.KH * d.KW, OHW = d.OH * d.OW, HW = d.H * d.W;
    const int ncols = d.IC * KHW;
    const int oc0 = blockIdx.y * ROWS, col0 = blockIdx.x * COLS;

    auto chunk_len = [&](const GkChunk &c) {
        const int rows = min(R, d.OH - c.oh0);
        return segW == d.OW ? rows * d.OW : min(segW, d.OW - c.ow0);
    };
    auto advance = [&](GkChunk &c) {
        c.ow0 += segW;
        if (c.ow0 >= d.OW) {
            c.ow0 = 0;
            c.oh0 += R;
            if (c.oh0 >= d.OH) c.oh0 = 0, c.n++;
        }
    };
    // The two roles run separate loops (so that neither holds the other's registers) and meet at a
    // named barrier once per chunk: after it chunk ci is visible to all and chunk ci - 1 is done with.
    auto chunk_barrier = []() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); };
    GkChunk cur = {0, 0, 0};
    int stage = 0;  // stage of chunk ci; the chunk issued in iteration ci goes to the stage before it
    bool unsafe = false;
    float acc = 0.0f, accb = 0.0f;
    const bool bias_only = BIAS && bias_sep && blockIdx.x == gridDim.x - 1;  // this CTA only adds up rows
    const bool bias_too = BIAS && !bias_sep && blockIdx.x == 0;              // second chain per thread
    // Multiplying role: which output of the CTA's tile a thread owns.  Shared memory serves a 16-byte
    // load eight lanes at a time, and passes of one load that fetch the same addresses in the same
    // lanes are merged.  So the lanes of a warp's 4 x 8 patch are laid out with all four rows in
    // every group of eight lanes (the row operand then costs one pass instead of four) and two of
    // the eight columns per group.
    const int cw = t / 32, lane = t % 32;
    const int prow = (lane % 8) / 2, pcol = 2 * (lane / 8) + lane % 2;
    const int crow = 4 * (cw / CB) + prow, ccol = 8 * (cw % CB) + pcol;

    if (producer) {
        // Thread t copies steps t, t + 256, ... of every row and column of a chunk (GKR_KPT of them at
        // most).  Rows and columns past the end are clamped to the last valid one: they are copied
        // twice and feed outputs nobody stores, which is cheaper than predicating every copy.
        int boff[GKR_KPT], hb[GKR_KPT], wb[GKR_KPT];
#pragma unroll
        for (int m = 0; m < GKR_KPT; m++) {
            const int k = t + m * GKR_STAGERS;
            const int sr = k / segW, sc = k - sr * segW;
            boff[m] = sr * d.sH * d.W + sc * d.sW;
            hb[m] = sr * d.sH - d.pH, wb[m] = sc * d.sW - d.pW;
        }
        int col_off[COLS], col_hw[COLS];
#pragma unroll
        for (int c = 0; c < COLS; c++) {
            const int col = min(col0 + c, ncols - 1);
            const int ic = col / KHW, r = col - ic * KHW;
            const int kh = r / d.KW, kw = r - kh * d.KW;
            col_off[c] = ic * HW + (kh - d.pH) * d.W + (kw - d.pW);
            col_hw[c] = (kh << 16) | kw;
        }
        // 16-byte copies of grad_output: LPR threads per row, along k
        constexpr int LPR = GKR_STAGERS / ROWS;
        const int a16r = t / LPR, a16l = t % LPR;
        const int a16src = min(oc0 + a16r, d.OC - 1) - oc0;

        auto issue = [&](int st, const GkChunk &c) {
            float *As = gkr_smem + st * STAGE, *Bs = As + ROWS * pitch;
            const int len = chunk_len(c);
            const float *ga = GO + ((int64_t)c.n * d.OC + oc0) * OHW + c.oh0 * d.OW + c.ow0;
            if (a16) {
                const float *src = ga + (int64_t)a16src * OHW;
                for (int q = 4 * a16l; q < len; q += 4 * LPR) cp_async_16(&As[a16r * pitch + q], src + q);
            }
            const float *gi = I + ((int64_t)c.n * d.IC * HW + (c.oh0 * d.sH) * d.W + c.ow0 * d.sW);
#pragma unroll 1
            for (int m = 0; m < GKR_KPT; m++) {
                const int k = t + m * GKR_STAGERS;
                if (k >= len) break;
                if (!a16) {
#pragma unroll
                    for (int row = 0; row < ROWS; row++) {
                        const int rr = min(oc0 + row, d.OC - 1) - oc0;
                        cp_async_4(&As[row * pitch + k], ga + (int64_t)rr * OHW + k);
                    }
                }
                if (bias_only) continue;
                const float *gim = gi + boff[m];
                const int hj = c.oh0 * d.sH + hb[m], wj = c.ow0 * d.sW + wb[m];
#pragma unroll
                for (int cc = 0; cc < COLS; cc++) {
                    if (PADDED) {
                        const bool ok = (unsigned)(hj + (col_hw[cc] >> 16)) < (unsigned)d.H &&
                                        (unsigned)(wj + (col_hw[cc] & 0xFFFF)) < (unsigned)d.W;
                        cp_async_4z(&Bs[cc * pitch + k], ok ? gim + col_off[cc] : I, ok);
                    } else {
                        cp_async_4(&Bs[cc * pitch + k], gim + col_off[cc]);
                    }
                }
            }
            // pad the chunk to whole rings of the multiplying warps with the identity of the chains
            for (int q = len + t; q < gkr_padded(len); q += GKR_STAGERS) {
#pragma unroll
                for (int row = 0; row < ROWS; row++) As[row * pitch + q] = -0.0f;
                if (bias_only) continue;
#pragma unroll
                for (int cc = 0; cc < COLS; cc++) Bs[cc * pitch + q] = 0.0f;
            }
        };
        // operand watch of a landed chunk: every staging thread looks at the elements it copied itself
        auto watch = [&](int st, const GkChunk &c) {
            const float *As = gkr_smem + st * STAGE, *Bs = As + ROWS * pitch;
            const int len = chunk_len(c);
            if (a16) {
                for (int q = 4 * a16l; q < len; q += 4 * LPR) {
                    const float4 v = *reinterpret_cast<const float4 *>(&As[a16r * pitch + q]);
                    unsafe |= cg_unsafe(v.x) | cg_unsafe(v.y) | cg_unsafe(v.z) | cg_unsafe(v.w);
                }
            }
#pragma unroll 1
            for (int m = 0; m < GKR_KPT; m++) {
                const int k = t + m * GKR_STAGERS;
                if (k >= len) break;
                if (!a16) {
#pragma unroll
                    for (int row = 0; row < ROWS; row++) unsafe |= cg_unsafe(As[row * pitch + k]);
                }
                if (bias_only) continue;
#pragma unroll
                for (int cc = 0; cc < COLS; cc++) unsafe |= cg_unsafe(Bs[cc * pitch + k]);
            }
        };

        GkChunk iss = {0, 0, 0};
#pragma unroll
        for (int s = 0; s < GKR_STAGES - 1; s++) {
            if (s < nchunks) issue(s, iss);
            cp_async_commit();
            advance(iss);
        }
        for (long long ci = 0; ci < nchunks; ci++) {
            cp_async_wait<GKR_STAGES - 2>();
            if (PADDED) watch(stage, cur);
            chunk_barrier();
            if (ci + GKR_STAGES - 1 < nchunks) issue(stage == 0 ? GKR_STAGES - 1 : stage - 1, iss);
            cp_async_commit();
            advance(iss);
            advance(cur);
            stage = stage + 1 == GKR_STAGES ? 0 : stage + 1;
        }
        cp_async_wait<0>();
    } else {
        // A group is 4 steps: one 16-byte load of the row operand, one of the column operand, four
        // dependent FMAs.  The loads of a group are issued GKR_RING groups (about 100 cycles of FMAs)
        // before its FMAs, into a ring of register sets whose loop is unrolled so that every set has
        // fixed registers.  Measured on B200: a 16-byte shared-memory load that the warp has to wait
        // for costs it far more than the 16 cycles of a group, loads it does not wait for cost
        // nothing (4.4 cycles per step for the whole loop), a second dependent chain in the same
        // thread costs 0.5 to 0.9 cycles per step.  The loop has no branch but its own: chunks are
        // padded to whole rings by the staging warps (row operand -0, column operand +0:
        // acc + (-0 * +0) = acc and accb + -0 = accb for every value, -0 included).
        // The pipeline does not drain between chunks: when the loads of a chunk have all been issued
        // the warp passes the barrier of the next chunk (loads issued before a barrier have read their
        // data when it completes, so the staging warps may refill the stage) and loads the first ring
        // of that chunk while it multiplies the last ring of this one.
        auto walk = [&](auto mode) {
            constexpr int MODE = decltype(mode)::value;  // 0: multiply, 1: multiply and add up rows, 2: add up rows
            constexpr bool BO = MODE == 2;
            auto step4 = [&](const float4 &a, const float4 &b) {
                if (MODE != 2) {
                    acc = __fmaf_rn(a.x, b.x, acc);
                    acc = __fmaf_rn(a.y, b.y, acc);
                    acc = __fmaf_rn(a.z, b.z, acc);
                    acc = __fmaf_rn(a.w, b.w, acc);
                }
                if (MODE != 0) {
                    accb = __fadd_rn(accb, a.x);
                    accb = __fadd_rn(accb, a.y);
                    accb = __fadd_rn(accb, a.z);
                    accb = __fadd_rn(accb, a.w);
                }
            };
            float4 ra[GKR_RING], rb[GKR_RING];
            const float4 *ar = nullptr, *br = nullptr;
            auto enter_chunk = [&]() {  // barrier of the next chunk; this thread's operand rows in its stage
                chunk_barrier();
                ar = reinterpret_cast<const float4 *>(gkr_smem + stage * STAGE + crow * pitch);
                br = reinterpret_cast<const float4 *>(gkr_smem + stage * STAGE + (ROWS + ccol) * pitch);
            };
            auto load = [&](int i, int g) {
                ra[i] = ar[g];
                if (!BO) rb[i] = br[g];
            };
            if (nchunks > 0) {
                enter_chunk();
#pragma unroll
                for (int i = 0; i < GKR_RING; i++) load(i, i);
            }
            for (long long ci = 0; ci < nchunks; ci++) {
                const int ngroups = gkr_padded(chunk_len(cur)) >> 2;  // a multiple of GKR_RING
                for (int g = GKR_RING; g < ngroups; g += GKR_RING) {
#pragma unroll
                    for (int i = 0; i < GKR_RING; i++) {
                        step4(ra[i], rb[i]);
                        load(i, g + i);
                    }
                }
                advance(cur);
                stage = stage + 1 == GKR_STAGES ? 0 : stage + 1;
                if (ci + 1 < nchunks) {
                    enter_chunk();
#pragma unroll
                    for (int i = 0; i < GKR_RING; i++) {
                        step4(ra[i], rb[i]);
                        load(i, i);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < GKR_RING; i++) step4(ra[i], rb[i]);
                }
            }
        };
        // (a copy of the loop per mode: a test inside it would cost the chain a branch per group)
        if (bias_only)
            walk(std::integral_constant<int, 2>{});
        else if (bias_too)
            walk(std::integral_constant<int, 1>{});
        else
            walk(std::integral_constant<int, 0>{});
    }
    const bool redo = PADDED ? (__syncthreads_or(unsafe ? 1 : 0) != 0) : false;
    if (!producer) {
        const int oc = oc0 + crow, col = col0 + ccol;
        if ((bias_only || bias_too) && ccol == 0 && oc < d.OC) GB[oc] = accb;
        if (!bias_only && oc < d.OC && col < ncols) {
            float v = acc;
            if (redo) {
                const int ic = col / KHW, r = col - ic * KHW;
                v = conv2d_grad_kernel_exact(GO, I, d, oc, ic, r / d.KW, r % d.KW);
            }
            GK[(int64_t)oc * ncols + col] = v;
        }
    }
}

// Chunk geometry for a tile of `lines` operand rows + columns.  Chunks are as long as three stages
// of them fit in half of an SM's shared memory (so that two CTAs, of this convolution or of the next
// layer's, share an SM) and GKR_KMAX allows: every chunk costs the multiplying warps a hand-over, and
// its padding.  An image is split into equal runs of whole output rows (segW = OW), or, when a row is
// longer than a chunk, rows into segments.
struct GkGeom {
    int segW, R, pitch, smem;
};
constexpr int GKR_SMEM_BUDGET = 112 * 1024;
static GkGeom gk_geometry(const ConvDims &d, int lines)
{
    int kmax = GKR_KMAX;
    while (GKR_STAGES * lines * gkr_pitch(kmax) * (int)sizeof(float) > GKR_SMEM_BUDGET) kmax -= 8;
    GkGeom g;
    if (d.OW <= kmax) {
        const int rows_max = kmax / d.OW < d.OH ? kmax / d.OW : d.OH;
        const int parts = (d.OH + rows_max - 1) / rows_max;
        g.segW = d.OW, g.R = (d.OH + parts - 1) / parts;
        g.pitch = gkr_pitch(g.R * d.OW);
    } else {
        g.segW = kmax, g.R = 1;
        g.pitch = gkr_pitch(kmax);
    }
    g.smem = GKR_STAGES * lines * g.pitch * (int)sizeof(float);
    return g;
}

template <bool PADDED, int RW, int CB, bool BIAS>
int launch_gk_rows(const float *go, const float *in, float *gk, float *gb, const ConvDims &d, cudaStream_t st)
{
    static unsigned long long done = 0;
    constexpr int ROWS = 4 * RW, COLS = 8 * CB;
    const GkGeom g = gk_geometry(d, ROWS + COLS);
    int e = ensure_smem(conv_gk_rows_kernel<PADDED, RW, CB, BIAS>, GKR_SMEM_BUDGET, &done);
    if (e) return e;
    const int ncols = d.IC * d.KH * d.KW;
    const long long nchunks = (long long)d.N * ((d.OH + g.R - 1) / g.R) * ((d.OW + g.segW - 1) / g.segW);
    // 16-byte copies of grad_output need every chunk to start on a 16-byte boundary and to hold a
    // multiple of 4 elements
    const bool a16 = ((uintptr_t)go % 16 == 0) && ((int64_t)d.OH * d.OW % 4 == 0) &&
                     (g.segW == d.OW ? ((int64_t)g.R * d.OW % 4 == 0) : (d.OW % 4 == 0));
    dim3 grid((unsigned)((ncols + COLS - 1) / COLS), (unsigned)((d.OC + ROWS - 1) / ROWS));
    // the bias chains in CTAs of their own if every CTA then still has an SM to itself
    const bool bias_sep = BIAS && (int64_t)(grid.x + 1) * grid.y <= sm_count();
    if (bias_sep) grid.x++;
    conv_gk_rows_kernel<PADDED, RW, CB, BIAS><<<grid, RW * CB * 32 + GKR_STAGERS, g.smem, st>>>(
        go, in, gk, gb, d, g.segW, g.R, g.pitch, a16 ? 1 : 0, bias_sep ? 1 : 0, nchunks);
    return launch_status();
}

// few outputs: patches of 4 x 8 (one multiplying warp per CTA) put them on four times as many SMs
template <bool BIAS>
int launch_gk_rows_any(const float *go, const float *in, float *gk, float *gb, const ConvDims &d,
                       cudaStream_t st)
{
    const int ncols = d.IC * d.KH * d.KW;
    const bool padded = (d.pH | d.pW) != 0;
    const int64_t big_tiles = (int64_t)((ncols + 15) / 16) * ((d.OC + 7) / 8);
    if (2 * big_tiles < sm_count())
        return padded ? launch_gk_rows<true, 1, 1, BIAS>(go, in, gk, gb, d, st)
                      : launch_gk_rows<false, 1, 1, BIAS>(go, in, gk, gb, d, st);
    return padded ? launch_gk_rows<true, 2, 2, BIAS>(go, in, gk, gb, d, st)
                  : launch_gk_rows<false, 2, 2, BIAS>(go, in, gk, gb, d, st);
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
    d.bias = nullptr, d.relu = 0;
    d.OH = (int)((H + 2 * pH - KH) / sH + 1);
    d.OW = (int)((W + 2 * pW - KW) / sW + 1);
    const unsigned long long khw = (unsigned long long)(KH * KW), kwv = (unsigned long long)KW;
    d.m40_khw = ((1ull << 40) + khw - 1) / khw;
    d.m40_kw = ((1ull << 40) + kwv - 1) / kwv;
    d.m40_ow = ((1ull << 40) + (unsigned long long)d.OW - 1) / (unsigned long long)d.OW;
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
    return repdl_b200_conv2d_bias_act(input, kernel, nullptr, output, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW,
                                      groups, 0, stream);
}

extern "C" int repdl_b200_conv2d_bias_act(const float *input, const float *kernel, const float *bias,
                                          float *output, int64_t N, int64_t IC, int64_t H, int64_t W, int64_t OC,
                                          int64_t KH, int64_t KW, int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                                          int64_t groups, int relu, void *stream)
{
    clear_stale_error();
    ConvDims d;
    int e = fill_dims(d, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW, groups);
    if (e) return e;
    d.bias = bias, d.relu = relu ? 1 : 0;
    int64_t total = (int64_t)d.N * d.OC * d.OH * d.OW;
    if (total == 0) return REPDL_OK;
    if (!input || !kernel || !output) return REPDL_E_NULL;
    if ((int64_t)d.KH * d.KW <= 64 && (int64_t)d.IC * d.KH * d.KW < (1 << 24) &&
        (int64_t)d.N * d.OH * d.OW >= 64)
        return launch_conv_gemm<0>(input, kernel, output, d, (cudaStream_t)stream);
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
    if ((int64_t)d.KH * d.KW <= 64 && (int64_t)d.OC * d.KH * d.KW < (1 << 24) &&
        (int64_t)d.N * d.H * d.W >= 64)
        return launch_conv_gemm<1>(grad_output, kernel, grad_input, d, (cudaStream_t)stream);
    unsigned blocks;
    if ((e = blocks_for(total, blocks))) return e;
    conv2d_grad_input_direct_kernel<<<blocks, CONV_THREADS, 0, (cudaStream_t)stream>>>(
        grad_output, kernel, grad_input, d, total);
    return launch_status();
}

// grad_bias != nullptr: the fused form, which only the row-chunk kernel offers (REPDL_E_UNSUPPORTED
// for shapes that take another kernel: the caller then uses the two separate entry points).
static int conv2d_grad_kernel_impl(const float *grad_output, const float *input, float *grad_kernel,
                                   float *grad_bias, int64_t N, int64_t IC, int64_t H, int64_t W,
                                   int64_t OC, int64_t KH, int64_t KW, int64_t sH, int64_t sW, int64_t pH,
                                   int64_t pW, void *stream, bool rows_only = false)
{
    clear_stale_error();
    ConvDims d;
    int e = fill_dims(d, N, IC, H, W, OC, KH, KW, sH, sW, pH, pW, 1);
    if (e) return e;
    int64_t total = (int64_t)d.OC * d.IC * d.KH * d.KW;
    if (!grad_output || !input || !grad_kernel) return REPDL_E_NULL;
    if ((int64_t)d.N * d.OH * d.OW >= 256 && (int64_t)d.IC * d.KH * d.KW < 0x7FFFFFFF &&
        (int64_t)d.IC * d.H * d.W < 0x7FFFFFFF) {
        const int ncols = d.IC * d.KH * d.KW;
        const unsigned gy = (unsigned)((d.OC + GK_ROWS - 1) / GK_ROWS);
        // few outputs: one chain per thread spreads them over twice as many SMs
        const bool narrow = (int64_t)((ncols + 31) / 32) * gy < 2 * (int64_t)sm_count();
        // the row-chunk kernel, unless its chunks would be too short to pay for their hand-over
        const GkGeom g = gk_geometry(d, 12);
        if ((d.OC + 3) / 4 <= 65535 && (int64_t)g.R * g.segW >= 64 && d.KH < 32768 && d.KW < 32768 &&
            (int64_t)d.OH * d.OW < (1 << 30) && ((int64_t)d.H + 2 * d.pH) * d.W < (1 << 30)) {
            return grad_bias ? launch_gk_rows_any<true>(grad_output, input, grad_kernel, grad_bias, d,
                                                        (cudaStream_t)stream)
                             : launch_gk_rows_any<false>(grad_output, input, grad_kernel, nullptr, d,
                                                         (cudaStream_t)stream);
        }
        if (grad_bias || rows_only) return REPDL_E_UNSUPPORTED;
        if (gy <= 65535 && d.OW < 65536 && (int64_t)d.OH * d.OW < (1 << 24)) {
            if (narrow)
                conv_gk_kernel<16><<<dim3((unsigned)((ncols + 15) / 16), gy), GK_THREADS, 0,
                                     (cudaStream_t)stream>>>(grad_output, input, grad_kernel, d);
            else
                conv_gk_kernel<32><<<dim3((unsigned)((ncols + 31) / 32), gy), GK_THREADS, 0,
                                     (cudaStream_t)stream>>>(grad_output, input, grad_kernel, d);
            return launch_status();
        }
    }
    if (grad_bias || rows_only) return REPDL_E_UNSUPPORTED;
    unsigned blocks;
    if ((e = blocks_for(total, blocks))) return e;
    conv2d_grad_kernel_direct_kernel<<<blocks, CONV_THREADS, 0, (cudaStream_t)stream>>>(
        grad_output, input, grad_kernel, d, total);
    return launch_status();
}

namespace repdl_b200 {
int mm_long_k(const float *A, const float *B, float *C, int M, int N, int K, cudaStream_t st)
{
    // grad_output = A as [1, M, 1, K], input = B as [1, N, 1, K], kernel 1 x 1: grad_kernel[m][n]
    return conv2d_grad_kernel_impl(A, B, C, nullptr, 1, N, 1, K, M, 1, 1, 1, 1, 0, 0, (void *)st, true);
}
}  // namespace repdl_b200

extern "C" int repdl_b200_conv2d_grad_kernel(const float *grad_output, const float *input,
                                             float *grad_kernel, int64_t N, int64_t IC, int64_t H,
                                             int64_t W, int64_t OC, int64_t KH, int64_t KW,
                                             int64_t sH, int64_t sW, int64_t pH, int64_t pW,
                                             void *stream)
{
    return conv2d_grad_kernel_impl(grad_output, input, grad_kernel, nullptr, N, IC, H, W, OC, KH, KW, sH,
                                   sW, pH, pW, stream);
}

extern "C" int repdl_b200_conv2d_grad_kernel_bias(const float *grad_output, const float *input,
                                                  float *grad_kernel, float *grad_bias, int64_t N,
                                                  int64_t IC, int64_t H, int64_t W, int64_t OC,
                                                  int64_t KH, int64_t KW, int64_t sH, int64_t sW,
                                                  int64_t pH, int64_t pW, void *stream)
{
    if (!grad_bias) return REPDL_E_NULL;
    return conv2d_grad_kernel_impl(grad_output, input, grad_kernel, grad_bias, N, IC, H, W, OC, KH, KW,
                                   sH, sW, pH, pW, stream);
}
