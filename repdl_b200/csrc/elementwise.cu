// Elementwise fp32 math for sm_100a: div, sqrt, exp, log with the bits of the reference's CPU run.
//
// All four are HBM-bound streams (4 B in, 4 B out per element): 128-bit loads and stores, four
// independent 16-byte groups in flight per thread, a grid of a few CTAs per SM walking the array
// with a grid stride.  The arithmetic per element is in crmath.cuh.
#include "common.cuh"
#include "crmath.cuh"

namespace repdl_b200 {
namespace {

struct OpSqrt {
    __device__ __forceinline__ float operator()(float x) const { return cr_sqrt(x); }
};
struct OpExp {
    __device__ __forceinline__ float operator()(float x) const { return cr_exp(x); }
};
struct OpLog {
    __device__ __forceinline__ float operator()(float x) const { return cr_log(x); }
};
struct OpDivScalar {
    float d;
    __device__ __forceinline__ float operator()(float x) const { return cr_div(x, d); }
};

constexpr int EW_THREADS = 256;
constexpr int EW_VEC_PER_THREAD = 4;  // float4 groups in flight per thread per iteration

template <class Op>
__global__ void __launch_bounds__(EW_THREADS)
unary_vec_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t nvec, Op op)
{
    // nvec = number of float4 groups; x and y are 16-byte aligned
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS * EW_VEC_PER_THREAD;
    for (int64_t base = (int64_t)blockIdx.x * EW_THREADS * EW_VEC_PER_THREAD + threadIdx.x;
         base < nvec; base += stride) {
        float4 v[EW_VEC_PER_THREAD];
#pragma unroll
        for (int u = 0; u < EW_VEC_PER_THREAD; u++) {
            int64_t i = base + (int64_t)u * EW_THREADS;
            if (i < nvec) v[u] = ldg_stream_f4(x + 4 * i);
        }
#pragma unroll
        for (int u = 0; u < EW_VEC_PER_THREAD; u++) {
            int64_t i = base + (int64_t)u * EW_THREADS;
            if (i < nvec) {
                float4 r;
                r.x = op(v[u].x);
                r.y = op(v[u].y);
                r.z = op(v[u].z);
                r.w = op(v[u].w);
                stg_stream_f4(y + 4 * i, r);
            }
        }
    }
}

template <class Op>
__global__ void __launch_bounds__(EW_THREADS)
unary_scalar_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t n, Op op)
{
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    for (int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += stride)
        y[i] = op(__ldg(x + i));
}

__global__ void __launch_bounds__(EW_THREADS)
div_tensor_kernel(const float *__restrict__ x, const float *__restrict__ d, float *__restrict__ y,
                  int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    for (int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += stride)
        y[i] = cr_div(__ldg(x + i), __ldg(d + i));
}

static unsigned grid_for(int64_t work_items, int per_block)
{
    int64_t blocks = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

template <class Op>
int launch_unary(const float *x, float *y, int64_t n, Op op, void *stream)
{
    if (n < 0) return REPDL_E_SHAPE;
    if (n == 0) return REPDL_OK;
    if (!x || !y) return REPDL_E_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    if (aligned16(x) && aligned16(y)) {
        int64_t nvec = n / 4;
        if (nvec > 0) {
            unary_vec_kernel<Op><<<grid_for(nvec, EW_THREADS * EW_VEC_PER_THREAD), EW_THREADS, 0,
                                   st>>>(x, y, nvec, op);
            int e = launch_status();
            if (e) return e;
        }
        int64_t done = nvec * 4;
        if (done < n) {
            unary_scalar_kernel<Op><<<1, EW_THREADS, 0, st>>>(x + done, y + done, n - done, op);
            return launch_status();
        }
        return REPDL_OK;
    }
    unary_scalar_kernel<Op><<<grid_for(n, EW_THREADS), EW_THREADS, 0, st>>>(x, y, n, op);
    return launch_status();
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_exp(const float *x, float *y, int64_t n, void *stream)
{
    return launch_unary(x, y, n, OpExp{}, stream);
}

extern "C" int repdl_b200_log(const float *x, float *y, int64_t n, void *stream)
{
    return launch_unary(x, y, n, OpLog{}, stream);
}

extern "C" int repdl_b200_sqrt(const float *x, float *y, int64_t n, void *stream)
{
    return launch_unary(x, y, n, OpSqrt{}, stream);
}

extern "C" int repdl_b200_div_scalar(const float *x, float divisor, float *y, int64_t n,
                                     void *stream)
{
    return launch_unary(x, y, n, OpDivScalar{divisor}, stream);
}

extern "C" int repdl_b200_div(const float *x, const float *divisor, float *y, int64_t n,
                              void *stream)
{
    if (n < 0) return REPDL_E_SHAPE;
    if (n == 0) return REPDL_OK;
    if (!x || !y || !divisor) return REPDL_E_NULL;
    div_tensor_kernel<<<grid_for(n, EW_THREADS), EW_THREADS, 0, (cudaStream_t)stream>>>(x, divisor,
                                                                                        y, n);
    return launch_status();
}
