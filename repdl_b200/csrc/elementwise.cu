// Elementwise fp32 math for sm_100a: div, sqrt, exp, log with the bits of the reference's CPU run.
//
// All four are HBM-bound streams (4 B in, 4 B out per element): 128-bit loads and stores, three or
// four independent 16-byte groups in flight per thread, a grid of a few CTAs per SM walking the array
// with a grid stride.  The arithmetic per element is in crmath.cuh.
#include "common.cuh"
#include "crmath.cuh"

namespace repdl_b200 {
namespace {

// exp/log read one table entry per element at a data-dependent index; the tables (1 KB and
// 2 KB) are staged in shared memory once per CTA so that those reads never leave the SM.
// (Replicating every entry once per lane to make the lookups bank-conflict-free was tried and is
// slower: 32-48 KB per CTA costs more occupancy than the conflicts cost bandwidth.)
struct SmemTables {
    const double *p;  // [0, N_exp) 2^(j/N); then N_log pairs (c_i, -log c_i), 16-byte aligned
    __device__ __forceinline__ double exp_t(int j) const { return p[j]; }
    __device__ __forceinline__ void log_ct(int i, double &c, double &t_hi) const
    {
        const double2 v = *reinterpret_cast<const double2 *>(p + CRM_EXP_N + 2 * i);
        c = v.x, t_hi = v.y;
    }
};
constexpr int TABLE_DOUBLES = CRM_EXP_N + 2 * CRM_LOG_N;

__device__ __forceinline__ void stage_tables(double *sm)
{
    for (int i = threadIdx.x; i < TABLE_DOUBLES; i += blockDim.x) {
        unsigned long long b;
        if (i < CRM_EXP_N) {
            b = CRM_EXP_T_HI[i];
        } else {
            const int e = i - CRM_EXP_N;
            b = (e & 1) ? CRM_LOG_T_HI[e >> 1] : CRM_LOG_C[e >> 1];
        }
        sm[i] = __longlong_as_double((long long)b);
    }
    __syncthreads();
}

// An Op gives fast(x, tab, slow): the result of the branch-free path plus a flag "this element
// needs slow(x)".  The kernels evaluate four elements, OR the flags and branch once.
struct OpSqrt {
    static constexpr bool kTables = false;
    static constexpr int kGroups = 3;
    __device__ __forceinline__ float fast(float x, SmemTables, bool &slow) const
    {
        slow = false;
        return cr_sqrt(x);
    }
    __device__ __forceinline__ float slow(float x) const { return cr_sqrt(x); }
};
struct OpExp {
    static constexpr bool kTables = true;
    static constexpr int kGroups = 4;
    __device__ __forceinline__ float fast(float x, SmemTables t, bool &slow) const
    {
        return cr_exp_fast(x, t, slow);
    }
    __device__ __forceinline__ float slow(float x) const { return crm_exp_slow(x); }
};
struct OpLog {
    static constexpr bool kTables = true;
    static constexpr int kGroups = 3;
    __device__ __forceinline__ float fast(float x, SmemTables t, bool &slow) const
    {
        return cr_log_fast(x, t, slow);
    }
    __device__ __forceinline__ float slow(float x) const { return crm_log_slow(x); }
};
// x / d for one divisor d (cr_div_by_reciprocal: one fp64 multiply, exact division only for
// subnormal and NaN results).
struct OpDivScalar {
    static constexpr bool kTables = false;
    static constexpr int kGroups = 4;
    float d;
    double rd;
    __device__ __forceinline__ float fast(float x, SmemTables, bool &slow) const
    {
        return cr_div_by_reciprocal(x, rd, slow);
    }
    __device__ __forceinline__ float slow(float x) const { return cr_div(x, d); }
};

template <class Op>
__device__ __forceinline__ float4 apply4(const Op &op, float4 v, SmemTables tab)
{
    bool s0, s1, s2, s3;
    float4 r;
    r.x = op.fast(v.x, tab, s0);
    r.y = op.fast(v.y, tab, s1);
    r.z = op.fast(v.z, tab, s2);
    r.w = op.fast(v.w, tab, s3);
    if (s0 | s1 | s2 | s3) {  // rare
        if (s0) r.x = op.slow(v.x);
        if (s1) r.y = op.slow(v.y);
        if (s2) r.z = op.slow(v.z);
        if (s3) r.w = op.slow(v.w);
    }
    return r;
}

constexpr int EW_THREADS = 256;

// Op::kGroups 16-byte groups are in flight per thread (measured per operator: three for log and
// sqrt, four for exp and the division).  At least four CTAs per SM: exp and log would otherwise take
// 80 registers and run three (exp 0.80 instead of 0.85 of the HBM peak).
template <class Op>
__global__ void __launch_bounds__(EW_THREADS, 4)
unary_vec_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t nvec, Op op)
{
    // nvec = number of float4 groups; x and y are 16-byte aligned
    __shared__ __align__(16) double tables[Op::kTables ? TABLE_DOUBLES : 2];
    if (Op::kTables) stage_tables(tables);
    const SmemTables tab{tables};
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS * Op::kGroups;
    int64_t base = (int64_t)blockIdx.x * EW_THREADS * Op::kGroups + threadIdx.x;
    // whole blocks of Op::kGroups groups per thread: no bounds tests
    for (; base + (Op::kGroups - 1) * EW_THREADS < nvec; base += stride) {
        float4 v[Op::kGroups];
#pragma unroll
        for (int u = 0; u < Op::kGroups; u++) v[u] = ldg_stream_f4(x + 4 * (base + u * EW_THREADS));
#pragma unroll
        for (int u = 0; u < Op::kGroups; u++)
            stg_stream_f4(y + 4 * (base + u * EW_THREADS), apply4(op, v[u], tab));
    }
    // the ragged end of the array (at most one pass per thread)
#pragma unroll 1
    for (int u = 0; u < Op::kGroups; u++) {
        const int64_t i = base + (int64_t)u * EW_THREADS;
        if (i < nvec) stg_stream_f4(y + 4 * i, apply4(op, ldg_stream_f4(x + 4 * i), tab));
    }
}

template <class Op>
__global__ void __launch_bounds__(EW_THREADS)
unary_scalar_kernel(const float *__restrict__ x, float *__restrict__ y, int64_t n, Op op)
{
    __shared__ __align__(16) double tables[Op::kTables ? TABLE_DOUBLES : 2];
    if (Op::kTables) stage_tables(tables);
    const SmemTables tab{tables};
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    for (int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += stride)
    {
        bool slow;
        const float v = __ldg(x + i);
        float r = op.fast(v, tab, slow);
        if (slow) r = op.slow(v);
        y[i] = r;
    }
}

__global__ void __launch_bounds__(EW_THREADS)
div_tensor_kernel(const float *__restrict__ x, const float *__restrict__ d, float *__restrict__ y,
                  int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    for (int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += stride)
        y[i] = cr_div(__ldg(x + i), __ldg(d + i));
}

static unsigned grid_for(int64_t work_items, int per_block, int per_sm = 8)
{
    int64_t blocks = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)sm_count() * per_sm;
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
            unary_vec_kernel<Op><<<grid_for(nvec, EW_THREADS * Op::kGroups), EW_THREADS, 0,
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
    clear_stale_error();
    return launch_unary(x, y, n, OpExp{}, stream);
}

extern "C" int repdl_b200_log(const float *x, float *y, int64_t n, void *stream)
{
    clear_stale_error();
    return launch_unary(x, y, n, OpLog{}, stream);
}

extern "C" int repdl_b200_sqrt(const float *x, float *y, int64_t n, void *stream)
{
    clear_stale_error();
    return launch_unary(x, y, n, OpSqrt{}, stream);
}

extern "C" int repdl_b200_div_scalar(const float *x, float divisor, float *y, int64_t n,
                                     void *stream)
{
    clear_stale_error();
    return launch_unary(x, y, n, OpDivScalar{divisor, 1.0 / (double)divisor}, stream);
}

extern "C" int repdl_b200_div(const float *x, const float *divisor, float *y, int64_t n,
                              void *stream)
{
    clear_stale_error();
    if (n < 0) return REPDL_E_SHAPE;
    if (n == 0) return REPDL_OK;
    if (!x || !y || !divisor) return REPDL_E_NULL;
    div_tensor_kernel<<<grid_for(n, EW_THREADS), EW_THREADS, 0, (cudaStream_t)stream>>>(x, divisor,
                                                                                        y, n);
    return launch_status();
}
