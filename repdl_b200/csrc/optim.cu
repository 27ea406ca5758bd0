// Multi-tensor optimizer steps with the operation order of the Python updates they replace, every
// operation rounded separately in fp32 exactly where the element-wise ATen calls round:
//   SGD  : p <- p + (g * -lr)                                  (two roundings; the update style of
//          microsoft/RepDL repdl/optim.py:83)
//   Adam : microsoft/RepDL repdl/optim.py:56-83, including the two places where ATen's
//          `add(x, alpha=a)` is ONE fused multiply-add on CPUs and GPUs with FMA
//          (weight decay, first-moment update), the correctly rounded sqrt / division of
//          repdl.ops.sqrt / repdl.ops.div, and the optional running maximum (amsgrad).
// One launch covers up to kMaxTensors parameter tensors: their pointers travel in the kernel's
// parameter block, so nothing is allocated or copied for the pointer table.
#include "common.cuh"
#include "crmath.cuh"

namespace repdl_b200 {
namespace {

constexpr int kMaxTensors = 24;
constexpr int OPT_THREADS = 256;

struct SgdTable {
    float *p[kMaxTensors];
    const float *g[kMaxTensors];
    long long n[kMaxTensors];
};
struct AdamTable {
    float *p[kMaxTensors];
    const float *g[kMaxTensors];
    float *m[kMaxTensors];
    float *v[kMaxTensors];
    float *vmax[kMaxTensors];  // all null without amsgrad
    long long n[kMaxTensors];
};
struct AdamScalars {
    float beta1, one_minus_beta1, beta2, one_minus_beta2, sqrt_bc2, eps, neg_step_size, weight_decay;
};

// blockIdx.y: tensor; blockIdx.x / gridDim.x: grid-stride over its elements
__global__ void __launch_bounds__(OPT_THREADS) sgd_kernel(const SgdTable t, float neg_lr)
{
    float *__restrict__ p = t.p[blockIdx.y];
    const float *__restrict__ g = t.g[blockIdx.y];
    const long long n = t.n[blockIdx.y];
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n;
         i += (long long)gridDim.x * OPT_THREADS)
        p[i] = __fadd_rn(p[i], __fmul_rn(g[i], neg_lr));
}

__global__ void __launch_bounds__(OPT_THREADS) adam_kernel(const AdamTable t, const AdamScalars s)
{
    float *__restrict__ p = t.p[blockIdx.y];
    const float *__restrict__ g = t.g[blockIdx.y];
    float *__restrict__ m = t.m[blockIdx.y];
    float *__restrict__ v = t.v[blockIdx.y];
    float *__restrict__ vmax = t.vmax[blockIdx.y];
    const long long n = t.n[blockIdx.y];
    for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n;
         i += (long long)gridDim.x * OPT_THREADS) {
        const float pi = p[i];
        float gi = g[i];
        if (s.weight_decay != 0.0f) gi = __fmaf_rn(pi, s.weight_decay, gi);       // grad.add(param, alpha=wd)
        const float mi = __fmaf_rn(gi, s.one_minus_beta1, __fmul_rn(m[i], s.beta1));  // mul_(b1).add_(g, alpha=1-b1)
        const float vi = __fadd_rn(__fmul_rn(v[i], s.beta2),
                                   __fmul_rn(__fmul_rn(gi, gi), s.one_minus_beta2));  // mul_(b2).add_(mul(g,g).mul(1-b2))
        m[i] = mi;
        v[i] = vi;
        float root = vi;
        if (vmax) {
            // torch.maximum: a NaN in either operand is the result
            const float old = vmax[i];
            root = (old != old) ? old : ((vi != vi) ? vi : fmaxf(old, vi));
            vmax[i] = root;
        }
        const float denom = __fadd_rn(cr_div(cr_sqrt(root), s.sqrt_bc2), s.eps);
        p[i] = __fadd_rn(pi, __fmul_rn(cr_div(mi, denom), s.neg_step_size));
    }
}

unsigned blocks_for_max(const long long *n, int count)
{
    long long mx = 0;
    for (int i = 0; i < count; i++) mx = n[i] > mx ? n[i] : mx;
    long long b = (mx + OPT_THREADS * 4 - 1) / (OPT_THREADS * 4);  // four elements per thread
    const long long cap = (long long)sm_count() * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

extern "C" int repdl_b200_sgd_step(float *const *params, const float *const *grads,
                                   const int64_t *sizes, int ntensors, float neg_lr, void *stream)
{
    clear_stale_error();
    if (ntensors < 0) return REPDL_E_SHAPE;
    if (ntensors == 0) return REPDL_OK;
    if (!params || !grads || !sizes) return REPDL_E_NULL;
    for (int i = 0; i < ntensors; i++) {
        if (sizes[i] < 0) return REPDL_E_SHAPE;
        if (sizes[i] > 0 && (!params[i] || !grads[i])) return REPDL_E_NULL;
    }
    for (int base = 0; base < ntensors; base += kMaxTensors) {
        SgdTable t = {};
        const int count = ntensors - base < kMaxTensors ? ntensors - base : kMaxTensors;
        for (int i = 0; i < count; i++)
            t.p[i] = params[base + i], t.g[i] = grads[base + i], t.n[i] = sizes[base + i];
        sgd_kernel<<<dim3(blocks_for_max(t.n, count), (unsigned)count), OPT_THREADS, 0,
                     (cudaStream_t)stream>>>(t, neg_lr);
        const int e = launch_status();
        if (e) return e;
    }
    return REPDL_OK;
}

extern "C" int repdl_b200_adam_step(float *const *params, const float *const *grads,
                                    float *const *exp_avg, float *const *exp_avg_sq,
                                    float *const *max_exp_avg_sq, const int64_t *sizes, int ntensors,
                                    float beta1, float one_minus_beta1, float beta2,
                                    float one_minus_beta2, float sqrt_bias_correction2, float eps,
                                    float neg_step_size, float weight_decay, void *stream)
{
    clear_stale_error();
    if (ntensors < 0) return REPDL_E_SHAPE;
    if (ntensors == 0) return REPDL_OK;
    if (!params || !grads || !exp_avg || !exp_avg_sq || !sizes) return REPDL_E_NULL;
    for (int i = 0; i < ntensors; i++) {
        if (sizes[i] < 0) return REPDL_E_SHAPE;
        if (sizes[i] > 0 && (!params[i] || !grads[i] || !exp_avg[i] || !exp_avg_sq[i] ||
                             (max_exp_avg_sq && !max_exp_avg_sq[i])))
            return REPDL_E_NULL;
    }
    const AdamScalars s = {beta1, one_minus_beta1, beta2, one_minus_beta2, sqrt_bias_correction2,
                           eps, neg_step_size, weight_decay};
    for (int base = 0; base < ntensors; base += kMaxTensors) {
        AdamTable t = {};
        const int count = ntensors - base < kMaxTensors ? ntensors - base : kMaxTensors;
        for (int i = 0; i < count; i++) {
            t.p[i] = params[base + i], t.g[i] = grads[base + i];
            t.m[i] = exp_avg[base + i], t.v[i] = exp_avg_sq[base + i];
            t.vmax[i] = max_exp_avg_sq ? max_exp_avg_sq[base + i] : nullptr;
            t.n[i] = sizes[base + i];
        }
        adam_kernel<<<dim3(blocks_for_max(t.n, count), (unsigned)count), OPT_THREADS, 0,
                      (cudaStream_t)stream>>>(t, s);
        const int e = launch_status();
        if (e) return e;
    }
    return REPDL_OK;
}
