// BENCHMARK HELPER, not part of the operator library: built into its own shared object
// (librepdl_b200_probe.so), which only bench.py loads.
//
// Peak-rate probes: dependent-free FFMA / DFMA loops that keep every FMA lane of the GPU busy.
// bench.py times them to obtain the FP32 (and FP64) FMA-pipe peak of the very GPU, clocks and
// power state the benchmark runs on; the GEMM roofline is quoted against that number.
#include "../common.cuh"

namespace repdl_b200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) fma_probe_kernel(T *out, int iters, T seed)
{
    T a[16];
#pragma unroll
    for (int i = 0; i < 16; i++) a[i] = seed + (T)(threadIdx.x + i);
    const T m = (T)1.0000001, c = (T)1e-9;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if constexpr (sizeof(T) == 4)
                a[i] = __fmaf_rn(a[i], m, c);
            else
                a[i] = __fma_rn(a[i], m, c);
        }
    }
    T s = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) s += a[i];
    if (s == (T)12345.678) out[0] = s;  // never true; keeps the loop alive
}

// Packed variant: fma.rn.f32x2, two FP32 FMAs per instruction.
__global__ void __launch_bounds__(256) fma2_probe_kernel(float *out, int iters, float seed)
{
    unsigned long long a[16], m, c;
    asm("mov.b64 %0, {%1,%2};" : "=l"(m) : "f"(1.0000001f), "f"(0.9999999f));
    asm("mov.b64 %0, {%1,%2};" : "=l"(c) : "f"(1e-9f), "f"(2e-9f));
#pragma unroll
    for (int i = 0; i < 16; i++)
        asm("mov.b64 %0, {%1,%2};" : "=l"(a[i]) : "f"(seed + threadIdx.x + i), "f"(seed + i));
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 16; i++) asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(a[i]) : "l"(m), "l"(c));
    }
    float s = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        float lo, hi;
        asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a[i]));
        s += lo + hi;
    }
    if (s == 12345.678f) out[0] = s;
}

}  // namespace
}  // namespace repdl_b200

using namespace repdl_b200;

// Launches blocks_per_sm * SMs CTAs of 256 threads; each thread issues 16 * iters FMAs
// (fp64 = 0: scalar fp32 FFMA; 1: fp64 DFMA; 2: packed fp32 fma.rn.f32x2, 2 FMAs per instruction).
extern "C" int repdl_b200_probe_fma(int fp64, int iters, int blocks_per_sm, void *scratch_out,
                                    double *flops_issued, void *stream)
{
    clear_stale_error();
    if (iters <= 0 || blocks_per_sm <= 0) return REPDL_E_SHAPE;
    if (!scratch_out) return REPDL_E_NULL;
    int dev = 0, sms = kNumSMsB200;
    if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    unsigned blocks = (unsigned)(sms * blocks_per_sm);
    if (fp64 == 2) {
        fma2_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((float *)scratch_out, iters, 1.0f);
        if (flops_issued) *flops_issued = 4.0 * 16.0 * (double)iters * 256.0 * (double)blocks;
        return launch_status();
    }
    if (fp64)
        fma_probe_kernel<double><<<blocks, 256, 0, (cudaStream_t)stream>>>((double *)scratch_out,
                                                                           iters, 1.0);
    else
        fma_probe_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float *)scratch_out,
                                                                          iters, 1.0f);
    if (flops_issued) *flops_issued = 2.0 * 16.0 * (double)iters * 256.0 * (double)blocks;
    return launch_status();
}
