// Shared helpers for the repdl_b200 kernels (sm_100a).
//
// Numerical ground rules for every file that includes this header:
//   * compiled with -fmad=false, -ftz=false, -prec-div=true, -prec-sqrt=true: the compiler never
//     fuses a multiply with an add on its own and never flushes subnormals;
//   * every fused multiply-add that is part of an accumulation chain is written as an explicit
//     __fmaf_rn / __fma_rn, every chain add as __fadd_rn, so the evaluation order in the source
//     is the evaluation order on the GPU.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/repdl_b200.h"

namespace repdl_b200 {

constexpr int kNumSMsB200 = 148;

// The CUDA runtime keeps one "last error" per host thread, shared with every other library in the
// process (PyTorch included).  Each entry point drops whatever an earlier, unrelated call left
// there, so that launch_status() reports only this library's own launches.
static inline void clear_stale_error() { (void)cudaGetLastError(); }
// Status of the launch that was just enqueued on this thread (0 or a cudaError_t).
static inline int launch_status() { return (int)cudaGetLastError(); }

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per thread; 148 on B200).
int sm_count();

// conv.cu: C[m][n] = chain over k of A[m][k] * B[n][k] for dense, k-contiguous operands, on the chain kernel
// of conv2d_grad_kernel (REPDL_E_UNSUPPORTED when the shape does not suit it).
int mm_long_k(const float *A, const float *B, float *C, int M, int N, int K, cudaStream_t st);

// The plain single-thread chain walk of sum1d.cu for short chains (no scratch): out[0] = factor * chain.
int sum1d_plain(const float *x, float *out, int64_t n, float factor, cudaStream_t st);

__device__ __forceinline__ float4 ldg_f4(const float *p)
{
    return __ldg(reinterpret_cast<const float4 *>(p));
}

// Streaming 128-bit load / store (cache-streaming hint) for data that is touched exactly once.
__device__ __forceinline__ float4 ldg_stream_f4(const float *p)
{
    return __ldcs(reinterpret_cast<const float4 *>(p));
}

__device__ __forceinline__ void stg_stream_f4(float *p, float4 v)
{
    __stcs(reinterpret_cast<float4 *>(p), v);
}

// cp.async (LDGSTS): 16-byte global -> shared copy that bypasses registers.
__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src)
{
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
// 4-byte global -> shared copy; copies nothing and writes zero when `valid` is false (the source
// address must still be a mapped one).
__device__ __forceinline__ void cp_async_4_zfill(void *smem_dst, const void *gmem_src, bool valid)
{
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gmem_src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Opt in to more than 48 KB of dynamic shared memory, once per device, for one kernel.  `done_mask`
// must be a static that belongs to that kernel alone (bit d set: applied on device d).
template <class Kern>
int ensure_smem(Kern kern, int bytes, unsigned long long *done_mask)
{
    if (bytes <= 48 * 1024) return 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    unsigned long long bit = 1ull << (dev & 63);
    if (__atomic_load_n(done_mask, __ATOMIC_ACQUIRE) & bit) return 0;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    __atomic_fetch_or(done_mask, bit, __ATOMIC_RELEASE);
    return 0;
}

}  // namespace repdl_b200
