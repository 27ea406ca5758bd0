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

// Status of the launch that was just enqueued on this thread (0 or a cudaError_t).
static inline int launch_status() { return (int)cudaGetLastError(); }

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per thread; 148 on B200).
int sm_count();

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

}  // namespace repdl_b200
