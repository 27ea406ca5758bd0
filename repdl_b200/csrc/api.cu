// Library identification and status text for the repdl_b200 C ABI.
#include "common.cuh"

extern "C" int repdl_b200_version(void) { return 100; }

extern "C" int repdl_b200_sm_arch(void) { return 100; }

extern "C" const char *repdl_b200_strerror(int status)
{
    switch (status) {
        case REPDL_OK: return "success";
        case REPDL_E_NULL: return "a required pointer is NULL";
        case REPDL_E_SHAPE: return "a dimension is negative or inconsistent";
        case REPDL_E_RANGE: return "a size exceeds what the kernel can index";
        case REPDL_E_SCRATCH: return "scratch buffer missing or too small";
        case REPDL_E_UNSUPPORTED: return "unsupported argument combination";
        case REPDL_E_STATIC_MAX:
            return "input is larger than the built-in scratch array of this entry point supports "
                   "(see repdl_b200_sum1d_static_max_n); use the variant that takes caller scratch";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown repdl_b200 status";
}

// Strided sub-matrix copy on a stream (cudaMemcpy2DAsync): `rows` rows of `width_bytes` bytes each.
// direction 0: host -> device, 1: device -> host, 2: device -> device.  Host memory should be pinned,
// or the copy is not asynchronous.
extern "C" int repdl_b200_copy2d(void *dst, int64_t dst_pitch_bytes, const void *src, int64_t src_pitch_bytes,
                                 int64_t width_bytes, int64_t rows, int direction, void *stream)
{
    repdl_b200::clear_stale_error();
    if (width_bytes < 0 || rows < 0 || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes)
        return REPDL_E_SHAPE;
    if (width_bytes == 0 || rows == 0) return REPDL_OK;
    if (!dst || !src) return REPDL_E_NULL;
    const cudaMemcpyKind kind = direction == 0   ? cudaMemcpyHostToDevice
                                : direction == 1 ? cudaMemcpyDeviceToHost
                                : direction == 2 ? cudaMemcpyDeviceToDevice
                                                 : cudaMemcpyDefault;
    if (direction < 0 || direction > 2) return REPDL_E_UNSUPPORTED;
    return (int)cudaMemcpy2DAsync(dst, (size_t)dst_pitch_bytes, src, (size_t)src_pitch_bytes, (size_t)width_bytes,
                                  (size_t)rows, kind, (cudaStream_t)stream);
}
