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
