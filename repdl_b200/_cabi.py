"""ctypes binding of the C ABI declared in include/repdl_b200.h.

The shared library is the product: if it is missing or a symbol is absent, importing this module
raises.  There is no CPU fallback and no other backend.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librepdl_b200.so")

_i64, _int, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_float
_ptr, _size = ctypes.c_void_p, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/repdl_b200.h declaration by declaration
SIGNATURES = {
    "repdl_b200_sgd_step": (_int, [_ptr, _ptr, _ptr, _int, _f32, _ptr]),
    "repdl_b200_adam_step": (_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _int] + [_f32] * 8 + [_ptr]),
    "repdl_b200_version": (_int, []),
    "repdl_b200_sm_arch": (_int, []),
    "repdl_b200_strerror": (ctypes.c_char_p, [_int]),
    "repdl_b200_mm": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _i64, _int, _int, _i64, _i64, _i64, _ptr]),
    "repdl_b200_mm_allgather": (_int, [_ptr, _ptr, _ptr, _int, _i64, _i64, _i64, _i64, _int, _int,
                                       _i64, _i64, _i64, _ptr]),
    "repdl_b200_conv2d": (_int, [_ptr, _ptr, _ptr] + [_i64] * 12 + [_ptr]),
    "repdl_b200_conv2d_bias_act": (_int, [_ptr, _ptr, _ptr, _ptr] + [_i64] * 12 + [_int, _ptr]),
    "repdl_b200_maxpool2d": (_int, [_ptr, _ptr, _ptr] + [_i64] * 5 + [_ptr]),
    "repdl_b200_maxpool2d_backward": (_int, [_ptr, _ptr, _ptr] + [_i64] * 5 + [_ptr]),
    "repdl_b200_cross_entropy_grad": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _ptr]),
    "repdl_b200_copy2d": (_int, [_ptr, _i64, _ptr, _i64, _i64, _i64, _int, _ptr]),
    "repdl_b200_conv2d_grad_input": (_int, [_ptr, _ptr, _ptr] + [_i64] * 11 + [_ptr]),
    "repdl_b200_conv2d_grad_kernel": (_int, [_ptr, _ptr, _ptr] + [_i64] * 11 + [_ptr]),
    "repdl_b200_conv2d_grad_kernel_bias": (_int, [_ptr, _ptr, _ptr, _ptr] + [_i64] * 11 + [_ptr]),
    "repdl_b200_sum1d_scratch_bytes": (_size, [_i64]),
    "repdl_b200_sum1d": (_int, [_ptr, _ptr, _i64, _f32, _ptr, _size, _ptr]),
    "repdl_b200_sum1d_stats": (_int, [_ptr, _ptr]),
    "repdl_b200_sum1d_static_max_n": (_i64, []),
    "repdl_b200_sum1d_static": (_int, [_ptr, _ptr, _i64, _f32, _ptr]),
    "repdl_b200_sum2d_dim0": (_int, [_ptr, _ptr, _i64, _i64, _f32, _ptr]),
    "repdl_b200_sum2d_dim1": (_int, [_ptr, _ptr, _i64, _i64, _f32, _ptr]),
    "repdl_b200_sum4d_dim023": (_int, [_ptr, _ptr, _i64, _i64, _i64, _f32, _ptr]),
    "repdl_b200_exp": (_int, [_ptr, _ptr, _i64, _ptr]),
    "repdl_b200_log": (_int, [_ptr, _ptr, _i64, _ptr]),
    "repdl_b200_sqrt": (_int, [_ptr, _ptr, _i64, _ptr]),
    "repdl_b200_div_scalar": (_int, [_ptr, _f32, _ptr, _i64, _ptr]),
    "repdl_b200_div": (_int, [_ptr, _ptr, _ptr, _i64, _ptr]),
    "repdl_b200_softmax": (_int, [_ptr, _ptr, _i64, _i64, _ptr]),
    "repdl_b200_cross_entropy": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _ptr, _ptr]),
}


class ReproError(RuntimeError):
    """A repdl_b200 C-ABI call returned a non-zero status."""


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "repdl_b200: %s is missing. Build it with `python -m repdl_b200.build`; "
            "there is no fallback implementation." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(status, what):
    if status != 0:
        msg = lib.repdl_b200_strerror(status).decode()
        raise ReproError("%s failed: status %d (%s)" % (what, status, msg))
