"""TEST INFRASTRUCTURE -- builds oracle/_ref/refmath.so and oracle/_ref/refmath_cuda.so.

The reference implements exp2d/log1d on the CPU (backend/cpu/math.cpp:19-47) but
its module init (backend/cpu/bind.cpp:6-19) never exports them.  This script
compiles the reference's unmodified math.cpp together with a pybind shim that
only declares and exports those two functions, so that the oracle can be checked
against them and so that they can be timed as the CPU baseline.  The same is
done for the reference's CUDA versions (backend/cuda/math.cu:15-66, compiled for
sm_100a; refmath_cuda.so), which its module init does not export either and
which the benchmark times as "the reference's own GPU kernels" next to this
repository's.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("REPDL_REFERENCE", "")
OUT = os.path.join(HERE, "_ref")

SHIM = r"""
#include <torch/extension.h>
namespace repdl { namespace cpu { namespace math {
torch::Tensor exp2d(const torch::Tensor &input);
torch::Tensor log1d(const torch::Tensor &input);
}}}
PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("exp2d", &repdl::cpu::math::exp2d);
    m.def("log1d", &repdl::cpu::math::log1d);
}
"""


SHIM_CUDA = SHIM.replace("namespace cpu", "namespace cuda").replace("repdl::cpu::", "repdl::cuda::")


def main():
    if not REF or not os.path.isdir(REF):
        print("no reference tree; refmath not built")
        return
    os.environ["CXX"] = "/usr/bin/g++"
    os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension

    bdir = os.path.join(OUT, "refmath_build")
    os.makedirs(bdir, exist_ok=True)
    shim = os.path.join(bdir, "refmath_shim.cpp")
    with open(shim, "w") as f:
        f.write(SHIM)
    cpp_extension.load(
        name="refmath",
        sources=[shim, os.path.join(REF, "backend/cpu/math.cpp")],
        extra_cflags=["-O2", "-fopenmp"],
        extra_ldflags=["-fopenmp"],
        build_directory=bdir,
        verbose=False,
    )
    import shutil

    shutil.copy(os.path.join(bdir, "refmath.so"), os.path.join(OUT, "refmath.so"))
    print("built", os.path.join(OUT, "refmath.so"))
    if os.environ.get("REF_SKIP_CUDA", "0") == "1":
        return
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    cdir = os.path.join(OUT, "refmath_cuda_build")
    os.makedirs(cdir, exist_ok=True)
    shim = os.path.join(cdir, "refmath_cuda_shim.cpp")
    with open(shim, "w") as f:
        f.write(SHIM_CUDA)
    cpp_extension.load(
        name="refmath_cuda",
        sources=[shim, os.path.join(REF, "backend/cuda/math.cu")],
        extra_cflags=["-O2"],
        with_cuda=True,
        build_directory=cdir,
        verbose=False,
    )
    shutil.copy(os.path.join(cdir, "refmath_cuda.so"), os.path.join(OUT, "refmath_cuda.so"))
    print("built", os.path.join(OUT, "refmath_cuda.so"))


if __name__ == "__main__":
    sys.exit(main())
