"""Builds the native parts of repdl_b200 in-tree.

  librepdl_b200.so            the CUDA kernels behind the C ABI of include/repdl_b200.h
                              (nvcc, sm_100a only, no torch dependency)
  librepdl_b200_probe.so      benchmark helper (an FMA-pipe peak probe kernel), loaded by bench.py only
  backend/cuda*.so            the PyTorch extension that registers those kernels under the
                              names microsoft/RepDL's backend/cuda/bind.cpp:12-19 exports, so that
                              it can stand in for `repdl.backend.cuda`

Usage: python -m repdl_b200.build [--force] [--no-ext]
"""
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "librepdl_b200.so")
PROBE_LIB = os.path.join(HERE, "librepdl_b200_probe.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

# Numerics flags are part of the contract: no implicit FMA contraction, no flush-to-zero,
# IEEE division and square root.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++",
]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_lib(force=False, verbose=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
            + [os.path.join(HERE, "..", "include", "repdl_b200.h")])
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC, *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((s, subprocess.Popen(cmd)))
    for s, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed on " + s)
    if force or procs or _newer(LIB, objs):
        subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-ccbin", "/usr/bin/g++",
                        "-cudart", "shared"], check=True)
    # the benchmark's peak probe: a library of its own, outside the operator ABI
    probe_src = os.path.join(CSRC, "probe", "probe.cu")
    if force or _newer(PROBE_LIB, [probe_src] + hdrs):
        subprocess.run([NVCC, *NVCC_FLAGS, "-shared", "-o", PROBE_LIB, probe_src, "-cudart", "shared"],
                       check=True)
    return LIB


def build_ext(force=False):
    """The drop-in `cuda` extension module (PyInit_cuda), linked against librepdl_b200.so."""
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(HERE, "backend", "cuda", "bind.cpp")
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(HERE, "backend", "cuda" + suffix)
    if not force and not _newer(out, [src, LIB, os.path.join(HERE, "..", "include", "repdl_b200.h")]):
        return out
    incs = cpp_extension.include_paths(device_type="cuda")
    libdirs = cpp_extension.library_paths(device_type="cuda")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=cuda",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(HERE, "..", "include")]
    cmd += ["-I" + i for i in incs]
    cmd += [src, "-o", out, "-L" + HERE, "-lrepdl_b200", "-Wl,-rpath,$ORIGIN/.."]
    for d in libdirs:
        cmd += ["-L" + d, "-Wl,-rpath," + d]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(cmd, check=True)
    return out


def main(argv):
    force = "--force" in argv
    print(build_lib(force=force, verbose="-v" in argv))
    if "--no-ext" not in argv:
        print(build_ext(force=force))


if __name__ == "__main__":
    main(sys.argv[1:])
