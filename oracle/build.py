"""TEST INFRASTRUCTURE -- compiles oracle/repdl_oracle.c into oracle/librepdl_oracle.so.

Usage: python oracle/build.py [--ref]   (--ref also runs oracle/build_ref.sh on the
reference tree that the environment variable REPDL_REFERENCE names; that takes a few
minutes because the reference's CUDA backend is compiled too).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "repdl_oracle.c")
LIB = os.path.join(HERE, "librepdl_oracle.so")

# -ffp-contract=off: only the explicit fmaf() calls may fuse.  -march=x86-64-v3 (AVX2+FMA)
# rather than native, so that the object built on one host runs on another.
CFLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
          "-fPIC", "-shared", "-Wall"]


def build_oracle(force=False):
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cmd = ["/usr/bin/gcc", *CFLAGS, "-o", LIB, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


def build_ref():
    ref = os.environ.get("REPDL_REFERENCE", "")
    if not ref or not os.path.isdir(ref):
        return False
    subprocess.run(["bash", os.path.join(HERE, "build_ref.sh")], check=True)
    return True


if __name__ == "__main__":
    print(build_oracle(force=True))
    if "--ref" in sys.argv:
        build_ref()
