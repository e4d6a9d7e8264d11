"""Builds libarraydiff_host.so: the C++ op-graph layer (context / spatial comm / ops / zoo / optimizer)
over the C ABI.  Usage: python -m arraydiff_cuda_b200.host.build"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libarraydiff_host.so")
SOURCES = ["host.cc", "ops.cc", "zoo.cc", "optimize.cc", "capi.cc"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, "src", s) for s in SOURCES] + [os.path.join(HERE, "tools", "train_dummy.cc")]
    if not os.path.exists(os.path.join(HERE, "tools", "train_dummy")):
        return True
    inc = os.path.join(HERE, "include", "arraydiff")
    deps += [os.path.join(inc, f) for f in os.listdir(inc)] + [os.path.join(ROOT, "include", "arraydiff_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False):
    from arraydiff_cuda_b200 import build as kbuild
    kbuild.build()
    if not force and not _stale():
        return LIB
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cxx = os.environ.get("HOST_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wno-unused-function",
           "-I", os.path.join(HERE, "include"), "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           *[os.path.join(HERE, "src", s) for s in SOURCES], "-o", LIB,
           "-L", PKG, "-larraydiff_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    # the training driver on synthetic data (the reference's tools/train_imagenet.cc loop over DummyData)
    tool = os.path.join(HERE, "tools", "train_dummy")
    subprocess.check_call([cxx, "-O2", "-std=c++17", "-Wall", "-Wno-unused-function", "-I", os.path.join(HERE, "include"),
                           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
                           os.path.join(HERE, "tools", "train_dummy.cc"), "-o", tool, "-L", PKG, "-larraydiff_host",
                           "-larraydiff_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN/../.."])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
