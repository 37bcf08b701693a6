"""Builds the ``pyCAHEL`` extension module (binding.cpp) in this folder with the host compiler.

The module is what lancelot-main-GPU imports (``import pyCAHEL as cahel``): put this folder on PYTHONPATH.
It links ``../liblancelot_b200.so`` (found at run time relative to the module) and the CUDA runtime."""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)


def target():
    return os.path.join(HERE, "pyCAHEL" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build(force=False):
    import pybind11

    out = target()
    deps = [os.path.join(HERE, "binding.cpp"), os.path.join(ROOT, "include", "cahel_b200.hpp"), os.path.join(ROOT, "include", "lancelot_b200.h")]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(cuda, "include"), deps[0], "-o", out + ".tmp",
           "-L" + PKG, "-llancelot_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building pyCAHEL failed: %s\n%s" % (" ".join(cmd), r.stderr))
    os.replace(out + ".tmp", out)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
