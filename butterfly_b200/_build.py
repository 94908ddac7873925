"""In-tree build of the native libraries (no JIT cache: the built files sit beside the
package so that they travel with the source tree).

    libbfly_b200.so   CUDA kernels + C ABI (include/bfly.h), nvcc, sm_100a only
    _butterfly.so     torch operator layer over the C ABI (torch_butterfly::* operators)
    _version.so       torch_butterfly::cuda_version

The two torch libraries carry the file names the reference package loads
(torch_butterfly/__init__.py:8-11), so they can be dropped into it unchanged.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_CORE = os.path.join(HERE, "libbfly_b200.so")
LIB_OPS = os.path.join(HERE, "_butterfly.so")
LIB_VERSION = os.path.join(HERE, "_version.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)


def build(force=False, verbose=False):
    """Compile whatever is out of date.  Needs nvcc and g++; needs no GPU."""
    import torch
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not os.path.exists(nvcc):
        nvcc = "nvcc"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    headers = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".h")]
    headers.append(os.path.join(HERE, "..", "include", "bfly.h"))
    units = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]
    # one object per translation unit (compiled side by side), linked into one library
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, jobs = [], []
    for cu in units:
        obj = os.path.join(objdir, os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [cu] + headers):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", cu, "-o", obj]
            if verbose:
                print(" ".join(cmd), file=sys.stderr)
            jobs.append((cmd, subprocess.Popen(cmd)))
    for cmd, proc in jobs:
        if proc.wait() != 0:
            raise subprocess.CalledProcessError(proc.returncode, cmd)
    if force or jobs or _newer(LIB_CORE, objs):
        _run([nvcc, "-shared", "-o", LIB_CORE] + objs, verbose)

    tdir = os.path.dirname(torch.__file__)
    inc = ["-I" + os.path.join(tdir, "include"), "-I" + os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(cuda_home, "include")]
    common = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + inc
    tlibs = ["-L" + os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
             "-Wl,-rpath," + os.path.join(tdir, "lib")]
    ops_src = [os.path.join(CSRC, "torch_binding.cpp"), os.path.join(HERE, "..", "include", "bfly.h")]
    if force or _newer(LIB_OPS, ops_src + [LIB_CORE]):
        _run(common + ["-DBFLY_SEPARATE_VERSION_LIB", os.path.join(CSRC, "torch_binding.cpp"), "-o", LIB_OPS,
                       "-L" + HERE, "-lbfly_b200", "-Wl,-rpath,$ORIGIN"] + tlibs, verbose)
    if force or _newer(LIB_VERSION, [os.path.join(CSRC, "version.cpp")]):
        _run(common + [os.path.join(CSRC, "version.cpp"), "-o", LIB_VERSION] + tlibs, verbose)
    return LIB_CORE, LIB_OPS, LIB_VERSION


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
