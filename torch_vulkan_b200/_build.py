"""Builds the package's native code in-tree, for sm_100a only.

  lib/libtvb200.so   the runtime and the CUDA kernels behind the C ABI of
                     include/tvb200.h (nvcc; no torch, no libcuda link)
  _native*.so        the ATen layer: the PrivateUse1 backend "vk" and the four
                     quantised ops, compiled against libtorch and linked to
                     libtvb200.so (see csrc/aten)

The reference builds its shaders with slangc per dtype variant and its C++
objects against libtorch from crates/*/build.rs; here nvcc cross-compiles the
kernels (no GPU needed) and a plain g++ invocation builds the extension.
Run as `python -m torch_vulkan_b200._build` or through __graft_entry__.build().
"""

import concurrent.futures
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libtvb200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _headers():
    return glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True) + \
        glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True) + [os.path.join(ROOT, "include", "tvb200.h")]


def build_core(verbose=False, ptxas_info=False):
    """Compiles csrc/core and csrc/kernels into lib/libtvb200.so."""
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "core", "*.cu")) + glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    headers = _headers()
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if _newer(obj, [src] + headers):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, r in pool.map(run, jobs):
            if verbose or ptxas_info or r.returncode != 0:
                sys.stderr.write(" ".join(cmd[-3:]) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or _newer(LIB, objects):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objects + ["-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.check_call(cmd)
    return LIB


def native_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "_native" + suffix)


def build_native(verbose=False):
    """Compiles csrc/aten (the PrivateUse1 backend and the ops) into _native.so."""
    import torch
    from torch.utils import cpp_extension

    build_core(verbose)
    out = native_path()
    sources = sorted(glob.glob(os.path.join(CSRC, "aten", "*.cpp")))
    if not _newer(out, sources + _headers() + [LIB]):
        return out
    os.makedirs(OBJ, exist_ok=True)
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], os.path.join(ROOT, "include")]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DTORCH_EXTENSION_NAME=_native",
              "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-Wno-deprecated-declarations"]
    for inc in includes:
        cflags += ["-isystem", inc]
    objects, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJ, "aten_" + os.path.basename(src)[:-4] + ".o")
        objects.append(obj)
        if _newer(obj, [src] + _headers()):
            jobs.append(["g++"] + cflags + ["-c", src, "-o", obj])

    def run(cmd):
        return cmd, subprocess.run(cmd, capture_output=True, text=True)

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, r in pool.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd[-3:]) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("g++ failed for " + cmd[-3])
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-shared", "-o", out] + objects + [
        "-L", torch_lib, "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
        "-L", os.path.dirname(LIB), "-ltvb200", "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath," + torch_lib]
    subprocess.check_call(cmd)
    return out


def build_all(verbose=False):
    build_core(verbose)
    return build_native(verbose)


if __name__ == "__main__":
    if "--ptxas" in sys.argv:
        build_core(verbose=True, ptxas_info=True)
    elif "--core" in sys.argv:
        print(build_core(verbose="-v" in sys.argv))
    else:
        print(build_all(verbose="-v" in sys.argv))
