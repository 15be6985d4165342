"""In-tree build of the two native artefacts of this package.

* ``libbsa_b200.so`` -- the torch-free C-ABI kernel library (``csrc/*.cu``,
  declared in ``include/bsa.h``), compiled by nvcc for sm_100a only.
* ``sparse/sparse_ops*.so`` -- the torch-extension binding
  (``native/sparse_ops.cc``), compiled by g++ against the installed torch and
  linked to the kernel library through an ``$ORIGIN``-relative rpath.

Run ``python build.py`` (add ``--force`` to rebuild everything).  Nothing is
installed outside this directory, so the built files travel with the tree.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
INCLUDE_DIR = os.path.join(REPO_DIR, "include")
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libbsa_b200.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
OPS_PATH = os.path.join(PKG_DIR, "sparse", "sparse_ops" + EXT_SUFFIX)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return path


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s" % (" ".join(cmd), proc.stdout))
    if verbose and proc.stdout.strip():
        print(proc.stdout)


def kernel_sources():
    return sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def build_kernel_library(force=False, verbose=False):
    """Compile csrc/*.cu into libbsa_b200.so (one object per source, then link)."""
    sources = kernel_sources()
    headers = [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE_DIR, "bsa.h"))
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    objects, rebuilt = [], False
    for src in sources:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or not _newer(obj, [src] + headers):
            _run([_nvcc()] + NVCC_FLAGS + ["-I", INCLUDE_DIR, "-I", CSRC_DIR, "-c", src, "-o", obj], verbose)
            rebuilt = True
    if rebuilt or not os.path.exists(LIB_PATH):
        _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objects, verbose)
    return LIB_PATH


def build_torch_binding(force=False, verbose=False):
    """Compile native/sparse_ops.cc into sparse/sparse_ops<EXT_SUFFIX>."""
    src = os.path.join(PKG_DIR, "native", "sparse_ops.cc")
    deps = [src, os.path.join(INCLUDE_DIR, "bsa.h")]   # the kernel library is linked dynamically
    if not force and _newer(OPS_PATH, deps):
        return OPS_PATH
    import torch
    from torch.utils import cpp_extension
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], INCLUDE_DIR]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes.append(os.path.join(cuda_home, "include"))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=sparse_ops",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", OPS_PATH, "-L", PKG_DIR, "-lbsa_b200", "-L", torch_lib,
            "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + torch_lib]
    _run(cmd, verbose)
    return OPS_PATH


def build(force=False, verbose=False):
    build_kernel_library(force, verbose)
    build_torch_binding(force, verbose)
    return LIB_PATH, OPS_PATH


if __name__ == "__main__":
    lib, ops = build(force="--force" in sys.argv, verbose=True)
    print("built", lib)
    print("built", ops)
