"""Builds the reference's own CUDA extension for sm_100 -- TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--force]

Compiles the two source files of tukisuwa/CAME's extension (came_pytorch/came_cuda/csrc/came_bindings.cpp and
came_kernels.cu) from where they lie in the reference checkout, with the flags the reference's setup.py:54-66
passes (`--use_fast_math -lineinfo`, C++17) plus the sm_100 code generation its build would pick up from the
visible GPU, straight with nvcc / g++ and torch's include paths (the reference's setup.py is not run).  The only
output is oracle/_ref/came_cuda_ext.so, a pybind11 module; it is git-ignored and never part of the product: the
tests and the benchmark's reference arm load it as the second oracle / the GPU baseline when it is present.
No reference source is copied anywhere.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "came_cuda_ext.so")
MODULE = "came_cuda_ext"


def reference_root() -> str | None:
    for cand in (os.environ.get("CAME_REFERENCE_ROOT"), "/root/reference"):
        if cand and os.path.exists(os.path.join(cand, "came_pytorch", "came_cuda", "csrc", "came_kernels.cu")):
            return cand
    return None


def build(force: bool = False, verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when no reference checkout is present (then an
    already-built module, if any, is left alone)."""
    root = reference_root()
    if root is None:
        return OUT if os.path.exists(OUT) else None
    csrc = os.path.join(root, "came_pytorch", "came_cuda", "csrc")
    srcs = [os.path.join(csrc, "came_bindings.cpp"), os.path.join(csrc, "came_kernels.cu")]
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(s) for s in srcs):
        return OUT
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    obj_cpp, obj_cu = os.path.join(OUT_DIR, "came_bindings.o"), os.path.join(OUT_DIR, "came_kernels.o")
    cmds = [
        ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc, "-c", srcs[0], "-o", obj_cpp],
        # torch's CUDAExtension adds the three -D__CUDA_NO_* switches and --expt-relaxed-constexpr to every nvcc line
        [nvcc, "-O3", "-std=c++17", "--use_fast_math", "-lineinfo", "-gencode", "arch=compute_100,code=sm_100",
         "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__",
         "-D__CUDA_NO_HALF2_OPERATORS__", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", *defs, *inc,
         "-c", srcs[1], "-o", obj_cu],
    ]
    procs = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for c in cmds]
    for c, p in zip(cmds, procs):
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"reference extension: {os.path.basename(c[0])} failed on {c[-3]}")
    libs = []
    for p in ce.library_paths("cuda"):
        libs += ["-L", p, f"-Wl,-rpath,{p}"]
    link = ["g++", "-shared", obj_cpp, obj_cu, "-o", OUT + ".tmp", *libs, "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("reference extension: link failed:\n" + res.stderr)
    os.replace(OUT + ".tmp", OUT)
    for o in (obj_cpp, obj_cu):
        os.remove(o)
    return OUT


def load():
    """Imports the built module (torch must be imported first: the module links against it); None when absent."""
    if not os.path.exists(OUT):
        return None
    import importlib.util
    import torch  # noqa: F401
    spec = importlib.util.spec_from_file_location(MODULE, OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
