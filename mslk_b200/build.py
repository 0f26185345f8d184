"""In-tree build of the native libraries (sm_100a only).

``build()`` compiles every ``csrc/*.cu`` with nvcc into ``mslk_b200/libmslk_b200.so``
(the C-ABI library: no torch dependency, CUDA runtime linked statically) and,
with ``torch_ops=True``, ``csrc/torch_ops.cpp`` into ``mslk_b200/_torch_ops.so``
(the thin PyTorch extension that registers the ``mslk::`` operators over the C ABI).
Objects are cached under ``csrc/_build`` and rebuilt when a source or header is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_build")
LIB = os.path.join(PKG, "libmslk_b200.so")
TORCH_LIB = os.path.join(PKG, "_torch_ops.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the mslk_b200 kernels cannot be built")


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)


def build(force: bool = False, verbose: bool = False, torch_ops: bool = True) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    hdr_time = _newest(headers)
    cus = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    nvcc = _nvcc()
    jobs, objs = [], []
    for f in cus:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or not os.path.exists(LIB):
        _run([nvcc, "-shared", "-o", LIB, *objs, "-cudart", "static"], verbose)
    if torch_ops:
        build_torch_ops(force=force or bool(jobs), verbose=verbose)
    return LIB


def build_torch_ops(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_ops.cpp")
    if not os.path.exists(src):
        return ""
    hdr = os.path.join(INCLUDE, "mslk_b200.h")
    if not force and os.path.exists(TORCH_LIB) and os.path.getmtime(TORCH_LIB) >= max(
            os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(LIB)):
        return TORCH_LIB
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{INCLUDE}", "-I/usr/local/cuda/include"]
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [
        # the system g++: its libstdc++.so is the one libtorch uses.  ($CXX may point at a toolchain that links
        # libstdc++ statically; a second copy of the stream/locale state inside this library crashes on the first
        # formatted TORCH_CHECK message.)
        os.environ.get("MSLK_B200_CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_EXTENSION_NAME=_torch_ops",
        *inc, src, "-o", TORCH_LIB,
        f"-L{PKG}", "-lmslk_b200", f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd, verbose)
    return TORCH_LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
