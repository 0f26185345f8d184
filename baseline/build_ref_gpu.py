"""Builds the reference's own sm_100 GEMM kernels as an on-box comparator: baseline/_ref/libmslk_ref_gpu.so.

    python baseline/build_ref_gpu.py --ref-root <checkout of meta-pytorch/MSLK> [--jobs 5]

The instance files the reference's heuristics pick for the benchmark shapes are compiled WHERE THEY LIE in
the reference checkout (nothing is copied into this repository) against the stock CUTLASS headers that ship
inside the flashinfer wheel -- the reference pins a CUTLASS fork whose checkout is empty, so numbers from this
library are "reference sources at stock CUTLASS", not the pinned fork:

  csrc/gemm/cutlass/f8f8bf16_rowwise/f8f8bf16_rowwise_128_256_128_2_1_1_10_f_f.cu   (M > 1024 on sm_100)
  csrc/gemm/cutlass/f8f8bf16_rowwise/f8f8bf16_rowwise_128_64_128_1_1_1_10_f_f.cu    (M <= 128, N > 1024)
  csrc/gemm/cutlass/f8f8bf16_rowwise_grouped_sm100/f8f8bf16_rowwise_grouped_256_256_128_2_1_1_10_f.cu
  csrc/gemm/cutlass/f4f4bf16/f4f4bf16_256_256_2_1_1.cu, f4f4bf16_256_128_4_1_1.cu   (8192^3; M = 1 / 32)

The two NVFP4 files name a type that exists only in the fork (`mx_float4_16_t`, the 1x16 MXFP4 mode); they are
compiled from temporary copies (in a scratch directory outside the repository) with that alias, its trait
specialisation and the branch that uses it removed -- the NVFP4 branch is untouched.
`baseline/ref_gpu_shim.cpp` registers the instances under `torch.ops.mslk_ref`.  Objects and the library go to
baseline/_ref/ only (git-ignored; it still travels to the GPU box).

`--python` also mirrors the reference's pure-Python package (its Triton quantizers) to baseline/_ref/pyref/mslk so
that `triton_quantize_fp8_row` can be timed on the GPU box, where the reference checkout does not exist
(import it with MSLK_PYTHON_ONLY=1 and baseline/_ref/pyref on sys.path).
"""

from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

ROWWISE = ["f8f8bf16_rowwise/f8f8bf16_rowwise_128_256_128_2_1_1_10_f_f.cu",
           "f8f8bf16_rowwise/f8f8bf16_rowwise_128_64_128_1_1_1_10_f_f.cu"]
GROUPED = ["f8f8bf16_rowwise_grouped_sm100/f8f8bf16_rowwise_grouped_256_256_128_2_1_1_10_f.cu"]
NVFP4 = ["f4f4bf16/f4f4bf16_256_256_2_1_1.cu", "f4f4bf16/f4f4bf16_256_128_4_1_1.cu"]
# grouped FP4 (NVFP4 and MXFP4 branches; stacked, 2D-3D and 2D-2D forms): the instance the heuristic picks for the MoE shapes
GROUPED_FP4 = ["f4f4bf16_grouped/f4f4bf16_grouped_256_256_256_2_1_1.cu"]


def cutlass_include_dirs():
    import flashinfer
    root = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
    dirs = [os.path.join(root, "include"), os.path.join(root, "tools", "util", "include")]
    for d in dirs:
        if not os.path.isdir(d):
            raise RuntimeError(f"stock CUTLASS headers not found at {d}")
    return dirs


def patched_nvfp4_copy(ref_cutlass_dir, rel, scratch):
    """Temporary copy of an NVFP4 instance file and of f4f4bf16_common.cuh without the fork-only 1x16 MXFP4 type."""
    d = os.path.join(scratch, "f4f4bf16")
    os.makedirs(d, exist_ok=True)
    common = open(os.path.join(ref_cutlass_dir, "f4f4bf16", "f4f4bf16_common.cuh")).read()
    common = re.sub(r"using MXFP4_16 =[^;]*;\n", "", common)
    common = re.sub(r"template <typename F4>\s*struct ultra_sf_vec_size<cutlass::mx_float4_16_t<F4>> \{[^}]*\};\n", "", common)
    if "mx_float4_16_t" in common:
        raise RuntimeError("f4f4bf16_common.cuh: the 1x16 MXFP4 type is still named after patching")
    with open(os.path.join(d, "f4f4bf16_common.cuh"), "w") as f:
        f.write(common)
    inst = open(os.path.join(ref_cutlass_dir, rel)).read()
    inst = re.sub(r"\} else if \(mxfp4_block_size == 16\) \{.*?\} else \{", "} else {", inst, flags=re.S)
    if "MXFP4_16" in inst:
        raise RuntimeError(f"{rel}: the 1x16 MXFP4 branch is still present after patching")
    dst = os.path.join(d, os.path.basename(rel))
    with open(dst, "w") as f:
        f.write(inst)
    return dst


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=os.environ.get("MSLK_REF_ROOT", ""),
                    help="checkout of the reference (meta-pytorch/MSLK); default: $MSLK_REF_ROOT")
    ap.add_argument("--jobs", type=int, default=5)
    ap.add_argument("--only", default="", help="comma-separated substrings of instance names to (re)build")
    ap.add_argument("--python", action="store_true", help="mirror the reference's Python package to _ref/pyref/mslk")
    args = ap.parse_args()
    if not os.path.isdir(os.path.join(args.ref_root, "csrc", "gemm", "cutlass")):
        sys.exit("build_ref_gpu.py: pass --ref-root <checkout of the reference> (or set MSLK_REF_ROOT)")
    if args.python:
        import shutil
        dst = os.path.join(OUT, "pyref", "mslk")
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        # only what the quantizer imports: the package root, mslk/quantize and mslk/utils
        os.makedirs(dst)
        shutil.copy(os.path.join(args.ref_root, "mslk", "__init__.py"), dst)
        for sub in ("quantize", "utils"):
            shutil.copytree(os.path.join(args.ref_root, "mslk", sub), os.path.join(dst, sub),
                            ignore=shutil.ignore_patterns("*.so", "__pycache__", "*.pyc"))
        print(dst)
    import torch
    from torch.utils import cpp_extension as ce
    ref_cutlass = os.path.join(args.ref_root, "csrc", "gemm", "cutlass")
    os.makedirs(OUT, exist_ok=True)
    scratch = tempfile.mkdtemp(prefix="mslk_ref_gpu_")
    inc = [os.path.join(args.ref_root, "include"), *cutlass_include_dirs(), *ce.include_paths(),
           sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "-O2", "--expt-relaxed-constexpr",
             "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
             "-DMSLK_DISABLE_SM90_CUTLASS", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-Xcompiler", "-fPIC", "-w"]
    jobs = []
    for rel in ROWWISE + GROUPED + GROUPED_FP4:
        jobs.append((os.path.join(ref_cutlass, rel), [os.path.join(ref_cutlass, os.path.dirname(rel))]))
    for rel in NVFP4:
        jobs.append((patched_nvfp4_copy(ref_cutlass, rel, scratch), [os.path.join(scratch, "f4f4bf16")]))
    only = [s for s in args.only.split(",") if s]

    def compile_one(job):
        src, extra_inc = job
        obj = os.path.join(OUT, os.path.basename(src)[:-3] + ".o")
        if os.path.exists(obj) and (not only or not any(s in src for s in only)):
            return obj, 0, "cached"
        cmd = ["nvcc", *flags, *[f"-I{d}" for d in extra_inc + inc], "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return obj, r.returncode, (r.stdout + r.stderr)[-4000:]

    with ThreadPoolExecutor(max_workers=args.jobs) as ex:
        results = list(ex.map(compile_one, jobs))
    ok = True
    for obj, rc, msg in results:
        print(f"[{'ok' if rc == 0 else 'FAILED'}] {os.path.basename(obj)} {msg if rc else ''}", flush=True)
        ok = ok and rc == 0
    if not ok:
        sys.exit(1)
    shim_obj = os.path.join(OUT, "ref_gpu_shim.o")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
                           *[f"-I{d}" for d in ce.include_paths()], f"-I{sysconfig.get_paths()['include']}",
                           "-c", os.path.join(HERE, "ref_gpu_shim.cpp"), "-o", shim_obj])
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    lib = os.path.join(OUT, "libmslk_ref_gpu.so")
    subprocess.check_call(["nvcc", "-shared", "-o", lib, shim_obj, *[o for o, _, _ in results],
                           f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcuda",
                           "-Xlinker", f"-rpath={torch_lib}"])
    print(lib)


if __name__ == "__main__":
    main()
