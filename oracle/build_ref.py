"""Compiles the reference's own C++ library (its six TorchScript classes over its NVRTC-compiled kernels) from
the sources where they lie in a read-only reference checkout.  TEST AND BASELINE INFRASTRUCTURE ONLY: the product
(`cuda_mace_b200/`) never loads, links or imports what this builds.

    python -m oracle.build_ref [--reference /path/to/reference] [--force]

Output: oracle/_ref/libcuda_mace.so (git-ignored).  Nothing else is kept; no reference source is copied into
the repository.

What the recipe does instead of the reference's CMake project (cuda_mace/CMakeLists.txt:42-114):
  * the ten translation units of `add_library(cuda_mace SHARED ...)` (CMakeLists.txt:42-54) are compiled with g++
    against the installed torch headers, straight from the checkout;
  * each wrapper includes "generated/wrapped_<name>_impl.cu", which CMake makes by concatenating
    cuda/include/<name>_impl.cuh, cuda/include/cuda_utils.hpp and cuda/src/<name>_impl.cu
    (cmake/PrependHeadersToSource.cmake:5-30) inside a C++ raw string literal R"======( ... )======"
    (cmake/MakeIncludeable.cmake:8-17).  The same five files are written to a temporary directory that is
    deleted after the compile; the kernels are compiled by NVRTC at their first launch, on the GPU box.

The library needs CUDA_HOME at run time (jit_wrappers/include/cuda_cache.hpp:20-27) and resolves libcuda.so,
libcudart.so and libnvrtc.so by dlopen (jit_wrappers/include/dynamic_cuda.hpp:76-338).
"""
import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libcuda_mace.so")
# the reference checkout: $CUDA_MACE_REFERENCE, else a directory "reference" next to this repository
DEFAULT_REFERENCE = os.environ.get("CUDA_MACE_REFERENCE",
                                   os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))

KERNEL_FILES = ["cubic_spline_impl", "invariant_message_passing_impl", "spherical_harmonics_impl", "linear_impl",
                "symmetric_contraction_impl"]
UNITS = ["jit_wrappers/src/cubic_spline_wrapper.cpp", "jit_wrappers/src/invariant_message_passing_wrapper.cpp",
         "jit_wrappers/src/spherical_harmonics_wrapper.cpp", "jit_wrappers/src/linear_wrapper.cpp",
         "jit_wrappers/src/symmetric_contraction_wrapper.cpp", "src/linear.cpp", "src/invariant_message_passing.cpp",
         "src/symmetric_contraction.cpp", "src/cubic_spline.cpp", "src/spherical_harmonics.cpp"]


def available(reference=DEFAULT_REFERENCE):
    return os.path.isfile(os.path.join(reference, "cuda_mace", "CMakeLists.txt"))


def build(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of the built library, or None when there is no reference checkout to build from (then a
    library built earlier, if any, is what the tests and the baseline use)."""
    if not available(reference):
        return LIB_PATH if os.path.isfile(LIB_PATH) else None
    root = os.path.join(reference, "cuda_mace")
    srcs = [os.path.join(root, u) for u in UNITS]
    if not force and os.path.isfile(LIB_PATH) and os.path.getmtime(LIB_PATH) > max(os.path.getmtime(s) for s in srcs):
        return LIB_PATH
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    tmp = tempfile.mkdtemp(prefix="cuda_mace_ref_")
    try:
        gen = os.path.join(tmp, "generated")
        os.makedirs(gen)
        for name in KERNEL_FILES:
            parts = [os.path.join(root, "cuda", "include", name + ".cuh"),
                     os.path.join(root, "cuda", "include", "cuda_utils.hpp"),
                     os.path.join(root, "cuda", "src", name + ".cu")]
            body = "".join("\n" + open(p).read() for p in parts)
            with open(os.path.join(gen, f"wrapped_{name}.cu"), "w") as f:
                f.write('R"======(\n' + body + '\n)======"')
        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        inc = [os.path.join(root, "cuda", "include"), os.path.join(root, "include"),
               os.path.join(root, "jit_wrappers", "include"), tmp, os.path.join(cuda_home, "include")]
        inc += cpp_extension.include_paths()
        flags = ["-O2", "-std=c++17", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        flags += ["-I" + p for p in inc]

        def compile_one(src):
            obj = os.path.join(tmp, os.path.basename(src)[:-4] + ".o")
            r = subprocess.run(["g++"] + flags + ["-c", src, "-o", obj], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {src}:\n{r.stderr[-4000:]}")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            objs = list(ex.map(compile_one, srcs))
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["g++", "-shared", "-o", LIB_PATH] + objs + ["-L" + torch_lib, "-lc10", "-ltorch", "-ltorch_cpu",
                                                          "-lc10_cuda", "-ltorch_cuda", "-ldl",
                                                          "-Wl,-rpath," + torch_lib]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print(p if p else "no reference checkout and no library built earlier")
    sys.exit(0 if p else 1)
