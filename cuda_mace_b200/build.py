"""Builds the C-ABI library in-tree with nvcc, and the TorchScript classes on top of it with g++.

    python -m cuda_mace_b200.build [--force] [-v]

Output: cuda_mace_b200/lib/libcuda_mace_b200.so (sm_100a cubin + compute_100a PTX).  nvcc
cross-compiles, so this runs on a machine without a GPU.  Sources are compiled one object per
file in parallel and only rebuilt when they (or a header) changed.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(LIB_DIR, "libcuda_mace_b200.so")
TORCH_LIB_PATH = os.path.join(LIB_DIR, "libcuda_mace_b200_torch.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".inc"))]
    headers.append(os.path.join(HERE, "..", "include", "cuda_mace_b200.h"))
    hdr_time = _newest(headers)

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        srcp = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(srcp), hdr_time):
            return obj, None
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", srcp, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < _newest(objs):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_torch_classes(force)
    return LIB_PATH


def build_torch_classes(force=False):
    """The TorchScript custom classes with the reference's names (csrc/torch_classes.cpp) on top of the C-ABI
    library: compiled with g++ against the installed torch, linked to libcuda_mace_b200.so next to it."""
    src = os.path.join(CSRC, "torch_classes.cpp")
    hdr = os.path.join(HERE, "..", "include", "cuda_mace_b200.h")
    if not force and os.path.exists(TORCH_LIB_PATH) and \
            os.path.getmtime(TORCH_LIB_PATH) > max(os.path.getmtime(src), os.path.getmtime(hdr)):
        return TORCH_LIB_PATH
    import torch
    from torch.utils import cpp_extension

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w", src, "-o", TORCH_LIB_PATH,
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += ["-I" + p for p in cpp_extension.include_paths()] + ["-I" + os.path.join(cuda_home, "include")]
    cmd += ["-L" + torch_lib, "-lc10", "-ltorch", "-ltorch_cpu", "-lc10_cuda", "-ltorch_cuda",
            "-L" + LIB_DIR, "-lcuda_mace_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for torch_classes.cpp:\n{r.stdout}\n{r.stderr[-4000:]}")
    return TORCH_LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    sys.exit(0)
