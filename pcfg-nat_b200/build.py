"""Builds libpcfgnat.so (the C-ABI library of include/pcfgnat.h) in-tree with nvcc for sm_100a.

The DP kernels are compiled WITHOUT fast-math: their tables must be bit-identical to the
reference kernels', which are built with plain ``-O3`` (fs_plugins/custom_ops/pcfg_loss.py:42-43).
Kernels that want fast intrinsics call them by name.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpcfgnat.so")
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = ["cabi.cu", "loss_fwd.cu", "loss_bwd.cu", "loss_balanced.cu", "loss_cluster.cu", "loss_linear.cu", "best_tree.cu", "viterbi.cu", "lookahead.cu", "logsoftmax_gather.cu", "proj_fused.cu", "proj_bwd_gemm.cu", "no_alloc.cu", "criterion_glue.cu", "extract_links.cu", "stage_inputs.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc_path():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def _deps_mtime():
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _compile(nvcc, src, verbose):
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    cmd = [nvcc, *ARCH, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force=False, verbose=False):
    """Compile every translation unit (in parallel) and link the shared library."""
    if not force and os.path.isfile(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        results = list(ex.map(lambda s: _compile(nvcc, s, verbose), SOURCES))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    cmd = [nvcc, *ARCH, "-shared", "-o", LIB, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
