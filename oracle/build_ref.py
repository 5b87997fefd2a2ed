"""Build recipe for the UNMODIFIED reference extension (test infrastructure only).

Compiles the six reference sources where they lie (fs_plugins/custom_ops/pcfg_loss.cpp,
pcfg_loss.cu, pcfg_loss_backward.cu, pcfg_best_tree.cu, pcfg_viterbi.cu,
logsoftmax_gather.cu) for sm_100a into ``oracle/_ref/pcfg_loss_fn.so`` with the same
compiler flags the reference's own loader uses (fs_plugins/custom_ops/pcfg_loss.py:32-45:
``-DOF_SOFTMAX_USE_FAST_MATH -O3 -lineinfo``).  Nothing is copied into the repository:
the output directory is git-ignored and only holds build products.

The resulting module is the checker the golden fixtures are generated from
(tests/golden/make_golden_ref.py) and is never imported by the product package.

Beside the extension it stages a byte-for-byte copy of the reference's Python wrapper
(fs_plugins/custom_ops/pcfg_loss.py) into the same git-ignored directory, so that a test can run the
UNMODIFIED wrapper on top of this package's extension object where the reference checkout is not mounted.

Usage:  python oracle/build_ref.py --reference /path/to/PCFG-NAT      (or PCFGNAT_REFERENCE=/path/to/PCFG-NAT)
"""
import argparse
import importlib.machinery
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MODULE_NAME = "pcfg_loss_fn"  # the name the reference gives its extension (pcfg_loss.py:33)
SOURCES = [
    "pcfg_loss.cpp",
    "pcfg_loss.cu",
    "pcfg_loss_backward.cu",
    "pcfg_best_tree.cu",
    "pcfg_viterbi.cu",
    "logsoftmax_gather.cu",
]


WRAPPER_COPY = "reference_pcfg_loss_wrapper.py"


def ref_so_path():
    return os.path.join(REF_DIR, MODULE_NAME + ".so")


def ref_wrapper_path():
    return os.path.join(REF_DIR, WRAPPER_COPY)


def find_reference():
    """The reference checkout: $PCFGNAT_REFERENCE, else a directory ``reference`` beside this repository.
    None when neither holds fs_plugins/custom_ops."""
    cands = [os.environ.get("PCFGNAT_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "fs_plugins", "custom_ops")):
            return c
    return None


def stage_wrapper(reference_root):
    """Copies the reference's own Python wrapper, unchanged, beside the built extension."""
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copyfile(os.path.join(reference_root, "fs_plugins", "custom_ops", "pcfg_loss.py"), ref_wrapper_path())
    return ref_wrapper_path()


def build_if_stale(reference_root):
    if not os.path.isfile(ref_so_path()):
        build(reference_root)
    if not os.path.isfile(ref_wrapper_path()):
        stage_wrapper(reference_root)


def build(reference_root, verbose=False):
    """Compile the reference sources in place; returns the path of the built module."""
    import torch  # noqa: F401
    from torch.utils.cpp_extension import load

    src_dir = os.path.join(reference_root, "fs_plugins", "custom_ops")
    sources = [os.path.join(src_dir, s) for s in SOURCES]
    for s in sources:
        if not os.path.isfile(s):
            raise FileNotFoundError(s)
    os.makedirs(REF_DIR, exist_ok=True)
    # An empty arch list stops torch from appending its own -gencode flags; the
    # explicit sm_100a flag below is then the only target.
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    load(
        MODULE_NAME,
        sources=sources,
        extra_cflags=["-DOF_SOFTMAX_USE_FAST_MATH", "-O3"],
        extra_cuda_cflags=["-DOF_SOFTMAX_USE_FAST_MATH", "-O3", "-lineinfo"],
        build_directory=REF_DIR,
        is_python_module=False,  # only build; loading a CUDA module needs no GPU but we import lazily
        verbose=verbose,
    )
    return ref_so_path()


def load_ref():
    """Import the prebuilt reference module (raises if it has not been built)."""
    import torch  # noqa: F401  (the module links against libtorch)

    path = ref_so_path()
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not built; run oracle/build_ref.py where the reference is mounted")
    loader = importlib.machinery.ExtensionFileLoader(MODULE_NAME, path)
    spec = importlib.util.spec_from_file_location(MODULE_NAME, path, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=find_reference(), help="root of the PCFG-NAT checkout")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    if not a.reference:
        ap.error("no reference checkout found: pass --reference or set PCFGNAT_REFERENCE")
    p = build(a.reference, a.verbose)
    stage_wrapper(a.reference)
    print("built", p, file=sys.stderr)
