"""B200-native (sm_100a) implementation of PCFG-NAT's structured-loss and decoding path.

Drop-in for ``fs_plugins/custom_ops`` of the reference: the five public operators live in
``custom_ops`` (same names, signatures and return structure), hand-written CUDA kernels
behind a C-ABI shared library (``include/pcfgnat.h``) do the work.  There is no CPU
fallback: operators raise if the library or a GPU is missing.
"""
__version__ = "0.1.0"

from . import sharding, support_tree, synthetic  # noqa: F401
