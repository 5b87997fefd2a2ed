"""ctypes binding of libpcfgnat.so (include/pcfgnat.h).  No torch types cross this boundary:
only raw device pointers, sizes and the CUDA stream handle."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpcfgnat.so")
_lib = None

c_int, c_i64, c_size, c_void = ctypes.c_int, ctypes.c_int64, ctypes.c_size_t, ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol include/pcfgnat.h declares
SIGNATURES = {
    "pcfgnat_version": (c_int, []),
    "pcfgnat_error_string": (ctypes.c_char_p, [c_int]),
    "pcfgnat_loss_fwd": (c_int, [c_void] * 4 + [c_int] * 4 + [c_void] * 4),
    "pcfgnat_loss_bwd": (c_int, [c_void] * 6 + [c_int] * 4 + [c_void] * 5),
    "pcfgnat_loss_workspace_bytes": (c_size, [c_int] * 4),
    "pcfgnat_loss_fwd_bwd_kernels": (c_int, [c_int] * 4),
    "pcfgnat_loss_fwd_bwd": (c_int, [c_void] * 4 + [c_int] * 4 + [c_void, c_size] + [c_void] * 5),
    "pcfgnat_loss_fwd_bwd_static": (c_int, [c_void] * 4 + [c_int] * 4 + [c_void] * 5),
    "pcfgnat_best_tree": (c_int, [c_void] * 5 + [c_int] * 4 + [c_void] * 3),
    "pcfgnat_viterbi": (c_int, [c_void] * 3 + [c_int] * 3 + [c_void] * 6),
    "pcfgnat_viterbi_backtrace": (c_int, [c_void] * 7 + [c_int, c_i64] + [c_int] * 4 + [c_void] * 4),
    "pcfgnat_viterbi_decode": (c_int, [c_void] * 8 + [c_int, c_i64] + [c_int] * 4 + [c_void] * 5),
    "pcfgnat_lookahead_decode": (c_int, [c_void] * 5 + [c_int, ctypes.c_float, c_int, c_i64] + [c_int] * 4 + [c_void] * 4),
    "pcfgnat_logsoftmax_gather": (c_int, [c_void, c_int, c_void] + [c_i64] * 5 + [c_int] * 3 + [c_void] * 3),
    "pcfgnat_proj_workspace_bytes": (c_size, [c_int] * 4),
    "pcfgnat_proj_logsoftmax_gather": (c_int, [c_void] * 5 + [c_int] * 5 + [c_void] * 5 + [c_size] + [c_void] * 2),
    "pcfgnat_proj_dlogits": (c_int, [c_void] * 7 + [c_int] * 5 + [c_void] * 2 + [c_size] + [c_void] * 2),
    "pcfgnat_proj_dlogits_compact": (c_int, [c_void] * 7 + [c_int] * 6 + [c_void] * 4 + [c_size] + [c_void] * 2),
    "pcfgnat_proj_backward_gemms": (c_int, [c_void] * 3 + [c_int] * 3 + [c_void] * 4),
    "pcfgnat_links_gather_features": (c_int, [c_void] * 3 + [c_int] + [c_void] + [c_int] * 5 + [c_void] * 4),
    "pcfgnat_links_scores": (c_int, [c_void] * 3 + [c_int] * 4 + [c_void] * 3),
    "pcfgnat_links_backward": (c_int, [c_void] * 13 + [c_int] * 6 + [c_void] * 8),
    "pcfgnat_links_from_scores": (c_int, [c_void] * 11 + [c_int] * 6 + [c_void] * 2),
    "pcfgnat_copy_links_main_rows": (c_int, [c_void] * 2 + [c_int] * 3 + [c_void]),
    "pcfgnat_plan_real_rows": (c_int, [c_void] + [c_int] * 4 + [c_void] + [c_int]),
    "pcfgnat_copy_real_rows": (c_int, [c_void] * 3 + [c_int] * 3 + [c_size] + [c_int] + [c_void] * 2),
    "pcfgnat_stage_inputs": (c_int, [c_void] * 2 + [c_int] + [c_void] * 3 + [c_int] * 3 + [c_void]),
    "pcfgnat_loss_stats": (c_int, [c_void] * 2 + [c_int] + [c_void] * 2),
    "pcfgnat_loss_stats_exchange": (c_int, [c_void] * 2 + [c_int] + [c_void] + [c_int] * 2 + [c_void] * 3),
    "pcfgnat_glance_select": (c_int, [c_void] * 7 + [c_int, ctypes.c_float] + [c_int] * 3 + [c_void] * 7),
    "pcfgnat_force_emit": (c_int, [c_void] * 3 + [c_int] * 3 + [c_void] * 2),
    "pcfgnat_force_emit_grad": (c_int, [c_void] * 2 + [c_int] * 3 + [c_void] * 2),
}


class LibraryMissing(RuntimeError):
    pass


def lib():
    """Loads the library; raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} is missing: build it with `python pcfg-nat_b200/build.py` (needs nvcc); "
                "there is no CPU fallback")
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().pcfgnat_error_string(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")
