"""ctypes binding of libinfllmv2_b200.so (the C ABI of include/infllmv2_b200.h).

The product path has no fallback: if the shared object is missing or a call fails, an exception
is raised.  Nothing here imports the CPU oracle.
"""
import ctypes
import os
import re
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libinfllmv2_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG_DIR), "include", "infllmv2_b200.h")

_lib = None
_lock = threading.Lock()

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> argtypes, mirroring include/infllmv2_b200.h (every pointer is passed as an address)
SIGNATURES = {
    "ifv2_check_status": [c_void_p, c_void_p],
    "ifv2_selftest_umma": [c_int] + [c_void_p] * 5,
    "ifv2_selftest_wait_timeout": [c_void_p, c_int64, c_int, c_void_p, c_void_p],
    "ifv2_topk_to_uint64": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
    "ifv2_blockmask_to_uint64": [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    "ifv2_uint64_to_bool": [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p],
    "ifv2_transpose_blockmask": [c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p],
    "ifv2_compress_keys": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int,
                           c_int, c_int, c_void_p],
    "ifv2_compress_keys_append": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int,
                                  c_int, c_int, c_void_p],
    "ifv2_max_pooling_1d": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ifv2_max_pooling_1d_varlen": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int64, c_int, c_int64, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p],
    "ifv2_topk_select": [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int64, c_int,
                         c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ifv2_topk_select_mask": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int64,
                              c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "ifv2_stage1_scores": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int64, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                           c_int64, c_float, c_int, c_void_p, c_void_p],
    "ifv2_stage1_decode_scores": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int,
                                  c_int, c_int, c_int, c_int64, c_float, c_int, c_void_p, c_int64, c_void_p],
    "ifv2_decode_select": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ifv2_stage1_decode_select": [c_void_p] * 7 + [c_int, c_int64] + [c_int] * 12 + [c_float, c_int, c_void_p,
                                                                               c_int64, c_void_p],
    "ifv2_cache_fill": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int,
                        c_void_p],
    "ifv2_decode_append": [c_void_p] * 10 + [c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_void_p],
    "ifv2_stage1_block_scores": [c_void_p] * 8 + [c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int,
                                                  c_int, c_int, c_int, c_int, c_int64, c_int, c_int,
                                                  c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ifv2_sparse_attn_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int,
                             c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ifv2_sparse_attn_fwd_paged": [c_void_p] * 6 + [c_int] + [c_void_p] * 5 + [c_int, c_int, c_int, c_int64,
                                                                              c_int64, c_int, c_int, c_int, c_int,
                                                                              c_int, c_float, c_int, c_void_p,
                                                                              c_void_p],
    "ifv2_stage1_paged": [c_void_p] * 9 + [c_int, c_int, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int,
                                           c_int, c_int, c_int64, c_int, c_int, c_int, c_int, c_float, c_int,
                                           c_void_p, c_void_p],
    "ifv2_sparse_attn_bwd": [c_void_p] * 9 + [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int,
                                              c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                                              c_float, c_int, c_void_p, c_int64, c_void_p,
                                              c_void_p],
    "ifv2_sparse_attn_bwd_noalloc": [c_void_p] * 9 + [c_void_p, c_int, c_void_p, c_int64, c_void_p,
                                                      c_void_p, c_int, c_int64, c_int64, c_int,
                                                      c_int, c_int, c_int, c_int, c_float, c_int,
                                                      c_void_p, c_void_p],
    "ifv2_decode": [c_void_p] * 8 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int64,
                                     c_int64, c_float, c_void_p, c_int64, c_void_p],
    "ifv2_decode_rotary": [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "ifv2_decode_paged": [c_void_p] * 8 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                           c_void_p, c_int, c_int, c_void_p, c_void_p, c_float,
                                           c_void_p, c_int64, c_void_p],
}
_INT64_RETURNS = {
    "ifv2_sparse_attn_bwd_workspace_bytes": [c_int64, c_int, c_int],
    "ifv2_decode_workspace_bytes": [c_int, c_int, c_int, c_int],
    "ifv2_stage1_decode_workspace_bytes": [c_int, c_int, c_int],
}


class Ifv2Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def declared_symbols():
    """Every function name declared in include/infllmv2_b200.h."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(ifv2_[a-z0-9_]+)\s*\(", text)))


def load():
    """Load the shared object (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m infllmv2_cuda_impl_b200.build` "
                "(needs nvcc; the kernels target sm_100a).  There is no CPU fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, c_int
        for name, args in _INT64_RETURNS.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, c_int64
        lib.ifv2_last_error.restype = ctypes.c_char_p
        lib.ifv2_version.restype = c_int
        _lib = lib
    return _lib


def call(name, *args):
    """Invoke an int-returning entry point and raise on a non-zero status."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.ifv2_last_error().decode(errors="replace")
        kind = {-1: ValueError, -2: NotImplementedError}.get(rc, Ifv2Error)
        raise kind(f"{name} failed (status {rc}): {msg}")
    return rc
