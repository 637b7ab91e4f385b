"""ctypes binding of libuniql_b200.so (the C ABI declared in include/uniql_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os

from ._build import LIB_PATH

_c = ctypes
_lib = None


class Prefetch(ctypes.Structure):
    """uniql_prefetch of include/uniql_b200.h: a byte range to pull into L2 when a decode launch ends."""
    _fields_ = [("ptr", _c.c_void_p), ("bytes", _c.c_size_t)]


class Proj(ctypes.Structure):
    """uniql_w4a16_proj of include/uniql_b200.h: one projection of a grouped decode launch."""
    _fields_ = [("B", _c.c_void_p), ("s", _c.c_void_p), ("bias", _c.c_void_p), ("D", _c.c_void_p),
                ("ldd", _c.c_int64), ("n", _c.c_int64), ("n_out", _c.c_int64)]


# name -> (restype, argtypes); must list every symbol include/uniql_b200.h declares
SYMBOLS = {
    "uniql_abi_version": (_c.c_int, []),
    "uniql_strerror": (_c.c_char_p, [_c.c_int]),
    "uniql_last_cuda_error": (_c.c_int, []),
    "uniql_w4a16_linear": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_size_t,
        _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_linear_static": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_linear_allreduce": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64,
        _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_scratch_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64]),
    "uniql_w4a16_linear_group": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.POINTER(Proj), _c.c_int, _c.c_int, _c.c_void_p, _c.c_int64,
        _c.c_int64, _c.POINTER(Prefetch), _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_group_scratch_bytes": (_c.c_size_t, [
        _c.c_int64, _c.c_int64, _c.POINTER(_c.c_int64), _c.c_int, _c.c_int, _c.c_int64]),
    "uniql_w4a16_linear_group_tp": (_c.c_int, [
        _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64,
        _c.POINTER(Proj), _c.c_int, _c.c_int, _c.c_void_p, _c.c_int64, _c.c_int64, _c.POINTER(Prefetch), _c.c_int,
        _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_plan_selftest": (_c.c_int, [
        _c.c_int64, _c.c_int64, _c.POINTER(_c.c_int64), _c.c_int, _c.c_int, _c.c_int64, _c.c_int64,
        _c.POINTER(_c.c_int)]),
    "uniql_w4a16_gemv_plan_check": (_c.c_int, [
        _c.c_int64, _c.c_int64, _c.POINTER(_c.c_int64), _c.c_int, _c.c_int, _c.POINTER(_c.c_int64)]),
    "uniql_w4_embedding": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64,
        _c.c_void_p, _c.c_void_p]),
    "uniql_silu_mul": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p]),
    "uniql_hadamard": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_float, _c.c_int, _c.c_void_p]),
    "uniql_hadamard_base_matrix": (_c.c_int, [_c.c_int, _c.c_void_p]),
    "uniql_hadamard_set_base_matrix": (_c.c_int, [_c.c_int, _c.c_void_p]),
    "uniql_w4a16_gather_columns": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p,
        _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_dequantize_rows": (_c.c_int, [
        _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p,
        _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "uniql_w4a16_quantize": (_c.c_int, [
        _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
        _c.c_int64, _c.c_void_p]),
    "uniql_comm_handle_bytes": (_c.c_size_t, []),
    "uniql_comm_create": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int64, _c.POINTER(_c.c_void_p), _c.c_void_p]),
    "uniql_comm_connect": (_c.c_int, [_c.c_void_p, _c.c_void_p]),
    "uniql_comm_destroy": (_c.c_int, [_c.c_void_p]),
    "uniql_allreduce_push": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p]),
}


def lib() -> ctypes.CDLL:
    """Load (once) and return the library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m uniql_b200._build` "
                "(needs nvcc). uniql_b200 has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


_ext = None
_ext_tried = False


def torch_ext():
    """The torch binding of the same library (uniql_b200/_torch_ext.so, built from csrc/torch_binding.cpp), or None.

    The modules' forward goes through it when it is there: the C++ binding does in a few microseconds what the ctypes
    path below does in tens.  Both end in the same C-ABI calls of libuniql_b200.so.  UNIQL_B200_TORCH_EXT=0 keeps
    everything on ctypes; a missing or unloadable binding does the same with a warning (it is built by
    `python -m uniql_b200._build`)."""
    global _ext, _ext_tried
    if _ext_tried:
        return _ext
    _ext_tried = True
    if os.environ.get("UNIQL_B200_TORCH_EXT", "1") == "0":
        return None
    try:
        lib()
        import torch  # noqa: F401  (libtorch must be loaded before the binding)
        from . import _torch_ext as ext
        if ext.abi_version() != lib().uniql_abi_version():
            raise RuntimeError("torch binding and library disagree on the ABI version")
        _ext = ext
    except Exception as e:  # noqa: BLE001
        import warnings
        warnings.warn(f"uniql_b200: torch binding not loaded ({e}); module calls go through ctypes")
        _ext = None
    return _ext


class UniqlError(RuntimeError):
    def __init__(self, code: int, where: str):
        msg = lib().uniql_strerror(code).decode()
        if code == -5:
            msg += f" [cudaError {lib().uniql_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (code {code})")
        self.code = code


def check(code: int, where: str) -> None:
    if code != 0:
        raise UniqlError(code, where)
