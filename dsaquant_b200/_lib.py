"""ctypes binding of libb200w4a4.so (the C ABI declared in include/b200w4a4.h).

There is no CPU fallback: if the library cannot be loaded every op raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p, POINTER
from typing import Optional

from .csrc import build as _build

ABI_VERSION = 1

# name -> (restype, argtypes); must list every symbol of include/b200w4a4.h.
SIGNATURES = {
    "b200w4a4_version": (c_int, []),
    "b200w4a4_strerror": (c_char_p, [c_int]),
    "b200w4a4_query": (c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "b200w4a4_pack_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200w4a4_repack_bytes": (c_size_t, [c_int, c_int]),
    "b200w4a4_repack_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200w4a4_qact_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200w4a4_quantize_act": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]),
    "b200w4a4_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200w4a4_linear_workspace_bytes": (c_size_t, [c_int, c_int]),
    "b200w4a4_linear": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_float, c_void_p]),
    "b200w4a4_quantize_act_fused": (c_int, [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_float, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "b200w4a4_gemm_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_void_p]),
    "b200w4a4_gemm_split": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200w4a4_qk_norm_rope": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, ctypes.c_longlong, c_int, c_int, c_void_p]),
    "b200w4a4_qk_norm_rope_push": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong, c_void_p, c_int, ctypes.c_uint32, c_void_p, c_int, c_int, c_void_p]),
    "b200w4a4_attn_merge": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_void_p]),
    "b200w4a4_wait_flags": (c_int, [c_void_p, c_int, ctypes.c_uint32, c_int, c_void_p]),
    "b200w4a4_signal_flags": (c_int, [c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p]),
    "b200w4a4_linear_fused": (c_int, [c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_size_t, c_int, c_int, c_int, c_float, c_void_p]),
    "b200w4a4_linear_noalloc": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "b200w4a4_linear_noalloc_max_codes": (c_size_t, []),
    "b200w4a4_linear_noalloc_max_rows": (c_int, []),
    "b200w4a4_unpack_codes": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200w4a4_set_cta_group": (c_int, [c_int]),
    "b200w4a4_set_weight_staging": (c_int, [c_int]),
    "b200w4a4_last_device_status": (c_int, [c_int]),
    "b200w4a4_check_device": (c_int, [c_int]),
    "b200w4a4_map_cache_stats": (None, [POINTER(ctypes.c_ulonglong), POINTER(ctypes.c_ulonglong)]),
}

_LIB: Optional[ctypes.CDLL] = None
_LOAD_ERROR: Optional[BaseException] = None
_LOCK = threading.Lock()


class B200W4A4Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        text = strerror(code)
        super().__init__(f"{where}: {text} (code {code})")


def load() -> ctypes.CDLL:
    """Loads the in-tree library, rebuilding it first when it is missing or older than its
    sources.  A stale library is never loaded silently: without nvcc it is refused.
    B200W4A4_NO_JIT=1 means "use the prebuilt file as it is": nothing is built or compared.
    Raises on failure."""
    global _LIB, _LOAD_ERROR
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        try:
            path = _build.lib_path()
            no_jit = os.environ.get("B200W4A4_NO_JIT", "0") == "1"
            if no_jit:
                if not path.exists():
                    raise FileNotFoundError(f"{path} is missing and B200W4A4_NO_JIT=1")
            elif _build.is_stale(path):
                if _build.nvcc_path() is None:
                    raise RuntimeError(f"{path} is missing or older than its sources and nvcc was not found")
                path = _build.build()
            lib = ctypes.CDLL(str(path))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            got = lib.b200w4a4_version()
            if got != ABI_VERSION:
                raise RuntimeError(f"{path}: ABI version {got}, expected {ABI_VERSION}")
            _LIB, _LOAD_ERROR = lib, None
            return lib
        except BaseException as exc:  # keep the original exception for diagnostics
            _LOAD_ERROR = exc
            raise


def load_error() -> Optional[BaseException]:
    return _LOAD_ERROR


def strerror(code: int) -> str:
    try:
        return load().b200w4a4_strerror(int(code)).decode()
    except BaseException:
        return f"error {code}"


def check(code: int, where: str) -> None:
    if code != 0:
        raise B200W4A4Error(code, where)
