"""ctypes binding of ``libchb.so`` (the C ABI declared in ``csrc/api/chb.h``)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libchb.so"
_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load (building first if necessary and possible) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists() or os.environ.get("CHB_REBUILD") == "1":
        from . import _build

        _build.build()
    if not _LIB_PATH.exists():
        raise NativeLibraryMissing(f"{_LIB_PATH} is missing and could not be built")
    L = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    _declare(L)
    _lib = L
    return L


def _declare(L: C.CDLL) -> None:
    vp, i32, i64, u64, cp = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_char_p
    L.chb_program_create.restype = vp
    L.chb_program_create.argtypes = [cp, cp, i32, i32, i32, i64, i32, i32, i32, cp, i32]
    L.chb_program_create_alltoallv.restype = vp
    L.chb_program_create_alltoallv.argtypes = [i32, i32, i32, C.POINTER(i64), cp, i32]
    L.chb_program_destroy.restype = None
    L.chb_program_destroy.argtypes = [vp]
    L.chb_program_info.restype = i32
    L.chb_program_info.argtypes = [vp, C.POINTER(i64), i32]
    L.chb_program_name.restype = cp
    L.chb_program_name.argtypes = [vp]
    L.chb_program_verify.restype = i32
    L.chb_program_verify.argtypes = [vp, cp, i32]
    L.chb_program_simulate.restype = i32
    L.chb_program_simulate.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), u64, cp, i32]
    L.chb_program_run_threads.restype = i32
    L.chb_program_run_threads.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), i32, C.POINTER(C.c_double)]
    L.chb_program_run_threads_late.restype = i32
    L.chb_program_run_threads_late.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), i32, i32]
    L.chb_program_ll_lines.restype = C.c_longlong
    L.chb_program_ll_lines.argtypes = [vp, i32]
    L.chb_program_ll_info.restype = i32
    L.chb_program_ll_info.argtypes = [vp, i32, C.POINTER(C.c_longlong), i32]
    L.chb_program_simulate_ll.restype = i32
    L.chb_program_simulate_ll.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), u64, i32, i32, i32, cp, i32]
    L.chb_program_export.restype = i32
    L.chb_program_export.argtypes = [vp, vp, vp, vp, vp, vp]
    L.chb_list_algorithms.restype = i32
    L.chb_list_algorithms.argtypes = [cp, cp, i32]
    L.chb_dtype_size.restype = i32
    L.chb_dtype_size.argtypes = [i32]
    L.chb_version.restype = cp
    for name, (res, args) in _OPTIONAL.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args


# declared lazily because the GPU half of the library may be absent in a
# host-only build
_OPTIONAL: dict = {}


def optional(name: str, restype, argtypes) -> None:
    _OPTIONAL[name] = (restype, argtypes)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes


# error codes / enums mirrored from chb.h
SUCCESS, ERR_NO_MEM, ERR_OTHER, ERR_COUNT, ERR_OP, ERR_ARG, ERR_TIMEOUT, ERR_CUDA, ERR_UNSUPPORTED = range(9)
F32, BF16, F16, I32, F64, I64, U8 = range(7)
SUM, MAX, MIN, PROD = range(4)
ERR_NAMES = {
    0: "success", 1: "out of memory", 2: "error", 3: "bad count", 4: "unsupported reduction",
    5: "invalid argument", 6: "timeout", 7: "CUDA error", 8: "unsupported",
}
