"""ctypes binding of libswiglu_b200.so (the C ABI declared in include/swiglu_b200.h).

There is no fallback.  The library is bound on first use (``lib.<entry point>`` or ``load()``):
if it is missing or was built from other sources than the ones in the tree, it is rebuilt with
nvcc then; if that is impossible, or the library does not export a declared symbol, that first use
raises ImportError.  Importing the package alone does not map the library, so host-only helpers
(the synthetic workloads, the row partition) can be used by processes that never touch a GPU.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libswiglu_b200.so"

F32, F16, BF16 = 0, 1, 2
OK = 0

_c_i64 = ctypes.c_int64
_c_ptr = ctypes.c_void_p

# name -> (restype, argtypes); one entry per declaration in include/swiglu_b200.h
SIGNATURES = {
    "swiglu_b200_version": (ctypes.c_int, []),
    "swiglu_b200_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "swiglu_b200_last_cuda_error": (ctypes.c_int, []),
    "swiglu_b200_launch_count": (ctypes.c_uint64, []),
    "swiglu_b200_fwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int, ctypes.c_float, ctypes.c_float,
         ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_bwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int,
         ctypes.c_float, ctypes.c_float, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_plan_fwd": (ctypes.c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int]),
    "swiglu_b200_plan_bwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int],
    ),
    "swiglu_b200_geglu_fwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_geglu_bwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_bwd_recompute": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, ctypes.c_int, ctypes.c_float, ctypes.c_float,
         ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_host_fwd_bwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, ctypes.c_int, ctypes.c_float,
         ctypes.c_float, _c_ptr, ctypes.c_uint64, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_host_workspace_bytes": (ctypes.c_uint64, [_c_i64, _c_i64, ctypes.c_int]),
    "swiglu_b200_gemm_fwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, ctypes.c_float, ctypes.c_float,
         _c_ptr, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_geglu_gemm_fwd": (
        ctypes.c_int,
        [_c_ptr] * 6 + [_c_i64] * 3 + [ctypes.c_int, _c_ptr, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_lora_geglu_gemm_fwd": (
        ctypes.c_int,
        [_c_ptr] * 9 + [_c_i64] * 4 + [ctypes.c_int, _c_ptr, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_geglu_bwd_recompute": (
        ctypes.c_int,
        [_c_ptr] * 6 + [_c_i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_lora_gemm_fwd": (
        ctypes.c_int,
        [_c_ptr] * 9 + [_c_i64] * 4 + [ctypes.c_float, ctypes.c_float, _c_ptr, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_gemm_fwd_noalloc": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, ctypes.c_float, ctypes.c_float, _c_ptr,
         ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_gemm_launch_count": (ctypes.c_uint64, []),
    "swiglu_b200_lora_swiglu_fwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64,
         ctypes.c_float, ctypes.c_float, _c_ptr, ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_lora_launch_count": (ctypes.c_uint64, []),
    "swiglu_b200_gemm_bwd": (
        ctypes.c_int,
        [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr,
         ctypes.c_int, _c_ptr],
    ),
    "swiglu_b200_gemm_bwd_launch_count": (ctypes.c_uint64, []),
    "swiglu_b200_selftest_wait_timeout": (
        ctypes.c_int, [_c_ptr, ctypes.c_int, _c_i64, ctypes.c_int, ctypes.c_int, _c_ptr]),
}


def _load() -> ctypes.CDLL:
    from . import build as _build

    if _build.is_stale():
        try:
            _build.build()
        except Exception as exc:
            raise ImportError(
                f"{LIB_PATH} is missing or out of date and could not be built ({exc}); "
                "there is no non-CUDA fallback"
            ) from exc
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


class _LazyLibrary:
    """Stands for the bound library; binds it the first time an entry point is looked up."""

    __slots__ = ("_cdll",)

    def __init__(self):
        self._cdll = None

    def _bound(self) -> ctypes.CDLL:
        if self._cdll is None:
            self._cdll = _load()
        return self._cdll

    def __getattr__(self, name: str):
        return getattr(self._bound(), name)


lib = _LazyLibrary()


def load() -> ctypes.CDLL:
    """Binds the library now (building it first when stale) and returns the ctypes handle."""
    return lib._bound()


def is_loaded() -> bool:
    return lib._cdll is not None


class SwigluB200Error(RuntimeError):
    """A non-zero return code from the C ABI."""

    def __init__(self, where: str, code: int):
        text = lib.swiglu_b200_strerror(code).decode()
        cuda = lib.swiglu_b200_last_cuda_error()
        super().__init__(f"{where}: swiglu_b200 error {code} ({text}); last CUDA error {cuda}")
        self.code = code
        self.cuda_error = cuda


def check(where: str, code: int) -> None:
    if code != OK:
        raise SwigluB200Error(where, code)


def launch_count() -> int:
    return int(lib.swiglu_b200_launch_count())
