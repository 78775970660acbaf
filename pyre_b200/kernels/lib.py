"""ctypes bindings of the kernel libraries.

Each library is loaded the first time one of its functions is called (building it first
if needed).  There is no fallback: if a library cannot be built or loaded, or a launch
returns an error, the call raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build

P, I, LL, F = c_void_p, c_int, c_longlong, c_float

# function name -> (library, argument types).  Every function returns int: 0 or an error code.
SIGNATURES: dict[str, tuple[str, list]] = {
    "pyre_embedding": ("elementwise", [P, I, P, P, I, I, I, P, P]),
    "pyre_add_rmsnorm": ("elementwise", [P, P, P, I, LL, P, P, P, I, I, F, I, I, P]),
    "pyre_add_residual": ("elementwise", [P, P, LL, I, P]),
    "pyre_rope_table": ("elementwise", [P, P, P, P, I, I, P]),
    "pyre_qkv_rope_write": ("elementwise", [P, P, I, LL, P, P, P, P, P, P, I, I, I, I, I, I, I, P]),
    "pyre_silu_mul": ("elementwise", [P, P, I, I, I, I, P]),
    "pyre_sum_partials": ("elementwise", [P, I, LL, P, LL, I, P]),
    "pyre_feed_tokens": ("elementwise", [P, P, P, P, I, P]),
    "pyre_gemm_tc": ("gemm_tc", [P, I, LL, P, I, LL, I, P, I, LL, LL, LL, I, I, I, I, I, P, P]),
    "pyre_sample": ("sampling", [P, LL, P, P, P, P, I, I, P, P]),
    "pyre_sample_slices": ("sampling", [I]),
    "pyre_paged_attention_generic": ("attention_generic", [P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, P]),
    "pyre_sgemm_nt": ("gemm_f32", [P, LL, P, LL, P, LL, P, I, I, I, P]),
    "pyre_paged_attention_mma": ("attention_mma", [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, LL, I, P, P]),
    "pyre_attention_prefill_tc": ("attention_tc", [P, P, P, P, I, P, P, I, I, I, I, I, I, I, LL, I, F, I, P, P]),
    "pyre_attention_prefill": ("attention_prefill", [P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P]),
}

_ERRORS = {100001: "bad argument", 100002: "unsupported size"}


class KernelError(RuntimeError):
    pass


_libs: dict[str, ctypes.CDLL] = {}
_funcs: dict[str, ctypes._CFuncPtr] = {}
launch_count = 0  # kernels launched through this module since import (one per call)


def register_function(name: str, library: str, argtypes: list) -> None:
    SIGNATURES[name] = (library, argtypes)


def load_library(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        build.ensure_built([name])
        path = build.library_path(name)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load kernel library {path}: {e}") from e
        _libs[name] = lib
    return lib


def loaded_libraries() -> list[str]:
    return [str(build.library_path(n)) for n in _libs]


def function(name: str):
    fn = _funcs.get(name)
    if fn is None:
        libname, argtypes = SIGNATURES[name]
        fn = getattr(load_library(libname), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _funcs[name] = fn
    return fn


def call_value(name: str, *args) -> int:
    """Call a function that returns a plain number (no launch, no error code)."""
    return int(function(name)(*args))


def call(name: str, *args) -> None:
    global launch_count
    code = function(name)(*args)
    launch_count += 1
    if code != 0:
        what = _ERRORS.get(code)
        if what is None:
            what = f"CUDA error {code}"
            try:
                import torch
                what += f" ({torch.cuda.cudart().cudaGetErrorString(code)})"  # type: ignore[attr-defined]
            except Exception:
                pass
        raise KernelError(f"{name} failed: {what}")
