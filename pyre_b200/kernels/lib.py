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


class GemmFix(ctypes.Structure):
    """``PyreGemmFix`` of csrc/gemm_tc.cu: work folded into a product of few tokens (field for field)."""

    _fields_ = [("fix", I), ("scale_tiles", I), ("scale_n", F), ("scale_eps", F), ("scale_ssq", P),
                ("tile_counters", P), ("resid", P), ("norm_w", P), ("h_out", P), ("ssq_out", P), ("bias", P),
                ("cos_t", P), ("sin_t", P), ("q_out", P), ("kv_cache", P), ("slot_mapping", P),
                ("nh", I), ("nkv", I), ("hd", I), ("rot", I), ("page_size", I), ("n_pages", LL)]

# function name -> (library, argument types).  Every function returns int: 0 or an error code.
SIGNATURES: dict[str, tuple[str, list]] = {
    "pyre_embedding": ("elementwise", [P, I, P, P, I, I, I, P, P]),
    "pyre_add_rmsnorm": ("elementwise", [P, P, P, I, LL, P, P, P, I, I, F, I, I, P]),
    "pyre_add_residual": ("elementwise", [P, P, LL, I, P]),
    "pyre_rope_table": ("elementwise", [P, P, P, P, I, I, P]),
    "pyre_qkv_rope_write": ("elementwise", [P, P, I, LL, P, P, P, P, P, P, I, I, I, I, I, I, I, LL, P, P]),
    "pyre_silu_mul": ("elementwise", [P, P, I, I, I, I, P]),
    "pyre_sum_partials": ("elementwise", [P, I, LL, P, LL, I, P]),
    "pyre_feed_tokens": ("elementwise", [P, P, P, P, I, P]),
    "pyre_delay": ("elementwise", [LL, P]),
    "pyre_gemm_tc": ("gemm_tc", [P, I, LL, P, I, LL, I, P, I, LL, LL, LL, I, I, I, I, I, P, P, P]),
    "pyre_scale_rows": ("elementwise", [P, P, I, P, I, I, F, P]),
    "pyre_sample": ("sampling", [P, LL, P, P, P, P, I, I, P, P]),
    "pyre_sample_slices": ("sampling", [I]),
    "pyre_paged_attention_generic": ("attention_generic", [P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, LL, P, P]),
    "pyre_sgemm_nt": ("gemm_f32", [P, LL, P, LL, P, LL, P, I, I, I, P]),
    "pyre_paged_attention_mma": ("attention_mma", [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, LL, I, P, P]),
    "pyre_attention_prefill_tc": ("attention_tc", [P, P, P, P, I, P, P, I, I, I, I, I, I, I, LL, I, F, I, I, P, P, P, P]),
    "pyre_attention_prefill": ("attention_prefill", [P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, LL, P, P]),
}

_ERRORS = {100001: "bad argument", 100002: "unsupported size"}


class KernelError(RuntimeError):
    pass


# ---------------------------------------------------------------------------------- per-kernel timing
# Which class of the decoder step a function belongs to when no part has named one.  The matrix product is
# one function for five classes (q/k/v, output projection, gate/up, down, head): the parts name those with
# ``section``.
DEFAULT_CLASS = {
    "pyre_embedding": "embed", "pyre_add_rmsnorm": "norm", "pyre_add_residual": "norm", "pyre_rope_table": "rotary+write",
    "pyre_qkv_rope_write": "rotary+write", "pyre_silu_mul": "activation", "pyre_sum_partials": "sum_partials",
    "pyre_feed_tokens": "feed", "pyre_delay": "delay", "pyre_gemm_tc": "product", "pyre_sgemm_nt": "product", "pyre_scale_rows": "norm", "pyre_sample": "sampler",
    "pyre_paged_attention_generic": "attention", "pyre_paged_attention_mma": "attention",
    "pyre_attention_prefill_tc": "attention", "pyre_attention_prefill": "attention",
}


class KernelTimer:
    """CUDA events around every launch made through ``call`` while the timer is installed (``timing``).

    An event between two launches also ends the overlap that the programmatic dependent launch gives two
    neighbours, so the classes' times add up to a step in which every kernel runs alone.  One event stands
    between two launches (the end of one is the start of the next), so the times of a run of launches add up
    to the time from its first event to its last.  The caller should keep the GPU behind the host (a queued
    delay before the step) so that no event waits for a launch."""

    def __init__(self):
        self.records: list = []      # (class, function, start event, end event)
        self.last = None             # the event recorded after the latest launch

    def totals(self) -> dict:
        """class -> {"us": summed device time, "launches": n}; synchronises."""
        import torch
        torch.cuda.synchronize()
        out: dict = {}
        for cls, _fn, a, b in self.records:
            d = out.setdefault(cls, {"us": 0.0, "launches": 0})
            d["us"] += a.elapsed_time(b) * 1e3
            d["launches"] += 1
        return out


_timer: "KernelTimer | None" = None
_sections: list[str] = []


class _Section:
    __slots__ = ("name",)

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        _sections.append(self.name)

    def __exit__(self, *exc):
        _sections.pop()
        return False


class _NoSection:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SECTION = _NoSection()


def section(name: "str | None"):
    """``with lib.section("qkv"):`` names the class of the launches inside for the per-kernel timer.
    Costs nothing while no timer is installed (or the name is None)."""
    return _Section(name) if _timer is not None and name is not None else _NO_SECTION


def current_section() -> "str | None":
    return _sections[-1] if _sections else None


class timing:
    """``with lib.timing() as t:`` installs a KernelTimer for the launches inside."""

    def __enter__(self) -> KernelTimer:
        global _timer
        if _timer is not None:
            raise RuntimeError("a kernel timer is already installed")
        _timer = KernelTimer()
        return _timer

    def __exit__(self, *exc):
        global _timer
        _timer = None
        del _sections[:]
        return False


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
    if _timer is None:
        code = function(name)(*args)
    else:
        import torch
        fn = function(name)
        a = _timer.last
        if a is None:
            a = torch.cuda.Event(enable_timing=True)
            a.record()
        code = fn(*args)
        b = torch.cuda.Event(enable_timing=True)
        b.record()
        _timer.last = b
        _timer.records.append((_sections[-1] if _sections else DEFAULT_CLASS.get(name, name), name, a, b))
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
