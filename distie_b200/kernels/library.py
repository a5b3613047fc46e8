"""``ctypes`` bindings of the CUDA launchers.

Each kernel unit is a shared library built by :mod:`distie_b200.csrc.build`; a unit
is compiled and loaded when the first function of it is asked for.  Launchers take
raw device pointers (``tensor.data_ptr()``) and the current stream's handle, start
no allocation and no synchronisation, and return 0 or an error code, which
:func:`check` turns into an exception.  There is no fallback: when the library
cannot be built or loaded the engine stops with the reason.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

P = c_void_p
I = c_int
F = c_float
L = c_longlong

# name -> (unit, argument types); every launcher returns int unless listed in _RESULT.
_SIGNATURES: dict[str, tuple[str, list]] = {
    "distie_embed": ("base", [P, P, P, I, I, I, I, P, P]),
    "distie_add_rmsnorm": ("base", [P, P, P, P, P, I, I, F, I, P]),
    "distie_rope_kv_write": ("base", [P, P, P, P, P, I, P, F, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P]),
    "distie_swiglu": ("base", [P, P, I, I, I, P]),
    "distie_add_rmsnorm_split": ("base", [P, I, L, P, P, P, P, I, I, F, I, P]),
    "distie_rope_kv_write_split": (
        "base", [P, I, L, I, P, P, I, P, P, P, P, I, P, F, P, P, I, I, I, I, I, I, I, I, I, I, P, P]
    ),
    "distie_rope_rows": ("base", [P, P, P, P, I, P, F, I, I, I, I, I, P, P, P, P]),
    "distie_bias_cast": ("base", [P, P, P, L, I, I, P]),
    "distie_attention_generic": ("base", [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P, P]),
    "distie_attention_decode": ("base", [P, I, P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, P, P]),
    "distie_attention_decode_scratch_floats": ("base", [I, I, I, I]),
    "distie_sample": ("base", [P, L, I, I, P, P, P, P]),
    "distie_attention_prefill": ("bf16", [P, I, P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P, P]),
    "distie_attention_prefill_tile": ("bf16", []),
    "distie_attention_prefill_tcgen05": (
        "bf16", [P, I, P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, P, P]
    ),
    "distie_attention_decode_mma_stages": ("bf16", [I, I, I, I]),
    "distie_attention_decode_mma": ("bf16", [P, I, P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P, P]),
    "distie_attention_decode_mma_qkv": (
        "bf16", [P, I, L, I, P, P, F, I, P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P, P]
    ),
    "distie_gemm_tcgen05": ("bf16", [P, I, P, P, I, I, I, I, I, I, I, P, P]),
    "distie_gemm_tcgen05_qkv": ("bf16", [P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, P, P]),
    "distie_gemm_tcgen05_skinny_splits": ("bf16", [I, I, I]),
    "distie_gemm_tcgen05_skinny": ("bf16", [P, I, P, P, P, I, I, I, I, I, I, I, P, P]),
}
_RESULT = {"distie_attention_decode_scratch_floats": c_longlong}

_libraries: dict[str, ctypes.CDLL] = {}
_functions: dict[str, object] = {}


class KernelError(RuntimeError):
    pass


def register_signature(name: str, unit: str, argtypes: list, restype=None) -> None:
    _SIGNATURES[name] = (unit, argtypes)
    if restype is not None:
        _RESULT[name] = restype


def load_unit(unit: str) -> ctypes.CDLL:
    lib = _libraries.get(unit)
    if lib is None:
        from ..csrc import build

        path = build.build_cuda_unit(unit)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise KernelError(f"cannot load kernel library {path}: {exc}") from exc
        _libraries[unit] = lib
    return lib


def function(name: str):
    fn = _functions.get(name)
    if fn is None:
        unit, argtypes = _SIGNATURES[name]
        lib = load_unit(unit)
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise KernelError(f"kernel library of unit {unit!r} has no symbol {name}") from exc
        fn.argtypes = argtypes
        fn.restype = _RESULT.get(name, c_int)
        _functions[name] = fn
    return fn


_ARG_ERRORS = {-1: "invalid argument", -2: "size or dtype not supported by this kernel"}


def check(code: int, name: str) -> None:
    if code == 0:
        return
    if code in _ARG_ERRORS:
        raise KernelError(f"{name}: {_ARG_ERRORS[code]}")
    raise KernelError(f"{name}: CUDA error {code} at launch")
