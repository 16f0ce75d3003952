"""Loads the kernel library and declares the C signature of every exported launcher.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is present, the
first op raises.  Launchers return 0, a cudaError_t (> 0) or a negative library code.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build

_lib = None

P = c_void_p
I = c_int
F = c_float
LL = c_longlong

# name -> argument types (the stream is always last)
SIGNATURES = {
    "rlis_embedding": [P, P, P, I, I, I, F, I, P],
    "rlis_embedding_sink": [P, P, P, P, P, P, I, I, I, F, P],
    "rlis_logit_transform": [P, I, I, LL, F, F, P],
    "rlis_attention_prefill_tile": [],
    "rlis_rmsnorm": [P, P, P, P, P, I, I, F, I, P],
    "rlis_swiglu": [P, P, I, I, I, I, P],
    "rlis_gemm_f32_nt": [P, P, P, I, I, I, P],
    "rlis_rope_cache": [P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "rlis_attention_generic": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
    "rlis_attention_decode": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P],
    "rlis_attention_decode_pages": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P],
    "rlis_attention_decode_qkv": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P],
    "rlis_attention_prefill": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, P],
    "rlis_attention_prefill_tc": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P],
    "rlis_attention_prefill_tc_takes": [I, I, I, I],
    "rlis_repetition_penalty": [P, P, P, P, P, I, I, LL, P],
    "rlis_sample_rows": [P, P, P, I, I, LL, P],
    "rlis_sample_filtered": [P, P, P, I, I, LL, P],
    "rlis_nll_rows": [P, P, P, I, I, LL, P],
    "rlis_gemm_tcgen05": [P, P, P, I, I, I, I, P],
    "rlis_stream_gemm_bf16": [P, P, P, I, I, I, I, I, P],
    "rlis_stream_gemm_fused": [P, P, P, I, I, I, I, I, P, I, I, F, P, P, P, P, P],
    "rlis_take_errors": [P, P],
    "rlis_stream_gemm_timeline": [I],
    "rlis_stream_gemm_timeline_read": [P, P],
    "rlis_attention_decode_last_variant": [],
}

OPTIONAL_SIGNATURES: dict = {}


class KernelError(RuntimeError):
    pass


# Switches for measurements and tests; nothing in the engine sets one.  In the library
# (csrc/kernels/runtime_switches.cu): pdl, stream_ctas, stream_min_stages, decode_stages, decode_cluster,
# decode_tma, prefill_splits, gemm_pair, filtered_cluster.  In Python (ops/__init__.py): fuse_norms, prefill_tcgen05, stream_rows.
# `RLIS_DEBUG=name=value,name=value` in the environment sets them when the library is loaded.
PYTHON_SWITCHES: dict = {}


def debug_set(name: str, value: int) -> None:
    """Holds one of the kernels' own choices fixed (see the list above)."""
    if name in PYTHON_SWITCHES:
        PYTHON_SWITCHES[name](int(value))
        return
    if lib().rlis_debug_set(name.encode(), int(value)) != 0:
        raise KernelError(f"no debug switch {name!r}")


def lib():
    global _lib
    if _lib is None:
        path = build.build_kernels()
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from e
        for name, args in {**SIGNATURES, **OPTIONAL_SIGNATURES}.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise KernelError(f"kernel library {path} lacks symbol {name}") from e
            fn.argtypes = args
            fn.restype = c_int
        for name in ("rlis_gemm_tcgen05_error", "rlis_stream_gemm_error", "rlis_attention_prefill_tc_error",
                     "rlis_attention_decode_error"):
            fn = getattr(handle, name)
            fn.argtypes = []
            fn.restype = c_int
        handle.rlis_debug_set.argtypes = [ctypes.c_char_p, c_int]
        handle.rlis_debug_set.restype = c_int
        _lib = handle
        for item in filter(None, os.environ.get("RLIS_DEBUG", "").split(",")):
            name, _, value = item.partition("=")
            debug_set(name.strip(), int(value))
    return _lib


_CUDA_ERRORS = {1: "invalid value", 2: "out of memory", 9: "invalid configuration",
                98: "invalid device function", 209: "no kernel image for this device",
                700: "illegal address", 715: "illegal instruction", 719: "launch failure"}


def check(code: int, name: str) -> None:
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{name}: this kernel does not take these sizes or this element type")
    if code < 0:
        raise KernelError(f"{name}: library error {code}")
    raise KernelError(f"{name}: CUDA error {code} ({_CUDA_ERRORS.get(code, 'see cudaError_t')})")
