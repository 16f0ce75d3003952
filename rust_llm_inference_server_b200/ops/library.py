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
    "rlis_embedding": [P, P, P, I, I, I, I, P],
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
}

OPTIONAL_SIGNATURES: dict = {}


class KernelError(RuntimeError):
    pass


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
        handle.rlis_gemm_tcgen05_error.argtypes = []
        handle.rlis_gemm_tcgen05_error.restype = c_int
        handle.rlis_attention_prefill_tc_set_splits.argtypes = [c_int]
        handle.rlis_attention_prefill_tc_set_splits.restype = None
        handle.rlis_attention_prefill_tc_error.argtypes = []
        handle.rlis_attention_prefill_tc_error.restype = c_int
        handle.rlis_stream_gemm_error.argtypes = []
        handle.rlis_stream_gemm_error.restype = c_int
        handle.rlis_stream_gemm_set_target.argtypes = [c_int]
        handle.rlis_stream_gemm_set_target.restype = None
        handle.rlis_attention_decode_set_stages.argtypes = [c_int]
        handle.rlis_attention_decode_set_stages.restype = None
        handle.rlis_sample_filtered_set_cluster.argtypes = [c_int]
        handle.rlis_sample_filtered_set_cluster.restype = None
        handle.rlis_attention_decode_set_tma.argtypes = [c_int]
        handle.rlis_attention_decode_set_tma.restype = None
        handle.rlis_attention_decode_error.argtypes = []
        handle.rlis_attention_decode_error.restype = c_int
        handle.rlis_attention_decode_set_cluster.argtypes = [c_int]
        handle.rlis_attention_decode_set_cluster.restype = None
        handle.rlis_set_pdl.argtypes = [c_int]
        handle.rlis_set_pdl.restype = None
        if os.environ.get("RLIS_PDL", "1") == "0":      # programmatic dependent launch is on unless switched off
            handle.rlis_set_pdl(0)
        if os.environ.get("RLIS_STREAM_CTAS"):           # for measurements: CTAs a streaming product is cut into
            handle.rlis_stream_gemm_set_target(int(os.environ["RLIS_STREAM_CTAS"]))
        if os.environ.get("RLIS_DECODE_STAGES"):         # for measurements: stages of keys in decode attention
            handle.rlis_attention_decode_set_stages(int(os.environ["RLIS_DECODE_STAGES"]))
        _lib = handle
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
